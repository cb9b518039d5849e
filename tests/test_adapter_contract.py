"""The user-defined adapter contract: the reference's validation rules (compile_tvm.py:29-93), the probes that
decide whether a class is the low-rank pair the kernels implement, and the lowering of its parameters."""
import importlib

import pytest
import torch

from conftest import load

ac = load("adapter_contract")
Tensor, nn, op = ac.Tensor, ac.nn, ac.op


def _init(self, in_features: int, out_features: int, config: ac.LoraConfig):
    self.scaling = config.alpha / config.r


def test_reference_example_class_is_accepted_and_lowered():
    has_wc, n = ac.verify_adapter_def(ac.Lora)
    assert (has_wc, n) == (False, 2)
    fam = ac.probe_family(ac.Lora, 64, 48, ac.LoraConfig(r=8, alpha=16))
    assert fam.rank == 8 and abs(fam.scale - 2.0) < 1e-6
    p0, p1 = torch.randn(64, 8), torch.randn(8, 48)
    A, B = fam.lower([p0, p1])
    assert torch.equal(A, p0.t()) and torch.equal(B, p1.t())
    # forward synthesised by the reference (take by wid, apply, post-process: compile_tvm.py:106-112) == lowered form
    x = torch.randn(3, 64)
    want = fam.instance.post_computation(fam.instance.weight_application(x, p0, p1))
    torch.testing.assert_close(fam.scale * (x @ A.t()) @ B.t(), want)


@pytest.mark.parametrize("drop,msg", [("define_parameters", "define_parameters method must be defined"),
                                      ("weight_application", "weight_application method must be defined"),
                                      ("post_computation", "post_computation method must be defined")])
def test_missing_methods_are_rejected_with_the_rule(drop, msg):
    ns = {k: v for k, v in vars(ac.Lora).items() if k in ("define_parameters", "weight_application", "post_computation")}
    ns["__init__"] = _init
    ns.pop(drop)
    cls = type("Broken", (nn.Module,), ns)
    with pytest.raises(AssertionError, match=msg):
        ac.verify_adapter_def(cls)


def test_annotation_rules():
    class NoInitTypes(nn.Module):
        def __init__(self, in_features, out_features: int, config: ac.LoraConfig):
            pass
        define_parameters = ac.Lora.define_parameters
        weight_application = ac.Lora.weight_application
        post_computation = ac.Lora.post_computation
    with pytest.raises(AssertionError, match="in_features: int"):
        ac.verify_adapter_def(NoInitTypes)

    class WrongApplication(nn.Module):
        __init__ = _init
        define_parameters = ac.Lora.define_parameters
        post_computation = ac.Lora.post_computation

        def weight_application(self, x: Tensor, only_one: Tensor) -> Tensor:
            return x
    with pytest.raises(AssertionError, match="weight_application must have as input what define_params returns"):
        ac.verify_adapter_def(WrongApplication)

    class PostTakesTwo(nn.Module):
        __init__ = _init
        define_parameters = ac.Lora.define_parameters
        weight_application = ac.Lora.weight_application

        def post_computation(self, y: Tensor, z: Tensor) -> Tensor:
            return y
    with pytest.raises(AssertionError, match="single Tensor as input"):
        ac.verify_adapter_def(PostTakesTwo)


@pytest.fixture
def scaled_class():
    @__import__("dataclasses").dataclass(frozen=True)
    class MagConfig:
        r: int
        alpha: float

    class MagnitudeLora(nn.Module):
        """Three declared parameters; weight_computation folds a per-output magnitude into the second factor
        (the kind of variant the optional method exists for): done once at load, then it is a plain pair."""
        def __init__(self, in_features: int, out_features: int, config: MagConfig):
            super().__init__()
            self.c = config.alpha / config.r

        def define_parameters(self, in_features: int, out_features: int, config: MagConfig) -> tuple[Tensor, Tensor, Tensor]:
            return (nn.Parameter((in_features, config.r)), nn.Parameter((config.r, out_features)),
                    nn.Parameter((1, out_features)))

        def weight_computation(self, a: Tensor, b: Tensor, m: Tensor) -> tuple[Tensor, Tensor]:
            return a, op.multiply(b, m)

        def weight_application(self, x: Tensor, a: Tensor, bm: Tensor) -> Tensor:
            return op.matmul(op.matmul(x, a), bm)

        def post_computation(self, y: Tensor) -> Tensor:
            return y * self.c
    return MagConfig, MagnitudeLora


def test_weight_computation_runs_once_at_load(scaled_class):
    MagConfig, MagnitudeLora = scaled_class
    assert ac.verify_adapter_def(MagnitudeLora) == (True, 3)
    fam = ac.probe_family(MagnitudeLora, 32, 24, MagConfig(4, 2.0))
    assert fam.rank == 4 and abs(fam.scale - 0.5) < 1e-6
    a, b, m = torch.randn(32, 4), torch.randn(4, 24), torch.rand(1, 24) + 0.5
    A, B = fam.lower([a, b, m])
    x = torch.randn(6, 32)
    torch.testing.assert_close(0.5 * (x @ A.t()) @ B.t(), 0.5 * (x @ a) @ (b * m))
    # through the file form: p2 rides next to lora_A / lora_B
    ac.register_adapter(MagConfig, MagnitudeLora)
    tensors = {"layers.0.self_attn.q_proj.lora_A.weight": a.t().contiguous(), "layers.0.self_attn.q_proj.lora_B.weight": b.t().contiguous(),
               "layers.0.self_attn.q_proj.p2.weight": m}
    low, scale = ac.lower_adapter_file(tensors, MagConfig(4, 2.0), {})
    assert abs(scale - 0.5) < 1e-6
    torch.testing.assert_close(low["layers.0.self_attn.q_proj.lora_B.weight"], (b * m).t())


def test_classes_outside_the_family_are_refused(scaled_class):
    class TanhPost(nn.Module):
        __init__ = _init
        define_parameters = ac.Lora.define_parameters
        weight_application = ac.Lora.weight_application

        def post_computation(self, y: Tensor) -> Tensor:
            return op.tanh(y)
    with pytest.raises(ac.UnsupportedAdapter, match="post_computation is not multiplication by a constant"):
        ac.probe_family(TanhPost, 16, 16, ac.LoraConfig(4, 8))

    class NotBilinear(nn.Module):
        __init__ = _init
        define_parameters = ac.Lora.define_parameters
        post_computation = ac.Lora.post_computation

        def weight_application(self, x: Tensor, a: Tensor, b: Tensor) -> Tensor:
            return op.matmul(op.tanh(op.matmul(x, a)), b)
    with pytest.raises(ac.UnsupportedAdapter, match="not \\(x @ P0\\) @ P1"):
        ac.probe_family(NotBilinear, 16, 16, ac.LoraConfig(4, 8))

    class ThreeFactors(nn.Module):
        __init__ = _init
        post_computation = ac.Lora.post_computation

        def define_parameters(self, in_features: int, out_features: int, config: ac.LoraConfig) -> tuple[Tensor, Tensor, Tensor]:
            return nn.Parameter((in_features, config.r)), nn.Parameter((config.r, config.r)), nn.Parameter((config.r, out_features))

        def weight_application(self, x: Tensor, a: Tensor, s: Tensor, b: Tensor) -> Tensor:
            return op.matmul(op.matmul(op.matmul(x, a), s), b)
    with pytest.raises(ac.UnsupportedAdapter, match="two-factor form"):
        ac.probe_family(ThreeFactors, 16, 16, ac.LoraConfig(4, 8))
