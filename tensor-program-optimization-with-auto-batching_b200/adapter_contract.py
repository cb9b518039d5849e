"""User-defined adapter classes: the reference's contract, checked the same way, lowered onto the kernels.

The reference lets a user describe an adapter as a small class
(``tvm/llama_auto_batcher/lora.py:10-24``) with four methods --
``define_parameters``, optional ``weight_computation``, ``weight_application`` and
``post_computation`` -- validates the class by its annotations
(``tvm/llama_auto_batcher/compile_tvm.py:29-93``), gives every parameter a leading
"adapter" axis and synthesises ``forward(x, wids)`` = take the rows' parameters, apply, post-process
(``compile_tvm.py:95-113``); TVM then compiles whatever arithmetic the methods contain.

Here there is no compiler: the kernels implement one family, the low-rank pair
``y = c * (x @ P0) @ P1``.  So a class is (1) validated by exactly the reference's rules, (2) *probed*:
its methods are executed on small random tensors to establish that ``weight_application`` is that
bilinear form in its two (possibly ``weight_computation``-derived) tensors and that
``post_computation`` is multiplication by a constant ``c``; (3) lowered: ``weight_computation`` runs
once at load time per adapter and the result is handed to the packed stacks as ``A = P0^T [r, in]``,
``B = P1^T [out, r]``, ``scale = c``.  Anything outside the family is refused with
:class:`UnsupportedAdapter` naming the probe that failed -- never approximated.

The stand-ins ``nn`` / ``op`` / ``Tensor`` carry just enough of ``tvm.relax.frontend.nn`` for such
classes to be written the way the reference writes them, over torch tensors on the host.
"""
import dataclasses
import types
from typing import get_args, get_origin, get_type_hints

import torch

Tensor = torch.Tensor


class UnsupportedAdapter(TypeError):
    """The class is well-formed but its arithmetic is not the low-rank pair the kernels implement."""


# ---- the small part of the front-end namespace adapter classes use -------------------------------------
class _ParamSpec:
    """What ``nn.Parameter(shape, dtype)`` declares (compile_tvm.py:99-102 reads ``.shape`` / ``.dtype``)."""

    def __init__(self, shape, dtype="float16"):
        self.shape, self.dtype = [int(s) for s in shape], dtype


class _NN:
    class Module:
        def __init__(self):
            pass

    Parameter = _ParamSpec
    Tensor = Tensor


class _Op:
    matmul = staticmethod(torch.matmul)
    add = staticmethod(torch.add)
    subtract = staticmethod(torch.sub)
    multiply = staticmethod(torch.mul)
    divide = staticmethod(torch.div)
    sqrt = staticmethod(torch.sqrt)
    square = staticmethod(torch.square)
    tanh = staticmethod(torch.tanh)
    sigmoid = staticmethod(torch.sigmoid)

    @staticmethod
    def take(x, indices, axis=0):
        return torch.index_select(x, axis, indices.long())

    @staticmethod
    def sum(x, axis=None, keepdims=False):
        return torch.sum(x) if axis is None else torch.sum(x, dim=axis, keepdim=keepdims)

    @staticmethod
    def permute_dims(x, axes=None):
        return x.permute(*axes) if axes is not None else x.transpose(-1, -2)


nn, op = _NN, _Op


# ---- validation: the rules of compile_tvm.py:29-93 ----------------------------------------------------------
def _tensors_with_count(annotation):
    if isinstance(annotation, types.GenericAlias):
        args = get_args(annotation)
        return get_origin(annotation) is tuple and all(a is Tensor for a in args), len(args)
    if isinstance(annotation, type):
        return annotation is Tensor, 1
    return False, 0


def _hints(fn):
    """Annotations as objects, also when the defining module postpones their evaluation."""
    try:
        return dict(get_type_hints(fn))
    except Exception:
        return dict(getattr(fn, "__annotations__", {}))


def verify_adapter_def(adapter_class):
    """Returns ``(weight_computation_defined, number_of_parameters)``; raises AssertionError with the rule
    that is broken.  The three mandatory methods, the ``__init__(in_features: int, out_features: int, config)``
    signature, ``define_parameters`` taking a subset of those and returning Tensor(s), the optional
    ``weight_computation`` mapping exactly those Tensors to Tensor(s), ``weight_application(x: Tensor, ...)
    -> Tensor`` over them, ``post_computation(Tensor) -> Tensor``."""
    for name in ("define_parameters", "weight_application", "post_computation"):
        assert hasattr(adapter_class, name), f"{name} method must be defined."
    has_wc = hasattr(adapter_class, "weight_computation")

    init = _hints(adapter_class.__init__)
    assert init.get("in_features") is int, "__init__ must take `in_features: int` as input"
    assert init.get("out_features") is int, "__init__ must take `out_features: int` as input"
    assert "config" in init, "__init__ must take `config: <Adapter>Config` as input"

    dp = _hints(adapter_class.define_parameters)
    assert "return" in dp, "define_params must indicate the return type with `-> <return_type>`"
    dp_ret = dp.pop("return")
    assert dp.items() <= init.items(), "define_params inputs must be a subset of __init__'s inputs"
    ok, n_params = _tensors_with_count(dp_ret)
    assert ok, "define_params must return a Tensor (`-> Tensor`) or a tuple of Tensors (`-> tuple[Tensor, ...]`)"

    n_applied = n_params
    if has_wc:
        wc = _hints(adapter_class.weight_computation)
        assert "return" in wc, "weight_computation must indicate the return type with `-> <return_type>`"
        wc_ret = wc.pop("return")
        assert len(wc) == n_params and all(t is Tensor for t in wc.values()), \
            "weight_computation must have exactly the input that define_params returns"
        ok, n_applied = _tensors_with_count(wc_ret)
        assert ok, "weight_computation must return a Tensor (`-> Tensor`) or a tuple of Tensors (`-> tuple[Tensor, ...]`)"

    wa = _hints(adapter_class.weight_application)
    assert wa.get("return") is Tensor, "weight_application must return a Tensor and indicate it with `-> Tensor`"
    wa.pop("return")
    assert wa.get("x") is Tensor, "weight_application must have `x: Tensor` as the first input argument"
    wa.pop("x")
    src = "weight_computation" if has_wc else "define_params"
    assert len(wa) == n_applied and all(t is Tensor for t in wa.values()), \
        f"weight_application must have as input what {src} returns"

    pc = _hints(adapter_class.post_computation)
    assert pc.get("return") is Tensor, "post_computation must return a Tensor and indicate it with `-> Tensor`"
    pc.pop("return")
    assert len(pc) == 1 and list(pc.values())[0] is Tensor, "post_computation must have a single Tensor as input"
    return has_wc, n_params


# ---- the reference's own example, written against the stand-ins (lora.py:5-24) -------------------------------------
@dataclasses.dataclass(frozen=True)
class LoraConfig:
    r: int
    alpha: float


class Lora(nn.Module):
    def __init__(self, in_features: int, out_features: int, config: LoraConfig):
        super().__init__()
        self.scaling = config.alpha / config.r

    def define_parameters(self, in_features: int, out_features: int, config: LoraConfig) -> tuple[Tensor, Tensor]:
        return nn.Parameter((in_features, config.r), "float16"), nn.Parameter((config.r, out_features), "float16")

    def weight_application(self, x: Tensor, lora_A: Tensor, lora_B: Tensor) -> Tensor:
        return op.matmul(op.matmul(x, lora_A), lora_B)

    def post_computation(self, y: Tensor) -> Tensor:
        return y * self.scaling


# ---- probing and lowering -------------------------------------------------------------------------------------
@dataclasses.dataclass
class Family:
    """What the probes established about (class, in_features, out_features, config)."""
    adapter_class: type
    instance: object
    has_weight_computation: bool
    param_shapes: list          # declared parameter shapes (without the adapter axis)
    rank: int                   # inner dimension of the pair
    scale: float                # the constant post_computation multiplies by

    def lower(self, params):
        """Declared parameters of ONE adapter -> ``(A [r, in], B [out, r])`` float32 (weight_computation applied)."""
        params = [torch.as_tensor(p, dtype=torch.float32) for p in params]
        for p, shp in zip(params, self.param_shapes):
            if list(p.shape) != shp:
                raise ValueError(f"parameter of shape {list(p.shape)} where {self.adapter_class.__name__} declares {shp}")
        if self.has_weight_computation:
            out = self.instance.weight_computation(*params)
            params = list(out) if isinstance(out, (tuple, list)) else [out]
        p0, p1 = params
        return p0.t().contiguous(), p1.t().contiguous()


_FAMILIES: dict = {}
_REGISTRY: dict = {LoraConfig: Lora}


def register_adapter(config_type, adapter_class):
    """Associates a config dataclass with the adapter class it configures (the reference hard-wires
    ``LoraConfig`` -> ``Lora`` at compile_tvm.py:331); validates the class first."""
    verify_adapter_def(adapter_class)
    _REGISTRY[config_type] = adapter_class


def adapter_class_for(config):
    for t, cls in _REGISTRY.items():
        if isinstance(config, t) or (type(config).__name__ == t.__name__ and hasattr(config, "r")):
            return cls
    raise UnsupportedAdapter(f"no adapter class registered for config type {type(config).__name__}")


def probe_family(adapter_class, in_features: int, out_features: int, config, seed: int = 0) -> Family:
    """Validates the class, then runs its methods on random float32 tensors to establish the family."""
    key = (adapter_class, in_features, out_features, repr(config))
    if key in _FAMILIES:
        return _FAMILIES[key]
    has_wc, n_params = verify_adapter_def(adapter_class)
    inst = adapter_class(in_features, out_features, config)
    dp_args = {k: v for k, v in (("in_features", in_features), ("out_features", out_features), ("config", config))
               if k in _hints(adapter_class.define_parameters)}
    specs = inst.define_parameters(**dp_args)
    specs = list(specs) if isinstance(specs, (tuple, list)) else [specs]
    if len(specs) != n_params:
        raise UnsupportedAdapter(f"define_parameters returned {len(specs)} parameters, its annotation says {n_params}")
    g = torch.Generator().manual_seed(seed)
    raw = [torch.randn(*s.shape, generator=g) for s in specs]
    applied = raw
    if has_wc:
        out = inst.weight_computation(*raw)
        applied = list(out) if isinstance(out, (tuple, list)) else [out]
    if len(applied) != 2:
        raise UnsupportedAdapter(f"{adapter_class.__name__}: weight_application takes {len(applied)} tensors; the kernels "
                                 "implement the two-factor form (x @ P0) @ P1")
    p0, p1 = applied
    if p0.dim() != 2 or p1.dim() != 2 or p0.shape[0] != in_features or p1.shape[1] != out_features or p0.shape[1] != p1.shape[0]:
        raise UnsupportedAdapter(f"{adapter_class.__name__}: factors of shapes {list(p0.shape)} and {list(p1.shape)} are not "
                                 f"[{in_features}, r] and [r, {out_features}]")
    x = torch.randn(5, in_features, generator=g)
    got = inst.weight_application(x, p0, p1)
    want = (x @ p0) @ p1
    if got.shape != want.shape or not torch.allclose(got, want, rtol=1e-4, atol=1e-4 * float(want.abs().max())):
        raise UnsupportedAdapter(f"{adapter_class.__name__}: weight_application is not (x @ P0) @ P1 on a random probe")
    y = torch.randn(4, out_features, generator=g)
    z1, z2, z0 = inst.post_computation(y), inst.post_computation(2.0 * y), inst.post_computation(torch.zeros_like(y))
    c = float((z1 * y).sum() / (y * y).sum())
    tol = 1e-5 * max(1.0, abs(c))
    if (z0.abs().max() > tol or not torch.allclose(z1, c * y, rtol=1e-5, atol=tol)
            or not torch.allclose(z2, 2.0 * c * y, rtol=1e-5, atol=2 * tol)):
        raise UnsupportedAdapter(f"{adapter_class.__name__}: post_computation is not multiplication by a constant")
    fam = Family(adapter_class, inst, has_wc, [s.shape for s in specs], int(p0.shape[1]), c)
    _FAMILIES[key] = fam
    return fam


def lower_adapter_file(tensors: dict, config, cfg_model: dict, adapter_class=None):
    """An adapter file of the reference's on-disk form (``layers.{L}.{block}.{proj}.lora_A/lora_B.weight``,
    A [r, in], B [out, r]: init_peft_weights/lora_weights.py:18-23; further parameters of a class with more
    than two as ``...p2.weight``, ``...p3.weight``) -> ``(same keys with the lowered A / B, scale)``.
    The reference feeds ``lora_A^T`` / ``lora_B^T`` as the class's p0 / p1 (compile_tvm.py:309-312)."""
    cls = adapter_class or adapter_class_for(config)
    out, scale = {}, None
    prefixes = sorted({k[: k.index(".lora_A.weight")] for k in tensors if k.endswith(".lora_A.weight")})
    for pre in prefixes:
        A, B = tensors[pre + ".lora_A.weight"], tensors[pre + ".lora_B.weight"]
        fam = probe_family(cls, int(A.shape[1]), int(B.shape[0]), config)
        params = [A.float().t(), B.float().t()]
        i = 2
        while pre + f".p{i}.weight" in tensors:
            params.append(tensors[pre + f".p{i}.weight"].float())
            i += 1
        a_low, b_low = fam.lower(params)
        out[pre + ".lora_A.weight"], out[pre + ".lora_B.weight"] = a_low.to(A.dtype), b_low.to(B.dtype)
        if scale is not None and abs(scale - fam.scale) > 1e-6 * max(1.0, abs(scale)):
            raise UnsupportedAdapter("post_computation constants differ between projections of one adapter")
        scale = fam.scale
    return out, scale
