"""Auto-batching front-end on top of :class:`vm.B200VM`.

Re-hosts the user-facing API of ``tvm/llama_auto_batcher/llama_auto_batcher.py`` (``create_var``,
``set_adapter``, ``generate``, ``print``, ``compile``, ``execute`` and the ``set_*`` configuration
calls, ``:29-136``) so that a script written like ``user_example.py:4-42`` / ``main.py:24-44`` runs
unchanged against the B200 kernels:

* a bipartite variable / operation graph is recorded while the user script runs
  (``exec_graph.py:3-42``); each ``generate`` adds ``encode_prompt -> prefill -> decode ->
  decode_answer`` for one sequence (``llama_auto_batcher.py:58-84``);
* ``compile`` merges all batchable operations ("decode") that sit on the same breadth-first level
  into one node (``exec_graph.py:85-107``) and loads the packed model;
* ``execute`` walks the levels and runs the nodes: per-sequence prefill and the batched greedy decode
  loop of ``llama_exec_graph.py:58-141`` (order the batch by adapter, pick the decode function by
  adapter types present, drop sequences that hit EOS or their own length limit, restore the original
  order at the end).

Differences: levels are ordered lists, not Python sets, so the execution order is deterministic; the
model comes from an in-memory state dict plus adapter files in the reference's on-disk format
(:mod:`adapters`) instead of a HuggingFace cache directory; TVM is replaced by :mod:`vm`.
"""
from __future__ import annotations

import dataclasses
import os

import numpy as np
import torch

from . import adapter_contract
from . import adapters as adapter_files
from . import vm as mvm
from .adapter_contract import LoraConfig  # same fields as tvm/llama_auto_batcher/lora.py:5-8
from .model import PackedLlama
from .seq_info import LlamaSeqInfo


@dataclasses.dataclass
class LlamaExecConfig:
    """Same fields as ``tvm/llama_auto_batcher/llama_exec_graph.py:10-14``."""
    max_prompt_len: int
    max_gen_len: int
    page_size: int


# ------------------------------------------------------------------------------------------------------
class _Var:
    def __init__(self, vid, value):
        self.id, self.var, self.ops = vid, value, []


class _Op:
    def __init__(self, op_type):
        self.op_type = op_type
        self.input_vars, self.output_vars, self.seqids = [], [], []


class ExecGraph:
    """Variables and operations, walked level by level from the source variables."""

    def __init__(self, batchable_op_types):
        self.sources, self.op_nodes = [], []
        self.batchable_op_types = list(batchable_op_types)
        self._next_id = 0

    def variable(self, value, source):
        v = _Var(self._next_id, value)
        self._next_id += 1
        if source:
            self.sources.append(v)
        return v

    def operation(self, input_var, op_type, seqid=None, output_var=None):
        op = _Op(op_type)
        input_var.ops.append(op)
        op.input_vars.append(input_var)
        if output_var is not None:
            op.output_vars.append(output_var)
        if seqid is not None:
            op.seqids.append(seqid)
        self.op_nodes.append(op)
        return op

    def levels(self):
        """Alternating levels of variables and operations (each node once, in first-seen order)."""
        frontier, out = list(self.sources), []
        while frontier:
            out.append(frontier)
            nxt, seen = [], set()
            for node in frontier:
                for child in (node.ops if isinstance(node, _Var) else node.output_vars):
                    if id(child) not in seen:
                        seen.add(id(child))
                        nxt.append(child)
            frontier = nxt
        return out

    def get_max_batch_sizes(self):
        sizes = {}
        for op in self.op_nodes:
            if op.op_type in self.batchable_op_types:
                sizes[op.op_type] = max(sizes.get(op.op_type, 0), len(op.input_vars))
        return sizes

    def fuse_batchable_ops(self):
        """All operations of a batchable type on one level become one operation; the merged ones are
        unhooked from their input variables, which now feed the survivor."""
        for level in self.levels():
            if not level or isinstance(level[0], _Var):
                continue
            keep = {}
            for op in level:
                if op.op_type not in self.batchable_op_types:
                    continue
                first = keep.setdefault(op.op_type, op)
                if first is op:
                    continue
                first.input_vars += op.input_vars
                first.output_vars += op.output_vars
                first.seqids += op.seqids
                for v in op.input_vars:
                    v.ops[v.ops.index(op)] = first
                self.op_nodes.remove(op)

    def execute_op(self, op):  # overridden
        raise NotImplementedError

    def execute(self):
        for level in self.levels():
            if level and isinstance(level[0], _Op):
                for op in level:
                    self.execute_op(op)

    def describe(self):
        lines = []
        for level in self.levels():
            if isinstance(level[0], _Var):
                lines.append(" ".join(f"Var(id={v.id})" for v in level))
            else:
                lines += [f"Op(type={o.op_type}, seqids={o.seqids}, in_ids={[v.id for v in o.input_vars]}, "
                          f"out_ids={[v.id for v in o.output_vars]})" for o in level]
        return "\n".join(lines)


class LlamaExecGraph(ExecGraph):
    def __init__(self, batchable_op_types=("decode",)):
        super().__init__(batchable_op_types)
        self.kv_cache = None
        self.decode_steps = 0

    def set_exec_vars(self, vm, dev, params, tokenizer, seq_info, exec_config):
        self.vm, self.dev, self.params = vm, dev, params
        self.tokenizer, self.seq_info, self.exec_config = tokenizer, seq_info, exec_config
        self.set_kv_cache()

    def set_kv_cache(self):
        n = self.seq_info.get_num_sequences()
        c = self.exec_config
        self.kv_cache = self.vm["create_paged_kv_cache"](
            mvm.ShapeTuple([n]), mvm.ShapeTuple([n * (c.max_prompt_len + c.max_gen_len)]),
            mvm.ShapeTuple([c.max_prompt_len]), mvm.ShapeTuple([c.page_size]))

    # -- node types ------------------------------------------------------------------------------------------
    def execute_op(self, op):
        handler = {"encode_prompt": self._encode_prompt, "prefill": self._prefill, "decode": self._decode,
                   "decode_answer": self._decode_answer, "print": self._print}.get(op.op_type)
        if handler is None:
            print(f"[ERROR] unknown op_type: {op.op_type}")
            return
        handler(op)

    @staticmethod
    def _single(op, what, outputs=1):
        assert len(op.input_vars) == 1, f"{what} node must have exactly 1 input var but has {len(op.input_vars)}"
        assert len(op.output_vars) == outputs, f"{what} node must have exactly {outputs} output var but has {len(op.output_vars)}"
        assert len(op.seqids) == 1, f"{what} node must have exactly 1 seqid but has {len(op.seqids)}"

    def _encode_prompt(self, op):
        self._single(op, "encode_prompt")
        op.output_vars[0].var = self.tokenizer(op.input_vars[0].var, return_tensors="pt")["input_ids"]

    def _prefill(self, op):
        self._single(op, "prefill")
        sid, tokens = op.seqids[0], op.input_vars[0].var
        gf = mvm.get_global_func
        tokens_dev = mvm.array(np.asarray(tokens, dtype="int32"), self.dev)
        gf("vm.builtin.kv_state_add_sequence")(self.kv_cache, sid)
        hidden = self.vm["embed"](tokens_dev, self.params)
        ad = self.seq_info.get_adapter_info(sid)
        gf("vm.builtin.kv_state_begin_forward")(self.kv_cache, mvm.ShapeTuple([sid]), mvm.ShapeTuple([tokens.shape[1]]))
        if ad is None:
            logits, self.kv_cache = self.vm["prefill_no_adapter"](hidden, self.kv_cache, self.params)
        else:
            wid = mvm.array(np.asarray([ad["wid"]], dtype="int32"), self.dev)
            logits, self.kv_cache = self.vm[f"prefill_a{ad['tid']}"](hidden, self.kv_cache, wid, self.params)
        gf("vm.builtin.kv_state_end_forward")(self.kv_cache)
        op.output_vars[0].var = int(np.argmax(logits.numpy()))

    def _unfinished(self, live, outputs):
        eos = getattr(self.tokenizer, "eos_token_id", None)
        return [s for s in live if outputs[s][-1] != eos and len(outputs[s]) < self.seq_info.get_max_gen_len(s)]

    # ``device_loop`` (default): the batch state of a decode node lives on the device (model.DecodeSession): the
    # batch is ordered once with the device bucket sort, every step is a CUDA-graph replay, finished sequences leave
    # inside the step, and the host reads 4 bytes per ``sync_every`` steps plus all tokens once at the end.
    # ``device_loop = False`` runs the reference's host loop below, step for step (kept as the checked slow path).
    device_loop = True
    sync_every = 1

    def _decode_on_device(self, op):
        from .model import DecodeSession
        live, positions = self.seq_info.order_seqs(op.seqids)
        slots = [self.vm.slot_of(self.seq_info.get_adapter_info(s)) for s in live]
        first = [int(op.input_vars[positions[i]].var) for i in range(len(live))]
        max_gen = [self.seq_info.get_max_gen_len(s) for s in live]
        sess = DecodeSession(self.vm.engine_for(self.kv_cache), live, slots, first, max_gen,
                             getattr(self.tokenizer, "eos_token_id", None), use_lora=any(s >= 0 for s in slots))
        outs = sess.run(self.sync_every)
        self.decode_steps += sess.steps
        self.decode_d2h_bytes = getattr(self, "decode_d2h_bytes", 0) + sess.d2h_bytes
        for i in range(len(live)):
            op.output_vars[positions[i]].var = torch.tensor(outs[i])

    def _decode(self, op):
        assert len(op.input_vars) == len(op.output_vars) == len(op.seqids), "decode node: inputs, outputs and seqids differ"
        if self.device_loop and isinstance(self.vm, mvm.B200VM):
            return self._decode_on_device(op)
        gf = mvm.get_global_func
        live, positions = self.seq_info.order_seqs(op.seqids)
        outputs = {sid: [op.input_vars[positions[i]].var] for i, sid in enumerate(live)}
        ordered = list(live)
        while live:
            tok = mvm.array(np.array([[outputs[s][-1]] for s in live]).astype("int32"), self.dev)
            hidden = self.vm["embed"](tok, self.params)
            name, plist = self.seq_info.get_decode_method(live)
            plist = [mvm.array(np.asarray(ids, dtype="int32"), self.dev) for ids in plist]
            gf("vm.builtin.kv_state_begin_forward")(self.kv_cache, mvm.ShapeTuple(live), mvm.ShapeTuple([1] * len(live)))
            logits, self.kv_cache = self.vm[name](hidden, self.kv_cache, *plist, self.params)
            gf("vm.builtin.kv_state_end_forward")(self.kv_cache)
            self.decode_steps += 1
            lg = logits.numpy()
            for i, s in enumerate(live):
                outputs[s].append(int(np.argmax(lg[i])))
            live = self._unfinished(live, outputs)
        for i, sid in enumerate(ordered):
            op.output_vars[positions[i]].var = torch.tensor(outputs[sid])

    def _decode_answer(self, op):
        self._single(op, "decode_answer")
        op.output_vars[0].var = self.tokenizer.decode(op.input_vars[0].var)

    def _print(self, op):
        assert len(op.input_vars) == 1 and len(op.seqids) == 1, "print node must have exactly 1 input var and 1 seqid"
        print(f"Answer for Sequence {op.seqids[0]} {op.input_vars[0].var}")


# ------------------------------------------------------------------------------------------------------
class LlamaAutoBatcherClass:
    """The recorder / driver object; ``LlamaAutoBatcher`` below is the module-level instance scripts use."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.graph = LlamaExecGraph()
        self.current = {"sid": -1, "generated": True}
        self.device = torch.device("cuda", 0)
        self.model_config = None
        self.weights = None
        self.adapter_dir = None
        self.adapter_targets = ("q_proj", "v_proj")
        self.tokenizer = None
        self.exec_config = LlamaExecConfig(max_prompt_len=512, max_gen_len=32, page_size=16)
        self.seq_info = LlamaSeqInfo(self.exec_config.max_gen_len, self.device)
        self.vm = None

    # -- configuration (llama_auto_batcher.py:29-51) ---------------------------------------------------------
    def set_device(self, device):
        self.device = torch.device(device)
        self.seq_info.device = self.device

    def set_model_config(self, model_config):
        self.model_config = dict(model_config)

    def set_weights(self, state_dict):
        """HF-named state dict of the base model (stands in for the cache_dir + from_pretrained)."""
        self.weights = state_dict

    def set_cache_dir(self, cache_dir):
        """Directory holding ``lora_adapters/r{rank}_a{id}.safetensors`` (compile_tvm.py:302)."""
        self.adapter_dir = os.path.join(cache_dir, "lora_adapters")

    def set_tokenizer(self, tokenizer):
        self.tokenizer = tokenizer

    def set_exec_config(self, exec_config):
        self.seq_info.update_max_gen_len(exec_config.max_gen_len)
        self.exec_config = exec_config

    # -- recording (llama_auto_batcher.py:53-96) ------------------------------------------------------------
    def create_var(self, var, source=True):
        return self.graph.variable(var, source)

    def _ensure_sequence(self, generated_flag):
        if self.current["generated"]:
            self.current["sid"] += 1
            self.seq_info.add_sequence(self.current["sid"])
        self.current["generated"] = generated_flag

    def set_adapter(self, config, wid):
        if self.current["generated"]:
            self._ensure_sequence(False)
        self.seq_info.set_adapter(self.current["sid"], config, wid)

    def generate(self, input_var, max_gen_len=None):
        self._ensure_sequence(True)
        sid = self.current["sid"]
        self.seq_info.set_max_gen_len(sid, max_gen_len)
        v = input_var
        for op_type in ("encode_prompt", "prefill", "decode", "decode_answer"):
            out = self.create_var(None, False)
            self.graph.operation(v, op_type, seqid=sid, output_var=out)
            v = out
        return v

    def print(self, var):
        self.graph.operation(var, "print", seqid=self.current["sid"])

    # -- compile / execute (llama_auto_batcher.py:98-136) --------------------------------------------------------
    def compile(self, fuse_decode=True):
        if fuse_decode:
            self.graph.fuse_batchable_ops()
        configs = self.seq_info.get_adapter_configs()
        wids = self.seq_info.get_wids_per_type()
        adapters, scales, base = [], [], []
        for t, cfg in enumerate(configs):
            base.append(len(adapters))
            for wid in range(max(wids[t]) + 1 if wids[t] else 0):
                # the raw weight id indexes the type's stack (compile_tvm.py:298-313): ids are dense per type
                path = adapter_files.adapter_path(self.adapter_dir, cfg.r, wid)
                # the config's adapter class is validated and probed (adapter_contract), its optional
                # weight_computation runs here, once, and its post_computation constant becomes the scale
                lowered, scale = adapter_contract.lower_adapter_file(adapter_files.load_adapter(path), cfg, self.model_config)
                adapters.append(lowered)
                scales.append(scale)
        model = PackedLlama(self.model_config, self.weights, adapters, scales, device=self.device)
        self.vm = mvm.B200VM(model, type_slot_base=base or [0])
        self.graph.set_exec_vars(self.vm, self.device, self.vm.params, self.tokenizer, self.seq_info, self.exec_config)

    def execute(self):
        self.graph.execute()


LlamaAutoBatcher = LlamaAutoBatcherClass()
