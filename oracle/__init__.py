"""CPU oracle for the multi-LoRA decode hot path.  TEST INFRASTRUCTURE ONLY.

Nothing here is part of the product: the shipped package never imports this
directory.  It may be imported only by the tests, by the smoke check and by
the benchmark's CPU-baseline / reference legs, and there only as the checker
(or as the timed CPU baseline), never as the thing that produces results for
a user.

Each function restates, in plain numpy / torch-fp32 on the CPU, one piece of
the reference algorithm and cites the reference file:line it follows.

Pinning status
--------------
* bucketing (``oracle.bucketing``): pinned bit-exactly against outputs of the
  reference's own ``tvm/llama_auto_batcher/llama_seq_info.py`` and
  ``exec_graph.py`` (golden file ``tests/golden/bucketing_golden.json``).
* GatherBMM LoRA layer (``oracle.ops.gather_bmm_linear``): pinned against
  outputs of the reference's own ``GatherBMMLinear.forward`` executed over a
  stand-in for its third-party peft base class
  (``tests/golden/lora_layer_golden.npz``).
* paged-KV attention, RoPE, RMSNorm and the decoder body: the reference
  delegates these to TVM v0.18 ``TIRPagedKVCache`` / transformers, neither of
  which is vendored, and ships no golden vectors for them -> parity unpinned
  at those boundaries; the oracle is cross-checked against the transformers
  ``LlamaForCausalLM`` installed here (``tests/test_oracle_model.py``).
"""
