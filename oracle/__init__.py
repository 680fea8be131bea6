"""CPU oracle for the four Qwen3 hot-path ops.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain numpy, the arithmetic of the reference's ops
(aghilann/bastile, src/bastile/ops/*.py) so that the CUDA kernels can be checked
against it.  Nothing in ``bastile_b200`` imports it: only ``tests/``, the smoke
check and the CPU-baseline leg of the benchmark may.

Pinning: the reference's device kernels are CuTile JIT kernels that need a GPU
and the ``tileiras`` compiler (CUDA >= 13.1), neither of which exists where this
oracle was written, so they cannot be executed.  The oracle is pinned instead
against (a) the reference's own pure-torch implementation of the fused loss
(``_v_chunked_fwd`` through ``fused_linear_cross_entropy(..., v_chunk_size=)``,
src/bastile/ops/fused_linear_cross_entropy.py:198-298), executed on CPU,
(b) the HuggingFace eager modules the patches replace (``Qwen3RMSNorm``,
``apply_rotary_pos_emb``, ``Qwen3MLP``), which is what the reference's unit tests
compare with, and (c) the reference's patch engine run on CPU.  The outputs of
those runs are the committed fixtures under ``tests/golden/`` (made by
``tests/golden/make_golden.py``).  The reference's RoPE forward values have no
test of their own (tests/ops/test_rope.py:32-38 is skipped): HF eager is the
only pin for them.
"""

from .ops import (  # noqa: F401
    adamw_step,
    add_rms_norm_bwd,
    add_rms_norm_fwd,
    head_norm_rope_bwd,
    head_norm_rope_fwd,
    lce_fwd_bwd,
    lce_shard_stats,
    merge_shard_stats,
    mlp_bwd,
    mlp_fwd,
    rms_norm_bwd,
    rms_norm_fwd,
    rope,
    swiglu_bwd,
    swiglu_fwd,
)
