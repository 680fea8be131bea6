"""``import bastile`` resolves to this package under the reference's import name
(src/bastile/__init__.py:18-33); the import lines below are those of the reference's own
tests and benchmarks (tests/ops/test_*.py, tests/benchmarks/kernel/*.py), unmodified."""

import inspect


def test_reference_import_lines_run_unmodified():
    import bastile
    from bastile.ops.fused_linear_cross_entropy import fused_linear_cross_entropy
    from bastile.ops.fused_linear_cross_entropy import fused_linear_cross_entropy as bastile_lce  # noqa: F401
    from bastile.ops.fused_linear_cross_entropy import warmup_fused_lce  # noqa: F401
    from bastile.ops.rms_norm import rms_norm
    from bastile.ops.rms_norm import rms_norm as cutile_rms_norm  # noqa: F401
    from bastile.ops.rope import apply_rotary_pos_emb
    from bastile.ops.rope import apply_rotary_pos_emb as bastile_rope  # noqa: F401
    from bastile.ops.swiglu import SwiGLUFunction
    from bastile.ops.swiglu import swiglu as cutile_swiglu  # noqa: F401

    import bastile_b200
    from bastile_b200.ops import rms_norm as impl_rms

    assert bastile.apply is bastile_b200.apply and bastile.reset is bastile_b200.reset
    assert rms_norm is impl_rms.rms_norm
    assert set(bastile.__all__) == {"apply", "apply_to_model", "clear_autotune_cache", "get_patched_ops",
                                    "list_patches", "register_patch", "reset", "warmup_all_kernels"}
    for fn in (fused_linear_cross_entropy, apply_rotary_pos_emb, SwiGLUFunction.apply):
        assert callable(fn)
    # the reference's keyword surface of the fused loss (:405-414)
    params = list(inspect.signature(fused_linear_cross_entropy).parameters)
    assert params[:8] == ["hidden_states", "weight", "target", "bias", "ignore_index", "chunk_size", "reduction",
                          "v_chunk_size"]


def test_alias_shares_one_registry():
    import bastile
    import bastile.core
    import bastile.registry

    import bastile_b200.registry

    assert bastile.registry is bastile_b200.registry
    assert bastile.list_patches() == bastile_b200.list_patches() and "rms_norm_qwen3" in bastile.list_patches()
