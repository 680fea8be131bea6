"""apply()/reset()/get_patched_ops()/registry against the reference's recorded behaviour
(tests/golden/patch_engine.json, produced by running the reference package on CPU)."""

import importlib
import json

import pytest
import torch

import bastile_b200 as bastile
from conftest import GOLDEN


@pytest.fixture()
def qwen3():
    import transformers.models.qwen3.modeling_qwen3 as q3

    bastile.reset()
    yield q3
    bastile.reset()


@pytest.fixture(scope="module")
def golden():
    return json.loads((GOLDEN / "patch_engine.json").read_text())


def test_surface_matches_reference(golden):
    assert sorted(bastile.__all__) == golden["all"]
    assert bastile.__version__ == golden["version"]
    for name in golden["all"]:
        assert callable(getattr(bastile, name))


def test_apply_reset_sequence_matches_reference(qwen3, golden):
    import bastile_b200.ops  # noqa: F401

    assert bastile.list_patches() == golden["list_patches"]
    assert bastile.apply() == golden["apply_default"]
    assert bastile.get_patched_ops() == golden["get_patched_ops_after_apply"]
    assert bastile.apply() == golden["apply_again"]  # idempotent
    assert bastile.reset() == golden["reset_all"]
    assert bastile.get_patched_ops() == golden["get_patched_ops_after_reset"]
    assert bastile.apply(rms_norm=True, swiglu=False, rope=False,
                         fused_linear_cross_entropy=False) == golden["apply_only_rms"]
    assert bastile.reset(["rms_norm_qwen3"]) == golden["reset_named"]
    assert bastile.apply(model_type="llama") == golden["apply_llama"]
    bastile.reset()
    assert bastile.apply(model_type="qwen3", fused_linear_cross_entropy=False) == golden["apply_qwen3_no_lce"]


def test_apply_swaps_and_reset_restores_every_target(qwen3):
    orig = (qwen3.Qwen3RMSNorm, qwen3.Qwen3MLP, qwen3.apply_rotary_pos_emb, qwen3.Qwen3ForCausalLM.forward)
    bastile.apply()
    from bastile_b200.ops.fused_linear_cross_entropy import bastile_lce_forward
    from bastile_b200.ops.rms_norm import B200RMSNorm
    from bastile_b200.ops.rope import apply_rotary_pos_emb
    from bastile_b200.ops.swiglu import B200SwiGLUMLP

    assert qwen3.Qwen3RMSNorm is B200RMSNorm
    assert qwen3.Qwen3MLP is B200SwiGLUMLP
    assert qwen3.apply_rotary_pos_emb is apply_rotary_pos_emb
    assert qwen3.Qwen3ForCausalLM.forward is bastile_lce_forward
    bastile.reset()
    # unlike the reference, reset() also puts the original causal-LM forward back
    assert (qwen3.Qwen3RMSNorm, qwen3.Qwen3MLP, qwen3.apply_rotary_pos_emb,
            qwen3.Qwen3ForCausalLM.forward) == orig


def test_reference_import_names_exist():
    from bastile_b200.ops.fused_linear_cross_entropy import (  # noqa: F401
        bastile_lce_forward, fused_linear_cross_entropy, warmup_fused_lce)
    from bastile_b200.ops.rms_norm import CuTileRMSNorm, rms_norm, warmup_rms_norm  # noqa: F401
    from bastile_b200.ops.rope import RoPEFunction, apply_rotary_pos_emb  # noqa: F401
    from bastile_b200.ops.swiglu import CuTileSwiGLUMLP, SwiGLUFunction, swiglu  # noqa: F401
    from bastile_b200.ops.utils import ceildiv, get_sm_count, next_power_of_2  # noqa: F401

    assert next_power_of_2(12288) == 16384 and next_power_of_2(0) == 1 and ceildiv(7, 2) == 4


def test_replacement_modules_keep_hf_parameter_names(qwen3):
    from golden.make_golden import tiny_qwen3_config

    bastile.apply(fused_linear_cross_entropy=False)
    importlib.reload  # noqa: B018  (patched classes are picked up at construction time)
    from transformers import Qwen3ForCausalLM

    patched = Qwen3ForCausalLM(tiny_qwen3_config())
    bastile.reset()
    stock = Qwen3ForCausalLM(tiny_qwen3_config())
    assert list(patched.state_dict()) == list(stock.state_dict())
    assert {k: v.shape for k, v in patched.state_dict().items()} == {k: v.shape for k, v in stock.state_dict().items()}
    assert patched.model.norm.variance_epsilon == stock.model.norm.variance_epsilon
    stock.load_state_dict(patched.state_dict())


def test_mlp_rejects_other_activations():
    from golden.make_golden import tiny_qwen3_config
    from bastile_b200.ops.swiglu import B200SwiGLUMLP

    cfg = tiny_qwen3_config()
    cfg.hidden_act = "gelu"
    with pytest.raises(ValueError):
        B200SwiGLUMLP(cfg)


def test_ops_refuse_cpu_tensors():
    """There is no CPU path: CPU tensors raise instead of silently computing somewhere else."""
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.swiglu import swiglu

    with pytest.raises(RuntimeError, match="CUDA"):
        rms_norm(torch.randn(4, 64), torch.ones(64))
    with pytest.raises(RuntimeError, match="CUDA"):
        swiglu(torch.randn(4, 64), torch.randn(4, 64))


def test_warmup_is_silent_without_cuda():
    if not torch.cuda.is_available():
        assert bastile.warmup_all_kernels() is None
    bastile.clear_autotune_cache()


def test_register_patch_and_registry_roundtrip():
    from bastile_b200.registry import PatchRegistry

    reg = PatchRegistry()
    reg.register("a_x", "d", "math", "floor", replacement=len, priority=1, models=["m1"])
    reg.register("b_x", "d", "math", "ceil", replacement=len, has_backward=False, priority=5)
    assert reg.list_all() == ["a_x", "b_x"]
    assert reg.list_with_backward() == ["a_x"]
    assert [p.name for p in reg.get_for_model("m1")] == ["b_x", "a_x"]
    assert [p.name for p in reg.get_for_model("other")] == ["b_x"]
    reg.mark_applied("a_x", original=abs)
    assert reg.get_applied() == ["a_x"] and reg.get("a_x").original is abs
    reg.mark_reset("a_x")
    assert reg.get_applied() == [] and reg.get("missing") is None


def test_fused_layers_are_opt_in_and_reset_restores_the_hf_forwards(qwen3):
    """apply() alone leaves Qwen3DecoderLayer.forward / Qwen3Attention.forward untouched (the
    reference patches neither); fused_layers=True replaces both and every form of reset() that
    names them, or names nothing, puts the originals back."""
    from bastile_b200.ops import fused_layers

    hf_layer, hf_attn = qwen3.Qwen3DecoderLayer.forward, qwen3.Qwen3Attention.forward
    bastile.apply()
    assert qwen3.Qwen3DecoderLayer.forward is hf_layer and qwen3.Qwen3Attention.forward is hf_attn
    bastile.reset()

    applied = bastile.apply(fused_layers=True)
    assert applied == ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3", "decoder_layer_qwen3", "attention_qwen3",
                       "fused_linear_cross_entropy"]
    assert qwen3.Qwen3DecoderLayer.forward is fused_layers.decoder_layer_forward
    assert qwen3.Qwen3Attention.forward is fused_layers.attention_forward
    assert bastile.apply(fused_layers=True) == applied  # idempotent
    assert bastile.get_patched_ops() == ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3"]  # registry patches only
    bastile.reset(["attention_qwen3"])
    assert qwen3.Qwen3Attention.forward is hf_attn
    assert qwen3.Qwen3DecoderLayer.forward is fused_layers.decoder_layer_forward
    bastile.reset()
    assert qwen3.Qwen3DecoderLayer.forward is hf_layer and fused_layers.installed() == []

    # without the norm patch there is nothing to fuse into; without RoPE only the layer forward goes in
    assert "decoder_layer_qwen3" not in bastile.apply(fused_layers=True, rms_norm=False)
    bastile.reset()
    applied = bastile.apply(fused_layers=True, rope=False)
    assert "decoder_layer_qwen3" in applied and "attention_qwen3" not in applied
    bastile.reset()
    with pytest.raises(ValueError):
        fused_layers.install(qwen3, projections="sometimes")


def test_fused_forwards_fall_back_to_plain_modules_on_cpu(qwen3):
    """A model built BEFORE apply() keeps HF's own norm / MLP modules; the fused layer forward
    must then behave exactly like HF's (here on CPU, where none of the kernels can run; the RoPE
    patch is a module-level function that has no CPU form, so it stays off)."""
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_inputs

    model = build_tiny_qwen3().eval()  # HF modules inside
    ids, _ = tiny_qwen3_inputs()
    with torch.no_grad():
        want = model(input_ids=ids).logits
    applied = bastile.apply(fused_layers=True, rope=False, fused_linear_cross_entropy=False)
    assert "decoder_layer_qwen3" in applied
    try:
        with torch.no_grad():
            got = model(input_ids=ids).logits
    finally:
        bastile.reset()
    assert torch.equal(got, want)


def test_two_output_inplace_function_on_views_cannot_mark_dirty():
    """Why RoPEFunction mutates q and k without ``ctx.mark_dirty`` (as the reference does,
    src/bastile/ops/rope.py:125-130): HF passes transposed views, and torch rejects a Function
    that modifies view inputs in place and returns two tensors.  If this ever stops raising,
    RoPEFunction can mark its inputs dirty."""
    import torch

    class TwoInPlace(torch.autograd.Function):
        @staticmethod
        def forward(ctx, q, k):
            q.mul_(2.0)
            k.mul_(2.0)
            ctx.mark_dirty(q, k)
            return q, k

        @staticmethod
        def backward(ctx, dq, dk):
            return dq * 2.0, dk * 2.0

    lin = torch.nn.Linear(8, 16)
    h = torch.randn(1, 4, 8)
    q = lin(h).view(1, 4, 2, 8).transpose(1, 2)
    k = lin(h).view(1, 4, 2, 8).transpose(1, 2)
    with pytest.raises(RuntimeError, match="cannot return more than one Tensor"):
        TwoInPlace.apply(q, k)
