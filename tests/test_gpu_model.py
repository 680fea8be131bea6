"""Whole-model parity: tiny Qwen3ForCausalLM, HF eager on CPU fp32 (golden fixture) against the
patched model on the GPU in bf16 - loss and every gradient."""

import numpy as np
import pytest
import torch

from conftest import assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def patched():
    import bastile_b200

    bastile_b200.reset()
    applied = bastile_b200.apply()
    yield applied
    bastile_b200.reset()


def test_tiny_qwen3_loss_and_grads_match_hf_eager_fixture(patched):
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_inputs
    from transformers import Qwen3ForCausalLM
    import transformers.models.qwen3.modeling_qwen3 as q3

    from bastile_b200.ops.rms_norm import B200RMSNorm
    from bastile_b200.ops.swiglu import B200SwiGLUMLP

    assert patched == ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3", "fused_linear_cross_entropy"]
    g = load_golden("tiny_qwen3.npz")
    import bastile_b200

    bastile_b200.reset()
    stock = build_tiny_qwen3()  # CPU fp32, seed 0: the weights of the fixture
    bastile_b200.apply()
    from golden.make_golden import tiny_qwen3_config

    model = Qwen3ForCausalLM(tiny_qwen3_config())
    assert isinstance(model.model.norm, B200RMSNorm) and isinstance(model.model.layers[0].mlp, B200SwiGLUMLP)
    assert q3.apply_rotary_pos_emb.__module__.startswith("bastile_b200")
    model.load_state_dict(stock.state_dict())
    model = model.to(DEV, torch.bfloat16).train()
    ids, labels = tiny_qwen3_inputs()
    out = model(input_ids=ids.to(DEV), labels=labels.to(DEV))
    assert out.logits is None  # training path never materialises logits
    out.loss.backward()
    from bastile_b200 import _lib

    _lib.check_status(torch.device(DEV, torch.cuda.current_device()), "tiny model")
    loss_ref = float(g["loss"])
    assert abs(out.loss.item() - loss_ref) <= 5e-3 * loss_ref  # bf16 weights/activations end to end
    names = [str(n) for n in g["names"]]
    grads = dict(model.named_parameters())
    for name, ref_norm in zip(names, g["grad_norms"]):
        gn = grads[name].grad.float().norm().item()
        assert np.isfinite(gn)
        assert abs(gn - ref_norm) <= 0.08 * ref_norm + 1e-4, f"{name}: grad norm {gn} vs {ref_norm}"
    for key in g.files:
        if not key.startswith("grad::"):
            continue
        pname = key[len("grad::"):]
        if pname.endswith("[:64,:64]"):
            got = grads[pname[:-len("[:64,:64]")]].grad[:64, :64]
        else:
            got = grads[pname].grad
        ref = g[key]
        assert_close(got, ref, what=pname, rtol=5e-2, atol=5e-2 * float(np.abs(ref).max()))


def test_tiny_qwen3_fp32_on_gpu_matches_hf_eager_fixture(patched):
    """Same model kept in fp32 on the GPU (tf32 products in the MLP and the fused loss; the
    projections and attention run torch's fp32 kernels): loss within 1e-3, gradients within 2e-2."""
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_config, tiny_qwen3_inputs
    from transformers import Qwen3ForCausalLM

    import bastile_b200

    g = load_golden("tiny_qwen3.npz")
    bastile_b200.reset()
    stock = build_tiny_qwen3()
    bastile_b200.apply()
    model = Qwen3ForCausalLM(tiny_qwen3_config())
    model.load_state_dict(stock.state_dict())
    model = model.to(DEV).train()
    ids, labels = tiny_qwen3_inputs()
    out = model(input_ids=ids.to(DEV), labels=labels.to(DEV))
    out.loss.backward()
    assert abs(out.loss.item() - float(g["loss"])) <= 1e-3 * float(g["loss"])
    grads = dict(model.named_parameters())
    for name, ref_norm in zip([str(n) for n in g["names"]], g["grad_norms"]):
        gn = grads[name].grad.float().norm().item()
        assert abs(gn - ref_norm) <= 2e-2 * ref_norm + 1e-5, f"{name}: grad norm {gn} vs {ref_norm}"
    for key in g.files:
        if key.startswith("grad::") and not key.endswith("[:64,:64]"):
            ref = g[key]
            assert_close(grads[key[6:]].grad, ref, what=key, rtol=2e-2, atol=2e-2 * float(np.abs(ref).max()))


def test_eval_path_returns_logits_like_hf(patched):
    from golden.make_golden import tiny_qwen3_config, tiny_qwen3_inputs
    from transformers import Qwen3ForCausalLM

    torch.manual_seed(0)
    model = Qwen3ForCausalLM(tiny_qwen3_config()).to(DEV, torch.bfloat16).eval()
    ids, labels = tiny_qwen3_inputs()
    with torch.no_grad():
        out = model(input_ids=ids.to(DEV), labels=labels.to(DEV))
    assert out.logits is not None and out.logits.shape == (2, 128, 4096)
    assert torch.isfinite(out.loss)
