"""bt_set_dependent_launch: kernels launched as programmatic dependents of their predecessors
(the default) give bit-identical results to ordinary launches, over a chain of the library's ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _chain(seed):
    """RMSNorm -> SwiGLU MLP -> add + RMSNorm -> AdamW on the weights, forward and backward."""
    from bastile_b200.ops.fused_layers import add_rms_norm
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction
    from bastile_b200.optim import AdamW

    torch.manual_seed(seed)
    rows, hidden, inter = 515, 256, 384
    x = torch.randn(rows, hidden, device=DEV).to(torch.bfloat16).requires_grad_(True)
    w0 = (1 + 0.02 * torch.randn(hidden, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    w1 = (1 + 0.02 * torch.randn(hidden, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    wg = (0.05 * torch.randn(inter, hidden, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    wu = (0.05 * torch.randn(inter, hidden, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    wd = (0.05 * torch.randn(hidden, inter, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    opt = AdamW([w0, w1, wg, wu, wd], lr=1e-2, weight_decay=0.1)
    outs = []
    for _ in range(3):
        h = rms_norm(x, w0, 1e-6)
        m = SwiGLUMLPFunction.apply(h, wg, wu, wd)
        y, stream = add_rms_norm(m, x, w1, 1e-6)
        (y.float().square().mean() + stream.float().mean()).backward()
        outs += [y.detach().clone(), stream.detach().clone(), x.grad.detach().clone()]
        opt.step()
        opt.zero_grad()
        x.grad = None
    torch.cuda.synchronize()
    return outs + [p.detach().clone() for p in (w0, w1, wg, wu, wd)]


def test_switch_returns_previous_value_and_results_are_bit_identical():
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    prev = lib.bt_set_dependent_launch(-1)          # negative: query only
    assert prev in (0, 1) and lib.bt_set_dependent_launch(-1) == prev
    try:
        assert lib.bt_set_dependent_launch(1) == prev
        on = _chain(3)
        assert lib.bt_set_dependent_launch(0) == 1
        off = _chain(3)
        _lib.check_status(torch.device(DEV), "dependent launch off")
    finally:
        lib.bt_set_dependent_launch(prev)
    assert len(on) == len(off)
    for i, (a, b) in enumerate(zip(on, off)):
        assert torch.equal(a, b), f"tensor {i} differs between dependent and ordinary launches"


def test_rope_and_qk_norm_rope_identical_under_both_launch_modes():
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_layers import qk_norm_rope

    lib = _lib.get_lib()
    prev = lib.bt_set_dependent_launch(-1)
    t, d = 130, 128
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), -1)
    cos, sin = emb.cos()[None].to(DEV, torch.bfloat16), emb.sin()[None].to(DEV, torch.bfloat16)
    results = {}
    try:
        for mode in (1, 0):
            lib.bt_set_dependent_launch(mode)
            torch.manual_seed(11)
            q = torch.randn(1, t, 4, d, device=DEV).to(torch.bfloat16).requires_grad_(True)
            k = torch.randn(1, t, 2, d, device=DEV).to(torch.bfloat16).requires_grad_(True)
            wq = (1 + 0.02 * torch.randn(d, device=DEV)).to(torch.bfloat16).requires_grad_(True)
            wk = (1 + 0.02 * torch.randn(d, device=DEV)).to(torch.bfloat16).requires_grad_(True)
            qo, ko = qk_norm_rope(q, k, wq, wk, cos, sin, 1e-6)
            (qo.float().square().sum() + ko.float().sum()).backward()
            torch.cuda.synchronize()
            results[mode] = [t_.detach().clone() for t_ in (qo, ko, q.grad, k.grad, wq.grad, wk.grad)]
    finally:
        lib.bt_set_dependent_launch(prev)
    for a, b in zip(results[1], results[0]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("mode", [1, 0])
def test_launches_capture_into_a_cuda_graph_and_replay(mode):
    """The library's launches (programmatic dependents or ordinary) are captured by torch.cuda.graph
    and a replay on new input data gives the bits of an eager run."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_layers import add_rms_norm
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    lib = _lib.get_lib()
    prev = lib.bt_set_dependent_launch(-1)
    torch.manual_seed(0)
    x = torch.randn(515, 256, device=DEV).to(torch.bfloat16)
    w = (1 + 0.02 * torch.randn(256, device=DEV)).to(torch.bfloat16)
    wg = (0.05 * torch.randn(384, 256, device=DEV)).to(torch.bfloat16)
    wu = (0.05 * torch.randn(384, 256, device=DEV)).to(torch.bfloat16)
    wd = (0.05 * torch.randn(256, 384, device=DEV)).to(torch.bfloat16)

    def chain(inp):
        with torch.no_grad():
            h = rms_norm(inp, w, 1e-6)
            m = SwiGLUMLPFunction.apply(h, wg, wu, wd)
            return add_rms_norm(m, inp, w, 1e-6)

    try:
        lib.bt_set_dependent_launch(mode)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm-up off the capture: scratch, status words, tensor maps
            for _ in range(3):
                chain(x)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = chain(x)
        fresh = torch.randn_like(x)
        want = chain(fresh)
        x.copy_(fresh)
        graph.replay()
        torch.cuda.synchronize()
        _lib.check_all_status()
    finally:
        lib.bt_set_dependent_launch(prev)
    assert torch.equal(out[0], want[0]) and torch.equal(out[1], want[1])
