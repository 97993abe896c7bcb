"""tcgen05 grouped products: against the CPU oracle (2e-2) and, buffer by buffer,
against the SIMT products run on the same BF16 data."""
import numpy as np
import pytest
import torch

from mgpt_b200 import synth
from oracle import oracle
from tests.golden import make_golden as G
from tests.util import assert_routing_exact, assert_values, dims_of, rel_l2, run_layer

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2
ACT = ("Xg", "G", "U", "Hh", "Yg", "dYg", "dG", "dU", "dXg")


def _bf16_inputs(w, x, params, dy):
    return synth.bf16_round(x), [synth.bf16_round(p) for p in params], synth.bf16_round(dy)


def _buffers(got, w, blocked_gu=False):
    """Activation buffers as [rows, width].  The tcgen05 path keeps the buffers named G and U as
    [row tile][8-column chunk][128 rows][8] (include/mgpt_moe.h); ``blocked_gu`` undoes that."""
    layer = got["layer"]
    rows = int(got["padded_offsets"][-1])
    out = {}
    for name in ACT:
        width = w.C if name in ("Xg", "Yg", "dYg", "dXg") else w.H
        t = layer.workspace_view(name, torch.bfloat16)
        if blocked_gu and name in ("G", "U"):
            t = t.view(-1, width // 8, 128, 8).permute(0, 2, 1, 3).reshape(-1, width)
        else:
            t = t.view(-1, width)
        out[name] = t[:rows].float().cpu().numpy()
    return out


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_tc_matches_oracle_small(name):
    w, x, params, dy = G.build_case(name)
    x, params, dy = _bf16_inputs(w, x, params, dy)
    ref = oracle.run(dims_of(w), x, params, dy, threads=4)
    got = run_layer(w, x, params, dy, mode="bf16")
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)


@pytest.mark.parametrize("shape", [
    (1000, 256, 384, 8, 2, False),     # several row tiles per expert, full 64-wide k blocks
    (700, 192, 200, 5, 2, False),      # ragged k (200 = 3*64+8) and column tails
    (3000, 128, 96, 16, 4, True),      # skewed: empty and one-row experts next to large ones
    (600, 128, 64, 128, 8, False),     # the largest expert count and top-k the library takes
])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_tc_against_simt_and_oracle(shape, io):
    n, C, H, E, k, skew = shape
    w = synth.Workload("tc", n, C, H, E, k, "bf16", skew=skew)
    x, params, dy = synth.make_inputs(w, seed=11, bias_std=0.02)
    if skew:
        params[0] = synth.bf16_round(params[0] * np.float32(10.0))
    ref = oracle.run(dims_of(w), x, params, dy, threads=16)
    # BF16 tokens also take the tensor-core router backward (dx and gWr); FP32 tokens the CUDA-core one
    tc = run_layer(w, x, params, dy, mode="bf16", io=io)
    assert tc["status"] == 0
    simt = run_layer(w, x, params, dy, mode="bf16", gemm_impl=1, io=io)
    assert_routing_exact(tc, ref)
    a, b = _buffers(tc, w, blocked_gu=True), _buffers(simt, w)
    # the tensor-core path keeps, in the buffers named G and U, what backward needs of them:
    # P = U*sigmoid(G)*(1 + G*(1 - sigmoid(G))) and Q = silu(G)  (include/mgpt_moe.h)
    g64, u64 = b["G"].astype(np.float64), b["U"].astype(np.float64)
    sig = 1.0 / (1.0 + np.exp(-g64))
    b["G"], b["U"] = u64 * sig * (1.0 + g64 * (1.0 - sig)), g64 * sig
    for name in ACT:
        assert rel_l2(a[name], b[name]) < 6e-3, (name, rel_l2(a[name], b[name]))
    for i, (ga, gb) in enumerate(zip(tc["grads"], simt["grads"])):
        assert rel_l2(ga, gb) < 6e-3, (f"grad {i}", rel_l2(ga, gb))
    assert_values(tc, ref, TOL_BF16, w)


def test_tc_c2_reduced_tokens():
    """Config-2 dimensions (C=512, H=1376, E=16, k=2) on 2048 tokens."""
    w = synth.WORKLOADS["c2"].scaled(2048)
    x, params, dy = synth.make_inputs(w)
    ref = oracle.run(dims_of(w), x, params, dy, threads=32)
    got = run_layer(w, x, params, dy, mode="bf16", io=torch.bfloat16)
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)


@pytest.mark.parametrize("n", [8, 64])
def test_tc_decode_shapes_forward_only(n):
    """Config-5 dimensions (C=1024, H=2816, E=32, k=2), one new token per sequence, forward only."""
    w = synth.WORKLOADS["c5-64"].scaled(n)
    x, params, dy = synth.make_inputs(w)
    ref = oracle.run(dims_of(w), x, params, None, threads=32)
    got = run_layer(w, x, params, None, mode="bf16", io=torch.bfloat16)
    assert_routing_exact(got, ref)
    assert rel_l2(got["y"], ref["y"]) <= TOL_BF16


def test_weight_gradients_overwritten_equal_accumulated_into_zero():
    """Stores instead of read-modify-writes: same bits as accumulating into zeroed tensors, stale contents gone,
    experts without rows get zeros; bias and router gradients keep accumulating."""
    w = synth.Workload("ow", 900, 128, 200, 16, 2, "bf16", skew=True)
    x, params, dy = synth.make_inputs(w, seed=13, bias_std=0.02)
    params[1][0, -3:] = np.float32(-64.0)                               # the last three experts stay empty
    acc = run_layer(w, x, params, dy, mode="bf16", io=torch.bfloat16)
    assert (acc["counts"] == 0).any()
    from mgpt_b200 import MoELayer
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16", lb_alpha=w.alpha)
    layer.load_parameters(params)
    for p in layer.get_parameters():
        p.grad.fill_(123.0)                                             # what a forgotten zero_grad leaves behind
    for i in (0, 1):
        layer.get_parameters()[i].grad.zero_()
    for e in range(w.E):
        for j in (1, 3, 5):
            layer.get_parameters()[2 + 6 * e + j].grad.zero_()          # biases accumulate: zeroed by the caller
    layer.set_weight_grad_overwrite(True)
    xt, dyt = torch.from_numpy(x).cuda().bfloat16(), torch.from_numpy(dy).cuda().bfloat16()
    layer.forward(xt)
    layer.backward(dyt)
    torch.cuda.synchronize()
    layer.check_status()
    for i, (p, want) in enumerate(zip(layer.get_parameters(), acc["grads"])):
        got = p.grad.cpu().numpy()
        if i >= 2 and (i - 2) % 6 in (0, 2, 4):
            assert np.array_equal(got, want), f"weight gradient {i}"
        else:
            assert rel_l2(got, want) < 1e-5, f"gradient {i}"
