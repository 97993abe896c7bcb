"""The block's glue fused around the layer: x2 = x1 + moe(rmsnorm(x1)*gamma) and its backward
(layers/TransformerBlock.cpp:42-46, 80-84; RMSNorm utils/Tensor.cpp:785-800, 1674-1690)."""
import numpy as np
import pytest
import torch

from mgpt_b200 import MoELayer, synth
from oracle import oracle
from tests.util import dims_of, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,io,tol", [("fp32", torch.float32, 2e-5), ("bf16", torch.bfloat16, 2e-2)])
def test_block_forward_and_backward(mode, io, tol):
    w = synth.Workload("blk", 700, 256, 320, 8, 2, mode)
    x1, params, dout = synth.make_inputs(w, seed=41, bias_std=0.02)
    x1 = (x1 * np.float32(1.7) + np.float32(0.3)).astype(np.float32)            # not unit variance, not centred
    rng = np.random.default_rng(2)
    gamma = (1.0 + 0.1 * rng.standard_normal(w.C)).astype(np.float32)
    if mode == "bf16":
        x1, dout = synth.bf16_round(x1), synth.bf16_round(dout)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode=mode, lb_alpha=w.alpha)
    layer.load_parameters(params)
    layer.zero_grad()
    g_t = torch.from_numpy(gamma).cuda()
    dg_t = torch.zeros_like(g_t)
    x1_t = torch.from_numpy(x1).cuda().to(io)
    x2 = layer.block_forward(x1_t, g_t, eps=1e-5)
    ln2 = layer.block_input().float().cpu().numpy()                            # what the layer saw
    d_x1 = layer.block_backward(g_t, torch.from_numpy(dout).cuda().to(io), dg_t)
    torch.cuda.synchronize()
    layer.check_status()

    # 1. the norm itself against the reference's (the layer's input is rounded to the tokens' dtype)
    ref_out, ref_rs, _, _ = oracle.rmsnorm(x1, gamma, dout)
    want_ln2 = synth.bf16_round(ref_out) if mode == "bf16" else ref_out
    assert rel_l2(ln2, want_ln2) <= (4e-3 if mode == "bf16" else 1e-6)
    # 2. the layer on exactly that input: routing bit-exact, values within the mode's tolerance
    d = dims_of(w)
    moe = oracle.run(d, ln2, params, dout, threads=8)
    N, E, k = w.n_tokens, w.E, w.k
    assert np.array_equal(layer.workspace_view("top_idx", torch.int32, (N, k)).cpu().numpy(), moe["top_idx"])
    assert np.array_equal(layer.workspace_view("map", torch.int32).cpu().numpy(), moe["map"])
    assert rel_l2(x2.float().cpu().numpy(), x1 + moe["y"]) <= tol
    for i, (p, g) in enumerate(zip(layer.get_parameters(), moe["grads"])):
        assert rel_l2(p.grad.cpu().numpy(), g) <= tol, f"grad {i}"
    # 3. backward glue: d_x1 = dout + rmsnorm_backward(gradient w.r.t. the layer's input), d_gamma
    _, _, dn, dgam = oracle.rmsnorm(x1, gamma, moe["dx"])
    assert rel_l2(d_x1.float().cpu().numpy(), dout + dn) <= tol
    assert rel_l2(dg_t.cpu().numpy(), dgam) <= tol
    layer.close()
