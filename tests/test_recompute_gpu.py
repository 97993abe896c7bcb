"""Recompute forward with saved routing (activation checkpointing) equals the plain forward."""
import numpy as np
import pytest
import torch

from mgpt_b200 import MoELayer, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,shape", [("fp32", (200, 64, 96, 8, 2)), ("bf16", (1500, 256, 320, 16, 2)),
                                         ("bf16", (700, 128, 192, 16, 4))])
def test_recompute_matches_forward_and_feeds_backward(mode, shape):
    n, C, H, E, k = shape
    w = synth.Workload("rc", n, C, H, E, k, mode, skew=(k == 4))
    x, params, dy = synth.make_inputs(w, seed=21, bias_std=0.02)
    io = torch.bfloat16 if mode == "bf16" else torch.float32
    layer = MoELayer(C, H, E, k, mode=mode)
    layer.load_parameters(params)
    xt, dyt = torch.from_numpy(x).cuda().to(io), torch.from_numpy(dy).cuda().to(io)

    layer.zero_grad()
    y = layer.forward(xt)
    routing = layer.save_routing()
    dx = layer.backward(dyt)
    want_y, want_dx = y.clone(), dx.clone()
    want_g = [p.grad.clone() for p in layer.get_parameters()]
    counts = list(layer.get_expert_counts())

    layer._ws.fill_(0x7f)                    # the arena is rewound and reused between the two forwards
    layer.zero_grad()
    y2 = torch.empty_like(xt)
    layer.recompute_into(xt, y2, routing)
    dx2 = layer.backward(dyt)
    torch.cuda.synchronize()
    assert torch.equal(y2, want_y)
    assert torch.equal(dx2, want_dx)
    assert list(layer.get_expert_counts()) == counts
    for a, p in zip(want_g, layer.get_parameters()):
        # bias and router-bias gradients are sums of float atomics: equal up to the order of addition
        assert torch.allclose(p.grad, a, rtol=1e-4, atol=1e-6)


def test_recompute_checks_its_arguments():
    from mgpt_b200 import _lib
    layer = MoELayer(64, 64, 4, 2, mode="bf16")
    layer.sync_weights()
    with pytest.raises(_lib.MoeError):
        _lib.check(layer.lib.mgpt_moe_save_routing(layer._h, None, None))
    x = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    layer.forward(x)
    st = layer.save_routing()
    with pytest.raises(AssertionError):
        layer.recompute_into(torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda"),
                             torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda"), st)


@pytest.mark.parametrize("mode", ["fp32", "bf16"])
def test_forward_with_residual_equals_forward_plus_add(mode):
    w = synth.Workload("res", 333, 128, 160, 8, 2, mode)
    x, params, dy = synth.make_inputs(w, seed=31, bias_std=0.02)
    io = torch.bfloat16 if mode == "bf16" else torch.float32
    layer = MoELayer(w.C, w.H, w.E, w.k, mode=mode)
    layer.load_parameters(params)
    xt = torch.from_numpy(x).cuda().to(io)
    res = torch.from_numpy(dy).cuda().to(io)            # any tensor of the right shape
    y = layer.forward(xt)
    out = torch.empty_like(xt)
    layer.forward_into(xt, out, residual=res)
    torch.cuda.synchronize()
    if mode == "fp32":
        assert torch.equal(out, res + y)                # the residual is added last, as the reference's caller does
    else:
        # the fused sum is rounded once; forward + add rounds y first
        assert torch.allclose(out.float(), res.float() + y.float(), rtol=2e-2, atol=2e-2)
        assert float((out.float() - (res.float() + y.float())).abs().max()) <= 2 ** -6 * float(out.float().abs().max())
