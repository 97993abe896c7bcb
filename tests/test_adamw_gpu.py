"""Fused AdamW + BF16 copy refresh against the reference's AdamW arithmetic (bit-exact) on a B200."""
import numpy as np
import pytest
import torch

from mgpt_b200 import synth
from mgpt_b200.moe_layer import MoELayer
from oracle import oracle

pytestmark = pytest.mark.gpu

HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("mode,shape", [("fp32", (96, 64, 80, 4, 2)), ("bf16", (300, 128, 200, 8, 2)),
                                         ("bf16", (64, 72, 40, 1, 1))])
def test_adamw_matches_reference_bit_for_bit(mode, shape):
    n, C, H, E, k = shape
    w = synth.Workload("adamw", n, C, H, E, k, mode)
    x, params, dy = synth.make_inputs(w, seed=5, bias_std=0.02)
    layer = MoELayer(C, H, E, k, mode=mode)
    layer.load_parameters(params)
    io = torch.bfloat16 if mode == "bf16" else torch.float32
    xt, dyt = torch.from_numpy(x).cuda().to(io), torch.from_numpy(dy).cuda().to(io)
    want_w = [p.copy() for p in params]
    want_m = [np.zeros_like(p) for p in params]
    want_v = [np.zeros_like(p) for p in params]
    for t in (1, 2, 3):
        layer.zero_grad()
        layer.forward(xt)
        layer.backward(dyt)
        grads = [p.grad.cpu().numpy().copy() for p in layer.get_parameters()]
        layer.adamw_step(t, **HYPER)
        torch.cuda.synchronize()
        for i, g in enumerate(grads):          # the CPU restatement, fed the gradients the GPU produced
            nw, nm, nv = oracle.adamw(want_w[i], g, want_m[i], want_v[i], t=t, **HYPER)
            want_w[i], want_m[i], want_v[i] = nw.reshape(params[i].shape), nm.reshape(params[i].shape), nv.reshape(params[i].shape)
        for i, p in enumerate(layer.get_parameters()):
            assert np.array_equal(_bits(p.cpu().numpy()), _bits(want_w[i])), f"step {t}: parameter {i}"
            assert np.array_equal(_bits(layer.opt_m[i].cpu().numpy()), _bits(want_m[i])), f"step {t}: m of {i}"
            assert np.array_equal(_bits(layer.opt_v[i].cpu().numpy()), _bits(want_v[i])), f"step {t}: v of {i}"


def test_copies_written_by_adamw_equal_a_fresh_sync():
    """Forward right after adamw_step (no sync_weights) equals forward after an explicit sync_weights."""
    w = synth.Workload("adamw2", 500, 128, 192, 8, 2, "bf16")
    x, params, dy = synth.make_inputs(w, seed=9, bias_std=0.02)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16")
    layer.load_parameters(params)
    xt, dyt = torch.from_numpy(x).cuda().bfloat16(), torch.from_numpy(dy).cuda().bfloat16()
    layer.zero_grad()
    layer.forward(xt)
    layer.backward(dyt)
    layer.adamw_step(1, **HYPER)
    y_fused = layer.forward(xt).float().cpu().numpy().copy()
    layer.sync_weights()
    y_sync = layer.forward(xt).float().cpu().numpy()
    assert np.array_equal(y_fused, y_sync)


def test_adamw_needs_state_and_valid_step():
    from mgpt_b200 import _lib
    layer = MoELayer(64, 64, 2, 1, mode="bf16")
    with pytest.raises(_lib.MoeError):
        _lib.check(layer.lib.mgpt_moe_adamw_step(layer._h, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, None))
    with pytest.raises(_lib.MoeError):
        layer.adamw_step(0)


def test_guarded_step_skips_nonfinite_and_clamps_like_the_gpu_arm():
    """utils/cuda_ops.cu:727-728: an element whose gradient is NaN or Inf is left untouched, the others see the
    gradient clamped to [-10, 10]; after the guards the arithmetic is the CPU arm's, bit for bit."""
    w = synth.Workload("adamw3", 64, 64, 72, 2, 1, "bf16")
    _, params, _ = synth.make_inputs(w, seed=3, bias_std=0.02)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16")
    layer.load_parameters(params)
    rng = np.random.default_rng(1)
    grads = []
    for p in layer.get_parameters():
        g = (rng.standard_normal(p.shape) * 8.0).astype(np.float32)        # a good share beyond +-10
        flat = g.reshape(-1)
        flat[:: 7] = np.nan
        flat[3:: 11] = np.inf
        flat[5:: 13] = -np.inf
        p.grad.copy_(torch.from_numpy(g))
        grads.append(g)
    layer.adamw_step(1, grad_clip=10.0, skip_nonfinite=True, **HYPER)
    torch.cuda.synchronize()
    for i, (p0, g) in enumerate(zip(params, grads)):
        ok = np.isfinite(g).reshape(-1)
        gc = np.clip(np.where(np.isfinite(g), g, 0.0), -10.0, 10.0).astype(np.float32)
        nw, nm, nv = oracle.adamw(p0, gc, np.zeros_like(p0), np.zeros_like(p0), t=1, **HYPER)
        want_w = np.where(ok, nw, p0.reshape(-1))
        want_m = np.where(ok, nm, 0.0).astype(np.float32)
        got_w = layer.get_parameters()[i].cpu().numpy().reshape(-1)
        assert np.array_equal(_bits(got_w), _bits(want_w)), f"parameter {i}"
        assert np.array_equal(_bits(layer.opt_m[i].cpu().numpy().reshape(-1)), _bits(want_m)), f"m of {i}"
    # the BF16 copies were written from the guarded result: forward agrees with a fresh sync
    x = torch.randn(w.n_tokens, w.C, device="cuda").bfloat16()
    y0 = layer.forward(x).clone()
    layer.sync_weights()
    assert torch.equal(y0, layer.forward(x))
