"""mgpt_moe_step_host_async: pipelined steps with host buffers give what the one-step call gives.

Several steps with different tokens go through the pipelined call (two in flight) on one layer and through
mgpt_moe_step_host on a second layer with the same weights; outputs and input gradients must be identical
(same kernels on the same data), the accumulated parameter gradients equal up to the order of the
floating-point additions of the weight-gradient reductions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layers(mode, C, H, E, k):
    from mgpt_b200 import MoELayer
    a = MoELayer(C, H, E, k, mode=mode)
    b = MoELayer(C, H, E, k, mode=mode)
    g = torch.Generator(device="cuda").manual_seed(7)
    for pa, pb in zip(a.get_parameters(), b.get_parameters()):
        v = (torch.randn(pa.shape, generator=g, device="cuda") * 0.05)
        if mode == "bf16":
            v = v.bfloat16().float()
        pa.copy_(v)
        pb.copy_(v)
    a.sync_weights()
    b.sync_weights()
    a.zero_grad()
    b.zero_grad()
    return a, b


def _tokens(n_steps, N, C, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn(N, C, generator=g).to(dtype).pin_memory() for _ in range(n_steps)]
    dys = [(torch.randn(N, C, generator=g) * 0.1).to(dtype).pin_memory() for _ in range(n_steps)]
    return xs, dys


@pytest.mark.parametrize("mode,dtype", [("bf16", torch.bfloat16), ("fp32", torch.float32)])
def test_pipelined_steps_equal_single_steps(mode, dtype):
    C, H, E, k, N, steps = 256, 128, 8, 2, 640, 5
    a, b = _layers(mode, C, H, E, k)
    xs, dys = _tokens(steps, N, C, dtype, 3)
    ya = [torch.empty_like(x).pin_memory() for x in xs]
    dxa = [torch.empty_like(x).pin_memory() for x in xs]
    for i in range(steps):
        a.step_host_async(xs[i], dys[i], ya[i], dxa[i])
    a.step_host_wait()
    yb, dxb = torch.empty_like(xs[0]).pin_memory(), torch.empty_like(xs[0]).pin_memory()
    for i in range(steps):
        b.step_host(xs[i], dys[i], yb, dxb)
        assert torch.equal(ya[i], yb), f"y of step {i}"
        assert torch.equal(dxa[i], dxb), f"dx of step {i}"
    for pa, pb in zip(a.get_parameters(), b.get_parameters()):
        scale = float(pb.grad.abs().max()) + 1e-12
        assert float((pa.grad - pb.grad).abs().max()) <= 1e-4 * scale
    a.check_status()
    a.close()
    b.close()


def test_pipelined_forward_only_and_mixed_sizes():
    C, H, E, k = 256, 128, 8, 2
    a, b = _layers("bf16", C, H, E, k)
    for N in (96, 1024, 96):                     # staging grows in the middle of a sequence of calls
        xs, _ = _tokens(3, N, C, torch.bfloat16, N)
        ya = [torch.empty_like(x).pin_memory() for x in xs]
        for i in range(3):
            a.step_host_async(xs[i], None, ya[i], None)
        a.step_host_wait()
        yb = torch.empty_like(xs[0]).pin_memory()
        for i in range(3):
            b.step_host(xs[i], None, yb, None)
            assert torch.equal(ya[i], yb)
    # the one-step call still works on a layer that has used the pipelined one
    xs, dys = _tokens(1, 128, C, torch.bfloat16, 11)
    y1, dx1 = torch.empty_like(xs[0]).pin_memory(), torch.empty_like(xs[0]).pin_memory()
    y2, dx2 = torch.empty_like(xs[0]).pin_memory(), torch.empty_like(xs[0]).pin_memory()
    a.step_host(xs[0], dys[0], y1, dx1)
    b.step_host(xs[0], dys[0], y2, dx2)
    assert torch.equal(y1, y2) and torch.equal(dx1, dx2)
    a.close()
    b.close()


def test_wait_without_steps_is_a_no_op():
    from mgpt_b200 import MoELayer
    layer = MoELayer(64, 32, 4, 2, mode="fp32")
    layer.step_host_wait()
    layer.close()
