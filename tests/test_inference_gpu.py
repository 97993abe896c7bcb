"""Forward for generation (mgpt_moe_forward_inference): the reference's generator runs forward only, over a context
that grows by one token per step, and drops the activations (pipeline/Generator.cpp:10-31)."""
import numpy as np
import pytest
import torch

from mgpt_b200 import MoELayer, synth
from mgpt_b200._lib import MoeError
from oracle import oracle
from tests.util import dims_of, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [8, 64, 256])
def test_inference_forward_at_the_decode_shapes(n):
    """Config 5 (C=1024, H=2816, E=32, top-2), 8 / 64 / 256 tokens: routing bit-exact, y within 2e-2 of the oracle
    and identical to the training forward's."""
    w = synth.WORKLOADS["c5-256"].scaled(n)
    x, params, _ = synth.make_inputs(w)
    ref = oracle.run(dims_of(w), x, params, None, threads=16)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16", lb_alpha=w.alpha)
    layer.load_parameters(params)
    xt = torch.from_numpy(x).cuda().bfloat16()
    y_train = layer.forward(xt).clone()
    y = layer.forward_inference(xt)
    torch.cuda.synchronize()
    assert torch.equal(y, y_train)
    assert rel_l2(y.float().cpu().numpy(), ref["y"]) <= 2e-2
    assert np.array_equal(layer.workspace_view("top_idx", torch.int32, (n, w.k)).cpu().numpy(), ref["top_idx"])
    assert layer.get_expert_counts() == ref["counts"].tolist()
    assert int(layer.lib.mgpt_moe_inference_workspace_bytes(layer._h, n)) < layer.get_footprint(1, n)
    with pytest.raises(MoeError):
        layer.backward(torch.zeros_like(xt))            # nothing was kept for it
    layer.check_status()
    layer.close()


def test_generation_loop_over_a_growing_context():
    """Each step re-runs the whole context plus one token: the rows of the earlier tokens never change (the layer
    is per-token), and the last row is the new token's."""
    w = synth.Workload("gen", 40, 256, 384, 8, 2, "bf16")
    x, params, _ = synth.make_inputs(w, seed=17, bias_std=0.02)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16")
    layer.load_parameters(params)
    xt = torch.from_numpy(x).cuda().bfloat16()
    full = layer.forward_inference(xt).clone()
    for n in range(33, 41):
        y = layer.forward_inference(xt[:n].contiguous())
        assert torch.equal(y, full[:n]), n
    layer.check_status()
    layer.close()
