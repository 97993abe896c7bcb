"""Parity on the benchmark's own configurations, at their own dimensions.

The CPU oracle needs seconds per step for these widths (it walks every expert's weights), so each case takes
as many tokens as the oracle finishes in ~15 s: config 2 whole, config 3 on 4096 tokens of its 16384 (the
router bias keeps the load as skewed: most experts empty, a few with 1-3 rows, one with every token), config 4
on 512 tokens (forward AND backward: y, dx and all 2+6E gradients), config 5 forward at 256 tokens.  Routing
must be bit-exact, values within rel-L2 2e-2 (BF16 operands, FP32 accumulation).
"""
import numpy as np
import pytest
import torch

from mgpt_b200 import MoELayer, synth
from oracle import oracle
from tests.util import assert_routing_exact, assert_values, dims_of, rel_l2, run_layer

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2


def _case(name, n_tokens):
    w = synth.WORKLOADS[name]
    w = w if n_tokens == w.n_tokens else w.scaled(n_tokens)
    x, params, dy = synth.make_inputs(w)
    if not w.backward:
        dy = None
    ref = oracle.run(dims_of(w), x, params, dy, threads=32)
    got = run_layer(w, x, params, dy, mode="bf16", io=torch.bfloat16)
    return w, ref, got


def test_c4_forward_and_backward_on_512_tokens():
    """C=2048, H=1408, E=64, top-2: 32 and 22 k-blocks, 11 gate/up column tiles, and experts with only a
    handful of rows each (512 tokens over 64 experts), so every tile is mostly padding."""
    w, ref, got = _case("c4", 512)
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)
    assert got["status"] == 0


def test_c3_skewed_on_4096_tokens():
    """C=1024, H=512, E=64, top-4 with the router bias 2*ln(1/(e+1)): empty experts, experts with 1-3 rows and
    one expert that receives every token (the long reduction of the weight gradients)."""
    w, ref, got = _case("c3", 4096)
    counts = ref["counts"]
    assert (counts == 0).any() and ((counts >= 1) & (counts <= 3)).any() and counts.max() == w.n_tokens
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)
    assert got["status"] == 0


def test_c2_whole():
    """All 8192 tokens of config 2 (C=512, H=1376 = 21.5 k-blocks, E=16, top-2)."""
    w, ref, got = _case("c2", 8192)
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)
    assert got["status"] == 0


def test_c5_forward_values_at_256_tokens():
    w, ref, got = _case("c5-256", 256)
    assert_routing_exact(got, ref)
    assert rel_l2(got["y"], ref["y"]) <= TOL_BF16
    assert got["status"] == 0


def test_bf16_forward_is_bit_deterministic_at_c4():
    """The recompute forward of a checkpointed step relies on the BF16 forward giving the same bits every time.
    Ten forwards of the full 32768-token config 4 on plain stream launches and three replays of a CUDA graph of
    the same forward: y and the saved activations Hh and Yg must be identical to the first run's."""
    w = synth.WORKLOADS["c4"]
    gen = torch.Generator(device="cuda").manual_seed(77)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16", lb_alpha=w.alpha)
    for p in layer.get_parameters():
        p.copy_((torch.randn(p.shape, generator=gen, device="cuda") * 0.02).bfloat16().float())
    layer.sync_weights()
    x = torch.randn(w.n_tokens, w.C, generator=gen, device="cuda").bfloat16()
    y = torch.empty_like(x)
    bf = torch.bfloat16

    def snapshot():
        torch.cuda.synchronize()
        rows = int(layer.workspace_view("padded_offsets", torch.int32)[-1])
        return (y.clone(), layer.workspace_view("Hh", bf).view(-1, w.H)[:rows].clone(),
                layer.workspace_view("Yg", bf).view(-1, w.C)[:rows].clone())

    layer.forward_into(x, y)
    first = snapshot()
    for _ in range(9):
        y.zero_()
        layer.forward_into(x, y)
        for a, b in zip(snapshot(), first):
            assert torch.equal(a, b)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.forward_into(x, y)            # the graph's stream has seen one launch before capture
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        layer.forward_into(x, y)
    for _ in range(3):
        y.zero_()
        g.replay()
        for a, b in zip(snapshot(), first):
            assert torch.equal(a, b)
    layer.check_status()
    layer.close()
