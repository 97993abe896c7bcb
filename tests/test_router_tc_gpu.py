"""The router for BF16 tokens: tensor-core first pass + exact second pass (mgpt_b200/csrc/router_tc.cu).

Bar: top-k indices, counts and the slot permutation equal the CPU reference's bit for bit, whatever the first
pass's rounding did -- on the golden cases (exact ties, the clamp floor, k = E), on FP32 router weights that
no BF16 value represents, on weights built to sit on the decision boundary, and on large activations.
"""
import numpy as np
import pytest
import torch

from mgpt_b200 import synth
from oracle import oracle
from tests.golden import make_golden as G
from tests.util import assert_routing_exact, assert_values, dims_of, run_layer

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _always_take_the_tensor_core_router(monkeypatch):
    """The library keeps small problems on the exact kernel alone (it is faster there); these tests are about the
    two-pass router, whatever the size."""
    monkeypatch.setenv("MGPT_MOE_ROUTER_TC_MIN_WORK", "0")


def _route(w, x, params):
    ref = oracle.run(dims_of(w), x, params, route_only=True, threads=16)
    got = run_layer(w, x, params, None, mode="bf16", io=torch.bfloat16)
    assert got["screened"]
    return ref, got


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_golden_cases_with_bf16_tokens(name):
    w, x, params, dy = G.build_case(name)
    x, dy = synth.bf16_round(x), synth.bf16_round(dy)
    params = [synth.bf16_round(p) for p in params]
    ref = oracle.run(dims_of(w), x, params, dy, threads=4)
    got = run_layer(w, x, params, dy, mode="bf16", io=torch.bfloat16)
    assert_routing_exact(got, ref)
    assert_values(got, ref, 2e-2, w)


@pytest.mark.parametrize("shape", [(8192, 512, 64, 4), (4096, 2048, 64, 2), (3000, 200, 5, 2), (2048, 1024, 128, 8),
                                   (5000, 256, 24, 3)])
def test_fp32_router_weights(shape):
    """Router weights with all 24 significand bits in use (what an optimiser step leaves): the first pass sees
    them as two BF16 pieces; indices must still be exact.  Also checks that the first pass's logits sit far inside
    the error bound the screening assumes."""
    n, C, E, k = shape
    w = synth.Workload("rt", n, C, 64, E, k, "bf16")
    x, params, _ = synth.make_inputs(w, seed=31, bias_std=0.02)
    rng = np.random.default_rng(7)
    params[0] = (rng.standard_normal((C, E)) * 0.02).astype(np.float32)          # not rounded to BF16
    params[1] = (rng.standard_normal((1, E)) * 0.1).astype(np.float32)
    ref, got = _route(w, x, params)
    assert_routing_exact(got, ref)
    frac = got["router_recompute"] / n
    assert frac < 0.6, frac
    u = 2.0 ** -24
    bound = (1.5 * C * u + 2.0 ** -16) * np.linalg.norm(x, axis=1) * np.linalg.norm(params[0], axis=0).max()
    err = np.abs(got["logits"] - ref["logits"]).max(axis=1)
    assert (err <= 0.25 * bound + 1e-7).all(), float((err / bound).max())


def test_decisions_on_the_boundary():
    """Columns of Wr that are equal (exact ties: the lowest index must win) or differ in the last bit or two."""
    n, C, E, k = 4096, 256, 16, 3
    w = synth.Workload("rt2", n, C, 64, E, k, "bf16")
    x, params, _ = synth.make_inputs(w, seed=33)
    Wr = params[0]
    Wr[:, 1] = Wr[:, 0]                                              # exact tie everywhere
    Wr[:, 3] = np.nextafter(Wr[:, 2], np.float32(np.inf))            # one ulp apart in every weight
    Wr[:, 5] = Wr[:, 4] * np.float32(1.0 + 2.0 ** -12)
    Wr[:, 7] = -Wr[:, 6]
    ref, got = _route(w, x, params)
    assert_routing_exact(got, ref)
    assert got["router_recompute"] > 0


def test_large_and_tiny_activations():
    n, C, E, k = 2048, 512, 32, 2
    w = synth.Workload("rt3", n, C, 64, E, k, "bf16")
    x, params, _ = synth.make_inputs(w, seed=35)
    x[: n // 2] *= np.float32(200.0)             # saturated softmax: floor-clamped probabilities beyond the first
    x[n // 2:] *= np.float32(1e-3)               # near-uniform probabilities
    x = synth.bf16_round(x)
    ref, got = _route(w, x, params)
    for key in ("top_idx", "counts", "offsets", "map"):          # probabilities of logits ~100 move by ~1e-4 relative
        assert np.array_equal(got[key], ref[key]), key
    assert got["status"] == 0
