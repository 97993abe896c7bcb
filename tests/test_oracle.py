"""The CPU oracle against the reference's golden vectors (and, where the
reference build exists, against the reference itself, live)."""
import numpy as np
import pytest

from mgpt_b200 import synth
from oracle import oracle
from tests.golden import make_golden as G


def _dims(w):
    return oracle.Dims(w.n_tokens, w.C, w.H, w.E, w.k, w.alpha)


def _assert_same(got, want, keys=None):
    for key, ref in want.items():
        if keys is not None and key not in keys:
            continue
        if key == "grads":
            for i, (a, b) in enumerate(zip(got["grads"], ref)):
                assert np.array_equal(a.reshape(-1), b.reshape(-1)), f"grad {i}"
        elif key in got:
            assert np.array_equal(got[key], ref), key


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_oracle_matches_reference_golden(name):
    w, x, params, dy = G.build_case(name)
    gold = G.load_golden(name)
    assert bytes(gold.pop("input_sha256")).decode() == G.input_digest(x, params, dy), \
        "seeded inputs drifted from the ones the golden file was made with"
    gold.pop("n_grads")
    got = oracle.run(_dims(w), x, params, dy, threads=2)
    _assert_same(got, gold)


@pytest.mark.parametrize("name", ["tiny", "e64k4"])
def test_route_only_equals_full(name):
    w, x, params, dy = G.build_case(name)
    full = oracle.run(_dims(w), x, params, dy)
    route = oracle.run(_dims(w), x, params, route_only=True)
    _assert_same(route, {k: full[k] for k in ("logits", "probs", "top_idx", "top_p", "counts", "offsets", "map")})


def test_threads_do_not_change_results():
    w, x, params, dy = G.build_case("mid")
    a = oracle.run(_dims(w), x, params, dy, threads=1)
    b = oracle.run(_dims(w), x, params, dy, threads=5)
    _assert_same(a, b)


def test_known_answers_ties_and_floor():
    # equal probabilities keep the lowest expert index first (utils/Tensor.cpp:1319-1329)
    w, x, params, dy = G.build_case("ties")
    r = oracle.run(_dims(w), x, params, route_only=True)
    p = r["probs"]
    assert np.array_equal(p[:, 1], p[:, 2]) and np.array_equal(p[:, 1], p[:, 4])
    for t in range(w.n_tokens):
        sel = list(r["top_idx"][t])
        tied = [e for e in sel if e in (1, 2, 4)]
        assert tied == sorted(tied) and tied == [1, 2, 4][:len(tied)]
    # the clamp floor is exactly 1e-7 and ties there resolve to the lowest index
    w, x, params, dy = G.build_case("floor")
    r = oracle.run(_dims(w), x, params, route_only=True)
    assert np.all(r["probs"][:, [1, 2, 4, 5, 6, 7]] == np.float32(1e-7))
    assert np.all(r["top_idx"][:, 2:] == np.array([1, 2]))
    assert r["counts"].tolist() == [16, 16, 16, 16, 0, 0, 0, 0]


def test_plan_invariants():
    w, x, params, dy = G.build_case("e64k4")
    r = oracle.run(_dims(w), x, params, route_only=True)
    R = w.n_tokens * w.k
    assert r["counts"].sum() == R
    assert np.array_equal(r["offsets"], np.concatenate([[0], np.cumsum(r["counts"])[:-1]]))
    assert sorted(r["map"].tolist()) == list(range(R))
    flat_e = r["top_idx"].reshape(-1)
    for e in range(w.E):
        seg = r["map"][r["offsets"][e]: r["offsets"][e] + r["counts"][e]]
        assert np.all(flat_e[seg] == e) and np.all(np.diff(seg) > 0)   # stable within an expert


@pytest.mark.skipif(not oracle.have_ref(), reason="reference build (oracle/_ref) not present")
@pytest.mark.parametrize("shape", [(64, 32, 48, 8, 2), (37, 24, 40, 5, 3), (128, 64, 96, 16, 4)])
def test_oracle_matches_reference_live(shape):
    n, C, H, E, k = shape
    w = synth.Workload("live", n, C, H, E, k, "fp32")
    x, params, dy = synth.make_inputs(w, seed=99, bias_std=0.1)
    a = oracle.run(_dims(w), x, params, dy, threads=2)
    b = oracle.run(_dims(w), x, params, dy, which="ref")
    _assert_same(a, b)


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_numpy_plan_reference_matches_golden(name):
    """The numpy statement of the dispatch plan used by the operator-level GPU tests is itself pinned."""
    from tests.util import plan_reference
    w, x, params, dy = G.build_case(name)
    gold = G.load_golden(name)
    r = plan_reference(gold["top_idx"], w.E)
    for key in ("counts", "offsets", "map"):
        assert np.array_equal(r[key], gold[key]), key


def test_adamw_restatement_matches_reference_live():
    """oracle/moe_oracle.c:moe_oracle_adamw against the reference's Tensor::adamw_step (CPU arm), bit for bit."""
    if not oracle.have_ref():
        pytest.skip("reference build absent")
    rng = np.random.default_rng(3)
    n = 4099
    w = rng.normal(0, 0.02, n).astype(np.float32)
    g = rng.normal(0, 1e-2, n).astype(np.float32)
    m = rng.normal(0, 1e-3, n).astype(np.float32)
    v = (rng.random(n) * 1e-5).astype(np.float32)
    for t in (1, 2, 17, 5000):
        a = oracle.adamw(w, g, m, v, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, t=t)
        b = oracle.adamw(w, g, m, v, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, t=t, which="ref")
        for x, y in zip(a, b):
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


def test_adamw_restatement_matches_golden():
    """tests/golden/adamw.npz holds the reference build's own outputs (make_golden.py)."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "adamw.npz"))
    w, m, v = z["w"], z["m"], z["v"]
    for t in (1, 2, 3):
        w, m, v = oracle.adamw(w, z["g"], m, v, lr=float(z["lr"]), beta1=float(z["beta1"]), beta2=float(z["beta2"]),
                               eps=float(z["eps"]), weight_decay=float(z["weight_decay"]), t=t)
    for got, want in ((w, z["w3"]), (m, z["m3"]), (v, z["v3"])):
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_seeded_tokens_have_the_prefix_property():
    """bench.py checks the first rows of a full-size run against the oracle run on a token subset: the generator's
    first rows must not depend on the token count, and the per-tensor generators must equal make_inputs."""
    from mgpt_b200 import synth
    w = synth.WORKLOADS["c2"]
    x, params, dy = synth.make_inputs(w)
    xs, _, dys = synth.make_inputs(w.scaled(300))
    assert np.array_equal(x[:300], xs) and np.array_equal(dy[:300], dys)
    xt, dyt = synth.make_tokens(w)
    assert np.array_equal(x, xt) and np.array_equal(dy, dyt)
    for i in (0, 1, 2, 3, 6, 7, len(params) - 1):
        assert np.array_equal(params[i], synth.make_param(w, i))
    w3 = synth.WORKLOADS["c3"].scaled(16)
    assert np.array_equal(synth.make_inputs(w3)[1][1], synth.make_param(w3, 1))


def test_rmsnorm_restatement_matches_reference_live():
    """The numpy RMSNorm the block-glue tests use, against the reference's own Tensor code."""
    if not oracle.have_ref():
        pytest.skip("reference build not present")
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((37, 96)) * 1.5 + 0.2).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(96)).astype(np.float32)
    d = rng.standard_normal((37, 96)).astype(np.float32)
    a, b = oracle.rmsnorm(x, g, d), oracle.rmsnorm(x, g, d, which="ref")
    for u, v in zip(a, b):
        assert np.allclose(u, v, rtol=2e-6, atol=1e-6)
