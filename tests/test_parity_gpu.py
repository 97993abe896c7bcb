"""CUDA path against the CPU oracle and the reference's golden vectors (through the C ABI)."""
import numpy as np
import pytest
import torch

from mgpt_b200 import synth
from oracle import oracle
from tests.golden import make_golden as G
from tests.util import assert_routing_exact, assert_values, dims_of, rel_l2, run_layer

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5     # FP32 SIMT validation mode
TOL_BF16 = 2e-2     # BF16 operands, FP32 accumulate


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_fp32_mode_matches_reference_golden(name):
    w, x, params, dy = G.build_case(name)
    gold = G.load_golden(name)
    got = run_layer(w, x, params, dy, mode="fp32")
    assert_routing_exact(got, gold)
    assert_values(got, gold, TOL_FP32, w)


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_bf16_simt_products_match_oracle(name):
    w, x, params, dy = G.build_case(name)
    x, dy = synth.bf16_round(x), synth.bf16_round(dy)
    params = [synth.bf16_round(p) for p in params]
    ref = oracle.run(dims_of(w), x, params, dy, threads=4)
    got = run_layer(w, x, params, dy, mode="bf16", gemm_impl=1)
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_BF16, w)


def test_c1_fp32_full_size():
    w = synth.WORKLOADS["c1"]
    x, params, dy = synth.make_inputs(w, bias_std=0.02)
    ref = oracle.run(dims_of(w), x, params, dy, threads=8)
    got = run_layer(w, x, params, dy, mode="fp32")
    assert_routing_exact(got, ref)
    assert_values(got, ref, TOL_FP32, w)
    assert rel_l2(got["d_top_p"], ref["d_top_p"]) <= TOL_FP32
    assert rel_l2(got["dlogits"], ref["dlogits"]) <= 1e-4


@pytest.mark.parametrize("impl", [1, 0])
@pytest.mark.parametrize("name", ["c2", "c3", "c5-256"])
def test_routing_bit_exact_at_full_size(name, impl):
    """Router + plan at the benchmark sizes (the oracle's routing pass takes seconds).  impl 1: the exact
    CUDA-core router alone; impl 0: tensor-core first pass + exact second pass."""
    w = synth.WORKLOADS[name]
    x, params, dy = synth.make_inputs(w)
    ref = oracle.run(dims_of(w), x, params, route_only=True, threads=16)
    got = run_layer(w, x, params, None, mode="fp32" if w.dtype == "fp32" else "bf16", gemm_impl=impl,
                    io=torch.bfloat16)
    assert_routing_exact(got, ref)
    if impl == 0 and got["screened"]:
        assert got["router_recompute"] <= w.n_tokens // 2


def test_gradients_accumulate():
    """Two backward passes add up (Tensor::add_grad semantics, Tensor.cpp:638-650)."""
    w, x, params, dy = G.build_case("mid")
    got = run_layer(w, x, params, dy, mode="fp32")
    layer = got["layer"]
    g1 = [p.grad.clone() for p in layer.get_parameters()]
    xt = torch.from_numpy(x).cuda()
    layer.forward(xt)
    layer.backward(torch.from_numpy(dy).cuda())
    for a, p in zip(g1, layer.get_parameters()):
        assert torch.allclose(p.grad, 2 * a, rtol=1e-4, atol=1e-6)


def test_expert_counts_and_padding_invariants():
    w, x, params, dy = G.build_case("e64k4")
    got = run_layer(w, x, params, dy, mode="fp32")
    layer = got["layer"]
    assert layer.get_expert_counts() == got["counts"].tolist()
    po = got["padded_offsets"]
    assert np.all(np.diff(po) == (got["counts"] + 127) // 128 * 128)
    # every flat index lands inside its expert's padded segment at its stable rank
    flat_e = got["top_idx"].reshape(-1)
    slot_of = np.empty_like(got["map"])
    slot_of[got["map"]] = np.arange(len(got["map"]))
    assert np.array_equal(got["pos"], po[flat_e] + slot_of - got["offsets"][flat_e])


def test_forward_is_deterministic():
    """The reference recomputes forward under activation checkpointing (GPT.cpp:79-96)."""
    w, x, params, dy = G.build_case("mid")
    a = run_layer(w, x, params, None, mode="fp32")
    b = run_layer(w, x, params, None, mode="fp32")
    assert np.array_equal(a["y"], b["y"]) and np.array_equal(a["map"], b["map"])


def test_step_host_equals_device_path():
    w, x, params, dy = G.build_case("mid")
    got = run_layer(w, x, params, dy, mode="fp32")
    layer = got["layer"]
    layer.zero_grad()
    xh, dyh = torch.from_numpy(x).pin_memory(), torch.from_numpy(dy).pin_memory()
    yh, dxh = torch.empty_like(xh).pin_memory(), torch.empty_like(xh).pin_memory()
    layer.step_host(xh, dyh, yh, dxh)
    assert np.array_equal(yh.numpy(), got["y"])
    assert rel_l2(dxh.numpy(), got["dx"]) < 1e-6


def test_errors_are_reported():
    from mgpt_b200 import MoELayer, MoeError
    layer = MoELayer(16, 32, 4, 2, mode="fp32")
    with pytest.raises(MoeError):
        layer.backward(torch.zeros(4, 16, device="cuda"))          # backward before forward
    with pytest.raises(MoeError):
        layer.forward(torch.zeros(4, 16, device="cuda", dtype=torch.bfloat16))   # FP32 mode wants FP32
    bf = MoELayer(16, 32, 4, 2, mode="bf16", gemm_impl=1)
    bf._bind()                                                       # rebinding marks the shadows stale
    with pytest.raises(MoeError):
        bf.forward(torch.zeros(4, 16, device="cuda"))


@pytest.mark.parametrize("n_rows,E", [(0, 4), (1, 1), (37, 3), (5000, 16), (70000, 64), (4096, 128)])
def test_op_plan_matches_numpy(n_rows, E):
    """Operator-level dispatch plan through the C ABI: counts, offsets, slot map, padded rows."""
    import ctypes as ct
    from mgpt_b200 import _lib
    from tests.util import assert_plan_equal, plan_buffers, plan_reference, plan_row_cap
    lib = _lib.load()
    rng = np.random.default_rng(n_rows + E)
    # a skewed draw: low expert ids are much more likely, some experts may stay empty
    idx = np.minimum((rng.random(n_rows) ** 3 * E).astype(np.int32), E - 1)
    top_idx = torch.from_numpy(idx).cuda() if n_rows else torch.zeros(1, dtype=torch.int32, device="cuda")
    bufs = plan_buffers(n_rows, E)
    nbytes = lib.mgpt_moe_op_plan_scratch_bytes(n_rows, E)
    scratch = torch.empty(max(1, nbytes), dtype=torch.uint8, device="cuda")
    rc = lib.mgpt_moe_op_plan(top_idx.data_ptr(), n_rows, E, *[bufs[k].data_ptr() for k in
                              ("counts", "offsets", "padded_offsets", "tile_expert", "n_tiles", "map", "pos", "row_src")],
                              plan_row_cap(n_rows, E), bufs["status"].data_ptr(), scratch.data_ptr(), nbytes,
                              ct.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc)
    torch.cuda.synchronize()
    assert_plan_equal(bufs, plan_reference(idx, E), n_rows)
