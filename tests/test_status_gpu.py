"""Failure detection without a GPU fault: errors the kernels can meet are reported through a status word.

* an expert id outside [0, E) handed to the operator-level plan is skipped and reported (bit 32);
* a bounded wait that runs out sets its bit, the kernel returns, the host reads MGPT_MOE_ECUDA once, and the
  same layer then runs a normal step.  The wait that runs out is a self-test kernel waiting on a barrier nothing
  arrives on, with a limit of 4096 polls: no trap, no bad address, no endless loop.
"""
import ctypes as ct

import numpy as np
import pytest
import torch

from mgpt_b200 import MoELayer, _lib, synth
from mgpt_b200._lib import MoeError
from oracle import oracle
from tests.util import (assert_plan_equal, assert_routing_exact, dims_of, plan_buffers, plan_reference, plan_row_cap,
                        run_layer)

pytestmark = pytest.mark.gpu

ORDER = ("counts", "offsets", "padded_offsets", "tile_expert", "n_tiles", "map", "pos", "row_src")


def _plan(lib, idx, E):
    n = idx.size
    bufs = plan_buffers(n, E)
    top_idx = torch.from_numpy(idx).cuda()
    nbytes = lib.mgpt_moe_op_plan_scratch_bytes(n, E)
    scratch = torch.empty(max(1, nbytes), dtype=torch.uint8, device="cuda")
    _lib.check(lib.mgpt_moe_op_plan(top_idx.data_ptr(), n, E, *[bufs[k].data_ptr() for k in ORDER],
                                    plan_row_cap(n, E), bufs["status"].data_ptr(), scratch.data_ptr(), nbytes,
                                    ct.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    return bufs


def test_plan_reports_expert_ids_out_of_range():
    lib = _lib.load()
    rng = np.random.default_rng(3)
    E, n = 16, 5000
    idx = rng.integers(0, E, n).astype(np.int32)
    good = _plan(lib, idx, E)
    assert_plan_equal(good, plan_reference(idx, E), n)
    bad = idx.copy()
    bad[[7, 1234, 4999]] = [E, -1, 1 << 20]           # one past the end, negative, far outside
    got = _plan(lib, bad, E)
    assert int(got["status"].item()) == 32
    # the plan of the remaining entries is the plan of the valid ones
    keep = np.ones(n, bool)
    keep[[7, 1234, 4999]] = False
    want = plan_reference(bad[keep], E)
    assert np.array_equal(got["counts"].cpu().numpy(), want["counts"])
    assert np.array_equal(got["offsets"].cpu().numpy(), want["offsets"])
    assert np.array_equal(got["padded_offsets"].cpu().numpy(), want["padded_offsets"])
    flat = np.flatnonzero(keep).astype(np.int32)
    assert np.array_equal(got["map"].cpu().numpy()[: flat.size], flat[want["map"]])


def test_bounded_wait_runs_out_then_the_layer_recovers():
    w = synth.Workload("st", 300, 128, 192, 8, 2, "bf16")
    x, params, dy = synth.make_inputs(w, seed=5, bias_std=0.02)
    ref = oracle.run(dims_of(w), x, params, dy, threads=4)
    layer = MoELayer(w.C, w.H, w.E, w.k, mode="bf16")
    layer.load_parameters(params)
    layer.check_status()                                            # clean after creation
    _lib.check(layer.lib.mgpt_moe_selftest_bounded_wait(layer._h, layer._stream()))
    with pytest.raises(MoeError, match="bounded wait ran out"):
        layer.check_status()
    layer.check_status()                                            # reported once, then clear
    # an error that nobody checked for is still there at the next call that synchronises anyway
    _lib.check(layer.lib.mgpt_moe_selftest_bounded_wait(layer._h, layer._stream()))
    xt = torch.from_numpy(x).cuda().bfloat16()
    layer.forward(xt)
    with pytest.raises(MoeError, match="status 2"):
        layer.get_expert_counts()
    layer.close()
    # the context is intact: a fresh layer passes parity
    got = run_layer(w, x, params, dy, mode="bf16", io=torch.bfloat16)
    assert_routing_exact(got, ref)
    assert got["status"] == 0
