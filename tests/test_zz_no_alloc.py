"""The allocation-free dispatch plan (mgpt_moe_op_plan_noalloc) against mgpt_moe_op_plan.

For callers that cannot allocate: an engine whose arena already owns all device memory,
or a step loop that must not meet cudaMalloc's device-wide synchronisation.  The variant
keeps its scratch in a fixed array inside the library, shared by every call, so the test
calls it twice in a row with different inputs (the second, smaller call sees the first
call's leftovers) and compares every output, exactly, with the entry point that takes
caller-provided scratch.  Collected last on purpose: a run that stops at the first failure
has then already run every other test.
"""
import ctypes as ct

import numpy as np
import pytest
import torch

from mgpt_b200 import _lib
from tests.util import PLAN_OUTPUTS, plan_buffers, plan_row_cap

ORDER = ("counts", "offsets", "padded_offsets", "tile_expert", "n_tiles", "map", "pos", "row_src")


def _stream():
    return ct.c_void_p(torch.cuda.current_stream().cuda_stream)


def _with_scratch(lib, top_idx, n_rows, E):
    bufs = plan_buffers(n_rows, E)
    nbytes = lib.mgpt_moe_op_plan_scratch_bytes(n_rows, E)
    scratch = torch.empty(max(1, nbytes), dtype=torch.uint8, device="cuda")
    _lib.check(lib.mgpt_moe_op_plan(top_idx.data_ptr(), n_rows, E, *[bufs[k].data_ptr() for k in ORDER],
                                    plan_row_cap(n_rows, E), bufs["status"].data_ptr(), scratch.data_ptr(),
                                    nbytes, _stream()))
    return bufs


def _no_alloc(lib, top_idx, n_rows, E):
    bufs = plan_buffers(n_rows, E)
    _lib.check(lib.mgpt_moe_op_plan_noalloc(top_idx.data_ptr(), n_rows, E, *[bufs[k].data_ptr() for k in ORDER],
                                            plan_row_cap(n_rows, E), bufs["status"].data_ptr(), _stream()))
    return bufs


def _assert_same(got, want):
    nt = int(want["n_tiles"].item())
    assert int(got["status"].item()) == 0
    for key in PLAN_OUTPUTS:
        a, b = got[key], want[key]
        if key == "tile_expert":
            a, b = a[:nt], b[:nt]
        assert torch.equal(a, b), key              # integer outputs: bit-exact


@pytest.mark.gpu
def test_no_alloc_plan_equals_plan_with_scratch_twice_in_a_row():
    lib = _lib.load()
    rng = np.random.default_rng(5)
    # big first, then small (stale scratch beyond the small call); then the two edges of the fixed array: the
    # largest row count with the largest expert count (every one of its 512 KiB in use) and no rows at all
    for n_rows, E in ((200_000, 64), (3_001, 16), (_lib.PLAN_NOALLOC_MAX_ROWS, 128), (0, 8)):
        idx = np.minimum((rng.random(n_rows) ** 2 * E).astype(np.int32), E - 1)
        top_idx = torch.from_numpy(idx).cuda() if n_rows else torch.zeros(1, dtype=torch.int32, device="cuda")
        want = _with_scratch(lib, top_idx, n_rows, E)
        got = _no_alloc(lib, top_idx, n_rows, E)
        torch.cuda.synchronize()
        _assert_same(got, want)


@pytest.mark.gpu
def test_no_alloc_plan_leaves_free_device_memory_unchanged():
    """After a first call on the device (which may load the library's module), a call allocates nothing: the
    driver reports the same free bytes before and after.  Output buffers are made before the reading."""
    lib = _lib.load()
    n_rows, E = 50_000, 32
    idx = torch.randint(0, E, (n_rows,), dtype=torch.int32, device="cuda")
    _no_alloc(lib, idx, n_rows, E)                  # first call: looks up the array's address
    bufs = plan_buffers(n_rows, E)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _lib.check(lib.mgpt_moe_op_plan_noalloc(idx.data_ptr(), n_rows, E, *[bufs[k].data_ptr() for k in ORDER],
                                                plan_row_cap(n_rows, E), bufs["status"].data_ptr(), _stream()))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    _assert_same(bufs, _with_scratch(lib, idx, n_rows, E))


def test_no_alloc_plan_rejects_sizes_beyond_its_scratch():
    """No GPU work is needed to refuse: the size check comes first."""
    import os
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("libmgpt_moe.so is not built")
    lib = _lib.load()
    n_rows = _lib.PLAN_NOALLOC_MAX_ROWS + 1
    rc = lib.mgpt_moe_op_plan_noalloc(None, n_rows, 8, None, None, None, None, None, None, None, None,
                                      plan_row_cap(n_rows, 8), None, None)
    assert rc == 1
    assert b"at most 1048576" in lib.mgpt_moe_last_error()
