"""The layer driven by the reference's own engine through the adapter class.

``oracle/_ref/engine_moe_driver`` is the reference's Tensor, Scratchpad, cuda_ops (USE_CUDA) and AdamWOptimizer,
compiled from its sources by ``oracle/Makefile``, with ``mgpt_b200/adapter/MoELayer.cpp`` in place of the
reference's MoELayer.cpp and linked to ``libmgpt_moe.so``.  It sizes the arena from ``get_footprint`` x 1.05 as
pipeline/Trainer.cpp:211-224 does, runs forward / rewind / forward / backward / rewind as the checkpointed
GPT.cpp:39-51, 79-96 does, steps the engine's own AdamW and runs the next forward.  Everything it writes is
compared here with the CPU oracle on the same weights (rel-L2 <= 2e-2: the layer computes in BF16).
"""
import os
import struct
import subprocess

import numpy as np
import pytest

from mgpt_b200 import synth
from oracle import oracle
from tests.util import rel_l2

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2


def _run_engine(tmp_path, B, T, w, x, params, dy):
    if not os.path.exists(oracle.ENGINE_BIN):
        pytest.skip("oracle/_ref/engine_moe_driver was not built (needs a checkout of the reference)")
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        f.write(struct.pack("6i", B, T, w.C, w.H, w.E, w.k))
        for p in params:
            f.write(np.ascontiguousarray(p, np.float32).tobytes())
        f.write(np.ascontiguousarray(x, np.float32).tobytes())
        f.write(np.ascontiguousarray(dy, np.float32).tobytes())
    r = subprocess.run([oracle.ENGINE_BIN, str(fin), str(fout)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(fout, dtype=np.float32)
    shapes = synth.param_shapes(w.C, w.H, w.E)
    n = B * T * w.C
    pos = 0

    def take(count, shape=None):
        nonlocal pos
        a = raw[pos: pos + count]
        pos += count
        return a.reshape(shape) if shape else a

    out = {"y": take(n, (B * T, w.C)), "dx": take(n, (B * T, w.C))}
    out["grads"] = [take(s[0] * s[1], s) for s in shapes]
    out["counts"] = take(w.E)
    out["params_after"] = [take(s[0] * s[1], s) for s in shapes]
    out["y2"] = take(n, (B * T, w.C))
    assert pos == raw.size
    return out, r.stdout


def test_reference_engine_drives_the_layer(tmp_path):
    B, T = 4, 96
    w = synth.Workload("engine", B * T, 256, 320, 8, 2, "bf16")
    x, params, dy = synth.make_inputs(w, seed=21, bias_std=0.02)
    got, log = _run_engine(tmp_path, B, T, w, x, params, dy)
    assert "engine_moe_driver ok" in log
    which = "ref" if oracle.have_ref() else "oracle"
    d = oracle.Dims(w.n_tokens, w.C, w.H, w.E, w.k, w.alpha)
    ref = oracle.run(d, x, params, dy, which=which, threads=8)
    # forward twice (the second after the arena was rewound), then backward: same results as one pass
    assert np.array_equal(got["counts"].astype(np.int32), ref["counts"])
    assert rel_l2(got["y"], ref["y"]) <= TOL_BF16
    assert rel_l2(got["dx"], ref["dx"]) <= TOL_BF16
    for i, (a, b) in enumerate(zip(got["grads"], ref["grads"])):
        assert rel_l2(a, b) <= TOL_BF16, (f"grad {i}", rel_l2(a, b))
    # the engine's AdamW moved the FP32 masters (GPU arm of Tensor::adamw_step: same formula as the CPU arm up to
    # a few roundings while |g| < 10); the step is lr-sized, far above that
    for i, (p0, p1, g) in enumerate(zip(params, got["params_after"], got["grads"])):
        want, _, _ = oracle.adamw(p0, g, np.zeros_like(p0), np.zeros_like(p0), lr=1e-2, beta1=0.9, beta2=0.999,
                                  eps=1e-8, weight_decay=0.01, t=1)
        assert np.allclose(p1.ravel(), want, rtol=1e-4, atol=1e-6), f"param {i} after the engine's AdamW step"
    # ... and the next forward used the moved weights: the BF16 copies followed the masters without any call
    # from the engine
    ref2 = oracle.run(d, x, got["params_after"], None, which=which, threads=8)
    assert rel_l2(got["y2"], ref2["y"]) <= TOL_BF16
    assert rel_l2(got["y2"], got["y"]) > 0.1, "the second forward must see the optimiser's update"
