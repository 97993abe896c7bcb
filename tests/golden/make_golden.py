"""Golden vectors for the MoE layer, produced by the reference's own code.

Run in a container that has the reference sources (``oracle/Makefile`` builds
them into ``oracle/_ref/libmgpt_ref.so``):

    python tests/golden/make_golden.py

Each case is a small layer configuration plus seeded inputs (rebuilt by
``build_case`` below, so only the reference's OUTPUTS are stored).  The files
pin the CPU restatement in ``oracle/moe_oracle.c`` and the CUDA path; they are
needed because the reference's own tests assert output shapes only
(test/networkTest/moeTests.cpp:6-39).
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from mgpt_b200 import synth  # noqa: E402

# name -> (Workload, tweak)
CASES = {
    # the reference test's shape (B=2,T=4,C=16,E=4,k=2, hidden 4C) and its all-ones input
    "ones": (synth.Workload("ones", 8, 16, 64, 4, 2, "fp32"), "ones"),
    "tiny": (synth.Workload("tiny", 8, 16, 64, 4, 2, "fp32"), None),
    # exact probability ties: router columns 1,2 and 4 are identical -> lowest index first
    "ties": (synth.Workload("ties", 24, 16, 32, 6, 3, "fp32"), "ties"),
    # clamp floor: most experts sit at the 1e-7 floor and tie there
    "floor": (synth.Workload("floor", 16, 16, 32, 8, 4, "fp32"), "floor"),
    # Zipf-like router bias: several experts receive no rows
    "empty": (synth.Workload("empty", 40, 32, 48, 16, 2, "bf16", skew=True), "wide_router"),
    "k1": (synth.Workload("k1", 33, 24, 40, 3, 1, "fp32"), None),
    "kE": (synth.Workload("kE", 19, 16, 24, 4, 4, "fp32"), None),
    "e64k4": (synth.Workload("e64k4", 96, 16, 16, 64, 4, "bf16", skew=True), "wide_router"),
    "one_token": (synth.Workload("one_token", 1, 16, 32, 4, 2, "fp32"), None),
    "mid": (synth.Workload("mid", 200, 32, 64, 8, 2, "bf16"), None),
}


def build_case(name: str):
    """Returns (workload, x, params, dy) for a named case."""
    w, tweak = CASES[name]
    x, params, dy = synth.make_inputs(w, seed=4321, bias_std=0.05)
    if tweak == "ones":
        x = np.ones_like(x)
        dy = np.ones_like(dy)
    elif tweak == "ties":
        params[0][:, 2] = params[0][:, 1]
        params[0][:, 4] = params[0][:, 1]
        params[1][0, 2] = params[1][0, 1]
        params[1][0, 4] = params[1][0, 1]
    elif tweak == "wide_router":
        # spread the logits so the skewed bias leaves a ragged, partly empty load
        params[0] = synth.bf16_round(params[0] * np.float32(40.0))
    elif tweak == "floor":
        params[1][0, :] = np.array([0.0, -30.0, -40.0, 1.0, -35.0, -50.0, -60.0, -45.0], np.float32)
    return w, x, params, dy


def input_digest(x, params, dy) -> str:
    h = hashlib.sha256()
    for a in [x, dy] + list(params):
        h.update(np.ascontiguousarray(a, dtype=np.float32).tobytes())
    return h.hexdigest()


def golden_path(name: str) -> str:
    return os.path.join(HERE, f"{name}.npz")


def load_golden(name: str) -> dict:
    with np.load(golden_path(name)) as z:
        out = {k: z[k] for k in z.files if not k.startswith("grad_")}
        n = int(z["n_grads"])
        out["grads"] = [z[f"grad_{i}"] for i in range(n)]
    return out


def main() -> None:
    from oracle import oracle

    if not oracle.have_ref():
        oracle.build(ref=True)
    for name in CASES:
        w, x, params, dy = build_case(name)
        d = oracle.Dims(w.n_tokens, w.C, w.H, w.E, w.k, w.alpha)
        r = oracle.run(d, x, params, dy, which="ref")
        arrays = {k: v for k, v in r.items() if k != "grads"}
        for i, g in enumerate(r["grads"]):
            arrays[f"grad_{i}"] = g
        arrays["n_grads"] = np.int32(len(r["grads"]))
        arrays["input_sha256"] = np.frombuffer(input_digest(x, params, dy).encode(), dtype=np.uint8)
        np.savez_compressed(golden_path(name), **arrays)
        print(f"{name}: counts {r['counts'].tolist()} -> {os.path.getsize(golden_path(name))} bytes")
    make_adamw_golden()


def make_adamw_golden() -> None:
    """Three steps of the reference's own AdamW (Tensor::adamw_step, CPU arm) on a seeded flat tensor."""
    from oracle import oracle

    rng = np.random.default_rng(20240611)
    n = 1537
    w = rng.normal(0, 0.02, n).astype(np.float32)
    g = rng.normal(0, 1e-2, n).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    hyper = dict(lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
    w3, m3, v3 = w, m, v
    for t in (1, 2, 3):
        w3, m3, v3 = oracle.adamw(w3, g, m3, v3, t=t, which="ref", **hyper)
    np.savez_compressed(golden_path("adamw"), w=w, g=g, m=m, v=v, w3=w3, m3=m3, v3=v3,
                        **{k: np.float32(x) for k, x in hyper.items()})
    print(f"adamw: {os.path.getsize(golden_path('adamw'))} bytes")


if __name__ == "__main__":
    main()
