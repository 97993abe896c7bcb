"""ctypes front end for the CPU oracle of the MoE layer.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs, never by the ``mgpt_b200`` package.

Two libraries share one C signature (oracle/moe_oracle.h):

* ``liboracle.so``        -- the plain-C restatement (``moe_oracle.c``)
* ``_ref/libmgpt_ref.so`` -- the reference's own MoELayer compiled from its
  sources (``ref_harness.cpp``); present only where it was built.
"""
from __future__ import annotations

import ctypes as ct
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libmgpt_ref.so")


class _Dims(ct.Structure):
    _fields_ = [("n_tokens", ct.c_int), ("C", ct.c_int), ("H", ct.c_int), ("E", ct.c_int),
                ("k", ct.c_int), ("alpha", ct.c_float)]


_FP = ct.POINTER(ct.c_float)
_IP = ct.POINTER(ct.c_int32)


class _Inputs(ct.Structure):
    _fields_ = [("x", _FP), ("params", ct.POINTER(_FP)), ("dy", _FP)]


class _Outputs(ct.Structure):
    _fields_ = [("logits", _FP), ("probs", _FP), ("top_idx", _IP), ("top_p", _FP), ("counts", _IP),
                ("offsets", _IP), ("map", _IP), ("gathered_out", _FP), ("y", _FP), ("d_top_p", _FP),
                ("dlogits", _FP), ("dx", _FP), ("grads", ct.POINTER(_FP))]


@dataclass(frozen=True)
class Dims:
    n_tokens: int
    C: int
    H: int
    E: int
    k: int
    alpha: float = 0.01


def param_shapes(C: int, H: int, E: int):
    """Shapes of the 2+6E parameter tensors in the reference's get_parameters() order
    (layers/MoELayer.cpp:225-236)."""
    shapes = [(C, E), (1, E)]
    for _ in range(E):
        shapes += [(C, H), (1, H), (C, H), (1, H), (H, C), (1, C)]
    return shapes


ENGINE_BIN = os.path.join(HERE, "_ref", "engine_moe_driver")


def reference_dir():
    """Checkout of the reference to compile ``_ref`` from: ``$MGPT_REFERENCE_DIR``, else a directory named
    ``reference`` beside this repository.  None when neither has the MoE layer's sources."""
    cands = [os.environ.get("MGPT_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "src", "main", "neuralnetwork", "layers", "MoELayer.cpp")):
            return c
    return None


def build(ref: bool = True) -> None:
    """Compile liboracle.so and, when a checkout of the reference is at hand, ``_ref/libmgpt_ref.so`` (its own
    MoELayer, CPU arm) and ``_ref/engine_moe_driver`` (its engine around this repository's adapter; needs the
    CUDA library built first)."""
    rd = reference_dir() if ref else None
    if rd is None:
        subprocess.run(["make", "-C", HERE, ORACLE_SO], check=True, stdout=subprocess.DEVNULL)
    else:
        subprocess.run(["make", "-C", HERE, "all", f"REF={rd}"], check=True, stdout=subprocess.DEVNULL)


def have_ref() -> bool:
    return os.path.exists(REF_SO)


_libs = {}


def _load(which: str):
    if which in _libs:
        return _libs[which]
    path = ORACLE_SO if which == "oracle" else REF_SO
    if which == "oracle" and not os.path.exists(path):
        build(ref=False)
    lib = ct.CDLL(path)
    names = ("moe_oracle_run", "moe_oracle_route") if which == "oracle" else ("moe_ref_run", "moe_ref_route")
    for n in names:
        fn = getattr(lib, n)
        fn.argtypes = [ct.POINTER(_Dims), ct.POINTER(_Inputs), ct.POINTER(_Outputs), ct.c_int]
        fn.restype = ct.c_int
    _libs[which] = (getattr(lib, names[0]), getattr(lib, names[1]))
    return _libs[which]


def _fp(a):
    return a.ctypes.data_as(_FP)


def run(dims: Dims, x, params, dy=None, *, which: str = "oracle", threads: int = 1,
        route_only: bool = False) -> dict:
    """Run forward (and backward when ``dy`` is given) on the CPU.

    ``x``/``dy`` are [N,C] float32, ``params`` the 2+6E float32 arrays.  Returns a dict
    with logits, probs, top_idx, top_p, counts, offsets, map and, unless ``route_only``,
    gathered_out, y, dx, grads (list), d_top_p and dlogits (restatement only).
    """
    N, C, H, E, k = dims.n_tokens, dims.C, dims.H, dims.E, dims.k
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(N, C)
    params = [np.ascontiguousarray(p, dtype=np.float32) for p in params]
    shapes = param_shapes(C, H, E)
    assert len(params) == len(shapes), "expected 2+6E parameter arrays"
    for p, s in zip(params, shapes):
        assert p.size == s[0] * s[1], f"parameter size {p.shape} does not match {s}"
    if dy is not None:
        dy = np.ascontiguousarray(dy, dtype=np.float32).reshape(N, C)

    d = _Dims(N, C, H, E, k, dims.alpha)
    parr = (_FP * len(params))(*[_fp(p) for p in params])
    inp = _Inputs(_fp(x), parr, _fp(dy) if dy is not None else None)

    R = N * k
    res = {
        "logits": np.zeros((N, E), np.float32), "probs": np.zeros((N, E), np.float32),
        "top_idx": np.zeros((N, k), np.int32), "top_p": np.zeros((N, k), np.float32),
        "counts": np.zeros(E, np.int32), "offsets": np.zeros(E, np.int32), "map": np.zeros(R, np.int32),
    }
    out = _Outputs()
    out.logits, out.probs, out.top_p = _fp(res["logits"]), _fp(res["probs"]), _fp(res["top_p"])
    out.top_idx = res["top_idx"].ctypes.data_as(_IP)
    out.counts = res["counts"].ctypes.data_as(_IP)
    out.offsets = res["offsets"].ctypes.data_as(_IP)
    out.map = res["map"].ctypes.data_as(_IP)
    grads = None
    if not route_only:
        res["gathered_out"] = np.zeros((R, C), np.float32)
        res["y"] = np.zeros((N, C), np.float32)
        out.gathered_out, out.y = _fp(res["gathered_out"]), _fp(res["y"])
        if dy is not None:
            res["dx"] = np.zeros((N, C), np.float32)
            res["d_top_p"] = np.zeros((N, k), np.float32)
            res["dlogits"] = np.zeros((N, E), np.float32)
            grads = [np.zeros(s, np.float32) for s in shapes]
            res["grads"] = grads
            out.dx, out.d_top_p, out.dlogits = _fp(res["dx"]), _fp(res["d_top_p"]), _fp(res["dlogits"])
            garr = (_FP * len(grads))(*[_fp(g) for g in grads])
            out.grads = garr
    full, route = _load(which)
    rc = (route if route_only else full)(ct.byref(d), ct.byref(inp), ct.byref(out), int(threads))
    if rc != 0:
        raise RuntimeError(f"{which} oracle returned {rc}")
    if which == "ref":
        res.pop("d_top_p", None)   # locals of the reference's backward; not observable
        res.pop("dlogits", None)
    return res


def bench(dims: Dims, x, params, dy=None, *, which: str = "oracle", iters: int = 1, threads: int = 1):
    """Times forward (+backward) on the CPU; returns the list of per-iteration seconds.
    Layer construction, parameter loading and gradient clearing are outside the timed region."""
    N, C = dims.n_tokens, dims.C
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(N, C)
    params = [np.ascontiguousarray(p, dtype=np.float32) for p in params]
    if dy is not None:
        dy = np.ascontiguousarray(dy, dtype=np.float32).reshape(N, C)
    d = _Dims(N, C, dims.H, dims.E, dims.k, dims.alpha)
    parr = (_FP * len(params))(*[_fp(p) for p in params])
    inp = _Inputs(_fp(x), parr, _fp(dy) if dy is not None else None)
    secs = (ct.c_double * iters)()
    _load(which)
    lib = ct.CDLL(ORACLE_SO if which == "oracle" else REF_SO)
    if which == "oracle":
        fn = lib.moe_oracle_bench
        fn.argtypes = [ct.POINTER(_Dims), ct.POINTER(_Inputs), ct.c_int, ct.POINTER(ct.c_double), ct.c_int]
        rc = fn(ct.byref(d), ct.byref(inp), iters, secs, int(threads))
    else:
        fn = lib.moe_ref_bench
        fn.argtypes = [ct.POINTER(_Dims), ct.POINTER(_Inputs), ct.c_int, ct.POINTER(ct.c_double)]
        rc = fn(ct.byref(d), ct.byref(inp), iters, secs)
    if rc != 0:
        raise RuntimeError(f"{which} bench returned {rc}")
    return list(secs)


def adamw(w, g, m, v, *, lr, beta1, beta2, eps, weight_decay, t, which: str = "oracle"):
    """One AdamW step on flat float32 arrays; returns new (w, m, v).  ``which``: "oracle" (C restatement of
    utils/Tensor.cpp:683-699) or "ref" (the reference's own Tensor::adamw_step)."""
    w, m, v = (np.array(a, dtype=np.float32).ravel() for a in (w, m, v))
    g = np.ascontiguousarray(g, dtype=np.float32).ravel()
    _load(which)
    lib = ct.CDLL(ORACLE_SO if which == "oracle" else REF_SO)
    fn = lib.moe_oracle_adamw if which == "oracle" else lib.moe_ref_adamw
    fn.argtypes = [_FP, _FP, _FP, _FP, ct.c_long] + [ct.c_float] * 5 + [ct.c_int]
    fn.restype = ct.c_int
    rc = fn(_fp(w), _fp(g), _fp(m), _fp(v), w.size, lr, beta1, beta2, eps, weight_decay, int(t))
    if rc != 0:
        raise RuntimeError(f"{which} adamw returned {rc}")
    return w, m, v


def rmsnorm(x, scale, dout, eps=1e-5, *, which: str = "numpy"):
    """RMSNorm forward and backward of the reference (utils/Tensor.cpp:785-800, 1674-1690) on [n, c] float32 arrays:
    returns (out, rs, dx, dscale).  ``which``: "numpy" (a restatement, float32 arithmetic, sums in float64 rounded
    once: within 1e-6 of the reference's sequential float32 sums) or "ref" (the reference's own Tensor code)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32).ravel()
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    n, c = x.shape
    if which == "ref":
        lib = ct.CDLL(REF_SO)
        fn = lib.moe_ref_rmsnorm
        fn.argtypes = [_FP, _FP, _FP, ct.c_int, ct.c_int, ct.c_float, _FP, _FP, _FP, _FP]
        out, rs = np.zeros((n, c), np.float32), np.zeros(n, np.float32)
        dx, ds = np.zeros((n, c), np.float32), np.zeros(c, np.float32)
        if fn(_fp(x), _fp(scale), _fp(dout), n, c, eps, _fp(out), _fp(rs), _fp(dx), _fp(ds)) != 0:
            raise RuntimeError("moe_ref_rmsnorm failed")
        return out, rs, dx, ds
    ms = (x.astype(np.float64) ** 2).sum(1) / c
    rs = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    xh = x * rs[:, None]
    out = xh * scale[None, :]
    dxh = dout * scale[None, :]
    dot = (dxh.astype(np.float64) * xh).sum(1).astype(np.float32)
    dx = rs[:, None] * (dxh - xh * (dot / np.float32(c))[:, None])
    ds = (dout.astype(np.float64) * xh).sum(0).astype(np.float32)
    return out.astype(np.float32), rs, dx.astype(np.float32), ds
