"""Seeded synthetic workloads for the MoE layer.

The benchmark configurations are the five the baseline names; every tensor is
drawn on the host from one counter-based generator (Philox keyed by seed and
tensor id), so the CPU oracle and the GPU see identical bits.  No dataset is
involved anywhere on this path.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np


@dataclass(frozen=True)
class Workload:
    name: str
    n_tokens: int
    C: int          # embed_dim
    H: int          # SwiGLU hidden_dim
    E: int          # num_experts
    k: int          # top_k
    dtype: str      # "fp32" or "bf16"
    skew: bool = False      # router bias b_e = 2*ln(1/(e+1))
    backward: bool = True
    alpha: float = 0.01     # load-balance coefficient (layers/MoELayer.cpp:194)

    def scaled(self, n_tokens: int, name: str | None = None) -> "Workload":
        return replace(self, n_tokens=n_tokens, name=name or f"{self.name}@{n_tokens}")


WORKLOADS = {
    "c1": Workload("c1", 1024, 128, 512, 8, 2, "fp32"),
    "c2": Workload("c2", 8192, 512, 1376, 16, 2, "bf16"),
    "c3": Workload("c3", 16384, 1024, 512, 64, 4, "bf16", skew=True),
    "c4": Workload("c4", 32768, 2048, 1408, 64, 2, "bf16"),
    # a quarter of c4 (same rows per expert, so the same tiles per expert): small enough for multi-pass profiling
    "c4q": Workload("c4q", 8192, 2048, 1408, 16, 2, "bf16"),
    # c4's tokens, router and permutation with token experts of 64 hidden units: the router, dispatch and combine
    # kernels at their full-size shapes in ~1.5 GB, for multi-pass profiling
    "c4r": Workload("c4r", 32768, 2048, 64, 64, 2, "bf16"),
    "c5-8": Workload("c5-8", 8, 1024, 2816, 32, 2, "bf16", backward=False),
    "c5-64": Workload("c5-64", 64, 1024, 2816, 32, 2, "bf16", backward=False),
    "c5-256": Workload("c5-256", 256, 1024, 2816, 32, 2, "bf16", backward=False),
}


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even) and return it as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(a.shape)


def param_shapes(C: int, H: int, E: int):
    """2+6E parameter shapes in the reference's get_parameters() order
    (layers/MoELayer.cpp:225-236; layers/SwiGLU.cpp:98-104)."""
    shapes = [(C, E), (1, E)]
    for _ in range(E):
        shapes += [(C, H), (1, H), (C, H), (1, H), (H, C), (1, C)]
    return shapes


def _normal(seed: int, tensor_id: int, shape, std: float) -> np.ndarray:
    gen = np.random.Generator(np.random.Philox(key=[seed, tensor_id]))
    a = gen.standard_normal(size=shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return a


def make_param(w: Workload, i: int, seed: int = 1234, bias_std: float = 0.0) -> np.ndarray:
    """Parameter tensor ``i`` (index in the 2+6E order) of ``make_inputs(w, seed, bias_std)``, alone: what an
    expert-parallel rank calls for the tensors it owns."""
    s = param_shapes(w.C, w.H, w.E)[i]
    if s[0] == 1:
        p = _normal(seed, 2 + i, s, bias_std) if bias_std > 0 else np.zeros(s, np.float32)
        if i == 1 and w.skew:
            p = p + (2.0 * np.log(1.0 / (np.arange(w.E, dtype=np.float64) + 1.0))).astype(np.float32)[None, :]
    else:
        p = _normal(seed, 2 + i, s, 0.02)
    return bf16_round(p) if w.dtype == "bf16" else p


def make_tokens(w: Workload, seed: int = 1234):
    """(x, dy) of ``make_inputs(w, seed)``, alone."""
    x = _normal(seed, 0, (w.n_tokens, w.C), 1.0)
    dy = _normal(seed, 1, (w.n_tokens, w.C), 1.0)
    if w.dtype == "bf16":
        x, dy = bf16_round(x), bf16_round(dy)
    return x, dy


def make_inputs(w: Workload, seed: int = 1234, bias_std: float = 0.0):
    """Returns (x [N,C], params list, dy [N,C]) as float32 arrays.

    x, dy ~ N(0,1); weights ~ N(0,0.02); biases 0 (the reference's init,
    layers/LinearLayer.cpp:19) unless ``bias_std`` asks for trained-looking ones;
    with ``skew`` the router bias is 2*ln(1/(e+1)).  For bf16 workloads every
    tensor is rounded to bf16 once, so the oracle consumes the same values.
    """
    x = _normal(seed, 0, (w.n_tokens, w.C), 1.0)
    dy = _normal(seed, 1, (w.n_tokens, w.C), 1.0)
    params = []
    for i, s in enumerate(param_shapes(w.C, w.H, w.E)):
        if s[0] == 1:
            p = _normal(seed, 2 + i, s, bias_std) if bias_std > 0 else np.zeros(s, np.float32)
            if i == 1 and w.skew:
                p = p + (2.0 * np.log(1.0 / (np.arange(w.E, dtype=np.float64) + 1.0))).astype(np.float32)[None, :]
        else:
            p = _normal(seed, 2 + i, s, 0.02)
        params.append(p)
    if w.dtype == "bf16":
        x, dy = bf16_round(x), bf16_round(dy)
        params = [bf16_round(p) for p in params]
    return x, params, dy
