"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from mgpt_b200 import MoELayer
from oracle import oracle


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a))


def dims_of(w):
    return oracle.Dims(w.n_tokens, w.C, w.H, w.E, w.k, w.alpha)


def run_layer(w, x, params, dy, *, mode, gemm_impl=0, io=torch.float32):
    """Runs forward (+backward) through the C ABI; returns a dict shaped like the oracle's."""
    layer = MoELayer(w.C, w.H, w.E, w.k, mode=mode, gemm_impl=gemm_impl, lb_alpha=w.alpha)
    layer.load_parameters(params)
    layer.zero_grad()
    xt = torch.from_numpy(x).cuda().to(io).contiguous()
    y = layer.forward(xt)
    N, E, k = w.n_tokens, w.E, w.k
    out = {"layer": layer, "y": y.float().cpu().numpy()}
    # BF16 tokens on the tensor-core path take the screened router: indices exact, logits / probabilities close
    import os
    min_work = float(os.environ.get("MGPT_MOE_ROUTER_TC_MIN_WORK", "4e8"))      # the library's own rule
    out["screened"] = (mode == "bf16" and gemm_impl == 0 and io == torch.bfloat16
                       and float(w.n_tokens) * w.C * w.E >= min_work)
    out["router_recompute"] = int(layer.workspace_view("router_recompute", torch.int32).cpu().numpy()[0]) if out["screened"] else 0
    i32, f32 = torch.int32, torch.float32
    out["logits"] = layer.workspace_view("logits", f32, (N, E)).cpu().numpy()
    out["probs"] = layer.workspace_view("probs", f32, (N, E)).cpu().numpy()
    out["top_idx"] = layer.workspace_view("top_idx", i32, (N, k)).cpu().numpy()
    out["top_p"] = layer.workspace_view("top_p", f32, (N, k)).cpu().numpy()
    out["counts"] = layer.workspace_view("counts", i32).cpu().numpy()
    out["offsets"] = layer.workspace_view("offsets", i32).cpu().numpy()
    out["map"] = layer.workspace_view("map", i32).cpu().numpy()
    out["padded_offsets"] = layer.workspace_view("padded_offsets", i32).cpu().numpy()
    out["pos"] = layer.workspace_view("pos", i32).cpu().numpy()
    if dy is not None:
        dyt = torch.from_numpy(dy).cuda().to(io).contiguous()
        dx = layer.backward(dyt)
        out["dx"] = dx.float().cpu().numpy()
        out["grads"] = [p.grad.cpu().numpy() for p in layer.get_parameters()]
        out["d_top_p"] = layer.workspace_view("d_top_p", f32, (N, k)).cpu().numpy()
        out["dlogits"] = layer.workspace_view("dlogits", f32, (N, E)).cpu().numpy()
    torch.cuda.synchronize()
    # the per-step word of the plan in the workspace, and every bit any kernel of the layer has set since creation
    out["status"] = int(layer.workspace_view("status", i32).cpu().numpy()[0]) | layer.status_bits()
    return out


def assert_routing_exact(got, ref):
    """Routing indices, per-expert counts and the slot permutation must be bit-exact."""
    for key in ("top_idx", "counts", "offsets", "map"):
        assert np.array_equal(got[key], ref[key]), f"{key} differs from the CPU reference"
    if got.get("screened"):
        # tensor-core first pass: same sums in another order (tokens of the exact second pass are bit-exact)
        assert np.abs(got["logits"] - ref["logits"]).max() <= 2e-5 * (1.0 + np.abs(ref["logits"]).max())
        assert np.allclose(got["top_p"], ref["top_p"], rtol=1e-4, atol=0)
        assert np.allclose(got["probs"], ref["probs"], rtol=1e-4, atol=0)
    else:
        assert np.array_equal(got["logits"], ref["logits"]), "router logits are not bit-exact"
        # probabilities differ from glibc's expf by at most an ulp or two
        assert np.allclose(got["top_p"], ref["top_p"], rtol=1e-6, atol=0)
    assert got["status"] == 0


def assert_values(got, ref, tol, w):
    assert rel_l2(got["y"], ref["y"]) <= tol, ("y", rel_l2(got["y"], ref["y"]))
    if "dx" in ref:
        assert rel_l2(got["dx"], ref["dx"]) <= tol, ("dx", rel_l2(got["dx"], ref["dx"]))
        for i, (a, b) in enumerate(zip(got["grads"], ref["grads"])):
            e = rel_l2(a, b)
            # an expert with no rows has exactly zero gradients on both sides
            assert e <= tol, (f"grad {i}", e)


# ---- dispatch plan, operator level ---------------------------------------------------------------
PLAN_OUTPUTS = ("counts", "offsets", "padded_offsets", "tile_expert", "n_tiles", "map", "pos", "row_src", "status")


def plan_row_cap(n_rows: int, E: int) -> int:
    return max(1, (n_rows + E * 127) // 128) * 128


def plan_reference(top_idx: np.ndarray, E: int) -> dict:
    """numpy statement of the plan (stable slots, segments padded to 128 rows)."""
    flat = np.asarray(top_idx, dtype=np.int64).reshape(-1)
    R = flat.size
    counts = np.bincount(flat, minlength=E).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
    padded = (counts + 127) // 128 * 128
    poff = np.concatenate([[0], np.cumsum(padded)]).astype(np.int32)
    order = np.argsort(flat, kind="stable").astype(np.int32)          # slot -> flat index
    rank = np.empty(R, np.int64)
    rank[order] = np.arange(R) - offsets[flat[order]]
    pos = (poff[flat] + rank).astype(np.int32)
    row_cap = plan_row_cap(R, E)
    row_src = np.full(row_cap, -1, np.int32)
    row_src[pos] = np.arange(R, dtype=np.int32)
    n_tiles = int(poff[-1]) // 128
    tile_expert = np.repeat(np.arange(E, dtype=np.int32), padded // 128)
    return {"counts": counts, "offsets": offsets, "padded_offsets": poff, "tile_expert": tile_expert,
            "n_tiles": np.array([n_tiles], np.int32), "map": order, "pos": pos, "row_src": row_src,
            "status": np.array([0], np.int32)}


def plan_buffers(n_rows: int, E: int, device="cuda") -> dict:
    row_cap = plan_row_cap(n_rows, E)
    sizes = {"counts": E, "offsets": E, "padded_offsets": E + 1, "tile_expert": row_cap // 128, "n_tiles": 1,
             "map": max(1, n_rows), "pos": max(1, n_rows), "row_src": row_cap, "status": 1}
    return {k: torch.full((v,), -7, dtype=torch.int32, device=device) for k, v in sizes.items()}


def assert_plan_equal(bufs: dict, ref: dict, n_rows: int) -> None:
    """Integer work: every output must match exactly (tile_expert only over the tiles in use)."""
    nt = int(ref["n_tiles"][0])
    for key in PLAN_OUTPUTS:
        got = bufs[key].cpu().numpy()
        want = ref[key]
        if key == "tile_expert":
            got = got[:nt]
        elif key in ("map", "pos"):
            got = got[:n_rows]
        elif key == "row_src":            # defined for the rows of the plan's tiles; beyond them nothing is written
            got, want = got[:nt * 128], want[:nt * 128]
        assert np.array_equal(got, want), key
