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
    out["status"] = int(layer.workspace_view("status", i32).cpu().numpy()[0])
    if dy is not None:
        dyt = torch.from_numpy(dy).cuda().to(io).contiguous()
        dx = layer.backward(dyt)
        out["dx"] = dx.float().cpu().numpy()
        out["grads"] = [p.grad.cpu().numpy() for p in layer.get_parameters()]
        out["d_top_p"] = layer.workspace_view("d_top_p", f32, (N, k)).cpu().numpy()
        out["dlogits"] = layer.workspace_view("dlogits", f32, (N, E)).cpu().numpy()
    torch.cuda.synchronize()
    return out


def assert_routing_exact(got, ref):
    """Routing indices, per-expert counts and the slot permutation must be bit-exact."""
    for key in ("top_idx", "counts", "offsets", "map"):
        assert np.array_equal(got[key], ref[key]), f"{key} differs from the CPU reference"
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
