"""ctypes binding of ``libmgpt_moe.so`` (the C ABI in ``include/mgpt_moe.h``)."""
from __future__ import annotations

import ctypes as ct
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libmgpt_moe.so")

FP32, BF16 = 0, 1
IO_F32, IO_BF16 = 0, 1

# every symbol include/mgpt_moe.h declares
SYMBOLS = [
    "mgpt_moe_create", "mgpt_moe_destroy", "mgpt_moe_last_error", "mgpt_moe_num_params",
    "mgpt_moe_param_shape", "mgpt_moe_bind_params", "mgpt_moe_sync_weights", "mgpt_moe_workspace_bytes",
    "mgpt_moe_forward", "mgpt_moe_backward", "mgpt_moe_expert_counts", "mgpt_moe_workspace_view",
    "mgpt_moe_step_host", "mgpt_moe_step_host_async", "mgpt_moe_step_host_wait", "mgpt_moe_launch_count", "mgpt_moe_op_router",
    "mgpt_moe_set_profiling", "mgpt_moe_stage_ms", "mgpt_moe_stage_name", "mgpt_moe_set_sm_budget", "mgpt_moe_bind_optimizer_state", "mgpt_moe_adamw_step",
    "mgpt_moe_forward_residual", "mgpt_moe_routing_bytes", "mgpt_moe_save_routing", "mgpt_moe_forward_with_routing",
    "mgpt_moe_op_plan", "mgpt_moe_op_plan_scratch_bytes", "mgpt_moe_op_plan_noalloc",
    "mgpt_moe_stage_workspace_bytes", "mgpt_moe_route", "mgpt_moe_combine", "mgpt_moe_combine_backward",
    "mgpt_moe_route_backward", "mgpt_moe_experts_forward", "mgpt_moe_experts_backward",
    "mgpt_moe_check_status", "mgpt_moe_adamw_step_guarded", "mgpt_moe_selftest_bounded_wait",
    "mgpt_moe_ep_unique_id", "mgpt_moe_ep_create", "mgpt_moe_ep_destroy", "mgpt_moe_ep_num_params",
    "mgpt_moe_ep_global_expert", "mgpt_moe_ep_bind_params", "mgpt_moe_ep_sync_weights", "mgpt_moe_ep_forward",
    "mgpt_moe_ep_backward", "mgpt_moe_ep_received_counts", "mgpt_moe_ep_check_status",
    "mgpt_moe_route_plan", "mgpt_moe_route_rows",
    "mgpt_moe_peer_alloc", "mgpt_moe_peer_open", "mgpt_moe_peer_close", "mgpt_moe_peer_free", "mgpt_moe_peer_copy",
    "mgpt_moe_block_workspace_bytes", "mgpt_moe_block_forward", "mgpt_moe_block_backward",
    "mgpt_moe_set_weight_grad_overwrite", "mgpt_moe_inference_workspace_bytes", "mgpt_moe_forward_inference", "mgpt_moe_experts_backward_rows", "mgpt_moe_experts_backward_params",
]
PLAN_NOALLOC_MAX_ROWS = 1048576
PEER_HANDLE_BYTES = 64
N_STAGES = 12


class Config(ct.Structure):
    _fields_ = [("embed_dim", ct.c_int), ("hidden_dim", ct.c_int), ("num_experts", ct.c_int),
                ("top_k", ct.c_int), ("lb_alpha", ct.c_float), ("mode", ct.c_int), ("device", ct.c_int),
                ("gemm_impl", ct.c_int)]


class EpConfig(ct.Structure):
    _fields_ = [("embed_dim", ct.c_int), ("hidden_dim", ct.c_int), ("num_experts", ct.c_int), ("top_k", ct.c_int),
                ("lb_alpha", ct.c_float), ("mode", ct.c_int), ("device", ct.c_int), ("rank", ct.c_int),
                ("world", ct.c_int), ("n_chunks", ct.c_int), ("max_tokens", ct.c_int)]


EP_ID_BYTES = 128


class MoeError(RuntimeError):
    pass


_lib = None


def load() -> ct.CDLL:
    """Loads the CUDA library. There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MoeError(f"{LIB_PATH} is missing: build it with `python -m mgpt_b200.build` "
                       "(the layer has no CPU or PyTorch fallback)")
    lib = ct.CDLL(LIB_PATH)
    vp, i32, sz = ct.c_void_p, ct.c_int, ct.c_size_t
    lib.mgpt_moe_create.argtypes = [ct.POINTER(Config), ct.POINTER(vp)]
    lib.mgpt_moe_destroy.argtypes = [vp]
    lib.mgpt_moe_destroy.restype = None
    lib.mgpt_moe_last_error.restype = ct.c_char_p
    lib.mgpt_moe_num_params.argtypes = [vp]
    lib.mgpt_moe_param_shape.argtypes = [vp, i32, ct.POINTER(i32), ct.POINTER(i32)]
    lib.mgpt_moe_bind_params.argtypes = [vp, ct.POINTER(vp), ct.POINTER(vp), i32]
    lib.mgpt_moe_sync_weights.argtypes = [vp, vp]
    lib.mgpt_moe_workspace_bytes.argtypes = [vp, i32]
    lib.mgpt_moe_workspace_bytes.restype = sz
    lib.mgpt_moe_forward.argtypes = [vp, vp, vp, i32, i32, vp, sz, vp]
    lib.mgpt_moe_forward_inference.argtypes = [vp, vp, vp, i32, i32, vp, sz, vp]
    lib.mgpt_moe_inference_workspace_bytes.argtypes = [vp, i32]
    lib.mgpt_moe_inference_workspace_bytes.restype = sz
    lib.mgpt_moe_backward.argtypes = [vp, vp, vp, vp, i32, vp, sz, vp]
    lib.mgpt_moe_expert_counts.argtypes = [vp, ct.POINTER(ct.c_int32)]
    lib.mgpt_moe_workspace_view.argtypes = [vp, i32, ct.c_char_p, ct.POINTER(sz), ct.POINTER(sz)]
    lib.mgpt_moe_step_host.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp]
    lib.mgpt_moe_step_host_async.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp]
    lib.mgpt_moe_step_host_wait.argtypes = [vp]
    lib.mgpt_moe_launch_count.argtypes = [i32]
    lib.mgpt_moe_launch_count.restype = ct.c_long
    lib.mgpt_moe_set_profiling.argtypes = [vp, i32]
    lib.mgpt_moe_set_sm_budget.argtypes = [vp, i32]
    lib.mgpt_moe_set_weight_grad_overwrite.argtypes = [vp, i32]
    lib.mgpt_moe_forward_residual.argtypes = [vp, vp, vp, vp, i32, i32, vp, ct.c_size_t, vp]
    lib.mgpt_moe_routing_bytes.argtypes = [vp, i32]
    lib.mgpt_moe_routing_bytes.restype = ct.c_size_t
    lib.mgpt_moe_save_routing.argtypes = [vp, vp, vp]
    lib.mgpt_moe_forward_with_routing.argtypes = [vp, vp, vp, i32, i32, vp, ct.c_size_t, vp, vp]
    lib.mgpt_moe_bind_optimizer_state.argtypes = [vp, ct.POINTER(vp), ct.POINTER(vp), i32]
    lib.mgpt_moe_adamw_step.argtypes = [vp] + [ct.c_float] * 5 + [i32, vp]
    lib.mgpt_moe_adamw_step_guarded.argtypes = [vp] + [ct.c_float] * 5 + [i32, ct.c_float, i32, vp]
    lib.mgpt_moe_check_status.argtypes = [vp, ct.POINTER(ct.c_int32)]
    lib.mgpt_moe_selftest_bounded_wait.argtypes = [vp, vp]
    lib.mgpt_moe_stage_ms.argtypes = [vp, ct.POINTER(ct.c_float)]
    lib.mgpt_moe_stage_name.argtypes = [i32]
    lib.mgpt_moe_stage_name.restype = ct.c_char_p
    lib.mgpt_moe_op_router.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp]
    lib.mgpt_moe_op_plan_scratch_bytes.argtypes = [i32, i32]
    lib.mgpt_moe_op_plan_scratch_bytes.restype = sz
    lib.mgpt_moe_op_plan.argtypes = [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, sz, vp]
    lib.mgpt_moe_stage_workspace_bytes.argtypes = [vp, i32, i32]
    lib.mgpt_moe_stage_workspace_bytes.restype = sz
    lib.mgpt_moe_route.argtypes = [vp, vp, i32, i32, vp, sz, vp, vp]
    lib.mgpt_moe_route_plan.argtypes = [vp, vp, i32, i32, vp, sz, vp]
    lib.mgpt_moe_route_rows.argtypes = [vp, vp, i32, vp, sz, vp, vp]
    lib.mgpt_moe_combine.argtypes = [vp, vp, vp, i32, vp, sz, vp]
    lib.mgpt_moe_combine_backward.argtypes = [vp, vp, vp, i32, vp, vp, sz, vp]
    lib.mgpt_moe_route_backward.argtypes = [vp, vp, vp, vp, i32, vp, sz, vp]
    lib.mgpt_moe_experts_forward.argtypes = [vp, vp, vp, i32, i32, vp, vp, sz, vp]
    lib.mgpt_moe_experts_backward.argtypes = [vp, vp, vp, vp, sz, vp]
    lib.mgpt_moe_experts_backward_rows.argtypes = [vp, vp, vp, vp, sz, vp]
    lib.mgpt_moe_experts_backward_params.argtypes = [vp, vp, vp, vp, sz, vp]
    lib.mgpt_moe_ep_unique_id.argtypes = [vp]
    lib.mgpt_moe_ep_create.argtypes = [ct.POINTER(EpConfig), vp, ct.POINTER(vp)]
    lib.mgpt_moe_ep_destroy.argtypes = [vp]
    lib.mgpt_moe_ep_destroy.restype = None
    lib.mgpt_moe_ep_num_params.argtypes = [vp]
    lib.mgpt_moe_ep_global_expert.argtypes = [vp, i32]
    lib.mgpt_moe_ep_bind_params.argtypes = [vp, ct.POINTER(vp), ct.POINTER(vp), i32]
    lib.mgpt_moe_ep_sync_weights.argtypes = [vp, vp]
    lib.mgpt_moe_ep_forward.argtypes = [vp, vp, vp, i32, i32, vp]
    lib.mgpt_moe_ep_backward.argtypes = [vp, vp, vp, vp, i32, vp]
    lib.mgpt_moe_ep_received_counts.argtypes = [vp, ct.POINTER(ct.c_int32)]
    lib.mgpt_moe_ep_check_status.argtypes = [vp]
    lib.mgpt_moe_peer_alloc.argtypes = [i32, sz, ct.POINTER(vp), vp]
    lib.mgpt_moe_peer_open.argtypes = [i32, vp, ct.POINTER(vp)]
    lib.mgpt_moe_peer_close.argtypes = [i32, vp]
    lib.mgpt_moe_peer_free.argtypes = [i32, vp]
    lib.mgpt_moe_peer_copy.argtypes = [vp, vp, sz, vp]
    lib.mgpt_moe_block_workspace_bytes.argtypes = [vp, i32, i32]
    lib.mgpt_moe_block_workspace_bytes.restype = sz
    lib.mgpt_moe_block_forward.argtypes = [vp, vp, vp, ct.c_float, vp, i32, i32, vp, sz, vp]
    lib.mgpt_moe_block_backward.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp, sz, vp]
    lib.mgpt_moe_op_plan_noalloc.argtypes = [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp]
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().mgpt_moe_last_error()
        raise MoeError(f"mgpt_moe error {rc}: {msg.decode() if msg else '?'}")
