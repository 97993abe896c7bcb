// Stage-level entry points: the layer cut at its two exchange points, for
// expert-parallel execution.  A routing-side layer (router parameters only)
// turns tokens into expert-major rows and back; an expert-side layer (top_k
// = 1, expert parameters only) runs the grouped SwiGLU products on the rows it
// receives.  Between the two the caller moves rows with whatever transport it
// has (NCCL all-to-all in mgpt_b200/ep.py).
//
// Rows travel tile-aligned: every expert's segment is padded to whole 128-row
// tiles (zero rows) on the routing side, exactly the layout the single-GPU
// layer uses internally.  The block for a destination GPU is therefore one
// contiguous range, and what arrives - one block per source rank, inside it
// one padded segment per local expert - can be fed to the tensor-core kernels
// where it lands: the expert side moves no rows at all.
//
// The reference has no multi-GPU code; these calls split what its
// MoELayer::forward_into / backward_into do in one piece
// (layers/MoELayer.cpp:52-83 | 94-118 | 121-123 and 156 | 159-181 | 184-218).
#include "common.cuh"

using namespace mgpt;

namespace {

int check_ws(const mgpt_moe_layer* L, const void* ws, size_t ws_bytes, const Workspace& w)
{
    if (!ws || ((uintptr_t)ws & 255)) return fail(MGPT_MOE_EINVAL, "workspace must be 256-byte aligned");
    if (ws_bytes < w.total) return fail(MGPT_MOE_ENOMEM, "workspace smaller than mgpt_moe_stage_workspace_bytes()");
    (void)L;
    return 0;
}
int act_io(const Workspace& w) { return w.act_bytes == 2 ? MGPT_MOE_IO_BF16 : MGPT_MOE_IO_F32; }

int check_route_layer(const mgpt_moe_layer* L, int io)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->router_bound) return fail(MGPT_MOE_ESTATE, "router parameters are not bound");
    if (io != MGPT_MOE_IO_F32 && io != MGPT_MOE_IO_BF16) return fail(MGPT_MOE_EINVAL, "unknown io dtype");
    if (L->d.mode == MGPT_MOE_FP32 && io != MGPT_MOE_IO_F32) return fail(MGPT_MOE_EINVAL, "FP32 mode takes FP32 tokens");
    return 0;
}
int check_expert_layer(const mgpt_moe_layer* L)
{
    if (!L) return fail(MGPT_MOE_EINVAL, "null layer");
    if (!L->experts_bound) return fail(MGPT_MOE_ESTATE, "expert parameters are not bound");
    if (L->d.k != 1) return fail(MGPT_MOE_EINVAL, "the expert side is a layer created with top_k = 1");
    if (L->d.mode == MGPT_MOE_BF16 && !L->shadows_fresh)
        return fail(MGPT_MOE_ESTATE, "sync_weights after bind_params / optimiser step");
    return 0;
}

}  // namespace

extern "C" {

size_t mgpt_moe_stage_workspace_bytes(const mgpt_moe_layer* L, int n, int routing_side)
{
    if (!L || n < 0) return 0;
    return make_workspace(L->d, n, routing_side ? 1 : 2).total;
}

// router + plan: after this the per-expert counts are final (workspace view "counts")
int mgpt_moe_route_plan(mgpt_moe_layer* L, const void* x, int n_tokens, int io, void* workspace, size_t ws_bytes,
                        mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (n_tokens < 0 || (n_tokens > 0 && !x)) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    const Workspace w = make_workspace(L->d, n_tokens, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->fwd_done = false;
    if (n_tokens > 0) {
        if (tc_router_usable(L, x, io, n_tokens))
            MGPT_TRY(tc_router_fwd(L, w, ws, x, st));
        else
            MGPT_TRY(launch_router_fwd(x, io, L->p_data[0], L->p_data[1], n_tokens, d.C, d.E, d.k, (float*)(ws + w.logits),
                                       (float*)(ws + w.probs), (int32_t*)(ws + w.top_idx), (float*)(ws + w.top_p), st));
    }
    MGPT_TRY(launch_plan(d, w, ws, st, L->d_status));
    L->last_n = n_tokens;
    L->last_io = io;
    L->last_ws = workspace;
    L->last_stream = st;
    return 0;
}

// the permutation of the tokens into send_rows, for the plan mgpt_moe_route_plan left in the workspace
int mgpt_moe_route_rows(mgpt_moe_layer* L, const void* x, int io, void* workspace, size_t ws_bytes, void* send_rows,
                        mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (workspace != L->last_ws || io != L->last_io) return fail(MGPT_MOE_ESTATE, "route_rows follows route_plan on the same workspace");
    const int n_tokens = L->last_n;
    if (n_tokens > 0 && (!x || !send_rows)) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    const Workspace w = make_workspace(L->d, n_tokens, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    MGPT_CUDA(cudaSetDevice(L->device));
    char* ws = (char*)workspace;
    // expert-major rows, each expert padded to whole tiles with zero rows; stable within an expert
    MGPT_TRY(gather_rows(x, io, (const int32_t*)(ws + w.row_src), (const int32_t*)(ws + w.n_tiles), -1, w.row_cap, L->d.C,
                         L->d.k, send_rows, w.act_bytes, (cudaStream_t)stream));
    L->fwd_done = true;
    return 0;
}

int mgpt_moe_route(mgpt_moe_layer* L, const void* x, int n_tokens, int io, void* workspace, size_t ws_bytes,
                   void* send_rows, mgpt_stream_t stream)
{
    if (n_tokens > 0 && !send_rows) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    MGPT_TRY(mgpt_moe_route_plan(L, x, n_tokens, io, workspace, ws_bytes, stream));
    return mgpt_moe_route_rows(L, x, io, workspace, ws_bytes, send_rows, stream);
}

int mgpt_moe_combine(mgpt_moe_layer* L, const void* rows_back, void* y, int io, void* workspace, size_t ws_bytes,
                     mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (!L->fwd_done || workspace != L->last_ws) return fail(MGPT_MOE_ESTATE, "combine needs the workspace of the last route");
    const Workspace w = make_workspace(L->d, L->last_n, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    if (L->last_n > 0 && (!rows_back || !y)) return fail(MGPT_MOE_EINVAL, "null buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    char* ws = (char*)workspace;
    return combine_rows(rows_back, (const int32_t*)(ws + w.pos), (const float*)(ws + w.top_p), w.n_tokens, L->d.C,
                        L->d.k, y, io, w.act_bytes, (cudaStream_t)stream);
}

int mgpt_moe_combine_backward(mgpt_moe_layer* L, const void* rows_back, const void* dy, int io, void* d_rows,
                              void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (!L->fwd_done || workspace != L->last_ws) return fail(MGPT_MOE_ESTATE, "backward needs the workspace of the last route");
    const Workspace w = make_workspace(L->d, L->last_n, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    if (L->last_n > 0 && (!rows_back || !dy || !d_rows)) return fail(MGPT_MOE_EINVAL, "null buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    char* ws = (char*)workspace;
    return combine_rows_backward(dy, io, rows_back, (const int32_t*)(ws + w.row_src), (const float*)(ws + w.top_p),
                                 (const int32_t*)(ws + w.n_tiles), -1, w.row_cap, L->d.C, L->d.k, d_rows,
                                 (float*)(ws + w.d_top_p), w.act_bytes, (cudaStream_t)stream);
}

int mgpt_moe_route_backward(mgpt_moe_layer* L, const void* x, const void* d_rows_in, void* dx, int io,
                            void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (!L->fwd_done || workspace != L->last_ws) return fail(MGPT_MOE_ESTATE, "backward needs the workspace of the last route");
    const Workspace w = make_workspace(L->d, L->last_n, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    if (L->last_n == 0) return 0;
    if (!x || !d_rows_in || !dx) return fail(MGPT_MOE_EINVAL, "null buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    char* ws = (char*)workspace;
    return launch_router_bwd(L, w, ws, x, io, dx, (cudaStream_t)stream, d_rows_in, (const int32_t*)(ws + w.pos));
}

int mgpt_moe_experts_forward(mgpt_moe_layer* L, const void* rows, const int32_t* seg_counts, int n_src, int n_rows,
                             void* out_rows, void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    MGPT_TRY(check_expert_layer(L));
    if (n_rows < 0 || n_rows % ROW_TILE) return fail(MGPT_MOE_EINVAL, "n_rows must be a multiple of 128 (padded segments)");
    if (n_src < 1 || n_src > MAX_SOURCES) return fail(MGPT_MOE_EINVAL, "n_src must be in 1..64");
    if (!seg_counts || (n_rows > 0 && (!rows || !out_rows))) return fail(MGPT_MOE_EINVAL, "null buffer");
    const Workspace w = make_workspace(L->d, n_rows, 2);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->fwd_done = false;
    for (int s = 0; s < ST_COUNT; ++s) L->ev_used[s] = false;
    L->ext_Xg = const_cast<void*>(rows);
    L->ext_Yg = out_rows;
    L->ext_dYg = L->ext_dXg = nullptr;
    L->n_seg = n_src;
    // tile -> expert table in arrival order and every expert's segment list, from the real counts
    L->stage_begin(ST_PLAN, st);
    MGPT_TRY(launch_segment_tiles(d, w, ws, seg_counts, n_src, st, L->d_status));
    L->stage_end(ST_PLAN, st);
    if (n_rows > 0) {
        if (d.mode == MGPT_MOE_BF16 && d.gemm_impl == 0) MGPT_TRY(tc_experts_forward(L, w, ws, st));
        else MGPT_TRY(simt_experts_forward(L, w, ws, st));
    }
    L->last_n = n_rows;
    L->last_io = act_io(w);
    L->last_ws = workspace;
    L->last_stream = st;
    L->fwd_done = true;
    return 0;
}

static int experts_backward_impl(mgpt_moe_layer* L, const void* d_out_rows, void* d_in_rows, void* workspace,
                                 size_t ws_bytes, mgpt_stream_t stream, int phase)
{
    MGPT_TRY(check_expert_layer(L));
    if (!L->fwd_done || workspace != L->last_ws) return fail(MGPT_MOE_ESTATE, "backward needs the workspace of the last forward");
    const int n_rows = L->last_n;
    const Workspace w = make_workspace(L->d, n_rows, 2);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    if (n_rows == 0) return 0;
    if (!d_out_rows || !d_in_rows) return fail(MGPT_MOE_EINVAL, "null buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->ext_dYg = const_cast<void*>(d_out_rows);      // padding rows arrive as zeros from the routing side
    L->ext_dXg = d_in_rows;
    const bool tc = d.mode == MGPT_MOE_BF16 && d.gemm_impl == 0;
    if (tc) {
        MGPT_TRY(tc_experts_backward(L, w, ws, st, phase));
    } else if (phase & 1) {
        MGPT_TRY(simt_experts_backward(L, w, ws, st));     // the CUDA-core path computes both kinds in one go
    }
    if ((phase & 2) && L->has_grad && !(tc && tc_fused_bias_grads(d))) {      // else the tensor-core weight-gradient kernel sums them itself
        L->stage_begin(ST_BIAS_GRAD, st);
        MGPT_TRY(launch_bias_grads(L, w, ws, st));
        L->stage_end(ST_BIAS_GRAD, st);
    }
    return 0;
}

int mgpt_moe_experts_backward(mgpt_moe_layer* L, const void* d_out_rows, void* d_in_rows, void* workspace,
                              size_t ws_bytes, mgpt_stream_t stream)
{
    return experts_backward_impl(L, d_out_rows, d_in_rows, workspace, ws_bytes, stream, 3);
}

int mgpt_moe_experts_backward_rows(mgpt_moe_layer* L, const void* d_out_rows, void* d_in_rows, void* workspace,
                                   size_t ws_bytes, mgpt_stream_t stream)
{
    return experts_backward_impl(L, d_out_rows, d_in_rows, workspace, ws_bytes, stream, 1);
}

int mgpt_moe_experts_backward_params(mgpt_moe_layer* L, const void* d_out_rows, void* d_in_rows, void* workspace,
                                     size_t ws_bytes, mgpt_stream_t stream)
{
    return experts_backward_impl(L, d_out_rows, d_in_rows, workspace, ws_bytes, stream, 2);
}

}  // extern "C"
