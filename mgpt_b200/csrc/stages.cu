// Stage-level entry points: the layer cut at its two exchange points, for
// expert-parallel execution.  A routing-side layer (router parameters only)
// turns tokens into expert-ordered rows and back; an expert-side layer (top_k
// = 1, expert parameters only) runs the grouped SwiGLU products on rows that
// arrive already tagged with their expert.  Between the two the caller moves
// rows with whatever transport it has (NCCL all-to-all in mgpt_b200/ep.py).
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
    return make_workspace(L->d, n, routing_side ? 1 : 0).total;
}

int mgpt_moe_route(mgpt_moe_layer* L, const void* x, int n_tokens, int io, void* workspace, size_t ws_bytes,
                   void* send_rows, mgpt_stream_t stream)
{
    MGPT_TRY(check_route_layer(L, io));
    if (n_tokens < 0 || (n_tokens > 0 && (!x || !send_rows))) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    const Workspace w = make_workspace(L->d, n_tokens, 1);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    if (n_tokens > 0)
        MGPT_TRY(launch_router_fwd(x, io, L->p_data[0], L->p_data[1], n_tokens, d.C, d.E, d.k, (float*)(ws + w.logits),
                                   (float*)(ws + w.probs), (int32_t*)(ws + w.top_idx), (float*)(ws + w.top_p), st));
    MGPT_TRY(launch_plan(d, w, ws, st));
    // rows in the reference's compact slot order: expert after expert, stable within an expert
    MGPT_TRY(gather_rows(x, io, (const int32_t*)(ws + w.map), nullptr, w.R, w.R, d.C, d.k, send_rows, w.act_bytes, st));
    L->last_n = n_tokens;
    L->last_io = io;
    L->last_ws = workspace;
    L->last_stream = st;
    L->fwd_done = true;
    return 0;
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
    return combine_rows(rows_back, (const int32_t*)(ws + w.slot), (const float*)(ws + w.top_p), w.n_tokens, L->d.C,
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
    return combine_rows_backward(dy, io, rows_back, (const int32_t*)(ws + w.map), (const float*)(ws + w.top_p), nullptr,
                                 w.R, w.R, L->d.C, L->d.k, d_rows, (float*)(ws + w.d_top_p), w.act_bytes,
                                 (cudaStream_t)stream);
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
    return launch_router_bwd(L, w, ws, x, io, dx, (cudaStream_t)stream, d_rows_in, (const int32_t*)(ws + w.slot));
}

int mgpt_moe_experts_forward(mgpt_moe_layer* L, const void* rows, const int32_t* expert_of_row, int n_rows,
                             void* out_rows, void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    MGPT_TRY(check_expert_layer(L));
    if (n_rows < 0 || (n_rows > 0 && (!rows || !expert_of_row || !out_rows))) return fail(MGPT_MOE_EINVAL, "bad row buffer");
    const Workspace w = make_workspace(L->d, n_rows, 0);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->fwd_done = false;
    for (int s = 0; s < ST_COUNT; ++s) L->ev_used[s] = false;
    // rows grouped by expert (stable in arrival order), each expert padded to whole 128-row tiles
    MGPT_TRY(run_plan(n_rows > 0 ? expert_of_row : (const int32_t*)(ws + w.top_idx), n_rows, d.E,
                      (int32_t*)(ws + w.counts), (int32_t*)(ws + w.offsets), (int32_t*)(ws + w.padded_offsets),
                      (int32_t*)(ws + w.tile_expert), (int32_t*)(ws + w.n_tiles), w.max_tiles, (int32_t*)(ws + w.map),
                      (int32_t*)(ws + w.pos), (int32_t*)(ws + w.row_src), w.row_cap, (int32_t*)(ws + w.status),
                      (int32_t*)(ws + w.blk_cnt), st, (int32_t*)(ws + w.slot)));
    if (n_rows > 0) {
        L->stage_begin(ST_DISPATCH, st);
        MGPT_TRY(gather_rows(rows, act_io(w), (const int32_t*)(ws + w.row_src), (const int32_t*)(ws + w.n_tiles), -1,
                             w.row_cap, d.C, 1, ws + w.Xg, w.act_bytes, st));
        L->stage_end(ST_DISPATCH, st);
        if (d.mode == MGPT_MOE_BF16 && d.gemm_impl == 0) MGPT_TRY(tc_experts_forward(L, w, ws, st));
        else MGPT_TRY(simt_experts_forward(L, w, ws, st));
        L->stage_begin(ST_COMBINE, st);
        MGPT_TRY(gather_rows(ws + w.Yg, act_io(w), (const int32_t*)(ws + w.pos), nullptr, n_rows, n_rows, d.C, 1,
                             out_rows, w.act_bytes, st));
        L->stage_end(ST_COMBINE, st);
    }
    L->last_n = n_rows;
    L->last_io = act_io(w);
    L->last_ws = workspace;
    L->last_stream = st;
    L->fwd_done = true;
    return 0;
}

int mgpt_moe_experts_backward(mgpt_moe_layer* L, const void* d_out_rows, void* d_in_rows, void* workspace,
                              size_t ws_bytes, mgpt_stream_t stream)
{
    MGPT_TRY(check_expert_layer(L));
    if (!L->fwd_done || workspace != L->last_ws) return fail(MGPT_MOE_ESTATE, "backward needs the workspace of the last forward");
    const int n_rows = L->last_n;
    const Workspace w = make_workspace(L->d, n_rows, 0);
    MGPT_TRY(check_ws(L, workspace, ws_bytes, w));
    if (n_rows == 0) return 0;
    if (!d_out_rows || !d_in_rows) return fail(MGPT_MOE_EINVAL, "null buffer");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const Dims& d = L->d;
    L->stage_begin(ST_COMBINE_BWD, st);
    MGPT_TRY(gather_rows(d_out_rows, act_io(w), (const int32_t*)(ws + w.row_src), (const int32_t*)(ws + w.n_tiles), -1,
                         w.row_cap, d.C, 1, ws + w.dYg, w.act_bytes, st));
    L->stage_end(ST_COMBINE_BWD, st);
    if (d.mode == MGPT_MOE_BF16 && d.gemm_impl == 0) MGPT_TRY(tc_experts_backward(L, w, ws, st));
    else MGPT_TRY(simt_experts_backward(L, w, ws, st));
    if (L->has_grad) {
        L->stage_begin(ST_BIAS_GRAD, st);
        MGPT_TRY(launch_bias_grads(L, w, ws, st));
        L->stage_end(ST_BIAS_GRAD, st);
    }
    return gather_rows(ws + w.dXg, act_io(w), (const int32_t*)(ws + w.pos), nullptr, n_rows, n_rows, d.C, 1, d_in_rows,
                       w.act_bytes, st);
}

}  // extern "C"
