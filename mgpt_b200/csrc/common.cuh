// Shared declarations of the MoE layer library: layer state, workspace layout,
// error plumbing and the launch prototypes of every stage.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/mgpt_moe.h"

namespace mgpt {

typedef __nv_bfloat16 bf16;

constexpr int ROW_TILE = 128;   // rows of one expert segment are padded to this
constexpr int MAX_EXPERTS = 128;
constexpr int MAX_TOPK = 8;
constexpr int MAX_SOURCES = 64;  // source ranks an expert-side layer can receive row segments from
constexpr int MAX_SEGMENTS = 4096;  // sources x local experts

// Bits of the status words (the per-step word in the workspace and the layer's own, which keeps every bit
// until mgpt_moe_check_status reads it).  A set bit means results of that step are incomplete.
enum StatusBits {
    ST_PLAN_OVERFLOW = 1,     // more row tiles than the workspace holds (cannot happen with a workspace of the stated size)
    ST_FULL_WAIT = 2,         // a bounded wait of a tensor-core kernel ran out: operand tiles never arrived
    ST_EMPTY_WAIT = 4,        //   ... a stage of the operand ring was never released
    ST_ACC_WAIT = 8,          //   ... an accumulator was never completed / released
    ST_SCHED_WAIT = 16,       //   ... the work-item queue stalled
    ST_BAD_EXPERT = 32,       // an expert id outside [0, E) was met by the dispatch plan and skipped
};

enum Stage {
    ST_ROUTER = 0, ST_PLAN, ST_DISPATCH, ST_GATEUP, ST_DOWN, ST_COMBINE,
    ST_COMBINE_BWD, ST_DHH, ST_DXG, ST_WGRAD, ST_BIAS_GRAD, ST_ROUTER_BWD, ST_COUNT
};
static_assert(ST_COUNT == MGPT_MOE_N_STAGES, "stage list and header disagree");

// ---- errors ---------------------------------------------------------------
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);
void count_launch(int n = 1);

#define MGPT_CUDA(call)                                             \
    do {                                                            \
        cudaError_t e__ = (call);                                   \
        if (e__ != cudaSuccess) return ::mgpt::cuda_fail(e__, #call); \
    } while (0)

#define MGPT_LAUNCHED(name)                                          \
    do {                                                             \
        ::mgpt::count_launch();                                      \
        cudaError_t e__ = cudaGetLastError();                        \
        if (e__ != cudaSuccess) return ::mgpt::cuda_fail(e__, name); \
    } while (0)

#define MGPT_TRY(expr)                 \
    do {                               \
        int rc__ = (expr);             \
        if (rc__ != 0) return rc__;    \
    } while (0)

// ---- workspace ------------------------------------------------------------
// One arena per forward/backward pair, carved deterministically from
// (config, n_tokens).  Offsets are bytes, every buffer 256-byte aligned.
struct Workspace {
    // routing (kept for backward)
    size_t logits, probs, top_idx, top_p;
    // plan
    size_t counts, offsets, padded_offsets, tile_expert, n_tiles, status;
    size_t map, pos, row_src, blk_cnt, slot, seg, tile_order;
    size_t pairs, n_pairs;      // row tiles two by two within an expert ({first, second or -1}), in processing order
    // forward activations (kept for backward)
    size_t Xg, G, U, Hh, Yg;
    // backward temporaries
    size_t dYg, dG, dU, dXg, d_top_p, dlogits, rw_part, dl16;
    size_t rt_list, rt_count;   // screened router: tokens to recompute exactly, and how many
    size_t total;
    // derived sizes
    int n_tokens, R, max_tiles, row_cap, plan_blocks, rw_chunks;
    bool inference;     // forward-only layout: nothing is kept for a backward pass
    size_t act_bytes;   // bytes per activation element (2 or 4)
};

struct Dims {
    int C, H, E, k;
    float alpha;
    int mode;       // MGPT_MOE_FP32 / MGPT_MOE_BF16
    int gemm_impl;  // 0 default, 1 SIMT
};

// kind 0: whole layer; kind 1: routing side only (no activation buffers; rows are exchanged by the caller);
// kind 2: expert side (the four [rows, C] buffers belong to the caller); kind 3: whole layer, forward only (inference)
Workspace make_workspace(const Dims& d, int n_tokens, int kind = 0);

// Device-side tables of per-expert pointers (index = expert).
// The transposed BF16 weight copies (the B operands of the forward products) are stored tile-major: per expert the
// [rows, cols] matrix is cut into blocks of 128 rows x 64 columns, 16 KiB each and contiguous, ordered [row block]
// [column block] -- exactly the box one TMA load of a pipeline stage fetches.  A forward-only (decode) batch streams
// every weight byte from DRAM once; from the row-major copy a box was 128 pieces of 128 bytes at the row pitch.
// rows and cols are padded up to whole blocks; the padding is zero (allocation is cleared, writers never touch it).
__host__ __device__ inline size_t tile_major_elems(int rows, int cols)
{
    return (size_t)((rows + 127) / 128 * 128) * (size_t)((cols + 63) / 64 * 64);
}
__host__ __device__ inline size_t tile_major_index(int cols, int r, int c)
{
    const int kb = (cols + 63) / 64;
    return ((size_t)((r >> 7) * kb + (c >> 6)) * 128 + (r & 127)) * 64 + (c & 63);
}

struct ExpertPtrs {
    const void** Wg;  const void** Wu;  const void** Wd;     // [C,H],[C,H],[H,C]
    const float** bg; const float** bu; const float** bd;
    float** gWg; float** gWu; float** gWd; float** gbg; float** gbu; float** gbd;
};

}  // namespace mgpt

struct mgpt_moe_layer {
    mgpt::Dims d;
    int device;
    int n_params;
    std::vector<float*> p_data, p_grad;      // host copies of the bound pointers
    bool bound = false, has_grad = false, shadows_fresh = false;
    bool router_bound = false, experts_bound = false;

    // Error bits of every kernel of this layer since the last mgpt_moe_check_status (device word, zero at create)
    // and the pinned host word they are read into.
    int32_t* d_status = nullptr;
    int32_t* h_status = nullptr;
    bool router_dx_attr = false;             // shared-memory opt-in of router_dx_kernel done on this layer's device
    bool router_tc_attr = false;             // the same for tc_router_fwd_kernel

    // device tables: pointers to FP32 masters / grads per expert
    void* d_tables = nullptr;                // one allocation holding all tables
    void* d_opt = nullptr;                   // optimiser-state tables (m, v per tensor kind; router w, g, m, v)
    bool opt_bound = false;
    mgpt::ExpertPtrs master;                 // W pointers -> FP32 masters
    mgpt::ExpertPtrs shadow;                 // W pointers -> BF16 shadows (BF16 mode)

    // BF16 shadows, contiguous over experts (BF16 mode only)
    mgpt::bf16 *sWg = nullptr, *sWu = nullptr, *sWd = nullptr;      // [E][C][H],[E][C][H],[E][H][C]
    mgpt::bf16 *sWgT = nullptr, *sWuT = nullptr, *sWdT = nullptr;   // transposed copies ([H,C],[H,C],[C,H] per expert), tile-major: see tile_major_index
    mgpt::bf16* sWr = nullptr;                                      // router weight [C][E8], E8 = E rounded up to 8
    mgpt::bf16* sWrT2 = nullptr;     // router weight transposed and split in two BF16 pieces: [2][NE][C], Wr^T ~ hi + mid
    float* d_rstat = nullptr;        // {max_e ||Wr[:,e]||_2, max_e |br[e]|}, slightly inflated (screened router's error bound)
    int router_ne = 0;               // NE: experts rounded up to 16, 32, 64 or 128
    double router_tc_min_work = 4e8; // tokens*C*E from which the tensor-core first pass is used (MGPT_MOE_ROUTER_TC_MIN_WORK)

    // last forward (for backward / counts)
    int last_n = 0, last_io = 0;
    void* last_ws = nullptr;
    cudaStream_t last_stream = 0;
    bool fwd_done = false;
    bool last_inference = false;             // the last forward was mgpt_moe_forward_inference (counts readable, no backward)

    // host staging for mgpt_moe_step_host
    void *h_x = nullptr, *h_dy = nullptr, *h_y = nullptr, *h_dx = nullptr, *h_ws = nullptr;
    size_t h_io_bytes = 0, h_ws_bytes = 0;
    cudaStream_t copy_stream = nullptr;      // second stream of mgpt_moe_step_host (copies that overlap compute)
    cudaEvent_t copy_ev[5] = {};
    cudaEvent_t dx_ready_event = nullptr;    // when set, backward records it as soon as dx is complete
    void* host_pipe = nullptr;               // mgpt_moe_step_host_async: two slots of device staging, copy streams, events

    // TMA descriptors (opaque, built per workspace pointer)
    void* tc_state = nullptr;
    int sm_budget = 0;                       // > 0: persistent kernels launch at most this many CTAs
    bool bwd_overwrite = false;              // this backward writes the expert weight gradients instead of adding to them

    // expert side of an expert-parallel layer: row buffers owned by the caller (the exchange buffers) and the
    // number of row segments per expert (one per source rank); 0 = one contiguous padded range per expert
    void *ext_Xg = nullptr, *ext_Yg = nullptr, *ext_dYg = nullptr, *ext_dXg = nullptr;
    int n_seg = 0;

    // optional per-stage timing
    bool profiling = false;
    cudaEvent_t ev_begin[mgpt::ST_COUNT] = {}, ev_end[mgpt::ST_COUNT] = {};
    bool ev_used[mgpt::ST_COUNT] = {};
    void stage_begin(int s, cudaStream_t st) const
    {
        if (profiling) cudaEventRecord(ev_begin[s], st);
    }
    void stage_end(int s, cudaStream_t st)
    {
        if (profiling) {
            cudaEventRecord(ev_end[s], st);
            ev_used[s] = true;
        }
    }
};

namespace mgpt {

// the four [rows, C] buffers: in the workspace, or caller-owned on the expert side of an expert-parallel layer
inline char* buf_Xg(const mgpt_moe_layer* L, const Workspace& w, char* ws) { return L->ext_Xg ? (char*)L->ext_Xg : ws + w.Xg; }
inline char* buf_Yg(const mgpt_moe_layer* L, const Workspace& w, char* ws) { return L->ext_Yg ? (char*)L->ext_Yg : ws + w.Yg; }
inline char* buf_dYg(const mgpt_moe_layer* L, const Workspace& w, char* ws) { return L->ext_dYg ? (char*)L->ext_dYg : ws + w.dYg; }
inline char* buf_dXg(const mgpt_moe_layer* L, const Workspace& w, char* ws) { return L->ext_dXg ? (char*)L->ext_dXg : ws + w.dXg; }

// ---- stage launchers (each enqueues on `st`, returns 0 or an error code) ---

// router.cu
int launch_router_fwd(const void* x, int io, const float* Wr, const float* br, int N, int C, int E, int k,
                      float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st,
                      const int32_t* list = nullptr, const int32_t* list_count = nullptr);
// router_tc.cu: the router for BF16 tokens -- tensor-core first pass plus exact recompute of the tokens whose
// routing the first pass cannot prove
bool tc_router_usable(const mgpt_moe_layer* L, const void* x, int io, int n_tokens);
int tc_router_fwd(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, cudaStream_t st);
int launch_router_pieces(mgpt_moe_layer* L, cudaStream_t st);
int router_tc_ne(int E);
int launch_router_bwd(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, int io,
                      void* dx, cudaStream_t st, const void* dXg_rows = nullptr, const int32_t* pos_rows = nullptr);

// plan.cu
int launch_plan(const Dims& d, const Workspace& w, char* ws, cudaStream_t st, int32_t* sticky);
int launch_dispatch(const Dims& d, const Workspace& w, char* ws, const void* x, int io, cudaStream_t st);
int launch_combine_fwd(const Dims& d, const Workspace& w, char* ws, void* y, int io, cudaStream_t st,
                       const void* residual = nullptr);
int launch_combine_bwd(const Dims& d, const Workspace& w, char* ws, const void* dy, int io, cudaStream_t st);
int launch_bias_grads(const mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st);
int launch_segment_tiles(const Dims& d, const Workspace& w, char* ws, const int32_t* seg_counts, int n_src, cudaStream_t st,
                         int32_t* sticky);
int gather_rows(const void* src, int src_io, const int32_t* row_src, const int32_t* n_tiles, int rows, int grid_rows,
                int C, int k, void* dst, size_t act_bytes, cudaStream_t st);
int combine_rows(const void* rows, const int32_t* pos, const float* top_p, int N, int C, int k, void* y, int io,
                 size_t act_bytes, cudaStream_t st, const void* residual = nullptr);
int combine_rows_backward(const void* dy, int io, const void* rows, const int32_t* row_src, const float* top_p,
                          const int32_t* n_tiles, int n_rows, int grid_rows, int C, int k, void* d_rows, float* d_top_p,
                          size_t act_bytes, cudaStream_t st);
int run_plan(const int32_t* top_idx, int R, int E, int32_t* counts, int32_t* offsets, int32_t* padded_offsets,
             int32_t* tile_expert, int32_t* n_tiles, int max_tiles, int32_t* map, int32_t* pos,
             int32_t* row_src, int row_cap, int32_t* status, int32_t* blk, cudaStream_t st, int32_t* slot_of,
             int32_t* sticky, int32_t* pairs, int32_t* n_pairs);

// gemm_simt.cu
int simt_experts_forward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st);
int simt_experts_backward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st);

// gemm_tc.cu (tcgen05 / TMEM / TMA)
int tc_experts_forward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st);
int tc_experts_backward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st, int phase = 3);
int tc_init(mgpt_moe_layer* L);
bool tc_fused_bias_grads(const Dims& d);
int tc_selftest_bounded_wait(mgpt_moe_layer* L, cudaStream_t st);
void tc_destroy(mgpt_moe_layer* L);
void host_pipe_destroy(mgpt_moe_layer* L);          // frees the staging of mgpt_moe_step_host_async (waits for steps in flight)
int launch_sync_router_only(mgpt_moe_layer* L, cudaStream_t st);
int launch_adamw(mgpt_moe_layer* L, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                 cudaStream_t st, float grad_clip = 0.0f, int skip_nonfinite = 0);
int tc_router_dx(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* dXg, const int32_t* pos, void* dx,
                 cudaStream_t st);
int tc_router_wgrad(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, cudaStream_t st);

// weights.cu
int launch_sync_weights(mgpt_moe_layer* L, cudaStream_t st);

}  // namespace mgpt
