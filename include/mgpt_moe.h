/*
 * mgpt_moe.h -- C ABI of the B200 (sm_100a) Mixture-of-Experts layer.
 *
 * The library replaces the body of the reference's MoELayer
 * (src/main/neuralnetwork/layers/MoELayer.{h,cpp}) and, below it, the
 * cuda_ops MoE kernels (src/main/utils/cuda_ops.h:52-62, 29, 36-37, 95-96).
 * The reference engine keeps owning parameters (FP32 Tensor data/grad),
 * the Scratchpad arena and the optimiser; this ABI only sees raw device
 * pointers, sizes and a stream.
 *
 * Conventions
 *   - every function returns 0 on success, a MGPT_MOE_E* code otherwise;
 *     mgpt_moe_last_error() returns the message of the calling thread's
 *     last failure;
 *   - all work is enqueued on the stream passed in (0 = the legacy default
 *     stream the reference uses everywhere) and nothing synchronises unless
 *     the comment says so;
 *   - token tensors are row-major [n_tokens, embed_dim] (the reference's
 *     [B,T,C] flattened, MoELayer.cpp:30);
 *   - parameter order is the reference's get_parameters() order
 *     (MoELayer.cpp:225-236): Wr[C,E], br[E], then per expert
 *     Wg[C,H], bg[H], Wu[C,H], bu[H], Wd[H,C], bd[C]  (2+6E tensors).
 *   - there is no CPU fallback: without a CUDA device every compute entry
 *     point fails with MGPT_MOE_ECUDA.
 */
#ifndef MGPT_MOE_H
#define MGPT_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MGPT_MOE_OK       0
#define MGPT_MOE_EINVAL   1   /* bad argument / unsupported shape            */
#define MGPT_MOE_ECUDA    2   /* a CUDA runtime or driver call failed         */
#define MGPT_MOE_ESTATE   3   /* call order (e.g. backward before forward)    */
#define MGPT_MOE_ENOMEM   4   /* workspace too small                          */

/* arithmetic modes */
#define MGPT_MOE_FP32     0   /* FP32 SIMT validation mode (reference dtype)  */
#define MGPT_MOE_BF16     1   /* BF16 operands, FP32 accumulate, tcgen05/TMEM */

/* element type of x / y / dy / dx at the boundary */
#define MGPT_MOE_IO_F32   0
#define MGPT_MOE_IO_BF16  1

typedef struct mgpt_moe_layer mgpt_moe_layer;   /* opaque */
typedef void* mgpt_stream_t;                    /* cudaStream_t */

/* Mirrors MoELayer(int embed_dim, int hidden_dim, int num_experts, int top_k)
 * (MoELayer.h:37); hidden_dim -1 means 4*embed_dim (SwiGLU.cpp:4-8).
 * lb_alpha is the literal 0.01f at MoELayer.cpp:194. */
typedef struct {
    int   embed_dim;
    int   hidden_dim;
    int   num_experts;
    int   top_k;
    float lb_alpha;
    int   mode;        /* MGPT_MOE_FP32 | MGPT_MOE_BF16                       */
    int   device;      /* CUDA device ordinal                                 */
    int   gemm_impl;   /* 0 = default for the mode, 1 = force SIMT products   */
} mgpt_moe_config;

/* Replaces the MoELayer constructor (MoELayer.cpp:4-12). Allocates only the
 * layer's own BF16 weight shadows and small tables; parameters stay with the
 * caller. */
int  mgpt_moe_create(const mgpt_moe_config* cfg, mgpt_moe_layer** out);
void mgpt_moe_destroy(mgpt_moe_layer* layer);
const char* mgpt_moe_last_error(void);

/* get_parameters() (MoELayer.cpp:225-236): number of tensors and their shapes. */
int  mgpt_moe_num_params(const mgpt_moe_layer* layer);
int  mgpt_moe_param_shape(const mgpt_moe_layer* layer, int index, int* rows, int* cols);

/* Hands the layer the engine-owned FP32 device buffers: data[i] is
 * Tensor::cuda_data and grad[i] Tensor::cuda_grad of get_parameters()[i]
 * (Tensor.h:22-23). grad may be NULL for inference. Gradients are
 * accumulated (+=) like Tensor::add_grad (Tensor.cpp:638-650). */
int  mgpt_moe_bind_params(mgpt_moe_layer* layer, float* const* data, float* const* grad, int n);

/* Rebuilds the BF16 shadows from the FP32 masters. Call after binding and
 * after every optimiser step or checkpoint load (no-op in FP32 mode). */
int  mgpt_moe_sync_weights(mgpt_moe_layer* layer, mgpt_stream_t stream);

/* get_footprint() (MoELayer.cpp:238-251): bytes of arena the layer needs for
 * n_tokens (forward activations kept for backward + backward temporaries). */
size_t mgpt_moe_workspace_bytes(const mgpt_moe_layer* layer, int n_tokens);

/* forward_into() (MoELayer.cpp:28-128). x, y: device [n_tokens, C] of io_dtype.
 * workspace: device memory of at least mgpt_moe_workspace_bytes(n_tokens),
 * 256-byte aligned (Scratchpad::get_address alignment, Scratchpad.cpp:27-29);
 * it must stay untouched until the matching backward has run. */
int  mgpt_moe_forward(mgpt_moe_layer* layer, const void* x, void* y, int n_tokens, int io_dtype,
                      void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* backward_into() (MoELayer.cpp:135-223). dy, dx: device [n_tokens, C]; x is
 * the forward input (the reference keeps it as LinearLayer::cached_input,
 * LinearLayer.cpp:24). Accumulates all 2+6E parameter gradients. */
int  mgpt_moe_backward(mgpt_moe_layer* layer, const void* x, const void* dy, void* dx, int io_dtype,
                       void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* get_expert_counts() (MoELayer.h:39): per-expert routed rows of the last
 * forward, as integers. Synchronises the stream of that forward. */
int  mgpt_moe_expert_counts(mgpt_moe_layer* layer, int32_t* host_counts);

/* Offset and size of a named buffer inside the workspace for n_tokens, for
 * tests and for callers that read routing results in place. Names:
 * logits probs top_idx top_p counts offsets padded_offsets map pos row_src
 * tile_expert n_tiles Xg G U Hh Yg dYg dG dU dXg d_top_p dlogits status
 * router_recompute (one int32: tokens the BF16-token router recomputed exactly).
 * Activation buffers are row-major [padded rows, width], except G and U on
 * the tensor-core path (mode BF16, gemm_impl 0), which only its own epilogues
 * read: there the buffer named G holds U*sigmoid(G)*(1 + G*(1 - sigmoid(G))) and
 * the buffer named U holds silu(G) -- the two factors backward multiplies dHh by
 * (utils/Tensor.cpp:2020-2027) -- laid out [row tile][8-column chunk][128 rows][8 values]. */
int  mgpt_moe_workspace_view(const mgpt_moe_layer* layer, int n_tokens, const char* name,
                             size_t* offset, size_t* bytes);

/* Whole step with HOST buffers: copies x (and dy) to the device, runs forward
 * (and backward when dy != NULL), copies y (and dx) back and synchronises.
 * Stands where the reference's caller does Tensor::to(Device::CUDA) /
 * copy_to_host around the layer (Tensor.h:37-44). The layer keeps its own
 * device staging buffers, grown on demand. */
int  mgpt_moe_step_host(mgpt_moe_layer* layer, const void* x_host, const void* dy_host,
                        void* y_host, void* dx_host, int n_tokens, int io_dtype, mgpt_stream_t stream);

/* The same step, pipelined: the call enqueues the uploads, the kernels and
 * the downloads and returns without waiting, so that the next step's x and
 * dy go up, and the previous step's y and dx come down, beside this step's
 * kernels (one upload stream, one download stream, compute on `stream` in
 * call order; two slots of device staging inside the layer). At most two
 * steps are in flight: a third call first waits until the results of the
 * step before last are in host memory. A step's y_host / dx_host are valid
 * after the call after next has returned, or after mgpt_moe_step_host_wait,
 * which waits for every step in flight and returns the layer's status
 * (MGPT_MOE_ESTATE style errors of the kernels, as mgpt_moe_check_status).
 * The host buffers must stay valid (and pinned, for the copies to overlap)
 * until then. No reference counterpart: the reference's CPU layer works on
 * host memory in place (layers/MoELayer.cpp:58-135). */
int  mgpt_moe_step_host_async(mgpt_moe_layer* layer, const void* x_host, const void* dy_host,
                              void* y_host, void* dx_host, int n_tokens, int io_dtype, mgpt_stream_t stream);
int  mgpt_moe_step_host_wait(mgpt_moe_layer* layer);

/* Per-stage device timing for benchmarks. When enabled, forward and backward
 * bracket each stage with CUDA events on the caller's stream;
 * mgpt_moe_stage_ms synchronises those events and writes the milliseconds of
 * the LAST forward/backward pair, one float per stage (0 for stages that did
 * not run). Stage i is named by mgpt_moe_stage_name(i). No reference
 * counterpart (the reference times whole steps with std::chrono,
 * pipeline/Trainer.cpp:314-323). */
#define MGPT_MOE_N_STAGES 12
int  mgpt_moe_set_profiling(mgpt_moe_layer* layer, int enabled);
int  mgpt_moe_stage_ms(mgpt_moe_layer* layer, float* ms);
const char* mgpt_moe_stage_name(int stage);

/* Forward with the block's skip connection folded into the combine write:
 * y = residual + moe(x), where the reference's caller adds the two in a separate pass
 * (TransformerBlock.cpp:42-46: x2 = x1 + moe(ln2(x1)); residual = x1, same dtype and
 * shape as y). The sum over a token's experts is formed first and the residual added
 * last, which is the reference's order, so FP32 results are bit-identical to
 * forward followed by the add. Backward is unchanged: the residual's gradient is dy itself. */
int  mgpt_moe_forward_residual(mgpt_moe_layer* layer, const void* x, const void* residual, void* y, int n_tokens,
                               int io_dtype, void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* Forward for generation.  The reference's generator runs the whole model forward over the current context for every
 * new token and throws the activations away (pipeline/Generator.cpp:10-31: model.forward, reset_activations), so the
 * layer sees forward-only calls of a few to a few hundred tokens.  This entry point is mgpt_moe_forward without
 * anything kept for a backward pass: a workspace of mgpt_moe_inference_workspace_bytes(n_tokens) (no saved
 * activation factors, no backward buffers), the same routing and the same y.  Token batches too small to fill the
 * device take the low-latency form of the exact router.  mgpt_moe_backward cannot follow it (MGPT_MOE_ESTATE);
 * mgpt_moe_expert_counts can. */
size_t mgpt_moe_inference_workspace_bytes(const mgpt_moe_layer* layer, int n_tokens);
int  mgpt_moe_forward_inference(mgpt_moe_layer* layer, const void* x, void* y, int n_tokens, int io_dtype,
                                void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* The block's glue around the layer, fused (layers/TransformerBlock.cpp:42-46 forward, 80-84 backward):
 *   block_forward   x2 = x1 + moe(rmsnorm(x1) * rms_scale)   in place of  ln2.forward_into, mlp.forward_into, add_into
 *   block_backward  d_x1 = dout + rmsnorm_backward(d_moe_in), d_rms_scale += ...
 *                                                            in place of  mlp.backward_into, ln2.backward_into, add_into
 * RMSNorm as the reference's (utils/Tensor.cpp:785-800, 1674-1690; r = 1/sqrt(mean(x^2) + eps), rms_scale the
 * layer's gamma [C], FP32).  The norm writes the layer's input once (the reference also writes x_hat) and one float
 * per token; the skip connection rides on the combine write; backward recomputes x_hat from x1 and forms d_x1 in
 * the pass that adds dout.  x1 must still hold its forward values at block_backward.  workspace:
 * mgpt_moe_block_workspace_bytes(n_tokens, io_dtype) bytes, 256-byte aligned, untouched between the two calls; it
 * contains the layer's own workspace, which starts at workspace + block_workspace_bytes - mgpt_moe_workspace_bytes.
 * d_rms_scale may be NULL.  The layer's parameter gradients accumulate as in mgpt_moe_backward. */
size_t mgpt_moe_block_workspace_bytes(const mgpt_moe_layer* layer, int n_tokens, int io_dtype);
int  mgpt_moe_block_forward(mgpt_moe_layer* layer, const void* x1, const float* rms_scale, float eps, void* x2,
                            int n_tokens, int io_dtype, void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
int  mgpt_moe_block_backward(mgpt_moe_layer* layer, const void* x1, const float* rms_scale, float* d_rms_scale,
                             const void* dout, void* d_x1, int io_dtype, void* workspace, size_t workspace_bytes,
                             mgpt_stream_t stream);

/* Recompute forward for activation checkpointing. The reference runs every block's
 * forward twice per step (GPT.cpp:79-96: once without keeping activations, once more
 * before that block's backward, the arena rewound in between). The same tokens route
 * the same way, so the second run can skip router and plan: after the first forward
 * save_routing copies the routing results and the plan (routing_bytes(n_tokens) bytes:
 * probabilities, top-k, counts, offsets, tile list, row permutation) into memory the
 * caller keeps outside the arena; forward_with_routing takes them back instead of
 * recomputing them and then runs dispatch, the expert products and combine as
 * mgpt_moe_forward does. Backward follows it as usual. The caller guarantees that x,
 * the weights and n_tokens are those of the forward that was saved. */
size_t mgpt_moe_routing_bytes(const mgpt_moe_layer* layer, int n_tokens);
int  mgpt_moe_save_routing(mgpt_moe_layer* layer, void* dst, mgpt_stream_t stream);
int  mgpt_moe_forward_with_routing(mgpt_moe_layer* layer, const void* x, void* y, int n_tokens, int io_dtype,
                                   void* workspace, size_t workspace_bytes, const void* routing,
                                   mgpt_stream_t stream);

/* Optimiser step for the layer's own parameters, fused with the refresh of the
 * BF16 weight copies. Replaces, for these tensors, the per-tensor
 * Tensor::adamw_step calls of AdamWOptimizer::step
 * (optimisers/AdamWOptimiser.h:24-36, utils/Tensor.cpp:683-699,
 * utils/cuda_ops.cu:723-738) and the mgpt_moe_sync_weights call that would
 * have to follow them. bind_optimizer_state takes the first and second moment
 * buffers (FP32 device memory owned by the caller, zero at step 1, same order
 * and NULL rules as bind_params); rebinding parameters unbinds them.
 * adamw_step (t = 1-based step count) updates w, m, v in place with the CPU
 * arm's arithmetic, bit for bit, and leaves the layer ready for forward. */
int  mgpt_moe_bind_optimizer_state(mgpt_moe_layer* layer, float* const* m, float* const* v, int n);
int  mgpt_moe_adamw_step(mgpt_moe_layer* layer, float lr, float beta1, float beta2, float eps, float weight_decay,
                         int t, mgpt_stream_t stream);

/* The same step with the two guards the reference's GPU kernel applies to the gradient before the update
 * (utils/cuda_ops.cu:727-728): skip_nonfinite != 0 leaves an element whose gradient is NaN or Inf untouched
 * (w, m, v keep their values), grad_clip > 0 clamps the gradient to [-grad_clip, grad_clip] (the reference
 * uses 10).  With grad_clip = 0 and skip_nonfinite = 0 this is mgpt_moe_adamw_step.  The arithmetic after the
 * guards is the CPU arm's, as above. */
int  mgpt_moe_adamw_step_guarded(mgpt_moe_layer* layer, float lr, float beta1, float beta2, float eps,
                                 float weight_decay, int t, float grad_clip, int skip_nonfinite,
                                 mgpt_stream_t stream);

/* Error word of the layer's kernels.  Every wait inside the tensor-core kernels is bounded; a wait that runs
 * out, or an expert id outside [0, num_experts) met by the dispatch plan, sets a bit in a device word owned
 * by the layer instead of hanging or faulting (the reference's kernels abort the process on a CUDA error,
 * utils/cuda_ops.cu:10-18; there is nothing to return there).  check_status copies that word to the host on
 * the stream of the layer's last call, synchronises that stream, and returns MGPT_MOE_OK when it is zero, else
 * MGPT_MOE_ECUDA with the decoded bits in mgpt_moe_last_error() (the word is then cleared).  bits may be
 * NULL.  mgpt_moe_step_host, mgpt_moe_expert_counts and mgpt_moe_stage_ms, which synchronise anyway, make the
 * same check.  Bits: 1 plan overflow, 2/4/8/16 a bounded wait ran out (operands, stage release, accumulator,
 * work queue), 32 expert id out of range. */
int  mgpt_moe_check_status(mgpt_moe_layer* layer, int32_t* bits);

/* Self-test of the error path, for failure-detection tests: launches one tiny kernel that waits, with the
 * tensor-core kernels' own bounded wait and a limit of 4096 polls, on a barrier nothing arrives on.  The wait
 * runs out within microseconds, bit 2 is set in the layer's error word and the kernel returns; no fault, no
 * hang, the context stays usable.  The next mgpt_moe_check_status reports MGPT_MOE_ECUDA once.  No reference
 * counterpart. */
int  mgpt_moe_selftest_bounded_wait(mgpt_moe_layer* layer, mgpt_stream_t stream);

/* Expert weight gradients written instead of accumulated.  The reference adds into gradient tensors its trainer
 * zeroed at the start of the step (Tensor::add_grad, utils/Tensor.cpp:638-650; pipeline/Trainer.cpp:303-305): a
 * zero fill plus a read-modify-write of 12 bytes per expert weight.  With this switch on (tensor-core path only),
 * backward STORES gWg, gWu and gWd of every expert (zeros for an expert without rows), which equals accumulating
 * into zeroed tensors bit for bit and makes the caller's zero fill of those tensors unnecessary.  Only valid for
 * the first backward after the caller's zero_grad: with gradient accumulation over micro-batches
 * (pipeline/Trainer.cpp:311-325) later backwards must run with the switch off.  Bias and router gradients always
 * accumulate.  Default off. */
int  mgpt_moe_set_weight_grad_overwrite(mgpt_moe_layer* layer, int enabled);

/* Upper bound on the CTAs of the persistent tensor-core kernels of this layer
 * (one CTA per SM; 0 = every SM, the default). A caller that overlaps these
 * kernels with communication kernels on another stream leaves SMs free for
 * them this way; results do not depend on the value. No reference counterpart. */
int  mgpt_moe_set_sm_budget(mgpt_moe_layer* layer, int n_sms);

/* Number of kernels the library launched since the counter was last reset
 * (host-side count of its own launches; for benchmark bookkeeping). */
long mgpt_moe_launch_count(int reset);

/* ---- operator level: the cuda_ops seam (cuda_ops.h:52-62), typed ---------
 * Device pointers; indices are int32 (the reference stores them as floats). */

/* linear + softmax(clamp 1e-7..1) + top_k in one pass
 * (LinearLayer.cpp:23-28, Tensor.cpp:850-883, cuda_ops.h:53). logits may be NULL. */
int  mgpt_moe_op_router(const void* x, int io_dtype, const float* Wr, const float* br,
                        int n_tokens, int C, int E, int k,
                        float* logits, float* probs, int32_t* top_idx, float* top_p,
                        mgpt_stream_t stream);

/* histogram + prefix sum + stable slot assignment in one call, on the device
 * (cuda_ops.h:56-57 moe_histogram / moe_gather's slot claim, MoELayer.cpp:61-80's
 * host prefix sum). top_idx: [n_rows] expert id per flat index tok*k+j.
 * Outputs: counts[E], offsets[E] (compact), padded_offsets[E+1] (every expert's
 * segment rounded up to 128 rows), tile_expert[row_cap/128], n_tiles[1],
 * map[n_rows] (compact slot -> flat index, the reference's sorted_token_ids),
 * pos[n_rows] (flat index -> padded row), row_src[row_cap] (padded row -> flat
 * index, -1 for padding; written for the n_tiles*128 rows in use), status[1] (0 = ok;
 * 32 = some top_idx value was outside [0, E): those entries get no slot and are left
 * out of counts, map and pos stay unwritten for them).
 * row_cap: a multiple of 128, at least (n_rows + E*127) rounded down to 128.
 * scratch: device memory of mgpt_moe_op_plan_scratch_bytes(n_rows, E) bytes. */
size_t mgpt_moe_op_plan_scratch_bytes(int n_rows, int E);
int  mgpt_moe_op_plan(const int32_t* top_idx, int n_rows, int E,
                      int32_t* counts, int32_t* offsets, int32_t* padded_offsets,
                      int32_t* tile_expert, int32_t* n_tiles, int32_t* map, int32_t* pos,
                      int32_t* row_src, int row_cap, int32_t* status,
                      void* scratch, size_t scratch_bytes, mgpt_stream_t stream);

/* ---- stage level: the layer cut at its two exchange points ------------------
 * For expert-parallel execution (the reference has no multi-GPU code; these
 * calls split MoELayer::forward_into / backward_into, MoELayer.cpp:52-83 |
 * 94-118 | 121-123 and 156 | 159-181 | 184-218, where rows change owner).
 *
 * Routing side: a layer created with all E experts and top_k = k, bound with
 * mgpt_moe_bind_params(layer, data, grad, 2) (router tensors only).
 * Expert side: a layer created with the E_local experts this GPU owns and
 * top_k = 1, bound with all 2+6*E_local pointers of which data[0], data[1]
 * (router) may be NULL.  Rows are [n, C] in the mode's activation type (BF16
 * in BF16 mode, FP32 in FP32 mode) and travel TILE-ALIGNED: expert-major, each
 * expert's segment padded with zero rows to a multiple of 128 rows, so the
 * rows of experts e0..e1 are the contiguous range
 * [padded_offsets[e0], padded_offsets[e1+1]) (workspace view "padded_offsets";
 * real counts: view "counts").  Workspaces: mgpt_moe_stage_workspace_bytes.  */
size_t mgpt_moe_stage_workspace_bytes(const mgpt_moe_layer* layer, int n, int routing_side);

/* router + plan + permutation into send_rows[row_cap, C] (row_cap = rows of the
 * workspace view "row_src"): the layout above, stable within an expert like the
 * reference's slot order (Tensor.cpp:1368-1381). */
int  mgpt_moe_route(mgpt_moe_layer* layer, const void* x, int n_tokens, int io_dtype,
                    void* workspace, size_t workspace_bytes, void* send_rows, mgpt_stream_t stream);
/* mgpt_moe_route in two calls: _plan (router + plan; the counts are then final and their exchange can start) and
 * _rows (the permutation into send_rows, which can run while the counts travel). */
int  mgpt_moe_route_plan(mgpt_moe_layer* layer, const void* x, int n_tokens, int io_dtype,
                         void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
int  mgpt_moe_route_rows(mgpt_moe_layer* layer, const void* x, int io_dtype, void* workspace, size_t workspace_bytes,
                         void* send_rows, mgpt_stream_t stream);
/* y[tok,:] = sum_j p[tok,j] * rows_back[row(tok,j),:]   (Tensor.cpp:1398-1406); rows_back in the send layout */
int  mgpt_moe_combine(mgpt_moe_layer* layer, const void* rows_back, void* y, int io_dtype,
                      void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
/* d_rows[row,:] = p * dy[tok,:] (zero in padding rows) and d_top_p (Tensor.cpp:1424-1436) */
int  mgpt_moe_combine_backward(mgpt_moe_layer* layer, const void* rows_back, const void* dy, int io_dtype,
                               void* d_rows, void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
/* dx = gather-sum of d_rows_in + router backward; accumulates the router gradients
 * with this GPU's own counts in the load-balance term (MoELayer.cpp:184-218). */
int  mgpt_moe_route_backward(mgpt_moe_layer* layer, const void* x, const void* d_rows_in, void* dx, int io_dtype,
                             void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
/* The SwiGLU experts on received rows (MoELayer.cpp:94-118). rows[n_rows, C] is n_src
 * blocks (one per source rank, in rank order), each holding one padded segment per
 * local expert; seg_counts[n_src * E_local] (device, source-major) are the REAL row
 * counts. n_rows = sum of the padded segment lengths. The kernels read rows and write
 * out_rows (same layout) in place: no copy, no regrouping. Keeps what backward needs
 * in the workspace; rows must stay valid until backward. */
int  mgpt_moe_experts_forward(mgpt_moe_layer* layer, const void* rows, const int32_t* seg_counts, int n_src,
                              int n_rows, void* out_rows, void* workspace, size_t workspace_bytes,
                              mgpt_stream_t stream);
/* d_in_rows = gradient w.r.t. rows (same layout; d_out_rows must be zero in padding rows, as
 * mgpt_moe_combine_backward writes it); accumulates the expert parameter gradients (MoELayer.cpp:159-181). */
int  mgpt_moe_experts_backward(mgpt_moe_layer* layer, const void* d_out_rows, void* d_in_rows,
                               void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* mgpt_moe_experts_backward in two calls, for callers that overlap the exchange with compute: _rows computes
 * d_in_rows (everything the other GPUs are waiting for), _params then accumulates the expert parameter gradients
 * from the same buffers; the caller starts sending d_in_rows back between the two.  Same arguments; calling
 * _rows then _params equals one mgpt_moe_experts_backward.  (On the CUDA-core paths _rows does all the work.) */
int  mgpt_moe_experts_backward_rows(mgpt_moe_layer* layer, const void* d_out_rows, void* d_in_rows,
                                    void* workspace, size_t workspace_bytes, mgpt_stream_t stream);
int  mgpt_moe_experts_backward_params(mgpt_moe_layer* layer, const void* d_out_rows, void* d_in_rows,
                                      void* workspace, size_t workspace_bytes, mgpt_stream_t stream);

/* ---- expert parallelism behind the C ABI ------------------------------------------------------------------------
 * One process per GPU, one mgpt_moe_ep per process: every rank keeps a replica of the router and E/world experts
 * (with n_chunks > 1 expert e belongs to chunk e / (E/n_chunks) and, inside it, to rank
 * (e % (E/n_chunks)) / (E/(world*n_chunks)); n_chunks = 1: rank g owns experts [g*E/world, (g+1)*E/world)), tokens
 * stay on their GPU.  Forward: route -> exchange of the per-expert counts -> rows to the experts' owners -> experts ->
 * rows back -> combine; backward the mirror image, the gradients of the received rows travelling back while the
 * parameter gradients are formed.  The exchange is NCCL point-to-point (ncclSend / ncclRecv in groups) on a stream of
 * its own; a chunk's exchange overlaps the previous chunk's expert work.  The library loads libnccl.so.2 at the first
 * call (it does not link it), so single-GPU users need no NCCL.  The reference has no multi-GPU code: these calls
 * shard the expert loop of MoELayer::forward_into / backward_into (layers/MoELayer.cpp:94-118, 159-181).
 *
 * Set-up: rank 0 calls mgpt_moe_ep_unique_id and hands the 128 bytes to every rank by whatever means the engine
 * has; then every rank calls mgpt_moe_ep_create (a collective: it returns once all ranks have called it).
 * Parameters: 2 + 6*E/world tensors -- Wr, br, then this rank's experts in local order (chunk by chunk;
 * mgpt_moe_ep_global_expert gives the global index of local expert i) -- FP32 device buffers owned by the caller, like
 * mgpt_moe_bind_params.  x, y, dy, dx: device [n_tokens, C].  The layer owns its workspaces and exchange buffers and
 * grows them on demand (allocation only when n_tokens or the row counts exceed what was seen before).  The
 * load-balance term uses this rank's own counts; router gradients are this rank's (all-reduce them if the replicas
 * are to stay identical).  Each forward synchronises the host once (the row counts per peer). */
typedef struct mgpt_moe_ep mgpt_moe_ep;
typedef struct {
    int   embed_dim, hidden_dim, num_experts, top_k;
    float lb_alpha;
    int   mode;        /* MGPT_MOE_FP32 | MGPT_MOE_BF16 */
    int   device;
    int   rank, world;
    int   n_chunks;    /* experts per rank are split into this many chunks (1 = no overlap) */
    int   max_tokens;  /* > 0 (all ranks in one node with peer access, world > 1): the rows do not travel through
                          NCCL; every rank keeps its row buffers, sized for this many tokens per call, readable by
                          the others (CUDA IPC), and the rank that needs a block pulls it with a copy engine, which
                          takes no SM from the tensor-core kernels.  NCCL then carries the counts (an all-gather)
                          and the barriers.  Calls with more tokens fail with MGPT_MOE_EINVAL.  0: NCCL
                          point-to-point for the rows, buffers grown on demand */
} mgpt_moe_ep_config;
#define MGPT_MOE_EP_ID_BYTES 128
int  mgpt_moe_ep_unique_id(void* id_out);
int  mgpt_moe_ep_create(const mgpt_moe_ep_config* cfg, const void* id, mgpt_moe_ep** out);
void mgpt_moe_ep_destroy(mgpt_moe_ep* ep);
int  mgpt_moe_ep_num_params(const mgpt_moe_ep* ep);
int  mgpt_moe_ep_global_expert(const mgpt_moe_ep* ep, int local_index);
int  mgpt_moe_ep_bind_params(mgpt_moe_ep* ep, float* const* data, float* const* grad, int n);
int  mgpt_moe_ep_sync_weights(mgpt_moe_ep* ep, mgpt_stream_t stream);
int  mgpt_moe_ep_forward(mgpt_moe_ep* ep, const void* x, void* y, int n_tokens, int io_dtype, mgpt_stream_t stream);
int  mgpt_moe_ep_backward(mgpt_moe_ep* ep, const void* x, const void* dy, void* dx, int io_dtype, mgpt_stream_t stream);
/* Real rows this rank received per (source rank, local expert) in the last forward: int32 [world * E/world], host. */
int  mgpt_moe_ep_received_counts(mgpt_moe_ep* ep, int32_t* host_counts);
int  mgpt_moe_ep_check_status(mgpt_moe_ep* ep);

/* Row buffers that the other GPUs of the node read directly, for expert-
 * parallel callers that compose the stage calls themselves (mgpt_b200/ep.py).
 * A collective's copy kernels need SMs, and this library's persistent kernels
 * hold all of them; a copy engine needs none. So each rank allocates the
 * buffers it produces rows into with mgpt_moe_peer_alloc, hands the 64-byte
 * handle to the other processes of the node by its own transport, and the
 * rank that needs a block pulls it with mgpt_moe_peer_copy from the pointer
 * mgpt_moe_peer_open gave it (cudaMemcpyAsync over NVLink, beside the
 * kernels). Ordering between producer and reader is the caller's (a barrier of
 * its process group between "rows written" and "rows pulled"). A handle can
 * be opened once per process; close every mapping before the owner frees the
 * buffer. No reference counterpart (the reference has one device). */
#define MGPT_MOE_PEER_HANDLE_BYTES 64
int  mgpt_moe_peer_alloc(int device, size_t bytes, void** ptr, void* handle /* [MGPT_MOE_PEER_HANDLE_BYTES] out */);
int  mgpt_moe_peer_open(int device, const void* handle, void** ptr);
int  mgpt_moe_peer_close(int device, void* ptr);
int  mgpt_moe_peer_free(int device, void* ptr);
int  mgpt_moe_peer_copy(void* dst, const void* src, size_t bytes, mgpt_stream_t stream);

/* The same plan for callers that can neither pass scratch nor let the library
 * allocate: an engine whose arena already owns all device memory, or a step
 * loop that must never run into cudaMalloc (it synchronises the whole device).
 * This entry point has no counterpart in the reference. Identical outputs to
 * mgpt_moe_op_plan; its scratch is a fixed 512 KiB array inside the library,
 * held by every GPU that loads the library until the process exits, so:
 *   - n_rows may be at most MGPT_MOE_PLAN_NOALLOC_MAX_ROWS (else MGPT_MOE_EINVAL);
 *   - all calls on one GPU share that array: two calls whose kernels may overlap
 *     (different streams, no ordering between them) race on it; keep them in
 *     stream order or use mgpt_moe_op_plan with separate scratch;
 *   - the first call on each device looks up the array's device address
 *     (once, with that device current); that lookup may make the CUDA runtime
 *     load the library's module on the device, which allocates and
 *     synchronises inside the driver.  Make that first call during set-up,
 *     outside the step loop and before any stream capture begins.
 * The call itself makes no cudaMalloc, cudaFree or other allocating call. */
#define MGPT_MOE_PLAN_NOALLOC_MAX_ROWS 1048576
int  mgpt_moe_op_plan_noalloc(const int32_t* top_idx, int n_rows, int E,
                              int32_t* counts, int32_t* offsets, int32_t* padded_offsets,
                              int32_t* tile_expert, int32_t* n_tiles, int32_t* map, int32_t* pos,
                              int32_t* row_src, int row_cap, int32_t* status, mgpt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MGPT_MOE_H */
