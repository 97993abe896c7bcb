/*
 * CPU oracle for the mgpt Mixture-of-Experts layer (forward + backward).
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * CPU arithmetic, used to check the CUDA path and as a timed CPU baseline.
 * Nothing in the shipped library links, imports or calls it.
 *
 * Parity status: PINNED. The restatement is compared bit-for-bit against the
 * reference's own MoELayer (compiled from its sources into oracle/_ref by
 * oracle/Makefile) and against the committed vectors in tests/golden/, which
 * were produced by that build.
 */
#ifndef MOE_ORACLE_H
#define MOE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int n_tokens;   /* N = B*T                                        */
    int C;          /* embed_dim                                      */
    int H;          /* SwiGLU hidden_dim                              */
    int E;          /* num_experts                                    */
    int k;          /* top_k                                          */
    float alpha;    /* load-balance coefficient (reference: 0.01f)    */
} moe_oracle_dims;

/* Parameter order (MoELayer.cpp:225-236, SwiGLU.cpp:98-104, LinearLayer.cpp:87-89):
 *   [0] Wr [C,E]   [1] br [E]
 *   per expert e:  [2+6e] Wg [C,H]  [3+6e] bg [H]  [4+6e] Wu [C,H]
 *                  [5+6e] bu [H]    [6+6e] Wd [H,C] [7+6e] bd [C]         */
typedef struct {
    const float* x;               /* [N,C]                                */
    const float* const* params;   /* 2+6E pointers                        */
    const float* dy;              /* [N,C]; NULL = forward only           */
} moe_oracle_inputs;

/* Every pointer may be NULL (that result is then not reported). */
typedef struct {
    float*   logits;        /* [N,E]  router pre-softmax                     */
    float*   probs;         /* [N,E]  clamped softmax                        */
    int32_t* top_idx;       /* [N,k]  expert ids, best first                 */
    float*   top_p;         /* [N,k]                                         */
    int32_t* counts;        /* [E]                                           */
    int32_t* offsets;       /* [E]    exclusive prefix sum of counts         */
    int32_t* map;           /* [N*k]  slot -> flat index tok*k+j             */
    float*   gathered_out;  /* [N*k,C] expert outputs in slot order          */
    float*   y;             /* [N,C]                                         */
    float*   d_top_p;       /* [N,k]                                         */
    float*   dlogits;       /* [N,E]                                         */
    float*   dx;            /* [N,C]                                         */
    float* const* grads;    /* 2+6E pointers, accumulated into (+=)          */
} moe_oracle_outputs;

/* Returns 0 on success. n_threads > 1 splits independent output rows across
 * POSIX threads; every output element is still summed in the reference's
 * order, so results do not depend on n_threads. */
int moe_oracle_run(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                   moe_oracle_outputs* out, int n_threads);

/* Router + dispatch plan only (logits .. map); cheap at full benchmark sizes. */
int moe_oracle_route(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                     moe_oracle_outputs* out, int n_threads);

/* Timed runs for the CPU baseline (setup and gradient clearing are untimed). */
int moe_oracle_bench(const moe_oracle_dims* d, const moe_oracle_inputs* in, int iters, double* seconds,
                     int n_threads);

/* One AdamW step on a flat tensor of n floats, in place on w, m, v: the reference's CPU arithmetic
 * (utils/Tensor.cpp:683-699, driven by optimisers/AdamWOptimiser.h:24-36).  t is the 1-based step count. */
int moe_oracle_adamw(float* w, const float* g, float* m, float* v, long n, float lr, float beta1, float beta2,
                     float eps, float weight_decay, int t);

#ifdef __cplusplus
}
#endif
#endif
