// Router of the MoE layer: gating product, clamped softmax and top-k fused in
// one pass over x, and the matching backward kernels.
//
// Reference semantics reproduced here (paths relative to the reference's
// src/main/):
//   logits = x*Wr + br      layers/LinearLayer.cpp:23-28, utils/Tensor.cpp:567-577
//   P = clamp(softmax)      utils/Tensor.cpp:850-883 (inv = 1/max(sum,1e-15), clamp [1e-7,1])
//   top-k, strict '>'       utils/Tensor.cpp:1296-1334 (ties keep the lowest index)
//   backward                layers/MoELayer.cpp:189-218, utils/Tensor.cpp:885-909
//
// Routing must equal the CPU reference bit for bit, so the gating product is
// accumulated per (token, expert) sequentially over channels with a separate
// FP32 multiply and add, exactly the order of the reference's i-k-j loop.
#include "common.cuh"

namespace mgpt {

namespace {

constexpr int R_WARPS = 8;     // warps per CTA
constexpr int R_TPW = 8;       // tokens per warp (independent accumulation chains)
constexpr int R_TOK = R_WARPS * R_TPW;
constexpr int R_CK = 32;       // channels staged per step

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

// One warp owns R_TPW tokens; lane l owns experts l, l+32, ... (EPL of them).
template <typename TIn, int EPL>
__global__ void __launch_bounds__(R_WARPS * 32)
router_fwd_kernel(const TIn* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ br,
                  int N, int C, int E, int k,
                  float* __restrict__ logits, float* __restrict__ probs,
                  int32_t* __restrict__ top_idx, float* __restrict__ top_p)
{
    __shared__ __align__(16) float xs[R_TOK][R_CK];
    __shared__ float wsm[R_CK][EPL * 32];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tok0 = blockIdx.x * R_TOK;

    float acc[R_TPW][EPL];
#pragma unroll
    for (int t = 0; t < R_TPW; ++t)
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[t][i] = 0.0f;

    for (int c0 = 0; c0 < C; c0 += R_CK) {
        // stage x[tok0.., c0..c0+31] and Wr[c0..c0+31, :] (zero padded: adding 0*w is exact)
        for (int i = tid; i < R_TOK * R_CK; i += R_WARPS * 32) {
            int t = i / R_CK, j = i % R_CK;
            int tok = tok0 + t, c = c0 + j;
            xs[t][j] = (tok < N && c < C) ? to_f32(x[(size_t)tok * C + c]) : 0.0f;
        }
        for (int i = tid; i < R_CK * EPL * 32; i += R_WARPS * 32) {
            int j = i / (EPL * 32), e = i % (EPL * 32);
            int c = c0 + j;
            wsm[j][e] = (c < C && e < E) ? Wr[(size_t)c * E + e] : 0.0f;
        }
        __syncthreads();
#pragma unroll 2
        for (int j = 0; j < R_CK; j += 4) {
            float4 xv[R_TPW];
#pragma unroll
            for (int t = 0; t < R_TPW; ++t) xv[t] = *reinterpret_cast<const float4*>(&xs[warp * R_TPW + t][j]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float w[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) w[i] = wsm[j + jj][lane + 32 * i];
#pragma unroll
                for (int t = 0; t < R_TPW; ++t) {
                    const float xe = jj == 0 ? xv[t].x : jj == 1 ? xv[t].y : jj == 2 ? xv[t].z : xv[t].w;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) acc[t][i] = __fadd_rn(acc[t][i], __fmul_rn(xe, w[i]));
                }
            }
        }
        __syncthreads();
    }

    float bias[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) bias[i] = (lane + 32 * i < E) ? br[lane + 32 * i] : 0.0f;

    const unsigned full = 0xffffffffu;
#pragma unroll
    for (int t = 0; t < R_TPW; ++t) {
        const int tok = tok0 + warp * R_TPW + t;
        if (tok >= N) continue;                    // warp-uniform
        float lg[EPL], p[EPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            lg[i] = __fadd_rn(acc[t][i], bias[i]);
            if (lane + 32 * i < E) mx = fmaxf(mx, lg[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, o));
        // exp through double and one rounding: agrees with a correctly rounded expf
#pragma unroll
        for (int i = 0; i < EPL; ++i) p[i] = (float)exp((double)__fsub_rn(lg[i], mx));
        // the reference adds the E terms in index order
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int lim = min(32, E - 32 * i);
            for (int l = 0; l < lim; ++l) sum = __fadd_rn(sum, __shfl_sync(full, p[i], l));
        }
        const float inv = __fdiv_rn(1.0f, fmaxf(sum, 1e-15f));
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            p[i] = fminf(fmaxf(__fmul_rn(p[i], inv), 1e-7f), 1.0f);
            const int e = lane + 32 * i;
            if (e < E) {
                probs[(size_t)tok * E + e] = p[i];
                if (logits) logits[(size_t)tok * E + e] = lg[i];
            }
        }
        // k rounds of (value desc, index asc) arg-max == the reference's stable insertion
        unsigned taken = 0;
        int my_idx = -1;
        float my_val = 0.0f;
        for (int r = 0; r < k; ++r) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int e = lane + 32 * i;
                if (e < E && !(taken & (1u << i)) && p[i] > bv) {
                    bv = p[i];
                    bi = e;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(full, bv, o);
                const int oi = __shfl_xor_sync(full, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
            if (lane == r) {
                my_idx = bi;
                my_val = bv;
            }
        }
        if (lane < k) {
            top_idx[(size_t)tok * k + lane] = my_idx;
            top_p[(size_t)tok * k + lane] = my_val;
        }
    }
}

// dlogits = P * (dP - <dP,P>),  dP = scatter(d_top_p) + alpha*E*f_e/N
// (layers/MoELayer.cpp:189-210).  One warp per token.
template <int EPL>
__global__ void __launch_bounds__(256)
router_dlogits_kernel(const float* __restrict__ probs, const int32_t* __restrict__ top_idx,
                      const float* __restrict__ d_top_p, const int32_t* __restrict__ counts,
                      int N, int E, int k, float alpha, float* __restrict__ dlogits)
{
    const int lane = threadIdx.x & 31;
    const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= N) return;
    const unsigned full = 0xffffffffu;
    float p[EPL], dp[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        p[i] = 0.0f;
        dp[i] = 0.0f;
        if (e < E) {
            p[i] = probs[(size_t)tok * E + e];
            const float f = __fdiv_rn((float)counts[e], (float)N);
            const float lb = __fdiv_rn(__fmul_rn(__fmul_rn(alpha, (float)E), f), (float)N);
            float sel = 0.0f;
            for (int j = 0; j < k; ++j)
                if (top_idx[(size_t)tok * k + j] == e) sel = d_top_p[(size_t)tok * k + j];
            dp[i] = __fadd_rn(sel, lb);
        }
    }
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const float prod = __fmul_rn(dp[i], p[i]);
        const int lim = min(32, E - 32 * i);
        for (int l = 0; l < lim; ++l) dot = __fadd_rn(dot, __shfl_sync(full, prod, l));
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        if (e < E) dlogits[(size_t)tok * E + e] = __fmul_rn(p[i], __fsub_rn(dp[i], dot));
    }
}

// dx[tok,:] = sum_j dXg[pos(tok,j),:] (ascending slot order, as the reference's
// scatter-add visits them, utils/Tensor.cpp:1451-1458) + dlogits[tok,:] * Wr^T
// (layers/LinearLayer.cpp:68-69, layers/MoELayer.cpp:217).
constexpr int DX_TOK = 32;
template <typename TAct, typename TIo>
__global__ void __launch_bounds__(256)
router_dx_kernel(const TAct* __restrict__ dXg, const int32_t* __restrict__ pos, const float* __restrict__ dlogits,
                 const float* __restrict__ Wr, int N, int C, int E, int k, TIo* __restrict__ dx)
{
    extern __shared__ float dl[];                 // [DX_TOK][E]
    __shared__ int spos[DX_TOK][MAX_TOPK];
    const int tok0 = blockIdx.x * DX_TOK;
    for (int i = threadIdx.x; i < DX_TOK * E; i += blockDim.x) {
        const int t = i / E, e = i % E;
        dl[i] = (tok0 + t < N) ? dlogits[(size_t)(tok0 + t) * E + e] : 0.0f;
    }
    if (threadIdx.x < DX_TOK) {
        const int tok = tok0 + threadIdx.x;
        int v[MAX_TOPK];
        for (int j = 0; j < k; ++j) v[j] = tok < N ? pos[(size_t)tok * k + j] : 0;
        for (int a = 1; a < k; ++a) {             // insertion sort, k <= 8
            int key = v[a], b = a - 1;
            while (b >= 0 && v[b] > key) {
                v[b + 1] = v[b];
                --b;
            }
            v[b + 1] = key;
        }
        for (int j = 0; j < k; ++j) spos[threadIdx.x][j] = v[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc[DX_TOK];
#pragma unroll
        for (int t = 0; t < DX_TOK; ++t) acc[t] = 0.0f;
        for (int e0 = 0; e0 < E; e0 += 8) {
            float w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = (e0 + i < E) ? Wr[(size_t)c * E + e0 + i] : 0.0f;
#pragma unroll
            for (int t = 0; t < DX_TOK; ++t)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (e0 + i < E) acc[t] = __fadd_rn(acc[t], __fmul_rn(dl[t * E + e0 + i], w[i]));
        }
#pragma unroll
        for (int t = 0; t < DX_TOK; ++t) {
            const int tok = tok0 + t;
            if (tok >= N) continue;
            float s = 0.0f;
            for (int j = 0; j < k; ++j) s = __fadd_rn(s, to_f32(dXg[(size_t)spos[t][j] * C + c]));
            const float r = __fadd_rn(s, acc[t]);
            if constexpr (sizeof(TIo) == 4) dx[(size_t)tok * C + c] = r;
            else dx[(size_t)tok * C + c] = __float2bfloat16(r);
        }
    }
}

// gWr[c,e] += sum_tok x[tok,c]*dlogits[tok,e];  gbr[e] += sum_tok dlogits[tok,e]
// (layers/LinearLayer.cpp:56-66).  grid (ceil(C/32), token chunks).
constexpr int WG_CH = 32, WG_TT = 32, WG_CHUNK = 256;
template <typename TIo>
__global__ void __launch_bounds__(256)
router_wgrad_kernel(const TIo* __restrict__ x, const float* __restrict__ dlogits, int N, int C, int E,
                    float* __restrict__ gWr, float* __restrict__ gbr)
{
    extern __shared__ float sm[];
    float* xs = sm;                  // [WG_TT][WG_CH]
    float* dls = sm + WG_TT * WG_CH; // [WG_TT][E]
    const int c_l = threadIdx.x & 31, eg = threadIdx.x >> 5;
    const int c0 = blockIdx.x * WG_CH;
    const int t_begin = blockIdx.y * WG_CHUNK, t_end = min(N, t_begin + WG_CHUNK);
    float acc[MAX_EXPERTS / 8];
#pragma unroll
    for (int i = 0; i < MAX_EXPERTS / 8; ++i) acc[i] = 0.0f;
    float bsum = 0.0f;
    for (int t0 = t_begin; t0 < t_end; t0 += WG_TT) {
        for (int i = threadIdx.x; i < WG_TT * WG_CH; i += blockDim.x) {
            const int t = i / WG_CH, j = i % WG_CH;
            const int tok = t0 + t, c = c0 + j;
            xs[i] = (tok < t_end && c < C) ? to_f32(x[(size_t)tok * C + c]) : 0.0f;
        }
        for (int i = threadIdx.x; i < WG_TT * E; i += blockDim.x) {
            const int t = i / E;
            dls[i] = (t0 + t < t_end) ? dlogits[(size_t)(t0 + t) * E + (i % E)] : 0.0f;
        }
        __syncthreads();
        for (int t = 0; t < WG_TT; ++t) {
            const float xv = xs[t * WG_CH + c_l];
#pragma unroll
            for (int i = 0; i < MAX_EXPERTS / 8; ++i)
                if (eg + 8 * i < E) acc[i] = fmaf(xv, dls[t * E + eg + 8 * i], acc[i]);
        }
        if (blockIdx.x == 0 && threadIdx.x < E)
            for (int t = 0; t < WG_TT; ++t) bsum += dls[t * E + threadIdx.x];
        __syncthreads();
    }
    const int c = c0 + c_l;
    if (c < C) {
#pragma unroll
        for (int i = 0; i < MAX_EXPERTS / 8; ++i)
            if (eg + 8 * i < E) atomicAdd(&gWr[(size_t)c * E + eg + 8 * i], acc[i]);
    }
    if (blockIdx.x == 0 && threadIdx.x < E) atomicAdd(&gbr[threadIdx.x], bsum);
}

template <typename TIn>
int router_fwd_dispatch(const TIn* x, const float* Wr, const float* br, int N, int C, int E, int k,
                        float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st)
{
    const int grid = (N + R_TOK - 1) / R_TOK;
    if (E <= 32)
        router_fwd_kernel<TIn, 1><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p);
    else if (E <= 64)
        router_fwd_kernel<TIn, 2><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p);
    else
        router_fwd_kernel<TIn, 4><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p);
    MGPT_LAUNCHED("router_fwd_kernel");
    return 0;
}

}  // namespace

int launch_router_fwd(const void* x, int io, const float* Wr, const float* br, int N, int C, int E, int k,
                      float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st)
{
    if (N <= 0) return 0;
    if (io == MGPT_MOE_IO_F32)
        return router_fwd_dispatch((const float*)x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st);
    return router_fwd_dispatch((const bf16*)x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st);
}

int launch_router_bwd(const mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, int io,
                      void* dx, cudaStream_t st)
{
    const Dims& d = L->d;
    const int N = w.n_tokens, C = d.C, E = d.E, k = d.k;
    if (N <= 0) return 0;
    const float* probs = (const float*)(ws + w.probs);
    const int32_t* top_idx = (const int32_t*)(ws + w.top_idx);
    const float* dtp = (const float*)(ws + w.d_top_p);
    const int32_t* counts = (const int32_t*)(ws + w.counts);
    const int32_t* pos = (const int32_t*)(ws + w.pos);
    float* dl = (float*)(ws + w.dlogits);
    const float* Wr = L->p_data[0];

    {
        const int grid = (N + 7) / 8;
        if (E <= 32) router_dlogits_kernel<1><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl);
        else if (E <= 64) router_dlogits_kernel<2><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl);
        else router_dlogits_kernel<4><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl);
        MGPT_LAUNCHED("router_dlogits_kernel");
    }
    {
        const int grid = (N + DX_TOK - 1) / DX_TOK;
        const size_t sm = (size_t)DX_TOK * E * sizeof(float);
        const void* dXg = ws + w.dXg;
        if (w.act_bytes == 4) {
            if (io == MGPT_MOE_IO_F32)
                router_dx_kernel<float, float><<<grid, 256, sm, st>>>((const float*)dXg, pos, dl, Wr, N, C, E, k, (float*)dx);
            else
                router_dx_kernel<float, bf16><<<grid, 256, sm, st>>>((const float*)dXg, pos, dl, Wr, N, C, E, k, (bf16*)dx);
        } else {
            if (io == MGPT_MOE_IO_F32)
                router_dx_kernel<bf16, float><<<grid, 256, sm, st>>>((const bf16*)dXg, pos, dl, Wr, N, C, E, k, (float*)dx);
            else
                router_dx_kernel<bf16, bf16><<<grid, 256, sm, st>>>((const bf16*)dXg, pos, dl, Wr, N, C, E, k, (bf16*)dx);
        }
        MGPT_LAUNCHED("router_dx_kernel");
    }
    if (L->has_grad) {
        dim3 grid((C + WG_CH - 1) / WG_CH, (N + WG_CHUNK - 1) / WG_CHUNK);
        const size_t sm = (size_t)(WG_TT * WG_CH + WG_TT * E) * sizeof(float);
        if (io == MGPT_MOE_IO_F32)
            router_wgrad_kernel<float><<<grid, 256, sm, st>>>((const float*)x, dl, N, C, E, L->p_grad[0], L->p_grad[1]);
        else
            router_wgrad_kernel<bf16><<<grid, 256, sm, st>>>((const bf16*)x, dl, N, C, E, L->p_grad[0], L->p_grad[1]);
        MGPT_LAUNCHED("router_wgrad_kernel");
    }
    return 0;
}

}  // namespace mgpt
