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

constexpr int R_WARPS = 4;     // warps per CTA
constexpr int R_CK = 32;       // channels staged per step
constexpr int R_XPAD = 36;     // padded row of the staged x tile (floats): rows land in distinct banks

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

// Bias, softmax with the reference's summation order, clamp and top-k for the TPW token groups of a warp whose
// logit sums are in acc (layers/MoELayer.cpp:96-131).
template <int EL, int EPL, int TPW>
__device__ __forceinline__ void router_finish(const float (&acc)[TPW][EPL], const int* stok, int warp, int sub, int el,
                                              int E, int k, const float* __restrict__ br, float* __restrict__ logits,
                                              float* __restrict__ probs, int32_t* __restrict__ top_idx,
                                              float* __restrict__ top_p)
{
    constexpr int SUB = 32 / EL;
    constexpr int TOK_W = TPW * SUB;
    float bias[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) bias[i] = (el + 32 * i < E) ? br[el + 32 * i] : 0.0f;

    const unsigned full = 0xffffffffu;
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
        // every lane runs the warp-level steps (tokens past N compute on zeros and store nothing)
        const int tok = stok[warp * TOK_W + t * SUB + sub];
        const bool live = tok >= 0;
        float lg[EPL], p[EPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            lg[i] = __fadd_rn(acc[t][i], bias[i]);
            if (el + 32 * i < E) mx = fmaxf(mx, lg[i]);
        }
#pragma unroll
        for (int o = EL / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(full, mx, o));
        // exp through double and one rounding: agrees with a correctly rounded expf
#pragma unroll
        for (int i = 0; i < EPL; ++i) p[i] = (el + 32 * i < E) ? (float)exp((double)__fsub_rn(lg[i], mx)) : 0.0f;
        // the reference adds the E terms in index order
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int lim = min(EL, E - 32 * i);
            for (int l = 0; l < lim; ++l) sum = __fadd_rn(sum, __shfl_sync(full, p[i], l, EL));
        }
        const float inv = __fdiv_rn(1.0f, fmaxf(sum, 1e-15f));
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            p[i] = fminf(fmaxf(__fmul_rn(p[i], inv), 1e-7f), 1.0f);
            const int e = el + 32 * i;
            if (live && e < E) {
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
                const int e = el + 32 * i;
                if (e < E && !(taken & (1u << i)) && p[i] > bv) {
                    bv = p[i];
                    bi = e;
                }
            }
#pragma unroll
            for (int o = EL / 2; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(full, bv, o);
                const int oi = __shfl_xor_sync(full, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            if ((bi & 31) == el && bi != 0x7fffffff) taken |= 1u << (bi >> 5);
            if (el == r) {
                my_idx = bi;
                my_val = bv;
            }
        }
        if (live && el < k) {
            top_idx[(size_t)tok * k + el] = my_idx;
            top_p[(size_t)tok * k + el] = my_val;
        }
    }
}

// EL lanes share one token (lane % EL owns experts el, el+32, ...: EPL of them, EPL > 1 only
// with EL = 32); a warp therefore works on 32/EL tokens at once and on TPW such groups in
// sequence, which gives every lane TPW*EPL independent accumulation chains.
// FAST: C is a multiple of 32 and E fills the staged columns exactly, so both tiles are copied
// with 16-byte loads into registers one chunk ahead of the arithmetic (double-buffered tiles,
// one barrier per chunk); otherwise a plain staged loop handles ragged shapes.
template <typename TIn, int EL, int EPL, int TPW, bool FAST>
__global__ void __launch_bounds__(R_WARPS * 32)
router_fwd_kernel(const TIn* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ br,
                  int N, int C, int E, int k,
                  float* __restrict__ logits, float* __restrict__ probs,
                  int32_t* __restrict__ top_idx, float* __restrict__ top_p,
                  const int32_t* __restrict__ list, const int32_t* __restrict__ list_count)
{
    constexpr int SUB = 32 / EL;                    // tokens per warp pass
    constexpr int TOK_W = TPW * SUB;                // tokens per warp
    constexpr int TOK = R_WARPS * TOK_W;            // tokens per CTA
    constexpr int WCOLS = EPL * EL;                 // staged expert columns
    constexpr int NBUF = FAST ? 2 : 1;
    constexpr int THREADS = R_WARPS * 32;
    __shared__ __align__(16) float xs[NBUF][TOK][R_XPAD];
    __shared__ __align__(16) float wsm[NBUF][R_CK][WCOLS];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane / EL, el = lane % EL;
    const int tok0 = blockIdx.x * TOK;

    // The CTA's tokens: a contiguous range, or -- second pass of the screened router -- entries of a list of
    // token indices whose length is only known on the device (CTAs beyond it leave at once).
    __shared__ int stok[TOK];
    const int n_active = list ? *list_count : N;
    if (tok0 >= n_active) return;
    for (int i = tid; i < TOK; i += THREADS) {
        const int idx = tok0 + i;
        stok[i] = idx < n_active ? (list ? list[idx] : idx) : -1;
    }
    __syncthreads();
    if (list) {
        // Listed tokens are scattered rows the first pass read a while ago: ask for all of each row now, so that the
        // per-chunk loads below find it in L2 instead of paying a DRAM round trip per 32 channels.
        const int lines = (C * (int)sizeof(TIn) + 127) / 128;
        for (int i = tid; i < TOK * lines; i += THREADS) {
            const int tok = stok[i / lines];
            if (tok >= 0)
                asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)(x + (size_t)tok * C) + (size_t)(i % lines) * 128));
        }
    }

    float acc[TPW][EPL];
#pragma unroll
    for (int t = 0; t < TPW; ++t)
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[t][i] = 0.0f;

    // sequential over the 32 staged channels: acc = fadd(acc, fmul(x, w)), the reference's order
    auto compute = [&](int buf) {
#pragma unroll 2
        for (int j = 0; j < R_CK; j += 4) {
            float4 xv[TPW];
#pragma unroll
            for (int t = 0; t < TPW; ++t)
                xv[t] = *reinterpret_cast<const float4*>(&xs[buf][warp * TOK_W + t * SUB + sub][j]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float w[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) w[i] = wsm[buf][j + jj][el + 32 * i];
#pragma unroll
                for (int t = 0; t < TPW; ++t) {
                    const float xe = jj == 0 ? xv[t].x : jj == 1 ? xv[t].y : jj == 2 ? xv[t].z : xv[t].w;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) acc[t][i] = __fadd_rn(acc[t][i], __fmul_rn(xe, w[i]));
                }
            }
        }
    };

    if constexpr (FAST) {
        constexpr int XV = 16 / sizeof(TIn);            // elements per 16-byte piece
        constexpr int XPT = R_CK / XV;                  // pieces per token per chunk
        constexpr int X_VECS = TOK * XPT, X_PER = (X_VECS + THREADS - 1) / THREADS;
        constexpr int W_VECS = R_CK * WCOLS / 4, W_PER = (W_VECS + THREADS - 1) / THREADS;
        uint4 xr[X_PER];
        float4 wr[W_PER];
        auto gload = [&](int c0) {
#pragma unroll
            for (int u = 0; u < X_PER; ++u) {
                const int v = tid + u * THREADS;
                xr[u] = make_uint4(0, 0, 0, 0);
                if (v < X_VECS) {
                    const int tok = stok[v / XPT];
                    if (tok >= 0) xr[u] = *reinterpret_cast<const uint4*>(x + (size_t)tok * C + c0 + (v % XPT) * XV);
                }
            }
#pragma unroll
            for (int u = 0; u < W_PER; ++u) {
                const int v = tid + u * THREADS;
                if (v < W_VECS) wr[u] = *reinterpret_cast<const float4*>(Wr + (size_t)c0 * E + v * 4);
            }
        };
        auto sstore = [&](int buf) {
#pragma unroll
            for (int u = 0; u < X_PER; ++u) {
                const int v = tid + u * THREADS;
                if (v < X_VECS) {
                    float* dst = &xs[buf][v / XPT][(v % XPT) * XV];
                    if constexpr (sizeof(TIn) == 2) {
                        const uint32_t w4[4] = {xr[u].x, xr[u].y, xr[u].z, xr[u].w};
                        *reinterpret_cast<float4*>(dst) = make_float4(
                            __uint_as_float(w4[0] << 16), __uint_as_float(w4[0] & 0xffff0000u),
                            __uint_as_float(w4[1] << 16), __uint_as_float(w4[1] & 0xffff0000u));
                        *reinterpret_cast<float4*>(dst + 4) = make_float4(
                            __uint_as_float(w4[2] << 16), __uint_as_float(w4[2] & 0xffff0000u),
                            __uint_as_float(w4[3] << 16), __uint_as_float(w4[3] & 0xffff0000u));
                    } else {
                        *reinterpret_cast<uint4*>(dst) = xr[u];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < W_PER; ++u) {
                const int v = tid + u * THREADS;
                if (v < W_VECS) *reinterpret_cast<float4*>(&wsm[buf][0][0] + v * 4) = wr[u];
            }
        };
        const int nchunks = C / R_CK;
        gload(0);
        sstore(0);
        __syncthreads();
        for (int ci = 0; ci < nchunks; ++ci) {
            const bool more = ci + 1 < nchunks;
            if (more) gload((ci + 1) * R_CK);          // next chunk's loads fly during this chunk's arithmetic
            compute(ci & 1);
            if (more) sstore((ci + 1) & 1);
            __syncthreads();
        }
    } else {
        for (int c0 = 0; c0 < C; c0 += R_CK) {
            // stage x[tok0.., c0..c0+31] and Wr[c0..c0+31, :] (zero padded: adding 0*w is exact)
#pragma unroll 4
            for (int i = tid; i < TOK * R_CK; i += THREADS) {
                const int t = i / R_CK, j = i % R_CK;
                const int tok = stok[t], c = c0 + j;
                xs[0][t][j] = (tok >= 0 && c < C) ? to_f32(x[(size_t)tok * C + c]) : 0.0f;
            }
#pragma unroll 4
            for (int i = tid; i < R_CK * WCOLS; i += THREADS) {
                const int j = i / WCOLS, e = i % WCOLS;
                const int c = c0 + j;
                wsm[0][j][e] = (c < C && e < E) ? Wr[(size_t)c * E + e] : 0.0f;
            }
            __syncthreads();
            compute(0);
            __syncthreads();
        }
    }

    router_finish<EL, EPL, TPW>(acc, stok, warp, sub, el, E, k, br, logits, probs, top_idx, top_p);
}

// The exact pass over a LIST of tokens (second pass of the screened router): a few thousand tokens, so only a CTA or
// two per SM, and what decides the time is the latency of one CTA's 64 chunk steps.  The chunks therefore come
// through a ring of shared-memory stages filled by cp.async three chunks ahead (the kernel above loads one chunk
// ahead through registers, which is enough only when a dozen CTAs per SM hide each other's waits).  Same arithmetic:
// one warp pass per token, lane el owns experts el, el+32, ..., acc = fadd(acc, fmul(x, w)) in channel order.
// Needs C % 32 == 0, E == 32*EPL and 16-byte aligned x and Wr.
// TPW tokens per warp: 4 for the list pass (fewer instructions per token), 1 for decode batches without a list
// (tokens 0..N-1; the shortest chains per lane, so that a handful of CTAs finish soonest).
template <typename TIn, int EPL, int TPW>
__global__ void __launch_bounds__(R_WARPS * 32)
router_list_kernel(const TIn* __restrict__ x, const float* __restrict__ Wr, const float* __restrict__ br,
                   int N, int C, int E, int k, float* __restrict__ logits, float* __restrict__ probs,
                   int32_t* __restrict__ top_idx, float* __restrict__ top_p,
                   const int32_t* __restrict__ list, const int32_t* __restrict__ list_count)
{
    constexpr int TOK = R_WARPS * TPW, WCOLS = 32 * EPL, THREADS = R_WARPS * 32;
    constexpr int ST = EPL <= 2 ? 4 : 2;            // stages: 36 KiB of static shared memory at most
    constexpr int XV = 16 / sizeof(TIn);            // elements per 16-byte piece
    constexpr int XPT = R_CK / XV;                  // pieces per token per chunk
    constexpr int W_VECS = R_CK * WCOLS / 4;
    __shared__ __align__(16) TIn xs[ST][TOK][R_CK];
    __shared__ __align__(16) float wsm[ST][R_CK][WCOLS];
    __shared__ int stok[TOK];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_active = list ? *list_count : N;
    const int tok0 = blockIdx.x * TOK;
    if (tok0 >= n_active) return;
    for (int i = tid; i < TOK; i += THREADS) stok[i] = tok0 + i < n_active ? (list ? list[tok0 + i] : tok0 + i) : -1;
    __syncthreads();

    auto issue = [&](int ci, int buf) {
        const int c0 = ci * R_CK;
        for (int v = tid; v < W_VECS; v += THREADS) {
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&wsm[buf][0][0] + v * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(Wr + (size_t)c0 * E + v * 4) : "memory");
        }
        for (int v = tid; v < TOK * XPT; v += THREADS) {
            const int tok = stok[v / XPT];
            TIn* d = &xs[buf][v / XPT][(v % XPT) * XV];
            if (tok >= 0) {
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(d);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(x + (size_t)tok * C + c0 + (v % XPT) * XV) : "memory");
            } else {
                *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);      // adding 0*w is exact
            }
        }
    };

    float acc[TPW][EPL];
#pragma unroll
    for (int t = 0; t < TPW; ++t)
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[t][i] = 0.0f;

    auto compute = [&](int buf) {
#pragma unroll 2
        for (int j = 0; j < R_CK; j += 4) {
            float xv[TPW][4];
#pragma unroll
            for (int t = 0; t < TPW; ++t) {
                if constexpr (sizeof(TIn) == 2) {
                    const uint2 u = *reinterpret_cast<const uint2*>(&xs[buf][warp * TPW + t][j]);
                    xv[t][0] = __uint_as_float(u.x << 16); xv[t][1] = __uint_as_float(u.x & 0xffff0000u);
                    xv[t][2] = __uint_as_float(u.y << 16); xv[t][3] = __uint_as_float(u.y & 0xffff0000u);
                } else {
                    const float4 f = *reinterpret_cast<const float4*>(&xs[buf][warp * TPW + t][j]);
                    xv[t][0] = f.x; xv[t][1] = f.y; xv[t][2] = f.z; xv[t][3] = f.w;
                }
            }
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float w[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) w[i] = wsm[buf][j + jj][lane + 32 * i];
#pragma unroll
                for (int t = 0; t < TPW; ++t)
#pragma unroll
                    for (int i = 0; i < EPL; ++i) acc[t][i] = __fadd_rn(acc[t][i], __fmul_rn(xv[t][jj], w[i]));
            }
        }
    };

    const int nchunks = C / R_CK;
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) {
        if (s < nchunks) issue(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int ci = 0; ci < nchunks; ++ci) {
        asm volatile("cp.async.wait_group %0;" ::"n"(ST - 2) : "memory");
        __syncthreads();                               // chunk ci has landed for everyone; chunk ci-1's stage is free
        const int nxt = ci + ST - 1;
        if (nxt < nchunks) issue(nxt, nxt % ST);
        asm volatile("cp.async.commit_group;" ::: "memory");
        compute(ci % ST);
    }
    router_finish<32, EPL, TPW>(acc, stok, warp, 0, lane, E, k, br, logits, probs, top_idx, top_p);
}

// dlogits = P * (dP - <dP,P>),  dP = scatter(d_top_p) + alpha*E*f_e/N
// (layers/MoELayer.cpp:189-210).  One warp per token, grid-stride over tokens.  Optionally also
// writes a bf16 copy with rows padded to E8 columns (for the tensor-core backward) and adds
// the column sums to gbr (layers/LinearLayer.cpp:56-57).
template <int EPL>
__global__ void __launch_bounds__(256)
router_dlogits_kernel(const float* __restrict__ probs, const int32_t* __restrict__ top_idx,
                      const float* __restrict__ d_top_p, const int32_t* __restrict__ counts,
                      int N, int E, int k, float alpha, float* __restrict__ dlogits,
                      bf16* __restrict__ dl16, int E8, float* __restrict__ gbr)
{
    __shared__ float bred[8][EPL * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned full = 0xffffffffu;
    float lb[EPL], bsum[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = lane + 32 * i;
        bsum[i] = 0.0f;
        lb[i] = 0.0f;
        if (e < E) {
            const float f = __fdiv_rn((float)counts[e], (float)N);
            lb[i] = __fdiv_rn(__fmul_rn(__fmul_rn(alpha, (float)E), f), (float)N);
        }
    }
    for (int tok = blockIdx.x * 8 + warp; tok < N; tok += gridDim.x * 8) {
        float p[EPL], dp[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = lane + 32 * i;
            p[i] = 0.0f;
            dp[i] = 0.0f;
            if (e < E) {
                p[i] = probs[(size_t)tok * E + e];
                float sel = 0.0f;
                for (int j = 0; j < k; ++j)
                    if (top_idx[(size_t)tok * k + j] == e) sel = d_top_p[(size_t)tok * k + j];
                dp[i] = __fadd_rn(sel, lb[i]);
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
            const float v = e < E ? __fmul_rn(p[i], __fsub_rn(dp[i], dot)) : 0.0f;
            if (e < E) dlogits[(size_t)tok * E + e] = v;
            if (dl16 && e < E8) dl16[(size_t)tok * E8 + e] = __float2bfloat16(v);
            bsum[i] += v;
        }
    }
    if (gbr) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) bred[warp][lane + 32 * i] = bsum[i];
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            float t = 0.0f;
#pragma unroll
            for (int wv = 0; wv < 8; ++wv) t += bred[wv][e];
            atomicAdd(&gbr[e], t);
        }
    }
}

// dx[tok,:] = sum_j dXg[pos(tok,j),:] (ascending slot order, as the reference's
// scatter-add visits them, utils/Tensor.cpp:1451-1458) + dlogits[tok,:] * Wr^T
// (layers/LinearLayer.cpp:68-69, layers/MoELayer.cpp:217).
// One CTA: DX_TOK tokens x one channel chunk (8192/E_pad channels, Wr^T of the chunk in shared
// memory); a thread owns 8 consecutive channels and uses 16-byte accesses.
constexpr int DX_TOK = 64;
constexpr int DX_WS_FLOATS = 8192;
template <typename TAct, typename TIo>
__global__ void __launch_bounds__(256)
router_dx_kernel(const TAct* __restrict__ dXg, const int32_t* __restrict__ pos, const float* __restrict__ dlogits,
                 const float* __restrict__ Wr, int N, int C, int E, int k, int chunk, TIo* __restrict__ dx)
{
    extern __shared__ __align__(16) float sm_dx[];
    const int wstride = chunk + 4;                      // padded row: transposed staging without 32-way conflicts
    float* wt = sm_dx;                                  // [E][chunk+4]  (Wr^T of this channel chunk)
    float* dlT = sm_dx + DX_WS_FLOATS + 4 * MAX_EXPERTS;   // [E][DX_TOK]  (dlogits^T of this token tile)
    __shared__ int spos[DX_TOK][MAX_TOPK];
    const int tok0 = blockIdx.x * DX_TOK, c_base = blockIdx.y * chunk;
    for (int i = threadIdx.x; i < chunk * E; i += blockDim.x) {
        const int c = i / E, e = i % E;
        wt[e * wstride + c] = (c_base + c < C) ? Wr[(size_t)(c_base + c) * E + e] : 0.0f;
    }
    for (int i = threadIdx.x; i < DX_TOK * E; i += blockDim.x) {
        const int t = i / E, e = i % E;
        dlT[e * DX_TOK + t] = (tok0 + t < N) ? dlogits[(size_t)(tok0 + t) * E + e] : 0.0f;
    }
    if (threadIdx.x < DX_TOK) {
        const int tok = tok0 + threadIdx.x;
        int v[MAX_TOPK];
#pragma unroll
        for (int j = 0; j < MAX_TOPK; ++j) v[j] = (j < k && tok < N) ? pos[(size_t)tok * k + j] : 0x7fffffff;
#pragma unroll
        for (int a = 0; a < MAX_TOPK - 1; ++a)
#pragma unroll
            for (int b = 0; b < MAX_TOPK - 1 - a; ++b)
                if (v[b] > v[b + 1]) {
                    const int tmp = v[b];
                    v[b] = v[b + 1];
                    v[b + 1] = tmp;
                }
#pragma unroll
        for (int j = 0; j < MAX_TOPK; ++j) spos[threadIdx.x][j] = v[j];
    }
    __syncthreads();
    const int groups = chunk / 8;                       // 8-channel groups in the chunk
    const int g = threadIdx.x % groups, ql = threadIdx.x / groups, qstep = blockDim.x / groups;
    const int c = c_base + g * 8;
    if (c >= C) return;
    for (int tq = ql; tq < DX_TOK / 4; tq += qstep) {    // a thread owns 8 channels of 4 consecutive tokens
        if (tok0 + tq * 4 >= N) break;
        float acc[4][8];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[t][i] = 0.0f;
        for (int e = 0; e < E; ++e) {
            const float4 d = *reinterpret_cast<const float4*>(&dlT[e * DX_TOK + tq * 4]);
            const float4 w0 = *reinterpret_cast<const float4*>(&wt[e * wstride + g * 8]);
            const float4 w1 = *reinterpret_cast<const float4*>(&wt[e * wstride + g * 8 + 4]);
            const float dv[4] = {d.x, d.y, d.z, d.w};
            const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[t][i] = fmaf(dv[t], wv[i], acc[t][i]);
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int tl = tq * 4 + t, tok = tok0 + tl;
            if (tok >= N) break;
            float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j = 0; j < k; ++j) {
                const TAct* r = dXg + (size_t)spos[tl][j] * C + c;
                if constexpr (sizeof(TAct) == 2) {
                    const uint4 u = *reinterpret_cast<const uint4*>(r);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        s[2 * i] = __fadd_rn(s[2 * i], __uint_as_float(w[i] << 16));
                        s[2 * i + 1] = __fadd_rn(s[2 * i + 1], __uint_as_float(w[i] & 0xffff0000u));
                    }
                } else {
                    const float4 a = *reinterpret_cast<const float4*>(r), b = *reinterpret_cast<const float4*>(r + 4);
                    s[0] = __fadd_rn(s[0], a.x); s[1] = __fadd_rn(s[1], a.y); s[2] = __fadd_rn(s[2], a.z); s[3] = __fadd_rn(s[3], a.w);
                    s[4] = __fadd_rn(s[4], b.x); s[5] = __fadd_rn(s[5], b.y); s[6] = __fadd_rn(s[6], b.z); s[7] = __fadd_rn(s[7], b.w);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i] = __fadd_rn(s[i], acc[t][i]);
            TIo* o = dx + (size_t)tok * C + c;
            if constexpr (sizeof(TIo) == 4) {
                *reinterpret_cast<float4*>(o) = make_float4(s[0], s[1], s[2], s[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(s[4], s[5], s[6], s[7]);
            } else {
                uint4 u;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(s[0], s[1]), h1 = __floats2bfloat162_rn(s[2], s[3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(s[4], s[5]), h3 = __floats2bfloat162_rn(s[6], s[7]);
                u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
                u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(o) = u;
            }
        }
    }
}

// Router weight gradient in two deterministic steps (layers/LinearLayer.cpp:56-66):
//   part[chunk][c][e] = sum over the chunk's tokens of x[tok,c]*dlogits[tok,e]   (and column sums of dlogits)
//   gWr[c,e] += sum_chunk part[chunk][c][e];  gbr[e] += sum_chunk partb[chunk][e]
// A thread keeps a 4 channel x 4 expert block of accumulators.
template <typename TIo>
__global__ void __launch_bounds__(256)
router_wgrad_partial_kernel(const TIo* __restrict__ x, const float* __restrict__ dlogits, int N, int C, int E,
                            int tok_per_chunk, float* __restrict__ part, float* __restrict__ partb)
{
    const int E4 = (E + 3) / 4;                         // expert groups of 4
    const int cg_per_cta = 256 / E4;                    // channel groups of 4 handled by this CTA
    const int eg = threadIdx.x % E4, cgi = threadIdx.x / E4;
    if (cgi >= cg_per_cta) return;
    const int c = (blockIdx.x * cg_per_cta + cgi) * 4, e0 = eg * 4;
    const int t0 = blockIdx.y * tok_per_chunk, t1 = min(N, t0 + tok_per_chunk);
    const bool c_ok = c < C;
    float acc[4][4] = {};
    float bs[4] = {0, 0, 0, 0};
    constexpr int UN = 4;                               // tokens in flight per thread
    for (int tb = t0; tb < t1; tb += UN) {
        float xv[UN][4], dv[UN][4];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int tok = tb + u;
            const bool ok = tok < t1;
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[u][i] = 0.0f;
            if (ok && c_ok) {
                if constexpr (sizeof(TIo) == 2) {
                    const uint2 w = *reinterpret_cast<const uint2*>(x + (size_t)tok * C + c);
                    xv[u][0] = __uint_as_float(w.x << 16); xv[u][1] = __uint_as_float(w.x & 0xffff0000u);
                    xv[u][2] = __uint_as_float(w.y << 16); xv[u][3] = __uint_as_float(w.y & 0xffff0000u);
                } else {
                    const float4 f = *reinterpret_cast<const float4*>(x + (size_t)tok * C + c);
                    xv[u][0] = f.x; xv[u][1] = f.y; xv[u][2] = f.z; xv[u][3] = f.w;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) dv[u][j] = (ok && e0 + j < E) ? dlogits[(size_t)tok * E + e0 + j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[u][i], dv[u][j], acc[i][j]);
#pragma unroll
            for (int j = 0; j < 4; ++j) bs[j] += dv[u][j];
        }
    }
    if (c_ok) {
        float* dst = part + ((size_t)blockIdx.y * C + c) * E;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (e0 + j < E) dst[(size_t)i * E + e0 + j] = acc[i][j];
    }
    if (blockIdx.x == 0 && cgi == 0)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (e0 + j < E) partb[(size_t)blockIdx.y * E + e0 + j] = bs[j];
}

__global__ void __launch_bounds__(256)
router_wgrad_reduce_kernel(const float* __restrict__ part, const float* __restrict__ partb, int n_chunks, int CE, int E,
                           float* __restrict__ gWr, float* __restrict__ gbr)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < CE) {
        float s = 0.0f;
        for (int ch = 0; ch < n_chunks; ++ch) s += part[(size_t)ch * CE + i];
        gWr[i] += s;
    }
    if (i < E) {
        float s = 0.0f;
        for (int ch = 0; ch < n_chunks; ++ch) s += partb[(size_t)ch * E + i];
        gbr[i] += s;
    }
}

template <typename TIn, int EL, int EPL, int TPW>
int router_fwd_launch(const TIn* x, const float* Wr, const float* br, int N, int C, int E, int k,
                      float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st,
                      const int32_t* list, const int32_t* list_count)
{
    constexpr int TOK = R_WARPS * TPW * (32 / EL);
    const int grid = (N + TOK - 1) / TOK;
    const bool fast = C % R_CK == 0 && E == EPL * EL && ((uintptr_t)x & 15) == 0 && ((uintptr_t)Wr & 15) == 0;
    if (fast)
        router_fwd_kernel<TIn, EL, EPL, TPW, true><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, list, list_count);
    else
        router_fwd_kernel<TIn, EL, EPL, TPW, false><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, list, list_count);
    MGPT_LAUNCHED("router_fwd_kernel");
    return 0;
}

template <typename TIn>
int router_fwd_dispatch(const TIn* x, const float* Wr, const float* br, int N, int C, int E, int k,
                        float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st,
                        const int32_t* list, const int32_t* list_count)
{
    // Decode-sized batches: too few tokens to fill the device, what is left is the latency of one CTA, which is the
    // length of its dependent addition chains: one token per warp pass keeps it shortest.
    if (!list && N <= 1024 && C % R_CK == 0 && E % 32 == 0 && E <= 128 && E != 96 && ((uintptr_t)x & 15) == 0 &&
        ((uintptr_t)Wr & 15) == 0) {
        // the chunks through the cp.async ring: with a handful of CTAs, nothing else hides the loads of a chunk
        const int grid = (N + R_WARPS - 1) / R_WARPS;
        if (E == 32) router_list_kernel<TIn, 1, 1><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, nullptr, nullptr);
        else if (E == 64) router_list_kernel<TIn, 2, 1><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, nullptr, nullptr);
        else router_list_kernel<TIn, 4, 1><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, nullptr, nullptr);
        MGPT_LAUNCHED("router_list_kernel<decode>");
        return 0;
    }
    if (!list && N <= 1024) {
        if (E <= 8) return router_fwd_launch<TIn, 8, 1, 1>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
        if (E <= 16) return router_fwd_launch<TIn, 16, 1, 1>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
        if (E <= 32) return router_fwd_launch<TIn, 32, 1, 1>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
        if (E <= 64) return router_fwd_launch<TIn, 32, 2, 1>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
        return router_fwd_launch<TIn, 32, 4, 1>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    }
    // Second pass of the screened router: a fraction of the tokens, how many is only known on the device.  Small
    // CTAs (16 tokens) so that the few thousand listed tokens still spread over every SM.
    if (list && C % R_CK == 0 && E % 32 == 0 && E <= 128 && E != 96 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)Wr & 15) == 0) {
        const int grid = (N + 15) / 16;
        if (E == 32) router_list_kernel<TIn, 1, 4><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, list, list_count);
        else if (E == 64) router_list_kernel<TIn, 2, 4><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, list, list_count);
        else router_list_kernel<TIn, 4, 4><<<grid, R_WARPS * 32, 0, st>>>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, list, list_count);
        MGPT_LAUNCHED("router_list_kernel");
        return 0;
    }
    if (list && E > 32 && E <= 64)
        return router_fwd_launch<TIn, 32, 2, 4>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    if (list && E > 16 && E <= 32)
        return router_fwd_launch<TIn, 32, 1, 4>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    if (E <= 8) return router_fwd_launch<TIn, 8, 1, 4>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    if (E <= 16) return router_fwd_launch<TIn, 16, 1, 4>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    if (E <= 32) return router_fwd_launch<TIn, 32, 1, 8>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    if (E <= 64) return router_fwd_launch<TIn, 32, 2, 8>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    return router_fwd_launch<TIn, 32, 4, 4>(x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
}

}  // namespace

// list / list_count (device): run only on the tokens list[0 .. *list_count), at most N of them
int launch_router_fwd(const void* x, int io, const float* Wr, const float* br, int N, int C, int E, int k,
                      float* logits, float* probs, int32_t* top_idx, float* top_p, cudaStream_t st,
                      const int32_t* list, const int32_t* list_count)
{
    if (N <= 0) return 0;
    if (io == MGPT_MOE_IO_F32)
        return router_fwd_dispatch((const float*)x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
    return router_fwd_dispatch((const bf16*)x, Wr, br, N, C, E, k, logits, probs, top_idx, top_p, st, list, list_count);
}

int launch_router_bwd(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, int io,
                      void* dx, cudaStream_t st, const void* dXg_rows, const int32_t* pos_rows)
{
    const Dims& d = L->d;
    const int N = w.n_tokens, C = d.C, E = d.E, k = d.k;
    if (N <= 0) return 0;
    const float* probs = (const float*)(ws + w.probs);
    const int32_t* top_idx = (const int32_t*)(ws + w.top_idx);
    const float* dtp = (const float*)(ws + w.d_top_p);
    const int32_t* counts = (const int32_t*)(ws + w.counts);
    const int32_t* pos = pos_rows ? pos_rows : (const int32_t*)(ws + w.pos);
    const void* dXg = dXg_rows ? dXg_rows : (const void*)(ws + w.dXg);
    float* dl = (float*)(ws + w.dlogits);
    const float* Wr = L->p_data[0];
    // Tensor-core path: BF16 mode with BF16 tokens (x, dx are TMA operands); gWr rows need 16-byte pieces.
    const bool tc = d.mode == MGPT_MOE_BF16 && d.gemm_impl == 0 && io == MGPT_MOE_IO_BF16;
    const bool tc_wgrad = tc && L->has_grad && E % 4 == 0;
    const int E8 = (E + 7) / 8 * 8;
    {
        const int grid = min((N + 7) / 8, 1184);
        bf16* dl16 = tc ? (bf16*)(ws + w.dl16) : nullptr;
        float* gbr = tc_wgrad ? L->p_grad[1] : nullptr;
        if (E <= 32) router_dlogits_kernel<1><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl, dl16, E8, gbr);
        else if (E <= 64) router_dlogits_kernel<2><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl, dl16, E8, gbr);
        else router_dlogits_kernel<4><<<grid, 256, 0, st>>>(probs, top_idx, dtp, counts, N, E, k, d.alpha, dl, dl16, E8, gbr);
        MGPT_LAUNCHED("router_dlogits_kernel");
    }
    if (tc) {
        MGPT_TRY(tc_router_dx(L, w, ws, dXg, pos, dx, st));
    } else {
        int epad = 8;
        while (epad < E) epad <<= 1;
        const int chunk = DX_WS_FLOATS / epad;                 // channels per CTA (multiple of 8)
        dim3 grid((N + DX_TOK - 1) / DX_TOK, (C + chunk - 1) / chunk);
        const size_t sm = (size_t)(DX_WS_FLOATS + 4 * MAX_EXPERTS + DX_TOK * E) * sizeof(float);
        if (!L->router_dx_attr) {                   // a per-device attribute: one opt-in per layer (layers live on one device)
            MGPT_CUDA(cudaFuncSetAttribute(router_dx_kernel<float, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
            MGPT_CUDA(cudaFuncSetAttribute(router_dx_kernel<bf16, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
            MGPT_CUDA(cudaFuncSetAttribute(router_dx_kernel<bf16, bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
            L->router_dx_attr = true;
        }
        if (w.act_bytes == 4) {
            router_dx_kernel<float, float><<<grid, 256, sm, st>>>((const float*)dXg, pos, dl, Wr, N, C, E, k, chunk, (float*)dx);
        } else if (io == MGPT_MOE_IO_F32) {
            router_dx_kernel<bf16, float><<<grid, 256, sm, st>>>((const bf16*)dXg, pos, dl, Wr, N, C, E, k, chunk, (float*)dx);
        } else {
            router_dx_kernel<bf16, bf16><<<grid, 256, sm, st>>>((const bf16*)dXg, pos, dl, Wr, N, C, E, k, chunk, (bf16*)dx);
        }
        MGPT_LAUNCHED("router_dx_kernel");
    }
    if (tc_wgrad) {
        MGPT_TRY(tc_router_wgrad(L, w, ws, x, st));
    } else if (L->has_grad) {
        const int E4 = (E + 3) / 4, ch_per_cta = (256 / E4) * 4;
        const int cblocks = (C + ch_per_cta - 1) / ch_per_cta;
        float* part = (float*)(ws + w.rw_part);
        float* partb = part + (size_t)w.rw_chunks * C * E;
        const int tpc = (N + w.rw_chunks - 1) / w.rw_chunks;
        dim3 grid(cblocks, w.rw_chunks);
        if (io == MGPT_MOE_IO_F32)
            router_wgrad_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)x, dl, N, C, E, tpc, part, partb);
        else
            router_wgrad_partial_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x, dl, N, C, E, tpc, part, partb);
        MGPT_LAUNCHED("router_wgrad_partial_kernel");
        router_wgrad_reduce_kernel<<<(C * E + 255) / 256, 256, 0, st>>>(part, partb, w.rw_chunks, C * E, E,
                                                                      L->p_grad[0], L->p_grad[1]);
        MGPT_LAUNCHED("router_wgrad_reduce_kernel");
    }
    return 0;
}

}  // namespace mgpt
