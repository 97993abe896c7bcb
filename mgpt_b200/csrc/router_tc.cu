// Router forward for BF16 tokens at HBM speed: a tensor-core first pass that PROVES the routing of most tokens,
// and an exact second pass over the rest.
//
// The reference routes on FP32 logits accumulated channel by channel (utils/Tensor.cpp:567-577), clamped softmax
// (utils/Tensor.cpp:850-883) and a strict '>' top-k (utils/Tensor.cpp:1296-1334).  Indices, per-expert counts and
// the slot permutation must equal it bit for bit.  Redoing its 2*N*C*E separate multiplies and adds is bound by
// FP32 issue, far from the memory roofline, so the work is split:
//
//   pass 1 (this file): logits ~= x * Wr on the tensor cores.  x is BF16; Wr^T is kept as two BF16 pieces
//     (Wr = hi + mid up to 2^-16 relative), so every product is exact and only the accumulation order differs
//     from the reference.  For token t and every expert
//         |logit_ref - logit_tc| <= B_t = (1.5*C*u + 2^-16) * ||x_t||_2 * max_e ||Wr[:,e]||_2 + (bias roundings)
//     (u = 2^-24.  C*u*sum|x w| bounds the reference's sequential FP32 sum of C exact products.  The tensor core
//     adds 16 exact products to the FP32 accumulator per instruction and rounds once, at worst by truncation:
//     2*(C/16)*2u*sum|x w| = C*u/4*sum|x w| over the two pieces; it is given twice that.  sum|x w| <= ||x|| ||w||
//     by Cauchy-Schwarz).  ||x_t||_2 comes from the same shared-memory
//     tile the tensor core reads.  If the token's top-(k+1) logits are pairwise more than 2*B_t apart and its
//     k-th probability is clear of the clamp floor, the reference's order of those experts is the same, whatever
//     its rounding did: indices are final.  Probabilities are written from the pass-1 logits (they differ from
//     the reference's by ~1e-6 relative, far inside the layer's BF16 tolerance).
//   pass 2: every other token (a few percent to ~20 %) is appended to a list and recomputed by the exact
//     kernel of router.cu, which overwrites its logits, probabilities and top-k.
//
// One thread owns one token in the epilogue (TMEM lane = row), so softmax and top-k need no shuffles.
#include "tc_common.cuh"

namespace mgpt {

namespace {

using namespace tcx;

constexpr int RT_BM = 128, RT_BK = 64;
constexpr int RT_THREADS = 64 + 128 + 128;        // warp 0: TMA, warp 1: MMA, warps 2-5: row norms, warps 6-9: epilogue
constexpr uint32_t RT_A_BYTES = RT_BM * RT_BK * 2;
constexpr uint32_t RT_TMEM_COLS = 256;            // two accumulators of up to 128 columns

template <int NE> struct RtCfg {
    static constexpr uint32_t B_BYTES = 2u * NE * RT_BK * 2;     // hi and mid pieces
    static constexpr uint32_t STAGE = RT_A_BYTES + B_BYTES;
    static constexpr int STAGES = (int)((196608u) / STAGE) > 8 ? 8 : (int)((196608u) / STAGE);
    static constexpr uint32_t SMEM = STAGES * STAGE + 1024 + 256 + 1024;     // tiles, alignment slack, barriers, row norms
};

struct RtP {
    const float* br;
    const float* rstat;       // {max column norm of Wr, max |br|}
    float* logits;            // [N,E] or null
    float* probs;             // [N,E]
    int32_t* top_idx;         // [N,k]
    float* top_p;             // [N,k]
    int32_t* list;            // tokens for the exact pass
    int32_t* list_count;
    int32_t* status;
    int N, C, E, k, n_tiles, kblocks;
};

template <int NE>
__global__ void __launch_bounds__(RT_THREADS, 1)
tc_router_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const RtP p)
{
    using Cfg = RtCfg<NE>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((int)blockIdx.x >= p.n_tiles) return;

    const uint32_t base = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (base & 1023u)) & 1023u;
    uint8_t* tiles = smem_raw + pad;
    const uint32_t bars = smem_u32(tiles + STAGES * Cfg::STAGE);
    auto full = [&](int s) { return bars + 8u * s; };
    auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
    auto norm_full = [&](int b) { return bars + 8u * (2 * STAGES + 5 + b); };
    float* norm_s = reinterpret_cast<float*>(tiles + STAGES * Cfg::STAGE + 256);      // [2][128]: sum of squares per row

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1 + 4);          // the MMA's commit and the four warps that read the rows
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
            mbar_init(norm_full(b), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, RT_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x) {
                bool ok = true;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= (uint32_t)STAGES &&
                        !mbar_wait(empty(s), ((it / STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_u32(tiles + s * Cfg::STAGE);
                    mbar_expect_tx(full(s), Cfg::STAGE);
                    tma_load_2d(a_dst, &tmX, kb * RT_BK, tile * RT_BM, full(s));
                    tma_load_2d(a_dst + RT_A_BYTES, &tmW, kb * RT_BK, 0, full(s));     // rows 0..NE-1 hi, NE..2NE-1 mid
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(RT_BM, NE, 0, 0);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x, ++t) {
                const uint32_t buf = t & 1u;
                if (t >= 2 && !mbar_wait(acc_empty(buf), ((t >> 1) - 1) & 1, p.status, ERR_ACC_WAIT)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 128;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full(s), (it / STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * Cfg::STAGE), b_addr = a_addr + RT_A_BYTES;
#pragma unroll
                    for (int k = 0; k < RT_BK / 16; ++k) {
                        const uint64_t ad = make_desc(a_addr + k * 32, 16, 1024);
                        umma_bf16(d_tmem, ad, make_desc(b_addr + k * 32, 16, 1024), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        umma_bf16(d_tmem, ad, make_desc(b_addr + NE * 128 + k * 32, 16, 1024), idesc, 1u);
                    }
                    umma_commit(empty(s));
                }
                if (ok) umma_commit(acc_full(buf));
            }
        }
    } else if (warp < 6) {
        // Row norms: ||x_row||^2 from the tiles the tensor core reads (16-byte pieces of a row are permuted by the
        // 128-byte swizzle, which a sum of squares does not mind; lane l starts at piece l so a quarter warp covers all
        // banks).  Warps of their own: the epilogue of a tile takes about as long as the loads of the next one, and
        // while these warps did both, no stage was released during an epilogue and the ring stood still.
        const int row = (warp & 3) * 32 + lane;
        uint32_t it = 0, t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u;
            float ss4[4] = {0.0f, 0.0f, 0.0f, 0.0f};          // independent chains: one warp per scheduler hides no latency
            for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(full(s), (it / STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                    ok = false;
                    break;
                }
                const uint32_t rbase = smem_u32(tiles + s * Cfg::STAGE) + row * 128;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t w0, w1, w2, w3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(rbase + (((uint32_t)(i + lane) & 7u) << 4)));
                    const uint32_t ws4[4] = {w0, w1, w2, w3};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float lo = __uint_as_float(ws4[j] << 16), hi = __uint_as_float(ws4[j] & 0xffff0000u);
                        ss4[j] = fmaf(lo, lo, ss4[j]);
                        ss4[j] = fmaf(hi, hi, ss4[j]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty(s));
            }
            if (!ok) break;
            // the epilogue has read this buffer's norms of two tiles ago (it arrives on acc_empty after reading them)
            if (t >= 2 && !mbar_wait(acc_empty(buf), ((t >> 1) - 1) & 1, p.status, ERR_ACC_WAIT)) break;
            norm_s[buf * 128 + row] = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(norm_full(buf));
        }
    } else {
        const int q = warp & 3;                   // TMEM lane quarter of this warp
        const int row = q * 32 + lane;
        const float wmax = p.rstat[0], bmax = p.rstat[1];
        uint32_t t = 0;
        for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++t) {
            const uint32_t buf = t & 1u;
            if (!mbar_wait(acc_full(buf), (t >> 1) & 1, p.status, ERR_ACC_WAIT)) break;
            if (!mbar_wait(norm_full(buf), (t >> 1) & 1, p.status, ERR_ACC_WAIT)) break;
            tc_fence_after();
            const float ss = norm_s[buf * 128 + row];
            const uint32_t t_lane = tmem_base + buf * 128 + ((uint32_t)(q * 32) << 16);
            constexpr int NLD = NE < 32 ? 1 : NE / 32;
            float lg[NLD * 32];
#pragma unroll
            for (int i = 0; i < NLD; ++i) {
                float v[32];
                tmem_ld32(t_lane + i * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) lg[i * 32 + j] = v[j];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));

            const int tok = tile * RT_BM + row;
            const int E = p.E, k = p.k;
            const bool live = tok < p.N;
            // error bound of this token's logits against the reference's, and the margin that makes an order final
            const float u = 5.9604645e-8f;
            const float xn = sqrtf(ss) * 1.001f;
            const float bound = (1.5f * (float)p.C * u + 1.52587890625e-5f) * xn * wmax * 1.01f + 4.0f * u * (xn * wmax + bmax);
            const float tau = 2.0f * bound;

            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < NE; ++j) {
                lg[j] = j < E ? lg[j] + __ldg(p.br + (j < E ? j : 0)) : -INFINITY;
                mx = fmaxf(mx, lg[j]);
            }
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < NE; ++j)
                if (j < E) sum += __expf(lg[j] - mx);
            const float inv = 1.0f / fmaxf(sum, 1e-15f);
            if (live) {
                float* prow = p.probs + (size_t)tok * E;
                float* lrow = p.logits ? p.logits + (size_t)tok * E : nullptr;
                if ((E & 3) == 0) {
#pragma unroll
                    for (int j = 0; j < NE; j += 4) {
                        if (j < E) {
                            float4 pv;
                            pv.x = fminf(fmaxf(__expf(lg[j] - mx) * inv, 1e-7f), 1.0f);
                            pv.y = fminf(fmaxf(__expf(lg[j + 1] - mx) * inv, 1e-7f), 1.0f);
                            pv.z = fminf(fmaxf(__expf(lg[j + 2] - mx) * inv, 1e-7f), 1.0f);
                            pv.w = fminf(fmaxf(__expf(lg[j + 3] - mx) * inv, 1e-7f), 1.0f);
                            *reinterpret_cast<float4*>(prow + j) = pv;
                            if (lrow) *reinterpret_cast<float4*>(lrow + j) = make_float4(lg[j], lg[j + 1], lg[j + 2], lg[j + 3]);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NE; ++j) {
                        if (j < E) {
                            prow[j] = fminf(fmaxf(__expf(lg[j] - mx) * inv, 1e-7f), 1.0f);
                            if (lrow) lrow[j] = lg[j];
                        }
                    }
                }
            }
            // top-(k+1) by logit, lowest index first on equal values (the reference's strict '>')
            const int nsel = k + 1 < E ? k + 1 : E;
            bool unsure = false;
            float prev = 0.0f, pk = 0.0f;
#pragma unroll
            for (int r = 0; r < MAX_TOPK + 1; ++r) {
                if (r < nsel) {
                    float best = -INFINITY;
                    int bi = -1;
#pragma unroll
                    for (int j = 0; j < NE; ++j)
                        if (lg[j] > best) {
                            best = lg[j];
                            bi = j;
                        }
#pragma unroll
                    for (int j = 0; j < NE; ++j)
                        if (j == bi) lg[j] = -INFINITY;
                    if (bi < 0) unsure = true;
                    if (r > 0 && !(prev - best > tau)) unsure = true;
                    prev = best;
                    if (r < k) {
                        pk = fminf(fmaxf(__expf(best - mx) * inv, 1e-7f), 1.0f);
                        if (live) {
                            p.top_idx[(size_t)tok * k + r] = bi < 0 ? 0 : bi;
                            p.top_p[(size_t)tok * k + r] = pk;
                        }
                    }
                }
            }
            if (!(pk > 4e-7f)) unsure = true;          // the k-th probability must be clear of the clamp floor
            unsure = unsure && live;
            const unsigned m = __ballot_sync(0xffffffffu, unsure);
            if (m) {
                int slot0 = 0;
                if (lane == 0) slot0 = atomicAdd(p.list_count, __popc(m));
                slot0 = __shfl_sync(0xffffffffu, slot0, 0);
                if (unsure) p.list[slot0 + __popc(m & ((1u << lane) - 1u))] = tok;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, RT_TMEM_COLS);
    }
}

// Wr [C,E] fp32 -> transposed BF16 pieces [2][NE][C] (hi = bf16(w), mid = bf16(w - hi)) and the largest column
// norm / bias magnitude, for the error bound.  One block per expert row of the output.
__global__ void __launch_bounds__(256)
router_pieces_kernel(const float* __restrict__ Wr, const float* __restrict__ br, int C, int E, int NE,
                     bf16* __restrict__ out, float* __restrict__ rstat)
{
    __shared__ float red[8];
    const int e = blockIdx.x;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float w = Wr[(size_t)c * E + e];
        const bf16 hi = __float2bfloat16(w);
        const bf16 mid = __float2bfloat16(w - __bfloat162float(hi));
        out[(size_t)e * C + c] = hi;
        out[((size_t)NE + e) * C + c] = mid;
        ss = fmaf(w, w, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; ++i) t += red[i];
        // non-negative floats order like their bit patterns; a NaN (bits above +inf) stays the maximum, so a
        // poisoned weight makes every token take the exact pass
        atomicMax(reinterpret_cast<int*>(rstat), __float_as_int(sqrtf(t) * 1.001f));
        atomicMax(reinterpret_cast<int*>(rstat) + 1, __float_as_int(fabsf(br[e])));
    }
}

int router_ne(int E) { return E <= 16 ? 16 : E <= 32 ? 32 : E <= 64 ? 64 : 128; }

template <int NE>
int launch_rt(const CUtensorMap& mx, const CUtensorMap& mw, const RtP& p, int grid, cudaStream_t st, bool* attr_done)
{
    if (!*attr_done) {
        MGPT_CUDA(cudaFuncSetAttribute(tc_router_fwd_kernel<NE>, cudaFuncAttributeMaxDynamicSharedMemorySize, RtCfg<NE>::SMEM));
        *attr_done = true;
    }
    tc_router_fwd_kernel<NE><<<grid, RT_THREADS, RtCfg<NE>::SMEM, st>>>(mx, mw, p);
    MGPT_LAUNCHED("tc_router_fwd_kernel");
    return 0;
}

}  // namespace

// Rebuilds the router's transposed BF16 pieces and the norms of the error bound (after the masters changed).
int launch_router_pieces(mgpt_moe_layer* L, cudaStream_t st)
{
    const Dims& d = L->d;
    if (!L->sWrT2 || !L->router_bound) return 0;
    MGPT_CUDA(cudaMemsetAsync(L->d_rstat, 0, 2 * sizeof(float), st));
    router_pieces_kernel<<<d.E, 256, 0, st>>>(L->p_data[0], L->p_data[1], d.C, d.E, L->router_ne, L->sWrT2, L->d_rstat);
    MGPT_LAUNCHED("router_pieces_kernel");
    return 0;
}

// The two-pass router pays off once the exact kernel's 2*N*C*E multiply-adds take longer than two launches and a
// first pass over x: below ~4e8 of them (config 2: 6.7e7; decode batches) the exact kernel alone is faster.
bool tc_router_usable(const mgpt_moe_layer* L, const void* x, int io, int n_tokens)
{
    return L->d.mode == MGPT_MOE_BF16 && L->d.gemm_impl == 0 && io == MGPT_MOE_IO_BF16 && L->sWrT2 != nullptr &&
           ((uintptr_t)x & 15) == 0 && (double)n_tokens * L->d.C * L->d.E >= L->router_tc_min_work;
}

int tc_router_fwd(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, cudaStream_t st)
{
    const Dims& d = L->d;
    const int N = w.n_tokens, NE = L->router_ne;
    if (N <= 0) return 0;
    CUtensorMap mx, mw;
    MGPT_TRY(make_map_kind(&mx, x, (uint64_t)N, (uint64_t)d.C, RT_BM, false));
    MGPT_TRY(make_map_kind(&mw, L->sWrT2, (uint64_t)2 * NE, (uint64_t)d.C, 2 * NE, false));
    RtP p;
    p.br = L->p_data[1];
    p.rstat = L->d_rstat;
    p.logits = (float*)(ws + w.logits);
    p.probs = (float*)(ws + w.probs);
    p.top_idx = (int32_t*)(ws + w.top_idx);
    p.top_p = (float*)(ws + w.top_p);
    p.list = (int32_t*)(ws + w.rt_list);
    p.list_count = (int32_t*)(ws + w.rt_count);
    p.status = L->d_status;
    p.N = N; p.C = d.C; p.E = d.E; p.k = d.k;
    p.n_tiles = (N + RT_BM - 1) / RT_BM;
    p.kblocks = (d.C + RT_BK - 1) / RT_BK;
    int sms = 0;
    MGPT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, L->device));
    const int grid = p.n_tiles < sms ? p.n_tiles : sms;
    MGPT_CUDA(cudaMemsetAsync(p.list_count, 0, sizeof(int32_t), st));
    switch (NE) {
        case 16: MGPT_TRY(launch_rt<16>(mx, mw, p, grid, st, &L->router_tc_attr)); break;
        case 32: MGPT_TRY(launch_rt<32>(mx, mw, p, grid, st, &L->router_tc_attr)); break;
        case 64: MGPT_TRY(launch_rt<64>(mx, mw, p, grid, st, &L->router_tc_attr)); break;
        default: MGPT_TRY(launch_rt<128>(mx, mw, p, grid, st, &L->router_tc_attr)); break;
    }
    // exact pass over the listed tokens (how many is known only on the device: CTAs beyond the list leave at once)
    return launch_router_fwd(x, MGPT_MOE_IO_BF16, L->p_data[0], L->p_data[1], N, d.C, d.E, d.k, p.logits, p.probs,
                             p.top_idx, p.top_p, st, p.list, p.list_count);
}

int router_tc_ne(int E) { return router_ne(E); }

}  // namespace mgpt
