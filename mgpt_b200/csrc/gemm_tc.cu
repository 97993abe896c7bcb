// Grouped SwiGLU expert products on the 5th-generation tensor cores.
//
// BF16 operands, FP32 accumulation in TMEM (tcgen05.mma, one issuing thread
// per CTA), operand tiles staged in shared memory by TMA (cp.async.bulk.tensor,
// 128-byte swizzle), epilogues read the accumulator with tcgen05.ld.  No
// cluster multicast is used anywhere: every CTA loads its own tiles.
//
// What the reference does with ~8 launches per expert forward and ~26 per
// expert backward (layers/MoELayer.cpp:94-118, 159-181; layers/SwiGLU.cpp:23-96;
// layers/LinearLayer.cpp:23-80) becomes seven launches for all experts:
//
//   gate/up : [G|U] = Xg * [Wg|Wu] + [bg|bu],  Hh = silu(G)*U      (epilogue)
//   down    : Yg = Hh * Wd + bd
//   dHh     : dHh = dYg * Wd^T -> dG, dU (SwiGLU backward in the epilogue)
//   dXg     : dXg = dG * Wg^T + dU * Wu^T       (one accumulator, K = 2H)
//   wgrad x3: gWg += Xg^T dG, gWu += Xg^T dU, gWd += Hh^T dYg   (FP32 +=)
//
// Row tiles are whole 128-row tiles of one expert (the dispatch plan pads each
// expert's segment with zero rows), so no tile mixes experts and the reduction
// over rows in the weight gradients needs no masking.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets a bit in the
// workspace status word and the CTA leaves through its normal teardown
// (TMEM is released), so a fault in a descriptor cannot hang the device.
#include <cuda.h>

#include "common.cuh"

namespace mgpt {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr uint32_t A_BYTES = BM * BK * 2;            // 16 KiB
constexpr uint32_t B_BYTES = BN * BK * 2;            // 32 KiB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KiB
constexpr uint32_t HALF_B = B_BYTES / 2;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int TC_THREADS = 192;                      // warp0 TMA, warp1 MMA, warps2-5 epilogue

enum { ERR_FULL_WAIT = 2, ERR_EMPTY_WAIT = 4, ERR_ACC_WAIT = 8 };

// ---- PTX wrappers ------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and records why) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t* status, int code)
{
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try(bar, parity)) return true;
    atomicOr(status, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum)
{
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
// mbarrier arrives once every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread = TMEM lane (row), v[j] = column j
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version bits.
//   K-major  operand: rows of 64 bf16 (128 B), 8-row groups SBO apart (LBO unused)
//   MN-major operand: 64 contiguous MN elements per k, 8-k groups SBO apart,
//                     next 64 MN elements LBO apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;            // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D=F32, A=B=BF16, dense, M x N, operand majors.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_mn_major, int b_mn_major)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

// 32 floats -> 32 bf16, written as up to four 16-byte stores; `valid` columns (multiple of 8) are kept
__device__ __forceinline__ void store_bf16x32(bf16* dst, const float (&v)[32], int valid)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q * 8 < valid) {
            uint4 u;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
            u.x = *reinterpret_cast<uint32_t*>(&h0);
            u.y = *reinterpret_cast<uint32_t*>(&h1);
            u.z = *reinterpret_cast<uint32_t*>(&h2);
            u.w = *reinterpret_cast<uint32_t*>(&h3);
            reinterpret_cast<uint4*>(dst)[q] = u;
        }
    }
}
__device__ __forceinline__ void load_bf16x32(const bf16* src, float (&v)[32], int valid)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q * 8 < valid) {
            const uint4 u = reinterpret_cast<const uint4*>(src)[q];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
                v[q * 8 + 2 * i] = __low2float(h);
                v[q * 8 + 2 * i + 1] = __high2float(h);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[q * 8 + i] = 0.0f;
        }
    }
}

struct Pipe {
    uint32_t bars, acc, tmem_slot;     // shared-space addresses
    uint8_t* tiles;
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8u * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8u * (STAGES + s); }
};

// Carves dynamic shared memory: 1024-aligned tile ring, then the barriers.
__device__ __forceinline__ Pipe carve(uint8_t* raw)
{
    Pipe p;
    const uint32_t base = smem_u32(raw);
    const uint32_t pad = (1024u - (base & 1023u)) & 1023u;
    p.tiles = raw + pad;
    p.bars = smem_u32(p.tiles + STAGES * STAGE_BYTES);
    p.acc = p.bars + 8u * (2 * STAGES);
    p.tmem_slot = p.acc + 8u;
    return p;
}

// ---- token-major products ------------------------------------------------------
enum { MODE_GATEUP = 0, MODE_DOWN = 1, MODE_DHH = 2, MODE_DXG = 3 };

struct RowsP {
    const int32_t* tile_expert;
    const int32_t* n_tiles;
    int32_t* status;
    int kblocks;            // k-blocks (of 64) per operand pair
    int n_out;              // output columns (H or C)
    int b_rows_per_expert;  // rows of one expert in the B tensor map (= n_out)
    bf16 *D0, *D1, *D2;     // outputs, row stride n_out
    const bf16 *G, *U;      // saved pre-activations (MODE_DHH)
    const float* const* bias0;
    const float* const* bias1;
};

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_rows_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1, const RowsP p)
{
    extern __shared__ uint8_t smem_raw[];
    const int row_tile = blockIdx.y;
    if (row_tile >= *p.n_tiles) return;                 // whole CTA leaves before any barrier or TMEM use
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = p.tile_expert[row_tile];
    // GATEUP: 128 hidden units per CTA (128 gate + 128 up accumulator columns); others: 256 columns
    const int n0 = blockIdx.x * (MODE == MODE_GATEUP ? BN / 2 : BN);
    const int row0 = row_tile * BM;
    const int total_kb = (MODE == MODE_DXG ? 2 : 1) * p.kblocks;

    Pipe pipe = carve(smem_raw);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(pipe.full(s), 1);
            mbar_init(pipe.empty(s), 1);
        }
        mbar_init(pipe.acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(pipe.tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(pipe.tmem_slot));

    if (warp == 0) {
        if (lane == 0) {
            const int brow = e * p.b_rows_per_expert + n0;
            for (int kb = 0; kb < total_kb; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(pipe.empty(s), ((kb / STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT)) break;
                const uint32_t a_dst = smem_u32(pipe.tiles + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                mbar_expect_tx(pipe.full(s), STAGE_BYTES);
                const bool second = MODE == MODE_DXG && kb >= p.kblocks;
                const int kx = (second ? kb - p.kblocks : kb) * BK;
                tma_load_2d(a_dst, second ? &tmA1 : &tmA0, kx, row0, pipe.full(s));
                if (MODE == MODE_GATEUP) {
                    tma_load_2d(b_dst, &tmB0, kx, brow, pipe.full(s));
                    tma_load_2d(b_dst + HALF_B, &tmB1, kx, brow, pipe.full(s));
                } else {
                    const CUtensorMap* mb = second ? &tmB1 : &tmB0;
                    tma_load_2d(b_dst, mb, kx, brow, pipe.full(s));
                    tma_load_2d(b_dst + HALF_B, mb, kx, brow + BN / 2, pipe.full(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0);
            bool ok = true;
            for (int kb = 0; kb < total_kb && ok; ++kb) {
                const int s = kb % STAGES;
                ok = mbar_wait(pipe.full(s), (kb / STAGES) & 1, p.status, ERR_FULL_WAIT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(pipe.tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    const uint64_t ad = make_desc(a_addr + k * 32, 16, 1024);
                    const uint64_t bd = make_desc(b_addr + k * 32, 16, 1024);
                    umma_bf16(tmem_base, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(pipe.empty(s));            // frees the stage once these MMAs have read it
            }
            umma_commit(pipe.acc);                      // accumulator complete (arrives even after a failed wait)
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32*(warp%4) .. +31  (row = lane)
        const int quarter = warp & 3;
        const int row = row0 + quarter * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool ok = mbar_wait(pipe.acc, 0, p.status, ERR_ACC_WAIT);
        tc_fence_after();
        if (ok) {
            if (MODE == MODE_GATEUP) {
                const float* bg = p.bias0[e];
                const float* bu = p.bias1[e];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    const int n = n0 + c * 32;
                    const int valid = min(32, p.n_out - n);
                    if (valid <= 0) break;
                    float g[32], u[32];
                    tmem_ld32(t_lane + c * 32, g);
                    tmem_ld32(t_lane + BN / 2 + c * 32, u);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < valid) {
                            // round the stored pre-activations first: backward reads them back
                            g[j] = __bfloat162float(__float2bfloat16(g[j] + bg[n + j]));
                            u[j] = __bfloat162float(__float2bfloat16(u[j] + bu[n + j]));
                        }
                    }
                    const size_t o = (size_t)row * p.n_out + n;
                    store_bf16x32(p.D0 + o, g, valid);
                    store_bf16x32(p.D1 + o, u, valid);
#pragma unroll
                    for (int j = 0; j < 32; ++j) g[j] = silu(g[j]) * u[j];
                    store_bf16x32(p.D2 + o, g, valid);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int n = n0 + c * 32;
                    const int valid = min(32, p.n_out - n);
                    if (valid <= 0) break;
                    float v[32];
                    tmem_ld32(t_lane + c * 32, v);
                    const size_t o = (size_t)row * p.n_out + n;
                    if (MODE == MODE_DOWN) {
                        const float* b = p.bias0[e];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < valid) v[j] += b[n + j];
                        store_bf16x32(p.D0 + o, v, valid);
                    } else if (MODE == MODE_DHH) {
                        // utils/Tensor.cpp:2020-2027 with dd = dHh
                        float g[32], u[32];
                        load_bf16x32(p.G + o, g, valid);
                        load_bf16x32(p.U + o, u, valid);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float sig = 1.0f / (1.0f + __expf(-g[j]));
                            const float dd = v[j];
                            v[j] = (dd * u[j]) * (sig * (1.0f + g[j] * (1.0f - sig)));   // dG
                            u[j] = dd * (g[j] * sig);                                     // dU
                        }
                        store_bf16x32(p.D0 + o, v, valid);
                        store_bf16x32(p.D1 + o, u, valid);
                    } else {
                        store_bf16x32(p.D0 + o, v, valid);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, BN);
    }
}

// ---- weight gradients: grad[e][M,N] += A_e^T * B_e over the expert's rows ---------
struct WgradP {
    const int32_t* padded_offsets;
    int32_t* status;
    float* const* grad;
    int M, N, n_tiles_n;
};

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_wgrad_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const WgradP p)
{
    extern __shared__ uint8_t smem_raw[];
    const int e = blockIdx.y;
    const int r0 = p.padded_offsets[e], r1 = p.padded_offsets[e + 1];
    const int total_kb = (r1 - r0) / BK;
    if (total_kb <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = (blockIdx.x / p.n_tiles_n) * BM, n0 = (blockIdx.x % p.n_tiles_n) * BN;

    Pipe pipe = carve(smem_raw);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(pipe.full(s), 1);
            mbar_init(pipe.empty(s), 1);
        }
        mbar_init(pipe.acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(pipe.tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(pipe.tmem_slot));

    constexpr uint32_t BOX = 64 * BK * 2;      // one {64 MN elements, 64 rows} box = 8 KiB
    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < total_kb; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(pipe.empty(s), ((kb / STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT)) break;
                const uint32_t a_dst = smem_u32(pipe.tiles + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                mbar_expect_tx(pipe.full(s), STAGE_BYTES);
                const int r = r0 + kb * BK;
#pragma unroll
                for (int i = 0; i < BM / 64; ++i) tma_load_2d(a_dst + i * BOX, &tmA, m0 + 64 * i, r, pipe.full(s));
#pragma unroll
                for (int i = 0; i < BN / 64; ++i) tma_load_2d(b_dst + i * BOX, &tmB, n0 + 64 * i, r, pipe.full(s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);
            for (int kb = 0; kb < total_kb; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(pipe.full(s), (kb / STAGES) & 1, p.status, ERR_FULL_WAIT)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(pipe.tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) {
                    // 16 reduction rows = two 8-row groups (1 KiB each); 64-element MN blocks are BOX apart
                    const uint64_t ad = make_desc(a_addr + k * 2048, BOX, 1024);
                    const uint64_t bd = make_desc(b_addr + k * 2048, BOX, 1024);
                    umma_bf16(tmem_base, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(pipe.empty(s));
            }
            umma_commit(pipe.acc);
        }
    } else {
        const int quarter = warp & 3;
        const int m = m0 + quarter * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const bool ok = mbar_wait(pipe.acc, 0, p.status, ERR_ACC_WAIT);
        tc_fence_after();
        if (ok) {
            float* g = p.grad[e];
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int n = n0 + c * 32;
                const int valid = min(32, p.N - n);
                if (valid <= 0) break;
                float v[32];
                tmem_ld32(t_lane + c * 32, v);             // warp-collective: every lane takes part
                if (m < p.M) {
                    float4* dst = reinterpret_cast<float4*>(g + (size_t)m * p.N + n);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (q * 4 < valid) {
                            float4 t = dst[q];
                            t.x += v[q * 4 + 0]; t.y += v[q * 4 + 1]; t.z += v[q * 4 + 2]; t.w += v[q * 4 + 3];
                            dst[q] = t;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, BN);
    }
}

// ---- host side: tensor maps ------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D row-major bf16 tensor [rows, cols]; box = {64 columns (128 B), box_rows}; 128-byte swizzle; OOB reads 0.
int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MGPT_MOE_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * sizeof(bf16)};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MGPT_MOE_ECUDA, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
    return 0;
}

struct TcState {
    const void* ws = nullptr;
    int n_tokens = -1;
    bool attr_set = false;
    // K-major (box 64 x 128 rows)
    CUtensorMap Xg, Hh, dYg, dG, dU, WgT, WuT, WdT, Wg, Wu, Wd;
    // reduction-over-rows operands (box 64 x 64 rows)
    CUtensorMap Xg_t, Hh_t, dYg_t, dG_t, dU_t;
};

int prepare(mgpt_moe_layer* L, const Workspace& w, char* ws)
{
    if (!L->tc_state) L->tc_state = new TcState();
    TcState* s = (TcState*)L->tc_state;
    if (!s->attr_set) {
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DHH>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DXG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        s->attr_set = true;
    }
    if (s->ws == ws && s->n_tokens == w.n_tokens) return 0;
    const Dims& d = L->d;
    const uint64_t rc = w.row_cap, C = d.C, H = d.H, E = d.E;
    MGPT_TRY(make_map(&s->Xg, ws + w.Xg, rc, C, 128));
    MGPT_TRY(make_map(&s->Hh, ws + w.Hh, rc, H, 128));
    MGPT_TRY(make_map(&s->dYg, ws + w.dYg, rc, C, 128));
    MGPT_TRY(make_map(&s->dG, ws + w.dG, rc, H, 128));
    MGPT_TRY(make_map(&s->dU, ws + w.dU, rc, H, 128));
    MGPT_TRY(make_map(&s->WgT, L->sWgT, E * H, C, 128));
    MGPT_TRY(make_map(&s->WuT, L->sWuT, E * H, C, 128));
    MGPT_TRY(make_map(&s->WdT, L->sWdT, E * C, H, 128));
    MGPT_TRY(make_map(&s->Wg, L->sWg, E * C, H, 128));
    MGPT_TRY(make_map(&s->Wu, L->sWu, E * C, H, 128));
    MGPT_TRY(make_map(&s->Wd, L->sWd, E * H, C, 128));
    MGPT_TRY(make_map(&s->Xg_t, ws + w.Xg, rc, C, 64));
    MGPT_TRY(make_map(&s->Hh_t, ws + w.Hh, rc, H, 64));
    MGPT_TRY(make_map(&s->dYg_t, ws + w.dYg, rc, C, 64));
    MGPT_TRY(make_map(&s->dG_t, ws + w.dG, rc, H, 64));
    MGPT_TRY(make_map(&s->dU_t, ws + w.dU, rc, H, 64));
    s->ws = ws;
    s->n_tokens = w.n_tokens;
    return 0;
}

int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace

int tc_experts_forward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    MGPT_TRY(prepare(L, w, ws));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    RowsP p = {};
    p.tile_expert = (const int32_t*)(ws + w.tile_expert);
    p.n_tiles = (const int32_t*)(ws + w.n_tiles);
    p.status = (int32_t*)(ws + w.status);
    // gate/up + SwiGLU: K = C, 128 hidden units per CTA
    p.kblocks = cdiv(d.C, BK); p.n_out = d.H; p.b_rows_per_expert = d.H;
    p.D0 = (bf16*)(ws + w.G); p.D1 = (bf16*)(ws + w.U); p.D2 = (bf16*)(ws + w.Hh);
    p.bias0 = L->master.bg; p.bias1 = L->master.bu;
    L->stage_begin(ST_GATEUP, st);
    tc_rows_kernel<MODE_GATEUP><<<dim3(cdiv(d.H, BN / 2), w.max_tiles), TC_THREADS, SMEM_BYTES, st>>>(
        s->Xg, s->Xg, s->WgT, s->WuT, p);
    MGPT_LAUNCHED("tc_rows_kernel<gateup>");
    L->stage_end(ST_GATEUP, st);
    // down: K = H
    p.kblocks = cdiv(d.H, BK); p.n_out = d.C; p.b_rows_per_expert = d.C;
    p.D0 = (bf16*)(ws + w.Yg); p.D1 = p.D2 = nullptr; p.bias0 = L->master.bd; p.bias1 = nullptr;
    L->stage_begin(ST_DOWN, st);
    tc_rows_kernel<MODE_DOWN><<<dim3(cdiv(d.C, BN), w.max_tiles), TC_THREADS, SMEM_BYTES, st>>>(
        s->Hh, s->Hh, s->WdT, s->WdT, p);
    MGPT_LAUNCHED("tc_rows_kernel<down>");
    L->stage_end(ST_DOWN, st);
    return 0;
}

int tc_experts_backward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    MGPT_TRY(prepare(L, w, ws));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    RowsP p = {};
    p.tile_expert = (const int32_t*)(ws + w.tile_expert);
    p.n_tiles = (const int32_t*)(ws + w.n_tiles);
    p.status = (int32_t*)(ws + w.status);
    // dHh = dYg * Wd^T  (K = C), SwiGLU backward in the epilogue
    p.kblocks = cdiv(d.C, BK); p.n_out = d.H; p.b_rows_per_expert = d.H;
    p.D0 = (bf16*)(ws + w.dG); p.D1 = (bf16*)(ws + w.dU);
    p.G = (const bf16*)(ws + w.G); p.U = (const bf16*)(ws + w.U);
    L->stage_begin(ST_DHH, st);
    tc_rows_kernel<MODE_DHH><<<dim3(cdiv(d.H, BN), w.max_tiles), TC_THREADS, SMEM_BYTES, st>>>(
        s->dYg, s->dYg, s->Wd, s->Wd, p);
    MGPT_LAUNCHED("tc_rows_kernel<dhh>");
    L->stage_end(ST_DHH, st);
    // dXg = dG * Wg^T + dU * Wu^T  (K = 2H)
    p.kblocks = cdiv(d.H, BK); p.n_out = d.C; p.b_rows_per_expert = d.C;
    p.D0 = (bf16*)(ws + w.dXg); p.D1 = nullptr;
    L->stage_begin(ST_DXG, st);
    tc_rows_kernel<MODE_DXG><<<dim3(cdiv(d.C, BN), w.max_tiles), TC_THREADS, SMEM_BYTES, st>>>(
        s->dG, s->dU, s->Wg, s->Wu, p);
    MGPT_LAUNCHED("tc_rows_kernel<dxg>");
    L->stage_end(ST_DXG, st);
    if (!L->has_grad) return 0;

    WgradP g = {};
    g.padded_offsets = (const int32_t*)(ws + w.padded_offsets);
    g.status = (int32_t*)(ws + w.status);
    L->stage_begin(ST_WGRAD, st);
    // gWg += Xg^T dG, gWu += Xg^T dU   [C,H]
    g.M = d.C; g.N = d.H; g.n_tiles_n = cdiv(d.H, BN);
    dim3 gCH(cdiv(d.C, BM) * g.n_tiles_n, d.E);
    g.grad = L->master.gWg;
    tc_wgrad_kernel<<<gCH, TC_THREADS, SMEM_BYTES, st>>>(s->Xg_t, s->dG_t, g);
    MGPT_LAUNCHED("tc_wgrad_kernel<Wg>");
    g.grad = L->master.gWu;
    tc_wgrad_kernel<<<gCH, TC_THREADS, SMEM_BYTES, st>>>(s->Xg_t, s->dU_t, g);
    MGPT_LAUNCHED("tc_wgrad_kernel<Wu>");
    // gWd += Hh^T dYg   [H,C]
    g.M = d.H; g.N = d.C; g.n_tiles_n = cdiv(d.C, BN);
    g.grad = L->master.gWd;
    tc_wgrad_kernel<<<dim3(cdiv(d.H, BM) * g.n_tiles_n, d.E), TC_THREADS, SMEM_BYTES, st>>>(s->Hh_t, s->dYg_t, g);
    MGPT_LAUNCHED("tc_wgrad_kernel<Wd>");
    L->stage_end(ST_WGRAD, st);
    return 0;
}

void tc_destroy(mgpt_moe_layer* L)
{
    delete (TcState*)L->tc_state;
    L->tc_state = nullptr;
}

}  // namespace mgpt
