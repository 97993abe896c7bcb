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
//   gate/up : [G|U] = Xg * [Wg|Wu] + [bg|bu],  Hh = silu(G)*U; keeps silu(G) and dHh/dG's factor (epilogue)
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
#include <cstdio>
#include <cstdlib>

#include "tc_common.cuh"

namespace mgpt {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr uint32_t A_BYTES = BM * BK * 2;            // 16 KiB
constexpr uint32_t B_BYTES = BN * BK * 2;            // 32 KiB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KiB
constexpr uint32_t HALF_B = B_BYTES / 2;
constexpr int EPI_WARPS = 16;                        // four per TMEM lane quarter
constexpr uint32_t STAGING_BYTES = 2048;             // per epilogue warp: 32 rows x 64 B
constexpr uint32_t TMEM_COLS = 2 * BN;               // two accumulators
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * STAGING_BYTES + 1024 /*align slack*/ + 512 /*barriers, work queue*/;
constexpr int TC_THREADS = 64 + 32 * EPI_WARPS;      // warp0 TMA, warp1 MMA, warps2-17 epilogue
constexpr int CS_WARPS = 2;                          // weight-gradient kernel only: warps 18-19 sum operand columns (bias gradients)
constexpr int WG_THREADS = TC_THREADS + 32 * CS_WARPS;

constexpr int SCHED_Q = 8;                           // queue entries: the producer runs up to ~4 items ahead of the slowest epilogue warp

using namespace tcx;

// v[j] += bias[n + j] for 32 consecutive columns; 16-byte loads when the whole piece is inside the row
__device__ __forceinline__ void add_bias32(float (&v)[32], const float* __restrict__ bias, int n, int n_out)
{
    if (n + 32 <= n_out) {
        const float4* b4 = reinterpret_cast<const float4*>(bias + n);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 b = __ldg(b4 + q);
            v[4 * q] += b.x; v[4 * q + 1] += b.y; v[4 * q + 2] += b.z; v[4 * q + 3] += b.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (n + j < n_out) v[j] += bias[n + j];
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

// Shared memory of one CTA: operand ring, one 4 KiB staging tile per epilogue warp, barriers.
struct Pipe {
    uint32_t bars, tmem_slot;          // shared-space addresses
    uint8_t* tiles;
    uint8_t* staging;
    __device__ __forceinline__ uint32_t full(int s) const { return bars + 8u * s; }
    __device__ __forceinline__ uint32_t empty(int s) const { return bars + 8u * (STAGES + s); }
    __device__ __forceinline__ uint32_t acc_full(int b) const { return bars + 8u * (2 * STAGES + b); }
    __device__ __forceinline__ uint32_t acc_empty(int b) const { return bars + 8u * (2 * STAGES + 2 + b); }
    // work-item queue: slot i is full once the producer has written item(i), empty once every consumer has read it
    __device__ __forceinline__ uint32_t sched_full(int i) const { return bars + 8u * (2 * STAGES + 5 + i); }
    __device__ __forceinline__ uint32_t sched_empty(int i) const { return bars + 8u * (2 * STAGES + 5 + SCHED_Q + i); }
    __device__ __forceinline__ uint32_t sched_item(int i) const { return bars + 8u * (2 * STAGES + 5 + 2 * SCHED_Q) + 4u * i; }
};

__device__ __forceinline__ Pipe carve(uint8_t* raw)
{
    Pipe p;
    const uint32_t base = smem_u32(raw);
    const uint32_t pad = (1024u - (base & 1023u)) & 1023u;
    p.tiles = raw + pad;
    p.staging = p.tiles + STAGES * STAGE_BYTES;
    p.bars = smem_u32(p.staging + EPI_WARPS * STAGING_BYTES);
    p.tmem_slot = p.bars + 8u * (2 * STAGES + 4);
    return p;
}

// Common prologue: barriers, TMEM (both accumulators), returns the TMEM base address.
// `extra`: warps besides the MMA thread that read every operand stage and every work item (and release both).
__device__ __forceinline__ uint32_t cta_setup(const Pipe& pipe, int warp, int extra = 0)
{
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(pipe.full(s), 1);
            mbar_init(pipe.empty(s), 1 + extra);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(pipe.acc_full(b), 1);
            mbar_init(pipe.acc_empty(b), EPI_WARPS);
        }
#pragma unroll
        for (int i = 0; i < SCHED_Q; ++i) {
            mbar_init(pipe.sched_full(i), 1);
            mbar_init(pipe.sched_empty(i), 1 + EPI_WARPS + extra);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(pipe.tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(pipe.tmem_slot));
    return tmem_base;
}

__device__ __forceinline__ void cta_teardown(uint32_t tmem_base, int warp)
{
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- work distribution ---------------------------------------------------------
// Items are handed out by a device-wide counter instead of a fixed stride, so a CTA that starts late (its SM
// was busy with another stream's kernel) or meets longer items simply takes fewer of them.  The producer thread
// fetches the CTA's n-th item and passes it to the MMA thread and the epilogue warps through a small queue in
// shared memory.  counter[0] = next item, counter[1] = CTAs that have finished; the last CTA to finish clears
// both, so the pair is ready for the next launch on the stream without a memset.
// The value returned by the counter is first looked at in sched_publish (item >= total: no work left, published
// as -1 so that the other roles stop at this entry too); between request and use lie an item's loads.
// A CTA's first item is its own index (no round trip before the first loads); the counter hands out the rest.
__device__ __forceinline__ int sched_fetch(int32_t* counter) { return (int)gridDim.x + atomicAdd(counter, 1); }
// Hands the CTA's n-th item to the other roles.  False: the wait for a free queue slot ran out.
__device__ __forceinline__ bool sched_publish(const Pipe& pipe, uint32_t n, int& item, int total, int32_t* status)
{
    const int slot = n % SCHED_Q;
    if (item >= total) item = -1;
    if (n >= SCHED_Q && !mbar_wait(pipe.sched_empty(slot), ((n / SCHED_Q) - 1) & 1, status, ERR_SCHED_WAIT)) return false;
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(pipe.sched_item(slot)), "r"(item) : "memory");
    mbar_arrive(pipe.sched_full(slot));
    return true;
}
// The caller reads with every thread that needs the item, then one thread per consumer calls sched_release.
__device__ __forceinline__ int sched_consume(const Pipe& pipe, uint32_t n, int32_t* status)
{
    const int slot = n % SCHED_Q;
    if (!mbar_wait(pipe.sched_full(slot), (n / SCHED_Q) & 1, status, ERR_SCHED_WAIT)) return -1;
    int item;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(item) : "r"(pipe.sched_item(slot)) : "memory");
    return item;
}
__device__ __forceinline__ void sched_release(const Pipe& pipe, uint32_t n) { mbar_arrive(pipe.sched_empty(n % SCHED_Q)); }
// Once per CTA of the grid, by the producer thread after its last fetch (also CTAs that leave without fetching).
// `n`: how many callers there are (every CTA of the grid, or every pair's leader)
__device__ __forceinline__ void sched_finish(int32_t* counter, int n = -1)
{
    __threadfence();
    if (atomicAdd(counter + 1, 1) == (n < 0 ? (int)gridDim.x : n) - 1) {
        counter[0] = 0;
        counter[1] = 0;
        __threadfence();
    }
}

// Epilogue warp -> accumulator buffer is free again (all its tcgen05.ld of this tile are done).
// bar: a barrier of this CTA, or -- remote -- the shared::cluster address of a barrier of the pair's leader CTA.
__device__ __forceinline__ void release_acc(uint32_t bar, int lane, bool remote = false)
{
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
        if (remote) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
        else mbar_arrive(bar);
    }
}

// Writes this thread's row of a [32 rows x 32 bf16] tile into the warp's staging tile in the
// 64-byte swizzle a TMA store with SWIZZLE_64B expects (16-byte chunk j of row r at j ^ ((r >> 1) & 3)).
__device__ __forceinline__ void stage_row_bf16(uint8_t* stage, int lane, const uint32_t (&packed)[16])
{
    // the previous TMA store out of this tile must have finished reading it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
    const uint32_t row = smem_u32(stage) + lane * 64;
    const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a = row + (((uint32_t)j ^ sw) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(packed[4 * j]), "r"(packed[4 * j + 1]),
                     "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3]) : "memory");
    }
}
// The staged tile -> global through TMA (columns beyond the tensor are clipped by the hardware).
__device__ __forceinline__ void flush_stage(uint8_t* stage, const CUtensorMap* map, int x, int y, int lane)
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(map, x, y, smem_u32(stage));
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}
__device__ __forceinline__ void pack32(const float (&a)[32], uint32_t (&out)[16])
{
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        out[i] = *reinterpret_cast<uint32_t*>(&h);
    }
}
// The two saved activation-derivative arrays (buffers "G" and "U") are private to the gate/up and dHh epilogues, so they are kept in the layout
// both epilogues touch with full-width accesses: [row tile][8-column chunk][128 rows][8 bf16].  A thread owns one
// row (its TMEM lane); the 32 lanes of a warp then read or write 512 contiguous bytes per instruction.
// `chunk0` points at this thread's row in the first chunk of its 32 columns; `valid` = columns left in the tensor.
__device__ __forceinline__ void load_blocked32(const uint4* chunk0, uint32_t (&w)[16], int valid)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 u = make_uint4(0, 0, 0, 0);
        if (q * 8 < valid) u = __ldg(chunk0 + q * BM);
        w[4 * q] = u.x; w[4 * q + 1] = u.y; w[4 * q + 2] = u.z; w[4 * q + 3] = u.w;
    }
}
__device__ __forceinline__ void store_blocked32(uint4* chunk0, const uint32_t (&w)[16], int valid)
{
#pragma unroll
    for (int q = 0; q < 4; ++q)
        if (q * 8 < valid) chunk0[q * BM] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}
// this thread's row in chunk n/8 of row tile `row_tile` (n_out columns, a multiple of 8)
__device__ __forceinline__ size_t blocked_index(int row_tile, int n_out, int n, int row_in_tile)
{
    return ((size_t)row_tile * (n_out >> 3) + (n >> 3)) * BM + row_in_tile;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// ---- token-major products ------------------------------------------------------
enum { MODE_GATEUP = 0, MODE_DOWN = 1, MODE_DHH = 2, MODE_DXG = 3, MODE_DX = 4 };

struct RowsP {
    const int32_t* tile_expert;
    const int32_t* tile_order;  // optional: i-th row tile to work on (expert-major order over scattered tiles)
    const int32_t* n_tiles;
    const int32_t* pairs;       // pair kernel: {first tile, second tile or -1} per pair, in processing order
    const int32_t* n_pairs;
    int32_t* status;
    int32_t* sched;         // {next item, finished CTAs}, both zero between launches
    int kblocks;            // k-blocks (of 64) per operand pair
    int n_out;              // output columns (H or C)
    int n_col_tiles;        // column tiles per row tile
    int b_rows_per_expert;  // rows of one expert in the B tensor map (= n_out)
    bf16 *G, *U;            // P and Q (see the gate/up epilogue) in the blocked layout (written by MODE_GATEUP, read by MODE_DHH)
    const float* const* bias0;
    const float* const* bias1;
    // MODE_DX only: row tiles are token tiles (no experts); the epilogue adds the expert rows of each token
    int fixed_tiles;            // number of 128-token tiles
    int n_valid_rows;           // tokens
    // MODE_GATEUP / MODE_DOWN: the B operand is a tile-major weight copy (common.cuh): its map is [blocks * 128 rows,
    // 64 columns]; block (expert e, row block rb, column block kb) starts at row ((e * b_row_blocks + rb) * b_kb + kb) * 128
    int b_row_blocks, b_kb;
    const bf16* gather_src;     // dXg rows [*, n_out]
    const int32_t* gather_pos;  // [tokens, gather_k] row of dXg for (token, j)
    int gather_k;
};

// The epilogue of one work item for one of the 16 epilogue warps: TMEM lane quarter q (rows q*32..+31 of the row
// tile), column group h.  acc_empty_bar is where "this warp has read the accumulator" is signalled: a barrier of
// this CTA, or (remote) of the leader CTA of a pair.  store = false: the tile is a stand-in (a pair's missing
// second tile): the accumulator is released and nothing is written.  False: a bounded wait ran out.
template <int MODE>
__device__ __forceinline__ bool rows_epilogue(const RowsP& p, uint32_t acc_full_bar, uint32_t acc_empty_bar, bool remote,
                                              uint32_t tmem_base, uint32_t buf, uint32_t t, int row_tile, int n0, int e,
                                              int q, int h, int lane, uint8_t* stage, const CUtensorMap* tmD0,
                                              const CUtensorMap* tmD1, const CUtensorMap* tmD2, bool store)
{
    const int row_w = row_tile * BM + q * 32;           // first row of this warp
    if (!store) {
        if (!mbar_wait(acc_full_bar, (t >> 1) & 1, p.status, ERR_ACC_WAIT)) return false;
        tc_fence_after();
        release_acc(acc_empty_bar, lane, remote);
        return true;
    }
    // MODE_DHH: the saved G and U of this item come from HBM.  Unit 0's pieces are requested before the wait
    // for the accumulator, unit 1's while unit 0 is worked on, so their latency hides behind other work.
    uint32_t gq[2][16], uq[2][16];
    if (MODE == MODE_DHH) {
        const int n = n0 + h * 64;
        const size_t o = blocked_index(row_tile, p.n_out, n, q * 32 + lane);
        load_blocked32(reinterpret_cast<const uint4*>(p.G) + o, gq[0], p.n_out - n);
        load_blocked32(reinterpret_cast<const uint4*>(p.U) + o, uq[0], p.n_out - n);
    }
    if (!mbar_wait(acc_full_bar, (t >> 1) & 1, p.status, ERR_ACC_WAIT)) return false;
    tc_fence_after();
    const uint32_t t_lane = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
    if (MODE == MODE_GATEUP) {
        // this warp: hidden units n0 + h*32 .. +31  (gate columns h*32.., up columns 128 + h*32..)
        const int n = n0 + h * 32;
        float a[32], b[32];
        tmem_ld32(t_lane + h * 32, a);
        tmem_ld32(t_lane + BN / 2 + h * 32, b);
        tmem_ld_wait();
        release_acc(acc_empty_bar, lane, remote);
        if (n < p.n_out) {
            // What backward needs of G and U is not the values themselves but
            //   Q = silu(G)                       (dU = dHh * Q)
            //   P = U * sigmoid(G) * (1 + G * (1 - sigmoid(G)))      (dG = dHh * P)
            // (utils/Tensor.cpp:2020-2027), so those are what is kept: the sigmoid is evaluated once, here,
            // in FP32 on the unrounded sums, and the dHh epilogue is left with two multiplies per element.
            uint32_t pp[16], qp[16], hp[16];
            add_bias32(a, p.bias0[e], n, p.n_out);
            add_bias32(b, p.bias1[e], n, p.n_out);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float pv[2], qv[2], hv[2];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const float g = a[2 * i + hh], u = b[2 * i + hh];
                    const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
                    const float q = g * sig;
                    qv[hh] = q;
                    hv[hh] = q * u;
                    pv[hh] = (u * sig) * (1.0f + (g - q));
                }
                __nv_bfloat162 p2 = __floats2bfloat162_rn(pv[0], pv[1]);
                __nv_bfloat162 q2 = __floats2bfloat162_rn(qv[0], qv[1]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(hv[0], hv[1]);
                pp[i] = *reinterpret_cast<uint32_t*>(&p2);
                qp[i] = *reinterpret_cast<uint32_t*>(&q2);
                hp[i] = *reinterpret_cast<uint32_t*>(&h2);
            }
            if (p.G) {                                  // inference keeps nothing for a backward pass
                const size_t o = blocked_index(row_tile, p.n_out, n, q * 32 + lane);
                store_blocked32(reinterpret_cast<uint4*>(p.G) + o, pp, p.n_out - n);
                store_blocked32(reinterpret_cast<uint4*>(p.U) + o, qp, p.n_out - n);
            }
            stage_row_bf16(stage, lane, hp);
            flush_stage(stage, tmD2, n, row_w, lane);
        }
    } else {
        // this warp: columns n0 + h*64 .. +63, two units of 32
#pragma unroll
        for (int un = 0; un < 2; ++un) {
            const int n = n0 + h * 64 + un * 32;
            float v[32];
            tmem_ld32(t_lane + h * 64 + un * 32, v);
            tmem_ld_wait();
            if (un == 1) release_acc(acc_empty_bar, lane, remote);
            if (n >= p.n_out) continue;                      // warp-uniform
            uint32_t pk[16];
            if (MODE == MODE_DOWN) {
                add_bias32(v, p.bias0[e], n, p.n_out);
            } else if (MODE == MODE_DHH) {
                // utils/Tensor.cpp:2020-2027 with dd = dHh: dG = dd * P, dU = dd * Q (P, Q saved by the forward epilogue)
                if (un == 0) {
                    const int n1 = n + 32;
                    const size_t o1 = blocked_index(row_tile, p.n_out, n1, q * 32 + lane);
                    load_blocked32(reinterpret_cast<const uint4*>(p.G) + o1, gq[1], p.n_out - n1);
                    load_blocked32(reinterpret_cast<const uint4*>(p.U) + o1, uq[1], p.n_out - n1);
                }
                uint32_t (&gw)[16] = gq[un];
                uint32_t (&uw)[16] = uq[un];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float d0 = v[2 * i], d1 = v[2 * i + 1];
                    __nv_bfloat162 a2 = __floats2bfloat162_rn(d0 * bf_lo(gw[i]), d1 * bf_hi(gw[i]));
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(d0 * bf_lo(uw[i]), d1 * bf_hi(uw[i]));
                    gw[i] = *reinterpret_cast<uint32_t*>(&a2);      // dG, packed in place
                    uw[i] = *reinterpret_cast<uint32_t*>(&b2);      // dU, packed in place
                }
                stage_row_bf16(stage, lane, uw);
                flush_stage(stage, tmD1, n, row_w, lane);
                stage_row_bf16(stage, lane, gw);
                flush_stage(stage, tmD0, n, row_w, lane);
                continue;
            } else if (MODE == MODE_DX) {
                // dx = (sum of the token's expert rows, ascending row order) + dlogits * Wr^T
                const int tok = row_w + lane;
                if (tok < p.n_valid_rows) {
                    int ps[MAX_TOPK];
#pragma unroll
                    for (int j = 0; j < MAX_TOPK; ++j)
                        ps[j] = j < p.gather_k ? p.gather_pos[(size_t)tok * p.gather_k + j] : 0x7fffffff;
#pragma unroll
                    for (int a = 0; a < MAX_TOPK - 1; ++a)
#pragma unroll
                        for (int b = 0; b < MAX_TOPK - 1 - a; ++b)
                            if (ps[b] > ps[b + 1]) {
                                const int tmp = ps[b];
                                ps[b] = ps[b + 1];
                                ps[b + 1] = tmp;
                            }
                    const int valid = min(32, p.n_out - n);
#pragma unroll
                    for (int j = 0; j < MAX_TOPK; ++j) {
                        if (j < p.gather_k) {
                            float g[32];
                            load_bf16x32(p.gather_src + (size_t)ps[j] * p.n_out + n, g, valid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += g[i];
                        }
                    }
                }
            }
            pack32(v, pk);
            stage_row_bf16(stage, lane, pk);
            flush_stage(stage, tmD0, n, row_w, lane);
        }
    }
    return true;
}

// Persistent: CTA b works on items b, b+grid, ... where item = row_tile * n_col_tiles + col_tile.
// Two 256-column accumulators in TMEM alternate, so the epilogue of one item runs while the
// tensor core works on the next.
template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_rows_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
               const __grid_constant__ CUtensorMap tmD0, const __grid_constant__ CUtensorMap tmD1,
               const __grid_constant__ CUtensorMap tmD2, const RowsP p)
{
    extern __shared__ uint8_t smem_raw[];
    const int total_items = (MODE == MODE_DX ? p.fixed_tiles : *p.n_tiles) * p.n_col_tiles;
    if ((int)blockIdx.x >= total_items) {                // whole CTA leaves before any barrier or TMEM use
        if (threadIdx.x == 0) sched_finish(p.sched);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int COLS_PER_ITEM = MODE == MODE_GATEUP ? BN / 2 : BN;
    const int kb_per_item = (MODE == MODE_DXG ? 2 : 1) * p.kblocks;

    const Pipe pipe = carve(smem_raw);
    const uint32_t tmem_base = cta_setup(pipe, warp);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int item = blockIdx.x;
            ok = sched_publish(pipe, 0, item, total_items, p.status);
            for (uint32_t nf = 1; ok && item >= 0; ++nf) {
                const int row_i = item / p.n_col_tiles, n0 = (item % p.n_col_tiles) * COLS_PER_ITEM;
                const int row_tile = p.tile_order ? p.tile_order[row_i] : row_i;
                const int brow = (MODE == MODE_DX ? 0 : p.tile_expert[row_tile] * p.b_rows_per_expert) + n0;
                const int row0 = row_tile * BM;
                for (int kb = 0; kb < kb_per_item; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(pipe.empty(s), ((it / STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT)) {
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_u32(pipe.tiles + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(pipe.full(s), STAGE_BYTES);
                    const bool second = MODE == MODE_DXG && kb >= p.kblocks;
                    const int kx = (second ? kb - p.kblocks : kb) * BK;
                    tma_load_2d(a_dst, second ? &tmA1 : &tmA0, kx, row0, pipe.full(s));
                    if (MODE == MODE_GATEUP) {
                        const int y = ((p.tile_expert[row_tile] * p.b_row_blocks + (n0 >> 7)) * p.b_kb + kb) * 128;
                        tma_load_2d(b_dst, &tmB0, 0, y, pipe.full(s));
                        tma_load_2d(b_dst + HALF_B, &tmB1, 0, y, pipe.full(s));
                    } else if (MODE == MODE_DOWN) {
                        const int y = ((p.tile_expert[row_tile] * p.b_row_blocks + (n0 >> 7)) * p.b_kb + kb) * 128;
                        tma_load_2d(b_dst, &tmB0, 0, y, pipe.full(s));
                        tma_load_2d(b_dst + HALF_B, &tmB0, 0, y + p.b_kb * 128, pipe.full(s));
                    } else {
                        const CUtensorMap* mb = second ? &tmB1 : &tmB0;
                        tma_load_2d(b_dst, mb, kx, brow, pipe.full(s));
                        tma_load_2d(b_dst + HALF_B, mb, kx, brow + BN / 2, pipe.full(s));
                    }
                }
                // the next item is claimed as late as possible (the ring is full by now, so the round trip to the
                // counter does not starve the tensor core): early claims would sit behind this CTA's unfinished work
                int next = sched_fetch(p.sched);
                if (ok) ok = sched_publish(pipe, nf, next, total_items, p.status);
                item = next;
            }
            sched_finish(p.sched);                       // this CTA asks for no more items
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (; ok; ++t) {
                const int item = sched_consume(pipe, t, p.status);
                if (item >= 0) sched_release(pipe, t);
                if (item < 0) break;
                const uint32_t buf = t & 1u;
                if (t >= 2 && !mbar_wait(pipe.acc_empty(buf), ((t >> 1) - 1) & 1, p.status, ERR_ACC_WAIT)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < kb_per_item; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(pipe.full(s), (it / STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(pipe.tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = make_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = make_desc(b_addr + k * 32, 16, 1024);
                        umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(pipe.empty(s));           // frees the stage once these MMAs have read it
                }
                umma_commit(pipe.acc_full(buf));          // accumulator of this item complete
            }
        }
    } else {
        // 16 epilogue warps: TMEM lane quarter q = warp % 4 (rows q*32..+31), column group h = 0..3
        const int q = warp & 3, h = (warp - 2) >> 2;
        uint8_t* stage = pipe.staging + (warp - 2) * STAGING_BYTES;
        uint32_t t = 0;
        for (;; ++t) {
            const int item = __shfl_sync(0xffffffffu, sched_consume(pipe, t, p.status), 0);   // warp-uniform
            if (item < 0) break;
            if (lane == 0) sched_release(pipe, t);
            const uint32_t buf = t & 1u;
            const int row_i = item / p.n_col_tiles, n0 = (item % p.n_col_tiles) * COLS_PER_ITEM;
            const int row_tile = p.tile_order ? p.tile_order[row_i] : row_i;
            const int e = MODE == MODE_DX ? 0 : p.tile_expert[row_tile];
            if (!rows_epilogue<MODE>(p, pipe.acc_full(buf), pipe.acc_empty(buf), false, tmem_base, buf, t, row_tile, n0, e, q, h,
                                     lane, stage, &tmD0, &tmD1, &tmD2, true))
                break;
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // stores landed before exit
    }
    cta_teardown(tmem_base, warp);
}

#include "gemm_tc_pair.inl"

// ---- weight gradients: grad[e][M,N] += A_e^T * B_e over the expert's rows ---------
// One weight-gradient problem: grad[e][M,N] += A_e^T * B_e over the rows of "expert" e.
struct WgradProb {
    float* const* grad;     // per-expert output [M,N]
    float* single_grad;     // or one output all chunks add into (router gradient)
    int M, N, n_tiles_m, n_tiles_n;
    int n_groups;           // experts, or uniform token chunks
    int uniform_rows;       // > 0: group g covers rows [g*uniform_rows, +uniform_rows) instead of an expert's rows
    int item_begin;         // first item index of this problem
    int transposed;         // the tile is grad^T: element (m, n) of the product belongs at grad[n*M + m]
};
struct WgradP {
    const int32_t* padded_offsets;
    const int32_t* seg;     // [E][n_seg][2] {first row, rows}: an expert's rows in n_seg segments (0 = one padded range)
    int n_seg;
    int32_t* status;
    int32_t* sched;         // {next item, finished CTAs}, both zero between launches
    WgradProb prob[3];
    int n_probs, total_items;
    int overwrite;          // grad = product (zeros for experts without rows) instead of grad += product
    int block_loads;        // the tensor maps are the column-block form: one load per operand tile and stage
    // bias gradients from the same operand tiles (null: none): gb[pr][e][col] += column sums, over the expert's
    // rows, of the operand of problem pr whose columns are that bias's (the A operand when the problem is
    // computed transposed, else the B operand)
    float* const* gb[3];
};
struct WgradItem {
    int pr, e, m0, n0, r0, nkb;
};
__device__ __forceinline__ WgradItem wgrad_item(const WgradP& p, int item)
{
    WgradItem w;
    w.pr = (p.n_probs > 2 && item >= p.prob[2].item_begin) ? 2 : (p.n_probs > 1 && item >= p.prob[1].item_begin) ? 1 : 0;
    const WgradProb& q = p.prob[w.pr];
    const int local = item - q.item_begin, per = q.n_tiles_m * q.n_tiles_n;
    w.e = local / per;
    const int r = local % per;
    w.m0 = (r / q.n_tiles_n) * BM;
    w.n0 = (r % q.n_tiles_n) * BN;
    if (q.uniform_rows) {
        w.r0 = w.e * q.uniform_rows;
        w.nkb = q.uniform_rows / BK;
    } else if (p.n_seg > 0) {
        w.r0 = 0;
        w.nkb = 0;
        for (int sg = 0; sg < p.n_seg; ++sg) w.nkb += p.seg[(w.e * p.n_seg + sg) * 2 + 1] / BK;
    } else {
        w.r0 = p.padded_offsets[w.e];
        w.nkb = (p.padded_offsets[w.e + 1] - w.r0) / BK;
    }
    return w;
}

// Persistent over items (problem, expert, m tile, n tile); experts without rows are skipped.
__global__ void __launch_bounds__(WG_THREADS, 1)
tc_wgrad_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, const WgradP p)
{
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_items = p.total_items;
    if ((int)blockIdx.x >= total_items) {
        if (threadIdx.x == 0) sched_finish(p.sched);
        return;
    }

    const Pipe pipe = carve(smem_raw);
    const uint32_t tmem_base = cta_setup(pipe, warp, CS_WARPS);
    constexpr uint32_t BOX = 64 * BK * 2;      // one {64 MN elements, 64 rows} box = 8 KiB

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int item = blockIdx.x;
            ok = sched_publish(pipe, 0, item, total_items, p.status);
            for (uint32_t nf = 1; ok && item >= 0; ++nf) {
                const WgradItem w = wgrad_item(p, item);
                const CUtensorMap* mA = w.pr == 0 ? &tmA0 : w.pr == 1 ? &tmA1 : &tmA2;
                const CUtensorMap* mB = w.pr == 0 ? &tmB0 : w.pr == 1 ? &tmB1 : &tmB2;
                const bool segmented = p.n_seg > 0 && !p.prob[w.pr].uniform_rows;
                const int nseg = segmented ? p.n_seg : 1;
                for (int sg = 0; sg < nseg && ok; ++sg) {
                    const int seg_r0 = segmented ? p.seg[(w.e * p.n_seg + sg) * 2] : w.r0;
                    const int seg_kb = segmented ? p.seg[(w.e * p.n_seg + sg) * 2 + 1] / BK : w.nkb;
                    for (int kb = 0; kb < seg_kb; ++kb, ++it) {
                        const int s = it % STAGES;
                        if (it >= STAGES && !mbar_wait(pipe.empty(s), ((it / STAGES) - 1) & 1, p.status, ERR_EMPTY_WAIT)) {
                            ok = false;
                            break;
                        }
                        const uint32_t a_dst = smem_u32(pipe.tiles + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                        mbar_expect_tx(pipe.full(s), STAGE_BYTES);
                        const int row = seg_r0 + kb * BK;
                        if (p.block_loads) {
                            // two loads per stage instead of six: with 64-row stages this kernel waits for the
                            // producer thread's issue rate as much as for the bytes (measured: 1.44 -> 1.39 ms)
                            tma_load_3d(a_dst, mA, 0, row, w.m0 / 64, pipe.full(s));
                            tma_load_3d(b_dst, mB, 0, row, w.n0 / 64, pipe.full(s));
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < BM / 64; ++i) tma_load_2d(a_dst + i * BOX, mA, w.m0 + 64 * i, row, pipe.full(s));
#pragma unroll
                        for (int i = 0; i < BN / 64; ++i) tma_load_2d(b_dst + i * BOX, mB, w.n0 + 64 * i, row, pipe.full(s));
                    }
                }
                // the next item is claimed as late as possible (the ring is full by now, so the round trip to the
                // counter does not starve the tensor core): early claims would sit behind this CTA's unfinished work
                int next = sched_fetch(p.sched);
                if (ok) ok = sched_publish(pipe, nf, next, total_items, p.status);
                item = next;
            }
            sched_finish(p.sched);                       // this CTA asks for no more items
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (uint32_t nf = 0; ok; ++nf) {
                const int item = sched_consume(pipe, nf, p.status);
                if (item < 0) break;
                sched_release(pipe, nf);
                const WgradItem w = wgrad_item(p, item);
                if (w.nkb <= 0) continue;
                const uint32_t buf = t & 1u;
                if (t >= 2 && !mbar_wait(pipe.acc_empty(buf), ((t >> 1) - 1) & 1, p.status, ERR_ACC_WAIT)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < w.nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(pipe.full(s), (it / STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(pipe.tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 reduction rows = two 8-row groups (1 KiB each); 64-element MN blocks are BOX apart
                        const uint64_t ad = make_desc(a_addr + k * 2048, BOX, 1024);
                        const uint64_t bd = make_desc(b_addr + k * 2048, BOX, 1024);
                        umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(pipe.empty(s));
                }
                umma_commit(pipe.acc_full(buf));
                ++t;
            }
        }
    } else if (warp >= 2 + EPI_WARPS) {
        // Column sums of an operand over the expert's rows = a bias gradient (layers/LinearLayer.cpp:56-57).  The tiles
        // are in shared memory anyway, so these two warps add rows up while the tensor core works on the same stage.
        // The operand tile whose columns are the bias's is made of 64-column boxes, and it is loaded once per tile of
        // the OTHER output dimension: box b is summed by the item whose other-dimension tile index is b modulo the
        // number of such tiles, so the work is spread over items (at most two boxes each; the host falls back to a
        // separate kernel for shapes where that does not cover every box).  The two warps split a box's 64 rows.
        // They take part in every stage and every item (fixed barrier counts), summing or not.
        const int cw = warp - (2 + EPI_WARPS);
        const int c8 = lane & 7, rg = lane >> 3;           // 16-byte piece of a 128-byte row; rows rg + 4i
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t nf = 0; ok; ++nf) {
            const int item = __shfl_sync(0xffffffffu, sched_consume(pipe, nf, p.status), 0);
            if (item < 0) break;
            if (lane == 0) sched_release(pipe, nf);
            const WgradItem w = wgrad_item(p, item);
            if (w.nkb <= 0) continue;
            const WgradProb& pb = p.prob[w.pr];
            float* const* gbt = p.gb[w.pr];
            // boxes of the operand tile, tiles of the other dimension, this item's index among them
            const int nbox = pb.transposed ? BM / 64 : BN / 64;
            const int other_tiles = pb.transposed ? pb.n_tiles_n : pb.n_tiles_m;
            const int other = pb.transposed ? w.n0 / BN : w.m0 / BM;
            int box0 = -1, box1 = -1;                       // the (at most two) boxes this item sums
            if (gbt) {
                if (other < nbox) box0 = other;
                if (other + other_tiles < nbox) box1 = other + other_tiles;
            }
            float acc[2][8];
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[b][i] = 0.0f;
            for (int kb = 0; kb < w.nkb; ++kb, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(pipe.full(s), (it / STAGES) & 1, p.status, ERR_FULL_WAIT)) {
                    ok = false;
                    break;
                }
                if (box0 >= 0) {
                    const uint32_t tile = smem_u32(pipe.tiles + s * STAGE_BYTES) + (pb.transposed ? 0 : A_BYTES);
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const int bx = b ? box1 : box0;
                        if (bx >= 0) {
                            const uint32_t box = tile + (uint32_t)bx * BOX;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const uint32_t r = (uint32_t)(rg + 32 * cw + 4 * i);
                                uint32_t w0, w1, w2, w3;
                                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                             : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                                             : "r"(box + r * 128u + ((((uint32_t)c8) ^ (r & 7u)) << 4)));
                                acc[b][0] += bf_lo(w0); acc[b][1] += bf_hi(w0); acc[b][2] += bf_lo(w1); acc[b][3] += bf_hi(w1);
                                acc[b][4] += bf_lo(w2); acc[b][5] += bf_hi(w2); acc[b][6] += bf_lo(w3); acc[b][7] += bf_hi(w3);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(pipe.empty(s));
            }
            if (box0 >= 0 && ok) {
                float* gbe = gbt[w.e];
                const int limit = pb.transposed ? pb.M : pb.N;
                const int col0 = pb.transposed ? w.m0 : w.n0;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const int bx = b ? box1 : box0;
                    if (bx >= 0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float v = acc[b][i];
                            v += __shfl_xor_sync(0xffffffffu, v, 8);
                            v += __shfl_xor_sync(0xffffffffu, v, 16);
                            const int col = col0 + bx * 64 + c8 * 8 + i;
                            if (rg == 0 && col < limit) atomicAdd(gbe + col, v);      // two partial sums per column: one per warp
                        }
                    }
                }
            }
        }
    } else {
        const int q = warp & 3, h = (warp - 2) >> 2;
        float* stage = reinterpret_cast<float*>(pipe.staging + (warp - 2) * STAGING_BYTES);   // [32 rows][16 floats]
        uint32_t t = 0;
        for (uint32_t nf = 0;; ++nf) {
            const int item = __shfl_sync(0xffffffffu, sched_consume(pipe, nf, p.status), 0);  // warp-uniform
            if (item < 0) break;
            if (lane == 0) sched_release(pipe, nf);
            const WgradItem w = wgrad_item(p, item);
            const WgradProb& pb = p.prob[w.pr];
            float* g = pb.single_grad ? pb.single_grad : pb.grad[w.e];
            const int M = pb.M, N = pb.N;
            const int m_w = w.m0 + q * 32;             // first product row of this warp
            const int n_w = w.n0 + h * 64;             // first product column of this warp
            if (w.nkb <= 0) {
                // an expert without rows: nothing to add; when gradients are overwritten its tile is zeros
                if (p.overwrite) {
                    const int m = m_w + lane;
                    if (pb.transposed) {
                        for (int j = 0; j < 64; ++j)
                            if (m < M && n_w + j < N) g[(size_t)(n_w + j) * M + m] = 0.0f;
                    } else {
                        for (int r = 0; r < 32; ++r)
                            for (int j = lane; j < 64; j += 32)
                                if (m_w + r < M && n_w + j < N) g[(size_t)(m_w + r) * N + n_w + j] = 0.0f;
                    }
                }
                continue;
            }
            const uint32_t buf = t & 1u;
            if (!mbar_wait(pipe.acc_full(buf), (t >> 1) & 1, p.status, ERR_ACC_WAIT)) break;
            tc_fence_after();
            const uint32_t t_lane = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16) + h * 64;
            float v[2][32];
            tmem_ld32(t_lane, v[0]);
            tmem_ld32(t_lane + 32, v[1]);
            tmem_ld_wait();
            release_acc(pipe.acc_empty(buf), lane);
            if (pb.transposed) {
                // this thread's product row m is a COLUMN of grad: for one register the 32 lanes cover 32
                // consecutive floats of one grad row, so every scalar instruction is one full 128-byte line
                const int m = m_w + lane;
                if (m < M) {
                    float* gm = g + m;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const int n = n_w + j;
                        if (n < N) {
                            if (p.overwrite) gm[(size_t)n * M] = v[j >> 5][j & 31];
                            else atomicAdd(gm + (size_t)n * M, v[j >> 5][j & 31]);
                        }
                    }
                }
                ++t;
                continue;
            }
            const uint32_t sw_w = ((uint32_t)lane >> 1) & 3u;            // writer: row = lane
            const int sub = lane >> 2, piece = lane & 3;                 // reader: 8 rows x 4 pieces per pass
#pragma unroll
            for (int c = 0; c < 4; ++c) {                                // four groups of 16 columns
                const int n = n_w + c * 16;
                if (n >= N) break;
                // transpose through shared memory (16-byte pieces, XOR-swizzled by row) so that one vector
                // RED instruction covers eight full 64-byte row segments
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int s0 = (c & 1) * 16 + 4 * j;
                    *reinterpret_cast<float4*>(&stage[lane * 16 + (((uint32_t)j ^ sw_w) << 2)]) =
                        make_float4(v[c >> 1][s0], v[c >> 1][s0 + 1], v[c >> 1][s0 + 2], v[c >> 1][s0 + 3]);
                }
                __syncwarp();
                const int col = n + piece * 4;
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {
                    const int row = rr * 8 + sub, m = m_w + row;
                    const float4 x = *reinterpret_cast<const float4*>(
                        &stage[row * 16 + (((uint32_t)piece ^ (((uint32_t)row >> 1) & 3u)) << 2)]);
                    if (m < M && col < N) {
                        if (p.overwrite) *reinterpret_cast<float4*>(g + (size_t)m * N + col) = x;
                        else red_add_v4(g + (size_t)m * N + col, x);
                    }
                }
                __syncwarp();
            }
            ++t;
        }
    }
    cta_teardown(tmem_base, warp);
}

}  // namespace

// ---- host side: tensor maps ------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
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

// 2-D row-major bf16 tensor [rows, cols].  Loads: box = {64 columns (128 B), box_rows}, 128-byte swizzle,
// OOB reads 0.  Stores (box_rows == 32): box = {32 columns (64 B), 32 rows}, 64-byte swizzle.
int make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    return make_map_kind(m, base, rows, cols, box_rows, box_rows == 32);
}

int make_map_kind(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool store)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MGPT_MOE_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * sizeof(bf16)};
    cuuint32_t box[2] = {store ? 32u : 64u, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, store ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MGPT_MOE_ECUDA, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
    return 0;
}

bool make_map_blocks(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t n_blocks)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || cols % 64 != 0) return false;
    cuuint64_t dims[3] = {64, rows, cols / 64};
    cuuint64_t strides[2] = {cols * sizeof(bf16), 64 * sizeof(bf16)};
    cuuint32_t box[3] = {64, box_rows, n_blocks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

namespace {

struct TcState {
    const void* ws = nullptr;
    const void *xg = nullptr, *yg = nullptr, *dyg = nullptr, *dxg = nullptr;
    int n_tokens = -1;
    bool attr_set = false;
    int sms = 0;
    int max_pairs = 0;           // CTA pairs (clusters of two) that can be resident at once; 0 = pair kernels off
    int32_t* sched = nullptr;    // device: one {next item, finished CTAs} pair per kind of launch, zero between launches
    // K-major operand loads (box 64 x 128 rows)
    CUtensorMap Xg, Hh, dYg, dG, dU, WgT, WuT, WdT, Wg, Wu, Wd;
    // reduction-over-rows operand loads (box 64 x 64 rows)
    CUtensorMap Xg_t, Hh_t, dYg_t, dG_t, dU_t;
    // the same operands by column blocks (one load per operand tile): A side {64, 64 rows, 2}, B side {64, 64 rows, 4}
    CUtensorMap Xg_b4, dYg_b4, dG_b2, dU_b2, Hh_b2;
    bool blocks_ok = false;      // the driver took the block maps (else six 2-D loads per stage)
    // epilogue stores (box 32 x 32 rows, 64-byte swizzle)
    CUtensorMap Hh_s, Yg_s, dG_s, dU_s, dXg_s;
};

int prepare_attrs(mgpt_moe_layer* L);

int prepare(mgpt_moe_layer* L, const Workspace& w, char* ws)
{
    MGPT_TRY(prepare_attrs(L));
    TcState* s = (TcState*)L->tc_state;
    const void *xg = buf_Xg(L, w, ws), *yg = buf_Yg(L, w, ws), *dyg = buf_dYg(L, w, ws), *dxg = buf_dXg(L, w, ws);
    if (s->ws == ws && s->n_tokens == w.n_tokens && s->xg == xg && s->yg == yg && s->dyg == dyg && s->dxg == dxg) return 0;
    const Dims& d = L->d;
    const uint64_t rc = w.row_cap, C = d.C, H = d.H, E = d.E;
    MGPT_TRY(make_map(&s->Xg, xg, rc, C, 128));
    MGPT_TRY(make_map(&s->Hh, ws + w.Hh, rc, H, 128));
    MGPT_TRY(make_map(&s->dYg, dyg, rc, C, 128));
    MGPT_TRY(make_map(&s->dG, ws + w.dG, rc, H, 128));
    MGPT_TRY(make_map(&s->dU, ws + w.dU, rc, H, 128));
    // tile-major copies: one 16 KiB block per (128 rows, 64 columns), seen as a tall matrix of 64 columns
    MGPT_TRY(make_map(&s->WgT, L->sWgT, E * tile_major_elems(d.H, d.C) / 64, 64, 128));
    MGPT_TRY(make_map(&s->WuT, L->sWuT, E * tile_major_elems(d.H, d.C) / 64, 64, 128));
    MGPT_TRY(make_map(&s->WdT, L->sWdT, E * tile_major_elems(d.C, d.H) / 64, 64, 128));
    MGPT_TRY(make_map(&s->Wg, L->sWg, E * C, H, 128));
    MGPT_TRY(make_map(&s->Wu, L->sWu, E * C, H, 128));
    MGPT_TRY(make_map(&s->Wd, L->sWd, E * H, C, 128));
    MGPT_TRY(make_map(&s->Xg_t, xg, rc, C, 64));
    MGPT_TRY(make_map(&s->Hh_t, ws + w.Hh, rc, H, 64));
    MGPT_TRY(make_map(&s->dYg_t, dyg, rc, C, 64));
    MGPT_TRY(make_map(&s->dG_t, ws + w.dG, rc, H, 64));
    MGPT_TRY(make_map(&s->dU_t, ws + w.dU, rc, H, 64));
    s->blocks_ok = make_map_blocks(&s->Xg_b4, xg, rc, C, 64, BN / 64) && make_map_blocks(&s->dYg_b4, dyg, rc, C, 64, BN / 64) &&
                   make_map_blocks(&s->dG_b2, ws + w.dG, rc, H, 64, BM / 64) && make_map_blocks(&s->dU_b2, ws + w.dU, rc, H, 64, BM / 64) &&
                   make_map_blocks(&s->Hh_b2, ws + w.Hh, rc, H, 64, BM / 64);
    MGPT_TRY(make_map(&s->Hh_s, ws + w.Hh, rc, H, 32));
    MGPT_TRY(make_map(&s->Yg_s, yg, rc, C, 32));
    MGPT_TRY(make_map(&s->dG_s, ws + w.dG, rc, H, 32));
    MGPT_TRY(make_map(&s->dU_s, ws + w.dU, rc, H, 32));
    MGPT_TRY(make_map(&s->dXg_s, dxg, rc, C, 32));
    s->ws = ws;
    s->n_tokens = w.n_tokens;
    s->xg = xg; s->yg = yg; s->dyg = dyg; s->dxg = dxg;
    return 0;
}

int prepare_attrs(mgpt_moe_layer* L)
{
    if (!L->tc_state) L->tc_state = new TcState();
    TcState* s = (TcState*)L->tc_state;
    if (!s->attr_set) {
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DHH>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DXG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_kernel<MODE_DX>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaDeviceGetAttribute(&s->sms, cudaDevAttrMultiProcessorCount, L->device));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_pair_kernel<MODE_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_pair_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_pair_kernel<MODE_DHH>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        MGPT_CUDA(cudaFuncSetAttribute(tc_rows_pair_kernel<MODE_DXG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        {
            // The CTA-pair kernels (gemm_tc_pair.inl) are opt-in, MGPT_MOE_CTA_PAIRS=1 in the environment: measured on
            // B200 they match the single-CTA kernels at the 64-expert shapes (both sit at ~82-90 % of what cuBLAS
            // sustains under the 1 kW power cap) and lose a little on small shapes.  How many clusters of two CTAs
            // fit on the device at once is asked of the driver (SMs pair up within a GPC).
            const char* env = getenv("MGPT_MOE_CTA_PAIRS");
            s->max_pairs = 0;
            if (env && env[0] == '1') {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(2 * (unsigned)s->sms, 1, 1);
                cfg.blockDim = dim3(TC_THREADS, 1, 1);
                cfg.dynamicSmemBytes = SMEM_BYTES;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
                cfg.attrs = at;
                cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, tc_rows_pair_kernel<MODE_DOWN>, &cfg) == cudaSuccess && n > 0)
                    s->max_pairs = n;
                else
                    cudaGetLastError();       // no pairs on this device: the single-CTA kernels stay
            }
            if (getenv("MGPT_MOE_VERBOSE")) fprintf(stderr, "mgpt_moe: %d SMs, %d resident CTA pairs\n", s->sms, s->max_pairs);
        }
        // the work-item counters must read zero before the first launch on any stream: allocate and clear them
        // here, at layer creation, and wait for the clear (nothing orders the legacy stream with a caller's
        // non-blocking stream)
        MGPT_CUDA(cudaMalloc(&s->sched, 64 * sizeof(int32_t)));
        MGPT_CUDA(cudaMemset(s->sched, 0, 64 * sizeof(int32_t)));
        MGPT_CUDA(cudaDeviceSynchronize());
        s->attr_set = true;
    }
    return 0;
}

int cdiv(int a, int b) { return (a + b - 1) / b; }
int imin(int a, int b) { return a < b ? a : b; }
// persistent CTAs to launch: every SM, or the caller's budget when other kernels must stay resident beside these
int grid_sms(const mgpt_moe_layer* L, const TcState* s) { return L->sm_budget > 0 ? imin(L->sm_budget, s->sms) : s->sms; }

}  // namespace

// The weight-gradient kernel also sums the bias gradients when every 64-column box of its operand tiles finds an
// item to sum it: the B tile of gWd has four boxes and is loaded once per 128-row tile of H, two boxes per item.
bool tc_fused_bias_grads(const Dims& d) { return cdiv(d.H, BM) >= 2; }

namespace {
// One of the four token-major products: on CTA pairs where the device takes them, else one CTA per tile.
template <int MODE>
int launch_rows(mgpt_moe_layer* L, TcState* s, const Workspace& w, const RowsP& p, const CUtensorMap& a0, const CUtensorMap& a1,
                const CUtensorMap& b0, const CUtensorMap& b1, const CUtensorMap& d0, const CUtensorMap& d1,
                const CUtensorMap& d2, cudaStream_t st, const char* what)
{
    const int budget = grid_sms(L, s);
    if (s->max_pairs > 0 && p.pairs) {
        const int pairs = imin(imin(s->max_pairs, budget / 2), w.max_tiles * p.n_col_tiles);
        tc_rows_pair_kernel<MODE><<<2 * (pairs > 0 ? pairs : 1), TC_THREADS, SMEM_BYTES, st>>>(a0, a1, b0, b1, d0, d1, d2, p);
    } else {
        tc_rows_kernel<MODE><<<imin(budget, w.max_tiles * p.n_col_tiles), TC_THREADS, SMEM_BYTES, st>>>(a0, a1, b0, b1, d0, d1, d2, p);
    }
    MGPT_LAUNCHED(what);
    return 0;
}
}  // namespace

int tc_experts_forward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    MGPT_TRY(prepare(L, w, ws));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    RowsP p = {};
    p.tile_expert = (const int32_t*)(ws + w.tile_expert);
    p.tile_order = L->n_seg > 0 ? (const int32_t*)(ws + w.tile_order) : nullptr;
    p.n_tiles = (const int32_t*)(ws + w.n_tiles);
    p.pairs = (const int32_t*)(ws + w.pairs);
    p.n_pairs = (const int32_t*)(ws + w.n_pairs);
    p.status = L->d_status;
    // gate/up + SwiGLU: K = C, 128 hidden units per item
    p.kblocks = cdiv(d.C, BK); p.n_out = d.H; p.b_rows_per_expert = d.H; p.n_col_tiles = cdiv(d.H, BN / 2);
    p.b_row_blocks = cdiv(d.H, 128); p.b_kb = cdiv(d.C, BK);
    p.bias0 = L->master.bg; p.bias1 = L->master.bu;
    p.G = w.inference ? nullptr : (bf16*)(ws + w.G);
    p.U = w.inference ? nullptr : (bf16*)(ws + w.U);
    L->stage_begin(ST_GATEUP, st);
    p.sched = s->sched + 0;
    MGPT_TRY(launch_rows<MODE_GATEUP>(L, s, w, p, s->Xg, s->Xg, s->WgT, s->WuT, s->Hh_s, s->Hh_s, s->Hh_s, st, "tc_rows<gateup>"));
    L->stage_end(ST_GATEUP, st);
    // down: K = H
    p.kblocks = cdiv(d.H, BK); p.n_out = d.C; p.b_rows_per_expert = d.C; p.n_col_tiles = cdiv(d.C, BN);
    p.b_row_blocks = cdiv(d.C, 128); p.b_kb = cdiv(d.H, BK);
    p.bias0 = L->master.bd; p.bias1 = nullptr;
    L->stage_begin(ST_DOWN, st);
    p.sched = s->sched + 2;
    MGPT_TRY(launch_rows<MODE_DOWN>(L, s, w, p, s->Hh, s->Hh, s->WdT, s->WdT, s->Yg_s, s->Yg_s, s->Yg_s, st, "tc_rows<down>"));
    L->stage_end(ST_DOWN, st);
    return 0;
}

// phase: 1 = gradients w.r.t. the rows (dHh, dXg), 2 = gradients w.r.t. the parameters, 3 = both
int tc_experts_backward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st, int phase)
{
    MGPT_TRY(prepare(L, w, ws));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    RowsP p = {};
    if (phase & 1) {
    p.tile_expert = (const int32_t*)(ws + w.tile_expert);
    p.tile_order = L->n_seg > 0 ? (const int32_t*)(ws + w.tile_order) : nullptr;
    p.n_tiles = (const int32_t*)(ws + w.n_tiles);
    p.pairs = (const int32_t*)(ws + w.pairs);
    p.n_pairs = (const int32_t*)(ws + w.n_pairs);
    p.status = L->d_status;
    // dHh = dYg * Wd^T  (K = C), SwiGLU backward in the epilogue
    p.kblocks = cdiv(d.C, BK); p.n_out = d.H; p.b_rows_per_expert = d.H; p.n_col_tiles = cdiv(d.H, BN);
    p.G = (bf16*)(ws + w.G); p.U = (bf16*)(ws + w.U);
    L->stage_begin(ST_DHH, st);
    p.sched = s->sched + 4;
    MGPT_TRY(launch_rows<MODE_DHH>(L, s, w, p, s->dYg, s->dYg, s->Wd, s->Wd, s->dG_s, s->dU_s, s->dU_s, st, "tc_rows<dhh>"));
    L->stage_end(ST_DHH, st);
    // dXg = dG * Wg^T + dU * Wu^T  (K = 2H)
    p.kblocks = cdiv(d.H, BK); p.n_out = d.C; p.b_rows_per_expert = d.C; p.n_col_tiles = cdiv(d.C, BN);
    L->stage_begin(ST_DXG, st);
    p.sched = s->sched + 6;
    MGPT_TRY(launch_rows<MODE_DXG>(L, s, w, p, s->dG, s->dU, s->Wg, s->Wu, s->dXg_s, s->dXg_s, s->dXg_s, st, "tc_rows<dxg>"));
    L->stage_end(ST_DXG, st);
    }
    if (!L->has_grad || !(phase & 2)) return 0;

    // all three weight gradients in one launch:
    //   gWg += Xg^T dG, gWu += Xg^T dU   [C,H];   gWd += Hh^T dYg   [H,C]
    // The first two are computed transposed, (dG^T Xg) [H,C]: H = 1408 splits into eleven 128-row tiles and C into
    // whole 256-column tiles, where the direct form leaves the last of six 256-column tiles over H half empty.
    // Writing the tile back transposed costs nothing: a thread's row index runs along a row of the gradient.
    WgradP g = {};
    g.padded_offsets = (const int32_t*)(ws + w.padded_offsets);
    g.seg = (const int32_t*)(ws + w.seg);
    g.n_seg = L->n_seg;
    g.status = L->d_status;
    g.n_probs = 3;
    g.overwrite = L->bwd_overwrite ? 1 : 0;
    float* const* grads[3] = {L->master.gWg, L->master.gWu, L->master.gWd};
    int items = 0;
    for (int i = 0; i < 3; ++i) {
        WgradProb& q = g.prob[i];
        q.grad = grads[i];
        q.M = d.H;
        q.N = d.C;
        q.transposed = i < 2 ? 1 : 0;
        q.n_tiles_m = cdiv(q.M, BM);
        q.n_tiles_n = cdiv(q.N, BN);
        q.n_groups = d.E;
        q.item_begin = items;
        items += d.E * q.n_tiles_m * q.n_tiles_n;
    }
    g.total_items = items;
    L->stage_begin(ST_WGRAD, st);
    g.sched = s->sched + 8;
    if (tc_fused_bias_grads(d)) {
        g.gb[0] = L->master.gbg; g.gb[1] = L->master.gbu; g.gb[2] = L->master.gbd;
    }
    g.block_loads = s->blocks_ok ? 1 : 0;
    if (g.block_loads)
        tc_wgrad_kernel<<<imin(grid_sms(L, s), items), WG_THREADS, SMEM_BYTES, st>>>(s->dG_b2, s->Xg_b4, s->dU_b2, s->Xg_b4,
                                                                           s->Hh_b2, s->dYg_b4, g);
    else
        tc_wgrad_kernel<<<imin(grid_sms(L, s), items), WG_THREADS, SMEM_BYTES, st>>>(s->dG_t, s->Xg_t, s->dU_t, s->Xg_t, s->Hh_t,
                                                                           s->dYg_t, g);
    MGPT_LAUNCHED("tc_wgrad_kernel");
    L->stage_end(ST_WGRAD, st);
    return 0;
}

// dx[N,C] (bf16) = gather-sum of the tokens' expert rows + dlogits * Wr^T on the tensor cores
// (K = experts, so the product is a single k-block; the kernel is bound by the row gather).
int tc_router_dx(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* dXg, const int32_t* pos, void* dx,
                 cudaStream_t st)
{
    MGPT_TRY(prepare_attrs(L));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    const int E8 = (d.E + 7) / 8 * 8;
    CUtensorMap mA, mB, mD;
    MGPT_TRY(make_map(&mA, ws + w.dl16, (uint64_t)w.n_tokens, (uint64_t)E8, 128));
    MGPT_TRY(make_map(&mB, L->sWr, (uint64_t)d.C, (uint64_t)E8, 128));
    MGPT_TRY(make_map(&mD, dx, (uint64_t)w.n_tokens, (uint64_t)d.C, 32));
    RowsP p = {};
    p.n_tiles = (const int32_t*)(ws + w.n_tiles);
    p.tile_expert = (const int32_t*)(ws + w.tile_expert);
    p.status = L->d_status;
    p.kblocks = cdiv(E8, BK); p.n_out = d.C; p.b_rows_per_expert = 0; p.n_col_tiles = cdiv(d.C, BN);
    p.fixed_tiles = cdiv(w.n_tokens, BM); p.n_valid_rows = w.n_tokens;
    p.gather_src = (const bf16*)dXg; p.gather_pos = pos; p.gather_k = d.k;
    p.sched = s->sched + 10;
    tc_rows_kernel<MODE_DX><<<imin(grid_sms(L, s), p.fixed_tiles * p.n_col_tiles), TC_THREADS, SMEM_BYTES, st>>>(
        mA, mA, mB, mB, mD, mD, mD, p);
    MGPT_LAUNCHED("tc_rows_kernel<dx>");
    return 0;
}

// gWr[C,E] += x^T * dlogits on the tensor cores, split over uniform token chunks (RED accumulation).
int tc_router_wgrad(mgpt_moe_layer* L, const Workspace& w, char* ws, const void* x, cudaStream_t st)
{
    MGPT_TRY(prepare_attrs(L));
    TcState* s = (TcState*)L->tc_state;
    const Dims& d = L->d;
    const int E8 = (d.E + 7) / 8 * 8;
    CUtensorMap mA, mB;
    MGPT_TRY(make_map(&mA, x, (uint64_t)w.n_tokens, (uint64_t)d.C, 64));
    MGPT_TRY(make_map(&mB, ws + w.dl16, (uint64_t)w.n_tokens, (uint64_t)E8, 64));
    WgradP g = {};
    g.status = L->d_status;
    g.n_probs = 1;
    WgradProb& q = g.prob[0];
    q.M = d.C; q.N = d.E; q.n_tiles_m = cdiv(d.C, BM); q.n_tiles_n = cdiv(d.E, BN);
    const int per_chunk = q.n_tiles_m * q.n_tiles_n;
    int chunks = imin(64, (2 * s->sms + per_chunk - 1) / per_chunk);
    int rows = cdiv(cdiv(w.n_tokens, chunks), BK) * BK;           // tokens per chunk, whole k-blocks
    chunks = cdiv(w.n_tokens, rows);
    q.n_groups = chunks; q.uniform_rows = rows; q.single_grad = L->p_grad[0]; q.item_begin = 0;
    g.total_items = chunks * per_chunk;
    g.sched = s->sched + 12;
    tc_wgrad_kernel<<<imin(grid_sms(L, s), g.total_items), WG_THREADS, SMEM_BYTES, st>>>(mA, mB, mA, mB, mA, mB, g);
    MGPT_LAUNCHED("tc_wgrad_kernel<Wr>");
    return 0;
}

// One barrier nothing ever arrives on, waited for with the kernels' own bounded wait and a short limit: the wait
// runs out after a few thousand polls, the error bit is set and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int32_t* status)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_wait(smem_u32(&bar), 0, status, ERR_FULL_WAIT, 1u << 12);
    }
}

int tc_selftest_bounded_wait(mgpt_moe_layer* L, cudaStream_t st)
{
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(L->d_status);
    MGPT_LAUNCHED("bounded_wait_selftest_kernel");
    L->last_stream = st;
    return 0;
}

// Called once from mgpt_moe_create (the layer's device is current): function attributes, SM count, work counters.
int tc_init(mgpt_moe_layer* L) { return prepare_attrs(L); }

void tc_destroy(mgpt_moe_layer* L)
{
    TcState* s = (TcState*)L->tc_state;
    if (s && s->sched) cudaFree(s->sched);
    delete s;
    L->tc_state = nullptr;
}

}  // namespace mgpt
