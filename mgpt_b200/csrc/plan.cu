// Dispatch plan, token permutation and combine of the MoE layer.
//
// Reference semantics (paths relative to the reference's src/main/):
//   counts / offsets   utils/Tensor.cpp:1336-1352, layers/MoELayer.cpp:61-80
//   slot assignment    utils/Tensor.cpp:1368-1381 (flat index ascending => stable)
//   combine            utils/Tensor.cpp:1398-1406
//   combine backward   utils/Tensor.cpp:1424-1436
//
// The reference claims slots with a float atomicAdd on the GPU and a host
// round trip for the prefix sum.  Here the plan is built on the device with
// no atomics on the slot order and no host synchronisation: block histograms,
// one scan, then a stable rank per flat index.  The slot map therefore equals
// the CPU reference's bit for bit.
//
// Rows are stored expert-major with every expert's segment padded to a
// multiple of ROW_TILE rows; padding rows are zero.  Every product tile is
// then a full tile of one expert, and zero rows contribute nothing to the
// weight gradients.
#include <mutex>

#include "common.cuh"

namespace mgpt {

namespace {

constexpr int PLAN_BLOCK = 1024;   // flat indices per block

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16(v); }

// (1) per-block expert histogram
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_count_kernel(const int32_t* __restrict__ top_idx, int R, int E, int32_t* __restrict__ blk_cnt)
{
    __shared__ int cnt[MAX_EXPERTS];
    if (threadIdx.x < E) cnt[threadIdx.x] = 0;
    __syncthreads();
    const int i = blockIdx.x * PLAN_BLOCK + threadIdx.x;
    if (i < R) {
        const int e = top_idx[i];
        if ((unsigned)e < (unsigned)E) atomicAdd(&cnt[e], 1);      // ids outside [0, E) are reported by plan_assign_kernel
    }
    __syncthreads();
    if (threadIdx.x < E) blk_cnt[(size_t)blockIdx.x * E + threadIdx.x] = cnt[threadIdx.x];
}

// (2) scan: per expert over blocks, then over experts (compact and padded), tile list
__global__ void __launch_bounds__(MAX_EXPERTS)
plan_scan_kernel(int32_t* __restrict__ blk_cnt, int n_blocks, int E,
                 int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                 int32_t* __restrict__ padded_offsets, int32_t* __restrict__ tile_expert,
                 int32_t* __restrict__ n_tiles, int max_tiles, int32_t* __restrict__ status,
                 int32_t* __restrict__ sticky, int32_t* __restrict__ pairs, int32_t* __restrict__ n_pairs)
{
    __shared__ int tot[MAX_EXPERTS];
    __shared__ int poff[MAX_EXPERTS + 1];
    __shared__ int pair0[MAX_EXPERTS + 1];
    const int e = threadIdx.x;
    if (e < E) {
        int run = 0;
        for (int b = 0; b < n_blocks; ++b) {
            const int c = blk_cnt[(size_t)b * E + e];
            blk_cnt[(size_t)b * E + e] = run;      // becomes the block's base within the expert
            run += c;
        }
        tot[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (e == 0) {
        int off = 0, p = 0;
        for (int i = 0; i < E; ++i) {
            offsets[i] = off;
            poff[i] = p;
            padded_offsets[i] = p;
            off += tot[i];
            p += (tot[i] + ROW_TILE - 1) / ROW_TILE * ROW_TILE;
        }
        poff[E] = p;
        padded_offsets[E] = p;
        const int nt = p / ROW_TILE;
        *n_tiles = nt;
        // pairs of row tiles of one expert, for the kernels in which two CTAs share a tile of the weights
        int np = 0;
        for (int i = 0; i < E; ++i) {
            pair0[i] = np;
            np += ((poff[i + 1] - poff[i]) / ROW_TILE + 1) / 2;
        }
        pair0[E] = np;
        if (n_pairs) *n_pairs = np;
        *status = nt > max_tiles ? ST_PLAN_OVERFLOW : 0;      // cannot happen: max_tiles bounds sum(ceil); also clears the word
        if (sticky && nt > max_tiles) atomicOr(sticky, ST_PLAN_OVERFLOW);
    }
    __syncthreads();
    if (e < E) {
        const int t0 = poff[e] / ROW_TILE, t1 = poff[e + 1] / ROW_TILE;
        for (int t = t0; t < t1 && t < max_tiles; ++t) tile_expert[t] = e;
        if (pairs) {
            int pi = pair0[e];
            for (int t = t0; t < t1 && t < max_tiles; t += 2, ++pi) {
                pairs[2 * pi] = t;
                pairs[2 * pi + 1] = (t + 1 < t1 && t + 1 < max_tiles) ? t + 1 : -1;     // a lone last tile has no partner
            }
        }
    }
}

// (3) stable rank of every flat index within its expert -> map / pos / row_src
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_assign_kernel(const int32_t* __restrict__ top_idx, int R, int E,
                   const int32_t* __restrict__ blk_base, const int32_t* __restrict__ counts,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ padded_offsets,
                   int32_t* __restrict__ map, int32_t* __restrict__ pos, int32_t* __restrict__ row_src,
                   int32_t* __restrict__ slot_of, int32_t* __restrict__ status, int32_t* __restrict__ sticky)
{
    __shared__ int warp_cnt[PLAN_BLOCK / 32][MAX_EXPERTS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (PLAN_BLOCK / 32) * MAX_EXPERTS; i += PLAN_BLOCK) (&warp_cnt[0][0])[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * PLAN_BLOCK + threadIdx.x;
    bool valid = i < R;
    int e = valid ? top_idx[i] : 0;
    if (valid && (unsigned)e >= (unsigned)E) {                    // an id no expert has: no slot, and the caller is told
        atomicOr(status, ST_BAD_EXPERT);
        if (sticky) atomicOr(sticky, ST_BAD_EXPERT);
        valid = false;
    }
    if (!valid) e = -1 - lane;                                    // distinct keys for idle lanes
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (valid) {
        int base = 0;
        for (int w = 0; w < warp; ++w) base += warp_cnt[w][e];
        const int r = blk_base[(size_t)blockIdx.x * E + e] + base + rank_in_warp;
        const int slot = offsets[e] + r;
        const int p = padded_offsets[e] + r;
        map[slot] = i;
        pos[i] = p;
        row_src[p] = i;
        if (slot_of) slot_of[i] = slot;
    }
    // padding rows of every expert's segment carry no source (block 0, one thread per expert)
    if (blockIdx.x == 0 && threadIdx.x < E) {
        const int e2 = threadIdx.x;
        for (int q = padded_offsets[e2] + counts[e2]; q < padded_offsets[e2 + 1]; ++q) row_src[q] = -1;
    }
}

// The whole plan in one block, for up to PLAN_BLOCK routed rows (decode-sized batches): histogram, prefix sums, tile
// and pair lists and the stable slot assignment without leaving the SM -- one launch instead of three.
__global__ void __launch_bounds__(PLAN_BLOCK)
plan_small_kernel(const int32_t* __restrict__ top_idx, int R, int E, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ padded_offsets, int32_t* __restrict__ tile_expert,
                  int32_t* __restrict__ n_tiles, int max_tiles, int32_t* __restrict__ map, int32_t* __restrict__ pos,
                  int32_t* __restrict__ row_src, int32_t* __restrict__ slot_of, int32_t* __restrict__ status,
                  int32_t* __restrict__ sticky, int32_t* __restrict__ pairs, int32_t* __restrict__ n_pairs)
{
    __shared__ int warp_cnt[PLAN_BLOCK / 32][MAX_EXPERTS];
    __shared__ int tot[MAX_EXPERTS], off[MAX_EXPERTS + 1], poff[MAX_EXPERTS + 1], pair0[MAX_EXPERTS + 1];
    __shared__ int bad;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (PLAN_BLOCK / 32) * MAX_EXPERTS; i += PLAN_BLOCK) (&warp_cnt[0][0])[i] = 0;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    const int i = threadIdx.x;
    bool valid = i < R;
    int e = valid ? top_idx[i] : 0;
    if (valid && (unsigned)e >= (unsigned)E) {
        bad = 1;
        valid = false;
    }
    if (!valid) e = -1 - lane;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (threadIdx.x < E) {
        int t = 0;
        for (int w = 0; w < PLAN_BLOCK / 32; ++w) t += warp_cnt[w][threadIdx.x];
        tot[threadIdx.x] = t;
        counts[threadIdx.x] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, p = 0, np = 0;
        for (int x = 0; x < E; ++x) {
            off[x] = o; poff[x] = p; pair0[x] = np;
            offsets[x] = o; padded_offsets[x] = p;
            const int tiles = (tot[x] + ROW_TILE - 1) / ROW_TILE;
            o += tot[x]; p += tiles * ROW_TILE; np += (tiles + 1) / 2;
        }
        off[E] = o; poff[E] = p; pair0[E] = np;
        padded_offsets[E] = p;
        *n_tiles = p / ROW_TILE;
        if (n_pairs) *n_pairs = np;
        const int st = (p / ROW_TILE > max_tiles ? ST_PLAN_OVERFLOW : 0) | (bad ? ST_BAD_EXPERT : 0);
        *status = st;
        if (sticky && st) atomicOr(sticky, st);
    }
    __syncthreads();
    if (threadIdx.x < E) {
        const int x = threadIdx.x;
        const int t0 = poff[x] / ROW_TILE, t1 = poff[x + 1] / ROW_TILE;
        int pi = pair0[x];
        for (int t = t0; t < t1 && t < max_tiles; ++t) tile_expert[t] = x;
        if (pairs)
            for (int t = t0; t < t1 && t < max_tiles; t += 2, ++pi) {
                pairs[2 * pi] = t;
                pairs[2 * pi + 1] = (t + 1 < t1 && t + 1 < max_tiles) ? t + 1 : -1;
            }
        for (int q = poff[x] + tot[x]; q < poff[x + 1]; ++q) row_src[q] = -1;
    }
    if (valid) {
        int base = 0;
        for (int w = 0; w < warp; ++w) base += warp_cnt[w][e];
        const int r = base + rank_in_warp;
        const int slot = off[e] + r, p = poff[e] + r;
        map[slot] = i;
        pos[i] = p;
        row_src[p] = i;
        if (slot_of) slot_of[i] = slot;
    }
}

// Xg[p,:] = x[row_src[p]/k,:]  (zero for padding rows).  One warp per row, 16-byte accesses.
template <typename TIn, typename TAct>
__global__ void __launch_bounds__(256)
dispatch_rows_kernel(const TIn* __restrict__ x, const int32_t* __restrict__ row_src,
                     const int32_t* __restrict__ n_tiles, int fixed_rows, int C, int k, TAct* __restrict__ Xg)
{
    const int lane = threadIdx.x & 31;
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // rows in use: all tiles of the plan, or a count the host already knows
    if (p >= (fixed_rows >= 0 ? fixed_rows : *n_tiles * ROW_TILE)) return;
    const int src = row_src[p];
    TAct* dst = Xg + (size_t)p * C;
    constexpr int VIN = 16 / sizeof(TIn), VOUT = 16 / sizeof(TAct);
    constexpr int V = VIN < VOUT ? VIN : VOUT;     // elements per lane per step
    if (src < 0) {
        for (int c = lane * V; c < C; c += 32 * V)
#pragma unroll
            for (int i = 0; i < V; ++i) dst[c + i] = from_f32<TAct>(0.0f);
        return;
    }
    const TIn* s = x + (size_t)(src / k) * C;
    if constexpr (sizeof(TIn) == sizeof(TAct)) {
        const uint4* s4 = reinterpret_cast<const uint4*>(s);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        const int n4 = C / VIN;
        for (int i = lane; i < n4; i += 32) d4[i] = s4[i];
        for (int c = n4 * VIN + lane; c < C; c += 32) dst[c] = from_f32<TAct>(to_f32(s[c]));
    } else {
        for (int c = lane; c < C; c += 32) dst[c] = from_f32<TAct>(to_f32(s[c]));
    }
}

// 8 consecutive elements <-> 8 floats (16 bytes of bf16, 32 bytes of float)
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8])
{
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8])
{
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8])
{
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<bf16>(bf16* p, const float (&v)[8])
{
    uint4 u;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(p) = u;
}

// y[tok,:] = sum_j p[tok,j] * Yg[pos(tok,j),:], slots visited in ascending order
// like the reference's scatter-add.  One warp per token, 8 channels per lane per step; K = top-k rounded up
// to a power of two, so the sort is a fixed network and the kernel fits 32 registers (all 64 warps resident).
template <typename TAct, typename TIo, int K>
__global__ void __launch_bounds__(256, 8)
combine_fwd_kernel(const TAct* __restrict__ Yg, const int32_t* __restrict__ pos, const float* __restrict__ top_p,
                   int N, int C, int k, const TIo* __restrict__ residual, TIo* __restrict__ y)
{
    const int lane = threadIdx.x & 31;
    const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= N) return;
    int ps[K];
    float pr[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
        ps[j] = j < k ? pos[(size_t)tok * k + j] : 0x7fffffff;
        pr[j] = j < k ? top_p[(size_t)tok * k + j] : 0.0f;
    }
#pragma unroll
    for (int a = 0; a < K - 1; ++a)                 // tiny sorting network (bubble), static indices
#pragma unroll
        for (int b = 0; b < K - 1 - a; ++b)
            if (ps[b] > ps[b + 1]) {
                int ti = ps[b]; ps[b] = ps[b + 1]; ps[b + 1] = ti;
                float tf = pr[b]; pr[b] = pr[b + 1]; pr[b + 1] = tf;
            }
    for (int c = lane * 8; c < C; c += 256) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < K; ++j) {
            if (j < k) {
                float v[8];
                load8(Yg + (size_t)ps[j] * C + c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(v[i], pr[j]));
            }
        }
        if (residual) {                 // y = residual + moe(x): the block's skip connection (TransformerBlock.cpp:44)
            float r[8];
            load8(residual + (size_t)tok * C + c, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(r[i], acc[i]);
        }
        store8(y + (size_t)tok * C + c, acc);
    }
}

// dYg[p,:] = p * dy[tok,:],  d_top_p[flat] = <Yg[p,:], dy[tok,:]>; padding rows -> 0.
template <typename TAct, typename TIo>
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const TIo* __restrict__ dy, const TAct* __restrict__ Yg, const int32_t* __restrict__ row_src,
                   const float* __restrict__ top_p, const int32_t* __restrict__ n_tiles, int fixed_rows, int C, int k,
                   TAct* __restrict__ dYg, float* __restrict__ d_top_p)
{
    const int lane = threadIdx.x & 31;
    const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (p >= (fixed_rows >= 0 ? fixed_rows : *n_tiles * ROW_TILE)) return;
    const int src = row_src[p];
    TAct* dst = dYg + (size_t)p * C;
    if (src < 0) {
        const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = lane * 8; c < C; c += 256) store8(dst + c, z);
        return;
    }
    const float prob = top_p[src];
    const TIo* g = dy + (size_t)(src / k) * C;
    const TAct* yg = Yg + (size_t)p * C;
    float dot = 0.0f;
    for (int c = lane * 8; c < C; c += 256) {
        float gv[8], yv[8], o[8];
        load8(g + c, gv);
        load8(yg + c, yv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i] = __fmul_rn(gv[i], prob);
            dot = fmaf(yv[i], gv[i], dot);
        }
        store8(dst + c, o);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) d_top_p[src] = dot;
}

// Column sums over each expert's rows, for the three bias gradients in one launch:
// gbd[e] += colsum(dYg), gbg[e] += colsum(dG), gbu[e] += colsum(dU)  (layers/LinearLayer.cpp:56-57).
// One CTA = one 128-row tile (one expert) x 256 columns; a thread reads 8 columns (16 bytes) of
// every 8th row, the 8 row lanes are folded in shared memory, then one atomicAdd per column.
struct BiasGradArgs {
    const void* M[3];
    float* const* gb[3];
    int cols[3];
    const int32_t* tile_expert;
    const int32_t* n_tiles;
};

template <typename TAct>
__global__ void __launch_bounds__(256) bias_grad_kernel(BiasGradArgs a)
{
    __shared__ float red[8][256 + 8];
    const int tile = blockIdx.x, which = blockIdx.z;
    if (tile >= *a.n_tiles) return;
    const int cols = a.cols[which];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.y * 256 + tx * 8;
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (c < cols) {
        const TAct* base = (const TAct*)a.M[which] + (size_t)tile * ROW_TILE * cols + c;
#pragma unroll 4
        for (int r = ty; r < ROW_TILE; r += 8) {
            const TAct* p = base + (size_t)r * cols;
            if constexpr (sizeof(TAct) == 2) {
                const uint4 u = *reinterpret_cast<const uint4*>(p);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[2 * i] += __uint_as_float(w[i] << 16);
                    s[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
                }
            } else {
                const float4 f0 = *reinterpret_cast<const float4*>(p), f1 = *reinterpret_cast<const float4*>(p + 4);
                s[0] += f0.x; s[1] += f0.y; s[2] += f0.z; s[3] += f0.w;
                s[4] += f1.x; s[5] += f1.y; s[6] += f1.z; s[7] += f1.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[ty][tx * 8 + i] = s[i];
    __syncthreads();
    const int col = blockIdx.y * 256 + threadIdx.x;
    if (col < cols) {
        float t = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) t += red[r][threadIdx.x];
        atomicAdd(&a.gb[which][a.tile_expert[tile]][col], t);
    }
}

}  // namespace

// The three plan kernels on explicit buffers.  `blk` is scratch of plan_blocks*E ints:
// every element is written by plan_count_kernel before it is read, so it needs no clearing.
int run_plan(const int32_t* top_idx, int R, int E, int32_t* counts, int32_t* offsets, int32_t* padded_offsets,
             int32_t* tile_expert, int32_t* n_tiles, int max_tiles, int32_t* map, int32_t* pos,
             int32_t* row_src, int row_cap, int32_t* status, int32_t* blk, cudaStream_t st, int32_t* slot_of,
             int32_t* sticky, int32_t* pairs, int32_t* n_pairs)
{
    const int plan_blocks = R > 0 ? (R + PLAN_BLOCK - 1) / PLAN_BLOCK : 1;
    if (R <= PLAN_BLOCK) {
        plan_small_kernel<<<1, PLAN_BLOCK, 0, st>>>(top_idx, R, E, counts, offsets, padded_offsets, tile_expert, n_tiles,
                                                    max_tiles, map, pos, row_src, slot_of, status, sticky, pairs, n_pairs);
        MGPT_LAUNCHED("plan_small_kernel");
        return 0;
    }
    (void)row_cap;      // rows beyond the plan's tiles are never read; padding rows are marked by plan_assign_kernel
    plan_count_kernel<<<plan_blocks, PLAN_BLOCK, 0, st>>>(top_idx, R, E, blk);
    MGPT_LAUNCHED("plan_count_kernel");
    plan_scan_kernel<<<1, MAX_EXPERTS, 0, st>>>(blk, plan_blocks, E, counts, offsets, padded_offsets, tile_expert,
                                                n_tiles, max_tiles, status, sticky, pairs, n_pairs);
    MGPT_LAUNCHED("plan_scan_kernel");
    plan_assign_kernel<<<plan_blocks, PLAN_BLOCK, 0, st>>>(top_idx, R, E, blk, counts, offsets, padded_offsets, map, pos,
                                                           row_src, slot_of, status, sticky);
    MGPT_LAUNCHED("plan_assign_kernel");
    return 0;
}

int launch_plan(const Dims& d, const Workspace& w, char* ws, cudaStream_t st, int32_t* sticky)
{
    return run_plan((const int32_t*)(ws + w.top_idx), w.R, d.E, (int32_t*)(ws + w.counts), (int32_t*)(ws + w.offsets),
                    (int32_t*)(ws + w.padded_offsets), (int32_t*)(ws + w.tile_expert), (int32_t*)(ws + w.n_tiles),
                    w.max_tiles, (int32_t*)(ws + w.map), (int32_t*)(ws + w.pos), (int32_t*)(ws + w.row_src),
                    w.row_cap, (int32_t*)(ws + w.status), (int32_t*)(ws + w.blk_cnt), st, (int32_t*)(ws + w.slot), sticky,
                    (int32_t*)(ws + w.pairs), (int32_t*)(ws + w.n_pairs));
}

// dst[p,:] = src[row_src[p]/k,:] for p < rows (zero where row_src[p] < 0).  rows < 0: every tile of the plan.
int gather_rows(const void* src, int src_io, const int32_t* row_src, const int32_t* n_tiles, int rows, int grid_rows,
                int C, int k, void* dst, size_t act_bytes, cudaStream_t st)
{
    if (grid_rows <= 0) return 0;
    const int grid = (grid_rows + 7) / 8;
    if (act_bytes == 4) {
        if (src_io != MGPT_MOE_IO_F32) return fail(MGPT_MOE_EINVAL, "FP32 mode takes FP32 rows");
        dispatch_rows_kernel<float, float><<<grid, 256, 0, st>>>((const float*)src, row_src, n_tiles, rows, C, k, (float*)dst);
    } else if (src_io == MGPT_MOE_IO_F32) {
        dispatch_rows_kernel<float, bf16><<<grid, 256, 0, st>>>((const float*)src, row_src, n_tiles, rows, C, k, (bf16*)dst);
    } else {
        dispatch_rows_kernel<bf16, bf16><<<grid, 256, 0, st>>>((const bf16*)src, row_src, n_tiles, rows, C, k, (bf16*)dst);
    }
    MGPT_LAUNCHED("dispatch_rows_kernel");
    return 0;
}

int launch_dispatch(const Dims& d, const Workspace& w, char* ws, const void* x, int io, cudaStream_t st)
{
    return gather_rows(x, io, (const int32_t*)(ws + w.row_src), (const int32_t*)(ws + w.n_tiles), -1, w.row_cap, d.C, d.k,
                       ws + w.Xg, w.act_bytes, st);
}

// y = weighted gather-sum of rows[pos[tok,j]]
int combine_rows(const void* rows, const int32_t* pos, const float* top_p, int N, int C, int k, void* y, int io,
                 size_t act_bytes, cudaStream_t st, const void* residual)
{
    if (N <= 0) return 0;
    const int grid = (N + 7) / 8;
#define MGPT_COMBINE(KK)                                                                                                  \
    do {                                                                                                                  \
        if (act_bytes == 4)                                                                                               \
            combine_fwd_kernel<float, float, KK><<<grid, 256, 0, st>>>((const float*)rows, pos, top_p, N, C, k, (const float*)residual, (float*)y); \
        else if (io == MGPT_MOE_IO_F32)                                                                                   \
            combine_fwd_kernel<bf16, float, KK><<<grid, 256, 0, st>>>((const bf16*)rows, pos, top_p, N, C, k, (const float*)residual, (float*)y); \
        else                                                                                                              \
            combine_fwd_kernel<bf16, bf16, KK><<<grid, 256, 0, st>>>((const bf16*)rows, pos, top_p, N, C, k, (const bf16*)residual, (bf16*)y);   \
    } while (0)
    if (k <= 1) MGPT_COMBINE(1);
    else if (k <= 2) MGPT_COMBINE(2);
    else if (k <= 4) MGPT_COMBINE(4);
    else MGPT_COMBINE(8);
#undef MGPT_COMBINE
    MGPT_LAUNCHED("combine_fwd_kernel");
    return 0;
}

int launch_combine_fwd(const Dims& d, const Workspace& w, char* ws, void* y, int io, cudaStream_t st, const void* residual)
{
    return combine_rows(ws + w.Yg, (const int32_t*)(ws + w.pos), (const float*)(ws + w.top_p), w.n_tokens, d.C, d.k, y,
                        io, w.act_bytes, st, residual);
}

// d_rows[p] = top_p * dy[tok], d_top_p[flat] = <rows[p], dy[tok]> for p < rows (rows < 0: every tile of the plan)
int combine_rows_backward(const void* dy, int io, const void* rows, const int32_t* row_src, const float* top_p,
                          const int32_t* n_tiles, int n_rows, int grid_rows, int C, int k, void* d_rows, float* d_top_p,
                          size_t act_bytes, cudaStream_t st)
{
    if (grid_rows <= 0) return 0;
    const int grid = (grid_rows + 7) / 8;
    if (act_bytes == 4)
        combine_bwd_kernel<float, float><<<grid, 256, 0, st>>>((const float*)dy, (const float*)rows, row_src, top_p,
                                                               n_tiles, n_rows, C, k, (float*)d_rows, d_top_p);
    else if (io == MGPT_MOE_IO_F32)
        combine_bwd_kernel<bf16, float><<<grid, 256, 0, st>>>((const float*)dy, (const bf16*)rows, row_src, top_p,
                                                              n_tiles, n_rows, C, k, (bf16*)d_rows, d_top_p);
    else
        combine_bwd_kernel<bf16, bf16><<<grid, 256, 0, st>>>((const bf16*)dy, (const bf16*)rows, row_src, top_p,
                                                             n_tiles, n_rows, C, k, (bf16*)d_rows, d_top_p);
    MGPT_LAUNCHED("combine_bwd_kernel");
    return 0;
}

int launch_combine_bwd(const Dims& d, const Workspace& w, char* ws, const void* dy, int io, cudaStream_t st)
{
    return combine_rows_backward(dy, io, ws + w.Yg, (const int32_t*)(ws + w.row_src), (const float*)(ws + w.top_p),
                                 (const int32_t*)(ws + w.n_tiles), -1, w.row_cap, d.C, d.k, ws + w.dYg,
                                 (float*)(ws + w.d_top_p), w.act_bytes, st);
}

int launch_bias_grads(const mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    const Dims& d = L->d;
    BiasGradArgs a;
    a.M[0] = buf_dYg(L, w, ws); a.M[1] = ws + w.dG; a.M[2] = ws + w.dU;
    a.gb[0] = L->master.gbd; a.gb[1] = L->master.gbg; a.gb[2] = L->master.gbu;
    a.cols[0] = d.C; a.cols[1] = d.H; a.cols[2] = d.H;
    a.tile_expert = (const int32_t*)(ws + w.tile_expert);
    a.n_tiles = (const int32_t*)(ws + w.n_tiles);
    const int mc = d.C > d.H ? d.C : d.H;
    dim3 grid(w.max_tiles, (mc + 255) / 256, 3);
    if (w.act_bytes == 4) bias_grad_kernel<float><<<grid, 256, 0, st>>>(a);
    else bias_grad_kernel<bf16><<<grid, 256, 0, st>>>(a);
    MGPT_LAUNCHED("bias_grad_kernel");
    return 0;
}

// Expert side of an expert-parallel layer: rows arrive as one block per source rank, inside it one
// 128-row-padded segment per local expert.  From the [n_src][E] real row counts this builds the tile ->
// expert table in arrival order, the per-expert segment list {first row, padded rows} and the totals.
__global__ void __launch_bounds__(256)
segment_tiles_kernel(const int32_t* __restrict__ seg_counts, int n_src, int E, int32_t* __restrict__ counts,
                     int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_order,
                     int32_t* __restrict__ n_tiles, int max_tiles, int32_t* __restrict__ seg,
                     int32_t* __restrict__ status, int32_t* __restrict__ sticky,
                     int32_t* __restrict__ pairs, int32_t* __restrict__ n_pairs)
{
    __shared__ int first_tile[MAX_SEGMENTS + 1];     // in arrival order (s, e)
    __shared__ int first_item[MAX_SEGMENTS];         // in processing order (e, s)
    __shared__ int pair0[MAX_EXPERTS + 1];
    __shared__ int item0[MAX_EXPERTS + 1];           // first position of an expert in the processing order
    const int n = n_src * E;
    if (threadIdx.x == 0) {
        int t = 0;
        for (int i = 0; i < n; ++i) {            // i = s*E + e, arrival order
            first_tile[i] = t;
            t += (seg_counts[i] + ROW_TILE - 1) / ROW_TILE;
        }
        first_tile[n] = t;
        *n_tiles = t;
        *status = t > max_tiles ? ST_PLAN_OVERFLOW : 0;
        if (sticky && t > max_tiles) atomicOr(sticky, ST_PLAN_OVERFLOW);
        int it = 0, np = 0;
        for (int e = 0; e < E; ++e) {
            item0[e] = it;
            pair0[e] = np;
            for (int s_ = 0; s_ < n_src; ++s_) {
                first_item[e * n_src + s_] = it;
                it += (seg_counts[s_ * E + e] + ROW_TILE - 1) / ROW_TILE;
            }
            np += (it - item0[e] + 1) / 2;
        }
        item0[E] = it;
        pair0[E] = np;
        *n_pairs = np;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int s_ = i / E, e = i % E;
        const int t0 = first_tile[i], t1 = first_tile[i + 1];
        seg[(e * n_src + s_) * 2] = t0 * ROW_TILE;
        seg[(e * n_src + s_) * 2 + 1] = (t1 - t0) * ROW_TILE;
        const int o0 = first_item[e * n_src + s_];
        for (int t = t0; t < t1 && t < max_tiles; ++t) {
            tile_expert[t] = e;
            // tiles are worked on expert after expert (one expert's weights stay in L2), wherever they landed
            if (o0 + (t - t0) < max_tiles) tile_order[o0 + (t - t0)] = t;
        }
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int s_ = 0; s_ < n_src; ++s_) c += seg_counts[s_ * E + e];
        counts[e] = c;
    }
    __syncthreads();        // tile_order is complete (written above by this block)
    // pairs of tiles of one expert, in processing order (the two tiles may have arrived from different sources)
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int pi = pair0[e];
        for (int i = item0[e]; i < item0[e + 1] && i < max_tiles; i += 2, ++pi) {
            pairs[2 * pi] = tile_order[i];
            pairs[2 * pi + 1] = (i + 1 < item0[e + 1] && i + 1 < max_tiles) ? tile_order[i + 1] : -1;
        }
    }
}

int launch_segment_tiles(const Dims& d, const Workspace& w, char* ws, const int32_t* seg_counts, int n_src, cudaStream_t st,
                         int32_t* sticky)
{
    if (n_src * d.E > MAX_SEGMENTS) return fail(MGPT_MOE_EINVAL, "sources x local experts must not exceed 4096");
    segment_tiles_kernel<<<1, 256, 0, st>>>(seg_counts, n_src, d.E, (int32_t*)(ws + w.counts),
                                            (int32_t*)(ws + w.tile_expert), (int32_t*)(ws + w.tile_order),
                                            (int32_t*)(ws + w.n_tiles), w.max_tiles, (int32_t*)(ws + w.seg),
                                            (int32_t*)(ws + w.status), sticky, (int32_t*)(ws + w.pairs),
                                            (int32_t*)(ws + w.n_pairs));
    MGPT_LAUNCHED("segment_tiles_kernel");
    return 0;
}

static int check_plan_args(const int32_t* top_idx, int n_rows, int E, const void* const* outs, int n_outs,
                           int row_cap)
{
    if (!top_idx) return fail(MGPT_MOE_EINVAL, "null top_idx");
    for (int i = 0; i < n_outs; ++i)
        if (!outs[i]) return fail(MGPT_MOE_EINVAL, "null output buffer");
    if (E <= 0 || E > MAX_EXPERTS) return fail(MGPT_MOE_EINVAL, "num_experts must be in 1..128");
    if (n_rows < 0) return fail(MGPT_MOE_EINVAL, "negative row count");
    const long long need = ((long long)n_rows + (long long)E * (ROW_TILE - 1)) / ROW_TILE * ROW_TILE;
    if (row_cap < need || row_cap % ROW_TILE) return fail(MGPT_MOE_EINVAL, "row_cap too small or not a multiple of 128");
    return 0;
}

}  // namespace mgpt

using namespace mgpt;

extern "C" size_t mgpt_moe_op_plan_scratch_bytes(int n_rows, int E)
{
    if (n_rows < 0 || E <= 0) return 0;
    const size_t blocks = n_rows > 0 ? ((size_t)n_rows + PLAN_BLOCK - 1) / PLAN_BLOCK : 1;
    return blocks * (size_t)E * sizeof(int32_t);
}

extern "C" int mgpt_moe_op_plan(const int32_t* top_idx, int n_rows, int E, int32_t* counts, int32_t* offsets,
                                int32_t* padded_offsets, int32_t* tile_expert, int32_t* n_tiles, int32_t* map,
                                int32_t* pos, int32_t* row_src, int row_cap, int32_t* status, void* scratch,
                                size_t scratch_bytes, mgpt_stream_t stream)
{
    const void* outs[] = {counts, offsets, padded_offsets, tile_expert, n_tiles, map, pos, row_src, status, scratch};
    MGPT_TRY(check_plan_args(top_idx, n_rows, E, outs, 10, row_cap));
    if (scratch_bytes < mgpt_moe_op_plan_scratch_bytes(n_rows, E))
        return fail(MGPT_MOE_ENOMEM, "scratch smaller than mgpt_moe_op_plan_scratch_bytes()");
    return run_plan(top_idx, n_rows, E, counts, offsets, padded_offsets, tile_expert, n_tiles, row_cap / ROW_TILE, map,
                    pos, row_src, row_cap, status, (int32_t*)scratch, (cudaStream_t)stream, nullptr, nullptr, nullptr, nullptr);
}

// ---- dispatch plan without any allocation ------------------------------------------
// Some callers cannot give the plan scratch memory of their own and cannot let the
// library allocate it either: an engine that has already handed all device memory to
// its own arena (the reference sizes its Scratchpad from a footprint predictor and
// leaves nothing over), or a step loop that must not meet cudaMalloc's device-wide
// synchronisation.  For them the per-block histogram lives in a fixed array inside the
// library image.  Every GPU that loads the library holds these 512 KiB until exit.
#define PLAN_STATIC_BLOCKS (MGPT_MOE_PLAN_NOALLOC_MAX_ROWS / 1024)
static __device__ __align__(256) int32_t g_plan_scratch[PLAN_STATIC_BLOCKS * mgpt::MAX_EXPERTS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
int32_t* g_scratch_dev_ptr[kMaxDevices] = {};   // device address of g_plan_scratch, per device

// In host code `g_plan_scratch` names a host-side shadow, not device memory; the
// address a kernel may use has to be asked for, on the device that will run it.
int plan_static_scratch(int32_t** out)
{
    int dev = -1;
    MGPT_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(MGPT_MOE_EINVAL, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_dev_ptr[dev]) {
        void* p = nullptr;
        MGPT_CUDA(cudaGetSymbolAddress(&p, g_plan_scratch));
        if (!p) return fail(MGPT_MOE_ECUDA, "cudaGetSymbolAddress returned a null address");
        g_scratch_dev_ptr[dev] = (int32_t*)p;
    }
    *out = g_scratch_dev_ptr[dev];
    return 0;
}
}  // namespace

extern "C" int mgpt_moe_op_plan_noalloc(const int32_t* top_idx, int n_rows, int E, int32_t* counts, int32_t* offsets,
                                        int32_t* padded_offsets, int32_t* tile_expert, int32_t* n_tiles,
                                        int32_t* map, int32_t* pos, int32_t* row_src, int row_cap, int32_t* status,
                                        mgpt_stream_t stream)
{
    if (n_rows > MGPT_MOE_PLAN_NOALLOC_MAX_ROWS)
        return fail(MGPT_MOE_EINVAL, "mgpt_moe_op_plan_noalloc handles at most " +
                                         std::to_string(MGPT_MOE_PLAN_NOALLOC_MAX_ROWS) + " routed rows, got " +
                                         std::to_string(n_rows) + "; use mgpt_moe_op_plan with your own scratch");
    const void* outs[] = {counts, offsets, padded_offsets, tile_expert, n_tiles, map, pos, row_src, status};
    MGPT_TRY(check_plan_args(top_idx, n_rows, E, outs, 9, row_cap));
    int32_t* scratch = nullptr;
    MGPT_TRY(plan_static_scratch(&scratch));
    // The array still holds the previous call's block bases.  Nothing has to be cleared:
    // plan_count_kernel writes all plan_blocks*E entries this call reads before they are read.
    return run_plan(top_idx, n_rows, E, counts, offsets, padded_offsets, tile_expert, n_tiles, row_cap / ROW_TILE, map,
                    pos, row_src, row_cap, status, scratch, (cudaStream_t)stream, nullptr, nullptr, nullptr, nullptr);
}
