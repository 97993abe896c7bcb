// BF16 weight shadows of the expert projections.
//
// The engine keeps FP32 masters (Tensor::cuda_data) for AdamW and checkpoints
// (optimisers/AdamWOptimiser.h:24-36, GPT.cpp:128-206); the tensor-core
// products read BF16 copies.  Each weight is kept twice, as stored and
// transposed, so that every product finds its reduction dimension contiguous:
//   forward  gate/up : B = Wg^T, Wu^T [H,C]     forward down : B = Wd^T [C,H]
//   dHh = dYg*Wd^T   : B = Wd [H,C]             dXg          : B = Wg, Wu [C,H]
#include "common.cuh"

namespace mgpt {

namespace {

// One 32x32 tile per block: dst[r,c] = src[r,c] (bf16) and dstT[c,r] = src[r,c].
__global__ void __launch_bounds__(256)
shadow_kernel(const void* const* __restrict__ src_ptrs, int rows, int cols,
              bf16* __restrict__ dst, bf16* __restrict__ dstT)
{
    __shared__ float tile[32][33];
    const int e = blockIdx.z;
    const float* src = (const float*)src_ptrs[e];
    bf16* d = dst + (size_t)e * rows * cols;
    bf16* dT = dstT + (size_t)e * tile_major_elems(cols, rows);       // the transposed matrix is [cols, rows]
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + tx;
        if (r < rows && c < cols) {
            const float v = src[(size_t)r * cols + c];
            tile[i][tx] = v;
            d[(size_t)r * cols + c] = __float2bfloat16(v);
        }
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + tx;
        if (r < rows && c < cols) dT[tile_major_index(rows, c, r)] = __float2bfloat16(tile[tx][i]);
    }
}

// Wr [C,E] fp32 -> [C,E8] bf16, zero in the padding columns
__global__ void __launch_bounds__(256)
router_shadow_kernel(const float* __restrict__ Wr, int C, int E, int E8, bf16* __restrict__ out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= C * E8) return;
    const int c = i / E8, e = i % E8;
    out[i] = __float2bfloat16(e < E ? Wr[(size_t)c * E + e] : 0.0f);
}

}  // namespace

// After an optimiser step that wrote the expert copies itself: only the router's padded BF16 copy is rebuilt.
int launch_sync_router_only(mgpt_moe_layer* L, cudaStream_t st)
{
    const Dims& d = L->d;
    if (d.mode == MGPT_MOE_BF16 && L->router_bound) {
        const int E8 = (d.E + 7) / 8 * 8;
        router_shadow_kernel<<<(d.C * E8 + 255) / 256, 256, 0, st>>>(L->p_data[0], d.C, d.E, E8, L->sWr);
        MGPT_LAUNCHED("router_shadow_kernel");
        MGPT_TRY(launch_router_pieces(L, st));
    }
    L->shadows_fresh = true;
    return 0;
}

int launch_sync_weights(mgpt_moe_layer* L, cudaStream_t st)
{
    const Dims& d = L->d;
    if (d.mode != MGPT_MOE_BF16) return 0;
    if (L->router_bound) {
        const int E8 = (d.E + 7) / 8 * 8;
        router_shadow_kernel<<<(d.C * E8 + 255) / 256, 256, 0, st>>>(L->p_data[0], d.C, d.E, E8, L->sWr);
        MGPT_LAUNCHED("router_shadow_kernel");
        MGPT_TRY(launch_router_pieces(L, st));
    }
    if (!L->experts_bound) {
        L->shadows_fresh = true;
        return 0;
    }
    dim3 gCH((d.H + 31) / 32, (d.C + 31) / 32, d.E), gHC((d.C + 31) / 32, (d.H + 31) / 32, d.E);
    shadow_kernel<<<gCH, 256, 0, st>>>(L->master.Wg, d.C, d.H, L->sWg, L->sWgT);
    MGPT_LAUNCHED("shadow_kernel<Wg>");
    shadow_kernel<<<gCH, 256, 0, st>>>(L->master.Wu, d.C, d.H, L->sWu, L->sWuT);
    MGPT_LAUNCHED("shadow_kernel<Wu>");
    shadow_kernel<<<gHC, 256, 0, st>>>(L->master.Wd, d.H, d.C, L->sWd, L->sWdT);
    MGPT_LAUNCHED("shadow_kernel<Wd>");
    L->shadows_fresh = true;
    return 0;
}

}  // namespace mgpt
