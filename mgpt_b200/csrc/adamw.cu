// AdamW over the layer's own parameters, fused with the refresh of the BF16 weight copies.
//
// The reference's optimiser calls Tensor::adamw_step once per parameter tensor
// (optimisers/AdamWOptimiser.h:24-36; CPU arithmetic utils/Tensor.cpp:683-699, GPU kernel
// utils/cuda_ops.cu:723-738) and the tensor-core products would then need a separate pass that
// re-reads every FP32 master to rebuild its two BF16 copies.  Here one launch per kind of
// tensor updates w, m, v for all experts and writes both copies from the value it just
// computed, so an optimiser step costs the AdamW traffic plus 4 bytes per weight.
//
// Arithmetic: the CPU arm's, operation for operation (separate FP32 roundings, IEEE sqrt and
// divide), so w, m, v match the reference bit for bit:
//   m = b1*m + (1-b1)*g;  v = b2*v + ((1-b2)*g)*g;  w = w - (lr*wd)*w;
//   w = w - (lr*(m*ms)) / (sqrt(v*vs) + eps),   ms = 1/(1-b1^t), vs = 1/(1-b2^t)  (host, powf)
#include <cmath>

#include "common.cuh"

namespace mgpt {

namespace {

struct AdamwScalars {
    float b1, b2, omb1, omb2, eps, lr, lrwd, ms, vs;
    float clip;       // > 0: the gradient is clamped to [-clip, clip] first (the GPU arm's 10, utils/cuda_ops.cu:728)
    int skip_bad;     // != 0: an element whose gradient is NaN or Inf is left as it is (utils/cuda_ops.cu:727)
};

__device__ __forceinline__ void adamw_elem(float& w, float g, float& m, float& v, const AdamwScalars& a)
{
    if (a.skip_bad && !isfinite(g)) return;
    if (a.clip > 0.0f) g = fminf(fmaxf(g, -a.clip), a.clip);
    m = __fadd_rn(__fmul_rn(a.b1, m), __fmul_rn(a.omb1, g));
    v = __fadd_rn(__fmul_rn(a.b2, v), __fmul_rn(__fmul_rn(a.omb2, g), g));
    const float mh = __fmul_rn(m, a.ms), vh = __fmul_rn(v, a.vs);
    w = __fsub_rn(w, __fmul_rn(a.lrwd, w));
    w = __fsub_rn(w, __fdiv_rn(__fmul_rn(a.lr, mh), __fadd_rn(__fsqrt_rn(vh), a.eps)));
}

// One 32x32 tile of one expert's [rows, cols] matrix per block: AdamW in place, then
// dst[r,c] = bf16(w) and dstT[c,r] = bf16(w) (both optional: FP32 mode keeps no copies).
__global__ void __launch_bounds__(256)
adamw_matrix_kernel(float* const* __restrict__ w_ptrs, const float* const* __restrict__ g_ptrs,
                    float* const* __restrict__ m_ptrs, float* const* __restrict__ v_ptrs, int rows, int cols,
                    bf16* __restrict__ dst, bf16* __restrict__ dstT, const AdamwScalars a)
{
    __shared__ float tile[32][33];
    const int e = blockIdx.z;
    float* w = w_ptrs[e];
    const float* g = g_ptrs[e];
    float* m = m_ptrs[e];
    float* v = v_ptrs[e];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + tx;
        if (r < rows && c < cols) {
            const size_t o = (size_t)r * cols + c;
            float wv = w[o], mv = m[o], vv = v[o];
            adamw_elem(wv, g[o], mv, vv, a);
            w[o] = wv; m[o] = mv; v[o] = vv;
            tile[i][tx] = wv;
            if (dst) dst[(size_t)e * rows * cols + o] = __float2bfloat16(wv);
        }
    }
    if (!dstT) return;
    __syncthreads();
#pragma unroll
    for (int i = ty; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + tx;
        if (r < rows && c < cols)       // the transposed copy [cols, rows] is tile-major (common.cuh)
            dstT[(size_t)e * tile_major_elems(cols, rows) + tile_major_index(rows, c, r)] = __float2bfloat16(tile[tx][i]);
    }
}

// Flat tensors of one length: blockIdx.y selects the tensor (one expert's bias, or the single router tensor).
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* const* __restrict__ w_ptrs, const float* const* __restrict__ g_ptrs,
                  float* const* __restrict__ m_ptrs, float* const* __restrict__ v_ptrs, int len, const AdamwScalars a)
{
    const int e = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= len) return;
    float wv = w_ptrs[e][i], mv = m_ptrs[e][i], vv = v_ptrs[e][i];
    adamw_elem(wv, g_ptrs[e][i], mv, vv, a);
    w_ptrs[e][i] = wv; m_ptrs[e][i] = mv; v_ptrs[e][i] = vv;
}

}  // namespace

int launch_adamw(mgpt_moe_layer* L, float lr, float beta1, float beta2, float eps, float weight_decay, int t,
                 cudaStream_t st, float grad_clip, int skip_nonfinite)
{
    const Dims& d = L->d;
    AdamwScalars a;
    a.b1 = beta1; a.b2 = beta2; a.omb1 = 1.0f - beta1; a.omb2 = 1.0f - beta2; a.eps = eps; a.lr = lr;
    a.lrwd = lr * weight_decay;
    a.ms = 1.0f / (1.0f - std::pow(beta1, (float)t));
    a.vs = 1.0f / (1.0f - std::pow(beta2, (float)t));
    a.clip = grad_clip;
    a.skip_bad = skip_nonfinite;
    void** tab = (void**)L->d_opt;     // [m: Wg Wu Wd bg bu bd | v: same | router: w g m v for Wr, br][E]
    const int E = d.E, S = E < 2 ? 2 : E;          // table stride (the router rows hold two entries)
    auto T = [&](int i) { return tab + (size_t)i * S; };
    const bool bf = d.mode == MGPT_MOE_BF16;
    if (L->experts_bound) {
        dim3 gCH((d.H + 31) / 32, (d.C + 31) / 32, E), gHC((d.C + 31) / 32, (d.H + 31) / 32, E);
        adamw_matrix_kernel<<<gCH, 256, 0, st>>>((float* const*)L->master.Wg, (const float* const*)L->master.gWg,
                                                 (float* const*)T(0), (float* const*)T(6), d.C, d.H,
                                                 bf ? L->sWg : nullptr, bf ? L->sWgT : nullptr, a);
        MGPT_LAUNCHED("adamw_matrix_kernel<Wg>");
        adamw_matrix_kernel<<<gCH, 256, 0, st>>>((float* const*)L->master.Wu, (const float* const*)L->master.gWu,
                                                 (float* const*)T(1), (float* const*)T(7), d.C, d.H,
                                                 bf ? L->sWu : nullptr, bf ? L->sWuT : nullptr, a);
        MGPT_LAUNCHED("adamw_matrix_kernel<Wu>");
        adamw_matrix_kernel<<<gHC, 256, 0, st>>>((float* const*)L->master.Wd, (const float* const*)L->master.gWd,
                                                 (float* const*)T(2), (float* const*)T(8), d.H, d.C,
                                                 bf ? L->sWd : nullptr, bf ? L->sWdT : nullptr, a);
        MGPT_LAUNCHED("adamw_matrix_kernel<Wd>");
        adamw_flat_kernel<<<dim3((d.H + 255) / 256, E), 256, 0, st>>>((float* const*)L->master.bg, (const float* const*)L->master.gbg,
                                                                      (float* const*)T(3), (float* const*)T(9), d.H, a);
        MGPT_LAUNCHED("adamw_flat_kernel<bg>");
        adamw_flat_kernel<<<dim3((d.H + 255) / 256, E), 256, 0, st>>>((float* const*)L->master.bu, (const float* const*)L->master.gbu,
                                                                      (float* const*)T(4), (float* const*)T(10), d.H, a);
        MGPT_LAUNCHED("adamw_flat_kernel<bu>");
        adamw_flat_kernel<<<dim3((d.C + 255) / 256, E), 256, 0, st>>>((float* const*)L->master.bd, (const float* const*)L->master.gbd,
                                                                      (float* const*)T(5), (float* const*)T(11), d.C, a);
        MGPT_LAUNCHED("adamw_flat_kernel<bd>");
    }
    if (L->router_bound) {
        // router tables: rows 12..15 hold {w, g, m, v}, entry 0 = Wr, entry 1 = br
        float* const* rw = (float* const*)T(12);
        const float* const* rg = (const float* const*)T(13);
        float* const* rm = (float* const*)T(14);
        float* const* rv = (float* const*)T(15);
        adamw_flat_kernel<<<dim3((d.C * E + 255) / 256, 1), 256, 0, st>>>(rw, rg, rm, rv, d.C * E, a);
        MGPT_LAUNCHED("adamw_flat_kernel<Wr>");
        adamw_flat_kernel<<<dim3((E + 255) / 256, 1), 256, 0, st>>>(rw + 1, rg + 1, rm + 1, rv + 1, E, a);
        MGPT_LAUNCHED("adamw_flat_kernel<br>");
    }
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "adamw launch");
    // the copies of the expert weights are current; the router's small BF16 copy is rebuilt from the new Wr
    L->shadows_fresh = false;
    return launch_sync_router_only(L, st);
}

}  // namespace mgpt
