// Grouped expert products on CUDA cores (FP32 accumulate).
//
// This is the FP32 validation mode of the layer (the reference's own dtype,
// parity bar 1e-5) and, with BF16 operands, the cross-check for the tcgen05
// path in gemm_tc.cu.  Same math as the reference's per-expert loop
// (layers/MoELayer.cpp:94-118, 159-181; layers/SwiGLU.cpp:23-50, 57-96;
// layers/LinearLayer.cpp:36-80) but grouped: one launch covers every expert,
// reading the row tiles and the tile->expert table built by the plan.
#include "common.cuh"

namespace mgpt {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16(v); }

// acc[4][4] += A(m0.., 0..K) * B(0..K, n0..) with element (m,k) of A at A[m*sAm + k*sAk]
// and (k,n) of B at B[k*sBk + n*sBn]; out-of-range rows/cols read as zero.
template <typename TA, typename TB>
__device__ __forceinline__ void tile_mac(const TA* __restrict__ A, long sAm, long sAk, int m0, int M,
                                         const TB* __restrict__ B, long sBk, long sBn, int n0, int N,
                                         int K, float (&acc)[4][4], float (*As)[TM + 4], float (*Bs)[TN + 4])
{
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            int m, k;
            if (sAk == 1) { k = idx % TK; m = idx / TK; } else { m = idx % TM; k = idx / TM; }
            const int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? to_f32(A[gm * sAm + gk * sAk]) : 0.0f;
            int n, kb;
            if (sBk == 1) { kb = idx % TK; n = idx / TK; } else { n = idx % TN; kb = idx / TN; }
            const int gn = n0 + n, gkb = k0 + kb;
            Bs[kb][n] = (gn < N && gkb < K) ? to_f32(B[gkb * sBk + gn * sBn]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
}

enum { EPI_GATEUP = 0, EPI_DOWN = 1, EPI_DHH = 2, EPI_DXG = 3 };

struct RowsArgs {
    const void* A;  const void* A2;            // activations [rows, K]
    const void* const* B; const void* const* B2;   // per-expert weights
    const float* const* bias; const float* const* bias2;
    void* D; void* D2; void* D3;               // outputs [rows, Nout]
    const void* G; const void* U;              // saved pre-activations (EPI_DHH)
    const int32_t* tile_expert; const int32_t* n_tiles;
    int K, Nout;
};

template <typename TAct, typename TW, int EPI>
__global__ void __launch_bounds__(256) simt_rows_kernel(RowsArgs a)
{
    __shared__ __align__(16) float As[TK][TM + 4];
    __shared__ __align__(16) float Bs[TK][TN + 4];
    const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    const int rows = *a.n_tiles * ROW_TILE;
    if (m0 >= rows) return;
    const int e = a.tile_expert[m0 / ROW_TILE];
    const int K = a.K, N = a.Nout;
    const TAct* A = (const TAct*)a.A;
    const TW* B = (const TW*)a.B[e];
    float acc[4][4] = {}, acc2[4][4] = {};
    if (EPI == EPI_GATEUP) {           // B = Wg, B2 = Wu, both [K=C, N=H] row-major
        tile_mac(A, (long)K, 1L, m0, rows, B, (long)N, 1L, n0, N, K, acc, As, Bs);
        tile_mac(A, (long)K, 1L, m0, rows, (const TW*)a.B2[e], (long)N, 1L, n0, N, K, acc2, As, Bs);
    } else if (EPI == EPI_DOWN) {      // B = Wd [K=H, N=C]
        tile_mac(A, (long)K, 1L, m0, rows, B, (long)N, 1L, n0, N, K, acc, As, Bs);
    } else if (EPI == EPI_DHH) {       // B(k=c, n=h) = Wd[h*C + c]
        tile_mac(A, (long)K, 1L, m0, rows, B, 1L, (long)K, n0, N, K, acc, As, Bs);
    } else {                           // dXg = dG*Wg^T + dU*Wu^T ; B(k=h, n=c) = W[c*H + h]
        tile_mac(A, (long)K, 1L, m0, rows, B, 1L, (long)K, n0, N, K, acc, As, Bs);
        tile_mac((const TAct*)a.A2, (long)K, 1L, m0, rows, (const TW*)a.B2[e], 1L, (long)K, n0, N, K, acc, As, Bs);
    }
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)m * N + n;
            if (EPI == EPI_GATEUP) {
                // layers/SwiGLU.cpp:32-40, utils/Tensor.cpp:1997-2002
                const float g = acc[i][j] + a.bias[e][n], u = acc2[i][j] + a.bias2[e][n];
                // downstream stages read the stored (rounded) values, so round first
                const TAct gs = from_f32<TAct>(g), us = from_f32<TAct>(u);
                const float gr = to_f32(gs), ur = to_f32(us);
                ((TAct*)a.D)[o] = gs;
                ((TAct*)a.D2)[o] = us;
                ((TAct*)a.D3)[o] = from_f32<TAct>((gr / (1.0f + expf(-gr))) * ur);
            } else if (EPI == EPI_DOWN) {
                ((TAct*)a.D)[o] = from_f32<TAct>(acc[i][j] + a.bias[e][n]);
            } else if (EPI == EPI_DHH) {
                // utils/Tensor.cpp:2020-2027
                const float dd = acc[i][j];
                const float g = to_f32(((const TAct*)a.G)[o]), u = to_f32(((const TAct*)a.U)[o]);
                const float sig = 1.0f / (1.0f + expf(-g));
                ((TAct*)a.D)[o] = from_f32<TAct>((dd * u) * (sig * (1.0f + g * (1.0f - sig))));   // dG
                ((TAct*)a.D2)[o] = from_f32<TAct>(dd * (g * sig));                                 // dU
            } else {
                ((TAct*)a.D)[o] = from_f32<TAct>(acc[i][j]);
            }
        }
    }
}

// grad[e][m,n] += sum over the expert's rows p of A[p,m] * B[p,n]
// (layers/LinearLayer.cpp:60-66: dW = X^T * dOut, accumulated like Tensor::add_grad).
struct WgradArgs {
    const void* A; int lda;      // [rows, M]
    const void* B; int ldb;      // [rows, N]
    float* const* grad;          // per expert [M, N]
    const int32_t* padded_offsets;
    int M, N;
    const int32_t* seg;          // [E][n_seg][2] {first row, rows} when an expert's rows come in several segments
    int n_seg;
};

template <typename TAct>
__global__ void __launch_bounds__(256) simt_wgrad_kernel(WgradArgs a)
{
    __shared__ __align__(16) float As[TK][TM + 4];
    __shared__ __align__(16) float Bs[TK][TN + 4];
    const int e = blockIdx.z;
    const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    float acc[4][4] = {};
    const int nseg = a.n_seg > 0 ? a.n_seg : 1;
    int total = 0;
    for (int sgi = 0; sgi < nseg; ++sgi) {
        const int r0 = a.n_seg > 0 ? a.seg[(e * a.n_seg + sgi) * 2] : a.padded_offsets[e];
        const int len = a.n_seg > 0 ? a.seg[(e * a.n_seg + sgi) * 2 + 1] : a.padded_offsets[e + 1] - r0;
        if (len <= 0) continue;               // uniform over the CTA
        total += len;
        const TAct* A = (const TAct*)a.A + (size_t)r0 * a.lda;
        const TAct* B = (const TAct*)a.B + (size_t)r0 * a.ldb;
        tile_mac(A, 1L, (long)a.lda, m0, a.M, B, (long)a.ldb, 1L, n0, a.N, len, acc, As, Bs);
    }
    if (total == 0) return;
    float* g = a.grad[e];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < a.N) g[(size_t)m * a.N + n] += acc[i][j];
        }
    }
}

template <typename TAct, typename TW>
int experts_forward_t(mgpt_moe_layer* L, const ExpertPtrs& P, const Workspace& w, char* ws, cudaStream_t st)
{
    const Dims& d = L->d;
    RowsArgs a = {};
    a.tile_expert = (const int32_t*)(ws + w.tile_expert);
    a.n_tiles = (const int32_t*)(ws + w.n_tiles);
    // gate/up + SwiGLU
    a.A = buf_Xg(L, w, ws); a.B = P.Wg; a.B2 = P.Wu; a.bias = P.bg; a.bias2 = P.bu;
    a.D = ws + w.G; a.D2 = ws + w.U; a.D3 = ws + w.Hh; a.K = d.C; a.Nout = d.H;
    L->stage_begin(ST_GATEUP, st);
    simt_rows_kernel<TAct, TW, EPI_GATEUP><<<dim3(w.row_cap / TM, (d.H + TN - 1) / TN), 256, 0, st>>>(a);
    MGPT_LAUNCHED("simt_rows_kernel<gateup>");
    L->stage_end(ST_GATEUP, st);
    // down
    a.A = ws + w.Hh; a.B = P.Wd; a.bias = P.bd; a.D = buf_Yg(L, w, ws); a.K = d.H; a.Nout = d.C;
    L->stage_begin(ST_DOWN, st);
    simt_rows_kernel<TAct, TW, EPI_DOWN><<<dim3(w.row_cap / TM, (d.C + TN - 1) / TN), 256, 0, st>>>(a);
    MGPT_LAUNCHED("simt_rows_kernel<down>");
    L->stage_end(ST_DOWN, st);
    return 0;
}

template <typename TAct, typename TW>
int experts_backward_t(mgpt_moe_layer* L, const ExpertPtrs& P, const Workspace& w, char* ws, cudaStream_t st)
{
    const Dims& d = L->d;
    RowsArgs a = {};
    a.tile_expert = (const int32_t*)(ws + w.tile_expert);
    a.n_tiles = (const int32_t*)(ws + w.n_tiles);
    // dHh = dYg * Wd^T, fused SwiGLU backward -> dG, dU
    a.A = buf_dYg(L, w, ws); a.B = P.Wd; a.G = ws + w.G; a.U = ws + w.U; a.D = ws + w.dG; a.D2 = ws + w.dU;
    a.K = d.C; a.Nout = d.H;
    L->stage_begin(ST_DHH, st);
    simt_rows_kernel<TAct, TW, EPI_DHH><<<dim3(w.row_cap / TM, (d.H + TN - 1) / TN), 256, 0, st>>>(a);
    MGPT_LAUNCHED("simt_rows_kernel<dhh>");
    L->stage_end(ST_DHH, st);
    // dXg = dG * Wg^T + dU * Wu^T
    a.A = ws + w.dG; a.A2 = ws + w.dU; a.B = P.Wg; a.B2 = P.Wu; a.D = buf_dXg(L, w, ws); a.K = d.H; a.Nout = d.C;
    L->stage_begin(ST_DXG, st);
    simt_rows_kernel<TAct, TW, EPI_DXG><<<dim3(w.row_cap / TM, (d.C + TN - 1) / TN), 256, 0, st>>>(a);
    MGPT_LAUNCHED("simt_rows_kernel<dxg>");
    L->stage_end(ST_DXG, st);
    if (!L->has_grad) return 0;
    L->stage_begin(ST_WGRAD, st);
    const int32_t* poff = (const int32_t*)(ws + w.padded_offsets);
    WgradArgs g = {};
    g.padded_offsets = poff;
    g.seg = (const int32_t*)(ws + w.seg); g.n_seg = L->n_seg;
    // dWg += Xg^T dG ; dWu += Xg^T dU   [C,H]
    g.A = buf_Xg(L, w, ws); g.lda = d.C; g.M = d.C; g.N = d.H; g.ldb = d.H;
    dim3 gCH((d.C + TM - 1) / TM, (d.H + TN - 1) / TN, d.E);
    g.B = ws + w.dG; g.grad = L->master.gWg;
    simt_wgrad_kernel<TAct><<<gCH, 256, 0, st>>>(g);
    MGPT_LAUNCHED("simt_wgrad_kernel<Wg>");
    g.B = ws + w.dU; g.grad = L->master.gWu;
    simt_wgrad_kernel<TAct><<<gCH, 256, 0, st>>>(g);
    MGPT_LAUNCHED("simt_wgrad_kernel<Wu>");
    // dWd += Hh^T dYg   [H,C]
    g.A = ws + w.Hh; g.lda = d.H; g.M = d.H; g.B = buf_dYg(L, w, ws); g.ldb = d.C; g.N = d.C; g.grad = L->master.gWd;
    dim3 gHC((d.H + TM - 1) / TM, (d.C + TN - 1) / TN, d.E);
    simt_wgrad_kernel<TAct><<<gHC, 256, 0, st>>>(g);
    MGPT_LAUNCHED("simt_wgrad_kernel<Wd>");
    L->stage_end(ST_WGRAD, st);
    return 0;
}

}  // namespace

int simt_experts_forward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    if (w.act_bytes == 4) return experts_forward_t<float, float>(L, L->master, w, ws, st);
    return experts_forward_t<bf16, bf16>(L, L->shadow, w, ws, st);
}

int simt_experts_backward(mgpt_moe_layer* L, const Workspace& w, char* ws, cudaStream_t st)
{
    if (w.act_bytes == 4) return experts_backward_t<float, float>(L, L->master, w, ws, st);
    return experts_backward_t<bf16, bf16>(L, L->shadow, w, ws, st);
}

}  // namespace mgpt
