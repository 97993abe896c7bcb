// The transformer block's glue around the MoE layer, fused:
//
//   forward   x2 = x1 + moe(rmsnorm(x1) * scale)            layers/TransformerBlock.cpp:42-46
//   backward  d_x1 = dout + rmsnorm_backward(d_moe_in)      layers/TransformerBlock.cpp:80-84
//
// The reference runs these as separate passes over [N, C]: rms_norm_into writes the normalised rows twice (x_hat
// and the scaled output, utils/Tensor.cpp:785-800), add_into makes the skip connection, rms_norm_backward_into
// reads x_hat back (utils/Tensor.cpp:1674-1690) and another add_into forms d_x1.  Here the norm writes only the
// layer's input (in the tokens' dtype) and one float per token; the skip connection is folded into the combine
// write; backward recomputes x_hat from x1 and the saved 1/rms and forms d_x1 in the same pass that adds dout.
#include "common.cuh"

namespace mgpt {

namespace {

__device__ __forceinline__ float ld_f32(const float* p) { return *p; }
__device__ __forceinline__ float ld_f32(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 cvt_out<bf16>(float v) { return __float2bfloat16(v); }

// one warp per token: r = 1/sqrt(mean(x^2) + eps), out = (x*r)*scale
template <typename TIo>
__global__ void __launch_bounds__(256)
block_rmsnorm_fwd_kernel(const TIo* __restrict__ x, const float* __restrict__ scale, float eps, int N, int C,
                         TIo* __restrict__ out, float* __restrict__ rs)
{
    const int lane = threadIdx.x & 31;
    const int tok = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (tok >= N) return;
    const TIo* xr = x + (size_t)tok * C;
    float ss = 0.0f;
    for (int c = lane; c < C; c += 32) {
        const float v = ld_f32(xr + c);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)C), eps)));
    if (lane == 0) rs[tok] = r;
    TIo* orow = out + (size_t)tok * C;
    for (int c = lane; c < C; c += 32) orow[c] = cvt_out<TIo>(__fmul_rn(__fmul_rn(ld_f32(xr + c), r), scale[c]));
}

// one warp per token, tokens grid-strided: d_x1 = dout + r*(g*scale - x_hat*<g*scale, x_hat>/C), x_hat = x1*r, g = d_in;
// d_scale[c] += sum over tokens of g*x_hat (per-CTA partial sums in shared memory, one atomic per column per CTA)
template <typename TIo>
__global__ void __launch_bounds__(256)
block_bwd_kernel(const TIo* __restrict__ x1, const float* __restrict__ scale, const float* __restrict__ rs,
                 const TIo* __restrict__ g_in, const TIo* __restrict__ dout, int N, int C, TIo* __restrict__ d_x1,
                 float* __restrict__ d_scale)
{
    extern __shared__ float part[];                 // [C]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < C; c += blockDim.x) part[c] = 0.0f;
    __syncthreads();
    for (int tok = blockIdx.x * 8 + warp; tok < N; tok += gridDim.x * 8) {
        const size_t o = (size_t)tok * C;
        const float r = rs[tok];
        float dot = 0.0f;
        for (int c = lane; c < C; c += 32) {
            const float xh = __fmul_rn(ld_f32(x1 + o + c), r);
            const float g = ld_f32(g_in + o + c);
            dot = fmaf(__fmul_rn(g, scale[c]), xh, dot);
            if (d_scale) atomicAdd(&part[c], g * xh);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        const float m = dot / (float)C;
        for (int c = lane; c < C; c += 32) {
            const float xh = __fmul_rn(ld_f32(x1 + o + c), r);
            const float dxh = __fmul_rn(ld_f32(g_in + o + c), scale[c]);
            const float dn = r * (dxh - xh * m);
            d_x1[o + c] = cvt_out<TIo>(ld_f32(dout + o + c) + dn);
        }
    }
    __syncthreads();
    if (d_scale)
        for (int c = threadIdx.x; c < C; c += blockDim.x) atomicAdd(d_scale + c, part[c]);
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct BlockWs {
    size_t ln2, rs, d_in, moe, total;
};
BlockWs block_ws(const mgpt_moe_layer* L, int n, int io)
{
    const size_t el = io == MGPT_MOE_IO_BF16 ? 2 : 4;
    BlockWs b;
    size_t off = 0;
    b.ln2 = off; off = align256(off + (size_t)n * L->d.C * el + 1);
    b.rs = off; off = align256(off + (size_t)n * 4 + 1);
    b.d_in = off; off = align256(off + (size_t)n * L->d.C * el + 1);
    b.moe = off;
    b.total = off + mgpt_moe_workspace_bytes(L, n);
    return b;
}

}  // namespace

}  // namespace mgpt

using namespace mgpt;

extern "C" {

size_t mgpt_moe_block_workspace_bytes(const mgpt_moe_layer* L, int n_tokens, int io)
{
    if (!L || n_tokens < 0) return 0;
    return block_ws(L, n_tokens, io).total;
}

int mgpt_moe_block_forward(mgpt_moe_layer* L, const void* x1, const float* rms_scale, float eps, void* x2, int n_tokens,
                           int io, void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    if (!L || !rms_scale) return fail(MGPT_MOE_EINVAL, "null argument");
    if (n_tokens <= 0 || !x1 || !x2) return fail(MGPT_MOE_EINVAL, "bad token buffer");
    if (io != MGPT_MOE_IO_F32 && io != MGPT_MOE_IO_BF16) return fail(MGPT_MOE_EINVAL, "unknown io dtype");
    if (!workspace || ((uintptr_t)workspace & 255)) return fail(MGPT_MOE_EINVAL, "workspace must be 256-byte aligned");
    const BlockWs b = block_ws(L, n_tokens, io);
    if (ws_bytes < b.total) return fail(MGPT_MOE_ENOMEM, "workspace smaller than mgpt_moe_block_workspace_bytes()");
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    const int grid = (n_tokens + 7) / 8;
    if (io == MGPT_MOE_IO_F32)
        block_rmsnorm_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x1, rms_scale, eps, n_tokens, L->d.C,
                                                              (float*)(ws + b.ln2), (float*)(ws + b.rs));
    else
        block_rmsnorm_fwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)x1, rms_scale, eps, n_tokens, L->d.C,
                                                             (bf16*)(ws + b.ln2), (float*)(ws + b.rs));
    MGPT_LAUNCHED("block_rmsnorm_fwd_kernel");
    // x2 = x1 + moe(ln2): the skip connection rides on the combine write
    return mgpt_moe_forward_residual(L, ws + b.ln2, x1, x2, n_tokens, io, ws + b.moe, ws_bytes - b.moe, stream);
}

int mgpt_moe_block_backward(mgpt_moe_layer* L, const void* x1, const float* rms_scale, float* d_rms_scale,
                            const void* dout, void* d_x1, int io, void* workspace, size_t ws_bytes, mgpt_stream_t stream)
{
    if (!L || !rms_scale) return fail(MGPT_MOE_EINVAL, "null argument");
    if (!L->fwd_done) return fail(MGPT_MOE_ESTATE, "backward without a forward");
    if (!x1 || !dout || !d_x1) return fail(MGPT_MOE_EINVAL, "null token buffer");
    const int n = L->last_n;
    const BlockWs b = block_ws(L, n, io);
    if (ws_bytes < b.total) return fail(MGPT_MOE_ENOMEM, "workspace smaller than mgpt_moe_block_workspace_bytes()");
    char* ws = (char*)workspace;
    if (ws + b.moe != (char*)L->last_ws) return fail(MGPT_MOE_ESTATE, "backward must reuse the forward's workspace");
    if (n == 0) return 0;
    MGPT_CUDA(cudaSetDevice(L->device));
    cudaStream_t st = (cudaStream_t)stream;
    // the layer's backward: input ln2 (kept by forward), upstream gradient dout, gradient w.r.t. ln2 into the block's buffer
    MGPT_TRY(mgpt_moe_backward(L, ws + b.ln2, dout, ws + b.d_in, io, ws + b.moe, ws_bytes - b.moe, stream));
    int sms = 0;
    MGPT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, L->device));
    const int grid = (n + 7) / 8 < 4 * sms ? (n + 7) / 8 : 4 * sms;
    const size_t sm = (size_t)L->d.C * sizeof(float);
    if (sm > 48 * 1024) return fail(MGPT_MOE_EINVAL, "embed_dim above 12288 is not supported by the block glue");
    if (io == MGPT_MOE_IO_F32)
        block_bwd_kernel<float><<<grid, 256, sm, st>>>((const float*)x1, rms_scale, (const float*)(ws + b.rs),
                                                       (const float*)(ws + b.d_in), (const float*)dout, n, L->d.C,
                                                       (float*)d_x1, d_rms_scale);
    else
        block_bwd_kernel<bf16><<<grid, 256, sm, st>>>((const bf16*)x1, rms_scale, (const float*)(ws + b.rs),
                                                      (const bf16*)(ws + b.d_in), (const bf16*)dout, n, L->d.C,
                                                      (bf16*)d_x1, d_rms_scale);
    MGPT_LAUNCHED("block_bwd_kernel");
    return 0;
}

}  // extern "C"
