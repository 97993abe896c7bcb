// Row buffers that the other GPUs of the node read directly.
//
// The expert-parallel layer moves rows between GPUs four times per step.  A collective's copy kernels need SMs,
// and the layer's persistent kernels hold every SM, so an exchange started beside them waits for the kernel to end.
// Copy engines need no SM: each rank allocates its send-side buffers here, exports them (CUDA IPC), the owners of
// the experts open them and PULL their blocks with cudaMemcpyAsync over NVLink while the SMs keep computing.
// The reference has no multi-GPU code (layers/MoELayer.cpp works on one device); there is no counterpart.
#include "common.cuh"

using namespace mgpt;

extern "C" {

int mgpt_moe_peer_alloc(int device, size_t bytes, void** ptr, void* handle)
{
    if (!ptr || !handle || bytes == 0) return fail(MGPT_MOE_EINVAL, "null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == MGPT_MOE_PEER_HANDLE_BYTES, "handle size");
    MGPT_CUDA(cudaSetDevice(device));
    void* p = nullptr;
    MGPT_CUDA(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(MGPT_MOE_ECUDA, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return 0;
}

int mgpt_moe_peer_open(int device, const void* handle, void** ptr)
{
    if (!ptr || !handle) return fail(MGPT_MOE_EINVAL, "null argument");
    MGPT_CUDA(cudaSetDevice(device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    MGPT_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return 0;
}

int mgpt_moe_peer_close(int device, void* ptr)
{
    if (!ptr) return 0;
    MGPT_CUDA(cudaSetDevice(device));
    MGPT_CUDA(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int mgpt_moe_peer_free(int device, void* ptr)
{
    if (!ptr) return 0;
    MGPT_CUDA(cudaSetDevice(device));
    MGPT_CUDA(cudaFree(ptr));
    return 0;
}

int mgpt_moe_peer_copy(void* dst, const void* src, size_t bytes, mgpt_stream_t stream)
{
    if (bytes == 0) return 0;
    if (!dst || !src) return fail(MGPT_MOE_EINVAL, "null argument");
    MGPT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return 0;
}

}  // extern "C"
