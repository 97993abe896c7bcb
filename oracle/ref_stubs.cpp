/*
 * Link-only definitions for the cuda_ops entry points that the reference's
 * no-CUDA stub block (utils/cuda_ops.cu:2009-2077) leaves out or declares with
 * a different parameter list than utils/cuda_ops.h.  None of them is ever
 * executed: with Device::CPU tensors every Tensor method takes its CPU arm.
 * TEST INFRASTRUCTURE ONLY (part of oracle/_ref).
 */
#include <cstddef>
#include "cuda_ops.h"

namespace cuda_ops {
void reset_memory_stats() {}
void print_memory_stats(const char*) {}
void top_k(const float*, float*, float*, int, int, int) {}
void moe_histogram(const float*, float*, int, int, int) {}
void moe_gather(const float*, const float*, float*, float*, float*, int, int, int) {}
void moe_scatter(const float*, const float*, const float*, float*, int, int, int) {}
void moe_scatter_backward(const float*, const float*, const float*, const float*, float*, float*, int, int, int) {}
void moe_gather_backward(const float*, const float*, float*, int, int, int) {}
void scatter_indices(const float*, const float*, float*, int, int, int) {}
float cross_entropy_loss_float(const float*, const float*, int, int) { return 0.0f; }
void cross_entropy_backward_float(const float*, const float*, float*, int, int) {}
void layer_norm(const float*, const float*, const float*, float, float*, float*, float*, float*, int, int) {}
}  // namespace cuda_ops
