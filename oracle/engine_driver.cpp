// Engine-driven run of the B200 MoE layer: TEST INFRASTRUCTURE, not part of the product.
//
// This program is the reference engine around the layer, unchanged: the reference's own Tensor, Scratchpad,
// cuda_ops (compiled with USE_CUDA by nvcc) and AdamWOptimizer sources, compiled where they lie, with ONE
// substitution -- mgpt_b200/adapter/MoELayer.{h,cpp} stands where the reference's MoELayer.{h,cpp} stood.
// It drives the layer the way the reference's own callers do:
//
//   construction + to(Device::CUDA)            pipeline/Trainer.cpp:200-207, layers/Layer.h:49-53
//   arena sized from get_footprint x 1.05       pipeline/Trainer.cpp:211-224
//   set_scratchpad                              layers/TransformerBlock.h:43-49
//   zero_grad on every parameter                pipeline/Trainer.cpp:303-305
//   forward, rewind; forward again, backward, rewind (activation checkpointing)
//                                               neuralnetwork/GPT.cpp:39-51, 79-96
//   AdamWOptimizer::step(parameters)            neuralnetwork/optimisers/AdamWOptimiser.h:24-36
//   forward again with the stepped weights
//
// and writes every observable result to a file the pytest compares with the CPU oracle.  Of the reference's GPU
// code only allocation, fills, copies and its AdamW kernel run here; its MoE kernels are not called.
//
//   engine_moe_driver <in.bin> <out.bin>
//   in : int32 B,T,C,H,E,k | params (2+6E tensors, get_parameters() order) | x[B*T*C] | dy[B*T*C]   (float32)
//   out: y | dx | grads (2+6E) | counts[E] | params after the step | y2          (float32)
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <stdexcept>
#include <vector>

#include "AdamWOptimiser.h"
#include "MoELayer.h"
#include "Scratchpad.h"
#include "Tensor.h"
#include "cuda_ops.h"

namespace {
std::vector<float> read_floats(FILE* f, size_t n)
{
    std::vector<float> v(n);
    if (n && fread(v.data(), sizeof(float), n, f) != n) throw std::runtime_error("short input file");
    return v;
}
void write_tensor(FILE* f, const Tensor& t)
{
    std::vector<float> h(t.size());
    t.copy_to_host(h.data());
    fwrite(h.data(), sizeof(float), h.size(), f);
}
}  // namespace

int main(int argc, char** argv)
{
    if (argc != 3) {
        std::cerr << "usage: engine_moe_driver <in.bin> <out.bin>\n";
        return 2;
    }
    try {
        FILE* in = fopen(argv[1], "rb");
        if (!in) throw std::runtime_error("cannot open input");
        int hdr[6];
        if (fread(hdr, sizeof(int), 6, in) != 6) throw std::runtime_error("short header");
        const int B = hdr[0], T = hdr[1], C = hdr[2], H = hdr[3], E = hdr[4], k = hdr[5];

        MoELayer moe(C, H, E, k);
        moe.to(Device::CUDA);
        std::vector<Tensor*> params = moe.get_parameters();
        if ((int)params.size() != 2 + 6 * E) throw std::runtime_error("unexpected parameter count");
        for (Tensor* p : params) {
            std::vector<float> w = read_floats(in, p->size());
            p->copy_from_host(w.data());          // as load_weights_bin does: through get_parameters() only
        }
        const size_t n = (size_t)B * T * C;
        Tensor x({B, T, C}, 0.0f, Device::CUDA), dy({B, T, C}, 0.0f, Device::CUDA);
        {
            std::vector<float> hx = read_floats(in, n), hdy = read_floats(in, n);
            x.copy_from_host(hx.data());
            dy.copy_from_host(hdy.data());
        }
        fclose(in);

        // the trainer's arena: footprint of the model (here: the layer) plus 5 %
        const ScratchpadFootprint fp = moe.get_footprint(B, T);
        const size_t peak = std::max(fp.fwd_peak(), fp.bwd_peak());
        Scratchpad pad((size_t)(peak * 1.05f), ScratchpadDevice::CUDA);
        moe.set_scratchpad(&pad);

        for (Tensor* p : params) p->zero_grad();

        Tensor y({B, T, C}, 0.0f, Device::CUDA), dx({B, T, C}, 0.0f, Device::CUDA);
        // forward pass of a checkpointed model: activations are dropped right after the block
        size_t sp = pad.get_savepoint();
        moe.forward_into(x, y);
        pad.restore_savepoint(sp);
        // backward pass: recompute the block's forward from its saved input, then backward, then rewind
        sp = pad.get_savepoint();
        moe.forward_into(x, y);
        moe.backward_into(dy, dx);
        pad.restore_savepoint(sp);
        const std::vector<float> counts = moe.get_expert_counts();

        FILE* out = fopen(argv[2], "wb");
        if (!out) throw std::runtime_error("cannot open output");
        write_tensor(out, y);
        write_tensor(out, dx);
        for (Tensor* p : params) {
            std::vector<float> g(p->size());
            cuda_ops::copy_device_to_host(g.data(), p->get_grad_ptr(), p->size());
            fwrite(g.data(), sizeof(float), g.size(), out);
        }
        fwrite(counts.data(), sizeof(float), counts.size(), out);

        // the engine's own optimiser, untouched, followed by the next step's forward
        AdamWOptimizer opt(1e-2f);
        opt.step(params);
        for (Tensor* p : params) write_tensor(out, *p);
        Tensor y2({B, T, C}, 0.0f, Device::CUDA);
        sp = pad.get_savepoint();
        moe.forward_into(x, y2);
        pad.restore_savepoint(sp);
        write_tensor(out, y2);
        fclose(out);
        std::cout << "engine_moe_driver ok: arena " << pad.get_capacity() << " floats, footprint " << peak << "\n";
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "engine_moe_driver failed: " << e.what() << "\n";
        return 1;
    }
}
