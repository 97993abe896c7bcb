/*
 * Drives the reference's own MoELayer (CPU arm) behind the same C signature as
 * moe_oracle_run, so the restatement in moe_oracle.c can be checked against
 * the real thing and golden vectors can be produced from it.
 *
 * TEST INFRASTRUCTURE ONLY. Compiled by oracle/Makefile together with the
 * reference's sources (read where they lie; none are copied) into
 * oracle/_ref/libmgpt_ref.so.  This file holds no reference code: it only
 * calls the layer's public interface (layers/MoELayer.h:37-50) and reads the
 * tensors the layer caches for its backward pass (layers/MoELayer.h:17-33).
 */
#include <chrono>
#include <cstdint>
#include <cstring>
#include <functional>
#include <iostream>
#include <stdexcept>
#include <vector>

/* The cached routing tensors are private members; open them for this one
 * translation unit (standard headers are already included above). */
#define private public
#include "MoELayer.h"
#undef private

#include "moe_oracle.h"

namespace {

void copy_as_int(const Tensor& t, int32_t* dst, size_t n)
{
    for (size_t i = 0; i < n; ++i) dst[i] = (int32_t)t.data[i];
}

int run(const moe_oracle_dims* d, const moe_oracle_inputs* in, moe_oracle_outputs* out, bool backward)
{
    const int N = d->n_tokens, C = d->C, H = d->H, E = d->E, k = d->k;
    MoELayer layer(C, H, E, k);
    std::vector<Tensor*> params = layer.get_parameters();
    if ((int)params.size() != 2 + 6 * E) return 2;
    for (size_t i = 0; i < params.size(); ++i) {
        std::memcpy(params[i]->data.data(), in->params[i], params[i]->size() * sizeof(float));
        params[i]->zero_grad();
    }
    /* One batch row of N tokens: the layer only uses B*T (MoELayer.cpp:30). */
    Tensor x({1, N, C}, 0.0f, Device::CPU);
    std::memcpy(x.data.data(), in->x, (size_t)N * C * sizeof(float));
    Tensor y = layer.forward(x);

    const size_t NE = (size_t)N * E, R = (size_t)N * k;
    if (out->logits) std::memcpy(out->logits, layer.cached_router_logits.data.data(), NE * sizeof(float));
    if (out->probs) std::memcpy(out->probs, layer.cached_router_probs.data.data(), NE * sizeof(float));
    if (out->top_idx) copy_as_int(layer.cached_top_indices, out->top_idx, R);
    if (out->top_p) std::memcpy(out->top_p, layer.cached_top_probs.data.data(), R * sizeof(float));
    if (out->counts)
        for (int e = 0; e < E; ++e) out->counts[e] = (int32_t)layer.get_expert_counts()[e];
    if (out->offsets)
        for (int e = 0; e < E; ++e) out->offsets[e] = (int32_t)layer.cached_cpu_offsets[e];
    if (out->map) copy_as_int(layer.cached_sorted_token_ids, out->map, R);
    if (out->gathered_out)
        std::memcpy(out->gathered_out, layer.cached_gathered_outputs.data.data(), R * C * sizeof(float));
    if (out->y) std::memcpy(out->y, y.data.data(), (size_t)N * C * sizeof(float));

    if (backward && in->dy) {
        Tensor dy({1, N, C}, 0.0f, Device::CPU);
        std::memcpy(dy.data.data(), in->dy, (size_t)N * C * sizeof(float));
        Tensor dx = layer.backward(dy);
        if (out->dx) std::memcpy(out->dx, dx.data.data(), (size_t)N * C * sizeof(float));
        if (out->grads)
            for (size_t i = 0; i < params.size(); ++i)
                if (out->grads[i])
                    for (size_t j = 0; j < params[i]->size(); ++j) out->grads[i][j] += params[i]->grad[j];
        /* d_top_p and dlogits are locals of MoELayer::backward_into and cannot be read. */
    }
    return 0;
}

}  // namespace

extern "C" int moe_ref_run(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                           moe_oracle_outputs* out, int /*n_threads*/)
{
    try {
        return run(d, in, out, true);
    } catch (const std::exception& e) {
        std::cerr << "moe_ref_run: " << e.what() << std::endl;
        return 1;
    }
}

/* Timed CPU baseline: the layer is built and loaded once (untimed); each of
 * `iters` iterations zeroes the gradients (untimed) and then times
 * forward()+backward() (forward only when dy is NULL) with std::chrono, the
 * clock the reference's trainer uses (pipeline/Trainer.cpp:314-323).
 * seconds[i] receives iteration i. */
extern "C" int moe_ref_bench(const moe_oracle_dims* d, const moe_oracle_inputs* in, int iters, double* seconds)
{
    try {
        const int N = d->n_tokens, C = d->C;
        MoELayer layer(C, d->H, d->E, d->k);
        std::vector<Tensor*> params = layer.get_parameters();
        for (size_t i = 0; i < params.size(); ++i)
            std::memcpy(params[i]->data.data(), in->params[i], params[i]->size() * sizeof(float));
        Tensor x({1, N, C}, 0.0f, Device::CPU), dy({1, N, C}, 0.0f, Device::CPU);
        std::memcpy(x.data.data(), in->x, (size_t)N * C * sizeof(float));
        if (in->dy) std::memcpy(dy.data.data(), in->dy, (size_t)N * C * sizeof(float));
        for (int it = 0; it < iters; ++it) {
            for (Tensor* p : params) p->zero_grad();
            auto t0 = std::chrono::steady_clock::now();
            Tensor y = layer.forward(x);
            if (in->dy) Tensor dx = layer.backward(dy);
            auto t1 = std::chrono::steady_clock::now();
            seconds[it] = std::chrono::duration<double>(t1 - t0).count();
        }
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "moe_ref_bench: " << e.what() << std::endl;
        return 1;
    }
}

extern "C" int moe_ref_route(const moe_oracle_dims* d, const moe_oracle_inputs* in,
                             moe_oracle_outputs* out, int /*n_threads*/)
{
    try {
        return run(d, in, out, false);
    } catch (const std::exception& e) {
        std::cerr << "moe_ref_route: " << e.what() << std::endl;
        return 1;
    }
}

/* The reference's own AdamW step (Tensor::adamw_step, CPU arm) on a flat tensor, in place on w, m, v. */
extern "C" int moe_ref_adamw(float* w, const float* g, float* m, float* v, long n, float lr, float beta1, float beta2,
                             float eps, float weight_decay, int t)
{
    try {
        Tensor p({(int)n}, 0.0f, Device::CPU), mt({(int)n}, 0.0f, Device::CPU), vt({(int)n}, 0.0f, Device::CPU);
        p.zero_grad();
        std::memcpy(p.data.data(), w, (size_t)n * sizeof(float));
        std::memcpy(p.grad.data(), g, (size_t)n * sizeof(float));
        std::memcpy(mt.data.data(), m, (size_t)n * sizeof(float));
        std::memcpy(vt.data.data(), v, (size_t)n * sizeof(float));
        p.adamw_step(mt, vt, lr, beta1, beta2, eps, weight_decay, t);
        std::memcpy(w, p.data.data(), (size_t)n * sizeof(float));
        std::memcpy(m, mt.data.data(), (size_t)n * sizeof(float));
        std::memcpy(v, vt.data.data(), (size_t)n * sizeof(float));
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "moe_ref_adamw: " << e.what() << std::endl;
        return 1;
    }
}

/* The reference's own RMSNorm (Tensor::rms_norm_into / rms_norm_backward_into, CPU arm), for pinning the numpy
 * restatement the block-glue tests use.  x, dout [n, c]; scale [c]; out, dx [n, c]; rs [n]; dscale [c] (accumulated from 0). */
extern "C" int moe_ref_rmsnorm(const float* x, const float* scale, const float* dout, int n, int c, float eps, float* out,
                               float* rs, float* dx, float* dscale)
{
    try {
        Tensor xt({n, c}, 0.0f, Device::CPU), st({c}, 0.0f, Device::CPU), dt({n, c}, 0.0f, Device::CPU);
        std::memcpy(xt.data.data(), x, (size_t)n * c * sizeof(float));
        std::memcpy(st.data.data(), scale, (size_t)c * sizeof(float));
        std::memcpy(dt.data.data(), dout, (size_t)n * c * sizeof(float));
        st.grad.assign((size_t)c, 0.0f);
        Tensor r, xh, o, dxt;
        xt.rms_norm_into(c, st, eps, r, xh, o);
        xt.rms_norm_backward_into(dt, xh, st, r, dxt);
        std::memcpy(out, o.data.data(), (size_t)n * c * sizeof(float));
        std::memcpy(rs, r.data.data(), (size_t)n * sizeof(float));
        std::memcpy(dx, dxt.data.data(), (size_t)n * c * sizeof(float));
        std::memcpy(dscale, st.grad.data(), (size_t)c * sizeof(float));
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "moe_ref_rmsnorm: " << e.what() << std::endl;
        return 1;
    }
}
