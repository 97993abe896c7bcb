// See MoELayer.h.  Error behaviour follows the reference: failures surface as
// std::runtime_error, which main() catches (src/main/main.cpp:24-27).
#include "MoELayer.h"

#include <cmath>
#include <stdexcept>
#include <string>

#include "Scratchpad.h"
#include "cuda_ops.h"

namespace {
void check(int rc, const char* what)
{
    if (rc != MGPT_MOE_OK)
        throw std::runtime_error(std::string("MoELayer: ") + what + ": " + mgpt_moe_last_error());
}
}  // namespace

MoELayer::MoELayer(int embed_dim_, int hidden_dim_, int num_experts_, int top_k_)
    : embed_dim(embed_dim_), hidden_dim(hidden_dim_ == -1 ? 4 * embed_dim_ : hidden_dim_),
      num_experts(num_experts_), top_k(top_k_)
{
    // Same tensors, same order, same initialiser calls as LinearLayer's constructor
    // (LinearLayer.cpp:15-20) run for the router and then gate/up/down of every expert,
    // so a seeded run starts from the reference's own weights.
    auto linear = [this](int in, int out) {
        params.emplace_back(new Tensor(Tensor::randn({in, out}, 0.0f, std::sqrt(2.0f / (float)in))));
        params.emplace_back(new Tensor({1, out}, 0.0f));
    };
    linear(embed_dim, num_experts);
    for (int e = 0; e < num_experts; ++e) {
        linear(embed_dim, hidden_dim);
        linear(embed_dim, hidden_dim);
        linear(hidden_dim, embed_dim);
    }
    mgpt_moe_config cfg = {embed_dim, hidden_dim, num_experts, top_k, 0.01f, MGPT_MOE_BF16, 0, 0};
    check(mgpt_moe_create(&cfg, &handle), "create");
}

MoELayer::MoELayer(MoELayer&& o) noexcept
    : Layer(std::move(o)), embed_dim(o.embed_dim), hidden_dim(o.hidden_dim), num_experts(o.num_experts),
      top_k(o.top_k), params(std::move(o.params)), handle(o.handle), bound(false), weights_dirty(true),
      owned_workspace(o.owned_workspace), owned_floats(o.owned_floats)
{
    o.handle = nullptr;
    o.owned_workspace = nullptr;
}

MoELayer::~MoELayer()
{
    mgpt_moe_destroy(handle);
    if (owned_workspace) cuda_ops::free_memory(owned_workspace);
}

void MoELayer::to(Device target_device)
{
    Layer::to(target_device);      // moves every parameter (Layer.h:49-53)
    bound = false;
    weights_dirty = true;
}

void MoELayer::ensure_bound()
{
    if (!bound) {
        std::vector<float*> data, grad;
        for (auto& p : params) {
            if (p->device != Device::CUDA) throw std::runtime_error("MoELayer: parameters must be on Device::CUDA");
            data.push_back(p->get_data_ptr());
            grad.push_back(p->get_grad_ptr());      // creates cuda_grad on first use (Tensor.cpp:239-246)
        }
        check(mgpt_moe_bind_params(handle, data.data(), grad.data(), (int)data.size()), "bind_params");
        bound = true;
        weights_dirty = true;
        opt_bound = false;
    }
    if (weights_dirty) {
        check(mgpt_moe_sync_weights(handle, nullptr), "sync_weights");
        weights_dirty = false;
    }
}

void MoELayer::adamw_step(const std::vector<Tensor*>& m, const std::vector<Tensor*>& v, float lr, float beta1,
                          float beta2, float eps, float weight_decay, int t)
{
    const bool rebound = !bound;
    ensure_bound();
    if (rebound || !opt_bound) {
        if (m.size() != params.size() || v.size() != params.size())
            throw std::runtime_error("MoELayer::adamw_step: expected one m and one v tensor per parameter");
        std::vector<float*> mp, vp;
        for (size_t i = 0; i < params.size(); ++i) {
            mp.push_back(m[i]->get_data_ptr());
            vp.push_back(v[i]->get_data_ptr());
        }
        check(mgpt_moe_bind_optimizer_state(handle, mp.data(), vp.data(), (int)mp.size()), "bind_optimizer_state");
        opt_bound = true;
    }
    check(mgpt_moe_adamw_step(handle, lr, beta1, beta2, eps, weight_decay, t, nullptr), "adamw_step");
    weights_dirty = false;      // the step wrote the BF16 copies itself
}

float* MoELayer::take_workspace(size_t n_tokens)
{
    const size_t bytes = mgpt_moe_workspace_bytes(handle, (int)n_tokens);
    const size_t floats = (bytes + sizeof(float) - 1) / sizeof(float);
    workspace_floats = floats;
    if (scratchpad) return scratchpad->get_address(floats);        // 256-byte aligned (Scratchpad.cpp:27-29)
    if (owned_floats < floats) {
        if (owned_workspace) cuda_ops::free_memory(owned_workspace);
        cuda_ops::allocate_memory(&owned_workspace, floats);
        owned_floats = floats;
    }
    return owned_workspace;
}

Tensor MoELayer::forward(const Tensor& input)
{
    forward_into(input, cached_out);
    return cached_out;
}

void MoELayer::forward_into(const Tensor& input, Tensor& output)
{
    if (input.device != Device::CUDA)
        throw std::runtime_error("MoELayer: this build has no CPU path; move the model to Device::CUDA");
    const size_t B = input.shape[0], T = input.shape[1], C = input.shape[2];
    ensure_bound();
    if (output.shape.empty()) output = Tensor({(int)B, (int)T, (int)C}, 0.0f, Device::CUDA);
    workspace = take_workspace(B * T);
    check(mgpt_moe_forward(handle, input.get_data_ptr(), output.get_data_ptr(), (int)(B * T), MGPT_MOE_IO_F32,
                           workspace, workspace_floats * sizeof(float), nullptr),
          "forward");
    cached_input = input.get_data_ptr();
    cached_tokens = (int)(B * T);
    cached_shape = input.shape;
    cached_out = output;
    // As in the reference (MoELayer.cpp:127) the arena is not rewound here: the saved
    // activations must survive until backward; the caller's savepoint releases them.
}

Tensor MoELayer::backward(const Tensor& dout)
{
    backward_into(dout, cached_dX);
    return cached_dX;
}

void MoELayer::backward_into(const Tensor& dout, Tensor& din)
{
    if (!cached_input) throw std::runtime_error("MoELayer: backward before forward");
    if (din.shape.empty()) din = Tensor(cached_shape, 0.0f, Device::CUDA);
    check(mgpt_moe_backward(handle, cached_input, dout.get_data_ptr(), din.get_data_ptr(), MGPT_MOE_IO_F32,
                            workspace, workspace_floats * sizeof(float), nullptr),
          "backward");
    cached_dX = din;
    // gradients exist now, so the optimiser is about to move the FP32 masters: the BF16 copies are stale
    if (auto_refresh) weights_dirty = true;
}

const std::vector<float>& MoELayer::get_expert_counts() const
{
    std::vector<int32_t> c(num_experts, 0);
    cached_cpu_counts.assign(num_experts, 0.0f);
    if (cached_input && mgpt_moe_expert_counts(handle, c.data()) == MGPT_MOE_OK)
        for (int e = 0; e < num_experts; ++e) cached_cpu_counts[e] = (float)c[e];
    return cached_cpu_counts;
}

std::vector<Tensor*> MoELayer::get_parameters()
{
    std::vector<Tensor*> out;
    for (auto& p : params) out.push_back(p.get());
    return out;
}

ScratchpadFootprint MoELayer::get_footprint(int B, int T)
{
    // Everything the layer needs is one block that lives from forward to backward.
    const size_t bytes = mgpt_moe_workspace_bytes(handle, B * T);
    const size_t floats = (bytes + sizeof(float) - 1) / sizeof(float) + 64;
    return {floats, 0, 0};
}
