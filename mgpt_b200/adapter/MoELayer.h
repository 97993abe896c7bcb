// Drop-in replacement for the reference engine's MoELayer
// (src/main/neuralnetwork/layers/MoELayer.h): same class name, constructor and
// Layer virtuals, so TransformerBlock, GPT, AdamW and the checkpoint code
// drive it unchanged.  The body forwards to the C ABI in include/mgpt_moe.h.
//
// Build: compile this pair in place of the reference's MoELayer.{h,cpp}, with
// the reference's include directories plus this repository's include/, and
// link libmgpt_moe.so.
#ifndef MOELAYER_H
#define MOELAYER_H

#include <memory>
#include <vector>

#include "Layer.h"
#include "mgpt_moe.h"

class MoELayer : public Layer {
private:
    int embed_dim;
    int hidden_dim;
    int num_experts;
    int top_k;

    // 2+6E engine-owned FP32 parameters in the reference's get_parameters() order:
    // Wr, br, then per expert Wg, bg, Wu, bu, Wd, bd (MoELayer.cpp:225-236).
    std::vector<std::unique_ptr<Tensor>> params;

    mgpt_moe_layer* handle = nullptr;
    bool bound = false;
    bool weights_dirty = true;
    bool opt_bound = false;

    Tensor cached_out;
    Tensor cached_dX;
    const float* cached_input = nullptr;   // device pointer of the forward input
    float* workspace = nullptr;
    size_t workspace_floats = 0;
    float* owned_workspace = nullptr;      // used when no Scratchpad is attached
    size_t owned_floats = 0;
    int cached_tokens = 0;
    std::vector<int> cached_shape;
    mutable std::vector<float> cached_cpu_counts;

    void ensure_bound();
    float* take_workspace(size_t n_tokens);

public:
    MoELayer(int embed_dim, int hidden_dim, int num_experts, int top_k);
    ~MoELayer() override;
    MoELayer(MoELayer&&) noexcept;
    MoELayer& operator=(MoELayer&&) = delete;

    // Per-expert routed rows of the last forward (reference: MoELayer.h:39).
    const std::vector<float>& get_expert_counts() const;

    // Call after an optimiser step or a checkpoint load: the BF16 weight copies are
    // rebuilt at the next forward.  Without it every forward rebuilds them.
    void weights_updated() { weights_dirty = true; }

    // Optional: one AdamW step over this layer's 2+6E tensors in a few launches, fused with the
    // rebuild of the BF16 weight copies (same arithmetic as Tensor::adamw_step, Tensor.cpp:683-699).
    // An optimiser that uses it skips these tensors in its own loop (AdamWOptimiser.h:24-36);
    // m and v are its moment tensors for get_parameters()[i], in the same order.
    void adamw_step(const std::vector<Tensor*>& m, const std::vector<Tensor*>& v, float lr, float beta1, float beta2,
                    float eps, float weight_decay, int t);

    Tensor forward(const Tensor& input) override;
    void forward_into(const Tensor& input, Tensor& output) override;

    Tensor backward(const Tensor& dout) override;
    void backward_into(const Tensor& dout, Tensor& din) override;

    std::vector<Tensor*> get_parameters() override;
    ScratchpadFootprint get_footprint(int B, int T) override;
    void to(Device target_device) override;
};

#endif  // MOELAYER_H
