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
    bool auto_refresh = true;
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

    // The tensor-core products read BF16 copies of the FP32 masters, so the copies must be rebuilt whenever the
    // masters change.  The engine changes them behind the layer's back (AdamWOptimizer::step, load_weights_bin,
    // --resume all go through get_parameters()), so the safe default is: the copies are marked stale when the
    // layer is created or moved, and after every backward (an optimiser step follows gradients), and rebuilt at
    // the next forward.  Under activation checkpointing that is still one rebuild per training step: the
    // recompute forward that precedes backward finds them fresh.  An engine that writes the masters at any other
    // moment (loading a checkpoint between two forwards without a backward) calls weights_updated() itself.
    void weights_updated() { weights_dirty = true; }

    // An engine that calls weights_updated() after each of its own parameter writes can switch the automatic
    // marking after backward off (saves the rebuild when several forward/backward pairs share one optimiser
    // step, i.e. gradient accumulation).
    void set_auto_refresh(bool on) { auto_refresh = on; }

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
