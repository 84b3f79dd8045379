// A mixture of gated feed-forward experts with a router.
//
// Router logits z = Wr x + b in float32 (the router's matrix is kept in float32 whatever the model's dtype; x is the
// normed row as the other products see it).  Each token takes the `top` experts with the largest logits (the lower
// index on a tie) with weights softmax(z over the chosen).  An expert is the gated unit of feed_forward.cpp without
// biases; the token's output is the weighted sum of its experts' outputs, added in the order of the choices.
//
// Everything stays on the device: the (token, choice) pairs are sorted by expert there, the experts' products run as
// one launch per matrix over row tiles that never cross from one expert to the next, and no count reaches the host,
// so a decode step with routing is captured as a graph like any other.
#include <array>

#include "gate.h"
#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, intermediate_size, experts, top, activation (as the gated feed-forward's), names{router,
// router_bias (optional)}, expert_names [{gate_proj, up_proj, down_proj} per expert].
class RoutedGLU : public FeedForward {
public:
    RoutedGLU(const Json& p, BuildContext& b)
        : FeedForward(p, b), hidden_(p.at("hidden_size").as_int()), inter_(p.at("intermediate_size").as_int()),
          experts_((int)p.at("experts").as_int()), top_((int)p.at("top").as_int()), gate_(GateSpec::read(p)) {
        if (experts_ < 1 || top_ < 1 || top_ > experts_)
            throw ConfigError("routed feed-forward: top " + std::to_string(top_) + " of " + std::to_string(experts_) + " experts");
        const Json& names = p.at("expert_names");
        if (!names.is_array() || (int)names.size() != experts_) throw ConfigError("routed feed-forward: expert_names must list every expert");
        for (const Json& n : names.items())
            expert_names_.push_back({n.at("gate_proj").as_string(), n.at("up_proj").as_string(), n.at("down_proj").as_string()});
        has_bias_ = names_.count("router_bias") != 0;
    }

    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("router"), {experts_, hidden_}, Role::Vector, Init::Normal}};
        if (has_bias_) s.push_back({name_of("router_bias"), {experts_}, Role::Vector, Init::Normal});
        for (const auto& n : expert_names_) {
            s.push_back({n[0], {inter_, hidden_}, Role::Matrix, Init::Normal});
            s.push_back({n[1], {inter_, hidden_}, Role::Matrix, Init::Normal});
            s.push_back({n[2], {hidden_, inter_}, Role::Matrix, Init::Normal});
        }
        return s;
    }

    void bind(WeightSource& src) override {
        router_ = Linear(src.fetch(name_of("router")), "router", "simple");
        if (has_bias_) router_bias_ = src.fetch(name_of("router_bias"));
        // the experts' matrices stacked: [experts, 2 ff, hidden] with gate and up rows interleaved (g0, u0, g1, u1, ...)
        // as the gated feed-forward lays them out, and [experts, hidden, ff]
        for (int e = 0; e < experts_; e++) {
            Tensor gate = src.fetch(expert_names_[e][0]), up = src.fetch(expert_names_[e][1]), down = src.fetch(expert_names_[e][2]);
            if (e == 0) {
                gate_up_ = src.arena().alloc(gate.dtype, {experts_, 2 * inter_, hidden_});
                down_ = src.arena().alloc(down.dtype, {experts_, hidden_, inter_});
            }
            if (gate.dtype != gate_up_.dtype || up.dtype != gate_up_.dtype || down.dtype != down_.dtype)
                throw WeightError("the experts of a routed feed-forward are stored in different precisions");
            const size_t row = (size_t)hidden_ * dtype_size(gate.dtype);
            char* gu = static_cast<char*>(gate_up_.data) + (size_t)e * 2 * inter_ * row;
            QE_CUDA(cudaMemcpy2DAsync(gu, 2 * row, gate.data, row, row, (size_t)inter_, cudaMemcpyDeviceToDevice, src.stream()));
            QE_CUDA(cudaMemcpy2DAsync(gu + row, 2 * row, up.data, row, row, (size_t)inter_, cudaMemcpyDeviceToDevice, src.stream()));
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(down_.data) + (size_t)e * down.bytes(), down.data, down.bytes(),
                                    cudaMemcpyDeviceToDevice, src.stream()));
            QE_CUDA(cudaStreamSynchronize(src.stream()));
            src.release(gate);
            src.release(up);
            src.release(down);
        }
    }

    Addend forward(const Tensor& x, StepContext& ctx) override {
        const int T = ctx.T, R = T * top_;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        Tensor logits = router_(x, ctx, "moe_router", DType::F32, T).tensor;
        Tensor choice = ws.get("moe_choice", {T, top_}, DType::I32), weight = ws.get("moe_weight", {T, top_}, DType::F32);
        QE_LAUNCH(k, k.route_topk(logits.as<float>(), router_bias_.defined() ? router_bias_.as<float>() : nullptr, T, experts_, top_,
                                  choice.as<int32_t>(), weight.as<float>(), ctx.stream));
        const int tiles = k.route_max_tiles(R, experts_);
        Tensor position = ws.get("moe_position", {R}, DType::I32), pair_at = ws.get("moe_pair_at", {R}, DType::I32);
        Tensor tile_list = ws.get("moe_tiles", {tiles, 3}, DType::I32), scratch = ws.get("moe_sort_scratch", {3 * experts_ + 1}, DType::I32);
        QE_LAUNCH(k, k.route_sort(choice.as<int32_t>(), R, experts_, position.as<int32_t>(), pair_at.as<int32_t>(),
                                  tile_list.as<int32_t>(), tiles, scratch.as<int32_t>(), ctx.stream));
        Tensor gu = ws.get("moe_gate_up", {R, 2 * inter_}, compute_dtype);
        QE_LAUNCH(k, k.gemm_grouped(x.data, x.code(), pair_at.as<int32_t>(), top_, gate_up_.data, gate_up_.code(), tile_list.as<int32_t>(),
                                    tiles, gu.data, gu.code(), (int)(2 * inter_), (int)hidden_, ctx.stream));
        Tensor act = ws.get("moe_act", {R, inter_}, compute_dtype);
        QE_LAUNCH(k, k.glu(gu.data, gu.code(), 1, 0, act.data, act.code(), R, (int)inter_, gate_.kind, gate_.alpha, gate_.limit,
                           gate_.shift, ctx.stream));
        Tensor y = ws.get("moe_down", {R, hidden_}, DType::F32);
        QE_LAUNCH(k, k.gemm_grouped(act.data, act.code(), nullptr, 1, down_.data, down_.code(), tile_list.as<int32_t>(), tiles, y.data,
                                    y.code(), (int)hidden_, (int)inter_, ctx.stream));
        Tensor out = ws.get("moe_out", {T, hidden_}, DType::F32);
        QE_LAUNCH(k, k.route_combine(y.data, y.code(), position.as<int32_t>(), weight.as<float>(), T, top_, (int)hidden_, out.as<float>(),
                                     ctx.stream));
        return Addend(out, 1);
    }

private:
    int64_t hidden_, inter_;
    int experts_, top_;
    GateSpec gate_;
    bool has_bias_ = false;
    std::vector<std::array<std::string, 3>> expert_names_;
    Linear router_;
    Tensor router_bias_, gate_up_, down_;
};

void register_routed_parts() {
    register_part("feed_forward", "routed_glu", [](const Json& p, BuildContext& b) { return std::make_shared<RoutedGLU>(p, b); });
}

}  // namespace qe
