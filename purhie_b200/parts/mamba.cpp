// A selective state-space mixer (the first Mamba form).
//
// [u | z] = W_in h; x = silu(conv(u)) with a causal convolution per channel over the last `conv` inputs (bias added,
// zeros before a request's start); [dt_low | B | C] = W_x x; dt = softplus(W_dt dt_low + b_dt) per channel;
// A = -exp(A_log); per channel c and state n: S[c][n] <- exp(dt_c A[c][n]) S[c][n] + dt_c x_c B_n,
// y_c = sum_n S[c][n] C_n + D_c x_c; the mixer's output is W_o (y * silu(z)).
//
// What a request carries from token to token is S (float32) and the last conv - 1 inputs of the convolution: one
// state slot of the cache manager per request, [inner x state | (conv - 1) x inner] floats, zero at admission.  A
// prompt cut anywhere walks the same recurrence: the convolution reads the kept inputs where a portion starts, and
// the scan starts from the kept S.  dt, the exponentials, the decays and S are float32 in every mode; the four
// products and the convolution's output follow the model's dtype.
//
// The step projection is run as one product over the whole [dt_low | B | C] row with zero columns under B and C
// (the weight is widened once, when the model is bound), so that no strided copy of dt_low is needed; a zero times a
// finite number adds nothing, so the sums are the ones of the narrow product.
#include <algorithm>
#include <cmath>

#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, inner, state, dt_rank, conv, names{in_proj, conv_weight, conv_bias, x_proj, dt_proj, dt_bias,
// a_log, d, out_proj}.
class Mamba1 : public Mixer {
public:
    Mamba1(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        inner_ = p.at("inner").as_int();
        state_ = (int)p.at("state").as_int();
        rank_ = (int)p.at("dt_rank").as_int();
        taps_ = (int)p.at("conv").as_int();
        if (inner_ < 1 || state_ < 1 || rank_ < 1 || taps_ < 1) throw ConfigError("mamba1: inner, state, dt_rank and conv must be positive");
        gemm_ = b.options.get_string("gemm", "auto");
        low_width_ = rank_ + 2 * state_;
    }

    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("in_proj"), {2 * inner_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("conv_weight"), {inner_, taps_}, Role::Vector, Init::Normal},
                {name_of("conv_bias"), {inner_}, Role::Vector, Init::Normal},
                {name_of("x_proj"), {low_width_, inner_}, Role::Matrix, Init::Normal},
                {name_of("dt_proj"), {inner_, rank_}, Role::Matrix, Init::Normal},
                {name_of("dt_bias"), {inner_}, Role::Vector, Init::Normal},
                {name_of("a_log"), {inner_, state_}, Role::Vector, Init::Normal},
                {name_of("d"), {inner_}, Role::Vector, Init::Scale},
                {name_of("out_proj"), {hidden_, inner_}, Role::Matrix, Init::Normal}};
    }

    void bind(WeightSource& src) override {
        in_proj_ = Linear(src.fetch(name_of("in_proj")), "in_proj", gemm_);
        conv_w_ = src.fetch(name_of("conv_weight"));
        conv_b_ = src.fetch(name_of("conv_bias"));
        x_proj_ = Linear(src.fetch(name_of("x_proj")), "x_proj", gemm_);
        // the step projection widened to the whole low row: zeros under B and C
        Tensor dt = src.fetch(name_of("dt_proj"));
        Tensor wide = src.arena().alloc(dt.dtype, {inner_, low_width_});
        const size_t elem = dtype_size(dt.dtype);
        QE_CUDA(cudaMemsetAsync(wide.data, 0, wide.bytes(), src.stream()));
        QE_CUDA(cudaMemcpy2DAsync(wide.data, (size_t)low_width_ * elem, dt.data, (size_t)rank_ * elem, (size_t)rank_ * elem, (size_t)inner_,
                                  cudaMemcpyDeviceToDevice, src.stream()));
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        src.release(dt);
        dt_proj_ = Linear(wide, "dt_proj", gemm_);
        dt_bias_ = src.fetch(name_of("dt_bias"));
        // A = -exp(A_log), once, in float32
        Tensor a_log = src.fetch(name_of("a_log"));
        std::vector<float> host((size_t)inner_ * state_);
        QE_CUDA(cudaMemcpy(host.data(), a_log.data, host.size() * sizeof(float), cudaMemcpyDeviceToHost));
        for (float& v : host) v = -std::exp(v);
        a_ = src.arena().alloc(DType::F32, {inner_, state_});
        QE_CUDA(cudaMemcpy(a_.data, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
        src.release(a_log);
        d_ = src.fetch(name_of("d"));
        out_proj_ = Linear(src.fetch(name_of("out_proj")), "out_proj", gemm_);
    }

    std::vector<std::string> required_libraries() const override {
        const bool fast = in_proj_.fast() || x_proj_.fast() || dt_proj_.fast() || out_proj_.fast();
        return fast ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }
    int preferred_row_multiple() const override { return (in_proj_.fast() || out_proj_.fast()) ? 256 : 0; }

    CacheNeed cache_need() const override { return CacheNeed::state({state_floats()}, DType::F32); }

    // A step with a long prompt portion cuts every request's rows into chunks for the scan (first row, rows, segment,
    // 1 if the request's last chunk), so that a prompt's tokens are spread over the device: the chunk list is this
    // mixer's own metadata, shared by all layers of its kind.
    void prepare_step(StepPlan& plan) override {
        if (plan.has("ssm.chunks")) return;
        int longest = 0;
        for (int n : plan.q_lens) longest = std::max(longest, n);
        if (longest < kChunkFrom) return;
        std::vector<int32_t> items, seg_items = {0};
        int row = 0;
        for (int s = 0; s < plan.S; s++) {
            const int n = plan.q_lens[s];
            for (int at = 0; at < n; at += kChunk) {
                items.push_back(row + at); items.push_back(std::min(kChunk, n - at)); items.push_back(s); items.push_back(at + kChunk >= n);
            }
            row += n;
            seg_items.push_back((int32_t)(items.size() / 4));
        }
        plan.add("ssm.chunks", std::move(items));
        plan.add("ssm.seg_chunks", std::move(seg_items));
    }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        if (cache.kind != CacheNeed::State || !cache.state.defined() || cache.state.dtype != DType::F32 ||
            cache.state.shape.size() != 2 || cache.state.shape[1] != state_floats())
            throw Error(kInvalidState, "mamba1: the cache manager gave no state of this mixer's shape");
        const int T = ctx.T;
        const DType dt = compute_dtype;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        Tensor uz = in_proj_(x, ctx, "ssm_uz", dt, T).tensor;                                   // [T, 2 inner]
        Tensor xc = ws.get("ssm_x", {T, inner_}, dt);
        const long long conv_at = (long long)inner_ * state_;
        const double es = (double)dtype_size(dt);
        if (LaunchProfile::get().on()) LaunchProfile::get().note_cost((double)T * inner_ * 2.0 * es, 2.0 * T * inner_ * taps_);
        QE_LAUNCH(k, k.causal_conv_silu(uz.data, uz.code(), 2 * inner_, (int)inner_, conv_w_.as<float>(), conv_b_.as<float>(), taps_,
                                        cache.state.as<float>(), state_floats(), conv_at, ctx.row_seg, ctx.seg_start, ctx.seg_slot,
                                        xc.data, xc.code(), T, ctx.stream));
        Tensor low = x_proj_(xc, ctx, "ssm_low", dt, T).tensor;                                 // [T, rank + 2 state]
        Tensor dt_raw = dt_proj_(low, ctx, "ssm_dt", DType::F32, T).tensor;                     // [T, inner]
        Tensor y = ws.get("ssm_y", {T, inner_}, dt);
        const StepArray chunks = ctx.array("ssm.chunks"), seg_chunks = ctx.array("ssm.seg_chunks");
        const int n_chunks = chunks.count / 4;
        float *carry = nullptr, *dt_sum = nullptr;
        if (n_chunks) {
            carry = ws.get("ssm_carry", {n_chunks, inner_, state_}, DType::F32).as<float>();
            dt_sum = ws.get("ssm_dt_sum", {n_chunks, inner_}, DType::F32).as<float>();
        }
        if (LaunchProfile::get().on())          // x, z, dt and y per token and channel, B and C per token, the state in and out
            LaunchProfile::get().note_cost((double)T * inner_ * (3.0 * es + 4.0) + (double)T * 2.0 * state_ * es +
                                               2.0 * ctx.S * (double)state_floats() * 4.0,
                                           (double)T * inner_ * state_ * 6.0);
        QE_LAUNCH(k, k.selective_scan(xc.data, dt_raw.as<float>(), dt_bias_.as<float>(), low.data, low_width_, rank_, rank_ + state_, state_,
                                      a_.as<float>(), d_.as<float>(), uz.data, 2 * inner_, (int)inner_, taps_, cache.state.as<float>(),
                                      state_floats(), ctx.seg_start, ctx.seg_slot, ctx.S, n_chunks ? chunks.data : nullptr, n_chunks,
                                      n_chunks ? seg_chunks.data : nullptr, carry, dt_sum, y.data, y.code(), ctx.stream));
        return out_proj_(y, ctx, "ssm_out", DType::F32, T, true);
    }

private:
    static constexpr int kChunk = 64;           // tokens of a chunk of the scan
    static constexpr int kChunkFrom = 192;      // the longest portion of a step from which its scan runs in chunks
    int64_t state_floats() const { return inner_ * state_ + (int64_t)(taps_ - 1) * inner_; }
    int64_t hidden_, inner_, low_width_;
    int state_, rank_, taps_;
    std::string gemm_;
    Linear in_proj_, x_proj_, dt_proj_, out_proj_;
    Tensor conv_w_, conv_b_, dt_bias_, a_, d_;
};

void register_state_space_parts() {
    register_part("mixer", "mamba1", [](const Json& p, BuildContext& b) { return std::make_shared<Mamba1>(p, b); });
}

}  // namespace qe
