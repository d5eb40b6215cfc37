// Part kinds for hybrid decoders: layers that mix softmax attention with recurrences, with norms on both
// sides of every sublayer.
//
//   norm          "rmsnorm"               x / sqrt(mean(x^2) + eps) * gain, in 32-bit; can also follow a sublayer
//   feed_forward  "gated_mlp"             down(act(gate h) * (up h))
//                 "none"                  a layer without a feed-forward
//   block         "sandwich_norm"         x += m * norm_b(mixer(norm_a(x)));  x += m * norm_d(ff(norm_c(x)))
//   mixer         "gated_delta"           short convolutions, unit q/k, gated delta rule, per-head norm, output gate
//                 "attention_beside_matrix_memory"
//                                         two mixers on one input: grouped-query attention (whole-row q/k norm, partial
//                                         rotary positions, a sink in the softmax, a gate per head) and a matrix
//                                         memory (mLSTM); result = left_scale * left + right_scale * right
//   remix         "concat_linear"         x <- W [x; x0]
//
// Every size and constant is a parameter of the part.  What the recurrences, the norms, the gates, the softmax
// and the residual sum compute is 32-bit in both compute types; the matrix products run in the compute type.
//
// Products are fused where several read the same input: each mixer has one wide product for everything that
// feeds its kernels in the compute type and one narrow product, written in float32, for its per-head gates
// (their values enter exponentials and recurrences).
#include <cmath>

#include "part_helpers.h"
#include "parts.h"

namespace sandy {
namespace part_helpers {

constexpr double kPi = 3.14159265358979323846;

// ---- host-side helpers: matrices put together from several tensors of the weight file ---------------------
std::shared_ptr<float> alloc_f32(size_t n) { return std::shared_ptr<float>(new float[std::max<size_t>(n, 1)](), std::default_delete<float[]>()); }

HostTensor host_f32(std::shared_ptr<float> data, std::vector<int64_t> shape) {
    HostTensor t;
    t.dtype = StoreDType::F32;
    t.shape = std::move(shape);
    t.data = data.get();
    t.owner = data;
    return t;
}

// Rows of several [n_i, cols] matrices one under the other.
HostTensor stack_rows(const std::vector<const HostTensor*>& parts, int64_t cols) {
    int64_t rows = 0;
    for (const HostTensor* p : parts) rows += p->numel() / cols;
    auto buf = alloc_f32((size_t)(rows * cols));
    size_t at = 0;
    for (const HostTensor* p : parts) {
        const std::vector<float> v = to_f32(*p);
        std::copy(v.begin(), v.end(), buf.get() + at);
        at += v.size();
    }
    return host_f32(buf, {rows, cols});
}

// Columns of several [rows, n_i] matrices side by side; `pad_to[i]` widens part i with zero columns, and with
// `group[i]` > 0 the padding goes behind every group of `group[i]` columns (heads padded to a larger head size).
HostTensor join_columns(const std::vector<ColumnPart>& parts, int64_t rows, int64_t total_cols) {
    auto buf = alloc_f32((size_t)(rows * total_cols));
    int64_t c0 = 0;
    for (const ColumnPart& p : parts) {
        const std::vector<float> v = to_f32(*p.t);
        const int64_t group = p.group > 0 ? p.group : p.cols, padded = p.group > 0 ? p.group_padded : p.cols;
        for (int64_t r = 0; r < rows; r++)
            for (int64_t c = 0; c < p.cols; c++)
                buf.get()[r * total_cols + c0 + (c / group) * padded + (c % group)] = v[(size_t)(r * p.cols + c)];
        c0 += (p.cols / group) * padded;
    }
    return host_f32(buf, {rows, total_cols});
}

TensorRequest want(std::vector<int64_t> shape, const char* init) {
    TensorRequest r;
    r.shape = std::move(shape);
    r.init = init;
    return r;
}

int64_t round_up(int64_t n, int64_t m) { return (n + m - 1) / m * m; }

// ---- rotary frequencies ----------------------------------------------------------------------------------------
// f_i = base^(-2i / dims), i < dims / 2.  With `scaling` {factor, low, high, original}: a frequency whose
// wavelength 2 pi / f is shorter than original / high stays, longer than original / low is divided by factor,
// and between the two is the blend (1 - s) f / factor + s f with s = (original / wavelength - low) / (high - low).
std::vector<float> rotary_frequencies(int dims, double base, const Json* scaling) {
    std::vector<float> out;
    for (int i = 0; i < dims / 2; i++) {
        double f = std::pow(base, -2.0 * i / dims);
        if (scaling && scaling->is_object()) {
            const double factor = scaling->at("factor").as_double(), low = scaling->at("low").as_double(),
                         high = scaling->at("high").as_double(), orig = scaling->at("original").as_double();
            const double wavelength = 2.0 * kPi / f;
            if (wavelength < orig / high) {
            } else if (wavelength > orig / low) {
                f /= factor;
            } else {
                const double s = (orig / wavelength - low) / (high - low);
                f = (1.0 - s) * f / factor + s * f;
            }
        }
        out.push_back((float)f);
    }
    return out;
}

DeviceWeight floats_to_device(const std::vector<float>& v) {
    auto buf = alloc_f32(v.size());
    std::copy(v.begin(), v.end(), buf.get());
    return to_device(host_f32(buf, {(int64_t)v.size()}), DType::F32);
}

}  // namespace part_helpers

namespace {
using namespace part_helpers;

// ---- RMS norm --------------------------------------------------------------------------------------------
// Parameters: width, eps.  Tensor: "weight" (a plain gain, not one-plus).
class RMSNorm : public Norm {
public:
    explicit RMSNorm(const PartSpec& s) : Norm(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")) {}
    TensorRequests requests() const override { return {{"weight", want({width_}, "gamma")}}; }
    void bind(const TensorMap& t, DType) override { gain_ = to_device(t.at("weight"), DType::F32); }
    size_t weight_bytes() const override { return gain_.bytes(); }
    void forward(StepContext& ctx, const Tensor& x, Tensor& out, const int* rows, int n_rows) override {
        ops::rmsnorm(ctx.launch, x, &gain_.view, eps_, out, rows, n_rows);
    }
    void forward_add(StepContext& ctx, const Tensor& y, float mult, Tensor& x) override {
        ops::rmsnorm_add(ctx.launch, y, &gain_.view, eps_, mult, x);
    }
    bool rms_params(RmsNormParams& p) const override {
        p.gain = &gain_.view;
        p.eps = eps_;
        return true;
    }
private:
    int64_t width_;
    float eps_;
    DeviceWeight gain_;
};

// ---- feed-forwards -----------------------------------------------------------------------------------------
// "gated_mlp": x (+)= down(act(gate h) * (up h)).  The gate and up matrices are one product.
// Parameters: width, inner, activation ("silu" | "gelu_tanh").  Tensors: "gate", "up", "down", all [out, in].
class GatedMLP : public FeedForward {
public:
    explicit GatedMLP(const PartSpec& s)
        : FeedForward(s), width_(s.get_int("width")), inner_(s.get_int("inner")),
          gate_up_(width_, 2 * inner_, false, "out_in", "gate_up"), down_(inner_, width_, false, "out_in", "down") {
        const std::string a = s.get_string("activation", "silu");
        if (a == "silu") act_ = ops::GluAct::Silu;
        else if (a == "gelu_tanh") act_ = ops::GluAct::GeluTanh;
        else throw ConfigError("gated_mlp: unknown activation '" + a + "'");
    }
    TensorRequests requests() const override {
        return {{"gate", want({inner_, width_})}, {"up", want({inner_, width_})}, {"down", want({width_, inner_})}};
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["gate_up.weight"] = stack_rows({&t.at("gate"), &t.at("up")}, width_);
        m["down.weight"] = t.at("down");
        gate_up_.bind(m, dtype);
        down_.bind(m, dtype);
    }
    size_t weight_bytes() const override { return gate_up_.weight_bytes() + down_.weight_bytes(); }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x) override {
        Workspace& ws = *ctx.workspace;
        Tensor gu = ws.get("ff_gate_up", h.rows(), 2 * inner_, ctx.compute_dtype);
        gate_up_.run(ctx, &h, nullptr, gu, ops::Act::None, nullptr);
        Tensor a = ws.get("ff_inner", h.rows(), inner_, ctx.compute_dtype);
        ops::glu(ctx.launch, gu.col_range(0, inner_), gu.col_range(inner_, 2 * inner_), act_, a);
        down_.run(ctx, nullptr, &a, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t width_, inner_;
    ops::GluAct act_ = ops::GluAct::Silu;
    Linear gate_up_, down_;
};

class NoFeedForward : public FeedForward {
public:
    using FeedForward::FeedForward;
    bool empty() const override { return true; }
    void forward(StepContext&, NormedInput&, Tensor&) override {}
};

// ---- block ---------------------------------------------------------------------------------------------------
// "sandwich_norm": a norm before and a norm after each sublayer; the normed branch joins the stream times a
// constant.  Norm names: "mixer", "mixer_out", "feed_forward", "feed_forward_out" (the last two are not used
// by a layer without a feed-forward).  Parameter: residual_mult.
class SandwichBlock : public Block {
public:
    SandwichBlock(BlockParts p)
        : Block(std::move(p.mixer), std::move(p.feed_forward), std::move(p.norms), p.width) {
        const Json* m = p.params.find("residual_mult");
        mult_ = m && !m->is_null() ? (float)m->as_double() : 1.0f;
    }
    void forward(StepContext& ctx, Tensor& x, const LayerCall& call) override {
        Tensor y = ctx.workspace->get("branch", x.rows, x.cols, DType::F32);
        {
            NormedInput h(ctx, *norms_.at("mixer"), x);
            begin_branch(ctx, y, mixer_->can_overwrite());
            mixer_->forward(ctx, h, y, call);
            ctx.overwrite = false;
            norms_.at("mixer_out")->forward_add(ctx, y, mult_, x);
        }
        if (!ff_->empty()) {
            NormedInput h(ctx, *norms_.at("feed_forward"), x);
            begin_branch(ctx, y, ff_->can_overwrite());
            ff_->forward(ctx, h, y);
            ctx.overwrite = false;
            norms_.at("feed_forward_out")->forward_add(ctx, y, mult_, x);
        }
    }
private:
    // A part that cannot write over its output adds to zeros.
    static void begin_branch(StepContext& ctx, Tensor& y, bool overwrites) {
        ctx.overwrite = overwrites;
        if (!overwrites)
            cuda_check(cudaMemsetAsync(y.data, 0, (size_t)y.numel() * sizeof(float), ctx.launch.stream), "clearing a branch");
    }
    float mult_ = 1.0f;
};

// ---- remix -----------------------------------------------------------------------------------------------------
// "concat_linear": x <- W [x; x0], W [width, 2 width] with the columns for x first.
class ConcatLinear : public Remix {
public:
    explicit ConcatLinear(const PartSpec& s) : Remix(s), width_(s.get_int("width")), linear_(2 * width_, width_, false, "out_in", "mix") {}
    TensorRequests requests() const override { return {{"weight", want({width_, 2 * width_})}}; }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["mix.weight"] = t.at("weight");
        linear_.bind(m, dtype);
    }
    size_t weight_bytes() const override { return linear_.weight_bytes(); }
    void forward(StepContext& ctx, Tensor& x, const Tensor& x0) override {
        Tensor both = ctx.workspace->get("remix_in", x.rows, 2 * width_, ctx.compute_dtype);
        Tensor left = both.col_range(0, width_), right = both.col_range(width_, 2 * width_);
        ops::cast_cols(ctx.launch, x, left);
        ops::cast_cols(ctx.launch, x0, right);
        linear_.run(ctx, nullptr, &both, x, ops::Act::None, nullptr);
    }
private:
    int64_t width_;
    Linear linear_;
};

// ---- attention beside a matrix memory ----------------------------------------------------------------------------
// Parameters: width, eps, left_scale, right_scale,
//   left:  n_heads, n_kv_heads, qk_dim, v_dim, scale, rot_dims, rot_base, rot_scaling (object or null), qk_norm, sink
//   right: n_heads, qk_dim, v_dim, gate_cap
// Tensors: left.q/k/v/o, left.q_norm, left.k_norm, left.sink, left.gate; right.q/k/v/gate/o, right.norm,
// right.i, right.i_bias, right.f, right.f_bias.
//
// Left, per token: q, k, v = W h; RMS norm over the whole q row and the whole k row; rotary on the first rot_dims
// entries of each head; causal softmax attention with exp(sink_h) in the denominator; head h's output times
// sigmoid(w_gate_h . h); output projection.  Keys and values live in pages whose head size is the larger of
// qk_dim and v_dim rounded up to 16, zeros beyond each one's own size.
// Right, per token and head: log i = cap tanh((w_i . h + b_i) / cap), log f = logsigmoid(cap tanh((w_f . h + b_f) / cap));
// the matrix memory's recurrence (csrc/matrix_state.cu) on q / sqrt(qk_dim), k, v; each head's read-out divided by
// its root mean square, times a gain, times sigmoid(W_gate h); output projection.
// The two output projections are one product over [left heads | right heads], the scales folded into the gates.
class AttentionBesideMatrixMemory : public Mixer {
public:
    explicit AttentionBesideMatrixMemory(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")),
          left_scale_((float)s.get_double("left_scale", 1.0)), right_scale_((float)s.get_double("right_scale", 1.0)),
          H_((int)s.get_int("left.n_heads")), G_((int)s.get_int("left.n_kv_heads")), d_((int)s.get_int("left.qk_dim")),
          e_((int)s.get_int("left.v_dim")), scale_((float)s.get_double("left.scale")), rot_dims_((int)s.get_int("left.rot_dims", 0)),
          qk_norm_(s.get_bool("left.qk_norm", true)), has_sink_(s.get_bool("left.sink", true)),
          Hr_((int)s.get_int("right.n_heads")), dr_((int)s.get_int("right.qk_dim")), er_((int)s.get_int("right.v_dim")),
          cap_((float)s.get_double("right.gate_cap")),
          pad_((int)round_up(std::max(d_, e_), 16)),
          n_wide_((int64_t)H_ * d_ + (int64_t)G_ * d_ + (int64_t)G_ * e_ + 2 * (int64_t)Hr_ * dr_ + 2 * (int64_t)Hr_ * er_),
          n_gates_(H_ + 2 * Hr_), k_right_(round_up((int64_t)Hr_ * er_, 8)),
          wide_(width_, n_wide_, false, "out_in", "wide"), gates_(width_, n_gates_, false, "out_in", "gates"),
          out_((int64_t)H_ * pad_ + k_right_, width_, false, "out_in", "out") {
        if (G_ <= 0 || H_ % G_) throw ConfigError("attention_beside_matrix_memory: " + std::to_string(H_) + " heads do not divide into " + std::to_string(G_) + " key/value heads");
        if (rot_dims_ < 0 || rot_dims_ > d_ || rot_dims_ % 2) throw ConfigError("attention_beside_matrix_memory: rot_dims must be even and at most qk_dim");
        if (pad_ > 256) throw ConfigError("attention_beside_matrix_memory: heads wider than 256 are not supported");
        if (dr_ > 256) throw ConfigError("attention_beside_matrix_memory: the matrix memory's qk_dim is at most 256");
        if (!(cap_ > 0)) throw ConfigError("attention_beside_matrix_memory: gate_cap must be positive");
        if (rot_dims_) freq_host_ = rotary_frequencies(rot_dims_, s.get_double("left.rot_base"), s.params.find("left.rot_scaling"));
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["left.q"] = want({(int64_t)H_ * d_, width_});
        r["left.k"] = want({(int64_t)G_ * d_, width_});
        r["left.v"] = want({(int64_t)G_ * e_, width_});
        r["left.o"] = want({width_, (int64_t)H_ * e_});
        r["left.gate"] = want({(int64_t)H_, width_});
        if (qk_norm_) {
            r["left.q_norm"] = want({(int64_t)H_ * d_}, "gamma");
            r["left.k_norm"] = want({(int64_t)G_ * d_}, "gamma");
        }
        if (has_sink_) r["left.sink"] = want({(int64_t)H_}, "bias");
        r["right.q"] = want({(int64_t)Hr_ * dr_, width_});
        r["right.k"] = want({(int64_t)Hr_ * dr_, width_});
        r["right.v"] = want({(int64_t)Hr_ * er_, width_});
        r["right.gate"] = want({(int64_t)Hr_ * er_, width_});
        r["right.o"] = want({width_, (int64_t)Hr_ * er_});
        r["right.norm"] = want({(int64_t)Hr_ * er_}, "gamma");
        r["right.i"] = want({(int64_t)Hr_, width_});
        r["right.i_bias"] = want({(int64_t)Hr_}, "bias");
        r["right.f"] = want({(int64_t)Hr_, width_});
        r["right.f_bias"] = want({(int64_t)Hr_}, "bias");
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["wide.weight"] = stack_rows({&t.at("left.q"), &t.at("left.k"), &t.at("left.v"), &t.at("right.q"), &t.at("right.k"),
                                       &t.at("right.v"), &t.at("right.gate")}, width_);
        m["gates.weight"] = stack_rows({&t.at("left.gate"), &t.at("right.i"), &t.at("right.f")}, width_);
        m["out.weight"] = join_columns({{&t.at("left.o"), (int64_t)H_ * e_, e_, pad_}, {&t.at("right.o"), (int64_t)Hr_ * er_, 0, 0}},
                                       width_, (int64_t)H_ * pad_ + k_right_);
        wide_.bind(m, dtype);
        gates_.bind(m, dtype);
        out_.bind(m, dtype);
        if (qk_norm_) {
            q_gain_ = to_device(t.at("left.q_norm"), DType::F32);
            k_gain_ = to_device(t.at("left.k_norm"), DType::F32);
        }
        if (has_sink_) sink_ = to_device(t.at("left.sink"), DType::F32);
        if (rot_dims_) freq_ = floats_to_device(freq_host_);
        right_gain_ = to_device(t.at("right.norm"), DType::F32);
        gate_bias_ = to_device(stack_rows({&t.at("right.i_bias"), &t.at("right.f_bias")}, 1), DType::F32);
    }
    size_t weight_bytes() const override { return wide_.weight_bytes() + gates_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override {
        return CacheSpec::paged_with_state(G_, pad_, 0, {ops::mlstm_state_floats(Hr_, dr_, er_)});
    }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        Tensor wide = ws.get("mix_wide", T, n_wide_, ctx.compute_dtype);
        wide_.run(ctx, &h, nullptr, wide, ops::Act::None, nullptr);
        Tensor gates = ws.get("mix_gates", T, n_gates_, DType::F32);
        gates_.run(ctx, &h, nullptr, gates, ops::Act::None, nullptr);

        const int64_t k_left = (int64_t)H_ * pad_;
        Tensor heads = ws.get("mix_heads", T, k_left + k_right_, ctx.compute_dtype);
        if (k_right_ != (int64_t)Hr_ * er_)      // the columns that only pad the product must not hold stale numbers
            cuda_check(cudaMemsetAsync(heads.data, 0, (size_t)heads.numel() * heads.elem_size(), l.stream), "clearing padded heads");

        // left: attention over the pages
        const KVView cache = ctx.caches->kv(call.cache);
        const int* table = ctx.block_tables.at((size_t)cache.group);
        Tensor q = ws.get("mix_q", T, k_left, ctx.compute_dtype);
        Tensor head_gate = ws.get("mix_head_gate", T, H_, DType::F32);
        ops::AttentionPrepare p;
        p.n_heads = H_; p.n_kv_heads = G_; p.qk_dim = d_; p.v_dim = e_;
        p.q_off = 0; p.k_off = H_ * d_; p.v_off = (H_ + G_) * d_;
        p.q_gain = qk_norm_ ? (const float*)q_gain_.view.data : nullptr;
        p.k_gain = qk_norm_ ? (const float*)k_gain_.view.data : nullptr;
        p.eps = eps_;
        p.freq = rot_dims_ ? (const float*)freq_.view.data : nullptr;
        p.rot_dims = rot_dims_;
        p.gate_in = (const float*)gates.data;
        p.ld_gate = (int)gates.ld;
        p.gate_out = (float*)head_gate.data;
        p.gate_scale = left_scale_;
        p.write_cache = call.write_cache;
        ops::attention_prepare(l, p, wide, cache, table, ctx.max_blocks, ctx.token_seq, ctx.positions, q);
        Tensor o_left = heads.col_range(0, k_left);
        ops::AttentionExtras extras;
        extras.sink = has_sink_ ? (const float*)sink_.view.data : nullptr;
        extras.out_gate = (const float*)head_gate.data;
        ops::attention(l, ctx.attention_step(cache.group), q, cache, o_left, H_, scale_, 0, ws, &extras);

        // right: the matrix memory
        const StateView state = ctx.caches->state(call.cache);
        ops::StepSeqs seqs{ctx.n_tokens, ctx.n_seqs, ctx.token_seq, ctx.q_start, ctx.seq_slots};
        ops::MlstmShape ms;
        ms.n_heads = Hr_; ms.qk_dim = dr_; ms.v_dim = er_;
        ms.q_off = (H_ + G_) * d_ + G_ * e_;
        ms.k_off = ms.q_off + Hr_ * dr_;
        ms.v_off = ms.k_off + Hr_ * dr_;
        ms.cap = cap_;
        ms.q_scale = 1.0f / std::sqrt((float)dr_);
        Tensor read = ws.get("mix_read", T, (int64_t)Hr_ * er_, DType::F32);
        Tensor gate_cols = gates.col_range(H_, H_ + 2 * Hr_);
        ops::mlstm_scan(l, seqs, ms, wide, gate_cols, (const float*)gate_bias_.view.data, state, read, ctx.max_q_len);
        Tensor o_right = heads.col_range(k_left, k_left + (int64_t)Hr_ * er_);
        Tensor out_gate = wide.col_range(ms.v_off + Hr_ * er_, ms.v_off + 2 * Hr_ * er_);
        ops::head_norm_gate(l, read, &right_gain_.view, &out_gate, ops::GateAct::Sigmoid, right_scale_, eps_, Hr_, o_right);

        out_.run(ctx, nullptr, &heads, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t width_;
    float eps_, left_scale_, right_scale_;
    int H_, G_, d_, e_;
    float scale_;
    int rot_dims_;
    bool qk_norm_, has_sink_;
    int Hr_, dr_, er_;
    float cap_;
    int pad_;
    int64_t n_wide_, n_gates_, k_right_;
    Linear wide_, gates_, out_;
    std::vector<float> freq_host_;
    DeviceWeight q_gain_, k_gain_, sink_, freq_, right_gain_, gate_bias_;
};

// ---- gated delta rule ------------------------------------------------------------------------------------------------
// Parameters: width, eps, n_heads, n_qk_heads, qk_dim, v_dim, conv_taps.
// Tensors: q, k, v, gate, o (matrices), q_conv, k_conv, v_conv ([channels, taps], the last column is the current
// token's), beta, decay ([heads, width]), a_log, dt_bias ([heads]), norm ([v_dim], shared by the heads).
//
// Per token: q, k (n_qk_heads x qk_dim) and v (n_heads x v_dim) = W h; each passes a short causal convolution over
// time per channel and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times
// qk_dim^(-1/2); beta = sigmoid(w_beta . h); decay g = exp(-exp(a_log) softplus(w_decay . h + dt_bias)); the rule
// S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q per head (head j reads q/k head j / (n_heads / n_qk_heads));
// o over its root mean square, times the gain, times silu(W_gate h); output projection.
// A request's state: S [heads][v_dim][qk_dim], then the last conv_taps - 1 inputs of the convolutions.
class GatedDelta : public Mixer {
public:
    explicit GatedDelta(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), H_((int)s.get_int("n_heads")),
          G_((int)s.get_int("n_qk_heads")), d_((int)s.get_int("qk_dim")), e_((int)s.get_int("v_dim")), taps_((int)s.get_int("conv_taps")),
          channels_(2 * (int64_t)G_ * d_ + (int64_t)H_ * e_), n_wide_(channels_ + (int64_t)H_ * e_),
          wide_(width_, n_wide_, false, "out_in", "wide"), gates_(width_, 2 * H_, false, "out_in", "gates"),
          out_((int64_t)H_ * e_, width_, false, "out_in", "out") {
        if (G_ <= 0 || H_ % G_) throw ConfigError("gated_delta: " + std::to_string(H_) + " heads do not divide into " + std::to_string(G_) + " query/key heads");
        if (taps_ < 1 || taps_ > 8) throw ConfigError("gated_delta: 1 to 8 convolution taps are supported, got " + std::to_string(taps_));
        if (d_ > 256) throw ConfigError("gated_delta: qk_dim is at most 256");
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["q"] = want({(int64_t)G_ * d_, width_});
        r["k"] = want({(int64_t)G_ * d_, width_});
        r["v"] = want({(int64_t)H_ * e_, width_});
        r["gate"] = want({(int64_t)H_ * e_, width_});
        r["o"] = want({width_, (int64_t)H_ * e_});
        r["q_conv"] = want({(int64_t)G_ * d_, taps_});
        r["k_conv"] = want({(int64_t)G_ * d_, taps_});
        r["v_conv"] = want({(int64_t)H_ * e_, taps_});
        r["beta"] = want({(int64_t)H_, width_});
        r["decay"] = want({(int64_t)H_, width_});
        r["a_log"] = want({(int64_t)H_}, "bias");
        r["dt_bias"] = want({(int64_t)H_}, "bias");
        r["norm"] = want({(int64_t)e_}, "gamma");
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["wide.weight"] = stack_rows({&t.at("q"), &t.at("k"), &t.at("v"), &t.at("gate")}, width_);
        m["gates.weight"] = stack_rows({&t.at("beta"), &t.at("decay")}, width_);
        m["out.weight"] = t.at("o");
        wide_.bind(m, dtype);
        gates_.bind(m, dtype);
        out_.bind(m, dtype);
        conv_ = to_device(stack_rows({&t.at("q_conv"), &t.at("k_conv"), &t.at("v_conv")}, taps_), DType::F32);
        a_log_ = to_device(t.at("a_log"), DType::F32);
        dt_bias_ = to_device(t.at("dt_bias"), DType::F32);
        gain_ = to_device(t.at("norm"), DType::F32);
    }
    size_t weight_bytes() const override { return wide_.weight_bytes() + gates_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override { return CacheSpec::state({state_floats()}); }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        Tensor wide = ws.get("mix_wide", T, n_wide_, ctx.compute_dtype);
        wide_.run(ctx, &h, nullptr, wide, ops::Act::None, nullptr);
        Tensor gates = ws.get("mix_gates", T, 2 * H_, DType::F32);
        gates_.run(ctx, &h, nullptr, gates, ops::Act::None, nullptr);

        const StateView state = ctx.caches->state(call.cache);
        const int64_t tail_off = (int64_t)H_ * e_ * d_;
        ops::StepSeqs seqs{ctx.n_tokens, ctx.n_seqs, ctx.token_seq, ctx.q_start, ctx.seq_slots};
        ops::DeltaShape ds{H_, G_, d_, e_, taps_};
        Tensor qkv = ws.get("delta_qkv", T, channels_, DType::F32);
        Tensor bg = ws.get("delta_gates", T, 2 * H_, DType::F32);
        ops::delta_prepare(l, seqs, ds, wide, conv_.view, gates, (const float*)a_log_.view.data, (const float*)dt_bias_.view.data,
                           state, tail_off, 1.0f / std::sqrt((float)d_), qkv, bg);
        ops::conv_tail(l, seqs, ds, wide, state, tail_off);
        Tensor read = ws.get("mix_read", T, (int64_t)H_ * e_, DType::F32);
        ops::delta_scan(l, seqs, ds, qkv, bg, state, read, ctx.max_q_len);
        Tensor normed = ws.get("delta_normed", T, (int64_t)H_ * e_, ctx.compute_dtype);
        Tensor out_gate = wide.col_range(channels_, n_wide_);
        ops::head_norm_gate(l, read, &gain_.view, &out_gate, ops::GateAct::Silu, 1.0f, eps_, H_, normed);
        out_.run(ctx, nullptr, &normed, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t state_floats() const { return (int64_t)H_ * e_ * d_ + (int64_t)(taps_ - 1) * channels_; }
    int64_t width_;
    float eps_;
    int H_, G_, d_, e_, taps_;
    int64_t channels_, n_wide_;
    Linear wide_, gates_, out_;
    DeviceWeight conv_, a_log_, dt_bias_, gain_;
};

template <typename T>
PartFactory simple() {
    PartFactory f;
    f.make = [](const PartSpec& s) { return std::unique_ptr<Part>(new T(s)); };
    return f;
}

}  // namespace

void register_hybrid_parts() {
    register_part("norm", "rmsnorm", simple<RMSNorm>());
    register_part("feed_forward", "gated_mlp", simple<GatedMLP>());
    register_part("feed_forward", "none", simple<NoFeedForward>());
    register_part("remix", "concat_linear", simple<ConcatLinear>());
    register_part("mixer", "attention_beside_matrix_memory", simple<AttentionBesideMatrixMemory>());
    register_part("mixer", "gated_delta", simple<GatedDelta>());
    PartFactory sandwich;
    sandwich.norm_names = {"mixer", "mixer_out"};          // "feed_forward" and "feed_forward_out" where the layer has one
    sandwich.make_block = [](BlockParts p) { return std::unique_ptr<Block>(new SandwichBlock(std::move(p))); };
    register_part("block", "sandwich_norm", std::move(sandwich));
}

}  // namespace sandy
