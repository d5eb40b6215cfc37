// Part kinds for decoders whose attention norms what it projects and caps its scores.
//
//   mixer   "normed_attention"   grouped-query softmax attention without positions in its scores, with any of:
//                                a token shift on its input, biases, an RMS norm over the whole query row and the whole
//                                key row, values of unit root mean square per head, a learned temperature per head,
//                                scores pressed through softcap * tanh(score / softcap), and chunks of positions
//                                (a query sees the keys of its own chunk only)
//   remix   "add_row"            x += x0 + row: the stream re-enters a looped span by addition (the embedding's
//                                output, and one row of a learned table per pass)
//
// Every size and constant is a parameter of the part.  Norms, the token shift, scores, softmax and the residual sum
// are 32-bit in both compute types; the matrix products run in the compute type.
#include <cmath>

#include "part_helpers.h"
#include "parts.h"

namespace sandy {
namespace {
using namespace part_helpers;

// ---- attention ------------------------------------------------------------------------------------------------
// Parameters: width, eps, n_heads, n_kv_heads, qk_dim, v_dim, scale, bias, qk_norm, v_norm, head_temperature,
//   softcap (0: none), chunk (0: none), window (null: none), token_shift.
// Tensors: q, k, v, o ([out, in]); with bias q_bias, k_bias, v_bias, o_bias; with qk_norm q_norm [H * qk_dim] and
//   k_norm [G * qk_dim] (plain gains); with head_temperature temperature [H]; with token_shift shift [width].
//
// Per token, h being the normed stream row the block hands over:
//   token shift   h <- h + (h_before - h) * shift, h_before the token before's h as the norm left it (zeros at a
//                 request's first token); the last h of a request is its state between steps.  The kernel runs the
//                 norm itself on the float32 stream, so the block's norm must be an RMS norm.
//   q, k, v       = W h + b, one product; RMS norm over all of q and over all of k with their gains; every value head
//                 over its own root mean square (no gain); the cache holds keys and values in this form
//   score(i, j)   = softcap * tanh((q_i . k_j) * scale * temperature[head] / softcap), j <= i in i's chunk / window
//   x            += W_o [heads] + b_o
// Keys and values live in pages whose head size is the larger of qk_dim and v_dim rounded up to 16, zeros beyond
// each one's own size; the temperature reaches the scores through the query.
class NormedAttention : public Mixer {
public:
    explicit NormedAttention(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), H_((int)s.get_int("n_heads")),
          G_((int)s.get_int("n_kv_heads", s.get_int("n_heads"))), d_((int)s.get_int("qk_dim")), e_((int)s.get_int("v_dim")),
          scale_((float)s.get_double("scale")), bias_(s.get_bool("bias", false)), qk_norm_(s.get_bool("qk_norm", false)),
          v_norm_(s.get_bool("v_norm", false)), temperature_(s.get_bool("head_temperature", false)),
          softcap_((float)s.get_double("softcap", 0.0)), chunk_((int)s.get_int("chunk", 0)),
          window_((int)s.get_optional_int("window").value_or(0)), shift_(s.get_bool("token_shift", false)),
          pad_((int)round_up(std::max(d_, e_), 16)), n_wide_((int64_t)H_ * d_ + (int64_t)G_ * d_ + (int64_t)G_ * e_),
          wide_(width_, n_wide_, bias_, "out_in", "wide"), out_((int64_t)H_ * pad_, width_, bias_, "out_in", "out") {
        if (G_ <= 0 || H_ <= 0 || H_ % G_)
            throw ConfigError("normed_attention: " + std::to_string(H_) + " heads do not divide into " + std::to_string(G_) + " key/value heads");
        if (d_ <= 0 || e_ <= 0 || pad_ > ops::kMaxHeadDim)
            throw ConfigError("normed_attention: head sizes must be 1 .. " + std::to_string(ops::kMaxHeadDim));
        if (softcap_ < 0.0f || chunk_ < 0) throw ConfigError("normed_attention: softcap and chunk must not be negative");
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["q"] = want({(int64_t)H_ * d_, width_});
        r["k"] = want({(int64_t)G_ * d_, width_});
        r["v"] = want({(int64_t)G_ * e_, width_});
        r["o"] = want({width_, (int64_t)H_ * e_});
        if (bias_) {
            r["q_bias"] = want({(int64_t)H_ * d_}, "bias");
            r["k_bias"] = want({(int64_t)G_ * d_}, "bias");
            r["v_bias"] = want({(int64_t)G_ * e_}, "bias");
            r["o_bias"] = want({width_}, "bias");
        }
        if (qk_norm_) {
            r["q_norm"] = want({(int64_t)H_ * d_}, "gamma");
            r["k_norm"] = want({(int64_t)G_ * d_}, "gamma");
        }
        if (temperature_) r["temperature"] = want({(int64_t)H_}, "gamma");
        if (shift_) r["shift"] = want({width_}, "bias");
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["wide.weight"] = stack_rows({&t.at("q"), &t.at("k"), &t.at("v")}, width_);
        m["out.weight"] = join_columns({{&t.at("o"), (int64_t)H_ * e_, e_, pad_}}, width_, (int64_t)H_ * pad_);
        if (bias_) {
            HostTensor b = stack_rows({&t.at("q_bias"), &t.at("k_bias"), &t.at("v_bias")}, 1);
            b.shape = {n_wide_};
            m["wide.bias"] = b;
            m["out.bias"] = t.at("o_bias");
        }
        wide_.bind(m, dtype);
        out_.bind(m, dtype);
        if (qk_norm_) {
            q_gain_ = to_device(t.at("q_norm"), DType::F32);
            k_gain_ = to_device(t.at("k_norm"), DType::F32);
        }
        if (temperature_) temp_ = to_device(t.at("temperature"), DType::F32);
        if (shift_) mix_ = to_device(t.at("shift"), DType::F32);
    }
    size_t weight_bytes() const override { return wide_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override {
        return shift_ ? CacheSpec::paged_with_state(G_, pad_, window_, {width_}) : CacheSpec::paged(G_, pad_, window_);
    }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        Tensor wide = ws.get("mix_wide", T, n_wide_, ctx.compute_dtype);
        if (shift_) {
            RmsNormParams norm;
            if (!h.rms(norm)) throw ConfigError("normed_attention: a token shift needs an RMS norm in front of the mixer");
            Tensor shifted = ws.get("mix_shifted", T, width_, ctx.compute_dtype);
            ops::StepSeqs seqs{ctx.n_tokens, ctx.n_seqs, ctx.token_seq, ctx.q_start, ctx.seq_slots};
            ops::rmsnorm_shift(l, seqs, norm.x, norm.gain, norm.eps, mix_.view, ctx.caches->state(call.cache), shifted, ctx.max_q_len);
            wide_.run(ctx, nullptr, &shifted, wide, ops::Act::None, nullptr);
        } else {
            wide_.run(ctx, &h, nullptr, wide, ops::Act::None, nullptr);
        }
        const KVView cache = ctx.caches->kv(call.cache);
        const int* table = ctx.block_tables.at((size_t)cache.group);
        Tensor q = ws.get("mix_q", T, (int64_t)H_ * pad_, ctx.compute_dtype);
        ops::AttentionPrepare p;
        p.n_heads = H_; p.n_kv_heads = G_; p.qk_dim = d_; p.v_dim = e_;
        p.q_off = 0; p.k_off = H_ * d_; p.v_off = (H_ + G_) * d_;
        p.q_gain = qk_norm_ ? (const float*)q_gain_.view.data : nullptr;
        p.k_gain = qk_norm_ ? (const float*)k_gain_.view.data : nullptr;
        p.eps = eps_;
        p.q_head_scale = temperature_ ? (const float*)temp_.view.data : nullptr;
        p.v_unit_eps = v_norm_ ? eps_ : 0.0f;
        p.write_cache = call.write_cache;
        ops::attention_prepare(l, p, wide, cache, table, ctx.max_blocks, ctx.token_seq, ctx.positions, q);
        Tensor heads = ws.get("mix_heads", T, (int64_t)H_ * pad_, ctx.compute_dtype);
        ops::AttentionExtras extras;
        extras.softcap = softcap_;
        extras.chunk = chunk_;
        ops::attention(l, ctx.attention_step(cache.group), q, cache, heads, H_, scale_, window_, ws, &extras);
        out_.run(ctx, nullptr, &heads, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t width_;
    float eps_;
    int H_, G_, d_, e_;
    float scale_;
    bool bias_, qk_norm_, v_norm_, temperature_;
    float softcap_;
    int chunk_, window_;
    bool shift_;
    int pad_;
    int64_t n_wide_;
    Linear wide_, out_;
    DeviceWeight q_gain_, k_gain_, temp_, mix_;
};

// ---- remix ------------------------------------------------------------------------------------------------------
// "add_row": x += x0 (with add_embedding) + table[row].  Parameters: width, rows, row, add_embedding.
// Tensor: "table" [rows, width]; the part keeps its own row, in 32-bit.
class AddRow : public Remix {
public:
    explicit AddRow(const PartSpec& s)
        : Remix(s), width_(s.get_int("width")), rows_(s.get_int("rows")), row_(s.get_int("row")),
          add_embedding_(s.get_bool("add_embedding", false)) {
        if (row_ < 0 || row_ >= rows_) throw ConfigError("add_row: row " + std::to_string(row_) + " of a table of " + std::to_string(rows_));
    }
    TensorRequests requests() const override { return {{"table", want({rows_, width_}, "bias")}}; }
    void bind(const TensorMap& t, DType) override {
        const std::vector<float> all = to_f32(t.at("table"));
        vec_ = floats_to_device(std::vector<float>(all.begin() + row_ * width_, all.begin() + (row_ + 1) * width_));
    }
    size_t weight_bytes() const override { return vec_.bytes(); }
    void forward(StepContext& ctx, Tensor& x, const Tensor& x0) override {
        ops::stream_add(ctx.launch, x, add_embedding_ ? &x0 : nullptr, &vec_.view);
    }
private:
    int64_t width_, rows_, row_;
    bool add_embedding_;
    DeviceWeight vec_;
};

template <typename T>
PartFactory simple() {
    PartFactory f;
    f.make = [](const PartSpec& s) { return std::unique_ptr<Part>(new T(s)); };
    return f;
}

}  // namespace

void register_capped_parts() {
    register_part("mixer", "normed_attention", simple<NormedAttention>());
    register_part("remix", "add_row", simple<AddRow>());
}

}  // namespace sandy
