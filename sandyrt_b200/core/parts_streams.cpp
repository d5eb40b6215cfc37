// Part kinds for decoders that keep the residual stream in several copies and mix attention with state-space layers.
//
//   embedding  "bigram_embedding"     x = E[token] + B[(token_before * a + token * b) mod n] + position table; a request's
//                                     first token reads row n of B; the token before is state of the request
//   wrap       "hyper_gated_conv"     around one sublayer: u = sum_s in[s] X_s; h = LayerNorm(u) (a gain, no offset);
//                                     the sublayer reads h + conv(h), a short causal convolution over time per channel;
//                                     its result y joins every copy, X_t <- sum_s mix[s, t] X_s + out[t] y sigmoid(W h + b)
//   block      "wrapped_sublayers"    mixer, then feed-forward, each inside its wrap; the write of the first sublayer and
//                                     the read of the second are one pass over the streams
//   mixer      "biased_attention"     grouped-query softmax attention without rotation: query and key heads over their own
//                                     root mean square, a factor on the query that grows with the logarithm of the position,
//                                     and a learned bias by distance in logarithmic buckets on the scores
//   mixer      "state_space"          Mamba-2: one input projection, a short convolution with silu, a matrix state per head
//                                     with one decay per head and step, a gate, a norm in groups, an output projection
//
// Every size and constant is a parameter of the part.  Norms, the streams and every sum into them, gates of the stream,
// positions, scores and softmax, step sizes, decays and the recurrent state are 32-bit in both compute types; the matrix
// products, the convolutions' inputs and the projections' outputs are in the compute type.
#include <cmath>

#include "part_helpers.h"
#include "parts.h"

namespace sandy {
namespace {
using namespace part_helpers;

ops::StepSeqs seqs_of(const StepContext& ctx) { return ops::StepSeqs{ctx.n_tokens, ctx.n_seqs, ctx.token_seq, ctx.q_start, ctx.seq_slots}; }

// Rows r0 .. r1-1 of a [rows, cols] matrix.
HostTensor slice_rows(const HostTensor& t, int64_t r0, int64_t r1, int64_t cols) {
    const std::vector<float> all = to_f32(t);
    auto buf = alloc_f32((size_t)((r1 - r0) * cols));
    std::copy(all.begin() + r0 * cols, all.begin() + r1 * cols, buf.get());
    return host_f32(buf, {r1 - r0, cols});
}

int64_t floats_of(const CacheSpec& s) {
    int64_t n = s.has_state() ? 1 : 0;
    for (int64_t d : s.state_shape) n *= d;
    return n;
}

// ---- embedding ---------------------------------------------------------------------------------------------------
// Parameters: vocab_size, width, buckets, mul_prev, mul_cur.  Tensors: "weight" [vocab, width], "bigram" [buckets + 1, width].
// The position encoding's table, where it has one, is added in the same pass.
class BigramEmbedding : public Embedding {
public:
    explicit BigramEmbedding(const PartSpec& s)
        : Embedding(s), vocab_(s.get_int("vocab_size")), width_(s.get_int("width")), buckets_(s.get_int("buckets")),
          mul_prev_(s.get_int("mul_prev")), mul_cur_(s.get_int("mul_cur")) {
        if (buckets_ < 1 || buckets_ > 0x7fffffff || mul_prev_ < 0 || mul_cur_ < 0 || mul_prev_ > 0x7fffffff || mul_cur_ > 0x7fffffff)
            throw ConfigError("bigram_embedding: buckets must be positive and the multipliers 0 .. 2^31 - 1");
    }
    TensorRequests requests() const override { return {{"weight", want({vocab_, width_})}, {"bigram", want({buckets_ + 1, width_})}}; }
    void bind(const TensorMap& t, DType dtype) override {
        weight_ = to_device(t.at("weight"), dtype);
        bigram_ = to_device(t.at("bigram"), dtype);
    }
    const Tensor* table() const override { return &weight_.view; }
    CacheSpec cache_spec() const override { return CacheSpec::state({1}, DType::I32); }
    void forward(StepContext& ctx, Tensor& x) override {
        if (ctx.embedding_cache < 0) throw ConfigError("bigram_embedding: the model's description names no cache entry for the token before");
        const Tensor* pos = ctx.position ? ctx.position->table() : nullptr;
        ops::BigramEmbed b;
        b.buckets = (int)buckets_;
        b.mul_prev = mul_prev_;
        b.mul_cur = mul_cur_;
        ops::embed_bigram(ctx.launch, seqs_of(ctx), ctx.token_ids, ctx.positions, weight_.view, bigram_.view, pos, b,
                          ctx.caches->state(ctx.embedding_cache), x, ctx.max_q_len);
    }
private:
    int64_t vocab_, width_, buckets_, mul_prev_, mul_cur_;
    DeviceWeight weight_, bigram_;
};

// ---- wrap ------------------------------------------------------------------------------------------------------------
// Parameters: width, streams, eps, taps (0: no convolution), gate (bool).
// Tensors: "norm" [width], "in" [streams], "out" [streams], "mix" [streams, streams] indexed [from, to]; with taps
// "conv" [width, taps] (the last column is the token's own); with gate "gate" [width, width] and "gate_bias" [width].
// Between steps a request keeps the last taps - 1 rows of h (zeros at its start).
class HyperGatedConv : public Wrap {
public:
    explicit HyperGatedConv(const PartSpec& s)
        : Wrap(s), width_(s.get_int("width")), S_((int)s.get_int("streams")), eps_((float)s.get_double("eps")),
          taps_((int)s.get_int("taps", 0)), gate_lin_(width_, width_, false, "out_in", "gate") {
        if (S_ < 1) throw ConfigError("hyper_gated_conv: at least one stream");
        if (taps_ < 0 || taps_ > 8) throw ConfigError("hyper_gated_conv: 0 to 8 convolution taps are supported, got " + std::to_string(taps_));
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["norm"] = want({width_}, "gamma");
        r["in"] = want({(int64_t)S_}, "gamma");
        r["out"] = want({(int64_t)S_}, "gamma");
        r["mix"] = want({(int64_t)S_, (int64_t)S_}, "gamma");
        if (taps_) r["conv"] = want({width_, (int64_t)taps_});
        r["gate"] = want({width_, width_});
        r["gate_bias"] = want({width_}, "bias");
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        gain_ = to_device(t.at("norm"), DType::F32);
        in_ = to_device(t.at("in"), DType::F32);
        out_ = to_device(t.at("out"), DType::F32);
        mix_ = to_device(t.at("mix"), DType::F32);
        if (taps_) conv_ = to_device(t.at("conv"), DType::F32);
        TensorMap m;
        m["gate.weight"] = t.at("gate");
        gate_lin_.bind(m, dtype);      // the product writes W h; the bias joins in the pass that uses the gate, in 32-bit
        gate_bias_ = to_device(t.at("gate_bias"), DType::F32);
        if (S_ > ops::streams_max()) throw ConfigError("hyper_gated_conv: at most " + std::to_string(ops::streams_max()) + " streams");
    }
    size_t weight_bytes() const override { return gate_lin_.weight_bytes() + gain_.bytes() + (taps_ ? conv_.bytes() : 0); }
    int64_t state_floats() const override { return taps_ > 1 ? (int64_t)(taps_ - 1) * width_ : 0; }
    void fill_write(ops::StreamsStep& st, const Tensor* y, const Input* in) const {
        st.y = y;
        st.gate = &in->gate;
        st.gate_bias = &gate_bias_.view;
        st.mix = &mix_.view;
        st.out_w = &out_.view;
    }
    Input read(StepContext& ctx, Tensor& X, const StateView* state, int64_t offset, Wrap* before, const Tensor* before_y,
               const Input* before_in) override {
        Workspace& ws = *ctx.workspace;
        const int64_t T = X.rows;
        Tensor h = ws.get("wrap_normed", T, width_, ctx.compute_dtype);
        ops::StreamsStep st;
        if (before) {
            auto* b = dynamic_cast<HyperGatedConv*>(before);
            if (!b) throw ConfigError("hyper_gated_conv: the wrap before is of another kind");
            b->fill_write(st, before_y, before_in);
        }
        st.in_w = &in_.view;
        st.gain = &gain_.view;
        st.eps = eps_;
        st.h = &h;
        Input out;
        StateView none;
        const StateView& sv = state ? *state : none;
        const ops::StepSeqs seqs = seqs_of(ctx);
        // a step of single tokens: the convolution and its tail ride in the same launch
        const bool fused = taps_ && ctx.max_q_len <= 1;
        if (taps_) out.sublayer_in = ws.get("wrap_sublayer_in", T, width_, ctx.compute_dtype);
        else out.sublayer_in = h;
        if (fused) {
            st.taps = &conv_.view;
            st.n_taps = taps_;
            st.state = &sv;
            st.tail_off = offset;
            st.seqs = &seqs;
            st.conv_out = &out.sublayer_in;
        }
        ops::streams_step(ctx.launch, X, S_, st);
        if (taps_ && !fused) {
            ops::canon_conv(ctx.launch, seqs, h, conv_.view, taps_, sv, offset, out.sublayer_in);
            if (taps_ > 1) ops::conv_tail(ctx.launch, seqs, h, taps_, sv, offset);
        }
        out.gate = ws.get("wrap_gate", T, width_, DType::F32);
        gate_lin_.run(ctx, nullptr, &h, out.gate, ops::Act::None, nullptr);
        return out;
    }
    void write(StepContext& ctx, Tensor& X, const Tensor& y, const Input& in, Tensor* sum_out) override {
        ops::StreamsStep st;
        fill_write(st, &y, &in);
        st.sum_out = sum_out;
        ops::streams_step(ctx.launch, X, S_, st);
    }
private:
    int64_t width_;
    int S_;
    float eps_;
    int taps_;
    Linear gate_lin_;
    DeviceWeight gain_, in_, out_, mix_, conv_, gate_bias_;
};

// ---- block -----------------------------------------------------------------------------------------------------------
// "wrapped_sublayers": wraps "mixer" and (where the layer has a feed-forward) "feed_forward".  The wraps' states follow
// the mixer's own in the layer's cache entry.
class WrappedSublayers : public Block {
public:
    explicit WrappedSublayers(BlockParts p) : Block(std::move(p.mixer), std::move(p.feed_forward), std::move(p.norms), p.width) {
        wraps_ = std::move(p.wraps);
        if (!wraps_.count("mixer") || (!ff_->empty() && !wraps_.count("feed_forward")))
            throw ConfigError("block 'wrapped_sublayers' needs a wrap for every sublayer");
    }
    CacheSpec cache_spec() const override {
        const CacheSpec m = mixer_->cache_spec();
        int64_t extra = 0;
        for (const auto& kv : wraps_) extra += kv.second->state_floats();
        if (extra == 0) return m;
        if (m.has_state() && m.state_dtype != DType::F32) throw ConfigError("wrapped_sublayers: the mixer's state must be float32");
        const int64_t own = floats_of(m);
        if (m.has_pages()) {
            if (m.planes != 2) throw ConfigError("wrapped_sublayers: one-plane pages beside a state are not supported");
            return CacheSpec::paged_with_state(m.n_kv_heads, m.head_dim, m.window, {own + extra});
        }
        return CacheSpec::state({own + extra});
    }
    bool settles_owed() const override { return true; }
    void forward(StepContext& ctx, Tensor& X, const LayerCall& call) override {
        Wrap& w1 = *wraps_.at("mixer");
        Wrap* w2 = ff_->empty() ? nullptr : wraps_.at("feed_forward").get();
        const int64_t own = floats_of(mixer_->cache_spec());
        const bool stateful = w1.state_floats() + (w2 ? w2->state_floats() : 0) > 0;
        StateView state;
        if (stateful) state = ctx.caches->state(call.cache);
        const StateView* sv = stateful ? &state : nullptr;
        // the write that the block before left owed rides in this block's first pass over the streams
        StepContext::OwedWrite owed = ctx.owed;
        ctx.owed = StepContext::OwedWrite();
        Wrap::Input owed_in;
        owed_in.gate = owed.gate;
        Wrap::Input in1 = w1.read(ctx, X, sv, own, owed.wrap, owed.wrap ? &owed.y : nullptr, owed.wrap ? &owed_in : nullptr);
        Tensor y = ctx.workspace->get("branch", X.rows, width_, DType::F32);
        {
            NormedInput h(ctx, in1.sublayer_in);
            begin_branch(ctx, y, mixer_->can_overwrite());
            mixer_->forward(ctx, h, y, call);
            ctx.overwrite = false;
        }
        if (!w2) {
            leave_owed(ctx, w1, y, in1);
            return;
        }
        Wrap::Input in2 = w2->read(ctx, X, sv, own + w1.state_floats(), &w1, &y, &in1);
        {
            NormedInput h(ctx, in2.sublayer_in);
            begin_branch(ctx, y, ff_->can_overwrite());
            ff_->forward(ctx, h, y);
            ctx.overwrite = false;
        }
        leave_owed(ctx, *w2, y, in2);
    }
private:
    // The last sublayer's write waits for the next pass over the streams (StepContext::owed): its result and its gate sit
    // in workspace buffers that nothing touches before that pass has read them.
    static void leave_owed(StepContext& ctx, Wrap& w, const Tensor& y, const Wrap::Input& in) {
        ctx.owed.wrap = &w;
        ctx.owed.y = y;
        ctx.owed.gate = in.gate;
    }
    static void begin_branch(StepContext& ctx, Tensor& y, bool overwrites) {
        ctx.overwrite = overwrites;
        if (!overwrites)
            cuda_check(cudaMemsetAsync(y.data, 0, (size_t)y.numel() * sizeof(float), ctx.launch.stream), "clearing a branch");
    }
};

// ---- attention with a bias by distance ---------------------------------------------------------------------------------
// Parameters: width, eps, n_heads, n_kv_heads, qk_dim, v_dim, scale, qk_unit_norm (bool), q_pos_coef, q_pos_every (0: no
//   factor by position), distance_bias (bool), bias_max, bias_rows (0 or absent: as many as the tensor has).
// Tensors: q, k, v, o ([out, in]); with distance_bias "rel" [bias_rows, n_heads].
//
// Per token: q, k, v = W h; with qk_unit_norm every query head and every key head over its own root mean square (eps
// inside the root, no gain); the query at position p times 1 + q_pos_coef ln(floor((p + 1) / q_pos_every) + 1);
//   score(i, j) = (q_i . k_j) scale + rel[bucket(i - j), head],  j <= i
//   bucket(n)   = n below half = bias_rows / 2, else min(bias_rows - 1, half + floor(ln(n / half) / ln(bias_max / half) (bias_rows - half)))
// softmax, x += W_o [heads].  The buckets are laid out by distance once, when the part binds: entry min(n, bias_max) of a
// head's row of a table [heads, bias_max + 1] (every distance from bias_max on falls into the last bucket).
// Keys and values live in pages whose head size is the larger of qk_dim and v_dim rounded up to 16.
class BiasedAttention : public Mixer {
public:
    explicit BiasedAttention(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), H_((int)s.get_int("n_heads")),
          G_((int)s.get_int("n_kv_heads", s.get_int("n_heads"))), d_((int)s.get_int("qk_dim")), e_((int)s.get_int("v_dim")),
          scale_((float)s.get_double("scale")), unit_(s.get_bool("qk_unit_norm", false)), pos_coef_((float)s.get_double("q_pos_coef", 0.0)),
          pos_every_((int)s.get_int("q_pos_every", 0)), biased_(s.get_bool("distance_bias", false)), rows_(s.get_int("bias_rows", 0)),
          far_(s.get_int("bias_max", 0)),
          pad_((int)round_up(std::max(d_, e_), 16)), n_wide_((int64_t)H_ * d_ + (int64_t)G_ * d_ + (int64_t)G_ * e_),
          wide_(width_, n_wide_, false, "out_in", "wide"), out_((int64_t)H_ * pad_, width_, false, "out_in", "out") {
        if (G_ <= 0 || H_ <= 0 || H_ % G_)
            throw ConfigError("biased_attention: " + std::to_string(H_) + " heads do not divide into " + std::to_string(G_) + " key/value heads");
        if (d_ <= 0 || e_ <= 0 || pad_ > ops::kMaxHeadDim)
            throw ConfigError("biased_attention: head sizes must be 1 .. " + std::to_string(ops::kMaxHeadDim));
        if (pos_every_ < 0) throw ConfigError("biased_attention: q_pos_every must not be negative");
        if (biased_) check_bias(rows_);
    }
    void check_bias(int64_t rows) const {
        if (rows < 0 || far_ < 2 || far_ > (1 << 24) || (rows > 0 && (rows < 2 || far_ <= rows / 2)))
            throw ConfigError("biased_attention: the bias table has at least 2 rows, and bias_max lies beyond half of them (at most 2^24); got " +
                              std::to_string(rows) + " rows and bias_max " + std::to_string(far_));
    }
    static int64_t bucket(int64_t n, int64_t rows, int64_t far) {
        const int64_t half = rows / 2;
        if (n < half) return n;
        const double f = std::log((double)n / (double)half) / std::log((double)far / (double)half) * (double)(rows - half);
        return std::min(rows - 1, half + (int64_t)std::floor(f));
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["q"] = want({(int64_t)H_ * d_, width_});
        r["k"] = want({(int64_t)G_ * d_, width_});
        r["v"] = want({(int64_t)G_ * e_, width_});
        r["o"] = want({width_, (int64_t)H_ * e_});
        if (biased_) r["rel"] = want({rows_ > 0 ? rows_ : -1, (int64_t)H_}, "bias");
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["wide.weight"] = stack_rows({&t.at("q"), &t.at("k"), &t.at("v")}, width_);
        m["out.weight"] = join_columns({{&t.at("o"), (int64_t)H_ * e_, e_, pad_}}, width_, (int64_t)H_ * pad_);
        wide_.bind(m, dtype);
        out_.bind(m, dtype);
        if (biased_) {
            const int64_t rows = t.at("rel").shape.at(0);
            check_bias(rows);
            if (rows < 2) throw ConfigError("biased_attention: the bias table has at least 2 rows");
            const std::vector<float> rel = to_f32(t.at("rel"));
            std::vector<float> by_distance((size_t)(far_ + 1) * H_);
            for (int64_t n = 0; n <= far_; n++) {
                const int64_t b = bucket(n, rows, far_);
                for (int h = 0; h < H_; h++) by_distance[(size_t)h * (far_ + 1) + n] = rel[(size_t)b * H_ + h];
            }
            bias_ = floats_to_device(by_distance);
        }
    }
    size_t weight_bytes() const override { return wide_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override { return CacheSpec::paged(G_, pad_, 0); }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        Tensor wide = ws.get("mix_wide", T, n_wide_, ctx.compute_dtype);
        wide_.run(ctx, &h, nullptr, wide, ops::Act::None, nullptr);
        const KVView cache = ctx.caches->kv(call.cache);
        const int* table = ctx.block_tables.at((size_t)cache.group);
        Tensor q = ws.get("mix_q", T, (int64_t)H_ * pad_, ctx.compute_dtype);
        ops::AttentionPrepare p;
        p.n_heads = H_; p.n_kv_heads = G_; p.qk_dim = d_; p.v_dim = e_;
        p.q_off = 0; p.k_off = H_ * d_; p.v_off = (H_ + G_) * d_;
        p.eps = eps_;
        p.per_head_norm = unit_;
        p.q_pos_coef = pos_coef_;
        p.q_pos_every = pos_every_;
        p.write_cache = call.write_cache;
        ops::attention_prepare(l, p, wide, cache, table, ctx.max_blocks, ctx.token_seq, ctx.positions, q);
        Tensor heads = ws.get("mix_heads", T, (int64_t)H_ * pad_, ctx.compute_dtype);
        ops::AttentionExtras extras;
        if (biased_) {
            extras.dist_bias = (const float*)bias_.view.data;
            extras.n_dist = (int)far_ + 1;
        }
        ops::attention(l, ctx.attention_step(cache.group), q, cache, heads, H_, scale_, 0, ws, &extras);
        out_.run(ctx, nullptr, &heads, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t width_;
    float eps_;
    int H_, G_, d_, e_;
    float scale_;
    bool unit_;
    float pos_coef_;
    int pos_every_;
    bool biased_;
    int64_t rows_, far_;
    int pad_;
    int64_t n_wide_;
    Linear wide_, out_;
    DeviceWeight bias_;
};

// ---- state-space mixer ----------------------------------------------------------------------------------------------------
// Parameters: width, eps, n_heads, n_groups, state, v_dim, conv_taps, norm_groups.
// Tensors: "in" [2 inner + 2 G N + H, width] laid out as (z: inner | x: inner | B: G N | C: G N | dt: H), inner = H * v_dim;
//   "conv" [inner + 2 G N, taps] (the last column is the token's own) and "conv_bias"; "dt_bias", "a_log", "d" [H];
//   "norm" [inner]; "o" [width, inner].
//
// Per token: (x, B, C) <- silu(causal conv + bias); dt <- softplus(dt + dt_bias), no clamp; per head (head h reads group
// h / (H / G)):  S <- exp(-exp(a_log) dt) S + dt B x^T,  y = S^T C + d x;  y (heads side by side) times silu(z), then over
// its root mean square in norm_groups equal parts (eps inside the root), times the gain; x += W_o y.
// The dt columns are a product of their own, written in float32: they enter exponentials and the recurrence.
// A request's state: S [H][v_dim][N] float32, then the last conv_taps - 1 inputs of the convolution.
class StateSpace : public Mixer {
public:
    explicit StateSpace(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), H_((int)s.get_int("n_heads")),
          G_((int)s.get_int("n_groups")), N_((int)s.get_int("state")), P_((int)s.get_int("v_dim")), taps_((int)s.get_int("conv_taps")),
          parts_((int)s.get_int("norm_groups", 1)), inner_((int64_t)H_ * P_), channels_(inner_ + 2 * (int64_t)G_ * N_),
          wide_(width_, inner_ + channels_, false, "out_in", "wide"), dt_(width_, H_, false, "out_in", "dt"),
          out_(inner_, width_, false, "out_in", "out") {
        if (G_ <= 0 || H_ <= 0 || H_ % G_) throw ConfigError("state_space: " + std::to_string(H_) + " heads do not divide into " + std::to_string(G_) + " groups");
        if (taps_ < 1 || taps_ > 8) throw ConfigError("state_space: 1 to 8 convolution taps are supported, got " + std::to_string(taps_));
        if (N_ < 1 || N_ > 256) throw ConfigError("state_space: the state size is 1 .. 256");
        if (P_ < 1) throw ConfigError("state_space: v_dim must be positive");
        if (parts_ < 1 || inner_ % parts_) throw ConfigError("state_space: norm_groups must divide heads * v_dim");
    }
    TensorRequests requests() const override {
        TensorRequests r;
        r["in"] = want({inner_ + channels_ + H_, width_});
        r["conv"] = want({channels_, (int64_t)taps_});
        r["conv_bias"] = want({channels_}, "bias");
        r["dt_bias"] = want({(int64_t)H_}, "bias");
        r["a_log"] = want({(int64_t)H_}, "bias");
        r["d"] = want({(int64_t)H_}, "gamma");
        r["norm"] = want({inner_}, "gamma");
        r["o"] = want({width_, inner_});
        return r;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["wide.weight"] = slice_rows(t.at("in"), 0, inner_ + channels_, width_);
        m["dt.weight"] = slice_rows(t.at("in"), inner_ + channels_, inner_ + channels_ + H_, width_);
        m["out.weight"] = t.at("o");
        wide_.bind(m, dtype);
        dt_.bind(m, dtype);
        out_.bind(m, dtype);
        conv_ = to_device(t.at("conv"), DType::F32);
        conv_bias_ = to_device(t.at("conv_bias"), DType::F32);
        dt_bias_ = to_device(t.at("dt_bias"), DType::F32);
        a_log_ = to_device(t.at("a_log"), DType::F32);
        d_ = to_device(t.at("d"), DType::F32);
        gain_ = to_device(t.at("norm"), DType::F32);
    }
    size_t weight_bytes() const override { return wide_.weight_bytes() + dt_.weight_bytes() + out_.weight_bytes(); }
    CacheSpec cache_spec() const override { return CacheSpec::state({ops::ssm_state_floats(shape()) + (int64_t)(taps_ - 1) * channels_}); }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        Tensor wide = ws.get("mix_wide", T, inner_ + channels_, ctx.compute_dtype);
        wide_.run(ctx, &h, nullptr, wide, ops::Act::None, nullptr);
        Tensor dt_raw = ws.get("mix_gates", T, H_, DType::F32);
        dt_.run(ctx, &h, nullptr, dt_raw, ops::Act::None, nullptr);

        const StateView state = ctx.caches->state(call.cache);
        const ops::SsmShape m = shape();
        const int64_t tail_off = ops::ssm_state_floats(m);
        const ops::StepSeqs seqs = seqs_of(ctx);
        Tensor z = wide.col_range(0, inner_), xbc_in = wide.col_range(inner_, inner_ + channels_);
        Tensor xbc = ws.get("ssm_xbc", T, channels_, DType::F32);
        Tensor dta = ws.get("ssm_dt", T, 2 * H_, DType::F32);
        ops::ssm_prepare(l, seqs, m, xbc_in, conv_.view, &conv_bias_.view, dt_raw, (const float*)dt_bias_.view.data,
                         (const float*)a_log_.view.data, state, tail_off, xbc, dta, ctx.max_q_len);
        Tensor read = ws.get("mix_read", T, inner_, DType::F32);
        ops::ssm_scan(l, seqs, m, xbc, dta, (const float*)d_.view.data, state, read);
        Tensor normed = ws.get("ssm_normed", T, inner_, ctx.compute_dtype);
        ops::gated_group_norm(l, read, z, &gain_.view, eps_, parts_, normed);
        out_.run(ctx, nullptr, &normed, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    ops::SsmShape shape() const { return ops::SsmShape{H_, G_, N_, P_, taps_}; }
    int64_t width_;
    float eps_;
    int H_, G_, N_, P_, taps_, parts_;
    int64_t inner_, channels_;
    Linear wide_, dt_, out_;
    DeviceWeight conv_, conv_bias_, dt_bias_, a_log_, d_, gain_;
};

template <typename T>
PartFactory simple() {
    PartFactory f;
    f.make = [](const PartSpec& s) { return std::unique_ptr<Part>(new T(s)); };
    return f;
}

}  // namespace

void register_stream_parts() {
    register_part("embedding", "bigram_embedding", simple<BigramEmbedding>());
    register_part("wrap", "hyper_gated_conv", simple<HyperGatedConv>());
    register_part("mixer", "biased_attention", simple<BiasedAttention>());
    register_part("mixer", "state_space", simple<StateSpace>());
    PartFactory wrapped;
    wrapped.make_block = [](BlockParts p) { return std::unique_ptr<Block>(new WrappedSublayers(std::move(p))); };
    register_part("block", "wrapped_sublayers", std::move(wrapped));
}

}  // namespace sandy
