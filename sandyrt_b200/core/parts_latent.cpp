// Part kinds for decoders whose attention runs over a low-rank latent of keys and values, and whose two sublayers
// read one normed input.
//
//   mixer         "latent_attention"      keys and values of all heads are linear in one short normed vector per token
//                                         (plus, optionally, one rotated key part shared by the heads); only that is
//                                         cached, and the attention runs in the latent's own space
//   feed_forward  "routed_experts"        each token goes through `top` of `n_experts` small feed-forwards, weighted by
//                                         the softmax over the chosen router logits
//   norm          "channel_scale"         follows a sublayer: x += gain * y, one learned factor per channel
//   block         "parallel_branches"     h = norm(x);  x += s1 * mixer(h) + s2 * ff(h)
//
// Every size and constant is a parameter of the part.  Norms, positions and angles, scores and softmax, router logits
// and expert weights, and the sum into the stream are 32-bit in both compute types.
#include <cmath>

#include "part_helpers.h"
#include "parts.h"

namespace sandy {
namespace {
using namespace part_helpers;

// ---- attention over a latent --------------------------------------------------------------------------------------
// Parameters: width, eps, n_heads H, qk_dim d (a head's unrotated query/key size), rot_dim r (its rotated size, 0 for
// none), v_dim e, kv_rank c, q_rank (0: queries straight from the input), scale, rot_dims (how many of the r entries
// turn; neighbours 2i, 2i+1 are a pair), rot_base, sink (a learned logit per head that joins the softmax's denominator).
// Tensors: "dkv" [c + r, width], "dkv_norm" [c], "uk" [H d, c], "uv" [H e, c], "o" [width, H e]; "q" [H (d + r), width]
// or, with a query latent, "dq" [q_rank, width], "dq_norm" [q_rank], "uq" [H d, q_rank]; "sink" [H].
//
// Per token: [latent | k_rot] = W_dkv h, the latent RMS-normed; k_h = U_k,h latent, v_h = U_v,h latent; q_h = [plain |
// rotated]; score = (q_plain . k_h + q_rot . k_rot) * scale; causal softmax; out = W_o [heads' weighted sums of v_h].
// Since k_h and v_h are linear in the latent, U_k,h^T is applied to the query and U_v,h to the weighted sum of latents
// instead: the cache holds one row [latent | k_rot] per token, key and value at once (a one-plane page, one "head"
// that all query heads share), and the attention kernels of every other model serve it with heads of that width.
class LatentAttention : public Mixer {
public:
    explicit LatentAttention(const PartSpec& s)
        : Mixer(s), width_(s.get_int("width")), eps_((float)s.get_double("eps")), H_((int)s.get_int("n_heads")),
          d_((int)s.get_int("qk_dim")), r_((int)s.get_int("rot_dim", 0)), e_((int)s.get_int("v_dim")), c_((int)s.get_int("kv_rank")),
          q_rank_((int)s.get_int("q_rank", 0)), scale_((float)s.get_double("scale")), rot_dims_((int)s.get_int("rot_dims", 0)),
          has_sink_(s.get_bool("sink", false)), pad_((int)round_up(c_ + r_, 16)),
          down_(width_, q_rank_ + c_ + r_, false, "out_in", "down"),
          q_(q_rank_ ? q_rank_ : width_, (int64_t)H_ * (d_ + r_), false, "out_in", "q"),
          out_((int64_t)H_ * e_, width_, false, "out_in", "out") {
        if (H_ <= 0 || d_ <= 0 || e_ <= 0 || c_ <= 0 || r_ < 0 || q_rank_ < 0) throw ConfigError("latent_attention: sizes must be positive");
        if (pad_ > ops::kMaxHeadDim)
            throw ConfigError("latent_attention: kv_rank + rot_dim is at most " + std::to_string(ops::kMaxHeadDim) + ", got " + std::to_string(c_ + r_));
        if (rot_dims_ < 0 || rot_dims_ > r_ || rot_dims_ % 2) throw ConfigError("latent_attention: rot_dims must be even and at most rot_dim");
        if (q_rank_ && r_) throw ConfigError("latent_attention: a query latent and a rotated part together are not supported");
        const std::string pairs = s.get_string("rot_pairs", "neighbours");
        if (pairs != "neighbours") throw ConfigError("latent_attention: rot_pairs must be 'neighbours', got '" + pairs + "'");
        if (rot_dims_) freq_host_ = rotary_frequencies(rot_dims_, s.get_double("rot_base"), nullptr);
    }
    TensorRequests requests() const override {
        TensorRequests t;
        t["dkv"] = want({(int64_t)c_ + r_, width_});
        t["dkv_norm"] = want({(int64_t)c_}, "gamma");
        t["uk"] = want({(int64_t)H_ * d_, (int64_t)c_});
        t["uv"] = want({(int64_t)H_ * e_, (int64_t)c_});
        t["o"] = want({width_, (int64_t)H_ * e_});
        if (q_rank_) {
            t["dq"] = want({(int64_t)q_rank_, width_});
            t["dq_norm"] = want({(int64_t)q_rank_}, "gamma");
            t["uq"] = want({(int64_t)H_ * d_, (int64_t)q_rank_});
        } else {
            t["q"] = want({(int64_t)H_ * (d_ + r_), width_});
        }
        if (has_sink_) t["sink"] = want({(int64_t)H_}, "bias");
        return t;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["down.weight"] = q_rank_ ? stack_rows({&t.at("dq"), &t.at("dkv")}, width_) : t.at("dkv");
        m["q.weight"] = q_rank_ ? t.at("uq") : t.at("q");
        m["out.weight"] = t.at("o");
        down_.bind(m, dtype);
        q_.bind(m, dtype);
        out_.bind(m, dtype);
        // U_k per head, turned: row h * c + i, column j holds uk[h * d + j, i]
        const std::vector<float> uk = to_f32(t.at("uk"));
        auto turned = alloc_f32((size_t)H_ * c_ * d_);
        for (int h = 0; h < H_; h++)
            for (int j = 0; j < d_; j++)
                for (int i = 0; i < c_; i++)
                    turned.get()[((size_t)h * c_ + i) * d_ + j] = uk[((size_t)h * d_ + j) * c_ + i];
        uk_t_ = to_device(host_f32(turned, {(int64_t)H_ * c_, (int64_t)d_}), dtype);
        uv_ = to_device(t.at("uv"), dtype);
        kv_gain_ = to_device(t.at("dkv_norm"), DType::F32);
        if (q_rank_) q_gain_ = to_device(t.at("dq_norm"), DType::F32);
        if (has_sink_) sink_ = to_device(t.at("sink"), DType::F32);
        if (rot_dims_) freq_ = floats_to_device(freq_host_);
    }
    size_t weight_bytes() const override {
        return down_.weight_bytes() + q_.weight_bytes() + out_.weight_bytes() + uk_t_.bytes() + uv_.bytes();
    }
    CacheSpec cache_spec() const override { return CacheSpec::paged_one_plane(1, pad_, 0); }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x, const LayerCall& call) override {
        const int64_t T = h.rows();
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        const DType dt = ctx.compute_dtype;
        // the down-projections, written in 32-bit: their norms read them
        Tensor down = ws.get("latent_down", T, q_rank_ + c_ + r_, DType::F32);
        down_.run(ctx, &h, nullptr, down, ops::Act::None, nullptr);
        Tensor q = ws.get("latent_q", T, (int64_t)H_ * (d_ + r_), dt);
        if (!q_rank_) q_.run(ctx, &h, nullptr, q, ops::Act::None, nullptr);

        const KVView cache = ctx.caches->kv(call.cache);
        const int* table = ctx.block_tables.at((size_t)cache.group);
        Tensor q_abs = ws.get("latent_q_absorbed", T, (int64_t)H_ * pad_, dt);
        Tensor q_latent;
        if (q_rank_) q_latent = ws.get("latent_q_latent", T, q_rank_, dt);
        ops::LatentPrepare p;
        p.q_rank = q_rank_; p.kv_rank = c_; p.rot_dim = r_;
        p.q_gain = q_rank_ ? (const float*)q_gain_.view.data : nullptr;
        p.kv_gain = (const float*)kv_gain_.view.data;
        p.eps = eps_;
        p.freq = rot_dims_ ? (const float*)freq_.view.data : nullptr;
        p.rot_dims = rot_dims_;
        p.n_heads = H_; p.qk_dim = d_;
        p.write_cache = call.write_cache;
        ops::latent_prepare(l, p, down, r_ ? &q : nullptr, cache, table, ctx.max_blocks, ctx.token_seq, ctx.positions,
                            q_rank_ ? &q_latent : nullptr, q_abs);
        if (q_rank_) q_.run(ctx, nullptr, &q_latent, q, ops::Act::None, nullptr);
        // queries into the latent's space: U_k,h^T q_h
        ops::head_product(l, q, d_ + r_, uk_t_.view, H_, q_abs, pad_);
        Tensor o_latent = ws.get("latent_attn_out", T, (int64_t)H_ * pad_, dt);
        ops::AttentionExtras extras;
        extras.sink = has_sink_ ? (const float*)sink_.view.data : nullptr;
        ops::attention(l, ctx.attention_step(cache.group), q_abs, cache, o_latent, H_, scale_, 0, ws, &extras);
        // and back: U_v,h on each head's weighted sum of latents
        Tensor heads = ws.get("latent_heads", T, (int64_t)H_ * e_, dt);
        ops::head_product(l, o_latent, pad_, uv_.view, H_, heads, e_);
        out_.run(ctx, nullptr, &heads, x, ops::Act::None, ctx.overwrite ? nullptr : &x);
    }
private:
    int64_t width_;
    float eps_;
    int H_, d_, r_, e_, c_, q_rank_;
    float scale_;
    int rot_dims_;
    bool has_sink_;
    int pad_;
    Linear down_, q_, out_;
    std::vector<float> freq_host_;
    DeviceWeight uk_t_, uv_, kv_gain_, q_gain_, sink_, freq_;
};

// ---- a routed mixture of experts ------------------------------------------------------------------------------------
// Parameters: width, inner (an expert's), n_experts, top,
//   activation   "relu_squared": an expert is down(relu(up h)^2);
//                "clamped_glu":  g = min(gate h, limit), u = clamp(up h, -limit, limit), down(g sigmoid(glu_alpha g) (u + 1))
//                (parameters limit, glu_alpha)
//                "silu_glu":     down(silu(gate h) (up h))
//   n_identity   that many further router outputs, behind the experts with matrices, are experts that hand their input
//                on: weight * h (gated activations only)
//   shared_inner > 0: one more expert of that inner size ("shared.gate", "shared.up", "shared.down"), which every token
//                passes and which is added unweighted
//   scoring      "softmax_top": the `top` largest router logits (+ router_bias) are chosen, weighted by the softmax over
//                the chosen logits alone (parameter router_bias);
//                "sigmoid": scores s = sigmoid(logit); the choice is by s + correction (parameter correction: whether
//                the tensor exists) among the experts of the keep_groups best of n_groups equal groups of neighbours (a
//                group's score: the sum of its group_rank largest choice scores); the weights are the chosen s over their
//                sum (+ weight_eps), times weight_scale;
//                "softmax_all": scores s = softmax over ALL router outputs; the choice is by s + correction; the weights
//                are the chosen s themselves times weight_scale (over their sum + weight_eps only with renormalize).
// Tensors: "router" [n_experts, width], "router_bias" / "correction" [n_experts], "up.<k>" [inner, width], "gate.<k>"
// likewise (clamped_glu), "down.<k>" [width, inner].
// x (+)= sum over a token's chosen experts of weight * expert_k(h).  Router logits are a product written in 32-bit;
// the routing lives on the device, so a recorded step serves every routing.
class RoutedExperts : public FeedForward {
public:
    explicit RoutedExperts(const PartSpec& s)
        : FeedForward(s), width_(s.get_int("width")), inner_(s.get_int("inner")), E_((int)s.get_int("n_experts")),
          top_((int)s.get_int("top")), identity_((int)s.get_int("n_identity", 0)), shared_inner_(s.get_int("shared_inner", 0)),
          has_bias_(s.get_bool("router_bias", false)), router_(width_, E_ + identity_, false, "out_in", "router"),
          shared_gate_up_(width_, 2 * std::max<int64_t>(shared_inner_, 1), false, "out_in", "shared_gate_up"),
          shared_down_(std::max<int64_t>(shared_inner_, 1), width_, false, "out_in", "shared_down") {
        if (E_ < 1 || identity_ < 0 || E_ + identity_ > 2048 || top_ < 1 || top_ > E_ + identity_)
            throw ConfigError("routed_experts: n_experts + n_identity must be 1 .. 2048 and top 1 .. their sum");
        if (shared_inner_ < 0) throw ConfigError("routed_experts: shared_inner must not be negative");
        const std::string a = s.get_string("activation", "relu_squared");
        if (a == "clamped_glu") {
            glu_ = true;
            limit_ = (float)s.get_double("limit");
            alpha_ = (float)s.get_double("glu_alpha", 1.0);
            if (!(limit_ > 0.0f)) throw ConfigError("routed_experts: limit must be positive");
        } else if (a == "silu_glu") {
            glu_ = true;
            plain_glu_ = true;
        } else if (a != "relu_squared") {
            throw ConfigError("routed_experts: unknown activation '" + a + "'");
        }
        const std::string sc = s.get_string("scoring", "softmax_top");
        if (sc == "sigmoid") {
            scored_ = true;
            has_bias_ = s.get_bool("correction", false);
            rule_.n_groups = (int)s.get_int("n_groups", 1);
            rule_.keep_groups = (int)s.get_int("keep_groups", rule_.n_groups);
            rule_.group_rank = (int)s.get_int("group_rank", 2);
            rule_.weight_scale = (float)s.get_double("weight_scale", 1.0);
            rule_.norm_eps = (float)s.get_double("weight_eps", 0.0);
            if (rule_.n_groups < 1 || E_ % rule_.n_groups || rule_.keep_groups < 1 || rule_.keep_groups > rule_.n_groups ||
                rule_.group_rank < 1 || top_ > E_ / rule_.n_groups * rule_.keep_groups)
                throw ConfigError("routed_experts: n_groups must divide n_experts, 1 <= keep_groups <= n_groups, and the kept groups must hold top experts");
        } else if (sc == "softmax_all") {
            softmax_all_ = true;
            has_bias_ = s.get_bool("correction", false);
            soft_.weight_scale = (float)s.get_double("weight_scale", 1.0);
            soft_.renormalize = s.get_bool("renormalize", false);
            soft_.norm_eps = (float)s.get_double("weight_eps", 0.0);
        } else if (sc != "softmax_top") {
            throw ConfigError("routed_experts: unknown scoring '" + sc + "'");
        }
        if ((identity_ > 0 || shared_inner_ > 0) && !glu_) throw ConfigError("routed_experts: identity and shared experts go with a gated activation");
    }
    TensorRequests requests() const override {
        TensorRequests t;
        t["router"] = want({(int64_t)(E_ + identity_), width_});
        if (has_bias_) t[scored_ || softmax_all_ ? "correction" : "router_bias"] = want({(int64_t)(E_ + identity_)}, "bias");
        if (shared_inner_) {
            t["shared.gate"] = want({shared_inner_, width_});
            t["shared.up"] = want({shared_inner_, width_});
            t["shared.down"] = want({width_, shared_inner_});
        }
        for (int e = 0; e < E_; e++) {
            t["up." + std::to_string(e)] = want({inner_, width_});
            if (glu_) t["gate." + std::to_string(e)] = want({inner_, width_});
            t["down." + std::to_string(e)] = want({width_, inner_});
        }
        return t;
    }
    void bind(const TensorMap& t, DType dtype) override {
        TensorMap m;
        m["router.weight"] = t.at("router");
        router_.bind(m, dtype);
        if (has_bias_) bias_ = to_device(t.at(scored_ || softmax_all_ ? "correction" : "router_bias"), DType::F32);
        if (shared_inner_) {
            TensorMap sm;
            sm["shared_gate_up.weight"] = stack_rows({&t.at("shared.gate"), &t.at("shared.up")}, width_);
            sm["shared_down.weight"] = t.at("shared.down");
            shared_gate_up_.bind(sm, dtype);
            shared_down_.bind(sm, dtype);
        }
        std::vector<const HostTensor*> ups, downs;
        for (int e = 0; e < E_; e++) {
            if (glu_) ups.push_back(&t.at("gate." + std::to_string(e)));      // an expert's rows: its gate, then its up
            ups.push_back(&t.at("up." + std::to_string(e)));
            downs.push_back(&t.at("down." + std::to_string(e)));
        }
        up_ = to_device(stack_rows(ups, width_), dtype);
        down_ = to_device(stack_rows(downs, inner_), dtype);
    }
    // a decode step reads the router and, per token, `top` experts
    size_t weight_bytes() const override {
        return router_.weight_bytes() + (up_.bytes() + down_.bytes()) / (size_t)E_ * (size_t)std::min(top_, E_) +
               (shared_inner_ ? shared_gate_up_.weight_bytes() + shared_down_.weight_bytes() : 0);
    }
    bool can_overwrite() const override { return true; }
    void forward(StepContext& ctx, NormedInput& h, Tensor& x) override {
        const int64_t T = h.rows(), slots = T * top_;
        Workspace& ws = *ctx.workspace;
        const ops::Launch& l = ctx.launch;
        const int routed = E_ + identity_;
        Tensor logits = ws.get("moe_logits", T, routed, DType::F32);
        router_.run(ctx, &h, nullptr, logits, ops::Act::None, nullptr);
        ops::Routing r;
        r.n_tokens = (int)T; r.n_experts = routed; r.top = top_;
        r.expert_of = (int*)ws.raw("moe_expert_of", (size_t)slots * sizeof(int));
        r.weight_of = (float*)ws.raw("moe_weight_of", (size_t)slots * sizeof(float));
        r.group_start = (int*)ws.raw("moe_group_start", (size_t)(routed + 1) * sizeof(int));
        r.entry_of_slot = (int*)ws.raw("moe_entry_of_slot", (size_t)slots * sizeof(int));
        r.slot_of_entry = (int*)ws.raw("moe_slot_of_entry", (size_t)slots * sizeof(int));
        if (scored_) ops::moe_route_scored(l, logits, has_bias_ ? &bias_.view : nullptr, rule_, r);
        else if (softmax_all_) ops::moe_route_softmax(l, logits, has_bias_ ? &bias_.view : nullptr, soft_, r);
        else ops::moe_route(l, logits, has_bias_ ? &bias_.view : nullptr, r);
        // Experts without matrices come last, so the slots of those with matrices are the first group_start[E_] of the
        // sorted order: the products walk the experts that have matrices and never see the others' slots.
        const ops::Routing all = r;
        r.n_experts = E_;
        Tensor a = ws.get("moe_inner", slots, inner_, ctx.compute_dtype);
        Tensor sorted = ws.get("moe_sorted_rows", slots, width_, ctx.compute_dtype);      // for steps whose products want them
        if (glu_) {
            Tensor gu = ws.get("moe_gate_up", slots, 2 * inner_, ctx.compute_dtype);
            ops::expert_product(l, r, h.tensor(), true, up_.view, ops::ExpertAct::None, gu, &sorted);
            if (plain_glu_) ops::glu(l, gu.col_range(0, inner_), gu.col_range(inner_, 2 * inner_), ops::GluAct::Silu, a);
            else ops::glu_clamped(l, gu.col_range(0, inner_), gu.col_range(inner_, 2 * inner_), limit_, alpha_, a);
        } else {
            ops::expert_product(l, r, h.tensor(), true, up_.view, ops::ExpertAct::ReluSquared, a, &sorted);
        }
        Tensor rows = ws.get("moe_rows", slots, width_, DType::F32);
        ops::expert_product(l, r, a, false, down_.view, ops::ExpertAct::None, rows);
        if (identity_) ops::moe_combine_identity(l, all, E_, h.tensor(), rows, x, !ctx.overwrite);
        else ops::moe_combine(l, r, rows, x, !ctx.overwrite);
        if (shared_inner_) {                        // an expert every token passes, added to the routed ones
            Tensor sgu = ws.get("ff_gate_up", T, 2 * shared_inner_, ctx.compute_dtype);
            shared_gate_up_.run(ctx, &h, nullptr, sgu, ops::Act::None, nullptr);
            Tensor sa = ws.get("ff_inner", T, shared_inner_, ctx.compute_dtype);
            ops::glu(l, sgu.col_range(0, shared_inner_), sgu.col_range(shared_inner_, 2 * shared_inner_), ops::GluAct::Silu, sa);
            shared_down_.run(ctx, nullptr, &sa, x, ops::Act::None, &x);
        }
    }
private:
    int64_t width_, inner_;
    int E_, top_, identity_;
    int64_t shared_inner_;
    bool has_bias_, glu_ = false, plain_glu_ = false, scored_ = false, softmax_all_ = false;
    float limit_ = 0.0f, alpha_ = 1.0f;
    ops::ScoredRoute rule_;
    ops::SoftmaxRoute soft_;
    Linear router_, shared_gate_up_, shared_down_;
    DeviceWeight bias_, up_, down_;
};

// ---- a factor per channel behind a sublayer ---------------------------------------------------------------------------
// Parameters: width.  Tensor: "weight" [width].  x += mult * weight * y, in 32-bit.
class ChannelScale : public Norm {
public:
    explicit ChannelScale(const PartSpec& s) : Norm(s), width_(s.get_int("width")) {}
    TensorRequests requests() const override { return {{"weight", want({width_}, "gamma")}}; }
    void bind(const TensorMap& t, DType) override { gain_ = to_device(t.at("weight"), DType::F32); }
    size_t weight_bytes() const override { return gain_.bytes(); }
    void forward(StepContext&, const Tensor&, Tensor&, const int*, int) override {
        throw ConfigError("norm kind 'channel_scale' only follows a sublayer");
    }
    void forward_add(StepContext& ctx, const Tensor& y, float mult, Tensor& x) override {
        if (mult != 1.0f) throw ConfigError("channel_scale: a multiplier beside the learned factors is not supported");
        ops::scale_add(ctx.launch, y, gain_.view, nullptr, nullptr, x);
    }
    const Tensor* channel_gain() const override { return &gain_.view; }
private:
    int64_t width_;
    DeviceWeight gain_;
};

// ---- block --------------------------------------------------------------------------------------------------------------
// "parallel_branches": one norm, both sublayers read its output, and their results join the stream together:
// h = norm(x); x += s1(mixer(h)) + s2(ff(h)).  Norm names: "input", "mixer_scale", and "feed_forward_scale" where the
// layer has a feed-forward; the two scales are parts that follow a sublayer (forward_add).  Where both hand out a
// factor per channel the branches are added first and join the stream in one pass.
class ParallelBranches : public Block {
public:
    using Block::Block;
    void forward(StepContext& ctx, Tensor& x, const LayerCall& call) override {
        NormedInput h(ctx, *norms_.at("input"), x);
        Tensor y1 = ctx.workspace->get("branch", x.rows, x.cols, DType::F32);
        begin_branch(ctx, y1, mixer_->can_overwrite());
        mixer_->forward(ctx, h, y1, call);
        ctx.overwrite = false;
        Norm& s1 = *norms_.at("mixer_scale");
        if (ff_->empty()) {
            s1.forward_add(ctx, y1, 1.0f, x);
            return;
        }
        Tensor y2 = ctx.workspace->get("branch_2", x.rows, x.cols, DType::F32);
        begin_branch(ctx, y2, ff_->can_overwrite());
        ff_->forward(ctx, h, y2);
        ctx.overwrite = false;
        Norm& s2 = *norms_.at("feed_forward_scale");
        if (s1.channel_gain() && s2.channel_gain()) {
            ops::scale_add(ctx.launch, y1, *s1.channel_gain(), &y2, s2.channel_gain(), x);
        } else {
            s1.forward_add(ctx, y1, 1.0f, x);
            s2.forward_add(ctx, y2, 1.0f, x);
        }
    }
private:
    static void begin_branch(StepContext& ctx, Tensor& y, bool overwrites) {
        ctx.overwrite = overwrites;
        if (!overwrites)
            cuda_check(cudaMemsetAsync(y.data, 0, (size_t)y.numel() * sizeof(float), ctx.launch.stream), "clearing a branch");
    }
};

template <typename T>
PartFactory simple() {
    PartFactory f;
    f.make = [](const PartSpec& s) { return std::unique_ptr<Part>(new T(s)); };
    return f;
}

}  // namespace

void register_latent_parts() {
    register_part("mixer", "latent_attention", simple<LatentAttention>());
    register_part("feed_forward", "routed_experts", simple<RoutedExperts>());
    register_part("norm", "channel_scale", simple<ChannelScale>());
    PartFactory parallel;
    parallel.norm_names = {"input", "mixer_scale"};          // "feed_forward_scale" where the layer has a feed-forward
    parallel.make_block = [](BlockParts p) {
        return std::unique_ptr<Block>(new ParallelBranches(std::move(p.mixer), std::move(p.feed_forward), std::move(p.norms), p.width));
    };
    register_part("block", "parallel_branches", std::move(parallel));
}

}  // namespace sandy
