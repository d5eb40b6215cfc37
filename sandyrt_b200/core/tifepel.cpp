// Tifepel: a decoder that keeps its residual stream in several copies, mixes attention layers with state-space layers,
// and routes every token through a few small experts.
//
// config.json (all sizes and every constant that differs between models come from it):
//   architecture  "Tifepel"
//   vocab, width, max_positions, streams
//   embedding.bigram {buckets, mul_prev, mul_cur}   the table row (token_before * mul_prev + token * mul_cur) mod buckets is
//                                                   added to a token's embedding; a request's first token reads row `buckets`
//   norm.eps, canon.taps                            the short convolution on every sublayer's input
//   layers[i]     {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, bias_max, q_temp: {coef, every}}, mlp}
//                 (the bias table 'rel' has as many rows as the weight file gives it; an optional 'bias_rows' states
//                 the number, which the random-weights mode needs)
//                 {type: "mamba2",    mixer: {heads, groups, state, vdim, conv, norm_groups}, mlp}
//     mlp  {kind: "moe", expert: {ff}, router: {experts, identity, top}, shared: {ff} | null} | null
//   loop          {start, stop, times} | absent: layers start .. stop-1 run `times` times on the same tensors, every pass
//                 with cache entries and states of its own; nothing else happens between passes
//
// The embedding is E[token] + bigram row + a learned position vector; every copy of the stream starts as that.  A
// sublayer q of a layer reads u = sum_s in_q[s] X_s through a LayerNorm without offset, passes h + conv(h) to the mixer
// or feed-forward, and its result y joins every copy: X_t <- sum_s mix_q[s, t] X_s + out_q[t] y sigmoid(W_q h + b_q).
// The output is the LayerNorm of the copies' sum and an untied head.
// Tensors: embed, bigram, pos, final.norm, head, and per layer l<i>.norm<q>, l<i>.hc<q>.{in, out, mix}, l<i>.canon<q>,
// l<i>.rg<q> and l<i>.rg<q>.b (q = 1 the mixer, 2 the feed-forward), l<i>.mix.{q, k, v, o, rel} or
// l<i>.mix.{in, conv, conv.b, dt_bias, A_log, D, norm, o}, l<i>.mlp.{router, correction, e<k>.{gate, up, down},
// shared.{gate, up, down}}; linear weights [out, in].
//
// What the design fixes and no file changes: the scores of the router are a softmax over all its outputs, the chosen
// experts' weights are those scores themselves, the experts are silu-gated, identity experts come last, the bias table
// of an attention layer has its first half for single distances and its second half for logarithmic buckets.
//
// The typed configuration below checks the file; `describe` turns it into parts of parts_streams.cpp, parts_latent.cpp
// and parts.cpp.  Nothing else in the engine knows this architecture.
#include <cmath>

#include "config.h"
#include "errors.h"

namespace sandy {

namespace {

[[noreturn]] void bad(const std::string& where, const std::string& what) { throw ConfigError("config.json: " + where + ": " + what); }

const Json& need(const Json& o, const std::string& where, const std::string& key) {
    const Json* v = o.is_object() ? o.find(key) : nullptr;
    if (!v || v->is_null()) bad(where, "required key '" + key + "' is missing");
    return *v;
}
int64_t need_int(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_int()) bad(where, "'" + key + "' must be int, got " + v.dump());
    return v.as_int();
}
double need_num(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_number()) bad(where, "'" + key + "' must be a number, got " + v.dump());
    return v.as_double();
}
const Json& need_obj(const Json& o, const std::string& where, const std::string& key) {
    const Json& v = need(o, where, key);
    if (!v.is_object()) bad(where, "'" + key + "' must be an object, got " + v.dump());
    return v;
}
const Json* maybe_obj(const Json& o, const std::string& where, const std::string& key) {
    const Json* v = o.find(key);
    if (!v || v->is_null()) return nullptr;
    if (!v->is_object()) bad(where, "'" + key + "' must be an object or null, got " + v->dump());
    return v;
}
void positive(int64_t v, const std::string& where, const std::string& key) {
    if (v <= 0) bad(where, "'" + key + "' must be > 0, got " + std::to_string(v));
}

}  // namespace

TifepelConfig TifepelConfig::from_json(const Json& raw) {
    if (!raw.is_object()) throw ConfigError("config.json: top level must be a JSON object");
    TifepelConfig c;
    c.vocab = need_int(raw, "top level", "vocab");
    c.width = need_int(raw, "top level", "width");
    c.max_positions = need_int(raw, "top level", "max_positions");
    c.streams = need_int(raw, "top level", "streams");
    c.norm_eps = need_num(need_obj(raw, "top level", "norm"), "norm", "eps");
    c.canon_taps = need_int(need_obj(raw, "top level", "canon"), "canon", "taps");
    const Json& bigram = need_obj(need_obj(raw, "top level", "embedding"), "embedding", "bigram");
    c.bigram_buckets = need_int(bigram, "embedding.bigram", "buckets");
    c.bigram_mul_prev = need_int(bigram, "embedding.bigram", "mul_prev");
    c.bigram_mul_cur = need_int(bigram, "embedding.bigram", "mul_cur");
    const Json& layers = need(raw, "top level", "layers");
    if (!layers.is_array() || layers.size() == 0) bad("layers", "must be a non-empty list");
    int i = 0;
    for (const Json& lj : layers.items()) {
        const std::string at = "layers[" + std::to_string(i++) + "]";
        if (!lj.is_object()) bad(at, "must be an object");
        Layer l;
        const Json& type = need(lj, at, "type");
        if (!type.is_string()) bad(at, "'type' must be a string");
        l.type = type.as_string();
        const Json& m = need_obj(lj, at, "mixer");
        const std::string ma = at + ".mixer";
        if (l.type == "attention") {
            l.heads = need_int(m, ma, "heads");
            l.kv_heads = need_int(m, ma, "kv_heads");
            l.dim = need_int(m, ma, "dim");
            l.vdim = need_int(m, ma, "vdim");
            l.scale = need_num(m, ma, "scale");
            l.bias_max = need_int(m, ma, "bias_max");
            if (const Json* rows = m.find("bias_rows"))
                if (!rows->is_null()) l.bias_rows = need_int(m, ma, "bias_rows");
            const Json& qt = need_obj(m, ma, "q_temp");
            l.q_temp_coef = need_num(qt, ma + ".q_temp", "coef");
            l.q_temp_every = need_int(qt, ma + ".q_temp", "every");
        } else if (l.type == "mamba2") {
            l.heads = need_int(m, ma, "heads");
            l.groups = need_int(m, ma, "groups");
            l.state = need_int(m, ma, "state");
            l.vdim = need_int(m, ma, "vdim");
            l.conv = need_int(m, ma, "conv");
            l.norm_groups = need_int(m, ma, "norm_groups");
        } else {
            bad(at, "unknown layer type '" + l.type + "'; one of ['attention', 'mamba2']");
        }
        if (const Json* mlp = maybe_obj(lj, at, "mlp")) {
            const std::string fa = at + ".mlp";
            const Json& kind = need(*mlp, fa, "kind");
            if (!kind.is_string() || kind.as_string() != "moe") bad(fa, "'kind' must be 'moe', got " + kind.dump());
            l.mlp = "moe";
            l.ff = need_int(need_obj(*mlp, fa, "expert"), fa + ".expert", "ff");
            const Json& router = need_obj(*mlp, fa, "router");
            l.experts = need_int(router, fa + ".router", "experts");
            l.identity = need_int(router, fa + ".router", "identity");
            l.top = need_int(router, fa + ".router", "top");
            if (const Json* shared = maybe_obj(*mlp, fa, "shared")) l.shared_ff = need_int(*shared, fa + ".shared", "ff");
        }
        c.layers.push_back(l);
    }
    if (const Json* loop = maybe_obj(raw, "top level", "loop")) {
        c.has_loop = true;
        c.loop_start = need_int(*loop, "loop", "start");
        c.loop_stop = need_int(*loop, "loop", "stop");
        c.loop_times = need_int(*loop, "loop", "times");
    }
    return c;
}

Json TifepelConfig::to_json() const {
    Json j = Json::object();
    j["architecture"] = kArchitecture;
    Json canon = Json::object();
    canon["taps"] = (long long)canon_taps;
    j["canon"] = canon;
    Json emb = Json::object(), bigram = Json::object();
    bigram["buckets"] = (long long)bigram_buckets;
    bigram["mul_cur"] = (long long)bigram_mul_cur;
    bigram["mul_prev"] = (long long)bigram_mul_prev;
    emb["bigram"] = bigram;
    j["embedding"] = emb;
    Json ls = Json::array();
    for (const Layer& l : layers) {
        Json lj = Json::object(), m = Json::object();
        if (l.type == "attention") {
            Json qt = Json::object();
            qt["coef"] = l.q_temp_coef;
            qt["every"] = (long long)l.q_temp_every;
            m["bias_max"] = (long long)l.bias_max;
            if (l.bias_rows > 0) m["bias_rows"] = (long long)l.bias_rows;
            m["dim"] = (long long)l.dim;
            m["heads"] = (long long)l.heads;
            m["kv_heads"] = (long long)l.kv_heads;
            m["q_temp"] = qt;
            m["scale"] = l.scale;
            m["vdim"] = (long long)l.vdim;
        } else {
            m["conv"] = (long long)l.conv;
            m["groups"] = (long long)l.groups;
            m["heads"] = (long long)l.heads;
            m["norm_groups"] = (long long)l.norm_groups;
            m["state"] = (long long)l.state;
            m["vdim"] = (long long)l.vdim;
        }
        lj["mixer"] = m;
        if (l.mlp == "moe") {
            Json mlp = Json::object(), expert = Json::object(), router = Json::object();
            expert["ff"] = (long long)l.ff;
            router["experts"] = (long long)l.experts;
            router["identity"] = (long long)l.identity;
            router["top"] = (long long)l.top;
            mlp["expert"] = expert;
            mlp["kind"] = "moe";
            mlp["router"] = router;
            if (l.shared_ff > 0) {
                Json shared = Json::object();
                shared["ff"] = (long long)l.shared_ff;
                mlp["shared"] = shared;
            } else {
                mlp["shared"] = Json();
            }
            lj["mlp"] = mlp;
        } else {
            lj["mlp"] = Json();
        }
        lj["type"] = l.type;
        ls.push(lj);
    }
    j["layers"] = ls;
    if (has_loop) {
        Json loop = Json::object();
        loop["start"] = (long long)loop_start;
        loop["stop"] = (long long)loop_stop;
        loop["times"] = (long long)loop_times;
        j["loop"] = loop;
    }
    j["max_positions"] = (long long)max_positions;
    Json norm = Json::object();
    norm["eps"] = norm_eps;
    j["norm"] = norm;
    j["streams"] = (long long)streams;
    j["vocab"] = (long long)vocab;
    j["width"] = (long long)width;
    return j;
}

void TifepelConfig::validate() const {
    positive(vocab, "top level", "vocab");
    positive(width, "top level", "width");
    positive(max_positions, "top level", "max_positions");
    if (streams < 1 || streams > 8) bad("top level", "'streams' must be 1 .. 8, got " + std::to_string(streams));
    if (!(norm_eps > 0.0)) bad("norm", "'eps' must be > 0");
    if (canon_taps < 1 || canon_taps > 8) bad("canon", "'taps' must be 1 .. 8, got " + std::to_string(canon_taps));
    positive(bigram_buckets, "embedding.bigram", "buckets");
    if (bigram_mul_prev < 0 || bigram_mul_cur < 0 || bigram_mul_prev > 0x7fffffff || bigram_mul_cur > 0x7fffffff || bigram_buckets > 0x7fffffff)
        bad("embedding.bigram", "'mul_prev' and 'mul_cur' must be 0 .. 2^31 - 1 and 'buckets' below 2^31");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer& l = layers[i];
        const std::string at = "layers[" + std::to_string(i) + "]";
        positive(l.heads, at + ".mixer", "heads");
        positive(l.vdim, at + ".mixer", "vdim");
        if (l.type == "attention") {
            positive(l.kv_heads, at + ".mixer", "kv_heads");
            positive(l.dim, at + ".mixer", "dim");
            if (l.heads % l.kv_heads) bad(at, std::to_string(l.heads) + " heads do not divide into " + std::to_string(l.kv_heads) + " kv_heads");
            if (std::max(l.dim, l.vdim) > 640) bad(at + ".mixer", "head sizes are at most 640 (the attention kernels' widest head)");
            positive(l.q_temp_every, at + ".mixer.q_temp", "every");
            if (!std::isfinite(l.q_temp_coef) || !std::isfinite(l.scale)) bad(at + ".mixer", "'scale' and 'q_temp.coef' must be finite numbers");
            if (l.bias_max < 2 || l.bias_max > (1 << 24)) bad(at + ".mixer", "'bias_max' must be 2 .. 2^24");
            if (l.bias_rows < 0 || l.bias_rows == 1 || (l.bias_rows > 0 && l.bias_max <= l.bias_rows / 2))
                bad(at + ".mixer", "'bias_rows', where given, must be at least 2 with 'bias_max' beyond half of it");
        } else {
            positive(l.groups, at + ".mixer", "groups");
            if (l.heads % l.groups) bad(at, std::to_string(l.heads) + " heads do not divide into " + std::to_string(l.groups) + " groups");
            if (l.state < 1 || l.state > 256) bad(at + ".mixer", "'state' must be 1 .. 256");
            if (l.conv < 1 || l.conv > 8) bad(at + ".mixer", "'conv' must be 1 .. 8");
            if (l.norm_groups < 1 || (l.heads * l.vdim) % l.norm_groups) bad(at + ".mixer", "'norm_groups' must divide heads * vdim");
        }
        if (l.mlp == "moe") {
            positive(l.ff, at + ".mlp.expert", "ff");
            positive(l.experts, at + ".mlp.router", "experts");
            if (l.identity < 0) bad(at + ".mlp.router", "'identity' must be >= 0");
            if (l.experts + l.identity > 2048) bad(at + ".mlp.router", "'experts' + 'identity' is at most 2048");
            if (l.top < 1 || l.top > l.experts + l.identity) bad(at + ".mlp.router", "'top' must be 1 .. experts + identity");
            if (l.shared_ff < 0) bad(at + ".mlp.shared", "'ff' must be > 0");
        }
    }
    if (has_loop) {
        if (loop_start < 0 || loop_stop <= loop_start || loop_stop > (int64_t)layers.size())
            bad("loop", "needs 0 <= start < stop <= " + std::to_string(layers.size()));
        if (loop_times < 1) bad("loop", "'times' must be >= 1");
    }
}

// The description: which parts every layer is made of, the run order (a looped span appears once per pass, each pass
// with cache entries of its own), and the tensor names.  The embedding's state has the cache entry after the layers'.
ModelSpec describe_tifepel(const TifepelConfig& cfg) {
    ModelSpec s;
    s.architecture = cfg.architecture();
    s.width = cfg.width;
    s.vocab_size = cfg.vocab;
    s.max_positions = cfg.max_positions;
    s.streams = (int)cfg.streams;
    auto wrap = [&](const std::string& p, int q) {
        const std::string n = std::to_string(q);
        PartSpec w;
        w.kind = "hyper_gated_conv";
        w.params["width"] = (long long)cfg.width;
        w.params["streams"] = (long long)cfg.streams;
        w.params["eps"] = cfg.norm_eps;
        w.params["taps"] = (long long)cfg.canon_taps;
        w.tensors = {{"norm", p + "norm" + n}, {"in", p + "hc" + n + ".in"}, {"out", p + "hc" + n + ".out"}, {"mix", p + "hc" + n + ".mix"},
                     {"conv", p + "canon" + n}, {"gate", p + "rg" + n}, {"gate_bias", p + "rg" + n + ".b"}};
        return w;
    };
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        const TifepelConfig::Layer& c = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        const std::string x = p + "mix.";
        LayerSpec l;
        l.block = "wrapped_sublayers";
        PartSpec& m = l.mixer;
        m.params["width"] = (long long)cfg.width;
        m.params["eps"] = cfg.norm_eps;
        m.params["n_heads"] = (long long)c.heads;
        m.params["v_dim"] = (long long)c.vdim;
        if (c.type == "attention") {
            m.kind = "biased_attention";
            m.params["n_kv_heads"] = (long long)c.kv_heads;
            m.params["qk_dim"] = (long long)c.dim;
            m.params["scale"] = c.scale;
            m.params["qk_unit_norm"] = true;
            m.params["q_pos_coef"] = c.q_temp_coef;
            m.params["q_pos_every"] = (long long)c.q_temp_every;
            m.params["distance_bias"] = true;
            m.params["bias_rows"] = (long long)c.bias_rows;
            m.params["bias_max"] = (long long)c.bias_max;
            m.tensors = {{"q", x + "q"}, {"k", x + "k"}, {"v", x + "v"}, {"o", x + "o"}, {"rel", x + "rel"}};
        } else {
            m.kind = "state_space";
            m.params["n_groups"] = (long long)c.groups;
            m.params["state"] = (long long)c.state;
            m.params["conv_taps"] = (long long)c.conv;
            m.params["norm_groups"] = (long long)c.norm_groups;
            m.tensors = {{"in", x + "in"}, {"conv", x + "conv"}, {"conv_bias", x + "conv.b"}, {"dt_bias", x + "dt_bias"},
                         {"a_log", x + "A_log"}, {"d", x + "D"}, {"norm", x + "norm"}, {"o", x + "o"}};
        }
        l.wraps["mixer"] = wrap(p, 1);
        PartSpec& f = l.feed_forward;
        if (c.mlp == "moe") {
            f.kind = "routed_experts";
            f.params["width"] = (long long)cfg.width;
            f.params["inner"] = (long long)c.ff;
            f.params["n_experts"] = (long long)c.experts;
            f.params["n_identity"] = (long long)c.identity;
            f.params["top"] = (long long)c.top;
            f.params["activation"] = "silu_glu";
            f.params["scoring"] = "softmax_all";
            f.params["correction"] = true;
            f.params["shared_inner"] = (long long)c.shared_ff;
            f.tensors = {{"router", p + "mlp.router"}, {"correction", p + "mlp.correction"}};
            for (int64_t e = 0; e < c.experts; e++) {
                const std::string ex = p + "mlp.e" + std::to_string(e) + ".";
                f.tensors["gate." + std::to_string(e)] = ex + "gate";
                f.tensors["up." + std::to_string(e)] = ex + "up";
                f.tensors["down." + std::to_string(e)] = ex + "down";
            }
            if (c.shared_ff > 0) {
                f.tensors["shared.gate"] = p + "mlp.shared.gate";
                f.tensors["shared.up"] = p + "mlp.shared.up";
                f.tensors["shared.down"] = p + "mlp.shared.down";
            }
            l.wraps["feed_forward"] = wrap(p, 2);
        } else {
            f.kind = "none";
            // what surrounds a feed-forward that is not there, if the file has it
            s.ignored_tensors.push_back("^l" + std::to_string(i) + R"(\.(norm2|canon2|rg2|rg2\.b|hc2\.(in|out|mix))$)");
        }
        s.layers.push_back(std::move(l));
    }
    const int n = (int)cfg.layers.size();
    int cache = 0;
    auto call = [&](int layer) {
        LayerCall c;
        c.layer = layer;
        c.cache = cache++;
        s.schedule.push_back(c);
    };
    if (cfg.has_loop) {
        for (int i = 0; i < (int)cfg.loop_start; i++) call(i);
        for (int64_t pass = 0; pass < cfg.loop_times; pass++)
            for (int i = (int)cfg.loop_start; i < (int)cfg.loop_stop; i++) call(i);
        for (int i = (int)cfg.loop_stop; i < n; i++) call(i);
    } else {
        for (int i = 0; i < n; i++) call(i);
    }
    s.embedding_cache = cache;
    s.embedding.kind = "bigram_embedding";
    s.embedding.params["vocab_size"] = (long long)cfg.vocab;
    s.embedding.params["width"] = (long long)cfg.width;
    s.embedding.params["buckets"] = (long long)cfg.bigram_buckets;
    s.embedding.params["mul_prev"] = (long long)cfg.bigram_mul_prev;
    s.embedding.params["mul_cur"] = (long long)cfg.bigram_mul_cur;
    s.embedding.tensors = {{"weight", "embed"}, {"bigram", "bigram"}};
    s.position.kind = "learned_absolute";
    s.position.params["width"] = (long long)cfg.width;
    s.position.params["max_positions"] = (long long)cfg.max_positions;
    s.position.tensors = {{"weight", "pos"}};
    s.final_norm.kind = "layernorm";
    s.final_norm.params["width"] = (long long)cfg.width;
    s.final_norm.params["eps"] = cfg.norm_eps;
    s.final_norm.params["bias"] = false;
    s.final_norm.tensors = {{"weight", "final.norm"}};
    s.head.kind = "output_head";
    s.head.params["vocab_size"] = (long long)cfg.vocab;
    s.head.params["width"] = (long long)cfg.width;
    s.head.params["tied"] = false;
    s.head.tensors = {{"weight", "head"}};
    return s;
}

}  // namespace sandy
