// Bilurax: a decoder whose attention has no positions in its scores, norms queries, keys and values, caps its scores
// and looks at chunks of positions, behind a token shift; dense or routed feed-forwards; a span of layers that may run
// several times.
//
// config.json (all sizes and every constant that differs between models come from it):
//   architecture  "Bilurax"
//   vocab, width, logit_softcap
//   embedding.scale                       the factor on a token's row of the table (the tied head reads the table itself)
//   norm.eps
//   layers[i]     {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, softcap, mask: {size}}, mlp: {...} | null}
//     mlp {kind: "dense", ff}                                      down(relu(up h)^2)
//         {kind: "moe", expert: {ff, limit},
//          router: {experts, top, scale, groups: {count, keep}}}   `top` of `experts` small gated feed-forwards, chosen by
//                                                                  sigmoid scores plus a correction inside the best groups
//   loop          {start, stop, times} | absent: layers start .. stop-1 run `times` times on the same tensors, every pass
//                 with cache entries and states of its own; before every pass but the first the embedding's output joins
//                 the stream, and before every pass row t of 'loop.step' [times, width] does
//
// A layer is x += mixer(shift(norm1(x))); x += ff(norm2(x)), RMS norms with plain gains.  The output is the final norm,
// the embedding table as the head, and logit_softcap * tanh(logits / logit_softcap).
// Tensors: embed, final.norm, loop.step, and per layer l<i>.norm1, l<i>.norm2, l<i>.shift, l<i>.mix.{q, k, v, o} with
// their biases '.b', l<i>.mix.{q.norm, k.norm, temp}, l<i>.mlp.{up, down | router, correction, e<k>.{gate, up, down}};
// linear weights [out, in].
//
// What the design fixes and no file changes: 1.702 in the experts' gate, 1e-20 in the weights' denominator, a group's
// score being the sum of its TWO largest choice scores.
//
// The typed configuration below checks the file; `describe` turns it into parts of parts_capped.cpp, parts_latent.cpp,
// parts_hybrid.cpp and parts.cpp.  Nothing else in the engine knows this architecture.
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

constexpr double kGluAlpha = 1.702;          // the experts' gate is g * sigmoid(1.702 g)
constexpr double kWeightEps = 1e-20;         // joins the sum the chosen scores are divided by
constexpr int kGroupRank = 2;                // a group's score: the sum of its two largest choice scores

}  // namespace

BiluraxConfig BiluraxConfig::from_json(const Json& raw) {
    if (!raw.is_object()) throw ConfigError("config.json: top level must be a JSON object");
    BiluraxConfig c;
    c.vocab = need_int(raw, "top level", "vocab");
    c.width = need_int(raw, "top level", "width");
    c.norm_eps = need_num(need_obj(raw, "top level", "norm"), "norm", "eps");
    c.logit_softcap = need_num(raw, "top level", "logit_softcap");
    c.embedding_scale = need_num(need_obj(raw, "top level", "embedding"), "embedding", "scale");
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
        if (l.type != "attention") bad(at, "unknown layer type '" + l.type + "'; one of ['attention']");
        const Json& m = need_obj(lj, at, "mixer");
        const std::string ma = at + ".mixer";
        l.heads = need_int(m, ma, "heads");
        l.kv_heads = need_int(m, ma, "kv_heads");
        l.dim = need_int(m, ma, "dim");
        l.vdim = need_int(m, ma, "vdim");
        l.scale = need_num(m, ma, "scale");
        l.softcap = need_num(m, ma, "softcap");
        l.chunk = need_int(need_obj(m, ma, "mask"), ma + ".mask", "size");
        if (const Json* mlp = maybe_obj(lj, at, "mlp")) {
            const std::string fa = at + ".mlp";
            const Json& kind = need(*mlp, fa, "kind");
            if (!kind.is_string()) bad(fa, "'kind' must be a string");
            l.mlp = kind.as_string();
            if (l.mlp == "dense") {
                l.ff = need_int(*mlp, fa, "ff");
            } else if (l.mlp == "moe") {
                const Json& expert = need_obj(*mlp, fa, "expert");
                l.ff = need_int(expert, fa + ".expert", "ff");
                l.limit = need_num(expert, fa + ".expert", "limit");
                const Json& router = need_obj(*mlp, fa, "router");
                const std::string ra = fa + ".router";
                l.experts = need_int(router, ra, "experts");
                l.top = need_int(router, ra, "top");
                l.router_scale = need_num(router, ra, "scale");
                const Json& groups = need_obj(router, ra, "groups");
                l.groups = need_int(groups, ra + ".groups", "count");
                l.keep = need_int(groups, ra + ".groups", "keep");
            } else {
                bad(fa, "'kind' must be 'dense' or 'moe', got " + kind.dump());
            }
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

Json BiluraxConfig::to_json() const {
    Json j = Json::object();
    j["architecture"] = kArchitecture;
    Json emb = Json::object();
    emb["scale"] = embedding_scale;
    j["embedding"] = emb;
    Json ls = Json::array();
    for (const Layer& l : layers) {
        Json lj = Json::object(), m = Json::object(), mask = Json::object();
        m["dim"] = (long long)l.dim;
        m["heads"] = (long long)l.heads;
        m["kv_heads"] = (long long)l.kv_heads;
        mask["size"] = (long long)l.chunk;
        m["mask"] = mask;
        m["scale"] = l.scale;
        m["softcap"] = l.softcap;
        m["vdim"] = (long long)l.vdim;
        lj["mixer"] = m;
        if (l.mlp == "dense") {
            Json mlp = Json::object();
            mlp["ff"] = (long long)l.ff;
            mlp["kind"] = "dense";
            lj["mlp"] = mlp;
        } else if (l.mlp == "moe") {
            Json mlp = Json::object(), expert = Json::object(), router = Json::object(), groups = Json::object();
            expert["ff"] = (long long)l.ff;
            expert["limit"] = l.limit;
            groups["count"] = (long long)l.groups;
            groups["keep"] = (long long)l.keep;
            router["experts"] = (long long)l.experts;
            router["groups"] = groups;
            router["scale"] = l.router_scale;
            router["top"] = (long long)l.top;
            mlp["expert"] = expert;
            mlp["kind"] = "moe";
            mlp["router"] = router;
            lj["mlp"] = mlp;
        } else {
            lj["mlp"] = Json();
        }
        lj["type"] = l.type;
        ls.push(lj);
    }
    j["layers"] = ls;
    j["logit_softcap"] = logit_softcap;
    if (has_loop) {
        Json loop = Json::object();
        loop["start"] = (long long)loop_start;
        loop["stop"] = (long long)loop_stop;
        loop["times"] = (long long)loop_times;
        j["loop"] = loop;
    }
    Json norm = Json::object();
    norm["eps"] = norm_eps;
    j["norm"] = norm;
    j["vocab"] = (long long)vocab;
    j["width"] = (long long)width;
    return j;
}

void BiluraxConfig::validate() const {
    positive(vocab, "top level", "vocab");
    positive(width, "top level", "width");
    if (!(norm_eps > 0.0)) bad("norm", "'eps' must be > 0");
    if (!(logit_softcap > 0.0)) bad("top level", "'logit_softcap' must be > 0");
    if (!std::isfinite(embedding_scale)) bad("embedding", "'scale' must be a finite number");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer& l = layers[i];
        const std::string at = "layers[" + std::to_string(i) + "]";
        positive(l.heads, at + ".mixer", "heads");
        positive(l.kv_heads, at + ".mixer", "kv_heads");
        positive(l.dim, at + ".mixer", "dim");
        positive(l.vdim, at + ".mixer", "vdim");
        positive(l.chunk, at + ".mixer.mask", "size");
        if (l.heads % l.kv_heads) bad(at, std::to_string(l.heads) + " heads do not divide into " + std::to_string(l.kv_heads) + " kv_heads");
        if (!(l.softcap > 0.0)) bad(at + ".mixer", "'softcap' must be > 0");
        if (std::max(l.dim, l.vdim) > 640) bad(at + ".mixer", "head sizes are at most 640 (the attention kernels' widest head)");
        if (l.mlp == "dense") positive(l.ff, at + ".mlp", "ff");
        if (l.mlp == "moe") {
            positive(l.ff, at + ".mlp.expert", "ff");
            if (!(l.limit > 0.0)) bad(at + ".mlp.expert", "'limit' must be > 0");
            positive(l.experts, at + ".mlp.router", "experts");
            if (l.experts > 2048) bad(at + ".mlp.router", "'experts' is at most 2048");
            positive(l.groups, at + ".mlp.router.groups", "count");
            if (l.experts % l.groups) bad(at + ".mlp.router.groups", "'count' must divide experts");
            if (l.keep < 1 || l.keep > l.groups) bad(at + ".mlp.router.groups", "'keep' must be 1 .. count");
            if (l.top < 1 || l.top > l.experts / l.groups * l.keep) bad(at + ".mlp.router", "'top' must be 1 .. the experts of the kept groups");
        }
    }
    if (has_loop) {
        if (loop_start < 0 || loop_stop <= loop_start || loop_stop > (int64_t)layers.size())
            bad("loop", "needs 0 <= start < stop <= " + std::to_string(layers.size()));
        if (loop_times < 1) bad("loop", "'times' must be >= 1");
    }
}

// The description: which parts every layer is made of, the run order (a looped span appears once per pass, each pass
// with cache entries of its own and entered through an addition to the stream), and the tensor names.
ModelSpec describe_bilurax(const BiluraxConfig& cfg) {
    ModelSpec s;
    s.architecture = cfg.architecture();
    s.width = cfg.width;
    s.vocab_size = cfg.vocab;
    auto norm = [&](const std::string& name) {
        PartSpec p;
        p.kind = "rmsnorm";
        p.params["width"] = (long long)cfg.width;
        p.params["eps"] = cfg.norm_eps;
        p.tensors = {{"weight", name}};
        return p;
    };
    for (size_t i = 0; i < cfg.layers.size(); i++) {
        const BiluraxConfig::Layer& c = cfg.layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        LayerSpec l;
        l.block = "pre_norm";
        PartSpec& m = l.mixer;
        m.kind = "normed_attention";
        m.params["width"] = (long long)cfg.width;
        m.params["eps"] = cfg.norm_eps;
        m.params["n_heads"] = (long long)c.heads;
        m.params["n_kv_heads"] = (long long)c.kv_heads;
        m.params["qk_dim"] = (long long)c.dim;
        m.params["v_dim"] = (long long)c.vdim;
        m.params["scale"] = c.scale;
        m.params["bias"] = true;
        m.params["qk_norm"] = true;
        m.params["v_norm"] = true;
        m.params["head_temperature"] = true;
        m.params["softcap"] = c.softcap;
        m.params["chunk"] = (long long)c.chunk;
        m.params["token_shift"] = true;
        const std::string x = p + "mix.";
        m.tensors = {{"q", x + "q"}, {"k", x + "k"}, {"v", x + "v"}, {"o", x + "o"}, {"q_bias", x + "q.b"}, {"k_bias", x + "k.b"},
                     {"v_bias", x + "v.b"}, {"o_bias", x + "o.b"}, {"q_norm", x + "q.norm"}, {"k_norm", x + "k.norm"},
                     {"temperature", x + "temp"}, {"shift", p + "shift"}};
        l.norms["mixer"] = norm(p + "norm1");
        PartSpec& f = l.feed_forward;
        if (c.mlp == "dense") {
            f.kind = "dense_mlp";
            f.params["width"] = (long long)cfg.width;
            f.params["inner"] = (long long)c.ff;
            f.params["activation"] = "relu_squared";
            f.params["bias"] = false;
            f.params["weight_layout"] = "out_in";
            f.tensors = {{"up.weight", p + "mlp.up"}, {"down.weight", p + "mlp.down"}};
        } else if (c.mlp == "moe") {
            f.kind = "routed_experts";
            f.params["width"] = (long long)cfg.width;
            f.params["inner"] = (long long)c.ff;
            f.params["n_experts"] = (long long)c.experts;
            f.params["top"] = (long long)c.top;
            f.params["activation"] = "clamped_glu";
            f.params["limit"] = c.limit;
            f.params["glu_alpha"] = kGluAlpha;
            f.params["scoring"] = "sigmoid";
            f.params["correction"] = true;
            f.params["n_groups"] = (long long)c.groups;
            f.params["keep_groups"] = (long long)c.keep;
            f.params["group_rank"] = (long long)kGroupRank;
            f.params["weight_scale"] = c.router_scale;
            f.params["weight_eps"] = kWeightEps;
            f.tensors = {{"router", p + "mlp.router"}, {"correction", p + "mlp.correction"}};
            for (int64_t e = 0; e < c.experts; e++) {
                const std::string ex = p + "mlp.e" + std::to_string(e) + ".";
                f.tensors["gate." + std::to_string(e)] = ex + "gate";
                f.tensors["up." + std::to_string(e)] = ex + "up";
                f.tensors["down." + std::to_string(e)] = ex + "down";
            }
        } else {
            f.kind = "none";
        }
        if (!c.mlp.empty()) l.norms["feed_forward"] = norm(p + "norm2");
        else s.ignored_tensors.push_back("^l" + std::to_string(i) + R"(\.norm2$)");      // a norm with nothing behind it, if the file has one
        s.layers.push_back(std::move(l));
    }
    // run order
    const int n = (int)cfg.layers.size();
    int cache = 0;
    auto call = [&](int layer, int remix) {
        LayerCall c;
        c.layer = layer;
        c.cache = cache++;
        c.remix = remix;
        s.schedule.push_back(c);
    };
    if (cfg.has_loop) {
        for (int64_t pass = 0; pass < cfg.loop_times; pass++) {
            PartSpec in;
            in.kind = "add_row";
            in.params["width"] = (long long)cfg.width;
            in.params["rows"] = (long long)cfg.loop_times;
            in.params["row"] = (long long)pass;
            in.params["add_embedding"] = pass > 0;
            in.tensors = {{"table", "loop.step"}};
            s.remixes.push_back(in);
        }
        for (int i = 0; i < (int)cfg.loop_start; i++) call(i, -1);
        for (int64_t pass = 0; pass < cfg.loop_times; pass++)
            for (int i = (int)cfg.loop_start; i < (int)cfg.loop_stop; i++) call(i, i == (int)cfg.loop_start ? (int)pass : -1);
        for (int i = (int)cfg.loop_stop; i < n; i++) call(i, -1);
    } else {
        for (int i = 0; i < n; i++) call(i, -1);
    }
    s.embedding.kind = "token_embedding";
    s.embedding.params["vocab_size"] = (long long)cfg.vocab;
    s.embedding.params["width"] = (long long)cfg.width;
    s.embedding.params["scale"] = cfg.embedding_scale;
    s.embedding.tensors = {{"weight", "embed"}};
    s.position.kind = "none";
    s.final_norm = norm("final.norm");
    s.head.kind = "output_head";
    s.head.params["vocab_size"] = (long long)cfg.vocab;
    s.head.params["width"] = (long long)cfg.width;
    s.head.params["tied"] = true;
    s.head.params["logit_softcap"] = cfg.logit_softcap;
    return s;
}

}  // namespace sandy
