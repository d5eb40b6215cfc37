// Typed model configuration and the architecture registry.
//
// A configuration is a typed object whose fields are the architecture's own config.json keys.
// Every size and constant the model code uses comes from one of these fields; the model code
// holds no literals of its own.  (The reference keeps every size as a literal in its model
// program, src/models/gpt2_small.sandy.go:7,18,36,52, and picks a model by an if/else chain over
// an `architecture` string, src/server/Model.cpp:100-160; here both are data and an open table.)
#pragma once

#include <functional>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "json.h"
#include "spec.h"

namespace sandy {

// Base of every architecture's typed configuration.
class ModelConfig {
public:
    virtual ~ModelConfig() = default;
    virtual std::string architecture() const = 0;     // the registry key ("GPT2LMHeadModel", ...)
    virtual Json to_json() const = 0;                 // what config.json holds
    virtual void validate() const = 0;                // throws ConfigError
};

// GPT-2's config.json.  Keys and defaults follow the reference's artefact
// experiments/gpt2_small/config.json:1-30 (n_layer :16, n_embd :14, n_head :15, n_positions :17,
// vocab_size :30, layer_norm_epsilon :11, activation_function :2, architectures :3-5, bos/eos
// :7,9).  Keys that file does not carry get the architecture's usual defaults: n_inner (null ->
// 4 * n_embd), scale_attn_weights (true), scale_attn_by_inverse_layer_idx (false),
// tie_word_embeddings (true).
class GPT2Config : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "GPT2LMHeadModel";
    int64_t n_layer = 0, n_embd = 0, n_head = 0, n_positions = 0, vocab_size = 0;
    std::optional<int64_t> n_inner;
    double layer_norm_epsilon = 1e-5;
    std::string activation_function = "gelu_new";
    bool scale_attn_weights = true;
    bool scale_attn_by_inverse_layer_idx = false;
    bool tie_word_embeddings = true;
    std::optional<int64_t> bos_token_id, eos_token_id;

    int64_t head_dim() const { return n_embd / n_head; }
    int64_t inner_dim() const { return n_inner ? *n_inner : 4 * n_embd; }

    static GPT2Config from_json(const Json& raw);     // type checks only; call validate() for the sizes
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
};

// Panupel's config.json (core/panupel.cpp says what the keys mean).  Layers are listed one by one, each with its
// own mixer type and sizes, so the typed form is a list of layer records.
class PanupelConfig : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "Panupel";
    struct Layer {
        std::string type;                                   // "parallel" | "delta"
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0; // delta: the mixer's; parallel: the left mixer's
        int64_t conv = 0;                                   // delta: taps of the short convolutions
        double scale = 1.0;                                 // parallel, left: the factor on q . k
        int64_t rot_dims = 0;                               // parallel, left: 0 = no rotary positions
        double rot_base = 10000.0;
        bool rot_scaling = false;
        double rot_factor = 1.0, rot_low = 1.0, rot_high = 1.0, rot_original = 1.0;
        int64_t right_heads = 0, right_dim = 0, right_vdim = 0;
        double gate_cap = 1.0, left_scale = 1.0, right_scale = 1.0;
        int64_t ff = 0;                                     // 0: the layer has no feed-forward
    };
    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6, residual_mult = 1.0;
    std::vector<Layer> layers;
    bool has_loop = false;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 1;

    static PanupelConfig from_json(const Json& raw);
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
};

// Sovezen's config.json (core/sovezen.cpp says what the keys mean): layers listed one by one, each an attention over
// a latent of keys and values in one of two forms, beside a dense or routed feed-forward, or none.
class SovezenConfig : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "Sovezen";
    struct Layer {
        std::string type;                                   // "latent_attention" | "latent_attention_2"
        int64_t heads = 0, dim = 0, vdim = 0, kv_rank = 0;
        int64_t rot_dim = 0;                                // latent_attention: rotated entries of a head's query and key
        int64_t q_rank = 0;                                 // latent_attention_2: size of the queries' own latent
        double scale = 1.0;
        int64_t rot_dims = 0;                               // how many of the rot_dim entries turn
        double rot_base = 10000.0;
        std::string mlp;                                    // "dense" | "moe" | "" (no feed-forward)
        int64_t ff = 0;                                     // dense: inner size; moe: an expert's inner size
        int64_t experts = 0, top = 0;
        int64_t weights_of = -1;                            // >= 0: the layer whose tensors this one uses
    };
    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6, logit_scale = 1.0;
    std::vector<Layer> layers;

    static SovezenConfig from_json(const Json& raw);
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
    int owner(int layer) const;                             // the layer whose tensors `layer` uses (itself, mostly)
};

// Bilurax's config.json (core/bilurax.cpp says what the keys mean): layers listed one by one, each an attention with
// normed queries, keys and values, capped scores and chunks of positions, behind a token shift; a dense or routed
// feed-forward, or none; a span of layers that may run several times.
class BiluraxConfig : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "Bilurax";
    struct Layer {
        std::string type;                                   // "attention"
        int64_t heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        double scale = 1.0, softcap = 0.0;
        int64_t chunk = 0;                                  // mask.size: a query sees the keys of its own chunk of positions
        std::string mlp;                                    // "dense" | "moe" | "" (no feed-forward)
        int64_t ff = 0;                                     // dense: inner size; moe: an expert's inner size
        double limit = 0.0;                                 // moe: where an expert's gate and up values are cut off
        int64_t experts = 0, top = 0, groups = 1, keep = 1;
        double router_scale = 1.0;
    };
    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6, logit_softcap = 0.0, embedding_scale = 1.0;
    std::vector<Layer> layers;
    bool has_loop = false;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 1;

    static BiluraxConfig from_json(const Json& raw);
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
};

// Tifepel's config.json (core/tifepel.cpp says what the keys mean): layers listed one by one, each an attention with
// a bias by distance or a state-space mixer, inside hyper-connections over several copies of the stream, with a short
// convolution on every sublayer's input and a gate on its result; routed feed-forwards; a span that may run several times.
class TifepelConfig : public ModelConfig {
public:
    static constexpr const char* kArchitecture = "Tifepel";
    struct Layer {
        std::string type;                                   // "attention" | "mamba2"
        int64_t heads = 0, vdim = 0;
        int64_t kv_heads = 0, dim = 0, bias_max = 0, bias_rows = 0, q_temp_every = 0;      // attention (bias_rows 0: the file's)
        double scale = 1.0, q_temp_coef = 0.0;
        int64_t groups = 0, state = 0, conv = 0, norm_groups = 1;                           // mamba2
        std::string mlp;                                    // "moe" | "" (no feed-forward)
        int64_t ff = 0, experts = 0, identity = 0, top = 0, shared_ff = 0;
    };
    int64_t vocab = 0, width = 0, max_positions = 0, streams = 1, canon_taps = 1;
    int64_t bigram_buckets = 0, bigram_mul_prev = 0, bigram_mul_cur = 0;
    double norm_eps = 1e-5;
    std::vector<Layer> layers;
    bool has_loop = false;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 1;

    static TifepelConfig from_json(const Json& raw);
    std::string architecture() const override { return kArchitecture; }
    Json to_json() const override;
    void validate() const override;
};

// A configuration of an architecture defined outside this library: its normalised config.json
// as the architecture's own `parse` returned it.
class ForeignConfig : public ModelConfig {
public:
    ForeignConfig(std::string arch, Json normalised) : arch_(std::move(arch)), json_(std::move(normalised)) {}
    std::string architecture() const override { return arch_; }
    Json to_json() const override { return json_; }
    void validate() const override {}
private:
    std::string arch_;
    Json json_;
};

struct Architecture {
    std::string name;
    // raw config.json -> typed configuration (type checks; throws ConfigError)
    std::function<std::unique_ptr<ModelConfig>(const Json&)> parse;
    // the parts of every layer, the run order and the tensor names
    std::function<ModelSpec(const ModelConfig&)> describe;
};

void register_architecture(Architecture arch);
const Architecture& get_architecture(const std::string& name);     // unknown -> ConfigError listing the known ones
std::vector<std::string> architectures();

Json read_config_json(const std::string& model_dir);
std::string architecture_name(const Json& raw);                    // architectures[0], or the string under "architecture"
std::unique_ptr<ModelConfig> parse_config(const Json& raw);         // chosen by the registry, validated
std::unique_ptr<ModelConfig> load_config(const std::string& model_dir);
std::string save_config(const ModelConfig& cfg, const std::string& model_dir);
ModelSpec describe(const ModelConfig& cfg);

ModelSpec describe_gpt2(const GPT2Config& cfg);
ModelSpec describe_panupel(const PanupelConfig& cfg);
ModelSpec describe_sovezen(const SovezenConfig& cfg);
ModelSpec describe_bilurax(const BiluraxConfig& cfg);
ModelSpec describe_tifepel(const TifepelConfig& cfg);

}  // namespace sandy
