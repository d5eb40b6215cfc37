#include "model.h"

namespace sandy {

Model::Model(ModelSpec spec) : spec_(std::move(spec)) {
    embedding_ = make_part<Embedding>("embedding", spec_.embedding);
    position_ = make_part<PositionEncoding>("position", spec_.position);
    for (const LayerSpec& l : spec_.layers) {
        const PartFactory& bf = get_part("block", l.block);
        BlockParts p;
        p.mixer = make_part<Mixer>("mixer", l.mixer);
        p.feed_forward = make_part<FeedForward>("feed_forward", l.feed_forward);
        for (const auto& kv : l.norms) p.norms[kv.first] = make_part<Norm>("norm", kv.second);
        for (const auto& kv : l.wraps) p.wraps[kv.first] = make_part<Wrap>("wrap", kv.second);
        std::string missing;
        for (const auto& n : bf.norm_names)
            if (!p.norms.count(n)) missing += (missing.empty() ? "" : ", ") + n;
        if (!missing.empty()) throw ConfigError("block '" + l.block + "' needs norms " + missing);
        p.width = spec_.width;
        p.params = l.block_params;
        if (!bf.make_block) throw ConfigError("part kind '" + l.block + "' is not a block");
        blocks_.push_back(bf.make_block(std::move(p)));
    }
    final_norm_ = make_part<Norm>("norm", spec_.final_norm);
    head_ = make_part<Head>("head", spec_.head);
    for (const PartSpec& r : spec_.remixes) remixes_.push_back(make_part<Remix>("remix", r));
    if (spec_.streams < 1) throw ConfigError("a model has at least one residual stream");
    if (spec_.streams > 1 && !remixes_.empty()) throw ConfigError("stream mixes between layers work on one residual stream");
    if ((spec_.embedding_cache >= 0) != embedding_->cache_spec().has_state())
        throw ConfigError("the embedding's state and the cache entry named for it do not go together");
    for (const LayerCall& c : spec_.schedule) {
        if (c.cache == spec_.embedding_cache) throw ConfigError("a layer uses the embedding's cache entry");
        if (c.layer < 0 || c.layer >= (int)blocks_.size())
            throw ConfigError("run order names layer " + std::to_string(c.layer) + ", the model has " + std::to_string(blocks_.size()));
        if (c.remix >= (int)remixes_.size())
            throw ConfigError("run order names stream mix " + std::to_string(c.remix) + ", the model has " + std::to_string(remixes_.size()));
    }
}

std::vector<Model::PartRef> Model::parts() const {
    std::vector<PartRef> out;
    out.push_back({embedding_.get(), &spec_.embedding});
    out.push_back({position_.get(), &spec_.position});
    for (size_t i = 0; i < blocks_.size(); i++) {
        const LayerSpec& l = spec_.layers[i];
        out.push_back({&blocks_[i]->mixer(), &l.mixer});
        out.push_back({&blocks_[i]->feed_forward(), &l.feed_forward});
        for (auto& kv : blocks_[i]->norms()) out.push_back({kv.second.get(), &l.norms.at(kv.first)});
        for (auto& kv : blocks_[i]->wraps()) out.push_back({kv.second.get(), &l.wraps.at(kv.first)});
    }
    for (size_t i = 0; i < remixes_.size(); i++) out.push_back({remixes_[i].get(), &spec_.remixes[i]});
    out.push_back({final_norm_.get(), &spec_.final_norm});
    out.push_back({head_.get(), &spec_.head});
    return out;
}

TensorRequests Model::tensor_requests() const {
    TensorRequests out;
    for (const PartRef& p : parts())
        for (const auto& kv : p.part->requests()) {
            auto name = p.spec->tensors.find(kv.first);
            if (name == p.spec->tensors.end())
                throw ConfigError(p.spec->kind + ": the model description names no tensor for '" + kv.first + "'");
            auto hit = out.find(name->second);
            if (hit != out.end() && hit->second.shape != kv.second.shape)
                throw ConfigError("tensor '" + name->second + "' is requested with two shapes");
            out[name->second] = kv.second;
        }
    return out;
}

void Model::bind(const TensorMap& tensors, DType dtype) {
    if (dtype != DType::F32 && dtype != DType::BF16) throw ValueError("compute dtype must be float32 or bfloat16");
    dtype_ = dtype;
    for (const PartRef& p : parts()) {
        TensorMap local;
        for (const auto& kv : p.part->requests()) {
            auto it = tensors.find(p.spec->tensors.at(kv.first));
            if (it == tensors.end()) throw ConfigError("tensor '" + p.spec->tensors.at(kv.first) + "' was not loaded");
            local[kv.first] = it->second;
        }
        if (p.part == head_.get()) head_->bind_head(local, dtype, head_->tied() ? embedding_->table() : nullptr);
        else p.part->bind(local, dtype);
    }
    bound_ = true;
}

std::vector<CacheSpec> Model::cache_specs() const {
    std::vector<CacheSpec> specs((size_t)spec_.n_caches());
    std::vector<char> seen(specs.size(), 0);
    for (const LayerCall& c : spec_.schedule) {
        const CacheSpec s = blocks_[(size_t)c.layer]->cache_spec();
        if (seen[(size_t)c.cache] && specs[(size_t)c.cache] != s)
            throw ConfigError("cache entry " + std::to_string(c.cache) + " is used by layers with different needs");
        specs[(size_t)c.cache] = s;
        seen[(size_t)c.cache] = 1;
    }
    if (spec_.embedding_cache >= 0) specs[(size_t)spec_.embedding_cache] = embedding_->cache_spec();
    return specs;
}

bool Model::graph_safe() const {
    for (const PartRef& p : parts())
        if (!p.part->graph_safe()) return false;
    return true;
}

size_t Model::weight_bytes() const {
    size_t total = head_->weight_bytes() + final_norm_->weight_bytes();
    for (const LayerCall& c : spec_.schedule) {
        Block& b = *blocks_[(size_t)c.layer];
        total += b.mixer().weight_bytes() + b.feed_forward().weight_bytes();
        for (auto& kv : b.norms()) total += kv.second->weight_bytes();
        for (auto& kv : b.wraps()) total += kv.second->weight_bytes();
        if (c.remix >= 0) total += remixes_[(size_t)c.remix]->weight_bytes();
    }
    return total;
}

Tensor Model::forward(StepContext& ctx) {
    Workspace& ws = *ctx.workspace;
    ctx.position = position_.get();
    ctx.embedding_cache = spec_.embedding_cache;
    Tensor x = ws.get("stream", ctx.n_tokens, spec_.width, DType::F32);
    embedding_->forward(ctx, x);
    const Tensor one_stream = x;
    if (spec_.streams > 1) {
        // the embedding's output enters every copy of the stream; the blocks work on all of them side by side
        x = ws.get("streams", ctx.n_tokens, spec_.width * spec_.streams, DType::F32);
        ops::streams_spread(ctx.launch, one_stream, x, spec_.streams);
    }
    Tensor x0;
    if (!remixes_.empty()) {
        // the embedding's output stays at hand for the stream mixes
        x0 = ws.get("stream_at_embedding", ctx.n_tokens, spec_.width, DType::F32);
        cuda_check(cudaMemcpyAsync(x0.data, x.data, (size_t)x.numel() * sizeof(float), cudaMemcpyDeviceToDevice, ctx.launch.stream),
                   "keeping the embedding's output");
    }
    ctx.owed = StepContext::OwedWrite();
    // a block may leave its last sublayer's write into the streams owed to whoever reads them next
    auto settle = [&](Tensor* sum_out) {
        if (!ctx.owed.wrap) return false;
        Wrap::Input in;
        in.gate = ctx.owed.gate;
        Wrap* w = ctx.owed.wrap;
        const Tensor y = ctx.owed.y;
        ctx.owed = StepContext::OwedWrite();
        w->write(ctx, x, y, in, sum_out);
        return true;
    };
    for (const LayerCall& c : spec_.schedule) {
        if (c.remix >= 0) {
            settle(nullptr);
            remixes_[(size_t)c.remix]->forward(ctx, x, x0);
        }
        if (!blocks_[(size_t)c.layer]->settles_owed()) settle(nullptr);
        blocks_[(size_t)c.layer]->forward(ctx, x, c);
    }
    if (spec_.streams > 1) {
        Tensor total = one_stream;            // the final norm reads the sum of the copies
        if (!settle(&total)) {
            ops::StreamsStep sum;
            sum.sum_out = &total;
            ops::streams_step(ctx.launch, x, spec_.streams, sum);
        }
        x = one_stream;
    } else {
        settle(nullptr);
    }
    Tensor logits = ws.get("logits", ctx.n_rows, spec_.vocab_size, DType::F32);
    if (ctx.n_rows) {
        Tensor y = ws.get("final_normed", ctx.n_rows, spec_.width, ctx.compute_dtype);
        final_norm_->forward(ctx, x, y, ctx.logit_rows, ctx.n_rows);
        head_->forward(ctx, y, logits);
    }
    return logits;
}

std::unique_ptr<Model> load_model(const std::string& model_dir, DType dtype) {
    std::shared_ptr<ModelConfig> config = load_config(model_dir);
    ModelSpec spec = describe(*config);
    std::unique_ptr<Model> model(new Model(std::move(spec)));
    const TensorMap tensors = load_weights(model_dir, model->tensor_requests(), model->spec().name_prefixes, model->spec().ignored_tensors);
    model->bind(tensors, dtype);
    model->set_config(std::move(config));
    return model;
}

std::string write_random_model(const ModelConfig& config, const std::string& out_dir, uint64_t seed, StoreDType store) {
    config.validate();
    Model model(describe(config));
    const TensorMap tensors = random_tensors(model.tensor_requests(), seed, store);
    save_config(config, out_dir);
    write_safetensors(out_dir + "/" + kWeightFile, tensors);
    return out_dir;
}

}  // namespace sandy
