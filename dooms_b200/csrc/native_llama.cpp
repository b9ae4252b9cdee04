// GGUF file -> decoder. The file's metadata supplies every hyperparameter and its tensors are handed to the decoder as host pointers into the mapping.
// The contract is the reference loader's (src/pipeline/native_llama.cpp:9-102): the metadata keys, the tensor names, which of them may be absent, the order
// in which a bad file is refused and the status code of each refusal. The structure is this backend's own: a small reader over the parsed file for the
// architecture-prefixed metadata, and a table of tensor rules walked once for the model-level tensors and once per layer.
#include <algorithm>
#include <fstream>
#include <optional>
#include <string>

#include "cuda_llama_decoder.h"
#include "gguf.h"

namespace dooms {

namespace {

// Metadata of one architecture ("llama." / "qwen2." keys) with the file's name kept for messages.
class ArchMetadata {
public:
    ArchMetadata(const GgufFile & file, const std::string & path, const std::string & arch) : file_(file), path_(path), prefix_(arch + ".") {}

    std::optional<int64_t> integer(const char * key) const {
        auto v = file_.get_uint(prefix_ + key);
        if (!v.is_ok()) return std::nullopt;
        return static_cast<int64_t>(v.value());
    }
    std::optional<double> real(const char * key) const {
        auto v = file_.get_float(prefix_ + key);
        if (!v.is_ok()) return std::nullopt;
        return v.value();
    }
    std::optional<std::string> text(const char * key) const {
        auto v = file_.get_string(prefix_ + key);
        if (!v.is_ok()) return std::nullopt;
        return v.value();
    }
    Status missing(const std::string & what) const { return invalid_argument("model file '" + path_ + "': metadata " + prefix_ + what + " is absent"); }
    std::string key(const char * k) const { return prefix_ + k; }

private:
    const GgufFile & file_;
    const std::string & path_;
    std::string prefix_;
};

// When a tensor has to be there.
enum class Need {
    Always,
    Optional,
    UnlessFusedQkv,     // attn_q / attn_k / attn_v weights: required when the file has no attn_qkv.weight, not looked at otherwise
    QueryBias,          // attn_q.bias: not looked at when attn_qkv.bias exists; required for qwen2, optional for llama
    KeyValueBias,       // attn_k.bias / attn_v.bias: as QueryBias, and required as soon as attn_q.bias is there (all three or none)
};

struct LayerRule { const char * suffix; WeightRef LlamaLayerWeights::* slot; Need need; };

// In the order the refusals are specified in.
const LayerRule kLayerRules[] = {
    {"attn_norm.weight", &LlamaLayerWeights::attn_norm, Need::Always},
    {"attn_qkv.weight", &LlamaLayerWeights::attn_qkv, Need::Optional},
    {"attn_q.weight", &LlamaLayerWeights::attn_q, Need::UnlessFusedQkv},
    {"attn_k.weight", &LlamaLayerWeights::attn_k, Need::UnlessFusedQkv},
    {"attn_v.weight", &LlamaLayerWeights::attn_v, Need::UnlessFusedQkv},
    {"attn_qkv.bias", &LlamaLayerWeights::attn_qkv_bias, Need::Optional},
    {"attn_q.bias", &LlamaLayerWeights::attn_q_bias, Need::QueryBias},
    {"attn_k.bias", &LlamaLayerWeights::attn_k_bias, Need::KeyValueBias},
    {"attn_v.bias", &LlamaLayerWeights::attn_v_bias, Need::KeyValueBias},
    {"attn_output.weight", &LlamaLayerWeights::attn_output, Need::Always},
    {"ffn_norm.weight", &LlamaLayerWeights::ffn_norm, Need::Always},
    {"ffn_gate.weight", &LlamaLayerWeights::ffn_gate, Need::Always},
    {"ffn_up.weight", &LlamaLayerWeights::ffn_up, Need::Always},
    {"ffn_down.weight", &LlamaLayerWeights::ffn_down, Need::Always},
};

// Points `out` at the named tensor's bytes: vectors as one row, matrices as [rows][cols]. An absent tensor leaves `out` untouched and is an error only
// when `required`.
Status bind_tensor(const GgufFile & file, const std::string & path, const std::string & name, bool required, WeightRef * out) {
    auto found = file.find_tensor(name);
    if (!found.is_ok()) {
        if (!required) return Status();
        return invalid_argument("model file '" + path + "': tensor " + name + " is absent");
    }
    const GgufTensorInfo & t = *found.value();
    if (t.rank != 1 && t.rank != 2) return invalid_argument("model file '" + path + "': tensor " + name + " has " + std::to_string(t.rank) + " dimensions, expected 1 or 2");
    out->data = file.tensor_data(t);
    out->dtype = t.dtype;
    out->rows = t.rank == 1 ? 1 : t.shape[0];
    out->cols = t.rank == 1 ? t.shape[0] : t.shape[1];
    return Status();
}

Status bind_layer(const GgufFile & file, const std::string & path, int32_t index, bool biased_arch, LlamaLayerWeights * layer) {
    const std::string stem = "blk." + std::to_string(index) + ".";
    for (const LayerRule & rule : kLayerRules) {
        bool look = true, required = false;
        switch (rule.need) {
            case Need::Always: required = true; break;
            case Need::Optional: break;
            case Need::UnlessFusedQkv: look = layer->attn_qkv.data == nullptr; required = true; break;
            case Need::QueryBias: look = layer->attn_qkv_bias.data == nullptr; required = biased_arch; break;
            case Need::KeyValueBias: look = layer->attn_qkv_bias.data == nullptr; required = biased_arch || layer->attn_q_bias.data != nullptr; break;
        }
        if (look) DOOMS_RETURN_IF_ERROR(bind_tensor(file, path, stem + rule.suffix, required, &(layer->*rule.slot)));
    }
    return Status();
}

}  // namespace

Result<std::unique_ptr<CudaLlamaDecoder>> load_native_llama(const std::string & path, const NativeLlamaOptions & options, const CudaOptions & cuda) {
    if (options.n_ctx < 1 || options.n_batch < 1) return invalid_argument("load_native_llama: n_ctx and n_batch have to be positive");
    if (!std::ifstream(path, std::ios::binary).good()) return not_found("model file '" + path + "' cannot be opened");
    auto parsed = GgufFile::open(path);
    if (!parsed.is_ok()) return unsupported("model file '" + path + "' is not a GGUF file this backend reads: " + parsed.status().message());
    const GgufFile & file = parsed.value();

    // Which block: llama rotates adjacent pairs; qwen2 is the same block with q / k / v biases and pairs split across the halves of a head.
    auto arch_name = file.get_string("general.architecture");
    if (!arch_name.is_ok()) return invalid_argument("model file '" + path + "': metadata general.architecture is absent");
    const bool qwen2 = arch_name.value() == "qwen2";
    if (!qwen2 && arch_name.value() != "llama") {
        return unsupported("model file '" + path + "' holds a '" + arch_name.value() + "' model; the CUDA decoder implements the llama and qwen2 blocks");
    }
    const ArchMetadata md(file, path, arch_name.value());
    if (const auto scaling = md.text("rope.scaling.type"); scaling && *scaling != "none") {
        return unsupported("model file '" + path + "' asks for rotary scaling of type '" + *scaling + "', which the CUDA decoder does not implement");
    }

    LlamaDecoderConfig cfg;
    const struct { const char * key; int32_t * field; } sizes[] = {
        {"block_count", &cfg.n_layer}, {"embedding_length", &cfg.n_embd}, {"attention.head_count", &cfg.n_head},
        {"attention.head_count_kv", &cfg.n_head_kv}, {"feed_forward_length", &cfg.n_ff},
    };
    for (const auto & s : sizes) {
        const auto v = md.integer(s.key);
        if (!v) return md.missing(s.key);
        *s.field = static_cast<int32_t>(*v);
    }
    if (cfg.n_head < 1 || cfg.n_embd % cfg.n_head != 0) return invalid_argument("model file '" + path + "': embedding_length does not divide into head_count heads");
    cfg.head_dim = cfg.n_embd / cfg.n_head;
    // Heads whose key, value or rotated width differs from embedding_length / head_count are another architecture variant.
    for (const char * key : {"attention.key_length", "attention.value_length", "rope.dimension_count"}) {
        const auto v = md.integer(key);
        if (v && *v != cfg.head_dim) {
            return unsupported("model file '" + path + "': " + md.key(key) + " is " + std::to_string(*v) + " but a head is " + std::to_string(cfg.head_dim) +
                               " wide; the CUDA decoder rotates and attends over whole heads only");
        }
    }
    const auto freq_base = md.real("rope.freq_base"), rms_eps = md.real("attention.layer_norm_rms_epsilon");
    if (!freq_base || !rms_eps) return md.missing("rope.freq_base / " + md.key("attention.layer_norm_rms_epsilon"));
    cfg.rope_base = static_cast<float>(*freq_base);
    cfg.rms_eps = static_cast<float>(*rms_eps);
    cfg.rope_neox = qwen2;
    const auto trained_context = md.integer("context_length");
    if (!trained_context) return md.missing("context_length");
    if (options.n_ctx > *trained_context) {
        return invalid_argument("load_native_llama: n_ctx = " + std::to_string(options.n_ctx) + " is more than the " + std::to_string(*trained_context) +
                                " positions the model was built for");
    }
    cfg.n_ctx = options.n_ctx;
    cfg.n_batch = std::min(options.n_batch, options.n_ctx);
    cfg.spin_wait = options.spin_wait;
    cfg.prefill_tile = options.prefill_tile;

    LlamaDecoderWeights weights;
    DOOMS_RETURN_IF_ERROR(bind_tensor(file, path, "token_embd.weight", true, &weights.token_embd));
    DOOMS_RETURN_IF_ERROR(bind_tensor(file, path, "output_norm.weight", true, &weights.output_norm));
    DOOMS_RETURN_IF_ERROR(bind_tensor(file, path, "output.weight", false, &weights.output));
    if (weights.output.data == nullptr) weights.output = weights.token_embd;      // tied: the output projection is the embedding table
    cfg.n_vocab = static_cast<int32_t>(weights.token_embd.rows);
    weights.layers.resize(static_cast<size_t>(std::max(cfg.n_layer, 0)));
    for (int32_t l = 0; l < cfg.n_layer; l++) DOOMS_RETURN_IF_ERROR(bind_layer(file, path, l, qwen2, &weights.layers[static_cast<size_t>(l)]));
    return CudaLlamaDecoder::create(cfg, weights, cuda);
}

}  // namespace dooms
