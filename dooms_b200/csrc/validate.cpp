#include "validate.h"

namespace dooms {

namespace {

constexpr int32_t kLargestHeadDim = 256;

bool holds_matrix(DType t) {
    switch (t) {
        case DType::F16: case DType::Q4_0: case DType::Q5_0: case DType::Q8_0: case DType::Q4_K: case DType::Q6_K: return true;
        default: return false;
    }
}

std::string dims(int64_t rows, int64_t cols) { return std::to_string(rows) + " x " + std::to_string(cols); }

}  // namespace

Status validate_config(const LlamaDecoderConfig & c, size_t n_layer_weights) {
    const bool sizes_ok = c.n_layer >= 1 && c.n_embd >= 4 && c.n_head >= 1 && c.n_head_kv >= 1 && c.head_dim >= 2 && c.n_ff >= 4 && c.n_vocab >= 1 &&
                          c.n_ctx >= 1 && c.n_batch >= 1;
    if (!sizes_ok || !(c.rope_base > 0.f) || !(c.rms_eps > 0.f)) {
        return invalid_argument("decoder configuration: a size is below its minimum, or rope_base / rms_eps is not a positive number");
    }
    if (c.n_head % c.n_head_kv != 0) {
        return invalid_argument("decoder configuration: " + std::to_string(c.n_head) + " query heads cannot be grouped over " + std::to_string(c.n_head_kv) + " key/value heads");
    }
    if (c.prefill_tile < 0 || c.prefill_tile > 2) return invalid_argument("decoder configuration: prefill_tile selects 0 (by chunk size), 1 (CUDA-core tiles) or 2 (tensor-core tiles)");
    const bool power_of_two = (c.head_dim & (c.head_dim - 1)) == 0;
    if (c.head_dim < 4 || c.head_dim > kLargestHeadDim || !power_of_two) {
        return unsupported("head_dim " + std::to_string(c.head_dim) + ": the attention kernels take powers of two from 4 to " + std::to_string(kLargestHeadDim));
    }
    if (c.n_embd % 4 != 0 || c.n_ff % 4 != 0 || (c.n_head * c.head_dim) % 4 != 0) {
        return unsupported("n_embd, n_ff and n_head x head_dim have to be multiples of 4 (the kernels move four floats at a time)");
    }
    if (n_layer_weights != size_t(c.n_layer)) {
        return invalid_argument("the weights describe " + std::to_string(n_layer_weights) + " layers, the configuration " + std::to_string(c.n_layer));
    }
    return Status();
}

Result<std::vector<ExpectedTensor>> expected_tensors(const LlamaDecoderConfig & c, const LlamaDecoderWeights & w) {
    const int64_t E = c.n_embd, F = c.n_ff, V = c.n_vocab, Q = int64_t(c.n_head) * c.head_dim, KV = int64_t(c.n_head_kv) * c.head_dim;
    std::vector<ExpectedTensor> list;
    list.reserve(3 + size_t(c.n_layer) * 12);
    auto matrix = [&](const WeightRef & r, std::string name, int64_t rows, int64_t cols) { list.push_back({&r, std::move(name), rows, cols, TensorRole::Matrix}); };
    auto vector = [&](const WeightRef & r, std::string name, int64_t n) { list.push_back({&r, std::move(name), 1, n, TensorRole::Vector}); };
    matrix(w.token_embd, "token_embd", V, E);
    vector(w.output_norm, "output_norm", E);
    matrix(w.output, "output", V, E);
    for (int32_t l = 0; l < c.n_layer; l++) {
        const LlamaLayerWeights & L = w.layers[size_t(l)];
        const std::string at = "blk." + std::to_string(l) + ".";
        vector(L.attn_norm, at + "attn_norm", E);
        // q, k, v: one fused matrix (rows q | k | v) or three
        if (L.attn_qkv.data) matrix(L.attn_qkv, at + "attn_qkv", Q + 2 * KV, E);
        else {
            matrix(L.attn_q, at + "attn_q", Q, E);
            matrix(L.attn_k, at + "attn_k", KV, E);
            matrix(L.attn_v, at + "attn_v", KV, E);
        }
        // biases: none, one fused vector, or all three
        const bool any_split_bias = L.attn_q_bias.data || L.attn_k_bias.data || L.attn_v_bias.data;
        if (any_split_bias && L.attn_qkv_bias.data) {
            // an entry cannot express "these two exclude each other": the list ends here and the caller reports it at this position
            list.push_back({nullptr, at + "attn", 0, 0, TensorRole::Vector});
            return list;
        }
        if (L.attn_qkv_bias.data) vector(L.attn_qkv_bias, at + "attn_qkv_bias", Q + 2 * KV);
        else if (any_split_bias) {
            vector(L.attn_q_bias, at + "attn_q_bias", Q);
            vector(L.attn_k_bias, at + "attn_k_bias", KV);
            vector(L.attn_v_bias, at + "attn_v_bias", KV);
        }
        matrix(L.attn_output, at + "attn_output", E, Q);
        vector(L.ffn_norm, at + "ffn_norm", E);
        matrix(L.ffn_gate, at + "ffn_gate", F, E);
        matrix(L.ffn_up, at + "ffn_up", F, E);
        matrix(L.ffn_down, at + "ffn_down", E, F);
    }
    return list;
}

Status validate_tensor(const ExpectedTensor & e) {
    if (e.given == nullptr) return invalid_argument(e.name + ": biases come either fused (attn_qkv_bias) or as attn_q / attn_k / attn_v biases, never both");
    const WeightRef & r = *e.given;
    if (r.data == nullptr) return invalid_argument("no data for weight '" + e.name + "'");
    if (r.rows != e.rows || r.cols != e.cols) return invalid_argument("weight '" + e.name + "': got " + dims(r.rows, r.cols) + ", the configuration implies " + dims(e.rows, e.cols));
    if (!dtype_valid(static_cast<int32_t>(r.dtype))) return invalid_argument("weight '" + e.name + "': dtype id " + std::to_string(static_cast<int32_t>(r.dtype)) + " is unknown");
    if (e.role == TensorRole::Vector) {
        if (r.dtype != DType::F32 && r.dtype != DType::F16) return unsupported("vector '" + e.name + "' is stored as " + dtype_name(r.dtype) + "; gains and biases are f32 or f16");
        return Status();
    }
    if (!holds_matrix(r.dtype)) return unsupported("matrix '" + e.name + "' is stored as " + std::string(dtype_name(r.dtype)) + "; the CUDA decoder holds f16, q4_0, q5_0, q8_0, q4_K and q6_K");
    if (r.cols % dtype_block_elems(r.dtype) != 0) return invalid_argument("matrix '" + e.name + "': rows of " + std::to_string(r.cols) + " are not whole " + dtype_name(r.dtype) + " blocks");
    if (r.dtype == DType::F16 && r.cols % 32 != 0) return unsupported("f16 matrix '" + e.name + "': the kernels read rows in groups of 32 elements");
    return Status();
}

Status validate_model(const LlamaDecoderConfig & c, const LlamaDecoderWeights & w) {
    DOOMS_RETURN_IF_ERROR(validate_config(c, w.layers.size()));
    auto list = expected_tensors(c, w);
    if (!list.is_ok()) return list.status();
    // the gate / up rule belongs to a layer: it is judged right after that layer's last tensor, before the next layer's first
    size_t layer = 0;
    for (const ExpectedTensor & e : list.value()) {
        DOOMS_RETURN_IF_ERROR(validate_tensor(e));
        if (layer < w.layers.size() && e.given == &w.layers[layer].ffn_down) {
            const LlamaLayerWeights & L = w.layers[layer];
            if (L.ffn_gate.dtype != L.ffn_up.dtype) {
                return unsupported("blk." + std::to_string(layer) + ": ffn_gate (" + dtype_name(L.ffn_gate.dtype) + ") and ffn_up (" + dtype_name(L.ffn_up.dtype) +
                                   ") differ in type; the fused gate / up kernels read both the same way");
            }
            layer++;
        }
    }
    return Status();
}

}  // namespace dooms
