// TEST INFRASTRUCTURE - not part of the product.
//
// A C entry point around the reference's own CPU statement of the decoder: the double-precision `Reference` class of its decoder test
// (tests/unit/test_metal_llama_decoder.cpp:110-192) together with the `TinyModel` it reads (:30-39) and `to_half_and_back` (:28). Nothing of the reference
// is copied into this repository: oracle/Makefile (target `ref`) cuts those three definitions out of the reference's test file where it lies, into
// oracle/_ref/reference_class.inc, and this file includes that text and compiles it unchanged. The only adaptation is the one the class needs on x86:
// `__fp16` (an Arm type) is mapped to `_Float16` on the compiler's command line; both are IEEE binary16 with round-to-nearest-even conversions.
// The tests hold oracle/oracle.c to this class on f16 models of the reference test's shapes (make_tiny, :57-82).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "backend/metal/metal_llama_decoder.h"   // LlamaDecoderConfig (the header exposes no Metal type)

using namespace dooms;

namespace {
#include "reference_class.inc"
}  // namespace

namespace {

struct Handle {
    TinyModel model;
    Reference * ref = nullptr;
    ~Handle() { delete ref; }
};

std::vector<__fp16> halves(const void * data, size_t n) {
    std::vector<__fp16> v(n);
    std::memcpy(v.data(), data, n * 2);
    return v;
}
std::vector<float> floats(const float * data, size_t n) { return std::vector<float>(data, data + n); }

}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

// The model is handed over tensor by tensor: f16 matrices as raw IEEE half bits, norms and biases as f32. qkv is the row-wise concatenation q | k | v and
// qkv_bias (optional) the concatenated biases, which is how TinyModel holds them.
REF_API void * ref_decoder_new(int32_t n_layer, int32_t n_embd, int32_t n_head, int32_t n_head_kv, int32_t head_dim, int32_t n_ff, int32_t n_vocab, float rope_base,
                               int32_t rope_neox, float rms_eps, const void * embd, const void * output, const float * output_norm) {
    Handle * h = new Handle;
    LlamaDecoderConfig & c = h->model.cfg;
    c.n_layer = n_layer; c.n_embd = n_embd; c.n_head = n_head; c.n_head_kv = n_head_kv; c.head_dim = head_dim; c.n_ff = n_ff; c.n_vocab = n_vocab;
    c.rope_base = rope_base; c.rope_neox = rope_neox != 0; c.rms_eps = rms_eps;
    h->model.embd = halves(embd, size_t(n_vocab) * size_t(n_embd));
    h->model.output = halves(output, size_t(n_vocab) * size_t(n_embd));
    h->model.output_norm = floats(output_norm, size_t(n_embd));
    return h;
}

REF_API void ref_decoder_add_layer(void * handle, const float * attn_norm, const float * ffn_norm, const float * qkv_bias, const void * qkv, const void * wo,
                                   const void * gate, const void * up, const void * down) {
    Handle * h = static_cast<Handle *>(handle);
    const LlamaDecoderConfig & c = h->model.cfg;
    const size_t E = size_t(c.n_embd), F = size_t(c.n_ff), Q = size_t(c.n_head) * size_t(c.head_dim), KV = size_t(c.n_head_kv) * size_t(c.head_dim);
    TinyModel::Layer L;
    L.attn_norm = floats(attn_norm, E);
    L.ffn_norm = floats(ffn_norm, E);
    if (qkv_bias) L.qkv_bias = floats(qkv_bias, Q + 2 * KV);
    L.qkv = halves(qkv, (Q + 2 * KV) * E);
    L.wo = halves(wo, E * Q);
    L.gate = halves(gate, F * E);
    L.up = halves(up, F * E);
    L.down = halves(down, E * F);
    h->model.layers.push_back(std::move(L));
}

// Call once after the last layer: Reference keeps a reference to the model and sizes its caches by the number of layers.
REF_API void ref_decoder_seal(void * handle) {
    Handle * h = static_cast<Handle *>(handle);
    delete h->ref;
    h->ref = new Reference(h->model);
}

// Restarts the sequence (a new Reference: the class has no reset, its position is the length of its caches).
REF_API void ref_decoder_reset(void * handle) { ref_decoder_seal(handle); }

// One position: n_embd input values in, n_vocab logits out (Reference::step).
REF_API void ref_decoder_step(void * handle, const double * input, double * logits) {
    Handle * h = static_cast<Handle *>(handle);
    const std::vector<double> in(input, input + h->model.cfg.n_embd);
    const std::vector<double> out = h->ref->step(in);
    std::memcpy(logits, out.data(), out.size() * sizeof(double));
}

// Row `token` of the embedding table (Reference::embedding).
REF_API void ref_decoder_embedding(void * handle, int32_t token, double * out) {
    Handle * h = static_cast<Handle *>(handle);
    const std::vector<double> e = h->ref->embedding(token);
    std::memcpy(out, e.data(), e.size() * sizeof(double));
}

REF_API void ref_decoder_free(void * handle) { delete static_cast<Handle *>(handle); }
