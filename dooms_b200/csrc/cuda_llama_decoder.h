#pragma once
// A llama / qwen2 text decoder on hand-written CUDA kernels for B200 (sm_100a). The class keeps the method set, argument meaning and error behaviour of the
// reference's MetalLlamaDecoder (src/backend/metal/metal_llama_decoder.h:63-106) so that its callers (src/pipeline/llm_pipeline.cpp:60,187-212,
// bench/bench_llm.cpp:92-114) compile against either: create / config / position / reset / eval_embeddings / eval_tokens / pending_token / logits /
// generate / profile_pass. Activations are f32, weight matrices stay in their GGUF block format in device memory (f16, q4_0, q5_0, q8_0, q4_K, q6_K),
// the KV cache is f16 in device memory. This header exposes no CUDA type. There is no CPU fallback: create() fails with Unsupported without a device.
#include <cstdint>
#include <functional>
#include <memory>
#include <vector>

#include "dtype.h"
#include "status.h"

namespace dooms {

// A tensor in host memory; copied at creation, not referenced afterwards (src/backend/weight_ref.h:11-15). Row-major [rows][cols], cols = input width.
struct WeightRef {
    const void * data = nullptr;
    DType dtype = DType::F32;
    int64_t rows = 0, cols = 0;
};

// metal_llama_decoder.h:20-39
struct LlamaDecoderConfig {
    int32_t n_layer = 0, n_embd = 0, n_head = 0, n_head_kv = 0, head_dim = 0, n_ff = 0, n_vocab = 0;
    float rope_base = 0.f;
    bool rope_neox = false;
    float rms_eps = 0.f;
    int32_t n_ctx = 0, n_batch = 0;
    bool spin_wait = true;      // generate(): poll the step's event on the calling thread instead of sleeping in the driver
    int32_t prefill_tile = 0;   // 0 automatic, 1 CUDA-core tiles, 2 tcgen05 tensor-core tiles (when the widths allow)
};

// metal_llama_decoder.h:42-58
struct LlamaLayerWeights {
    WeightRef attn_norm;
    WeightRef attn_q, attn_k, attn_v, attn_qkv;
    WeightRef attn_q_bias, attn_k_bias, attn_v_bias, attn_qkv_bias;
    WeightRef attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down;
};
struct LlamaDecoderWeights {
    WeightRef token_embd, output_norm, output;
    std::vector<LlamaLayerWeights> layers;
};

// Where and how this process's share of the model runs (no counterpart in the reference, which has one GPU).
struct CudaOptions {
    int32_t device = 0;
    int32_t tp_rank = 0, tp_size = 1;        // tensor parallelism: q/k/v/gate/up split by output rows, attn_output/ffn_down by input columns
    const void * nccl_unique_id = nullptr;   // 128 bytes shared by the ranks of the group (tp_size > 1)
    const char * nccl_library = nullptr;
    bool operand_bf16 = false;               // reserved: bf16 tensor-core operands; true is refused with Unsupported (the tiles hold f16, the reference's rounding)
    bool use_graphs = true;                  // decode steps replay a captured CUDA graph
    int32_t max_sequences = 1;               // independent KV caches ("slots") of n_ctx positions each; see select_sequence / decode_batch
};

// A rank's share of the model under tensor parallelism: whole heads, a slice of the feed-forward width, a slice of the vocabulary.
// Column shards have to be whole quantization blocks. The feed-forward width is therefore dealt in units of ffn_block columns, the first n_ff / ffn_block %
// tp_size ranks taking one unit more. The columns of attn_output follow the heads, which no choice can move; where a rank's columns [q_row0, q_row0 +
// q_rows) start or end inside a block, the rank holds the blocks that cover them, [attn_col0, attn_col0 + attn_cols), and multiplies them with an input
// that is zero outside its own columns: a block on the boundary is held by both neighbours, each using its own part of it.
struct TpShare {
    int64_t q_row0 = 0, q_rows = 0, kv_row0 = 0, kv_rows = 0, ff_row0 = 0, ff_rows = 0, vocab_row0 = 0, vocab_rows = 0;
    int64_t attn_col0 = 0, attn_cols = 0;
};
//   InvalidArgument  tp_rank outside [0, tp_size), a block size < 1
//   Unsupported  n_head or n_head_kv is not a multiple of tp_size, n_ff or the attention width is not whole blocks, fewer feed-forward units than ranks
Result<TpShare> tp_share(const LlamaDecoderConfig & config, int32_t tp_rank, int32_t tp_size, int64_t attn_block = 1, int64_t ffn_block = 1);

class CudaLlamaDecoder {
public:
    //   Unsupported  no CUDA device, a weight type the kernels do not take, a head_dim that is not a power of two in [4, 256]
    //   InvalidArgument  the weights do not have the shapes the config implies
    //   ResourceExhausted  device memory
    static Result<std::unique_ptr<CudaLlamaDecoder>> create(const LlamaDecoderConfig & config, const LlamaDecoderWeights & weights,
                                                            const CudaOptions & options = CudaOptions());
    ~CudaLlamaDecoder();
    CudaLlamaDecoder(const CudaLlamaDecoder &) = delete;
    CudaLlamaDecoder & operator=(const CudaLlamaDecoder &) = delete;

    const LlamaDecoderConfig & config() const;
    int32_t position() const;
    void reset();
    Status eval_embeddings(const float * embeddings, int32_t n);
    Status eval_tokens(const std::vector<int32_t> & tokens);
    Status eval_tokens(const int32_t * tokens, int32_t n);
    // Rows of the embedding table as f32 (n x n_embd floats into out), looked up and dequantized on the device by the kernel that eval_tokens uses: what
    // a caller that mixes token rows with rows of its own (image embeddings, src/pipeline/vlm_pipeline.cpp:180-189) hands to eval_embeddings.
    //   InvalidArgument  no ids, no room, an id outside the vocabulary
    Status embed_tokens(const int32_t * tokens, int32_t n, float * out);
    Result<int32_t> pending_token();
    Result<std::vector<float>> logits();
    Status logits_into(float * out, int64_t capacity);
    Status generate(int32_t max_tokens, int32_t depth, const std::function<bool(int32_t)> & on_token);

    // ---- several sequences on one decoder (no counterpart in the reference, which serves one request at a time: python/dooms/server.py:262-269) ----
    // The decoder holds max_sequences KV-cache slots. Every call above acts on the selected slot (0 at creation); select_sequence switches. logits() is
    // kept for the last evaluation only.   InvalidArgument  slot outside [0, max_sequences)
    int32_t max_sequences() const;
    int32_t selected_sequence() const;
    Status select_sequence(int32_t slot);
    // `steps` greedy decode steps for n slots at once, one pass over the weights per step for all of them (the chunk path's tensor-core kernels with one
    // row per sequence, each attending over its own slot). slots[i] < 0 marks an idle row. Every listed slot needs a pending token, as for generate();
    // out_tokens[t * n + i] receives the token step t produced for slots[i] (-1 for idle rows). Afterwards each slot's position has advanced by `steps` and
    // its pending token is the last one produced: as after `steps` calls of eval_tokens({pending}).
    //   Unsupported  built with max_sequences = 1, tensor parallelism, or shapes the tensor-core chunk path does not take (max_batch_rows() == 0)
    //   InvalidArgument  a slot out of range or listed twice, a slot without pending token, steps outside [1, 256]     ResourceExhausted  context, rows
    int32_t max_batch_rows() const;
    Status decode_batch(const int32_t * slots, int32_t n, int32_t steps, int32_t * out_tokens);

    struct KernelTime { const char * kind; int32_t dispatches; double gpu_ms; };
    Result<std::vector<KernelTime>> profile_pass(int32_t rows = 1);

    // Device-side measurements of the last calls (CUDA events on the decoder's stream).
    struct Timings {
        double last_eval_ms = 0, last_generate_ms = 0;
        int64_t last_eval_launches = 0, last_generate_launches = 0, weight_bytes = 0, kv_bytes = 0;
        double last_batch_ms = 0;            // device time of the last decode_batch call's steps
        int64_t last_batch_launches = 0;
        int64_t tp_peer_allreduce = 0;       // 1: decode steps reduce over peer memory (kernels/allreduce_peer.cu); 0: NCCL, or one GPU
        int64_t tp_symmetric_window = 0;     // 1: the buffers NCCL reduces lie in a registered symmetric window (its low-latency kernels apply)
    };
    Timings timings() const;

private:
    struct Impl;
    explicit CudaLlamaDecoder(std::unique_ptr<Impl> impl);
    std::unique_ptr<Impl> impl_;
};

struct NativeLlamaOptions {   // src/pipeline/native_llama.h:15-20
    int32_t n_ctx = 2048, n_batch = 512;
    bool spin_wait = true;
    int32_t prefill_tile = 0;
};
//   NotFound  no such file     Unsupported  not a GGUF this decoder runs     InvalidArgument  bad options or inconsistent metadata
Result<std::unique_ptr<CudaLlamaDecoder>> load_native_llama(const std::string & path, const NativeLlamaOptions & options = NativeLlamaOptions(),
                                                            const CudaOptions & cuda = CudaOptions());

}  // namespace dooms
