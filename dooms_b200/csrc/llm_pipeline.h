#pragma once
// A text language model on the CUDA decoder: the surface of the reference's `Llm` (src/pipeline/llm_pipeline.h:16-82) for the decoder's own engine:
// tokenization, seeded sampling, streaming with complete UTF-8 pieces and stop strings, timings. The reference takes vocabulary, tokenizer and sampler
// from llama.cpp (src/models/vlm/text_decoder.*), which is not part of this backend; here they are this file's own: the vocabulary is read from the GGUF
// metadata (tokenizer.ggml.*), byte-level BPE files are tokenized by merge rank within the words their pre-tokenizer pattern cuts, sentencepiece files
// by piece score, and the sampler is a plain temperature / top-k / top-p / repetition penalty chain on a seeded generator. Chat templates are not evaluated as Jinja: as llama.cpp's llama_chat_apply_template does (the call the reference
// makes, src/models/vlm/text_decoder.cpp:257-278), the file's template is recognised by the markers it contains and the conversation is written in that
// family's published format (ChatML, Llama 3, SmolVLM); any other template is Unsupported.
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "cuda_llama_decoder.h"
#include "gguf.h"

namespace dooms {

// text_decoder.h:24-30
struct SamplerOptions {
    float temperature = 0.f;       // 0: greedy
    int32_t top_k = 40;            // 0: off
    float top_p = 0.95f;           // in (0, 1]; 1: off
    float repeat_penalty = 1.f;    // > 0; 1: off; applied to the last 64 tokens
    uint32_t seed = 0;
};

struct ChatMessage {             // text_decoder.h:32-35
    std::string role, content;
};

// The vocabulary of a GGUF file: token id <-> bytes.
class Vocab {
public:
    //   InvalidArgument  the file has no tokenizer.ggml.tokens     Unsupported  a tokenizer model other than "gpt2" (byte-level BPE) or "llama" (sentencepiece)
    static Result<Vocab> from_gguf(const GgufFile & file);
    int32_t size() const { return int32_t(pieces_.size()); }
    // The bytes token `id` stands for (byte-level BPE: the GPT-2 byte alphabet undone; sentencepiece: U+2581 -> space, <0xHH> -> that byte); special
    // tokens give no text.
    const std::string & piece(int32_t id) const;
    bool is_end_of_generation(int32_t id) const;
    int32_t bos() const { return bos_; }
    bool add_bos() const { return add_bos_; }
    // Text -> ids.   InvalidArgument  empty text, or a byte the vocabulary has no token for
    //   byte-level BPE: the text is cut into words the way the file's pre-tokenizer does (tokenizer.ggml.pre: the Llama 3 pattern for "llama-bpe", the
    //   Qwen2 pattern for "qwen2", the GPT-2 pattern otherwise), each word's bytes are merged pairwise by rank;
    //   sentencepiece: spaces become U+2581 (one is put in front of the text unless tokenizer.ggml.add_space_prefix says no), the text's characters are merged pairwise, best-scoring vocabulary piece
    //   first (tokenizer.ggml.scores; leftmost on ties), and what is no piece at the end goes out byte by byte as <0xHH>.
    // parse_special: a control token's text inside `text` ("<|im_start|>") becomes that token's id instead of being tokenized as characters (what a
    // chat template's output needs); user-defined tokens are matched either way. The longest token at the earliest position wins.
    Result<std::vector<int32_t>> tokenize(const std::string & text, bool add_special, bool parse_special = false) const;

    // The conversation in the format of the file's chat template (tokenizer.chat_template), with the opening of the assistant's turn at the end when
    // add_generation_prompt (TextDecoder::apply_chat_template, text_decoder.cpp:257-278).
    //   InvalidArgument  no messages, a message with an empty role     Unsupported  the file has no template, or one of a family this library does not know
    Result<std::string> apply_chat_template(const std::vector<ChatMessage> & messages, bool add_generation_prompt = true) const;
    bool has_chat_template() const { return apply_chat_template({{"user", "x"}}, true).is_ok(); }      // llm_pipeline.cpp:82

private:
    Status tokenize_plain(const std::string & text, bool space_in_front, std::vector<int32_t> * out) const;
    std::vector<std::pair<std::string, int32_t>> marked_;       // control and user-defined tokens that are looked for in text, longest first
    std::vector<bool> control_;
    std::string chat_template_;
    std::vector<std::string> pieces_;                           // decoded bytes per id
    std::vector<std::string> raw_;                              // as stored
    std::unordered_map<std::string, int32_t> ids_;              // raw token -> id
    std::unordered_map<std::string, int32_t> merge_rank_;       // "left right" -> rank
    std::vector<float> scores_;                                 // sentencepiece: per id
    std::vector<bool> special_;
    std::vector<int32_t> eog_;
    int32_t bos_ = -1;
    bool add_bos_ = false, byte_level_ = false, ignore_merges_ = false;
    bool space_prefix_ = true;                                  // sentencepiece: a space goes in front of the text (tokenizer.ggml.add_space_prefix)
    int pre_ = 0;                                               // 0 GPT-2, 1 Llama 3, 2 Qwen2
};

// Seeded token choice from a row of logits.
class Sampler {
public:
    //   InvalidArgument  temperature < 0, top_p outside (0, 1], top_k < 0, repeat_penalty <= 0
    static Result<Sampler> create(const SamplerOptions & options);
    bool greedy() const { return o_.temperature == 0.f && o_.repeat_penalty == 1.f; }
    int32_t sample(const float * logits, int32_t n);      // also records the token for the repetition penalty
    void accept(int32_t token);                           // a token chosen elsewhere (greedy on the device)

private:
    SamplerOptions o_;
    uint64_t state_ = 0;
    std::vector<int32_t> recent_;
    double uniform();
};

struct LlmGenerateOptions {      // llm_pipeline.h:28-32
    int32_t max_new_tokens = 128;
    SamplerOptions sampler;
    std::vector<std::string> stop;
};
struct LlmTimings {              // llm_pipeline.h:34-40
    double prefill_ms = 0, first_token_ms = 0, decode_ms = 0;
    int64_t prompt_tokens = 0, generated_tokens = 0;
    double decode_ms_per_token() const { return generated_tokens > 1 ? decode_ms / double(generated_tokens - 1) : 0.0; }
};
struct LlmGeneration {           // llm_pipeline.h:42-47
    std::string text;
    std::vector<int32_t> tokens;
    bool stopped = false, cancelled = false;
};

// Generated tokens -> text, piece by piece: a piece is handed on only when it is complete UTF-8 and cannot be the beginning of a stop string; generation
// ends at an end-of-generation token, at a stop string (the text ends before it) or when the callback declines.
class TextStream {
public:
    TextStream(const Vocab & vocab, const std::vector<std::string> & stops, std::function<bool(const std::string &)> on_text, LlmGeneration * out);
    bool push(int32_t token);      // false: generation is over
    void finish();                 // hands on what was held back, where the ending allows it
private:
    bool release(size_t n);
    const Vocab & vocab_;
    const std::vector<std::string> & stops_;
    std::function<bool(const std::string &)> on_text_;
    LlmGeneration & out_;
    std::string held_;
};

struct LlmOptions {
    int32_t n_ctx = 4096, n_batch = 512;
    int32_t queue_depth = 4;       // decode steps kept queued on the GPU in greedy generation
    CudaOptions cuda;
};

class Llm {
public:
    //   NotFound / Unsupported / InvalidArgument  as load_native_llama, plus the vocabulary's
    static Result<std::unique_ptr<Llm>> load(const std::string & path, const LlmOptions & options = LlmOptions());
    int32_t vocab_size() const { return vocab_.size(); }
    int32_t context_size() const { return decoder_->config().n_ctx; }
    const Vocab & vocab() const { return vocab_; }
    CudaLlamaDecoder & decoder() { return *decoder_; }
    Result<std::vector<int32_t>> tokenize(const std::string & text, bool add_special = true) const { return vocab_.tokenize(text, add_special); }
    // Every call is a fresh conversation (llm_pipeline.h:72-75).   InvalidArgument  empty prompt, max_new_tokens outside [1, n_ctx), an empty stop string,
    // a bad sampler     ResourceExhausted  prompt + max_new_tokens exceed the context
    Result<LlmGeneration> generate(const std::string & prompt, const LlmGenerateOptions & options = LlmGenerateOptions(),
                                   const std::function<bool(const std::string &)> & on_text = nullptr, LlmTimings * timings = nullptr);
    Result<LlmGeneration> generate_tokens(const std::vector<int32_t> & prompt, const LlmGenerateOptions & options = LlmGenerateOptions(),
                                          const std::function<bool(const std::string &)> & on_text = nullptr, LlmTimings * timings = nullptr);
    // A conversation, formatted with the file's chat template and tokenized with its special tokens parsed and no BOS added: the template's text carries
    // what it needs (llm_pipeline.h:60-71, llm_pipeline.cpp:233-247).   Unsupported  no template, or an unknown family; otherwise as generate
    bool has_chat_template() const { return vocab_.has_chat_template(); }
    Result<std::vector<int32_t>> chat_tokens(const std::vector<ChatMessage> & messages) const;
    Result<LlmGeneration> chat(const std::vector<ChatMessage> & messages, const LlmGenerateOptions & options = LlmGenerateOptions(),
                               const std::function<bool(const std::string &)> & on_text = nullptr, LlmTimings * timings = nullptr);

    // The text side of a vision-language pipeline (generate_native, src/pipeline/vlm_pipeline.cpp:177-212): the whole prompt as ONE embedding sequence -
    // the rows of the tokens before the image, the image's embedding rows as the vision model produced them (image_rows x n_embd floats), the rows of the
    // tokens after it - through eval_embeddings, then greedy decoding with steps queued on the GPU.
    //   InvalidArgument  no rows at all, non-finite embeddings, max_new_tokens outside [1, n_ctx)     ResourceExhausted  the context
    Result<LlmGeneration> generate_from_embeddings(const std::vector<int32_t> & before, const float * image, int32_t image_rows, const std::vector<int32_t> & after,
                                                   int32_t max_new_tokens, const std::function<bool(const std::string &)> & on_text = nullptr, LlmTimings * timings = nullptr);

private:
    Llm(std::unique_ptr<CudaLlamaDecoder> d, Vocab v, int32_t depth) : decoder_(std::move(d)), vocab_(std::move(v)), depth_(depth) {}
    std::unique_ptr<CudaLlamaDecoder> decoder_;
    Vocab vocab_;
    int32_t depth_;
};

}  // namespace dooms
