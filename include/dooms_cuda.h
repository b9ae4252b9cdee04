#ifndef DOOMS_CUDA_H
#define DOOMS_CUDA_H
/* C ABI of the CUDA (sm_100a) backend for the llama / qwen2 GGUF decoder.
 *
 * This is the boundary a dooms.cpp build binds instead of its Metal decoder: the entry points below carry the method set of
 * dooms::MetalLlamaDecoder (src/backend/metal/metal_llama_decoder.h:63-106) and of load_native_llama (src/pipeline/native_llama.h:15-23) over plain
 * pointers and sizes. No C++, CUDA or torch type appears in a signature.
 *
 *  - Every function returns a dooms_code (the reference's values, include/dooms/dooms_c.h:23-32); DOOMS_OK is 0. On failure
 *    dooms_cuda_last_error() returns a message for the calling thread, valid until that thread's next call.
 *  - Handles are not thread-safe: one caller at a time per handle (metal_llama_decoder.h:61-62).
 *  - Weight pointers are HOST memory (for example a mapped GGUF file). They are copied to device memory at creation and never referenced afterwards
 *    (src/backend/weight_ref.h:9). Quantized blocks are uploaded byte for byte.
 *  - There is no CPU fallback: without a CUDA device every entry point that computes fails with DOOMS_UNSUPPORTED.
 *  - Structs start with struct_size (set it to sizeof(the struct)); zero is rejected (src/api/c_api.cpp:96-102).
 */
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DOOMS_CUDA_API __attribute__((visibility("default")))

typedef enum dooms_code {
    DOOMS_OK = 0,
    DOOMS_INVALID_ARGUMENT = 1,
    DOOMS_NOT_FOUND = 2,
    DOOMS_DATA_LOSS = 3,
    DOOMS_UNSUPPORTED = 4,
    DOOMS_RESOURCE_EXHAUSTED = 5,
    DOOMS_IO_ERROR = 6,
    DOOMS_INTERNAL = 7
} dooms_code;

/* Element types, numbered like dooms::DType (src/core/dtype.h:15). The quantized ones are ggml block formats (src/core/dtype.cpp:17-29). */
typedef enum dooms_dtype {
    DOOMS_F32 = 0, DOOMS_F16 = 1, DOOMS_BF16 = 2, DOOMS_I32 = 3,
    DOOMS_Q4_0 = 4, DOOMS_Q5_0 = 5, DOOMS_Q8_0 = 6, DOOMS_Q4_K = 7, DOOMS_Q6_K = 8
} dooms_dtype;

/* dooms::WeightRef (src/backend/weight_ref.h:11-15): a row-major [rows][cols] host tensor, cols = input width; vectors have rows = 1. */
typedef struct dooms_weight_ref {
    const void * data;
    int32_t dtype;       /* a dooms_dtype */
    int64_t rows, cols;
} dooms_weight_ref;

/* dooms::LlamaDecoderConfig (metal_llama_decoder.h:20-39). */
typedef struct dooms_llama_config {
    size_t struct_size;
    int32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab;
    float rope_base;
    int32_t rope_neox;      /* 0: adjacent rotary pairs (llama); 1: split halves (qwen2) */
    float rms_eps;
    int32_t n_ctx;          /* positions the KV cache holds */
    int32_t n_batch;        /* largest prefill chunk */
    int32_t spin_wait;      /* generate(): poll for each token instead of sleeping */
    int32_t prefill_tile;   /* 0: automatic; 1: the CUDA-core tile kernel; 2: the tcgen05 tensor-core kernel (when the widths allow) */
} dooms_llama_config;

/* dooms::LlamaLayerWeights (metal_llama_decoder.h:42-51). Unused refs have data == NULL. */
typedef struct dooms_llama_layer_weights {
    dooms_weight_ref attn_norm;
    dooms_weight_ref attn_q, attn_k, attn_v, attn_qkv;
    dooms_weight_ref attn_q_bias, attn_k_bias, attn_v_bias, attn_qkv_bias;
    dooms_weight_ref attn_output;
    dooms_weight_ref ffn_norm;
    dooms_weight_ref ffn_gate, ffn_up, ffn_down;
} dooms_llama_layer_weights;

/* dooms::LlamaDecoderWeights (metal_llama_decoder.h:53-58). output.data == token_embd.data means tied. */
typedef struct dooms_llama_weights {
    size_t struct_size;
    dooms_weight_ref token_embd, output_norm, output;
    const dooms_llama_layer_weights * layers;
    int32_t n_layers;
} dooms_llama_weights;

/* Placement; no counterpart in the reference (it has one GPU and no distributed code). */
typedef struct dooms_cuda_options {
    size_t struct_size;
    int32_t device;          /* CUDA device ordinal of this process */
    int32_t tp_rank;         /* tensor-parallel rank and degree; 0 / 1 for one GPU */
    int32_t tp_size;
    const void * nccl_unique_id;   /* tp_size > 1: the 128-byte ncclUniqueId every rank of the group passes (rank 0 makes it with dooms_cuda_nccl_unique_id) */
    const char * nccl_library;     /* path of libnccl.so.2 to load; NULL: the dynamic loader's search path */
    int32_t operand_bf16;    /* prefill tensor-core operands: 0 = f16 (the reference's rounding, llama_kernels.h:197); 1 (bf16) is refused: DOOMS_UNSUPPORTED */
    int32_t use_graphs;      /* 1: decode steps replay a CUDA graph; 0: plain launches */
    int32_t max_sequences;   /* independent KV caches ("slots") of n_ctx positions each; 0 or 1: one sequence, as the reference's class. Read only when
                              * struct_size covers it. */
} dooms_cuda_options;

/* dooms::NativeLlamaOptions (src/pipeline/native_llama.h:15-20). */
typedef struct dooms_native_llama_options {
    size_t struct_size;
    int32_t n_ctx, n_batch, spin_wait, prefill_tile;
} dooms_native_llama_options;

/* MetalLlamaDecoder::KernelTime (metal_llama_decoder.h:99). `kind` points at a string literal. */
typedef struct dooms_kernel_time {
    const char * kind;
    int32_t dispatches;
    double gpu_ms;
} dooms_kernel_time;

typedef struct dooms_cuda_llama dooms_cuda_llama;

DOOMS_CUDA_API const char * dooms_cuda_last_error(void);
DOOMS_CUDA_API const char * dooms_cuda_code_name(int32_t code);                  /* code_name, src/core/status.h:25 */
DOOMS_CUDA_API int32_t dooms_cuda_device_count(void);                            /* 0 without a usable CUDA device */

/* Block tables: dtype_block_elems / dtype_block_bytes / dtype_bytes (src/core/dtype.cpp:45-52). */
DOOMS_CUDA_API int64_t dooms_dtype_block_elems(int32_t dtype);
DOOMS_CUDA_API int64_t dooms_dtype_block_bytes(int32_t dtype);
DOOMS_CUDA_API int32_t dooms_dtype_bytes(int32_t dtype, int64_t n, uint64_t * out);
DOOMS_CUDA_API const char * dooms_dtype_name(int32_t dtype);

/* ---- GGUF reader: GgufFile (src/format/gguf.h:63-100, src/format/gguf.cpp:179-317). Host only. ---- */
typedef struct dooms_gguf dooms_gguf;
typedef struct dooms_gguf_tensor {
    const char * name;       /* owned by the file handle */
    int32_t dtype;
    int32_t rank;
    int64_t shape[4];        /* row-major, outermost first (the file stores the reverse) */
    uint64_t offset;         /* from the start of the file */
    uint64_t nbytes;
    const void * data;       /* inside the mapping; valid while the handle lives */
} dooms_gguf_tensor;
DOOMS_CUDA_API int32_t dooms_gguf_open(const char * path, dooms_gguf ** out);                         /* GgufFile::open */
DOOMS_CUDA_API int32_t dooms_gguf_parse(const void * data, size_t size, dooms_gguf ** out);            /* GgufFile::parse; data must outlive the handle */
DOOMS_CUDA_API void dooms_gguf_close(dooms_gguf * f);
DOOMS_CUDA_API uint32_t dooms_gguf_version(const dooms_gguf * f);
DOOMS_CUDA_API uint64_t dooms_gguf_alignment(const dooms_gguf * f);
DOOMS_CUDA_API int64_t dooms_gguf_tensor_count(const dooms_gguf * f);
DOOMS_CUDA_API int32_t dooms_gguf_tensor_at(const dooms_gguf * f, int64_t index, dooms_gguf_tensor * out);
DOOMS_CUDA_API int32_t dooms_gguf_find_tensor(const dooms_gguf * f, const char * name, dooms_gguf_tensor * out);   /* find_tensor + tensor_data */
DOOMS_CUDA_API int32_t dooms_gguf_get_string(const dooms_gguf * f, const char * key, const char ** out);
DOOMS_CUDA_API int32_t dooms_gguf_get_uint(const dooms_gguf * f, const char * key, uint64_t * out);
DOOMS_CUDA_API int32_t dooms_gguf_get_int(const dooms_gguf * f, const char * key, int64_t * out);
DOOMS_CUDA_API int32_t dooms_gguf_get_float(const dooms_gguf * f, const char * key, double * out);
DOOMS_CUDA_API int32_t dooms_gguf_get_bool(const dooms_gguf * f, const char * key, int32_t * out);

/* ---- The decoder: MetalLlamaDecoder's methods (metal_llama_decoder.h:63-106). ---- */
/* create (metal_llama_decoder.mm:425-689). options may be NULL (device 0, one GPU, f16 operands, graphs on). */
DOOMS_CUDA_API int32_t dooms_cuda_llama_create(const dooms_llama_config * config, const dooms_llama_weights * weights, const dooms_cuda_options * options,
                                               dooms_cuda_llama ** out);
/* load_native_llama (src/pipeline/native_llama.cpp:9-102): GGUF metadata -> config, tensor names -> weights, then create. */
DOOMS_CUDA_API int32_t dooms_cuda_llama_load(const char * gguf_path, const dooms_native_llama_options * options, const dooms_cuda_options * cuda_options,
                                             dooms_cuda_llama ** out);
DOOMS_CUDA_API void dooms_cuda_llama_destroy(dooms_cuda_llama * d);
DOOMS_CUDA_API int32_t dooms_cuda_llama_config(const dooms_cuda_llama * d, dooms_llama_config * out);   /* config() */
DOOMS_CUDA_API int32_t dooms_cuda_llama_position(const dooms_cuda_llama * d);                            /* position() */
DOOMS_CUDA_API int32_t dooms_cuda_llama_reset(dooms_cuda_llama * d);                                     /* reset(), .mm:691-695 */
DOOMS_CUDA_API int32_t dooms_cuda_llama_eval_tokens(dooms_cuda_llama * d, const int32_t * tokens, int32_t n);        /* .mm:712-724 */
DOOMS_CUDA_API int32_t dooms_cuda_llama_eval_embeddings(dooms_cuda_llama * d, const float * embeddings, int32_t n);  /* .mm:697-710 */
/* Rows of the embedding table as f32 (n x n_embd floats into out, host memory), dequantized on the device (embedq<Q>, llama_kernels.h:1289-1296): what a
 * caller that mixes token rows with rows of its own hands to eval_embeddings (vocab.embed_tokens in src/pipeline/vlm_pipeline.cpp:180-181). */
DOOMS_CUDA_API int32_t dooms_cuda_llama_embed_tokens(dooms_cuda_llama * d, const int32_t * tokens, int32_t n, float * out);
DOOMS_CUDA_API int32_t dooms_cuda_llama_pending_token(dooms_cuda_llama * d, int32_t * out);                           /* .mm:726-731 */
/* logits() (.mm:733-739): n_vocab floats of the last evaluated position into out (capacity floats; too small: DOOMS_RESOURCE_EXHAUSTED). */
DOOMS_CUDA_API int32_t dooms_cuda_llama_logits(dooms_cuda_llama * d, float * out, int64_t capacity);
/* generate() (.mm:741-787). callback returns non-zero to continue, zero to stop (the reference's `bool on_token(int32_t)`). */
typedef int32_t (*dooms_token_callback)(int32_t token, void * user);
DOOMS_CUDA_API int32_t dooms_cuda_llama_generate(dooms_cuda_llama * d, int32_t max_tokens, int32_t depth, dooms_token_callback callback, void * user);
/* profile_pass() (.mm:789-812): per-kind device time of one forward pass over `rows` positions; *count receives the number of entries written. */
DOOMS_CUDA_API int32_t dooms_cuda_llama_profile_pass(dooms_cuda_llama * d, int32_t rows, dooms_kernel_time * out, int32_t capacity, int32_t * count);

/* Measurement helpers without a counterpart in the reference's class: device time (CUDA events on the decoder's stream) of the last eval_* call and of
 * the last generate() call, and the number of kernels those calls launched. */
typedef struct dooms_cuda_timings {
    size_t struct_size;
    double last_eval_ms;         /* device time of the last eval_tokens / eval_embeddings call, all chunks */
    double last_generate_ms;     /* device time from the first queued decode step to the last delivered token */
    int64_t last_eval_launches;
    int64_t last_generate_launches;
    int64_t weight_bytes;        /* bytes of weight matrices resident on this GPU */
    int64_t kv_bytes;            /* bytes of the KV cache on this GPU */
    double last_batch_ms;        /* device time of the steps of the last dooms_cuda_llama_decode_batch call (written only when struct_size covers it) */
    int64_t last_batch_launches;
    int64_t tp_peer_allreduce;   /* 1: the tensor-parallel decode steps reduce over peer memory; 0: NCCL's all-reduce, or one GPU */
    int64_t tp_symmetric_window; /* 1: the buffers NCCL reduces are NCCL's own memory registered as a symmetric window (NCCL 2.27+); 0: plain device memory */
} dooms_cuda_timings;
DOOMS_CUDA_API int32_t dooms_cuda_llama_timings(const dooms_cuda_llama * d, dooms_cuda_timings * out);

/* ---- Several sequences on one decoder. No counterpart in the reference, which serves one request at a time (python/dooms/server.py:262-269); this is
 * the batched decode step the many-sequence serving load needs: one pass over the weights per step for all sequences of the batch. ----
 * A decoder created with max_sequences = S holds S KV-cache slots. Every call above acts on the selected slot (0 at creation); logits are kept for the
 * last evaluation only. */
DOOMS_CUDA_API int32_t dooms_cuda_llama_max_sequences(const dooms_cuda_llama * d);
DOOMS_CUDA_API int32_t dooms_cuda_llama_max_batch_rows(const dooms_cuda_llama * d);   /* rows one batched step can hold; 0: decode_batch is unsupported here */
DOOMS_CUDA_API int32_t dooms_cuda_llama_select_sequence(dooms_cuda_llama * d, int32_t slot);
/* `steps` greedy decode steps for the n listed slots at once (slots[i] < 0: an idle row). Every listed slot needs a pending token, as for generate.
 * out_tokens[t * n + i] = the token step t produced for slots[i] (-1 for idle rows). Afterwards each slot's position has advanced by `steps` and its pending
 * token is the last one produced. DOOMS_UNSUPPORTED when max_batch_rows is 0; DOOMS_INVALID_ARGUMENT for a bad / repeated slot, a slot without pending
 * token or steps outside [1, 256]; DOOMS_RESOURCE_EXHAUSTED when a slot's context or the step's rows would overflow. */
DOOMS_CUDA_API int32_t dooms_cuda_llama_decode_batch(dooms_cuda_llama * d, const int32_t * slots, int32_t n, int32_t steps, int32_t * out_tokens);

/* ---- Single kernels on DEVICE pointers, for parity tests and roofline measurement. `stream` is a cudaStream_t (NULL: the default stream). ---- */
/* dequant_half<Q> / Q::elem (llama_kernels.h:1012-1154, 1474-1480): rows x cols blocks -> f32 values, bit for bit the block formulas. */
DOOMS_CUDA_API int32_t dooms_cuda_dequantize(int32_t dtype, const void * d_blocks, int64_t rows, int64_t cols, float * d_out, void * stream);
/* matvec1q<Q> (llama_kernels.h:1197-1230): y[r] (+)= W[r] . x (+ bias[r]). flags: 2 accumulate into y, 4 add bias (MatvecParams flags, .mm:51). */
DOOMS_CUDA_API int32_t dooms_cuda_matvec(int32_t dtype, const void * d_w, const float * d_x, float * d_y, const float * d_bias, int64_t rows, int64_t cols,
                                         uint32_t flags, void * stream);
/* gate_up1q<Q> (llama_kernels.h:1232-1269): h[r] = silu(Wg[r] . x) * (Wu[r] . x). */
DOOMS_CUDA_API int32_t dooms_cuda_gate_up(int32_t dtype, const void * d_wg, const void * d_wu, const float * d_x, float * d_h, int64_t rows, int64_t cols,
                                          void * stream);
/* No counterpart in the reference. The q4_0 / q4_K kernel behind dooms_cuda_matvec / _gate_up multiplies int8 digits on the tensor cores: it works on the
 * input vector split per 32-element block into a power-of-two scale and four base-128 digits. Given an f32 input it makes that split in its prologue; inside
 * a decode step the kernel that produced the vector leaves it already split. These entry points are that second form: dooms_cuda_split_input writes the
 * split of d_x (cols floats) into d_split (dooms_cuda_split_input_bytes(cols) bytes of device memory), dooms_cuda_matvec_split is dooms_cuda_matvec on
 * it (with d_w2: dooms_cuda_gate_up). Results are bit for bit those of the f32 entry points. DOOMS_UNSUPPORTED for other types or shapes. */
DOOMS_CUDA_API int64_t dooms_cuda_split_input_bytes(int64_t cols);
DOOMS_CUDA_API int32_t dooms_cuda_split_input(const float * d_x, int64_t cols, void * d_split, void * stream);
DOOMS_CUDA_API int32_t dooms_cuda_matvec_split(int32_t dtype, const void * d_w, const void * d_w2, const void * d_split, float * d_y, const float * d_bias, int64_t rows,
                                               int64_t cols, uint32_t flags, void * stream);
/* matmul_bigq<Q> / matmul_gate_up_bigq<Q> (llama_kernels.h:1320-1382) on the tcgen05 tensor cores: Y[t][r] (+)= sum_k X[t][k] W[r][k] (+ bias[r]) for
 * `tokens` rows of X, an f16 [tokens][cols] device buffer (cols a multiple of 64; operands are rounded to f16 as the reference's tiles, llama_kernels.h:197).
 * With d_w2: Y[t][r] = silu(X[t] . W[r]) * (X[t] . W2[r]). Y is f32 [tokens][rows]. flags as dooms_cuda_matvec. */
DOOMS_CUDA_API int32_t dooms_cuda_matmul(int32_t dtype, const void * d_w, const void * d_w2, const void * d_x16, float * d_y, const float * d_bias,
                                         int32_t tokens, int64_t rows, int64_t cols, uint32_t flags, void * stream);
/* No counterpart in the reference (Metal command buffers report their own errors). The matvec / gate_up / matmul kernels above wait for their tensor copies
 * and tensor-core stages with a limit; a wait that runs out sets a process-wide error word instead of hanging the GPU, and the kernel's output is then
 * not valid. This call waits for `stream`, reads the word into *flag (may be NULL; 0: none, 2: matmul, 4: matvec / gate_up) and clears it; it returns
 * DOOMS_OK when the word was 0 and DOOMS_INTERNAL otherwise. */
DOOMS_CUDA_API int32_t dooms_cuda_kernel_status(void * stream, int32_t * flag);
/* norm_vec (llama_kernels.h:1272-1286): xn = x * rsqrt(mean(x^2) + eps) * gamma for `rows` rows of `cols`. */
DOOMS_CUDA_API int32_t dooms_cuda_rms_norm(const float * d_x, const float * d_gamma, float * d_out, int64_t rows, int64_t cols, float eps, void * stream);
/* argmax (llama_kernels.h:949-975) with the host rule that NaN never wins (src/core/argmax.h:15-16): *d_out = lowest index of the maximum. */
DOOMS_CUDA_API int32_t dooms_cuda_argmax(const float * d_logits, int64_t n, int32_t * d_out, void * stream);
/* No counterpart in the reference. The same reduction as dooms_cuda_argmax for callers that must not allocate device memory: code running where a
 * cudaMalloc is forbidden or would stall (inside a latency-critical serving loop that has handed all free device memory to a KV-cache pool, or a host
 * runtime that pre-plans its memory and treats any later allocation as a fault). Its partial results live in a fixed array inside the library's device
 * image (2 KB per GPU that loads the library, held until the process exits), which limits n to DOOMS_CUDA_ARGMAX_NOALLOC_MAX logits; larger n is refused
 * with DOOMS_INVALID_ARGUMENT. The first call on each device looks up the array's device address (no allocation, but a driver call): make that first
 * call before starting any stream capture. All calls on a device share the array: two calls that overlap on the GPU (different streams) race. */
#define DOOMS_CUDA_ARGMAX_NOALLOC_MAX 1048576
DOOMS_CUDA_API int32_t dooms_cuda_argmax_noalloc(const float * d_logits, int64_t n, int32_t * d_out, void * stream);
/* attention_split + attention_combine (llama_kernels.h:860-929): one query token, n_keys cached positions, grouped-query heads. q f32 [n_head][head_dim]
 * (already rotated), kc / vc f16 [n_keys][n_head_kv*head_dim], out f32 [n_head][head_dim]. d_scratch: dooms_cuda_attention_scratch_bytes(...) bytes. */
DOOMS_CUDA_API int64_t dooms_cuda_attention_scratch_bytes(int32_t n_head, int32_t head_dim, int32_t n_keys);
DOOMS_CUDA_API int32_t dooms_cuda_attention_decode(const float * d_q, const void * d_kc, const void * d_vc, float * d_out, void * d_scratch, int32_t n_head,
                                                   int32_t n_head_kv, int32_t head_dim, int32_t n_keys, void * stream);

/* ---- A text language model on the decoder: the `Llm` surface of the reference (src/pipeline/llm_pipeline.h:16-82) and its C face dooms_llm_*
 * (include/dooms/dooms_c.h:73-138, src/api/c_api.cpp:322-504) for the decoder's own engine. Vocabulary, byte-level BPE tokenizer and sampler are this
 * library's (the reference takes them from llama.cpp); chat templates are not evaluated. ---- */
typedef struct dooms_cuda_llm dooms_cuda_llm;
typedef struct dooms_cuda_vocab dooms_cuda_vocab;
typedef struct dooms_cuda_llm_options {     /* dooms_llm_options (dooms_c.h:75-81) */
    size_t struct_size;
    int32_t n_ctx;          /* positions of the KV cache (prompt + answer); 0: 4096 */
    int32_t n_batch;        /* largest prefill chunk; 0: 512 */
    int32_t queue_depth;    /* decode steps kept queued on the GPU in greedy generation; 0: 4 */
    int32_t device;         /* CUDA device ordinal */
} dooms_cuda_llm_options;
typedef struct dooms_cuda_sampling {        /* dooms_llm_sampling (dooms_c.h:85-92); NULL wherever one is taken: greedy */
    size_t struct_size;
    float temperature;
    int32_t top_k;
    float top_p;
    float repeat_penalty;
    uint32_t seed;
} dooms_cuda_sampling;
typedef int32_t (*dooms_cuda_text_callback)(const char * piece, void * user);   /* returns 0 to continue, non-zero to stop (dooms_text_callback, dooms_c.h:69) */
enum { DOOMS_CUDA_FINISH_NONE = 0, DOOMS_CUDA_FINISH_STOP = 1, DOOMS_CUDA_FINISH_LENGTH = 2, DOOMS_CUDA_FINISH_CANCELLED = 3 };   /* dooms_finish_reason, dooms_c.h:118-123 */
typedef struct dooms_cuda_generation_info { /* dooms_llm_generation_info (dooms_c.h:125-130) plus LlmTimings (llm_pipeline.h:34-40) */
    size_t struct_size;
    int32_t prompt_tokens, completion_tokens, finish_reason;
    double prefill_ms, first_token_ms, decode_ms;
} dooms_cuda_generation_info;

DOOMS_CUDA_API int32_t dooms_cuda_llm_open(const char * gguf_path, const dooms_cuda_llm_options * options, dooms_cuda_llm ** out);   /* dooms_llm_open */
DOOMS_CUDA_API void dooms_cuda_llm_close(dooms_cuda_llm * llm);
DOOMS_CUDA_API int32_t dooms_cuda_llm_context_size(const dooms_cuda_llm * llm);
/* dooms_llm_generate (dooms_c.h:103-107): the answer as a NUL-terminated UTF-8 string; *needed (optional) its length including the NUL; a smaller
 * capacity writes nothing and returns DOOMS_RESOURCE_EXHAUSTED. Every call starts a fresh conversation. */
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate(dooms_cuda_llm * llm, const char * prompt, int32_t max_new_tokens, const dooms_cuda_sampling * sampling,
                                               const char * const * stop, int32_t n_stop, char * out, size_t capacity, size_t * needed);
/* dooms_llm_generate_stream (dooms_c.h:108-110). */
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_stream(dooms_cuda_llm * llm, const char * prompt, int32_t max_new_tokens, const dooms_cuda_sampling * sampling,
                                                      const char * const * stop, int32_t n_stop, dooms_cuda_text_callback callback, void * user);
/* The same from token ids (files whose vocabulary this library does not tokenize, and tests). out_tokens (optional, token_capacity ids) receives the
 * generated ids, *n_tokens their number. */
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_tokens(dooms_cuda_llm * llm, const int32_t * prompt, int32_t n_prompt, int32_t max_new_tokens,
                                                      const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, char * out, size_t capacity,
                                                      size_t * needed, int32_t * out_tokens, int32_t token_capacity, int32_t * n_tokens);
/* The text side of the reference's vision-language pipeline (generate_native, src/pipeline/vlm_pipeline.cpp:177-212): the prompt as one embedding sequence
 * (rows of the tokens `before`, then image_rows x n_embd floats of image embeddings as given, then the rows of the tokens `after`) through
 * eval_embeddings, then greedy decoding. callback optional (as dooms_cuda_llm_generate_stream); the whole answer in out as dooms_cuda_llm_generate. */
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_from_embeddings(dooms_cuda_llm * llm, const int32_t * before, int32_t n_before, const float * image, int32_t image_rows,
                                                               const int32_t * after, int32_t n_after, int32_t max_new_tokens, dooms_cuda_text_callback callback,
                                                               void * user, char * out, size_t capacity, size_t * needed);
/* A conversation (dooms_chat_message, dooms_c.h:94-97), formatted with the file's chat template: dooms_llm_chat / dooms_llm_chat_stream /
 * dooms_llm_count_chat_tokens (dooms_c.h:111-116, 137-138). The template is recognised by the markers it contains, as the llama.cpp call the reference
 * makes does (src/models/vlm/text_decoder.cpp:268-277): ChatML, Llama 3 and SmolVLM are written; no template or another family: DOOMS_UNSUPPORTED. The
 * template's text is tokenized with its special tokens parsed and no BOS added (src/pipeline/llm_pipeline.cpp:233-238). */
typedef struct dooms_cuda_chat_message {
    const char * role;      /* "system", "user", "assistant" */
    const char * content;
} dooms_cuda_chat_message;
DOOMS_CUDA_API int32_t dooms_cuda_llm_chat(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t max_new_tokens,
                                           const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, char * out, size_t capacity, size_t * needed);
DOOMS_CUDA_API int32_t dooms_cuda_llm_chat_stream(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t max_new_tokens,
                                                  const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, dooms_cuda_text_callback callback,
                                                  void * user);
DOOMS_CUDA_API int32_t dooms_cuda_llm_count_chat_tokens(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t * count);
DOOMS_CUDA_API int32_t dooms_cuda_llm_last_generation(const dooms_cuda_llm * llm, dooms_cuda_generation_info * out);                 /* dooms_llm_last_generation */
DOOMS_CUDA_API int32_t dooms_cuda_llm_count_tokens(dooms_cuda_llm * llm, const char * text, int32_t add_special, int32_t * count);   /* dooms_llm_count_tokens */

/* The host-side pieces on their own (no GPU): the vocabulary of a GGUF file, the text assembly that turns a token stream into complete UTF-8 pieces with
 * stop strings (TokenSink, src/pipeline/llm_pipeline.cpp:91-135), and the sampler. */
DOOMS_CUDA_API int32_t dooms_cuda_vocab_open(const char * gguf_path, dooms_cuda_vocab ** out);
DOOMS_CUDA_API void dooms_cuda_vocab_close(dooms_cuda_vocab * vocab);
DOOMS_CUDA_API int32_t dooms_cuda_vocab_size(const dooms_cuda_vocab * vocab);
DOOMS_CUDA_API int32_t dooms_cuda_vocab_is_end_of_generation(const dooms_cuda_vocab * vocab, int32_t token);
/* The bytes a token stands for (not NUL-terminated: a piece may hold any byte); *n their number; capacity too small: DOOMS_RESOURCE_EXHAUSTED. */
DOOMS_CUDA_API int32_t dooms_cuda_vocab_piece(const dooms_cuda_vocab * vocab, int32_t token, char * out, int32_t capacity, int32_t * n);
DOOMS_CUDA_API int32_t dooms_cuda_vocab_tokenize(const dooms_cuda_vocab * vocab, const char * text, int32_t add_special, int32_t * out, int32_t capacity, int32_t * n);
/* The same with parse_special: the text of a control token inside `text` becomes that token's id (TextDecoder::tokenize's parse_special, text_decoder.h:51-53). */
DOOMS_CUDA_API int32_t dooms_cuda_vocab_tokenize_special(const dooms_cuda_vocab * vocab, const char * text, int32_t add_special, int32_t parse_special, int32_t * out,
                                                         int32_t capacity, int32_t * n);
/* TextDecoder::apply_chat_template (text_decoder.cpp:257-278): the conversation as the template's family writes it; the text as dooms_cuda_llm_generate returns one. */
DOOMS_CUDA_API int32_t dooms_cuda_vocab_apply_chat_template(const dooms_cuda_vocab * vocab, const dooms_cuda_chat_message * messages, int32_t n_messages,
                                                            int32_t add_generation_prompt, char * out, size_t capacity, size_t * needed);
/* Runs the text assembly over `tokens`: pieces go to `callback` (optional); *consumed = tokens taken before generation ended, *finish_reason how it ended
 * (DOOMS_CUDA_FINISH_LENGTH: the tokens ran out); the whole text as dooms_cuda_llm_generate returns it. */
DOOMS_CUDA_API int32_t dooms_cuda_text_stream(const dooms_cuda_vocab * vocab, const int32_t * tokens, int32_t n_tokens, const char * const * stop, int32_t n_stop,
                                              dooms_cuda_text_callback callback, void * user, char * out, size_t capacity, size_t * needed, int32_t * consumed,
                                              int32_t * finish_reason);
/* `draws` tokens drawn one after another from the same row of n logits (each draw joins the repetition-penalty history). */
DOOMS_CUDA_API int32_t dooms_cuda_sample(const float * logits, int32_t n, const dooms_cuda_sampling * sampling, int32_t draws, int32_t * out_tokens);

/* This rank's share of the model under tensor parallelism (no counterpart in the reference): rows [q_row0, q_row0 + q_rows) of attn_q and the same
 * columns of attn_output, rows [kv_row0, ..) of attn_k / attn_v (whole heads; the KV cache holds only these heads), rows [ff_row0, ..) of ffn_gate /
 * ffn_up and the same columns of ffn_down, rows [vocab_row0, ..) of the output matrix. The partial sums of attn_output and ffn_down are all-reduced.
 * Column shards are whole quantization blocks: the feed-forward width is dealt in units of ffn_block columns (the first n_ff / ffn_block % tp_size ranks
 * take one unit more), and of attn_output a rank holds the blocks [attn_col0, attn_col0 + attn_cols) that cover its heads' columns, multiplied with an
 * input that is zero outside them (a block on a boundary is held by both neighbours). dooms_cuda_tp_share is the case of both block sizes 1; a decoder
 * uses the largest block size among its layers' attn_output and ffn_down types (dooms_dtype_block_elems).
 * Host only. DOOMS_UNSUPPORTED when the heads do not divide by tp_size, or n_ff is not at least tp_size whole blocks. */
typedef struct dooms_tp_share {
    size_t struct_size;
    int64_t q_row0, q_rows, kv_row0, kv_rows, ff_row0, ff_rows, vocab_row0, vocab_rows;
    int64_t attn_col0, attn_cols;      /* written when struct_size covers them */
} dooms_tp_share;
DOOMS_CUDA_API int32_t dooms_cuda_tp_share(const dooms_llama_config * config, int32_t tp_rank, int32_t tp_size, dooms_tp_share * out);
DOOMS_CUDA_API int32_t dooms_cuda_tp_share_blocks(const dooms_llama_config * config, int32_t tp_rank, int32_t tp_size, int64_t attn_block, int64_t ffn_block,
                                                  dooms_tp_share * out);

/* Tensor-parallel set-up helper: fills 128 bytes with a fresh ncclUniqueId (rank 0 calls it and sends the bytes to the other ranks). */
DOOMS_CUDA_API int32_t dooms_cuda_nccl_unique_id(const char * nccl_library, void * out128);

#ifdef __cplusplus
}
#endif
#endif
