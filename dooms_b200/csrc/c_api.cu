// The C ABI of include/dooms_cuda.h over the C++ decoder, the GGUF reader and the single-kernel launchers.
#include "dooms_cuda.h"

#include <cuda_runtime.h>

#include <cstddef>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "cuda_llama_decoder.h"
#include "gguf.h"
#include "llm_pipeline.h"
#include "kernels/kernels.h"
#include "nccl_dyn.h"

using namespace dooms;

struct dooms_cuda_llama { std::unique_ptr<CudaLlamaDecoder> dec; };
struct dooms_gguf { std::unique_ptr<GgufFile> file; };
struct dooms_cuda_vocab { Vocab vocab; };
struct dooms_cuda_llm {
    std::unique_ptr<Llm> llm;
    dooms_cuda_generation_info last{};
};

namespace {

thread_local std::string g_last_error;

// dooms::Code -> the C numbering (the reference's src/api/c_api.cpp:36-47: OutOfRange folds into InvalidArgument).
int32_t c_code(Code c) {
    switch (c) {
        case Code::Ok: return DOOMS_OK;
        case Code::InvalidArgument: case Code::OutOfRange: return DOOMS_INVALID_ARGUMENT;
        case Code::NotFound: return DOOMS_NOT_FOUND;
        case Code::DataLoss: return DOOMS_DATA_LOSS;
        case Code::Unsupported: return DOOMS_UNSUPPORTED;
        case Code::ResourceExhausted: return DOOMS_RESOURCE_EXHAUSTED;
        case Code::IoError: return DOOMS_IO_ERROR;
        case Code::Internal: return DOOMS_INTERNAL;
    }
    return DOOMS_INTERNAL;
}
int32_t fail(int32_t code, std::string message) { g_last_error = std::move(message); return code; }
int32_t done(const Status & st) {
    if (st.is_ok()) return DOOMS_OK;
    return fail(c_code(st.code()), st.message());
}
// struct_size lets a newer library accept an older caller's smaller struct; zero (an uninitialised caller) is rejected.
template <class T>
bool struct_ok(const T * p, const char * name, int32_t * code) {
    if (!p) { *code = fail(DOOMS_INVALID_ARGUMENT, std::string(name) + " is NULL"); return false; }
    if (p->struct_size < sizeof(size_t) * 2) { *code = fail(DOOMS_INVALID_ARGUMENT, std::string(name) + ".struct_size is not set"); return false; }
    return true;
}

bool ref_of(const dooms_weight_ref & r, WeightRef * out, std::string * err) {
    if (r.data && !dtype_valid(r.dtype)) { *err = "a weight has dtype " + std::to_string(r.dtype) + ", which is not a dooms_dtype"; return false; }
    out->data = r.data;
    out->dtype = r.data ? static_cast<DType>(r.dtype) : DType::F32;
    out->rows = r.rows;
    out->cols = r.cols;
    return true;
}

CudaOptions options_of(const dooms_cuda_options * o) {
    CudaOptions c;
    if (!o) return c;
    c.device = o->device;
    c.tp_rank = o->tp_rank;
    c.tp_size = o->tp_size < 1 ? 1 : o->tp_size;
    c.nccl_unique_id = o->nccl_unique_id;
    c.nccl_library = o->nccl_library;
    c.operand_bf16 = o->operand_bf16 != 0;
    c.use_graphs = o->use_graphs != 0;
    if (o->struct_size >= offsetof(dooms_cuda_options, max_sequences) + sizeof(int32_t)) c.max_sequences = o->max_sequences < 1 ? 1 : o->max_sequences;
    return c;
}

void fill_tensor(const GgufFile & f, const GgufTensorInfo & t, dooms_gguf_tensor * out) {
    out->name = t.name.c_str();
    out->dtype = static_cast<int32_t>(t.dtype);
    out->rank = t.rank;
    for (int d = 0; d < 4; d++) out->shape[d] = d < t.rank ? t.shape[d] : 0;
    out->offset = t.offset;
    out->nbytes = t.nbytes;
    out->data = f.tensor_data(t);
}

// Scratch of the single-kernel entry points that need some (argmax partial results): one small buffer per device, made on first use.
struct DeviceScratch { void * ptr = nullptr; size_t bytes = 0; };
std::mutex g_scratch_mutex;
DeviceScratch g_scratch[64];
Status scratch_for(size_t bytes, void ** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return unsupported("no CUDA device"); }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    DeviceScratch & s = g_scratch[dev];
    if (s.bytes < bytes) {
        if (s.ptr) cudaFree(s.ptr);
        s.ptr = nullptr;
        s.bytes = 0;
        if (cudaMalloc(&s.ptr, bytes) != cudaSuccess) { (void)cudaGetLastError(); return resource_exhausted("could not allocate kernel scratch memory"); }
        s.bytes = bytes;
    }
    *out = s.ptr;
    return Status();
}

// The error word of the single-kernel entry points: kernels with bounded waits (tensor copies, mbarriers) set it instead of waiting for ever. One word of
// mapped pinned host memory per process, never freed, read and cleared by dooms_cuda_kernel_status.
int32_t * kernel_error_word() {
    static int32_t * word = [] {
        int32_t * w = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&w), 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { (void)cudaGetLastError(); return static_cast<int32_t *>(nullptr); }
        *w = 0;
        return w;
    }();
    return word;
}

int32_t launch_result(cudaError_t e, const char * what) {
    if (e == cudaSuccess) return DOOMS_OK;
    (void)cudaGetLastError();
    if (e == cudaErrorInvalidValue) return fail(DOOMS_UNSUPPORTED, std::string(what) + ": a type or shape the kernel does not take");
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) return fail(DOOMS_UNSUPPORTED, std::string(what) + ": no CUDA device");
    return fail(DOOMS_INTERNAL, std::string(what) + ": " + cudaGetErrorString(e));
}

// The integer tensor-core GEMV on an f32 input. Up to 8192 columns every block splits the input for itself in its prologue: one launch, no scratch. Longer
// inputs are split once by a kernel into the per-device scratch (shared by every call on the device, so such calls must not overlap on different streams).
int32_t fast_q4_0(const void * w, const void * w2, const float * x, float * y, const float * bias, int64_t rows, int64_t cols, uint32_t flags, bool q4_k,
                  cudaStream_t st, const char * what) {
    int32_t * err = kernel_error_word();
    if (cols < 8192) return launch_result(cuda::launch_gemv_q4_0(w, w2, nullptr, x, nullptr, 0.f, y, bias, rows, cols, flags, q4_k, st, nullptr, nullptr, err), what);
    void * scratch = nullptr;
    const Status ss = scratch_for((cuda::quantized_x_bytes(cols) + 15) & ~size_t(15), &scratch);
    if (!ss.is_ok()) return done(ss);
    cudaError_t e = cuda::launch_quantize_x(x, cols, scratch, st);
    if (e == cudaSuccess) e = cuda::launch_gemv_q4_0(w, w2, scratch, nullptr, nullptr, 0.f, y, bias, rows, cols, flags, q4_k, st, nullptr, nullptr, err);
    return launch_result(e, what);
}

// Scratch of dooms_cuda_argmax_noalloc: the per-block partial results (8 bytes each) for up to DOOMS_CUDA_ARGMAX_NOALLOC_MAX logits. It is part of the
// library's device image, so no call ever allocates. In host code the name below is only a handle for cudaGetSymbolAddress, never a device address.
constexpr int kNoAllocParts = DOOMS_CUDA_ARGMAX_NOALLOC_MAX / 4096;
static __device__ __align__(256) unsigned long long g_argmax_noalloc_scratch[kNoAllocParts];
void * g_argmax_noalloc_ptr[64];      // the array's device address, per device, looked up on the first call there
std::mutex g_argmax_noalloc_mutex;

bool matrix_dtype(int32_t dt) { return dt == DOOMS_F16 || dt == DOOMS_Q4_0 || dt == DOOMS_Q5_0 || dt == DOOMS_Q8_0 || dt == DOOMS_Q4_K || dt == DOOMS_Q6_K; }

}  // namespace

extern "C" {

DOOMS_CUDA_API const char * dooms_cuda_last_error(void) { return g_last_error.c_str(); }

DOOMS_CUDA_API const char * dooms_cuda_code_name(int32_t code) {
    switch (code) {
        case DOOMS_OK: return "Ok";
        case DOOMS_INVALID_ARGUMENT: return "InvalidArgument";
        case DOOMS_NOT_FOUND: return "NotFound";
        case DOOMS_DATA_LOSS: return "DataLoss";
        case DOOMS_UNSUPPORTED: return "Unsupported";
        case DOOMS_RESOURCE_EXHAUSTED: return "ResourceExhausted";
        case DOOMS_IO_ERROR: return "IoError";
        case DOOMS_INTERNAL: return "Internal";
    }
    return "Unknown";
}

DOOMS_CUDA_API int32_t dooms_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
}

DOOMS_CUDA_API int64_t dooms_dtype_block_elems(int32_t dtype) { const DTypeInfo * i = dtype_info(dtype); return i ? i->block_elems : 0; }
DOOMS_CUDA_API int64_t dooms_dtype_block_bytes(int32_t dtype) { const DTypeInfo * i = dtype_info(dtype); return i ? i->block_bytes : 0; }
DOOMS_CUDA_API const char * dooms_dtype_name(int32_t dtype) { const DTypeInfo * i = dtype_info(dtype); return i ? i->name : "unknown"; }
DOOMS_CUDA_API int32_t dooms_dtype_bytes(int32_t dtype, int64_t n, uint64_t * out) {
    if (!dtype_valid(dtype) || !out) return fail(DOOMS_INVALID_ARGUMENT, "unknown dtype or NULL output");
    auto r = dtype_bytes(static_cast<DType>(dtype), n);
    if (!r.is_ok()) return done(r.status());
    *out = r.value();
    return DOOMS_OK;
}

// ---------------------------------------------------------------- GGUF

DOOMS_CUDA_API int32_t dooms_gguf_open(const char * path, dooms_gguf ** out) {
    if (!path || !out) return fail(DOOMS_INVALID_ARGUMENT, "path or out is NULL");
    auto r = GgufFile::open(path);
    if (!r.is_ok()) return done(r.status());
    *out = new dooms_gguf{std::make_unique<GgufFile>(std::move(r).value())};
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_parse(const void * data, size_t size, dooms_gguf ** out) {
    if (!out) return fail(DOOMS_INVALID_ARGUMENT, "out is NULL");
    auto r = GgufFile::parse(static_cast<const uint8_t *>(data), size);
    if (!r.is_ok()) return done(r.status());
    *out = new dooms_gguf{std::make_unique<GgufFile>(std::move(r).value())};
    return DOOMS_OK;
}
DOOMS_CUDA_API void dooms_gguf_close(dooms_gguf * f) { delete f; }
DOOMS_CUDA_API uint32_t dooms_gguf_version(const dooms_gguf * f) { return f ? f->file->version() : 0; }
DOOMS_CUDA_API uint64_t dooms_gguf_alignment(const dooms_gguf * f) { return f ? f->file->alignment() : 0; }
DOOMS_CUDA_API int64_t dooms_gguf_tensor_count(const dooms_gguf * f) { return f ? static_cast<int64_t>(f->file->tensors().size()) : 0; }
DOOMS_CUDA_API int32_t dooms_gguf_tensor_at(const dooms_gguf * f, int64_t index, dooms_gguf_tensor * out) {
    if (!f || !out) return fail(DOOMS_INVALID_ARGUMENT, "file or out is NULL");
    if (index < 0 || index >= static_cast<int64_t>(f->file->tensors().size())) return fail(DOOMS_INVALID_ARGUMENT, "tensor index out of range");
    fill_tensor(*f->file, f->file->tensors()[static_cast<size_t>(index)], out);
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_find_tensor(const dooms_gguf * f, const char * name, dooms_gguf_tensor * out) {
    if (!f || !name || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, name or out is NULL");
    auto r = f->file->find_tensor(name);
    if (!r.is_ok()) return done(r.status());
    fill_tensor(*f->file, *r.value(), out);
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_get_string(const dooms_gguf * f, const char * key, const char ** out) {
    if (!f || !key || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, key or out is NULL");
    auto it = f->file->metadata().find(key);
    auto r = f->file->get_string(key);
    if (!r.is_ok()) return done(r.status());
    *out = it->second.s.c_str();   // owned by the file
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_get_uint(const dooms_gguf * f, const char * key, uint64_t * out) {
    if (!f || !key || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, key or out is NULL");
    auto r = f->file->get_uint(key);
    if (!r.is_ok()) return done(r.status());
    *out = r.value();
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_get_int(const dooms_gguf * f, const char * key, int64_t * out) {
    if (!f || !key || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, key or out is NULL");
    auto r = f->file->get_int(key);
    if (!r.is_ok()) return done(r.status());
    *out = r.value();
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_get_float(const dooms_gguf * f, const char * key, double * out) {
    if (!f || !key || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, key or out is NULL");
    auto r = f->file->get_float(key);
    if (!r.is_ok()) return done(r.status());
    *out = r.value();
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_gguf_get_bool(const dooms_gguf * f, const char * key, int32_t * out) {
    if (!f || !key || !out) return fail(DOOMS_INVALID_ARGUMENT, "file, key or out is NULL");
    auto r = f->file->get_bool(key);
    if (!r.is_ok()) return done(r.status());
    *out = r.value() ? 1 : 0;
    return DOOMS_OK;
}

// ---------------------------------------------------------------- decoder

DOOMS_CUDA_API int32_t dooms_cuda_llama_create(const dooms_llama_config * config, const dooms_llama_weights * weights, const dooms_cuda_options * options,
                                               dooms_cuda_llama ** out) {
    int32_t code = DOOMS_OK;
    if (!struct_ok(config, "config", &code) || !struct_ok(weights, "weights", &code)) return code;
    if (options && !struct_ok(options, "options", &code)) return code;
    if (!out) return fail(DOOMS_INVALID_ARGUMENT, "out is NULL");
    LlamaDecoderConfig c;
    c.n_layer = config->n_layer; c.n_embd = config->n_embd; c.n_head = config->n_head; c.n_head_kv = config->n_head_kv; c.head_dim = config->head_dim;
    c.n_ff = config->n_ff; c.n_vocab = config->n_vocab; c.rope_base = config->rope_base; c.rope_neox = config->rope_neox != 0; c.rms_eps = config->rms_eps;
    c.n_ctx = config->n_ctx; c.n_batch = config->n_batch; c.spin_wait = config->spin_wait != 0; c.prefill_tile = config->prefill_tile;
    LlamaDecoderWeights w;
    std::string err;
    bool ok = ref_of(weights->token_embd, &w.token_embd, &err) && ref_of(weights->output_norm, &w.output_norm, &err) && ref_of(weights->output, &w.output, &err);
    if (ok && weights->n_layers > 0 && !weights->layers) { ok = false; err = "weights.layers is NULL"; }
    for (int32_t l = 0; ok && l < weights->n_layers; l++) {
        const dooms_llama_layer_weights & s = weights->layers[l];
        LlamaLayerWeights L;
        ok = ref_of(s.attn_norm, &L.attn_norm, &err) && ref_of(s.attn_q, &L.attn_q, &err) && ref_of(s.attn_k, &L.attn_k, &err) && ref_of(s.attn_v, &L.attn_v, &err) &&
             ref_of(s.attn_qkv, &L.attn_qkv, &err) && ref_of(s.attn_q_bias, &L.attn_q_bias, &err) && ref_of(s.attn_k_bias, &L.attn_k_bias, &err) &&
             ref_of(s.attn_v_bias, &L.attn_v_bias, &err) && ref_of(s.attn_qkv_bias, &L.attn_qkv_bias, &err) && ref_of(s.attn_output, &L.attn_output, &err) &&
             ref_of(s.ffn_norm, &L.ffn_norm, &err) && ref_of(s.ffn_gate, &L.ffn_gate, &err) && ref_of(s.ffn_up, &L.ffn_up, &err) && ref_of(s.ffn_down, &L.ffn_down, &err);
        w.layers.push_back(L);
    }
    if (!ok) return fail(DOOMS_INVALID_ARGUMENT, err);
    auto r = CudaLlamaDecoder::create(c, w, options_of(options));
    if (!r.is_ok()) return done(r.status());
    *out = new dooms_cuda_llama{std::move(r).value()};
    return DOOMS_OK;
}

DOOMS_CUDA_API int32_t dooms_cuda_llama_load(const char * gguf_path, const dooms_native_llama_options * options, const dooms_cuda_options * cuda_options,
                                             dooms_cuda_llama ** out) {
    int32_t code = DOOMS_OK;
    if (!gguf_path || !out) return fail(DOOMS_INVALID_ARGUMENT, "gguf_path or out is NULL");
    if (options && !struct_ok(options, "options", &code)) return code;
    if (cuda_options && !struct_ok(cuda_options, "cuda_options", &code)) return code;
    NativeLlamaOptions o;
    if (options) { o.n_ctx = options->n_ctx; o.n_batch = options->n_batch; o.spin_wait = options->spin_wait != 0; o.prefill_tile = options->prefill_tile; }
    auto r = load_native_llama(gguf_path, o, options_of(cuda_options));
    if (!r.is_ok()) return done(r.status());
    *out = new dooms_cuda_llama{std::move(r).value()};
    return DOOMS_OK;
}

DOOMS_CUDA_API void dooms_cuda_llama_destroy(dooms_cuda_llama * d) { delete d; }

DOOMS_CUDA_API int32_t dooms_cuda_llama_config(const dooms_cuda_llama * d, dooms_llama_config * out) {
    if (!d || !out) return fail(DOOMS_INVALID_ARGUMENT, "decoder or out is NULL");
    const LlamaDecoderConfig & c = d->dec->config();
    std::memset(out, 0, sizeof *out);
    out->struct_size = sizeof *out;
    out->n_layer = c.n_layer; out->n_embd = c.n_embd; out->n_head = c.n_head; out->n_head_kv = c.n_head_kv; out->head_dim = c.head_dim; out->n_ff = c.n_ff;
    out->n_vocab = c.n_vocab; out->rope_base = c.rope_base; out->rope_neox = c.rope_neox ? 1 : 0; out->rms_eps = c.rms_eps; out->n_ctx = c.n_ctx;
    out->n_batch = c.n_batch; out->spin_wait = c.spin_wait ? 1 : 0; out->prefill_tile = c.prefill_tile;
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_position(const dooms_cuda_llama * d) { return d ? d->dec->position() : 0; }
DOOMS_CUDA_API int32_t dooms_cuda_llama_reset(dooms_cuda_llama * d) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    d->dec->reset();
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_eval_tokens(dooms_cuda_llama * d, const int32_t * tokens, int32_t n) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->eval_tokens(tokens, n));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_eval_embeddings(dooms_cuda_llama * d, const float * embeddings, int32_t n) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->eval_embeddings(embeddings, n));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_embed_tokens(dooms_cuda_llama * d, const int32_t * tokens, int32_t n, float * out) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->embed_tokens(tokens, n, out));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_pending_token(dooms_cuda_llama * d, int32_t * out) {
    if (!d || !out) return fail(DOOMS_INVALID_ARGUMENT, "decoder or out is NULL");
    auto r = d->dec->pending_token();
    if (!r.is_ok()) return done(r.status());
    *out = r.value();
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_logits(dooms_cuda_llama * d, float * out, int64_t capacity) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->logits_into(out, capacity));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_generate(dooms_cuda_llama * d, int32_t max_tokens, int32_t depth, dooms_token_callback callback, void * user) {
    if (!d || !callback) return fail(DOOMS_INVALID_ARGUMENT, "decoder or callback is NULL");
    return done(d->dec->generate(max_tokens, depth, [&](int32_t tok) { return callback(tok, user) != 0; }));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_profile_pass(dooms_cuda_llama * d, int32_t rows, dooms_kernel_time * out, int32_t capacity, int32_t * count) {
    if (!d || !count) return fail(DOOMS_INVALID_ARGUMENT, "decoder or count is NULL");
    auto r = d->dec->profile_pass(rows);
    if (!r.is_ok()) return done(r.status());
    const auto & v = r.value();
    if (static_cast<int32_t>(v.size()) > capacity || (!out && !v.empty())) {
        *count = static_cast<int32_t>(v.size());
        return fail(DOOMS_RESOURCE_EXHAUSTED, "profile_pass needs room for " + std::to_string(v.size()) + " entries");
    }
    for (size_t i = 0; i < v.size(); i++) out[i] = dooms_kernel_time{v[i].kind, v[i].dispatches, v[i].gpu_ms};
    *count = static_cast<int32_t>(v.size());
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_timings(const dooms_cuda_llama * d, dooms_cuda_timings * out) {
    int32_t code = DOOMS_OK;
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    if (!struct_ok(out, "out", &code)) return code;
    const CudaLlamaDecoder::Timings t = d->dec->timings();
    out->last_eval_ms = t.last_eval_ms; out->last_generate_ms = t.last_generate_ms; out->last_eval_launches = t.last_eval_launches;
    out->last_generate_launches = t.last_generate_launches; out->weight_bytes = t.weight_bytes; out->kv_bytes = t.kv_bytes;
    if (out->struct_size >= offsetof(dooms_cuda_timings, last_batch_launches) + sizeof(int64_t)) {
        out->last_batch_ms = t.last_batch_ms;
        out->last_batch_launches = t.last_batch_launches;
    }
    if (out->struct_size >= offsetof(dooms_cuda_timings, tp_peer_allreduce) + sizeof(int64_t)) out->tp_peer_allreduce = t.tp_peer_allreduce;
    if (out->struct_size >= offsetof(dooms_cuda_timings, tp_symmetric_window) + sizeof(int64_t)) out->tp_symmetric_window = t.tp_symmetric_window;
    return DOOMS_OK;
}

DOOMS_CUDA_API int32_t dooms_cuda_llama_max_sequences(const dooms_cuda_llama * d) { return d ? d->dec->max_sequences() : 0; }
DOOMS_CUDA_API int32_t dooms_cuda_llama_max_batch_rows(const dooms_cuda_llama * d) { return d ? d->dec->max_batch_rows() : 0; }
DOOMS_CUDA_API int32_t dooms_cuda_llama_select_sequence(dooms_cuda_llama * d, int32_t slot) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->select_sequence(slot));
}
DOOMS_CUDA_API int32_t dooms_cuda_llama_decode_batch(dooms_cuda_llama * d, const int32_t * slots, int32_t n, int32_t steps, int32_t * out_tokens) {
    if (!d) return fail(DOOMS_INVALID_ARGUMENT, "decoder is NULL");
    return done(d->dec->decode_batch(slots, n, steps, out_tokens));
}

// ---------------------------------------------------------------- the Llm surface

namespace {

SamplerOptions sampler_of(const dooms_cuda_sampling * s) {
    SamplerOptions o;      // greedy
    if (s) { o.temperature = s->temperature; o.top_k = s->top_k; o.top_p = s->top_p; o.repeat_penalty = s->repeat_penalty; o.seed = s->seed; }
    return o;
}
bool stops_of(const char * const * stop, int32_t n_stop, std::vector<std::string> * out, int32_t * code) {
    if (n_stop < 0 || (n_stop > 0 && !stop)) { *code = fail(DOOMS_INVALID_ARGUMENT, "stop strings: a count without an array"); return false; }
    for (int32_t i = 0; i < n_stop; i++) {
        if (!stop[i]) { *code = fail(DOOMS_INVALID_ARGUMENT, "stop strings: a NULL entry"); return false; }
        out->push_back(stop[i]);
    }
    return true;
}
int32_t text_out(const std::string & text, char * out, size_t capacity, size_t * needed) {
    if (needed) *needed = text.size() + 1;
    if (!out || capacity < text.size() + 1) return fail(DOOMS_RESOURCE_EXHAUSTED, "the text needs " + std::to_string(text.size() + 1) + " bytes");
    std::memcpy(out, text.c_str(), text.size() + 1);
    return DOOMS_OK;
}
int32_t finish_reason_of(const LlmGeneration & g) { return g.cancelled ? DOOMS_CUDA_FINISH_CANCELLED : g.stopped ? DOOMS_CUDA_FINISH_STOP : DOOMS_CUDA_FINISH_LENGTH; }

// One generation on a handle: the shared body of the three generate entry points.
bool messages_of(const dooms_cuda_chat_message * messages, int32_t n, std::vector<ChatMessage> * out, int32_t * code) {
    if (!messages || n < 1) { *code = fail(DOOMS_INVALID_ARGUMENT, "no messages"); return false; }
    for (int32_t i = 0; i < n; i++) {
        if (!messages[i].role || !messages[i].content) { *code = fail(DOOMS_INVALID_ARGUMENT, "a message has a NULL role or content"); return false; }
        out->push_back({messages[i].role, messages[i].content});
    }
    return true;
}

int32_t run_generation(dooms_cuda_llm * h, const std::vector<int32_t> * prompt_tokens, const char * prompt, int32_t max_new_tokens, const dooms_cuda_sampling * sampling,
                       const char * const * stop, int32_t n_stop, dooms_cuda_text_callback callback, void * user, LlmGeneration * result) {
    if (!h) return fail(DOOMS_INVALID_ARGUMENT, "llm is NULL");
    h->last = dooms_cuda_generation_info{};
    int32_t code = DOOMS_OK;
    LlmGenerateOptions o;
    o.max_new_tokens = max_new_tokens;
    o.sampler = sampler_of(sampling);
    if (!stops_of(stop, n_stop, &o.stop, &code)) return code;
    std::function<bool(const std::string &)> on_text;
    if (callback) on_text = [&](const std::string & piece) { return callback(piece.c_str(), user) == 0; };
    LlmTimings tm;
    Result<LlmGeneration> g = prompt_tokens ? h->llm->generate_tokens(*prompt_tokens, o, on_text, &tm)
                                            : (prompt && *prompt) ? h->llm->generate(prompt, o, on_text, &tm) : Result<LlmGeneration>(invalid_argument("generate: empty prompt"));
    if (!g.is_ok()) return done(g.status());
    h->last.struct_size = sizeof(h->last);
    h->last.prompt_tokens = int32_t(tm.prompt_tokens);
    h->last.completion_tokens = int32_t(g.value().tokens.size());
    h->last.finish_reason = finish_reason_of(g.value());
    h->last.prefill_ms = tm.prefill_ms; h->last.first_token_ms = tm.first_token_ms; h->last.decode_ms = tm.decode_ms;
    *result = std::move(g).value();
    return DOOMS_OK;
}

}  // namespace

DOOMS_CUDA_API int32_t dooms_cuda_llm_open(const char * gguf_path, const dooms_cuda_llm_options * options, dooms_cuda_llm ** out) {
    if (!gguf_path || !out) return fail(DOOMS_INVALID_ARGUMENT, "gguf_path or out is NULL");
    *out = nullptr;
    int32_t code = DOOMS_OK;
    if (options && !struct_ok(options, "options", &code)) return code;
    LlmOptions o;
    if (options) {
        if (options->n_ctx > 0) o.n_ctx = options->n_ctx;
        if (options->n_batch > 0) o.n_batch = options->n_batch;
        if (options->queue_depth > 0) o.queue_depth = options->queue_depth;
        o.cuda.device = options->device;
    }
    auto llm = Llm::load(gguf_path, o);
    if (!llm.is_ok()) return done(llm.status());
    *out = new dooms_cuda_llm{std::move(llm).value(), {}};
    return DOOMS_OK;
}
DOOMS_CUDA_API void dooms_cuda_llm_close(dooms_cuda_llm * llm) { delete llm; }
DOOMS_CUDA_API int32_t dooms_cuda_llm_context_size(const dooms_cuda_llm * llm) { return llm ? llm->llm->context_size() : 0; }

DOOMS_CUDA_API int32_t dooms_cuda_llm_generate(dooms_cuda_llm * llm, const char * prompt, int32_t max_new_tokens, const dooms_cuda_sampling * sampling,
                                               const char * const * stop, int32_t n_stop, char * out, size_t capacity, size_t * needed) {
    LlmGeneration g;
    const int32_t code = run_generation(llm, nullptr, prompt, max_new_tokens, sampling, stop, n_stop, nullptr, nullptr, &g);
    return code != DOOMS_OK ? code : text_out(g.text, out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_stream(dooms_cuda_llm * llm, const char * prompt, int32_t max_new_tokens, const dooms_cuda_sampling * sampling,
                                                      const char * const * stop, int32_t n_stop, dooms_cuda_text_callback callback, void * user) {
    if (!callback) return fail(DOOMS_INVALID_ARGUMENT, "callback is NULL");
    LlmGeneration g;
    return run_generation(llm, nullptr, prompt, max_new_tokens, sampling, stop, n_stop, callback, user, &g);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_tokens(dooms_cuda_llm * llm, const int32_t * prompt, int32_t n_prompt, int32_t max_new_tokens,
                                                      const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, char * out, size_t capacity,
                                                      size_t * needed, int32_t * out_tokens, int32_t token_capacity, int32_t * n_tokens) {
    if (!prompt || n_prompt < 1) return fail(DOOMS_INVALID_ARGUMENT, "generate: empty prompt");
    const std::vector<int32_t> p(prompt, prompt + n_prompt);
    LlmGeneration g;
    const int32_t code = run_generation(llm, &p, nullptr, max_new_tokens, sampling, stop, n_stop, nullptr, nullptr, &g);
    if (code != DOOMS_OK) return code;
    if (n_tokens) *n_tokens = int32_t(g.tokens.size());
    if (out_tokens) {
        if (token_capacity < int32_t(g.tokens.size())) return fail(DOOMS_RESOURCE_EXHAUSTED, "the tokens need room for " + std::to_string(g.tokens.size()) + " ids");
        std::copy(g.tokens.begin(), g.tokens.end(), out_tokens);
    }
    return text_out(g.text, out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_generate_from_embeddings(dooms_cuda_llm * llm, const int32_t * before, int32_t n_before, const float * image, int32_t image_rows,
                                                               const int32_t * after, int32_t n_after, int32_t max_new_tokens, dooms_cuda_text_callback callback,
                                                               void * user, char * out, size_t capacity, size_t * needed) {
    if (!llm) return fail(DOOMS_INVALID_ARGUMENT, "llm is NULL");
    if (n_before < 0 || n_after < 0 || (n_before > 0 && !before) || (n_after > 0 && !after)) return fail(DOOMS_INVALID_ARGUMENT, "token counts without arrays");
    llm->last = dooms_cuda_generation_info{};
    std::function<bool(const std::string &)> on_text;
    if (callback) on_text = [&](const std::string & piece) { return callback(piece.c_str(), user) == 0; };
    LlmTimings tm;
    auto g = llm->llm->generate_from_embeddings(std::vector<int32_t>(before, before + n_before), image, image_rows, std::vector<int32_t>(after, after + n_after), max_new_tokens,
                                                on_text, &tm);
    if (!g.is_ok()) return done(g.status());
    llm->last.struct_size = sizeof(llm->last);
    llm->last.prompt_tokens = int32_t(tm.prompt_tokens);
    llm->last.completion_tokens = int32_t(g.value().tokens.size());
    llm->last.finish_reason = finish_reason_of(g.value());
    llm->last.prefill_ms = tm.prefill_ms; llm->last.first_token_ms = tm.first_token_ms; llm->last.decode_ms = tm.decode_ms;
    return text_out(g.value().text, out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_last_generation(const dooms_cuda_llm * llm, dooms_cuda_generation_info * out) {
    int32_t code = DOOMS_OK;
    if (!llm) return fail(DOOMS_INVALID_ARGUMENT, "llm is NULL");
    if (!struct_ok(out, "out", &code)) return code;
    const size_t size = out->struct_size;
    std::memcpy(out, &llm->last, std::min(size, sizeof(llm->last)));
    out->struct_size = size;
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_chat(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t max_new_tokens,
                                           const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, char * out, size_t capacity, size_t * needed) {
    if (!llm) return fail(DOOMS_INVALID_ARGUMENT, "llm is NULL");
    int32_t code = DOOMS_OK;
    std::vector<ChatMessage> chat;
    if (!messages_of(messages, n_messages, &chat, &code)) return code;
    auto tokens = llm->llm->chat_tokens(chat);
    if (!tokens.is_ok()) return done(tokens.status());
    LlmGeneration g;
    code = run_generation(llm, &tokens.value(), nullptr, max_new_tokens, sampling, stop, n_stop, nullptr, nullptr, &g);
    return code != DOOMS_OK ? code : text_out(g.text, out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_chat_stream(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t max_new_tokens,
                                                  const dooms_cuda_sampling * sampling, const char * const * stop, int32_t n_stop, dooms_cuda_text_callback callback,
                                                  void * user) {
    if (!llm) return fail(DOOMS_INVALID_ARGUMENT, "llm is NULL");
    if (!callback) return fail(DOOMS_INVALID_ARGUMENT, "callback is NULL");
    int32_t code = DOOMS_OK;
    std::vector<ChatMessage> chat;
    if (!messages_of(messages, n_messages, &chat, &code)) return code;
    auto tokens = llm->llm->chat_tokens(chat);
    if (!tokens.is_ok()) return done(tokens.status());
    LlmGeneration g;
    return run_generation(llm, &tokens.value(), nullptr, max_new_tokens, sampling, stop, n_stop, callback, user, &g);
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_count_chat_tokens(dooms_cuda_llm * llm, const dooms_cuda_chat_message * messages, int32_t n_messages, int32_t * count) {
    if (!llm || !count) return fail(DOOMS_INVALID_ARGUMENT, "llm or count is NULL");
    int32_t code = DOOMS_OK;
    std::vector<ChatMessage> chat;
    if (!messages_of(messages, n_messages, &chat, &code)) return code;
    auto tokens = llm->llm->chat_tokens(chat);
    if (!tokens.is_ok()) return done(tokens.status());
    *count = int32_t(tokens.value().size());
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_llm_count_tokens(dooms_cuda_llm * llm, const char * text, int32_t add_special, int32_t * count) {
    if (!llm || !count) return fail(DOOMS_INVALID_ARGUMENT, "llm or count is NULL");
    if (!text || !*text) return fail(DOOMS_INVALID_ARGUMENT, "count_tokens: empty text");
    auto t = llm->llm->tokenize(text, add_special != 0);
    if (!t.is_ok()) return done(t.status());
    *count = int32_t(t.value().size());
    return DOOMS_OK;
}

DOOMS_CUDA_API int32_t dooms_cuda_vocab_open(const char * gguf_path, dooms_cuda_vocab ** out) {
    if (!gguf_path || !out) return fail(DOOMS_INVALID_ARGUMENT, "gguf_path or out is NULL");
    *out = nullptr;
    auto file = GgufFile::open(gguf_path);
    if (!file.is_ok()) return done(file.status());
    auto v = Vocab::from_gguf(file.value());
    if (!v.is_ok()) return done(v.status());
    *out = new dooms_cuda_vocab{std::move(v).value()};
    return DOOMS_OK;
}
DOOMS_CUDA_API void dooms_cuda_vocab_close(dooms_cuda_vocab * vocab) { delete vocab; }
DOOMS_CUDA_API int32_t dooms_cuda_vocab_size(const dooms_cuda_vocab * vocab) { return vocab ? vocab->vocab.size() : 0; }
DOOMS_CUDA_API int32_t dooms_cuda_vocab_is_end_of_generation(const dooms_cuda_vocab * vocab, int32_t token) { return vocab && vocab->vocab.is_end_of_generation(token) ? 1 : 0; }
DOOMS_CUDA_API int32_t dooms_cuda_vocab_piece(const dooms_cuda_vocab * vocab, int32_t token, char * out, int32_t capacity, int32_t * n) {
    if (!vocab || !n) return fail(DOOMS_INVALID_ARGUMENT, "vocab or n is NULL");
    if (token < 0 || token >= vocab->vocab.size()) return fail(DOOMS_INVALID_ARGUMENT, "token " + std::to_string(token) + " is outside the vocabulary");
    const std::string & p = vocab->vocab.piece(token);
    *n = int32_t(p.size());
    if (capacity < *n || (!out && *n > 0)) return fail(DOOMS_RESOURCE_EXHAUSTED, "the piece needs " + std::to_string(*n) + " bytes");
    if (*n > 0) std::memcpy(out, p.data(), p.size());
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_vocab_apply_chat_template(const dooms_cuda_vocab * vocab, const dooms_cuda_chat_message * messages, int32_t n_messages,
                                                            int32_t add_generation_prompt, char * out, size_t capacity, size_t * needed) {
    if (!vocab) return fail(DOOMS_INVALID_ARGUMENT, "vocab is NULL");
    int32_t code = DOOMS_OK;
    std::vector<ChatMessage> chat;
    if (!messages_of(messages, n_messages, &chat, &code)) return code;
    auto text = vocab->vocab.apply_chat_template(chat, add_generation_prompt != 0);
    if (!text.is_ok()) return done(text.status());
    return text_out(text.value(), out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_vocab_tokenize_special(const dooms_cuda_vocab * vocab, const char * text, int32_t add_special, int32_t parse_special, int32_t * out,
                                                         int32_t capacity, int32_t * n) {
    if (!vocab || !n) return fail(DOOMS_INVALID_ARGUMENT, "vocab or n is NULL");
    auto t = vocab->vocab.tokenize(text ? text : "", add_special != 0, parse_special != 0);
    if (!t.is_ok()) return done(t.status());
    *n = int32_t(t.value().size());
    if (!out || capacity < *n) return fail(DOOMS_RESOURCE_EXHAUSTED, "the ids need room for " + std::to_string(*n));
    std::copy(t.value().begin(), t.value().end(), out);
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_vocab_tokenize(const dooms_cuda_vocab * vocab, const char * text, int32_t add_special, int32_t * out, int32_t capacity, int32_t * n) {
    if (!vocab || !n) return fail(DOOMS_INVALID_ARGUMENT, "vocab or n is NULL");
    auto t = vocab->vocab.tokenize(text ? text : "", add_special != 0);
    if (!t.is_ok()) return done(t.status());
    *n = int32_t(t.value().size());
    if (!out || capacity < *n) return fail(DOOMS_RESOURCE_EXHAUSTED, "the ids need room for " + std::to_string(*n));
    std::copy(t.value().begin(), t.value().end(), out);
    return DOOMS_OK;
}
DOOMS_CUDA_API int32_t dooms_cuda_text_stream(const dooms_cuda_vocab * vocab, const int32_t * tokens, int32_t n_tokens, const char * const * stop, int32_t n_stop,
                                              dooms_cuda_text_callback callback, void * user, char * out, size_t capacity, size_t * needed, int32_t * consumed,
                                              int32_t * finish_reason) {
    if (!vocab || (n_tokens > 0 && !tokens) || n_tokens < 0) return fail(DOOMS_INVALID_ARGUMENT, "vocab or tokens is NULL");
    int32_t code = DOOMS_OK;
    std::vector<std::string> stops;
    if (!stops_of(stop, n_stop, &stops, &code)) return code;
    for (const std::string & s : stops) if (s.empty()) return fail(DOOMS_INVALID_ARGUMENT, "an empty stop string");
    LlmGeneration g;
    std::function<bool(const std::string &)> on_text;
    if (callback) on_text = [&](const std::string & piece) { return callback(piece.c_str(), user) == 0; };
    TextStream stream(vocab->vocab, stops, on_text, &g);
    int32_t taken = 0;
    while (taken < n_tokens) { taken++; if (!stream.push(tokens[taken - 1])) break; }
    stream.finish();
    if (consumed) *consumed = taken;
    if (finish_reason) *finish_reason = finish_reason_of(g);
    return text_out(g.text, out, capacity, needed);
}
DOOMS_CUDA_API int32_t dooms_cuda_sample(const float * logits, int32_t n, const dooms_cuda_sampling * sampling, int32_t draws, int32_t * out_tokens) {
    if (!logits || n < 1 || draws < 1 || !out_tokens) return fail(DOOMS_INVALID_ARGUMENT, "sample: logits, n, draws and out_tokens are required");
    auto s = Sampler::create(sampler_of(sampling));
    if (!s.is_ok()) return done(s.status());
    for (int32_t i = 0; i < draws; i++) out_tokens[i] = s.value().sample(logits, n);
    return DOOMS_OK;
}

// ---------------------------------------------------------------- single kernels

DOOMS_CUDA_API int32_t dooms_cuda_dequantize(int32_t dtype, const void * d_blocks, int64_t rows, int64_t cols, float * d_out, void * stream) {
    if (!matrix_dtype(dtype)) return fail(DOOMS_UNSUPPORTED, "dequantize takes f16, q4_0, q5_0, q8_0, q4_K and q6_K");
    if (!d_blocks || !d_out || rows < 0 || cols < 1 || cols % dooms_dtype_block_elems(dtype) != 0 || cols > INT32_MAX) {
        return fail(DOOMS_INVALID_ARGUMENT, "dequantize: NULL pointer or rows that are not whole blocks");
    }
    if (rows == 0) return DOOMS_OK;
    return launch_result(cuda::launch_dequantize(dtype, d_blocks, rows, cols, d_out, static_cast<cudaStream_t>(stream)), "dequantize");
}

DOOMS_CUDA_API int32_t dooms_cuda_matvec(int32_t dtype, const void * d_w, const float * d_x, float * d_y, const float * d_bias, int64_t rows, int64_t cols,
                                         uint32_t flags, void * stream) {
    if (!matrix_dtype(dtype)) return fail(DOOMS_UNSUPPORTED, "matvec takes f16, q4_0, q5_0, q8_0, q4_K and q6_K");
    if (!d_w || !d_x || !d_y || rows < 0 || cols < 32 || cols % 32 != 0 || cols % dooms_dtype_block_elems(dtype) != 0 || cols > INT32_MAX ||
        ((flags & cuda::kFlagBias) && !d_bias) || (flags & ~(cuda::kFlagAccumulate | cuda::kFlagBias))) {
        return fail(DOOMS_INVALID_ARGUMENT, "matvec: NULL pointer, unknown flag, or rows that are not whole blocks of at least 32 elements");
    }
    if (rows == 0) return DOOMS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == DOOMS_Q4_0 && cuda::gemv_q4_0_supported(d_w, rows, cols)) return fast_q4_0(d_w, nullptr, d_x, d_y, d_bias, rows, cols, flags, false, st, "matvec");
    if (dtype == DOOMS_Q4_K && cuda::gemv_q4_k_supported(d_w, rows, cols)) return fast_q4_0(d_w, nullptr, d_x, d_y, d_bias, rows, cols, flags, true, st, "matvec");
    if (dtype == DOOMS_Q6_K && cuda::gemv_q6_k_supported(d_w, rows, cols)) {
        void * scratch = nullptr;
        const Status ss = scratch_for((cuda::quantized_x_bytes(cols) + 15) & ~size_t(15), &scratch);
        if (!ss.is_ok()) return done(ss);
        cudaError_t e = cuda::launch_quantize_x(d_x, cols, scratch, st);
        if (e == cudaSuccess) e = cuda::launch_gemv_q6_k(d_w, scratch, d_y, d_bias, rows, cols, flags, st);
        return launch_result(e, "matvec");
    }
    return launch_result(cuda::launch_matvec(dtype, d_w, d_x, d_y, d_bias, rows, cols, flags, st), "matvec");
}

DOOMS_CUDA_API int64_t dooms_cuda_split_input_bytes(int64_t cols) {
    return cols >= 32 && cols % 32 == 0 ? int64_t((cuda::quantized_x_bytes(cols) + 15) & ~size_t(15)) : 0;
}

DOOMS_CUDA_API int32_t dooms_cuda_split_input(const float * d_x, int64_t cols, void * d_split, void * stream) {
    if (!d_x || !d_split || cols < 32 || cols % 32 != 0 || cols > INT32_MAX) return fail(DOOMS_INVALID_ARGUMENT, "split_input: NULL pointer, or a length that is not whole 32-element blocks");
    return launch_result(cuda::launch_quantize_x(d_x, cols, d_split, static_cast<cudaStream_t>(stream)), "split_input");
}

DOOMS_CUDA_API int32_t dooms_cuda_matvec_split(int32_t dtype, const void * d_w, const void * d_w2, const void * d_split, float * d_y, const float * d_bias, int64_t rows,
                                               int64_t cols, uint32_t flags, void * stream) {
    if (dtype != DOOMS_Q4_0 && dtype != DOOMS_Q4_K) return fail(DOOMS_UNSUPPORTED, "matvec_split takes q4_0 and q4_K rows (the integer tensor-core kernel)");
    if (!d_w || !d_split || !d_y || rows < 1 || cols < 32 || cols % 32 != 0 || cols > INT32_MAX || ((flags & cuda::kFlagBias) && !d_bias) ||
        (flags & ~(cuda::kFlagAccumulate | cuda::kFlagBias)) || (d_w2 && flags)) {
        return fail(DOOMS_INVALID_ARGUMENT, "matvec_split: NULL pointer, unknown flag, or rows that are not whole blocks");
    }
    const bool k4 = dtype == DOOMS_Q4_K;
    const bool ok = k4 ? cuda::gemv_q4_k_supported(d_w, rows, cols) && (!d_w2 || cuda::gemv_q4_k_supported(d_w2, rows, cols))
                       : cuda::gemv_q4_0_supported(d_w, rows, cols) && (!d_w2 || cuda::gemv_q4_0_supported(d_w2, rows, cols));
    if (!ok) return fail(DOOMS_UNSUPPORTED, "matvec_split: a shape or alignment the integer tensor-core kernel does not take");
    return launch_result(cuda::launch_gemv_q4_0(d_w, d_w2, d_split, nullptr, nullptr, 0.f, d_y, d_bias, rows, cols, flags, k4, static_cast<cudaStream_t>(stream), nullptr,
                                                nullptr, kernel_error_word()), "matvec_split");
}

DOOMS_CUDA_API int32_t dooms_cuda_gate_up(int32_t dtype, const void * d_wg, const void * d_wu, const float * d_x, float * d_h, int64_t rows, int64_t cols,
                                          void * stream) {
    if (!matrix_dtype(dtype)) return fail(DOOMS_UNSUPPORTED, "gate_up takes f16, q4_0, q5_0, q8_0, q4_K and q6_K");
    if (!d_wg || !d_wu || !d_x || !d_h || rows < 0 || cols < 32 || cols % 32 != 0 || cols % dooms_dtype_block_elems(dtype) != 0 || cols > INT32_MAX) {
        return fail(DOOMS_INVALID_ARGUMENT, "gate_up: NULL pointer or rows that are not whole blocks of at least 32 elements");
    }
    if (rows == 0) return DOOMS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == DOOMS_Q4_0 && cuda::gemv_q4_0_supported(d_wg, rows, cols) && cuda::gemv_q4_0_supported(d_wu, rows, cols)) {
        return fast_q4_0(d_wg, d_wu, d_x, d_h, nullptr, rows, cols, 0u, false, st, "gate_up");
    }
    if (dtype == DOOMS_Q4_K && cuda::gemv_q4_k_supported(d_wg, rows, cols) && cuda::gemv_q4_k_supported(d_wu, rows, cols)) {
        return fast_q4_0(d_wg, d_wu, d_x, d_h, nullptr, rows, cols, 0u, true, st, "gate_up");
    }
    return launch_result(cuda::launch_gate_up(dtype, d_wg, d_wu, d_x, d_h, rows, cols, st), "gate_up");
}

DOOMS_CUDA_API int32_t dooms_cuda_matmul(int32_t dtype, const void * d_w, const void * d_w2, const void * d_x16, float * d_y, const float * d_bias,
                                         int32_t tokens, int64_t rows, int64_t cols, uint32_t flags, void * stream) {
    if (!matrix_dtype(dtype)) return fail(DOOMS_UNSUPPORTED, "matmul takes f16, q4_0, q5_0, q8_0, q4_K and q6_K");
    if (!d_w || !d_x16 || !d_y || tokens < 1 || rows < 1 || cols < 64 || cols % 64 != 0 || cols % dooms_dtype_block_elems(dtype) != 0 || cols > INT32_MAX ||
        ((flags & cuda::kFlagBias) && !d_bias) || (flags & ~(cuda::kFlagAccumulate | cuda::kFlagBias)) || (d_w2 && flags)) {
        return fail(DOOMS_INVALID_ARGUMENT, "matmul: NULL pointer, unknown flag, or rows that are not whole blocks and a multiple of 64 elements");
    }
    // 128 tokens or more: room for the matrix (both, for gate/up) as f16 rows, so that it is dequantized once and both operands arrive by TMA
    const size_t w16_bytes = tokens >= 128 && dtype != DOOMS_F16 ? size_t(rows) * size_t(cols) * 2 * (d_w2 ? 2 : 1) : 0;
    void * scratch = nullptr;
    const Status ss = scratch_for(256 + w16_bytes, &scratch);
    if (!ss.is_ok()) return done(ss);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cuda::TensorMap map;
    cudaError_t e = cuda::make_activation_map(&map, d_x16, tokens, cols);
    if (e != cudaSuccess) return launch_result(e, "matmul (tensor map)");
    int32_t * err = kernel_error_word();
    if (!err) return fail(DOOMS_RESOURCE_EXHAUSTED, "matmul: could not allocate the kernel error word");
    {
        e = cuda::launch_gemm_tc(dtype, d_w, d_w2, &map, d_y, nullptr, d_bias, tokens, rows, cols, rows, 0, flags, err, st,
                                 w16_bytes ? static_cast<uint8_t *>(scratch) + 256 : nullptr, w16_bytes);
    }
    return launch_result(e, "matmul");
}

DOOMS_CUDA_API int32_t dooms_cuda_kernel_status(void * stream, int32_t * flag) {
    if (flag) *flag = 0;
    const cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return launch_result(e, "kernel_status");
    int32_t * err = kernel_error_word();
    const int32_t seen = err ? *err : 0;
    if (err) *err = 0;
    if (flag) *flag = seen;
    if (seen == 0) return DOOMS_OK;
    return fail(DOOMS_INTERNAL, "a kernel gave up a bounded wait (flag " + std::to_string(seen) + (seen == 2 ? ": matmul" : seen == 4 ? ": matvec / gate_up tensor copy" : "") +
                                    "); its output is not valid");
}

DOOMS_CUDA_API int32_t dooms_cuda_rms_norm(const float * d_x, const float * d_gamma, float * d_out, int64_t rows, int64_t cols, float eps, void * stream) {
    if (!d_x || !d_gamma || !d_out || rows < 0 || cols < 1 || rows > INT32_MAX || cols > INT32_MAX || !(eps > 0.f)) {
        return fail(DOOMS_INVALID_ARGUMENT, "rms_norm: NULL pointer, bad shape or eps <= 0");
    }
    if (rows == 0) return DOOMS_OK;
    return launch_result(cuda::launch_rms_norm(d_x, d_gamma, d_out, nullptr, nullptr, int(rows), int(cols), eps, static_cast<cudaStream_t>(stream)), "rms_norm");
}

DOOMS_CUDA_API int32_t dooms_cuda_argmax(const float * d_logits, int64_t n, int32_t * d_out, void * stream) {
    if (!d_logits || !d_out || n < 1 || n > INT32_MAX) return fail(DOOMS_INVALID_ARGUMENT, "argmax: NULL pointer or n outside [1, 2^31)");
    void * part = nullptr;
    const Status st = scratch_for(size_t(cuda::argmax_blocks(n)) * 8, &part);
    if (!st.is_ok()) return done(st);
    return launch_result(cuda::launch_argmax_plain(d_logits, n, d_out, part, static_cast<cudaStream_t>(stream)), "argmax");
}

DOOMS_CUDA_API int32_t dooms_cuda_argmax_noalloc(const float * d_logits, int64_t n, int32_t * d_out, void * stream) {
    if (!d_logits || !d_out || n < 1) return fail(DOOMS_INVALID_ARGUMENT, "argmax_noalloc: NULL pointer or n < 1");
    if (n > DOOMS_CUDA_ARGMAX_NOALLOC_MAX || cuda::argmax_blocks(n) > kNoAllocParts) {
        return fail(DOOMS_INVALID_ARGUMENT, "argmax_noalloc: n = " + std::to_string(n) + " exceeds the fixed scratch, which holds the partial results of at most " +
                                            std::to_string(DOOMS_CUDA_ARGMAX_NOALLOC_MAX) + " logits; use dooms_cuda_argmax");
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return fail(DOOMS_UNSUPPORTED, "argmax_noalloc: no CUDA device"); }
    void * part = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_argmax_noalloc_mutex);
        if (!g_argmax_noalloc_ptr[dev]) {      // once per device, with that device current
            void * p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_noalloc_scratch);
            if (e != cudaSuccess || !p) { (void)cudaGetLastError(); return fail(DOOMS_INTERNAL, std::string("argmax_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e)); }
            g_argmax_noalloc_ptr[dev] = p;
        }
        part = g_argmax_noalloc_ptr[dev];
    }
    // every partial result read by the final pass is written by the first pass of the same call: nothing in the array has to start at zero
    return launch_result(cuda::launch_argmax_plain(d_logits, n, d_out, part, static_cast<cudaStream_t>(stream)), "argmax_noalloc");
}

DOOMS_CUDA_API int64_t dooms_cuda_attention_scratch_bytes(int32_t n_head, int32_t head_dim, int32_t n_keys) {
    if (n_head < 1 || head_dim < 1 || n_keys < 1) return 0;
    // enough for either kernel: the grouped-query one uses at most one range per SM
    return int64_t(std::max(cuda::attention_splits(n_head, n_keys), cuda::attention_gqa_splits(1, n_keys))) * n_head * (2 + head_dim) * 4;
}

DOOMS_CUDA_API int32_t dooms_cuda_attention_decode(const float * d_q, const void * d_kc, const void * d_vc, float * d_out, void * d_scratch, int32_t n_head,
                                                   int32_t n_head_kv, int32_t head_dim, int32_t n_keys, void * stream) {
    if (!d_q || !d_kc || !d_vc || !d_out || !d_scratch || n_head < 1 || n_head_kv < 1 || n_head % n_head_kv != 0 || n_keys < 1) {
        return fail(DOOMS_INVALID_ARGUMENT, "attention_decode: NULL pointer or bad head counts");
    }
    if (head_dim < 4 || head_dim > 256 || (head_dim & (head_dim - 1)) != 0) return fail(DOOMS_UNSUPPORTED, "attention_decode: head_dim must be a power of two in [4, 256]");
    const cuda::AttnShape s{n_head, n_head_kv, head_dim, n_head * head_dim, n_head_kv * head_dim, n_head * head_dim, 0, 10000.f};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cuda::attention_gqa_supported(s) && (reinterpret_cast<uintptr_t>(d_kc) & 15u) == 0 && (reinterpret_cast<uintptr_t>(d_vc) & 15u) == 0) {
        // q alone is read of the row, so d_q stands for the whole row
        const int gs = cuda::attention_gqa_splits(n_head_kv, n_keys);
        const cudaError_t e = cuda::launch_attention_gqa(d_q, const_cast<void *>(d_kc), const_cast<void *>(d_vc), static_cast<float *>(d_scratch), nullptr, nullptr,
                                                         n_keys, gs, s, nullptr, nullptr, nullptr, st);
        if (e != cudaSuccess) return launch_result(e, "attention_decode");
        return launch_result(cuda::launch_attention_combine(static_cast<const float *>(d_scratch), d_out, nullptr, gs, s, st), "attention_decode");
    }
    const int splits = cuda::attention_splits(n_head, n_keys);
    return launch_result(cuda::launch_attention_decode(d_q, d_kc, d_vc, d_out, static_cast<float *>(d_scratch), nullptr, nullptr, n_keys, splits, s,
                                                       static_cast<cudaStream_t>(stream)), "attention_decode");
}

DOOMS_CUDA_API int32_t dooms_cuda_tp_share_blocks(const dooms_llama_config * config, int32_t tp_rank, int32_t tp_size, int64_t attn_block, int64_t ffn_block,
                                                  dooms_tp_share * out) {
    int32_t code = DOOMS_OK;
    if (!struct_ok(config, "config", &code) || !struct_ok(out, "out", &code)) return code;
    LlamaDecoderConfig c;
    c.n_head = config->n_head; c.n_head_kv = config->n_head_kv; c.head_dim = config->head_dim; c.n_ff = config->n_ff; c.n_vocab = config->n_vocab;
    auto r = tp_share(c, tp_rank, tp_size, attn_block, ffn_block);
    if (!r.is_ok()) return done(r.status());
    const TpShare & s = r.value();
    out->q_row0 = s.q_row0; out->q_rows = s.q_rows; out->kv_row0 = s.kv_row0; out->kv_rows = s.kv_rows; out->ff_row0 = s.ff_row0; out->ff_rows = s.ff_rows;
    out->vocab_row0 = s.vocab_row0; out->vocab_rows = s.vocab_rows;
    if (out->struct_size >= offsetof(dooms_tp_share, attn_cols) + sizeof(int64_t)) { out->attn_col0 = s.attn_col0; out->attn_cols = s.attn_cols; }
    return DOOMS_OK;
}

DOOMS_CUDA_API int32_t dooms_cuda_tp_share(const dooms_llama_config * config, int32_t tp_rank, int32_t tp_size, dooms_tp_share * out) {
    return dooms_cuda_tp_share_blocks(config, tp_rank, tp_size, 1, 1, out);
}

DOOMS_CUDA_API int32_t dooms_cuda_nccl_unique_id(const char * nccl_library, void * out128) {
    if (!out128) return fail(DOOMS_INVALID_ARGUMENT, "out128 is NULL");
    static NcclApi api;
    const Status st = load_nccl(nccl_library, &api);
    if (!st.is_ok()) return done(st);
    NcclUniqueId id;
    const int rc = api.GetUniqueId(&id);
    if (rc != 0) return fail(DOOMS_INTERNAL, std::string("ncclGetUniqueId: ") + api.GetErrorString(rc));
    std::memcpy(out128, &id, sizeof id);
    return DOOMS_OK;
}

}  // extern "C"
