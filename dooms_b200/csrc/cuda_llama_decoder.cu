#include "cuda_llama_decoder.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <string>
#include <utility>

#include "kernels/kernels.h"
#include "nccl_dyn.h"
#include "validate.h"

namespace dooms {

using cuda::AttnShape;
using cuda::DevState;
using cuda::kFlagAccumulate;
using cuda::kFlagBias;

namespace {

constexpr size_t kWeightAlign = 256;   // offset alignment of each tensor inside the weight buffer
constexpr size_t kWeightTail = 256;    // slack after the last tensor: kernels that read rows as 16-byte spans may run a few bytes past a matrix
constexpr int kMaxHeadDim = 256;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool is_matrix_type(DType t) {
    return t == DType::F16 || t == DType::Q4_0 || t == DType::Q5_0 || t == DType::Q8_0 || t == DType::Q4_K || t == DType::Q6_K;
}

std::string cuda_msg(const char * what, cudaError_t e) { return std::string(what) + ": " + cudaGetErrorString(e); }

// A matrix in the device weight buffer.
struct MatDev {
    const uint8_t * ptr = nullptr;
    DType dt = DType::F16;
    int64_t rows = 0, cols = 0;
    const __half * rows16 = nullptr;      // optional: the same matrix as f16 rows, for the projections of batched steps
    int64_t bytes() const { return rows * static_cast<int64_t>(dtype_bytes(dt, cols).value()); }
};
// q, k and v are one concatenated matrix when they share a type; otherwise one part each (rows row0.. of the qkv output).
struct QkvPart { MatDev w; int32_t row0 = 0; };
struct LayerDev {
    const float * attn_norm = nullptr, * ffn_norm = nullptr, * qkv_bias = nullptr;
    std::vector<QkvPart> qkv;
    MatDev attn_output, ffn_gate, ffn_up, ffn_down;
};

float half_bits_to_float(uint16_t h) { __half v; std::memcpy(&v, &h, 2); return __half2float(v); }

}  // namespace

struct CudaLlamaDecoder::Impl {
    LlamaDecoderConfig cfg;
    CudaOptions opt;
    int tp = 1, rank = 0;
    // this rank's share
    // attn_width / attn_pad: the attention rows are as wide as the blocks of attn_output this rank holds; its heads' columns start attn_pad into a row and
    // the rest stays zero (one GPU, or shards on block boundaries: attn_width = q_width, attn_pad = 0)
    int32_t attn_width = 0, attn_pad = 0;
    int32_t nh = 0, nkv = 0, q_width = 0, kv_width = 0, qkv_width = 0, ff = 0, vocab_rows = 0, vocab_row0 = 0, vocab_stride = 0;
    cudaStream_t stream = nullptr;
    uint8_t * weights = nullptr;
    size_t weight_bytes = 0, matrix_bytes = 0;
    MatDev token_embd, output;
    const float * output_norm = nullptr;
    std::vector<LayerDev> layers;
    __half * kc = nullptr, * vc = nullptr;
    size_t cache_layer_elems = 0, kv_bytes = 0;
    // Several sequences (CudaOptions::max_sequences): each layer's cache holds one slot of n_ctx positions per sequence. The calls of the single-sequence
    // interface act on the selected slot; its position and pending-token flag live in pos / has_pending, the other slots' in seqs.
    struct Sequence { int32_t pos = 0; bool has_pending = false; int32_t pending = 0; };
    std::vector<Sequence> seqs;
    int32_t cur = 0, graph_slot = 0, logits_slot = 0;
    size_t slot_elems = 0;          // f16 elements of one slot within a layer: n_ctx * kv_width
    // one decode step over several slots at once (decode_batch)
    int32_t max_rows = 0;           // rows such a step can hold
    int32_t * b_rows = nullptr;     // device: slot[max_rows], pos[max_rows], tok[max_rows]
    int32_t * b_out = nullptr;      // device: [kMaxBatchSteps][max_rows] tokens
    int32_t * b_step = nullptr;     // device: steps done in the current call
    int32_t * h_rows = nullptr, * h_out = nullptr;   // pinned staging of the same
    float * b_logits = nullptr, * b_part = nullptr;
    void * b_argmax_part = nullptr;
    int * b_counters = nullptr;
    int b_splits = 1;
    std::vector<std::pair<int32_t, cudaGraphExec_t>> batch_graphs;   // per number of rows
    int64_t batch_step_launches_count = 0;
    float * x = nullptr, * xn = nullptr, * qkv = nullptr, * attn = nullptr, * h = nullptr, * red = nullptr, * logits_buf = nullptr, * part = nullptr;
    void * argmax_part = nullptr;
    __half * xn16 = nullptr, * attn16 = nullptr, * h16 = nullptr;   // f16 activations of a prefill chunk, the tensor-core GEMM's token operands
    cuda::TensorMap map_xn, map_attn, map_h;
    bool tc_capable = false;       // every reduction length is a multiple of 64 and the TMA descriptors exist
    uint8_t * xq = nullptr;        // the current projection input split into int8 limbs (the staged q4_0 GEMV's operand)
    const float * xq_of = nullptr; // which f32 vector xq currently holds
    int32_t * tokens = nullptr, * in_tokens = nullptr, * host_tokens = nullptr, * host_in = nullptr;
    float * host_x = nullptr;     // pinned staging for eval_embeddings
    DevState * state = nullptr;
    int32_t * host_error = nullptr;   // mapped pinned word a kernel sets when a bounded wait ran out
    // tensor parallelism: x, red and tp_pairs in one allocation of NCCL's own (sym_base) registered as a symmetric window (sym_win), when the library
    // offers that; the three pointers then lie inside it and are not freed on their own
    void * sym_base = nullptr, * sym_win = nullptr;
    int32_t * tp_pairs = nullptr;  // tensor parallelism: every rank's (best logit, its index) of the current position
    bool logits_gathered = true;   // logits_buf holds every rank's rows (always true on one GPU)
    int splits = 1;
    static constexpr int kMaxShares = 32;
    __half * rows16_all = nullptr;   // batched decode steps: the matrices as f16 rows (MatDev::rows16 point into it), when memory allows
    float * b_shares = nullptr;  // batched decode steps: [share][max_rows][n_embd] sums of the blocks that share a tile's reduction
    bool rows_tc = false;        // batched decode steps: attention on the tensor cores (attention_rows.cu)
    bool gqa = false;            // decode attention: the grouped-query kernel (which also rotates and stores the new key / value)
    int gqa_splits = 1;
    double * inv_freq = nullptr;   // head_dim / 2 rotary frequencies
    void * rope_cs = nullptr;      // head_dim / 2 (cos, sin) pairs of the current decode step's position
    int * attn_counters = nullptr; // one per key/value head: blocks of the decode attention that have finished (zero between launches)
    void * w16 = nullptr;           // room for the largest matrix (pair) as f16 rows: chunks of 128 tokens or more dequantize a matrix once per call
    size_t w16_bytes = 0;
    // Chunks of 128 tokens or more: the f16 rows of the next projection are written on a second stream while the kernels before it run (two buffers taken
    // in turn; an event per buffer says when it is filled, another when the product that read it is done).
    cudaStream_t side = nullptr;
    __half * rows_buf[2] = {nullptr, nullptr};
    cudaEvent_t rows_filled[2] = {nullptr, nullptr}, rows_freed[2] = {nullptr, nullptr};
    int rows_next = 0;
    bool rows_ahead = false;
    int * split_counters = nullptr; // one per 32 rows of h: rows written by the gate/up GEMV's blocks (zero between launches)
    // The norm between two projections of a decode step, folded into the producer (kernels.h, GemvNormLink): the projection that finishes the residual row
    // x leaves x * (the next norm's gains) split in xq2 and its blocks' sums of squares in norm_ss; the next projection takes both instead of reading,
    // normalizing and splitting x in every one of its blocks.
    uint8_t * xq2 = nullptr;
    float * norm_ss = nullptr;
    int * norm_counters = nullptr;  // one per 32 rows of x
    bool link_ready = false;        // xq2 / norm_ss describe the current x
    int link_blocks = 0;
    // All layers of a one-sequence decode step as one cooperative launch (kernels.h, "the fused decode step"), when the model's shapes allow it.
    cuda::DecodeLayersPlan * fused = nullptr;
    int32_t fused_slot = -1;        // the plan holds the cache pointers of this slot
    bool fused_refused = false;     // the shapes do not fit: do not ask again
    int32_t pos = 0;
    bool has_pending = false;
    // decode graph
    cudaGraphExec_t step_graph = nullptr;
    std::vector<cudaEvent_t> step_events;
    cudaEvent_t ev_a = nullptr, ev_b = nullptr;
    Timings tm;
    int64_t launches = 0;
    // profiling
    std::vector<CudaLlamaDecoder::KernelTime> * profile = nullptr;
    // tensor parallelism
    NcclApi nccl;
    NcclComm comm = nullptr;
    // decode steps, when asked for: the all-reduce + residual add as one kernel over peer memory (kernels/allreduce_peer.cu); prefill chunks and any
    // group where the peer mapping could not be set up use NCCL
    cuda::PeerAllReduce par{};
    bool use_par = false;
    void * par_inbox = nullptr, * par_flags = nullptr, * par_words = nullptr;
    std::vector<void *> par_opened;
    Status failed;   // the first device error; every later call returns it

    ~Impl() {
        if (stream) cudaStreamSynchronize(stream);
        if (side) { cudaStreamSynchronize(side); cudaStreamDestroy(side); }
        for (int i = 0; i < 2; i++) {
            if (rows_filled[i]) cudaEventDestroy(rows_filled[i]);
            if (rows_freed[i]) cudaEventDestroy(rows_freed[i]);
            if (rows_buf[i]) cudaFree(rows_buf[i]);
        }
        if (step_graph) cudaGraphExecDestroy(step_graph);      // a graph that holds captured NCCL work has to go before its communicator
        cuda::decode_layers_destroy(fused);
        for (auto & g : batch_graphs) cudaGraphExecDestroy(g.second);
        for (void * p : {(void *)b_rows, (void *)b_out, (void *)b_step, (void *)b_logits, (void *)b_part, b_argmax_part, (void *)b_counters, (void *)b_shares, (void *)rows16_all}) if (p) cudaFree(p);
        for (void * p : {(void *)h_rows, (void *)h_out}) if (p) cudaFreeHost(p);
        for (void * p : par_opened) cudaIpcCloseMemHandle(p);
        for (void * p : {par_inbox, par_flags, par_words}) if (p) cudaFree(p);
        if (sym_win) nccl.CommWindowDeregister(comm, sym_win);
        if (sym_base) { nccl.MemFree(sym_base); x = nullptr; red = nullptr; tp_pairs = nullptr; }
        if (comm) nccl.CommDestroy(comm);
        for (cudaEvent_t e : step_events) cudaEventDestroy(e);
        if (ev_a) cudaEventDestroy(ev_a);
        if (ev_b) cudaEventDestroy(ev_b);
        for (void * p : {(void *)weights, (void *)kc, (void *)vc, (void *)x, (void *)xn, (void *)qkv, (void *)attn, (void *)h, (void *)red, (void *)logits_buf, (void *)part, (void *)inv_freq, rope_cs, (void *)attn_counters, (void *)split_counters, (void *)xq2, (void *)norm_ss, (void *)norm_counters, (void *)tp_pairs, w16,
                         argmax_part, (void *)xq, (void *)xn16, (void *)attn16, (void *)h16, (void *)tokens, (void *)in_tokens, (void *)state}) {
            if (p) cudaFree(p);
        }
        for (void * p : {(void *)host_tokens, (void *)host_in, (void *)host_x, (void *)host_error}) if (p) cudaFreeHost(p);
        if (stream) cudaStreamDestroy(stream);
    }

    Status check(cudaError_t e, const char * what) {
        if (e == cudaSuccess) return Status();
        Status st = internal_error(cuda_msg(what, e));
        if (failed.is_ok()) failed = st;
        return st;
    }

    Status wait_idle() {
        if (!failed.is_ok()) return failed;
        DOOMS_RETURN_IF_ERROR(check(cudaStreamSynchronize(stream), "a CUDA kernel of the decoder failed"));
        if (host_error && *host_error != 0) {   // a kernel gave up on a bounded wait and said so
            const int32_t flag = *host_error;
            const char * what = flag == 2 ? "the prefill GEMM gave up waiting on its shared-memory pipeline"
                              : flag == 3 ? "the peer-memory all-reduce gave up waiting for another rank"
                              : flag == 4 ? "a decode GEMV gave up waiting for a tensor copy"
                              : flag == 5 ? "the batched decode step gave up waiting at a grid barrier"
                                          : "a kernel reported an internal inconsistency";
            failed = internal_error(std::string(what) + " (error flag " + std::to_string(flag) + ")");
            return failed;
        }
        return Status();
    }

    // Every launch goes through here: counted, and timed on its own when a profile is being taken.
    template <class F>
    void run(const char * kind, F && f) {
        if (!failed.is_ok()) return;
        if (profile) {
            cudaEventRecord(ev_a, stream);
            const cudaError_t e = f();
            cudaEventRecord(ev_b, stream);
            cudaEventSynchronize(ev_b);
            float ms = 0.f;
            cudaEventElapsedTime(&ms, ev_a, ev_b);
            (void)check(e, kind);
            for (auto & k : *profile) if (std::strcmp(k.kind, kind) == 0) { k.dispatches++; k.gpu_ms += ms; return; }
            profile->push_back({kind, 1, ms});
            return;
        }
        launches++;
        (void)check(f(), kind);
    }

    AttnShape attn_shape() const {
        return AttnShape{nh, nkv, cfg.head_dim, qkv_width, kv_width, attn_width, cfg.rope_neox ? 1 : 0, cfg.rope_base};
    }

    void all_reduce(float * buf, size_t count) {
        if (tp == 1) return;
        run("all_reduce", [&] { return nccl.AllReduce(buf, buf, count, NcclApi::kFloat32, NcclApi::kSum, comm, stream) == 0 ? cudaSuccess : cudaErrorUnknown; });
    }

    // the integer tensor-core GEMV takes q4_0 and q4_K rows
    bool fast(const MatDev & w) const {
        return (w.dt == DType::Q4_0 && cuda::gemv_q4_0_supported(w.ptr, w.rows, w.cols)) || (w.dt == DType::Q4_K && cuda::gemv_q4_k_supported(w.ptr, w.rows, w.cols));
    }
    // One-token projection of `in`, RMS-normalized with gamma first when gamma is given. The streaming kernels do the norm (and the q4_0 kernel the split of
    // its input into int8 limbs) in their prologue; only shapes they do not take go through a norm launch and the row-per-warp kernel. A producer that
    // already wrote the split of `in` (the attention merge) leaves it in xq and says so in xq_of.
    // The q4_0 kernel splits an f32 input in its prologue, every block for itself. That beats a launch of its own for the model-width inputs (with the norm
    // folded in); for the feed-forward-width input of ffn_down (3.5x longer) one split kernel ahead of the projection measured 0.2 ms per token faster on
    // the 8B shape, so long plain inputs are still split once, by a kernel.
    void prepare_fast_input(const float *& in, const float *& gamma, int64_t cols) {
        if (!gamma && xq_of != in && cols >= 8192) {
            run("split", [&] { return cuda::launch_quantize_x(in, cols, xq, stream); });
            xq_of = in;
        }
    }
    // next_gamma: the gains of the norm that the next projection applies to `out` (= x); given when that projection can take the norm from here.
    void matvec(const char * kind, const MatDev & w, const float * in, const float * gamma, float * out, const float * bias, uint32_t flags,
                const float * next_gamma = nullptr) {
        const bool writes_x = out == x;
        if (fast(w)) {
            const bool consume = gamma && in == x && link_ready;
            const bool produce = next_gamma && writes_x && tp == 1 && w.rows % 32 == 0 && norm_counters;
            if (!consume) prepare_fast_input(in, gamma, w.cols);
            const void * split = consume ? xq2 : (xq_of == in && !gamma) ? xq : nullptr;
            const cuda::GemvNormLink link{produce ? next_gamma : nullptr, produce ? norm_ss : nullptr, consume ? norm_ss : nullptr, consume ? link_blocks : 0};
            run(kind, [&] {
                return cuda::launch_gemv_q4_0(w.ptr, nullptr, split, in, consume ? nullptr : gamma, cfg.rms_eps, out, bias, w.rows, w.cols, flags, w.dt == DType::Q4_K, stream,
                                              produce ? xq2 : nullptr, produce ? norm_counters : nullptr, host_error, &link);
            });
            if (writes_x) { link_ready = produce; link_blocks = cuda::gemv_q4_0_blocks(w.rows, w.cols, false, w.dt == DType::Q4_K); }
            return;
        }
        if (writes_x) link_ready = false;
        if (w.dt == DType::Q6_K && cuda::gemv_q6_k_supported(w.ptr, w.rows, w.cols) && (!gamma || (in == x && cfg.n_embd % 32 == 0))) {
            // the integer tensor-core kernel for q6_K works on the split input: left by the norm, or made by one small kernel
            if (gamma) {
                norm(in, gamma, 1, true);
            } else if (xq_of != in) {
                run("split", [&] { return cuda::launch_quantize_x(in, w.cols, xq, stream); });
                xq_of = in;
            }
            run(kind, [&] { return cuda::launch_gemv_q6_k(w.ptr, xq, out, bias, w.rows, w.cols, flags, stream); });
            return;
        }
        if (cuda::gemv_blocks_supported(int(w.dt), w.ptr, in, w.rows, w.cols)) {
            run(kind, [&] { return cuda::launch_gemv_blocks(int(w.dt), w.ptr, nullptr, in, gamma, cfg.rms_eps, out, bias, w.rows, w.cols, flags, stream); });
            return;
        }
        if (gamma) { norm(in, gamma, 1, false); in = xn; }
        run(kind, [&] { return cuda::launch_matvec(int(w.dt), w.ptr, in, out, bias, w.rows, w.cols, flags, stream); });
    }
    // xn = RMS-normalized rows; with split (one row) the kernel also leaves the row split for the staged q4_0 kernels (every producer of a projection
    // input invalidates the split copy).
    void norm(const float * in, const float * gamma, int M, bool split, bool f16_only = false) {
        const bool do_split = split && M == 1 && cfg.n_embd % 32 == 0;
        run("norm", [&] {
            return cuda::launch_rms_norm(in, gamma, f16_only ? nullptr : xn, f16_only ? xn16 : nullptr, do_split ? xq : nullptr, M, cfg.n_embd, cfg.rms_eps, stream);
        });
        xq_of = do_split ? xn : nullptr;
    }
    void gate_up(const MatDev & wg, const MatDev & wu, const float * in, const float * gamma, float * out, bool down_takes_split) {
        if (fast(wg) && fast(wu)) {
            const bool consume = gamma && in == x && link_ready;
            if (!consume) prepare_fast_input(in, gamma, wg.cols);
            const void * split = consume ? xq2 : (xq_of == in && !gamma) ? xq : nullptr;
            const cuda::GemvNormLink link{nullptr, nullptr, consume ? norm_ss : nullptr, consume ? link_blocks : 0};
            // a result that the integer GEMV reads next (ffn_down) is left split by the blocks that complete its 32-row groups: no split launch, and no
            // split in the next kernel's prologue
            const bool split_out = down_takes_split && wg.rows % 32 == 0 && split_counters;
            run("gate_up", [&] {
                return cuda::launch_gemv_q4_0(wg.ptr, wu.ptr, split, in, consume ? nullptr : gamma, cfg.rms_eps, out, nullptr, wg.rows, wg.cols, 0u, wg.dt == DType::Q4_K, stream,
                                              split_out ? xq : nullptr, split_out ? split_counters : nullptr, host_error, &link);
            });
            xq_of = split_out ? out : nullptr;
            return;
        }
        if (cuda::gemv_blocks_supported(int(wg.dt), wg.ptr, in, wg.rows, wg.cols) && cuda::gemv_blocks_supported(int(wu.dt), wu.ptr, in, wu.rows, wu.cols)) {
            run("gate_up", [&] { return cuda::launch_gemv_blocks(int(wg.dt), wg.ptr, wu.ptr, in, gamma, cfg.rms_eps, out, nullptr, wg.rows, wg.cols, 0u, stream); });
            return;
        }
        if (gamma) { norm(in, gamma, 1, false); in = xn; }
        run("gate_up", [&] { return cuda::launch_gate_up(int(wg.dt), wg.ptr, wu.ptr, in, out, wg.rows, wg.cols, stream); });
    }
    void matmul(const char * kind, const MatDev & w, const MatDev * w2, const float * in, int64_t in_stride, float * out, int64_t out_stride, const float * bias, int M,
                uint32_t flags) {
        run(kind, [&] { return cuda::launch_matmul_tile(int(w.dt), w.ptr, w2 ? w2->ptr : nullptr, in, in_stride, out, out_stride, bias, M, w.rows, w.cols, flags, stream); });
    }
    // Causal attention of a chunk: flash attention on the tensor cores for head_dim 64 / 128 (the reference's attention_prefill), the CUDA-core kernel
    // otherwise, or when prefill_tile = 1 asks for the plain kernels.
    void prefill_attention(__half * kcl, __half * vcl, __half * out16, int M, const AttnShape & as) {
        if (cfg.prefill_tile != 1 && cuda::attention_flash_supported(as)) {
            run("attention", [&] { return cuda::launch_attention_flash(qkv, kcl, vcl, attn + attn_pad, out16 ? out16 + attn_pad : nullptr, state, M, as, stream); });
        } else {
            run("attention", [&] { return cuda::launch_attention_prefill(qkv, kcl, vcl, attn + attn_pad, out16 ? out16 + attn_pad : nullptr, state, M, as, stream); });
        }
    }
    // Y[m][row0 + n] (+)= X16[m] . W[n] on the tensor cores; X16 is the f16 activation buffer behind map.
    void gemm_tc(const char * kind, const MatDev & w, const MatDev * w2, const cuda::TensorMap & map, float * out, __half * out16, const float * bias, int M,
                 int64_t out_stride, int64_t out16_stride, uint32_t flags) {
        run(kind, [&] {
            return cuda::launch_gemm_tc(int(w.dt), w.ptr, w2 ? w2->ptr : nullptr, &map, out, out16, bias, M, w.rows, w.cols, out_stride, out16_stride, flags,
                                        host_error, stream, w16, w16_bytes);
        });
    }
    // Starts writing the f16 rows of w into the next of the two buffers, on the second stream, as soon as the product that last read that buffer is done.
    int rows_prefetch(const MatDev & w) {
        const int s = rows_next;
        rows_next ^= 1;
        cudaStreamWaitEvent(side, rows_freed[s], 0);
        run("dequant", [&] { return cuda::launch_dequant_rows16(int(w.dt), w.ptr, rows_buf[s], w.rows, w.cols, side); });
        cudaEventRecord(rows_filled[s], side);
        return s;
    }
    // The product on the rows that rows_prefetch put into buffer s.
    void gemm_from_rows(const char * kind, const MatDev & w, int s, const cuda::TensorMap & map, float * out, const float * bias, int M, int64_t out_stride, uint32_t flags) {
        cudaStreamWaitEvent(stream, rows_filled[s], 0);
        run(kind, [&] { return cuda::launch_gemm_tc_rows16(rows_buf[s], nullptr, &map, out, nullptr, bias, M, w.rows, w.cols, out_stride, 0, flags, host_error, stream); });
        cudaEventRecord(rows_freed[s], stream);
    }
    // x[m] += X16[m] . W[n] for the rows of a batched step. Few weight rows against one token tile would run on a handful of SMs, so the reduction
    // dimension is dealt over several blocks per tile where that pays; their sums are added onto x in a fixed order.
    void gemm_tc_into_x(const char * kind, const MatDev & w, const cuda::TensorMap & map, int M) {
        const int E = cfg.n_embd;
        int shares = 1;
        if (b_shares) shares = w.rows16 ? cuda::gemm_tc_rows16_k_splits(M, w.rows, w.cols) : cuda::gemm_tc_k_splits(int(w.dt), M, w.rows, w.cols, false, w16 ? w16_bytes : 0);
        if (shares <= 1 || shares > kMaxShares) { gemm_rows(kind, w, nullptr, map, x, nullptr, nullptr, M, E, 0, kFlagAccumulate); return; }
        const int64_t share_stride = int64_t(max_rows) * E;
        run(kind, [&] {
            if (w.rows16) {
                return cuda::launch_gemm_tc_rows16(w.rows16, nullptr, &map, b_shares, nullptr, nullptr, M, w.rows, w.cols, E, 0, 0u, host_error, stream, shares, share_stride);
            }
            return cuda::launch_gemm_tc(int(w.dt), w.ptr, nullptr, &map, b_shares, nullptr, nullptr, M, w.rows, w.cols, E, 0, 0u, host_error, stream, w16, w16_bytes, shares,
                                        share_stride);
        });
        run("residual", [&] { return cuda::launch_add_shares(x, b_shares, shares, int64_t(M) * E, share_stride, stream); });
    }
    // A projection of a batched step: from the decoder's f16 copy of the matrix when it keeps one, else as any chunk's.
    void gemm_rows(const char * kind, const MatDev & w, const MatDev * w2, const cuda::TensorMap & map, float * out, __half * out16, const float * bias, int M,
                   int64_t out_stride, int64_t out16_stride, uint32_t flags) {
        if (!w.rows16 || (w2 && !w2->rows16)) { gemm_tc(kind, w, w2, map, out, out16, bias, M, out_stride, out16_stride, flags); return; }
        run(kind, [&] {
            return cuda::launch_gemm_tc_rows16(w.rows16, w2 ? w2->rows16 : nullptr, &map, out, out16, bias, M, w.rows, w.cols, out_stride, out16_stride, flags, host_error, stream);
        });
    }
    // x += partial sums of the other ranks' shares: with one GPU the projection accumulated into x directly.
    void reduce_into_x(int M) {
        if (tp == 1) return;
        const size_t n = size_t(M) * size_t(cfg.n_embd);
        if (M == 1 && use_par) {
            run("all_reduce", [&] { return cuda::launch_allreduce_add(par, red, x, int(n), stream); });
            return;
        }
        if (M == 1 && (tp & (tp - 1)) == 0) {      // the projection already wrote x / tp + its share into x
            all_reduce(x, n);
            return;
        }
        all_reduce(red, n);
        run("residual", [&] { return cuda::launch_add(x, red, int64_t(n), stream); });
    }

    // Maps every rank's inbox and flags into this process (CUDA IPC handles exchanged with an NCCL all-gather) for the peer-memory all-reduce of the decode
    // steps. Any failure on any rank leaves the whole group on NCCL: the ranks agree on that with one more all-reduce.
    struct PeerHandles { cudaIpcMemHandle_t inbox, flags; };
    static size_t peer_setup_scratch_bytes(int ranks) { return sizeof(PeerHandles) * size_t(ranks) + 256; }
    // scratch: peer_setup_scratch_bytes(tp) of device memory, allocated by create() like every other buffer, so that no rank can leave before the
    // collectives below: each rank takes part in both of them whether or not its own setup worked.
    void setup_peer_allreduce(void * scratch) {
        using Handles = PeerHandles;
        const char * env = getenv("DOOMS_TP_ALLREDUCE");
        const int E = cfg.n_embd;
        // Opt-in (DOOMS_TP_ALLREDUCE=peer): on two B200s the 8B decode step measured 2.72 ms with it against 2.60 ms with NCCL's 16 KB all-reduce plus the
        // add kernel, so NCCL stays the default until this path is faster.
        bool ok = env && std::string(env) == "peer" && tp <= cuda::kPeerMaxRanks && E % 4 == 0 && (E + 1023) / 1024 <= cuda::kPeerMaxBlocks;
        std::vector<Handles> all(size_t(tp), Handles{});
        Handles * d_all = static_cast<Handles *>(scratch);
        float * d_ok = reinterpret_cast<float *>(static_cast<char *>(scratch) + sizeof(Handles) * size_t(tp));
        const size_t inbox_bytes = cuda::peer_allreduce_inbox_bytes(tp, E), flag_bytes = cuda::peer_allreduce_flag_bytes(tp);
        ok = ok && cudaMalloc(&par_inbox, inbox_bytes) == cudaSuccess && cudaMalloc(&par_flags, flag_bytes) == cudaSuccess && cudaMalloc(&par_words, 64) == cudaSuccess;
        ok = ok && cudaMemset(par_inbox, 0, inbox_bytes) == cudaSuccess && cudaMemset(par_flags, 0, flag_bytes) == cudaSuccess && cudaMemset(par_words, 0, 64) == cudaSuccess;
        ok = ok && cudaIpcGetMemHandle(&all[size_t(rank)].inbox, par_inbox) == cudaSuccess && cudaIpcGetMemHandle(&all[size_t(rank)].flags, par_flags) == cudaSuccess;
        (void)cudaGetLastError();
        cudaMemcpy(d_all + rank, &all[size_t(rank)], sizeof(Handles), cudaMemcpyHostToDevice);
        bool exchanged = nccl.AllGather(d_all + rank, d_all, sizeof(Handles), NcclApi::kInt8, comm, stream) == 0 && cudaStreamSynchronize(stream) == cudaSuccess;
        exchanged = exchanged && cudaMemcpy(all.data(), d_all, sizeof(Handles) * size_t(tp), cudaMemcpyDeviceToHost) == cudaSuccess;
        ok = ok && exchanged;
        if (ok) {
            for (int r = 0; r < tp && ok; r++) {
                if (r == rank) { par.inbox[r] = static_cast<float *>(par_inbox); par.flags[r] = static_cast<uint32_t *>(par_flags); continue; }
                void * pi = nullptr, * pf = nullptr;
                ok = cudaIpcOpenMemHandle(&pi, all[size_t(r)].inbox, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
                if (ok) par_opened.push_back(pi);
                ok = ok && cudaIpcOpenMemHandle(&pf, all[size_t(r)].flags, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
                if (ok) par_opened.push_back(pf);
                par.inbox[r] = static_cast<float *>(pi);
                par.flags[r] = static_cast<uint32_t *>(pf);
            }
        }
        cudaGetLastError();
        const float mine = ok ? 0.f : 1.f;
        float sum = 1.f;
        cudaMemcpy(d_ok, &mine, 4, cudaMemcpyHostToDevice);
        if (nccl.AllReduce(d_ok, d_ok, 1, NcclApi::kFloat32, NcclApi::kSum, comm, stream) == 0 && cudaStreamSynchronize(stream) == cudaSuccess) {
            cudaMemcpy(&sum, d_ok, 4, cudaMemcpyDeviceToHost);
        }
        par.round = static_cast<uint32_t *>(par_words);
        par.ticket = par.round + 1;
        par.state = state;
        par.host_error = host_error;
        par.rank = rank;
        par.n = tp;
        par.max_floats = E;
        use_par = sum == 0.f;
    }

    // The plan of the fused decode step for the selected slot, or nullptr when this model / option set runs kernel by kernel.
    cuda::DecodeLayersPlan * fused_plan() {
        // Opt-in (DOOMS_FUSED_STEP=1). Measured on B200 with the 8B shape it is the slower way today: 2.13 ms per token against 1.84 ms for the chain of
        // early-launched kernels. Stamps inside the kernel show where a layer's 64 us go: not into launches (there are none) but into what every phase
        // boundary costs however it is implemented: waiting at the barrier for the slowest block of the phase before (1.5 - 4 us of spread per phase),
        // 2.5 - 3 us of epilogue where a projection also splits its output and leaves the norm's sums, and the attention merge (4 us on eight blocks).
        static const bool on = [] { const char * e = getenv("DOOMS_FUSED_STEP"); return e && *e == '1'; }();
        if (!on || fused_refused || tp != 1 || !gqa || profile) return nullptr;
        if (fused && fused_slot == cur) return fused;
        cuda::decode_layers_destroy(fused);
        fused = nullptr;
        std::vector<cuda::FusedLayer> fl;
        for (size_t l = 0; l < layers.size(); l++) {
            const LayerDev & L = layers[l];
            bool ok = L.qkv.size() == 1 && fast(L.qkv[0].w);
            for (const MatDev * w : {&L.attn_output, &L.ffn_gate, &L.ffn_up, &L.ffn_down}) ok = ok && fast(*w);
            if (!ok) { fused_refused = true; return nullptr; }
            auto mat = [](const MatDev & w) { return cuda::FusedMatrix{w.ptr, w.rows, w.cols, w.dt == DType::Q4_K}; };
            const float * next = l + 1 < layers.size() ? layers[l + 1].attn_norm : output_norm;
            fl.push_back(cuda::FusedLayer{mat(L.qkv[0].w), mat(L.attn_output), mat(L.ffn_gate), mat(L.ffn_up), mat(L.ffn_down), L.attn_norm, L.ffn_norm, L.qkv_bias, next,
                                          kc + l * cache_layer_elems + size_t(cur) * slot_elems, vc + l * cache_layer_elems + size_t(cur) * slot_elems});
        }
        const cuda::FusedBuffers fb{x, qkv, attn, h, xq, xq2, norm_ss, norm_counters, split_counters, attn_counters, part, state, inv_freq, rope_cs, host_error, cfg.rms_eps,
                                    attn_shape(), gqa_splits};
        if (cuda::decode_layers_create(fl.data(), int(fl.size()), fb, &fused) != cudaSuccess) {
            (void)cudaGetLastError();
            fused = nullptr;
            fused_refused = true;
            return nullptr;
        }
        fused_slot = cur;
        return fused;
    }

    // All layers for M positions starting at state->pos whose input rows are in x; then the logits and the greedy token of the last row
    // (encode_forward, metal_llama_decoder.mm:311-385).
    void forward(int M, bool advance) {
        const int E = cfg.n_embd;
        int rows_slot = 0;
        const AttnShape as = attn_shape();
        const bool single = tp == 1;
        link_ready = false;      // x was just written by the embedding (or by the caller)
        // one position: its rotary angles are the same for every head of every layer
        cuda::DecodeLayersPlan * const one_launch = M == 1 ? fused_plan() : nullptr;
        if (M == 1 && gqa) {
            run("rope_table", [&] { return cuda::launch_rope_table(state, inv_freq, rope_cs, cfg.head_dim, stream, one_launch ? cuda::decode_layers_barrier(one_launch) : nullptr); });
        }
        if (one_launch) {
            run("layers", [&] { return cuda::launch_decode_layers(one_launch, stream); });
            link_ready = true;          // its last ffn_down prepared the output norm
            link_blocks = cuda::decode_layers_blocks(one_launch);
            xq_of = nullptr;
        }
        for (size_t l = 0; l < (one_launch ? 0 : layers.size()); l++) {
            const LayerDev & L = layers[l];
            __half * kcl = kc + l * cache_layer_elems + size_t(cur) * slot_elems, * vcl = vc + l * cache_layer_elems + size_t(cur) * slot_elems;
            // Tensor-parallel decode steps with a power-of-two group: the projection leaves x / tp + its share of the product in x, and the in-place all-reduce
            // of x is the residual add (no buffer for the partial sums, no add kernel). Chunks and other group sizes reduce a separate buffer and add it.
            const bool share = !single && M == 1 && !use_par && (tp & (tp - 1)) == 0;
            uint32_t log2_tp = 0;
            while ((1 << log2_tp) < tp) log2_tp++;
            float * o_dst = (single || share) ? x : red;
            // (under tensor parallelism the kernel after these projections is a collective: they do not let it start early)
            const uint32_t o_flags = single ? kFlagAccumulate : (share ? (kFlagAccumulate | (log2_tp << cuda::kFlagShareShift)) : 0u) | cuda::kFlagLateDependents;
            const bool use_tc = M > 1 && tc_capable && cfg.prefill_tile != 1;
            if (M > 1) norm(x, L.attn_norm, M, false, use_tc);
            if (M == 1) {
                for (const QkvPart & q : L.qkv) {
                    matvec("qkv", q.w, x, L.attn_norm, qkv + q.row0, L.qkv_bias ? L.qkv_bias + q.row0 : nullptr, L.qkv_bias ? kFlagBias : 0u);
                }
                // (a padded attention row is split by the projection itself: its zero columns are not the attention kernel's to write)
                const bool split_attn = fast(L.attn_output) && cfg.head_dim % 32 == 0 && (gqa || splits > 1) && attn_width == q_width;
                if (gqa) {
                    run("attention", [&] {
                        return cuda::launch_attention_gqa(qkv, kcl, vcl, part, state, inv_freq, 0, gqa_splits, as, attn_counters, attn + attn_pad, split_attn ? xq : nullptr, stream, rope_cs);
                    });
                } else {
                    run("rope_store", [&] { return cuda::launch_rope_store(qkv, kcl, vcl, state, inv_freq, 1, as, stream); });
                    run("attention", [&] { return cuda::launch_attention_decode(qkv, kcl, vcl, attn + attn_pad, part, split_attn ? xq : nullptr, state, 0, splits, as, stream); });
                }
                xq_of = split_attn ? attn : nullptr;
                // the projections that finish x also prepare the norm of the projection after them, when that one is a kernel that can take it
                const bool gate_up_takes = fast(L.ffn_gate) && fast(L.ffn_up);
                matvec("attn_output", L.attn_output, attn, nullptr, o_dst, nullptr, o_flags, gate_up_takes ? L.ffn_norm : nullptr);
                xq_of = nullptr;
                reduce_into_x(1);
                gate_up(L.ffn_gate, L.ffn_up, x, L.ffn_norm, h, fast(L.ffn_down));
                const float * after_gamma = nullptr;
                if (l + 1 < layers.size()) {
                    const LayerDev & N = layers[l + 1];
                    if (std::all_of(N.qkv.begin(), N.qkv.end(), [&](const QkvPart & q) { return fast(q.w); })) after_gamma = N.attn_norm;
                } else if (output.rows > 0 && fast(output)) {
                    after_gamma = output_norm;
                }
                matvec("ffn_down", L.ffn_down, h, nullptr, o_dst, nullptr, o_flags, after_gamma);
                reduce_into_x(1);
            } else if (use_tc && rows_ahead && M >= 128 && !profile) {
                // (the chunk's norm above wrote xn16) Every projection but the fused gate / up reads f16 rows that were written while the kernels before
                // it ran: the rows of attn_output during the qkv product, those of ffn_down during attention, the next layer's qkv during gate / up.
                if (l == 0) rows_slot = rows_prefetch(L.qkv[0].w);
                const int slot_qkv = rows_slot, slot_o = rows_prefetch(L.attn_output);
                gemm_from_rows("qkv", L.qkv[0].w, slot_qkv, map_xn, qkv, L.qkv_bias, M, qkv_width, L.qkv_bias ? kFlagBias : 0u);
                run("rope_store", [&] { return cuda::launch_rope_store(qkv, kcl, vcl, state, inv_freq, M, as, stream); });
                prefill_attention(kcl, vcl, attn16, M, as);
                const int slot_down = rows_prefetch(L.ffn_down);
                gemm_from_rows("attn_output", L.attn_output, slot_o, map_attn, o_dst, nullptr, M, E, o_flags);
                reduce_into_x(M);
                norm(x, L.ffn_norm, M, false, true);
                gemm_tc("gate_up", L.ffn_gate, &L.ffn_up, map_xn, nullptr, h16, nullptr, M, 0, ff, 0u);
                if (l + 1 < layers.size()) rows_slot = rows_prefetch(layers[l + 1].qkv[0].w);
                gemm_from_rows("ffn_down", L.ffn_down, slot_down, map_h, o_dst, nullptr, M, E, o_flags);
                reduce_into_x(M);
            } else if (use_tc) {
                // (the chunk's norm above wrote xn16)
                for (const QkvPart & q : L.qkv) {
                    gemm_tc("qkv", q.w, nullptr, map_xn, qkv + q.row0, nullptr, L.qkv_bias ? L.qkv_bias + q.row0 : nullptr, M, qkv_width, 0, L.qkv_bias ? kFlagBias : 0u);
                }
                run("rope_store", [&] { return cuda::launch_rope_store(qkv, kcl, vcl, state, inv_freq, M, as, stream); });
                prefill_attention(kcl, vcl, attn16, M, as);
                gemm_tc("attn_output", L.attn_output, nullptr, map_attn, o_dst, nullptr, nullptr, M, E, 0, o_flags);
                reduce_into_x(M);
                norm(x, L.ffn_norm, M, false, true);
                gemm_tc("gate_up", L.ffn_gate, &L.ffn_up, map_xn, nullptr, h16, nullptr, M, 0, ff, 0u);
                gemm_tc("ffn_down", L.ffn_down, nullptr, map_h, o_dst, nullptr, nullptr, M, E, 0, o_flags);
                reduce_into_x(M);
            } else {
                for (const QkvPart & q : L.qkv) {
                    matmul("qkv", q.w, nullptr, xn, E, qkv + q.row0, qkv_width, L.qkv_bias ? L.qkv_bias + q.row0 : nullptr, M, L.qkv_bias ? kFlagBias : 0u);
                }
                run("rope_store", [&] { return cuda::launch_rope_store(qkv, kcl, vcl, state, inv_freq, M, as, stream); });
                prefill_attention(kcl, vcl, nullptr, M, as);
                matmul("attn_output", L.attn_output, nullptr, attn, attn_width, o_dst, E, nullptr, M, o_flags);
                reduce_into_x(M);
                norm(x, L.ffn_norm, M, false);
                matmul("gate_up", L.ffn_gate, &L.ffn_up, xn, E, h, ff, nullptr, M, 0u);
                matmul("ffn_down", L.ffn_down, nullptr, h, ff, o_dst, E, nullptr, M, o_flags);
                reduce_into_x(M);
            }
        }
        // The logits of the last row only (metal_llama_decoder.mm:375).
        if (output.rows > 0) matvec("output", output, x + size_t(M - 1) * E, output_norm, logits_buf + vocab_row0, nullptr, 0u);
        if (tp > 1) {
            // every rank reduces its own rows to one (value, index) pair; 8 bytes per rank are gathered instead of the logits (those only in logits())
            run("argmax", [&] { return cuda::launch_argmax_local_pair(logits_buf + vocab_row0, vocab_rows, vocab_row0, tp_pairs + rank * 2, argmax_part, stream); });
            run("all_gather", [&] { return nccl.AllGather(tp_pairs + rank * 2, tp_pairs, 8, NcclApi::kInt8, comm, stream) == 0 ? cudaSuccess : cudaErrorUnknown; });
            run("argmax", [&] { return cuda::launch_argmax_pairs(tp_pairs, tp, tokens, host_tokens, state, advance ? 1 : 0, stream); });
            logits_gathered = false;
        } else {
            run("argmax", [&] { return cuda::launch_argmax(logits_buf, int64_t(vocab_stride) * tp, tokens, host_tokens, state, argmax_part, advance ? 1 : 0, stream); });
        }
    }

    void embed(const int32_t * ids, const int32_t * index, int rows) {
        run("embed", [&] { return cuda::launch_embed(int(token_embd.dt), token_embd.ptr, ids, index, x, rows, cfg.n_embd, stream); });
    }

    // One chunk whose rows are in x (or whose ids are in in_tokens); the last row's greedy token lands in tokens[0] (run_chunk, metal_llama_decoder.mm:402-414).
    void run_chunk(int rows, bool from_tokens) {
        run("state", [&] { return cuda::launch_set_state(state, pos, 0, 0, stream); });
        if (from_tokens) embed(in_tokens, nullptr, rows);
        forward(rows, false);
        pos += rows;
        has_pending = true;
    }

    // One decode step: embeds tokens[state->tok_in], writes its greedy token to tokens[state->tok_out], advances the state.
    void decode_step_launches() {
        embed(tokens, &state->tok_in, 1);
        forward(1, true);
    }

    Status ensure_step_graph() {
        if (step_graph && graph_slot != cur) {      // the captured launches point into another slot's cache
            DOOMS_RETURN_IF_ERROR(wait_idle());
            cudaGraphExecDestroy(step_graph);
            step_graph = nullptr;
        }
        if (step_graph || !opt.use_graphs) return Status();
        graph_slot = cur;
        (void)fused_plan();      // built (device allocations, copies) before the capture starts
        DOOMS_RETURN_IF_ERROR(wait_idle());
        const int64_t before = launches;
        cudaGraph_t graph = nullptr;
        DOOMS_RETURN_IF_ERROR(check(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture"));
        decode_step_launches();
        const cudaError_t e = cudaStreamEndCapture(stream, &graph);
        step_launches = launches - before;
        launches = before;
        if (!failed.is_ok()) { if (graph) cudaGraphDestroy(graph); return failed; }
        DOOMS_RETURN_IF_ERROR(check(e, "cudaStreamEndCapture"));
        const cudaError_t ie = cudaGraphInstantiate(&step_graph, graph, 0);
        cudaGraphDestroy(graph);
        return check(ie, "cudaGraphInstantiate");
    }
    int64_t step_launches = 0;

    // ---- one decode step for several slots (rows) at once: the chunk path's kernels with one row per sequence. Every row's token comes from and goes
    // to device memory (b_rows), so the same captured launches serve any set of slots. ----
    static constexpr int32_t kMaxBatchSteps = 256;
    cuda::BatchRows batch_rows() const { return cuda::BatchRows{b_rows, b_rows + max_rows, b_rows + 2 * max_rows, int64_t(slot_elems)}; }
    void batch_step_launches(int32_t n) {
        const cuda::BatchRows rows = batch_rows();
        const int E = cfg.n_embd;
        const AttnShape as = attn_shape();
        embed(rows.tok, nullptr, n);
        for (size_t l = 0; l < layers.size(); l++) {
            const LayerDev & L = layers[l];
            norm(x, L.attn_norm, n, false, true);
            for (const QkvPart & q : L.qkv) {
                gemm_rows("qkv", q.w, nullptr, map_xn, qkv + q.row0, nullptr, L.qkv_bias ? L.qkv_bias + q.row0 : nullptr, n, qkv_width, 0, L.qkv_bias ? kFlagBias : 0u);
            }
            run("attention", [&] {
                if (rows_tc) {
                    return cuda::launch_attention_rows_tc(qkv, kc + l * cache_layer_elems, vc + l * cache_layer_elems, b_part, inv_freq, b_splits, cfg.n_ctx, as, b_counters,
                                                          attn, attn16, rows, n, stream);
                }
                return cuda::launch_attention_gqa_rows(qkv, kc + l * cache_layer_elems, vc + l * cache_layer_elems, b_part, inv_freq, b_splits, as, b_counters, attn, attn16,
                                                       rows, n, stream);
            });
            gemm_tc_into_x("attn_output", L.attn_output, map_attn, n);
            norm(x, L.ffn_norm, n, false, true);
            gemm_rows("gate_up", L.ffn_gate, &L.ffn_up, map_xn, nullptr, h16, nullptr, n, 0, ff, 0u);
            gemm_tc_into_x("ffn_down", L.ffn_down, map_h, n);
        }
        norm(x, output_norm, n, false, true);
        gemm_rows("output", output, nullptr, map_xn, b_logits, nullptr, nullptr, n, cfg.n_vocab, 0, 0u);
        run("argmax", [&] { return cuda::launch_argmax_rows(b_logits, cfg.n_vocab, cfg.n_vocab, rows, n, b_out, b_step, b_argmax_part, stream); });
    }
    Result<cudaGraphExec_t> batch_graph(int32_t n) {
        for (auto & g : batch_graphs) if (g.first == n) return g.second;
        DOOMS_RETURN_IF_ERROR(wait_idle());
        const int64_t before = launches;
        cudaGraph_t graph = nullptr;
        DOOMS_RETURN_IF_ERROR(check(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture"));
        batch_step_launches(n);
        const cudaError_t e = cudaStreamEndCapture(stream, &graph);
        batch_step_launches_count = launches - before;
        launches = before;
        if (!failed.is_ok()) { if (graph) cudaGraphDestroy(graph); return failed; }
        DOOMS_RETURN_IF_ERROR(check(e, "cudaStreamEndCapture"));
        cudaGraphExec_t exec = nullptr;
        const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        DOOMS_RETURN_IF_ERROR(check(ie, "cudaGraphInstantiate"));
        batch_graphs.emplace_back(n, exec);
        return exec;
    }
    // The selected slot's state to and from its entry in seqs (the stream is idle).
    void stash_selected() { seqs[size_t(cur)] = Sequence{pos, has_pending, has_pending ? host_tokens[0] : 0}; }
    void restore_selected() {
        const Sequence & q = seqs[size_t(cur)];
        pos = q.pos;
        has_pending = q.has_pending;
        if (has_pending) {
            host_tokens[0] = q.pending;
            (void)check(cudaMemcpy(tokens, &q.pending, sizeof(int32_t), cudaMemcpyHostToDevice), "restoring the pending token");
        }
    }
    class StepWindow;
    template <class Stage> Status append_positions(int32_t n, bool from_tokens, Stage && stage);

    void queue_decode_step() {
        logits_gathered = tp == 1;
        if (step_graph) {
            launches += step_launches;
            (void)check(cudaGraphLaunch(step_graph, stream), "cudaGraphLaunch");
        } else {
            decode_step_launches();
        }
    }
};

namespace cuda {
cudaError_t launch_add(float * x, const float * y, int64_t n, cudaStream_t stream);
}

Result<TpShare> tp_share(const LlamaDecoderConfig & c, int32_t rank, int32_t tp, int64_t attn_block, int64_t ffn_block) {
    if (tp < 1 || rank < 0 || rank >= tp) return invalid_argument("tp_rank must be in [0, tp_size)");
    if (attn_block < 1 || ffn_block < 1) return invalid_argument("block sizes must be at least 1");
    if (c.n_head < 1 || c.n_head_kv < 1 || c.n_head % tp != 0 || c.n_head_kv % tp != 0) {
        return unsupported("tensor parallelism over " + std::to_string(tp) + " GPUs needs n_head and n_head_kv to be multiples of it");
    }
    const int64_t q_width = int64_t(c.n_head) * c.head_dim;
    if (c.n_ff % ffn_block != 0 || c.n_ff / ffn_block < tp || q_width % attn_block != 0) {
        return unsupported("tensor parallelism over " + std::to_string(tp) + " GPUs: n_ff has to be at least that many whole blocks of " + std::to_string(ffn_block) +
                           " columns, and the attention width whole blocks of " + std::to_string(attn_block));
    }
    TpShare s;
    s.q_rows = int64_t(c.n_head / tp) * c.head_dim;
    s.q_row0 = s.q_rows * rank;
    s.kv_rows = int64_t(c.n_head_kv / tp) * c.head_dim;
    s.kv_row0 = s.kv_rows * rank;
    const int64_t units = c.n_ff / ffn_block, each = units / tp, more = units % tp;
    s.ff_row0 = (each * rank + std::min<int64_t>(rank, more)) * ffn_block;
    s.ff_rows = (each + (rank < more ? 1 : 0)) * ffn_block;
    s.attn_col0 = s.q_row0 / attn_block * attn_block;
    s.attn_cols = (s.q_row0 + s.q_rows + attn_block - 1) / attn_block * attn_block - s.attn_col0;
    const int64_t stride = (int64_t(c.n_vocab) + tp - 1) / tp;
    s.vocab_row0 = stride * rank;
    s.vocab_rows = std::max<int64_t>(0, std::min<int64_t>(stride, int64_t(c.n_vocab) - s.vocab_row0));
    return s;
}

CudaLlamaDecoder::CudaLlamaDecoder(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
CudaLlamaDecoder::~CudaLlamaDecoder() = default;

const LlamaDecoderConfig & CudaLlamaDecoder::config() const { return impl_->cfg; }
int32_t CudaLlamaDecoder::position() const { return impl_->pos; }
CudaLlamaDecoder::Timings CudaLlamaDecoder::timings() const { return impl_->tm; }

Result<std::unique_ptr<CudaLlamaDecoder>> CudaLlamaDecoder::create(const LlamaDecoderConfig & c, const LlamaDecoderWeights & w, const CudaOptions & opt) {
    DOOMS_RETURN_IF_ERROR(validate_model(c, w));      // validate.cpp: configuration ranges, every tensor's shape and type, in the contract's order
    if (opt.tp_size < 1 || opt.tp_rank < 0 || opt.tp_rank >= opt.tp_size) return invalid_argument("CUDA options: tp_rank has to lie in [0, tp_size)");
    const int64_t E = c.n_embd, F = c.n_ff, V = c.n_vocab, Qw = int64_t(c.n_head) * c.head_dim, KVw = int64_t(c.n_head_kv) * c.head_dim;

    // This rank's share under tensor parallelism: whole heads, and column shards that are whole blocks of the coarsest format any layer uses.
    const int tp = opt.tp_size;
    int64_t attn_block = 1, ffn_block = 1;
    for (const LlamaLayerWeights & L : w.layers) {
        attn_block = std::max<int64_t>(attn_block, dtype_block_elems(L.attn_output.dtype));
        ffn_block = std::max<int64_t>(ffn_block, dtype_block_elems(L.ffn_down.dtype));
    }
    const Result<TpShare> share = tp == 1 ? tp_share(c, 0, 1) : tp_share(c, opt.tp_rank, tp, attn_block, ffn_block);
    if (!share.is_ok()) return share.status();
    const int64_t attn_pad = share.value().q_row0 - share.value().attn_col0;
    if (attn_pad % 8 != 0) return unsupported("tensor parallelism: a rank's heads start " + std::to_string(attn_pad) + " columns into a block of attn_output; multiples of 8 are taken");

    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev < 1) { (void)cudaGetLastError(); return unsupported("no CUDA device"); }
    if (opt.device < 0 || opt.device >= n_dev) return invalid_argument("CUDA device " + std::to_string(opt.device) + " does not exist");
    if (cudaSetDevice(opt.device) != cudaSuccess) return unsupported(cuda_msg("cannot use the CUDA device", cudaGetLastError()));
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, opt.device) != cudaSuccess) return unsupported("cannot query the CUDA device");
    if (prop.major != 10) return unsupported(std::string("the kernels are built for sm_100a (B200); device is ") + prop.name);

    auto impl = std::make_unique<Impl>();
    Impl & m = *impl;
    m.cfg = c;
    m.opt = opt;
    m.tp = tp;
    m.rank = opt.tp_rank;
    m.nh = c.n_head / tp;
    m.nkv = c.n_head_kv / tp;
    m.q_width = m.nh * c.head_dim;
    m.kv_width = m.nkv * c.head_dim;
    m.qkv_width = m.q_width + 2 * m.kv_width;
    m.ff = int32_t(share.value().ff_rows);
    m.attn_width = int32_t(share.value().attn_cols);
    m.attn_pad = int32_t(attn_pad);
    m.vocab_stride = int32_t((V + tp - 1) / tp);
    m.vocab_row0 = int32_t(share.value().vocab_row0);
    m.vocab_rows = int32_t(share.value().vocab_rows);

    if (opt.operand_bf16) return unsupported("bf16 prefill operands are not built: the tensor-core tiles hold f16 operands, the reference's rounding");
    if (cudaStreamCreateWithFlags(&m.stream, cudaStreamNonBlocking) != cudaSuccess) return internal_error(cuda_msg("cudaStreamCreate", cudaGetLastError()));
    cudaEventCreate(&m.ev_a);
    cudaEventCreate(&m.ev_b);

    if (tp > 1) {
        if (!opt.nccl_unique_id) return invalid_argument("tp_size > 1 needs the group's nccl_unique_id");
        DOOMS_RETURN_IF_ERROR(load_nccl(opt.nccl_library, &m.nccl));
        NcclUniqueId id;
        std::memcpy(&id, opt.nccl_unique_id, sizeof id);
        const int rc = m.nccl.CommInitRank(&m.comm, tp, id, m.rank);
        if (rc != 0) return internal_error(std::string("ncclCommInitRank: ") + m.nccl.GetErrorString(rc));
    }

    // ---- the packed weight buffer: matrices as they are in the file (this rank's rows / column blocks), norms and biases as f32 ----
    struct Piece { const WeightRef * src; int64_t row0, rows, col0, cols; };   // a slice of a host tensor
    struct Plan { size_t off; std::vector<Piece> pieces; bool vector; };
    std::vector<Plan> plans;
    size_t total = 0;
    auto reserve = [&](size_t bytes) { const size_t off = total; total = align_up(total + bytes, kWeightAlign); return off; };
    auto piece_bytes = [](const Piece & p) { return size_t(p.rows) * size_t(dtype_bytes(p.src->dtype, p.cols).value()); };
    auto plan_mat = [&](std::vector<Piece> pieces, MatDev * out) {
        size_t bytes = 0;
        int64_t rows = 0;
        for (const Piece & p : pieces) { bytes += piece_bytes(p); rows += p.rows; }
        const size_t off = reserve(bytes);
        out->ptr = reinterpret_cast<const uint8_t *>(off);   // an offset until the buffer exists
        out->dt = pieces[0].src->dtype;
        out->rows = rows;
        out->cols = pieces[0].cols;
        m.matrix_bytes += bytes;
        plans.push_back({off, std::move(pieces), false});
    };
    auto plan_vec = [&](std::vector<Piece> pieces, const float ** out) {
        int64_t n = 0;
        for (const Piece & p : pieces) n += p.cols;
        const size_t off = reserve(size_t(n) * sizeof(float));
        *out = reinterpret_cast<const float *>(off);
        plans.push_back({off, std::move(pieces), true});
    };
    auto whole = [](const WeightRef & r) { return Piece{&r, 0, r.rows, 0, r.cols}; };
    auto rows_of = [](const WeightRef & r, int64_t row0, int64_t rows) { return Piece{&r, row0, rows, 0, r.cols}; };
    auto cols_of = [](const WeightRef & r, int64_t col0, int64_t cols) { return Piece{&r, 0, r.rows, col0, cols}; };

    plan_mat({whole(w.token_embd)}, &m.token_embd);
    const bool tied = w.output.data == w.token_embd.data && w.output.dtype == w.token_embd.dtype;
    if (tied) {
        m.output = m.token_embd;   // the rank's vocabulary rows are addressed inside the table below
    } else if (m.vocab_rows > 0) {
        plan_mat({rows_of(w.output, m.vocab_row0, m.vocab_rows)}, &m.output);
    }
    plan_vec({whole(w.output_norm)}, &m.output_norm);
    m.layers.resize(size_t(c.n_layer));
    const int64_t ql = m.q_width, kvl = m.kv_width, q0 = int64_t(m.rank) * ql, kv0 = int64_t(m.rank) * kvl;
    for (int32_t l = 0; l < c.n_layer; l++) {
        const LlamaLayerWeights & L = w.layers[size_t(l)];
        LayerDev & o = m.layers[size_t(l)];
        plan_vec({whole(L.attn_norm)}, &o.attn_norm);
        if (L.attn_qkv.data) {
            QkvPart p;
            plan_mat({rows_of(L.attn_qkv, q0, ql), rows_of(L.attn_qkv, Qw + kv0, kvl), rows_of(L.attn_qkv, Qw + KVw + kv0, kvl)}, &p.w);
            o.qkv.push_back(p);
        } else if (L.attn_q.dtype == L.attn_k.dtype && L.attn_k.dtype == L.attn_v.dtype) {
            QkvPart p;
            plan_mat({rows_of(L.attn_q, q0, ql), rows_of(L.attn_k, kv0, kvl), rows_of(L.attn_v, kv0, kvl)}, &p.w);
            o.qkv.push_back(p);
        } else {
            QkvPart a, b, d;
            plan_mat({rows_of(L.attn_q, q0, ql)}, &a.w);
            plan_mat({rows_of(L.attn_k, kv0, kvl)}, &b.w);
            plan_mat({rows_of(L.attn_v, kv0, kvl)}, &d.w);
            a.row0 = 0; b.row0 = int32_t(ql); d.row0 = int32_t(ql + kvl);
            o.qkv.push_back(a); o.qkv.push_back(b); o.qkv.push_back(d);
        }
        if (L.attn_qkv_bias.data) {
            plan_vec({cols_of(L.attn_qkv_bias, q0, ql), cols_of(L.attn_qkv_bias, Qw + kv0, kvl), cols_of(L.attn_qkv_bias, Qw + KVw + kv0, kvl)}, &o.qkv_bias);
        } else if (L.attn_q_bias.data) {
            plan_vec({cols_of(L.attn_q_bias, q0, ql), cols_of(L.attn_k_bias, kv0, kvl), cols_of(L.attn_v_bias, kv0, kvl)}, &o.qkv_bias);
        }
        plan_mat({cols_of(L.attn_output, share.value().attn_col0, m.attn_width)}, &o.attn_output);
        plan_vec({whole(L.ffn_norm)}, &o.ffn_norm);
        plan_mat({rows_of(L.ffn_gate, share.value().ff_row0, m.ff)}, &o.ffn_gate);
        plan_mat({rows_of(L.ffn_up, share.value().ff_row0, m.ff)}, &o.ffn_up);
        plan_mat({cols_of(L.ffn_down, share.value().ff_row0, m.ff)}, &o.ffn_down);
    }
    total += kWeightTail;
    m.weight_bytes = total;

    auto dev_alloc = [&](void ** p, size_t bytes, const char * what) -> Status {
        const cudaError_t e = cudaMalloc(p, std::max<size_t>(bytes, 16));
        if (e != cudaSuccess) { (void)cudaGetLastError(); return resource_exhausted(std::string("could not allocate ") + std::to_string(bytes) + " bytes for " + what); }
        return Status();
    };
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.weights), total, "the decoder weights"));
    cudaMemset(m.weights + total - kWeightTail, 0, kWeightTail);
    auto fix = [&](MatDev & d) { d.ptr = m.weights + reinterpret_cast<size_t>(d.ptr); };
    auto fixv = [&](const float *& p) { p = reinterpret_cast<const float *>(m.weights + reinterpret_cast<size_t>(p)); };
    fix(m.token_embd);
    if (tied) {
        m.output = m.token_embd;
        m.output.ptr += size_t(m.vocab_row0) * size_t(dtype_bytes(m.output.dt, E).value());
        m.output.rows = m.vocab_rows;
    } else if (m.vocab_rows > 0) fix(m.output);
    fixv(m.output_norm);
    for (LayerDev & o : m.layers) {
        fixv(o.attn_norm); fixv(o.ffn_norm);
        if (o.qkv_bias) fixv(o.qkv_bias);
        for (QkvPart & p : o.qkv) fix(p.w);
        fix(o.attn_output); fix(o.ffn_gate); fix(o.ffn_up); fix(o.ffn_down);
    }
    // qkv_bias == offset 0 cannot happen (token_embd is first), so a null pointer still means "no bias".

    std::vector<float> vec_tmp;
    for (const Plan & pl : plans) {
        uint8_t * dst = m.weights + pl.off;
        for (const Piece & p : pl.pieces) {
            const WeightRef & r = *p.src;
            cudaError_t e = cudaSuccess;
            if (pl.vector) {
                vec_tmp.resize(size_t(p.cols));
                for (int64_t i = 0; i < p.cols; i++) {
                    const uint8_t * s = static_cast<const uint8_t *>(r.data);
                    if (r.dtype == DType::F32) std::memcpy(&vec_tmp[size_t(i)], s + (p.col0 + i) * 4, 4);
                    else { uint16_t hb; std::memcpy(&hb, s + (p.col0 + i) * 2, 2); vec_tmp[size_t(i)] = half_bits_to_float(hb); }
                }
                e = cudaMemcpy(dst, vec_tmp.data(), size_t(p.cols) * 4, cudaMemcpyHostToDevice);
                dst += size_t(p.cols) * 4;
            } else {
                const size_t src_row = size_t(dtype_bytes(r.dtype, r.cols).value()), width = size_t(dtype_bytes(r.dtype, p.cols).value());
                const size_t col_off = size_t(dtype_bytes(r.dtype, p.col0).value());
                const uint8_t * s = static_cast<const uint8_t *>(r.data) + size_t(p.row0) * src_row + col_off;
                if (width == src_row) e = cudaMemcpy(dst, s, width * size_t(p.rows), cudaMemcpyHostToDevice);
                else e = cudaMemcpy2D(dst, width, s, src_row, width, size_t(p.rows), cudaMemcpyHostToDevice);
                dst += width * size_t(p.rows);
            }
            if (e != cudaSuccess) return internal_error(cuda_msg("copying the weights to the device", e));
        }
    }

    // ---- activations for the largest chunk, the KV cache, the logits and the token ring ----
    const size_t B = size_t(c.n_batch);
    const int32_t n_seq = std::max(1, opt.max_sequences);
    m.seqs.assign(size_t(n_seq), Impl::Sequence{});
    m.slot_elems = size_t(c.n_ctx) * size_t(m.kv_width);
    m.cache_layer_elems = size_t(n_seq) * m.slot_elems;
    m.kv_bytes = 2 * size_t(c.n_layer) * m.cache_layer_elems * sizeof(__half);
    m.splits = cuda::attention_splits(m.nh, c.n_ctx);
    m.gqa = cuda::attention_gqa_supported(m.attn_shape());
    {
        const char * e = getenv("DOOMS_ROWS_TC");
        m.rows_tc = cuda::attention_rows_tc_supported(m.attn_shape()) && !(e && *e == '0');
    }
    m.gqa_splits = cuda::attention_gqa_splits(m.nkv, c.n_ctx);
    const size_t part_floats = size_t(std::max(m.splits, m.gqa_splits)) * size_t(m.nh) * size_t(2 + c.head_dim);
    const size_t logits_floats = size_t(m.vocab_stride) * size_t(tp);
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.kc), m.kv_bytes / 2, "the key cache"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.vc), m.kv_bytes / 2, "the value cache"));
    if (tp > 1) {
        // The buffers the ranks reduce and gather: from NCCL's allocator, registered as one symmetric window, so that the 16 KB all-reduces of a decode step
        // run NCCL's low-latency kernels (DOOMS_TP_SYMMETRIC=0: plain device memory). Every rank takes the same branch: the registration is collective, and
        // whether the library has the entry points is the same for all of them.
        const char * sym = getenv("DOOMS_TP_SYMMETRIC");
        const size_t row_bytes = (B * size_t(E) * 4 + NcclApi::kWinAlignment - 1) & ~(NcclApi::kWinAlignment - 1);
        const size_t sym_bytes = 2 * row_bytes + NcclApi::kWinAlignment;
        if (m.nccl.has_windows() && !(sym && *sym == '0') && m.nccl.MemAlloc(&m.sym_base, sym_bytes) == 0 && m.sym_base) {
            if (m.nccl.CommWindowRegister(m.comm, m.sym_base, sym_bytes, &m.sym_win, NcclApi::kWinCollSymmetric) != 0) m.sym_win = nullptr;
            cudaMemset(m.sym_base, 0, sym_bytes);
            m.x = static_cast<float *>(m.sym_base);
            m.red = reinterpret_cast<float *>(static_cast<char *>(m.sym_base) + row_bytes);
            m.tp_pairs = reinterpret_cast<int32_t *>(static_cast<char *>(m.sym_base) + 2 * row_bytes);
        } else {
            m.sym_base = nullptr;
            (void)cudaGetLastError();
        }
    }
    if (!m.x) DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.x), B * size_t(E) * 4, "the residual rows"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.xn), B * size_t(E) * 4, "the normalized rows"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.qkv), B * size_t(m.qkv_width) * 4, "the q/k/v rows"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.attn), B * size_t(m.attn_width) * 4, "the attention rows"));
    cudaMemset(m.attn, 0, B * size_t(m.attn_width) * 4);
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.h), B * size_t(m.ff) * 4, "the feed-forward rows"));
    if (tp > 1 && !m.red) DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.red), B * size_t(E) * 4, "the all-reduce rows"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.logits_buf), logits_floats * 4, "the logits"));
    if (tp > 1 && !m.tp_pairs) DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.tp_pairs), size_t(tp) * 8, "the ranks' argmax pairs"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.part), part_floats * 4, "the attention partial results"));
    {
        std::vector<double> freq(size_t(c.head_dim / 2));
        for (size_t i = 0; i < freq.size(); i++) freq[i] = std::pow(double(c.rope_base), -2.0 * double(i) / double(c.head_dim));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.inv_freq), freq.size() * sizeof(double), "the rotary frequencies"));
        if (cudaMemcpy(m.inv_freq, freq.data(), freq.size() * sizeof(double), cudaMemcpyHostToDevice) != cudaSuccess) return internal_error("copying the rotary frequencies");
        DOOMS_RETURN_IF_ERROR(dev_alloc(&m.rope_cs, freq.size() * 2 * sizeof(float), "the rotary table of a decode step"));
    }
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.attn_counters), size_t(std::max(1, m.nkv)) * sizeof(int), "the attention counters"));
    cudaMemset(m.attn_counters, 0, size_t(std::max(1, m.nkv)) * sizeof(int));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.split_counters), (size_t(m.ff) / 32 + 1) * sizeof(int), "the split counters"));
    cudaMemset(m.split_counters, 0, (size_t(m.ff) / 32 + 1) * sizeof(int));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.xq2), cuda::quantized_x_bytes(E) + 64, "the split residual row"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.norm_ss), 4096 * sizeof(float), "the sums of squares of the residual row"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.norm_counters), (size_t(E) / 32 + 1) * sizeof(int), "the residual split counters"));
    cudaMemset(m.norm_counters, 0, (size_t(E) / 32 + 1) * sizeof(int));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.xq), cuda::quantized_x_bytes(std::max<int64_t>({E, int64_t(m.ff), int64_t(m.attn_width)})) + 64,
                                    "the split projection input"));
    if (E % 64 == 0 && m.attn_width % 64 == 0 && m.ff % 64 == 0) {
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.xn16), B * size_t(E) * 2, "the f16 normalized rows"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.attn16), B * size_t(m.attn_width) * 2, "the f16 attention rows"));
        cudaMemset(m.attn16, 0, B * size_t(m.attn_width) * 2);
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.h16), B * size_t(m.ff) * 2, "the f16 feed-forward rows"));
        m.tc_capable = cuda::make_activation_map(&m.map_xn, m.xn16, int64_t(B), E) == cudaSuccess &&
                       cuda::make_activation_map(&m.map_attn, m.attn16, int64_t(B), m.attn_width) == cudaSuccess &&
                       cuda::make_activation_map(&m.map_h, m.h16, int64_t(B), m.ff) == cudaSuccess;
        size_t largest = 0;
        for (const LayerDev & L : m.layers) {
            for (const QkvPart & q : L.qkv) largest = std::max(largest, size_t(q.w.rows) * size_t(q.w.cols) * 2);
            largest = std::max({largest, size_t(L.attn_output.rows) * size_t(L.attn_output.cols) * 2, size_t(L.ffn_down.rows) * size_t(L.ffn_down.cols) * 2,
                                size_t(L.ffn_gate.rows) * size_t(L.ffn_gate.cols) * 4});
        }
        if (B >= 128 && largest > 0 && cudaMalloc(&m.w16, largest) == cudaSuccess) m.w16_bytes = largest;      // optional: without it the GEMM dequantizes per tile
        else { (void)cudaGetLastError(); m.w16 = nullptr; }
        {
            // the two buffers of the rows written ahead: when every layer has one qkv matrix and none of these matrices is f16 already
            size_t single = 0;
            bool all = B >= 128 && m.w16 != nullptr;
            for (const LayerDev & L : m.layers) {
                all = all && L.qkv.size() == 1;
                for (const MatDev * w : {L.qkv.empty() ? &L.attn_output : &L.qkv[0].w, &L.attn_output, &L.ffn_down}) {
                    all = all && w->dt != DType::F16;
                    single = std::max(single, size_t(w->rows) * size_t(w->cols) * 2);
                }
            }
            const char * ahead = getenv("DOOMS_PREFILL_ROWS_AHEAD");
            if (all && single > 0 && !(ahead && *ahead == '0') && cudaStreamCreateWithFlags(&m.side, cudaStreamNonBlocking) == cudaSuccess) {
                bool ok = true;
                for (int i = 0; i < 2; i++) {
                    ok = ok && cudaMalloc(reinterpret_cast<void **>(&m.rows_buf[i]), single) == cudaSuccess;
                    ok = ok && cudaEventCreateWithFlags(&m.rows_filled[i], cudaEventDisableTiming) == cudaSuccess;
                    ok = ok && cudaEventCreateWithFlags(&m.rows_freed[i], cudaEventDisableTiming) == cudaSuccess;
                }
                m.rows_ahead = ok;
            }
            (void)cudaGetLastError();
        }
        for (const LayerDev & L : m.layers) {
            for (const QkvPart & q : L.qkv) m.tc_capable = m.tc_capable && cuda::gemm_tc_supported(int(q.w.dt), q.w.ptr, q.w.rows, q.w.cols);
            for (const MatDev * w : {&L.attn_output, &L.ffn_gate, &L.ffn_up, &L.ffn_down}) {
                m.tc_capable = m.tc_capable && cuda::gemm_tc_supported(int(w->dt), w->ptr, w->rows, w->cols);
            }
        }
    }
    DOOMS_RETURN_IF_ERROR(dev_alloc(&m.argmax_part, size_t(cuda::argmax_blocks(int64_t(logits_floats))) * 8, "the argmax partial results"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.tokens), (size_t(c.n_ctx) + 2) * 4, "the token ring"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.in_tokens), B * 4, "the input tokens"));
    DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.state), sizeof(DevState), "the position state"));
    cudaMemset(m.state, 0, sizeof(DevState));
    cudaMemset(m.tokens, 0, (size_t(c.n_ctx) + 2) * 4);
    {   // vocabulary padding rows (tp does not divide n_vocab) never win the argmax
        std::vector<float> ninf(logits_floats, -INFINITY);
        cudaMemcpy(m.logits_buf, ninf.data(), logits_floats * 4, cudaMemcpyHostToDevice);
    }
    if (cudaHostAlloc(reinterpret_cast<void **>(&m.host_tokens), (size_t(c.n_ctx) + 2) * 4, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void **>(&m.host_in), B * 4, cudaHostAllocDefault) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void **>(&m.host_error), 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void **>(&m.host_x), B * size_t(E) * 4, cudaHostAllocDefault) != cudaSuccess) {
        (void)cudaGetLastError();
        return resource_exhausted("could not allocate pinned host memory for the decoder");
    }
    *m.host_error = 0;
    // a decode step over several slots needs the tensor-core chunk path, the grouped-query attention kernel and the whole model on this GPU
    m.max_rows = (n_seq > 1 && tp == 1 && m.tc_capable && m.gqa && cuda::gemm_tc_supported(int(m.output.dt), m.output.ptr, m.output.rows, m.output.cols))
                     ? std::min<int32_t>({n_seq, c.n_batch, 1024}) : 0;
    if (m.max_rows > 0) {
        const size_t R = size_t(m.max_rows);
        // Rows attend over very different lengths (a fresh sequence beside one at the end of its context), so a row is cut into ranges of a fixed number of
        // positions, which bounds what one block does and lets the long rows spread over many SMs; a short row's later ranges are empty and leave at once.
        // 1024 positions measured best on 256 rows of 32 .. 4096 positions (4.23 ms per step; 512: 4.48, 256: 5.14).
        static const int range = [] { const char * e = getenv("DOOMS_ROWS_RANGE"); return e ? std::max(64, atoi(e)) : 1024; }();
        m.b_splits = std::max(1, std::min(64, (c.n_ctx + range - 1) / range));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_rows), 3 * R * sizeof(int32_t), "the rows of a batched decode step"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_out), size_t(Impl::kMaxBatchSteps) * R * sizeof(int32_t), "the tokens of a batched decode call"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_step), sizeof(int32_t), "the step counter"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_logits), R * size_t(c.n_vocab) * sizeof(float), "the logits of a batched decode step"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_part), R * size_t(m.b_splits) * size_t(m.nh) * size_t(2 + c.head_dim) * sizeof(float), "the batched attention partial results"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(&m.b_argmax_part, R * size_t(cuda::argmax_blocks(c.n_vocab)) * 8, "the batched argmax partial results"));
        DOOMS_RETURN_IF_ERROR(dev_alloc(reinterpret_cast<void **>(&m.b_counters), R * size_t(m.nkv) * sizeof(int), "the batched attention counters"));
        if (cudaMalloc(reinterpret_cast<void **>(&m.b_shares), size_t(Impl::kMaxShares) * R * size_t(E) * sizeof(float)) != cudaSuccess) {      // optional
            (void)cudaGetLastError();
            m.b_shares = nullptr;
        }
        // Batched steps run every projection from f16 rows. A copy of the matrices in that form, made once, saves dequantizing them in every step (11 % of
        // a 256-row step on the 0.5B shape); it is kept when it takes at most a quarter of the memory that is still free (DOOMS_BATCH_F16_ROWS=0: never).
        std::vector<MatDev *> mats;
        for (LayerDev & L : m.layers) {
            for (QkvPart & q : L.qkv) mats.push_back(&q.w);
            for (MatDev * w : {&L.attn_output, &L.ffn_gate, &L.ffn_up, &L.ffn_down}) mats.push_back(w);
        }
        mats.push_back(&m.output);
        size_t halves = 0;
        for (const MatDev * w : mats) halves += (size_t(w->rows) * size_t(w->cols) + 127) & ~size_t(127);
        size_t free_bytes = 0, total_bytes = 0;
        const char * keep = getenv("DOOMS_BATCH_F16_ROWS");
        if (!(keep && *keep == '0') && cudaMemGetInfo(&free_bytes, &total_bytes) == cudaSuccess && halves * 2 <= free_bytes / 4 &&
            cudaMalloc(reinterpret_cast<void **>(&m.rows16_all), halves * 2) == cudaSuccess) {
            size_t at = 0;
            bool ok = true;
            for (MatDev * w : mats) {
                if (w->dt == DType::F16) continue;      // (f16 matrices are their own f16 rows; they stay on the path of any chunk)
                __half * dst = m.rows16_all + at;
                ok = ok && cuda::launch_dequant_rows16(int(w->dt), w->ptr, dst, w->rows, w->cols, m.stream) == cudaSuccess;
                w->rows16 = dst;
                at += (size_t(w->rows) * size_t(w->cols) + 127) & ~size_t(127);
            }
            if (!ok || cudaStreamSynchronize(m.stream) != cudaSuccess) {
                (void)cudaGetLastError();
                for (MatDev * w : mats) w->rows16 = nullptr;
                cudaFree(m.rows16_all);
                m.rows16_all = nullptr;
            }
        } else {
            (void)cudaGetLastError();
        }
        cudaMemset(m.b_counters, 0, R * size_t(m.nkv) * sizeof(int));
        if (cudaHostAlloc(reinterpret_cast<void **>(&m.h_rows), 3 * R * sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess ||
            cudaHostAlloc(reinterpret_cast<void **>(&m.h_out), size_t(Impl::kMaxBatchSteps) * R * sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess) {
            (void)cudaGetLastError();
            return resource_exhausted("could not allocate pinned host memory for the batched decode step");
        }
    }
    if (tp > 1) {
        void * scratch = nullptr;
        DOOMS_RETURN_IF_ERROR(dev_alloc(&scratch, Impl::peer_setup_scratch_bytes(tp), "the exchange of the ranks' memory handles"));
        m.setup_peer_allreduce(scratch);
        cudaFree(scratch);
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return internal_error(cuda_msg("setting up the decoder", cudaGetLastError()));
    m.tm.tp_peer_allreduce = m.use_par ? 1 : 0;
    m.tm.tp_symmetric_window = m.sym_win ? 1 : 0;
    m.tm.weight_bytes = int64_t(m.matrix_bytes);
    m.tm.kv_bytes = int64_t(m.kv_bytes);
    return std::unique_ptr<CudaLlamaDecoder>(new CudaLlamaDecoder(std::move(impl)));
}

// ---- the calls of a sequence. Their observable behaviour is the reference decoder's (src/backend/metal/metal_llama_decoder.mm:691-787 and the cases of
// tests/unit/test_metal_llama_decoder.cpp:534-608): argument checks and their codes, results independent of chunking and of the queue depth, what
// generate() delivers and where position() stands afterwards. ----

void CudaLlamaDecoder::reset() {
    Impl & m = *impl_;
    (void)m.wait_idle();          // nothing of the old sequence may still be writing the cache
    m.pos = 0;
    m.has_pending = false;
}

namespace {
std::string context_full(const LlamaDecoderConfig & c, int64_t wanted) {
    return "the KV cache holds " + std::to_string(c.n_ctx) + " positions; this call would need " + std::to_string(wanted);
}
const char * const kNothingPending = "no position has been evaluated since the last reset() / generate(): there is no pending token";
}  // namespace

// Appends n positions in chunks of at most n_batch. `stage(first, rows)` puts rows first .. first + rows of the caller's input into the pinned staging
// buffer and queues its copy to the device; the chunk then runs from there. The host rewrites the staging buffer for every chunk, hence the wait before it.
template <class Stage>
Status CudaLlamaDecoder::Impl::append_positions(int32_t n, bool from_tokens, Stage && stage) {
    if (int64_t(pos) + n > cfg.n_ctx) return resource_exhausted(context_full(cfg, int64_t(pos) + n));
    cudaSetDevice(opt.device);
    launches = 0;
    for (int32_t done = 0; done < n;) {
        DOOMS_RETURN_IF_ERROR(wait_idle());
        const int32_t rows = std::min(cfg.n_batch, n - done);
        if (done == 0) cudaEventRecord(ev_a, stream);
        stage(done, rows);
        run_chunk(rows, from_tokens);
        logits_slot = cur;
        done += rows;
    }
    cudaEventRecord(ev_b, stream);
    DOOMS_RETURN_IF_ERROR(wait_idle());
    float ms = 0.f;
    cudaEventElapsedTime(&ms, ev_a, ev_b);
    tm.last_eval_ms = ms;
    tm.last_eval_launches = launches;
    return Status();
}

Status CudaLlamaDecoder::eval_embeddings(const float * embeddings, int32_t n) {
    Impl & m = *impl_;
    if (embeddings == nullptr || n < 1) return invalid_argument("eval_embeddings: no rows given");
    const int64_t E = m.cfg.n_embd;
    if (!std::all_of(embeddings, embeddings + int64_t(n) * E, [](float v) { return std::isfinite(v); })) {
        return invalid_argument("eval_embeddings: a value is NaN or infinite");
    }
    return m.append_positions(n, false, [&](int32_t first, int32_t rows) {
        const size_t bytes = size_t(rows) * size_t(E) * sizeof(float);
        std::memcpy(m.host_x, embeddings + int64_t(first) * E, bytes);
        (void)m.check(cudaMemcpyAsync(m.x, m.host_x, bytes, cudaMemcpyHostToDevice, m.stream), "copying the embeddings to the device");
    });
}

Status CudaLlamaDecoder::eval_tokens(const std::vector<int32_t> & ids) { return eval_tokens(ids.data(), int32_t(ids.size())); }

Status CudaLlamaDecoder::eval_tokens(const int32_t * ids, int32_t n) {
    Impl & m = *impl_;
    if (ids == nullptr || n < 1) return invalid_argument("eval_tokens: no tokens given");
    const int32_t * bad = std::find_if(ids, ids + n, [&](int32_t t) { return t < 0 || t >= m.cfg.n_vocab; });
    if (bad != ids + n) return invalid_argument("eval_tokens: id " + std::to_string(*bad) + " is not in the vocabulary of " + std::to_string(m.cfg.n_vocab));
    return m.append_positions(n, true, [&](int32_t first, int32_t rows) {
        std::memcpy(m.host_in, ids + first, size_t(rows) * sizeof(int32_t));
        (void)m.check(cudaMemcpyAsync(m.in_tokens, m.host_in, size_t(rows) * sizeof(int32_t), cudaMemcpyHostToDevice, m.stream), "copying the tokens to the device");
    });
}

Status CudaLlamaDecoder::embed_tokens(const int32_t * ids, int32_t n, float * out) {
    Impl & m = *impl_;
    if (ids == nullptr || out == nullptr || n < 1) return invalid_argument("embed_tokens: no tokens given, or no room for their rows");
    const int32_t * bad = std::find_if(ids, ids + n, [&](int32_t t) { return t < 0 || t >= m.cfg.n_vocab; });
    if (bad != ids + n) return invalid_argument("embed_tokens: id " + std::to_string(*bad) + " is not in the vocabulary of " + std::to_string(m.cfg.n_vocab));
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    cudaSetDevice(m.opt.device);
    const size_t E = size_t(m.cfg.n_embd);
    for (int32_t done = 0; done < n; done += m.cfg.n_batch) {      // through the chunk buffers: nothing is pending on them while the stream is idle
        const int32_t rows = std::min(m.cfg.n_batch, n - done);
        std::memcpy(m.host_in, ids + done, size_t(rows) * sizeof(int32_t));
        (void)m.check(cudaMemcpyAsync(m.in_tokens, m.host_in, size_t(rows) * sizeof(int32_t), cudaMemcpyHostToDevice, m.stream), "copying the tokens to the device");
        m.embed(m.in_tokens, nullptr, rows);
        (void)m.check(cudaMemcpyAsync(out + size_t(done) * E, m.x, size_t(rows) * E * sizeof(float), cudaMemcpyDeviceToHost, m.stream), "reading the embedding rows");
        DOOMS_RETURN_IF_ERROR(m.wait_idle());
    }
    return Status();
}

Result<int32_t> CudaLlamaDecoder::pending_token() {
    Impl & m = *impl_;
    if (!m.has_pending) return invalid_argument(kNothingPending);
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    return m.host_tokens[0];
}

Status CudaLlamaDecoder::logits_into(float * out, int64_t capacity) {
    Impl & m = *impl_;
    if (!m.has_pending) return invalid_argument(kNothingPending);
    if (out == nullptr || capacity < m.cfg.n_vocab) return resource_exhausted("logits: the buffer has to hold " + std::to_string(m.cfg.n_vocab) + " floats");
    if (m.logits_slot != m.cur) return invalid_argument("logits: another sequence (or a batched step) was evaluated since this one; only the last evaluation's logits are kept");
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    cudaSetDevice(m.opt.device);
    if (m.tp > 1 && !m.logits_gathered) {
        // Under tensor parallelism a rank holds its own rows only; the other ranks' arrive here. Collective: every rank of the group calls logits() at
        // the same point (as it calls eval_tokens and generate).
        if (m.nccl.AllGather(m.logits_buf + m.vocab_row0, m.logits_buf, size_t(m.vocab_stride), NcclApi::kFloat32, m.comm, m.stream) != 0) {
            return m.check(cudaErrorUnknown, "gathering the logits");
        }
        DOOMS_RETURN_IF_ERROR(m.wait_idle());
        m.logits_gathered = true;
    }
    return m.check(cudaMemcpy(out, m.logits_buf, size_t(m.cfg.n_vocab) * sizeof(float), cudaMemcpyDeviceToHost), "reading the logits");
}

Result<std::vector<float>> CudaLlamaDecoder::logits() {
    std::vector<float> row(size_t(impl_->cfg.n_vocab));
    DOOMS_RETURN_IF_ERROR(logits_into(row.data(), int64_t(row.size())));
    return row;
}

// The decode steps in flight during generate(): a ring of events, one per queued step, oldest first.
class CudaLlamaDecoder::Impl::StepWindow {
public:
    StepWindow(Impl & m, int32_t depth) : m_(m) {
        while (m_.step_events.size() < size_t(depth) + 1) {
            cudaEvent_t e = nullptr;
            cudaEventCreate(&e);
            m_.step_events.push_back(e);
        }
    }
    int32_t in_flight() const { return int32_t(slots_.size()); }
    void queue_step() {
        m_.queue_decode_step();
        const size_t slot = issued_++ % m_.step_events.size();
        cudaEventRecord(m_.step_events[slot], m_.stream);
        slots_.push_back(slot);
    }
    // Blocks (or spins, when the configuration asks for it) until the oldest queued step is done; its event is remembered as the end of the timed span.
    cudaError_t retire_oldest() {
        const size_t slot = slots_.front();
        slots_.pop_front();
        cudaEvent_t e = m_.step_events[slot];
        cudaError_t rc = cudaSuccess;
        if (m_.cfg.spin_wait) { do { rc = cudaEventQuery(e); } while (rc == cudaErrorNotReady); }
        else rc = cudaEventSynchronize(e);
        if (rc == cudaSuccess) last_done_ = e;
        return rc;
    }
    cudaEvent_t last_done() const { return last_done_; }

private:
    Impl & m_;
    std::deque<size_t> slots_;
    size_t issued_ = 0;
    cudaEvent_t last_done_ = nullptr;
};

// Token 0 is the pending one (already in the token ring); token i > 0 comes out of decode step i, which embeds token i - 1 straight from the ring on the
// device, writes the cache at position start + i - 1 and its own greedy token to ring slot i. Up to `depth` steps run ahead of the token the host is
// handing to the callback; the steps queued past the stopping point finish on their own and are discarded (every later call waits for the stream first).
Status CudaLlamaDecoder::generate(int32_t max_tokens, int32_t depth, const std::function<bool(int32_t)> & on_token) {
    Impl & m = *impl_;
    if (!m.has_pending) return invalid_argument(kNothingPending);
    if (max_tokens < 1 || depth < 1) return invalid_argument("generate: max_tokens and depth have to be at least 1");
    const int32_t start = m.pos;
    if (int64_t(start) + max_tokens - 1 > m.cfg.n_ctx) return resource_exhausted(context_full(m.cfg, int64_t(start) + max_tokens - 1));
    cudaSetDevice(m.opt.device);
    DOOMS_RETURN_IF_ERROR(m.ensure_step_graph());
    DOOMS_RETURN_IF_ERROR(m.wait_idle());          // the pending token is final and nothing of an earlier generate() is still running
    Impl::StepWindow window(m, depth);
    m.launches = 0;
    m.run("state", [&] { return cuda::launch_set_state(m.state, start, 0, 1, m.stream); });
    cudaEventRecord(m.ev_a, m.stream);

    Status outcome;
    int32_t delivered = 0, queued_tokens = 1;      // tokens handed to the callback; tokens that exist or are being computed (the pending one counts)
    for (bool more = true; more;) {
        while (queued_tokens < max_tokens && queued_tokens - delivered <= depth) { window.queue_step(); queued_tokens++; }
        if (delivered > 0) {                        // every token but the pending one waits for its step
            const cudaError_t rc = window.retire_oldest();
            if (rc != cudaSuccess) { outcome = m.check(rc, "a decode step failed"); break; }
        }
        if (!m.failed.is_ok()) { outcome = m.failed; break; }
        if (m.host_error && *m.host_error != 0) { outcome = m.wait_idle(); break; }      // a kernel gave up on a bounded wait: its token is not to be trusted
        const int32_t token = m.host_tokens[delivered++];
        more = on_token(token) && delivered < max_tokens;
    }
    if (outcome.is_ok()) {
        // device time from the first step to the step of the last delivered token; what was queued past it is not the caller's
        float ms = 0.f;
        if (window.last_done()) cudaEventElapsedTime(&ms, m.ev_a, window.last_done());
        m.tm.last_generate_ms = ms;
        m.tm.last_generate_launches = m.launches;
    } else {
        (void)cudaStreamSynchronize(m.stream);
    }
    // as if the delivered tokens except the last had been evaluated one by one
    m.pos = start + std::max(delivered, 1) - 1;
    m.has_pending = false;
    return outcome;
}

// ---- several sequences ----

int32_t CudaLlamaDecoder::max_sequences() const { return int32_t(impl_->seqs.size()); }
int32_t CudaLlamaDecoder::selected_sequence() const { return impl_->cur; }
int32_t CudaLlamaDecoder::max_batch_rows() const { return impl_->max_rows; }

Status CudaLlamaDecoder::select_sequence(int32_t slot) {
    Impl & m = *impl_;
    if (slot < 0 || slot >= int32_t(m.seqs.size())) return invalid_argument("select_sequence: slot " + std::to_string(slot) + " of " + std::to_string(m.seqs.size()));
    if (slot == m.cur) return Status();
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    cudaSetDevice(m.opt.device);
    m.stash_selected();
    m.cur = slot;
    m.restore_selected();
    return m.failed;
}

Status CudaLlamaDecoder::decode_batch(const int32_t * slots, int32_t n, int32_t steps, int32_t * out_tokens) {
    Impl & m = *impl_;
    if (m.max_rows == 0) {
        return unsupported("decode_batch needs max_sequences > 1, one GPU, head_dim 64 or 128 and widths that are multiples of 64 (the tensor-core chunk path)");
    }
    if (slots == nullptr || out_tokens == nullptr || n < 1 || steps < 1) return invalid_argument("decode_batch: no slots, no room for the tokens, or no steps");
    if (n > m.max_rows) return resource_exhausted("decode_batch: " + std::to_string(n) + " rows; one step holds " + std::to_string(m.max_rows));
    if (steps > Impl::kMaxBatchSteps) return invalid_argument("decode_batch: at most " + std::to_string(Impl::kMaxBatchSteps) + " steps per call");
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    cudaSetDevice(m.opt.device);
    m.stash_selected();
    std::vector<bool> taken(m.seqs.size(), false);
    for (int32_t i = 0; i < n; i++) {
        const int32_t s = slots[i];
        if (s < 0) continue;                        // an idle row
        if (s >= int32_t(m.seqs.size())) return invalid_argument("decode_batch: slot " + std::to_string(s) + " of " + std::to_string(m.seqs.size()));
        if (taken[size_t(s)]) return invalid_argument("decode_batch: slot " + std::to_string(s) + " is listed twice");
        taken[size_t(s)] = true;
        const Impl::Sequence & q = m.seqs[size_t(s)];
        if (!q.has_pending) return invalid_argument("decode_batch: slot " + std::to_string(s) + " has no pending token (evaluate its prompt first)");
        if (int64_t(q.pos) + steps > m.cfg.n_ctx) return resource_exhausted(context_full(m.cfg, int64_t(q.pos) + steps));
    }
    const size_t R = size_t(m.max_rows);
    for (int32_t i = 0; i < n; i++) {
        const int32_t s = slots[i];
        m.h_rows[i] = s;
        m.h_rows[R + size_t(i)] = s < 0 ? 0 : m.seqs[size_t(s)].pos;
        m.h_rows[2 * R + size_t(i)] = s < 0 ? 0 : m.seqs[size_t(s)].pending;
    }
    auto graph = m.opt.use_graphs ? m.batch_graph(n) : Result<cudaGraphExec_t>(cudaGraphExec_t(nullptr));
    if (!graph.is_ok()) return graph.status();
    m.launches = 0;
    for (int part = 0; part < 3; part++) {
        (void)m.check(cudaMemcpyAsync(m.b_rows + size_t(part) * R, m.h_rows + size_t(part) * R, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice, m.stream), "copying the rows to the device");
    }
    (void)m.check(cudaMemsetAsync(m.b_step, 0, sizeof(int32_t), m.stream), "clearing the step counter");
    cudaEventRecord(m.ev_a, m.stream);
    for (int32_t t = 0; t < steps; t++) {
        if (graph.value()) { m.launches += m.batch_step_launches_count; (void)m.check(cudaGraphLaunch(graph.value(), m.stream), "cudaGraphLaunch"); }
        else m.batch_step_launches(n);
    }
    cudaEventRecord(m.ev_b, m.stream);
    (void)m.check(cudaMemcpyAsync(m.h_out, m.b_out, size_t(steps) * size_t(n) * sizeof(int32_t), cudaMemcpyDeviceToHost, m.stream), "reading the tokens");
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    float ms = 0.f;
    cudaEventElapsedTime(&ms, m.ev_a, m.ev_b);
    m.tm.last_batch_ms = ms;
    m.tm.last_batch_launches = m.launches;
    std::memcpy(out_tokens, m.h_out, size_t(steps) * size_t(n) * sizeof(int32_t));
    for (int32_t i = 0; i < n; i++) {
        const int32_t s = slots[i];
        if (s < 0) continue;
        Impl::Sequence & q = m.seqs[size_t(s)];
        q.pos += steps;
        q.pending = m.h_out[size_t(steps - 1) * size_t(n) + size_t(i)];
    }
    m.logits_slot = -1;              // the single-sequence logits buffer no longer belongs to any slot's last position
    m.restore_selected();
    return m.failed;
}

Result<std::vector<CudaLlamaDecoder::KernelTime>> CudaLlamaDecoder::profile_pass(int32_t rows) {
    Impl & m = *impl_;
    if (rows < 1 || rows > m.cfg.n_batch) return invalid_argument("rows must be in [1, n_batch]");
    if (rows == 1 && !m.has_pending) return invalid_argument("nothing has been evaluated yet");
    if (m.pos + rows > m.cfg.n_ctx) return resource_exhausted("the cache is too full");
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    cudaSetDevice(m.opt.device);
    if (rows > 1) {
        for (int32_t i = 0; i < rows; i++) m.host_in[i] = i % m.cfg.n_vocab;
        (void)m.check(cudaMemcpyAsync(m.in_tokens, m.host_in, size_t(rows) * 4, cudaMemcpyHostToDevice, m.stream), "copying the tokens to the device");
    }
    std::vector<KernelTime> times;
    m.profile = &times;
    // tokens[0] holds the pending token; the pass writes its own token to tokens[1] and leaves position() alone.
    (void)m.check(cuda::launch_set_state(m.state, m.pos, 0, 1, m.stream), "state");
    m.embed(rows == 1 ? m.tokens : m.in_tokens, nullptr, rows);
    m.forward(rows, false);
    m.profile = nullptr;
    DOOMS_RETURN_IF_ERROR(m.wait_idle());
    return times;
}

}  // namespace dooms
