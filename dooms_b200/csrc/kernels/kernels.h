#pragma once
// Launchers of the decoder's CUDA kernels (internal interface between the host-side decoder and the .cu files). Every launcher enqueues on `stream` and
// returns the CUDA error of the launch; nothing here allocates or synchronizes unless it says so.
#include <cuda_runtime.h>
#include <cstdint>

namespace dooms {
namespace cuda {

// Position state of a sequence, kept in device memory so that a captured decode step can be replayed without new arguments: the kernels read it, the last
// kernel of a step advances it.
struct DevState {
    int32_t pos;       // cache position of the first row of the current call
    int32_t tok_in;    // index into the token ring of the token a decode step embeds
    int32_t tok_out;   // index into the token ring where the step's greedy token goes
    int32_t error;     // set non-zero by a kernel that found an inconsistency (never cleared by kernels)
};

enum : uint32_t { kFlagAccumulate = 2, kFlagBias = 4 };   // the reference's MatvecParams / GemmParams flags (metal_llama_decoder.mm:51)
// One-token projections only, with kFlagAccumulate: bits 8..11 = k > 0 scale the old value by 2^-k first, y = y 2^-k + W x. With 2^k tensor-parallel ranks
// an in-place all-reduce of y then gives y + the sum of the ranks' products on every rank (the scaling by a power of two is exact), without an add kernel.
constexpr uint32_t kFlagShareShift = 8;
// The kernel launched after this one is not one of this library's (an NCCL collective): this kernel then does not let its dependents start early. NCCL's
// symmetric-memory kernels start on the programmatic trigger of the kernel before them and read their input at once (measured: a tensor-parallel prompt
// went wrong when the projection before the all-reduce triggered at its start), so a producer of a collective's input triggers only by finishing.
constexpr uint32_t kFlagLateDependents = 1u << 12;
__host__ __device__ inline float accumulate_base(float y, uint32_t flags) {
    const uint32_t k = (flags >> kFlagShareShift) & 15u;
#ifdef __CUDA_ARCH__
    return k ? y * __uint_as_float((127u - k) << 23) : y;
#else
    return k ? y / float(1u << k) : y;
#endif
}

cudaError_t launch_set_state(DevState * st, int32_t pos, int32_t tok_in, int32_t tok_out, cudaStream_t stream);

// x[row][:] = table[ids[(index ? *index : 0) + row]][:], rows x E (embedq<Q>, llama_kernels.h:1289-1296).
cudaError_t launch_embed(int dt, const void * table, const int32_t * ids, const int32_t * index, float * x, int rows, int E, cudaStream_t stream);

// out[r][:] = x[r][:] * rsqrt(mean(x[r]^2) + eps) * gamma (norm_vec, llama_kernels.h:1272-1286). out16 (optional) also receives the rows as f16; xq
// (optional, one row, E a multiple of 32) the row split for the staged q4_0 GEMV.
cudaError_t launch_rms_norm(const float * x, const float * gamma, float * out, void * out16, void * xq, int rows, int E, float eps, cudaStream_t stream);

// y[r] (+)= W[r] . x (+ bias[r]) (matvec1q<Q>, llama_kernels.h:1197-1230).
cudaError_t launch_matvec(int dt, const void * W, const float * x, float * y, const float * bias, int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream);
// h[r] = silu(Wg[r] . x) * (Wu[r] . x) (gate_up1q<Q>, llama_kernels.h:1232-1269).
cudaError_t launch_gate_up(int dt, const void * Wg, const void * Wu, const float * x, float * h, int64_t rows, int64_t cols, cudaStream_t stream);

// Y[m][n] (+)= X[m] . W[n] (+ bias[n]) for M rows (matmulq<16,16,Q>, llama_kernels.h:1397-1429), CUDA-core tiles, f32 operands. With W2 the kernel computes
// silu(X . W[n]) * (X . W2[n]) instead (matmul_gate_upq, llama_kernels.h:1431-1468).
cudaError_t launch_matmul_tile(int dt, const void * W, const void * W2, const float * X, int64_t x_stride, float * Y, int64_t y_stride, const float * bias,
                               int M, int64_t N, int64_t K, uint32_t flags, cudaStream_t stream);

// x[i] += y[i].
cudaError_t launch_add(float * x, const float * y, int64_t n, cudaStream_t stream);

// Whole matrix to f32, bit for bit the block formulas (dequant_half<Q>, llama_kernels.h:1474-1480).
cudaError_t launch_dequantize(int dt, const void * blocks, int64_t rows, int64_t cols, float * out, cudaStream_t stream);

struct AttnShape { int n_head, n_head_kv, head_dim, qkv_stride, kv_stride, out_stride, neox; float rope_base; };

// Rotates q in place, rotates k into the f16 key cache and copies v into the f16 value cache for M rows at positions st->pos + t
// (rope_store, llama_kernels.h:521-545).
cudaError_t launch_rope_store(float * qkv, void * kc, void * vc, const DevState * st, const double * inv_freq, int M, const AttnShape & s,
                              cudaStream_t stream);   // inv_freq: head_dim / 2 rotary frequencies base^(-2i / head_dim)

// One query row against cache positions 0 .. st->pos (attention_split + attention_combine, llama_kernels.h:860-929). The cache is cut into `splits`
// ranges; part holds splits x n_head x (2 + head_dim) floats.
int attention_splits(int n_head, int n_ctx);
// xq (optional; needs splits > 1 and head_dim a multiple of 32): the output row also split for the staged q4_0 GEMV.
cudaError_t launch_attention_decode(const float * q, const void * kc, const void * vc, float * out, float * part, void * xq, const DevState * st,
                                    int n_keys_fixed, int splits, const AttnShape & s, cudaStream_t stream);

// The merge of the ranges alone: out[h] from part[h][splits][2 + head_dim]; xq (optional) receives the row split for the staged q4_0 GEMV.
cudaError_t launch_attention_combine(const float * part, float * out, void * xq, int splits, const AttnShape & s, cudaStream_t stream);

// Grouped-query decode attention (attention_decode.cu), head_dim 64 or 128, at most 8 query heads per key/value head, cache rows 16-byte aligned. qkv is
// the new token's row (query, key and value heads). With inv_freq (head_dim / 2 rotary frequencies base^(-2i / head_dim)) the kernel rotates the query and
// the key itself and writes key and value into the cache at st->pos (no launch_rope_store before it); without, q is used as it is, the cache is only read
// and n_keys_fixed gives the number of positions. Leaves part[n_head][splits][2 + head_dim] for launch_attention_combine.
// cs[i] = (cos, sin)(st->pos * inv_freq[i]) as float2 for the head_dim / 2 rotary pairs: one decode step's rotation, shared by its layers.
// zero (optional): a device word the kernel clears (the barrier counter of the fused decode step that follows it).
cudaError_t launch_rope_table(const DevState * st, const double * inv_freq, void * cs, int head_dim, cudaStream_t stream, unsigned * zero = nullptr);
bool attention_gqa_supported(const AttnShape & s);
int attention_gqa_splits(int n_head_kv, int n_ctx);
// With counters (n_head_kv zeroed ints, left zeroed) the last block of each key/value head merges the ranges itself into out (and xq): no combine launch.
cudaError_t launch_attention_gqa(const float * qkv, void * kc, void * vc, float * part, const DevState * st, const double * inv_freq, int n_keys_fixed,
                                 int splits, const AttnShape & s, int * counters, float * out, void * xq, cudaStream_t stream,
                                 const void * rope_cs = nullptr);   // rope_cs: launch_rope_table's output for st->pos, used instead of computing the angles

// ---- one decode step over several sequences at once ----
// Row r of the step belongs to the KV-cache slot slot[r] (negative: the row is idle, every kernel skips it) and sits at position pos[r] of that
// sequence; tok[r] is the token the row embeds and, after the step, the row's greedy token. Slots are slot_elems f16 elements apart within a layer's cache.
struct BatchRows { const int32_t * slot; int32_t * pos; int32_t * tok; int64_t slot_elems; };
// launch_attention_gqa for n_rows rows: qkv [n_rows][qkv_stride], out [n_rows][out_stride] (+ out16 [n_rows][n_head * head_dim] as f16, optional);
// part: n_rows x splits x n_head x (2 + head_dim) floats; counters: n_rows x n_head_kv zeroed ints (left zeroed). Each row rotates its query and key by
// its own position and appends key and value to its own slot's cache.
cudaError_t launch_attention_gqa_rows(const float * qkv, void * kc, void * vc, float * part, const double * inv_freq, int splits, const AttnShape & s, int * counters,
                                      float * out, void * out16, const BatchRows & rows, int n_rows, cudaStream_t stream);
// The same step on the tensor cores (attention_rows.cu) for head_dim 64 / 128 and at most 16 query heads per key/value head: ranges of a fixed number of
// positions (ceil(n_ctx / splits), rounded up to whole tiles), so that a row has as many blocks as its length asks for. Same buffers as above.
bool attention_rows_tc_supported(const AttnShape & s);
cudaError_t launch_attention_rows_tc(const float * qkv, void * kc, void * vc, float * part, const double * inv_freq, int splits, int n_ctx, const AttnShape & s,
                                     int * counters, float * out, void * out16, const BatchRows & rows, int n_rows, cudaStream_t stream);
// Greedy token of every row: logits [n_rows][stride], first n of each row. Active rows (slot >= 0): tok[r] = argmax, pos[r] += 1, and the token also goes
// to out[(*step) * n_rows + r]; idle rows write -1 there. *step is incremented once per launch. part: n_rows x argmax_blocks(n) x 2 words.
cudaError_t launch_argmax_rows(const float * logits, int64_t n, int64_t stride, const BatchRows & rows, int n_rows, int32_t * out, int32_t * step, void * part,
                               cudaStream_t stream);

// Causal attention of M query rows at positions st->pos + t over the cache (attention_prefill, llama_kernels.h:640-769; this version runs on CUDA cores).
// out16 (optional): the same rows as f16, for the tensor-core GEMM that follows.
cudaError_t launch_attention_prefill(const float * qkv, const void * kc, const void * vc, float * out, void * out16, const DevState * st, int M,
                                     const AttnShape & s, cudaStream_t stream);

// The same on the tensor cores (attention_flash.cu) for head_dim 64 or 128.
bool attention_flash_supported(const AttnShape & s);
cudaError_t launch_attention_flash(const float * qkv, const void * kc, const void * vc, float * out, void * out16, const DevState * st, int M, const AttnShape & s,
                                   cudaStream_t stream);

// tokens[st->tok_out] = first index of the maximum of logits[0..n) (NaN never wins); the token also goes to host_tokens[st->tok_out] when that is set
// (mapped pinned memory). With advance the state moves one decode step forward (pos, tok_in, tok_out += 1). part: argmax_blocks(n) x 2 words.
int argmax_blocks(int64_t n);
cudaError_t launch_argmax(const float * logits, int64_t n, int32_t * tokens, int32_t * host_tokens, DevState * st, void * part, int advance, cudaStream_t stream);
// Two stages for a vocabulary split over tensor-parallel ranks: *pair (8 bytes: value, index + offset; index -1 when the slice holds no number) = the
// best of this rank's logits[0..n); then, over the gathered pairs of all ranks, the token by the same first-index rule.
cudaError_t launch_argmax_local_pair(const float * logits, int64_t n, int32_t offset, void * pair, void * part, cudaStream_t stream);
cudaError_t launch_argmax_pairs(const void * pairs, int n_ranks, int32_t * tokens, int32_t * host_tokens, DevState * st, int advance, cudaStream_t stream);
// The same reduction without a state: *out = argmax.
cudaError_t launch_argmax_plain(const float * logits, int64_t n, int32_t * out, void * part, cudaStream_t stream);

// ---- the fast decode GEMV on q4_0 rows (gemv_q4_0.cu) ----
// q6_K rows on the int8 tensor-core path (gemv_q6_k.cu): y (+)= W x (+ bias) on an input that is already split (launch_quantize_x, or a norm that leaves
// the split). Takes 16-byte aligned matrices with rows of whole super-blocks, up to 40960 columns.
bool gemv_q6_k_supported(const void * W, int64_t rows, int64_t cols);
cudaError_t launch_gemv_q6_k(const void * W, const void * xq, float * y, const float * bias, int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream);

// The streaming GEMV for any block format (gemv_blocks.cu): y (+)= W x (+ bias), or with W2 the fused gate/up h = silu(W x) * (W2 x). Takes 16-byte aligned
// W and x and rows of whole blocks that fit its shared-memory plan; launch_matvec / launch_gate_up use it whenever it takes the call.
bool gemv_blocks_supported(int dt, const void * W, const void * x, int64_t rows, int64_t cols);
// gamma (optional): the input is RMS-normalized in the block's prologue first, as for launch_gemv_q4_0.
cudaError_t launch_gemv_blocks(int dt, const void * W, const void * W2, const float * x, const float * gamma, float eps, float * y, const float * bias,
                               int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream);

// The input vector split into int8 limbs: quantized_x_bytes(cols) bytes at a 16-byte aligned address, written by launch_quantize_x.
size_t quantized_x_bytes(int64_t cols);
cudaError_t launch_quantize_x(const float * x, int64_t cols, void * xq, cudaStream_t stream);
// Whether launch_gemv_q4_0 takes this matrix: a 16-byte aligned base and rows of an even number of blocks that fit the kernel's shared memory plan.
bool gemv_q4_0_supported(const void * W, int64_t rows, int64_t cols);
// y[r] (+)= W[r] . x (+ bias[r]); with W2: y[r] = silu(W[r] . x) * (W2[r] . x). The input comes either split (xq, from launch_quantize_x or from a kernel
// that writes the split itself) or as f32 (xq == nullptr, x != nullptr): then every block splits it in its prologue, after RMS-normalizing it when gamma is
// given (x[i] * rsqrt(mean(x^2) + eps) * gamma[i]), which saves the norm's and the split's own launches in a decode step.
// q4_k: the rows are q4_K super-blocks (same bytes per 256 elements, other unpacking); gemv_q4_k_supported says whether the kernel takes the matrix.
bool gemv_q4_k_supported(const void * W, int64_t rows, int64_t cols);
// xq_out (optional, rows a multiple of 32, with out_counters = rows / 32 zeroed ints that are left zeroed): the output row is also written split, for a
// following projection that takes it as xq; the block that completes a 32-row group of y splits it.
// link (optional): the RMS norm between two projections, moved to the producer. As producer (with xq_out): the split left in xq_out is of
// y[i] * gamma_out[i] and block b writes the sum of its rows' y^2 to ss_out[b] (gemv_q4_0_blocks(...) entries). As consumer (with xq): ss_in / ss_n are
// the producer's ss_out and its block count; the results are multiplied by rsqrt(sum(ss_in) / cols + eps), which is the norm's scale factor applied
// after the product instead of before it.
struct GemvNormLink { const float * gamma_out; float * ss_out; const float * ss_in; int ss_n; };
int gemv_q4_0_blocks(int64_t rows, int64_t cols, bool gate_up, bool q4_k);      // blocks a launch on this shape uses
cudaError_t launch_gemv_q4_0(const void * W, const void * W2, const void * xq, const float * x, const float * gamma, float eps, float * y, const float * bias,
                             int64_t rows, int64_t cols, uint32_t flags, bool q4_k, cudaStream_t stream, void * xq_out = nullptr, int * out_counters = nullptr,
                             int32_t * error = nullptr,    // error: optional mapped host word, set to 4 if a bounded wait for a tensor copy ran out
                             const GemvNormLink * link = nullptr);

// ---- the fused decode step (gemv_q4_0.cu): all layers of a one-sequence decode step in one cooperative launch ----
// Takes models whose layer matrices are all q4_0 / q4_K rows that the tensor-copy variant of the GEMV above streams (rows of whole 256-element groups,
// one q/k/v matrix per layer) and whose attention the grouped-query kernel handles; anything else is refused with cudaErrorNotSupported and runs kernel
// by kernel. The step around it stays as it is: embedding and rotary table before (the rotary table kernel also zeroes the barrier word), output
// projection and argmax after.
struct FusedMatrix { const void * w; int64_t rows, cols; bool q4_k; };
struct FusedLayer {
    FusedMatrix qkv, attn_output, ffn_gate, ffn_up, ffn_down;
    const float * attn_norm, * ffn_norm, * qkv_bias;      // qkv_bias: nullptr = none
    const float * next_norm;                               // gains of the norm after this layer: the next layer's attn_norm, or the output norm
    void * kc, * vc;                                       // this layer's key / value cache
};
struct FusedBuffers {
    float * x, * qkv, * attn, * h;
    void * xq, * xq2;                                      // split rows: attention / feed-forward output, and the residual row times the next norm's gains
    float * norm_ss;
    int * norm_counters, * split_counters, * attn_counters;
    float * part;                                          // max_splits x n_head x (2 + head_dim) floats
    const DevState * state;
    const double * inv_freq;
    const void * rope_cs;
    int32_t * error;
    float eps;
    AttnShape shape;
    int max_splits;
};
struct DecodeLayersPlan;
cudaError_t decode_layers_create(const FusedLayer * layers, int n_layers, const FusedBuffers & buffers, DecodeLayersPlan ** out);
void decode_layers_destroy(DecodeLayersPlan * plan);
int decode_layers_blocks(const DecodeLayersPlan * plan);            // blocks of the launch = entries of norm_ss its last projection leaves
unsigned * decode_layers_barrier(const DecodeLayersPlan * plan);    // the word the kernel before the launch has to zero
cudaError_t launch_decode_layers(const DecodeLayersPlan * plan, cudaStream_t stream);

// ---- the decode step's all-reduce + residual add over peer memory (allreduce_peer.cu) ----
constexpr int kPeerMaxRanks = 8, kPeerMaxBlocks = 64;
struct PeerAllReduce {
    float * inbox[kPeerMaxRanks];       // every rank's inbox [2][n][max_floats] as this process sees it (its own, and the peers' through CUDA IPC)
    uint32_t * flags[kPeerMaxRanks];    // every rank's flags [2][n][kPeerMaxBlocks]
    uint32_t * round;                   // this rank's count of rounds done (device memory, zero at start)
    uint32_t * ticket;                  // this rank's count of blocks done in the current round
    DevState * state;
    int32_t * host_error;               // mapped host word the decoder polls (optional)
    int rank, n, max_floats;
};
size_t peer_allreduce_inbox_bytes(int n_ranks, int max_floats);
size_t peer_allreduce_flag_bytes(int n_ranks);
// x[0..n) += sum over ranks of partial[0..n), the same bits on every rank. n a multiple of 4, at most max_floats. All ranks must call it the same number
// of times; waits are bounded and end with state->error = 3.
cudaError_t launch_allreduce_add(const PeerAllReduce & p, const float * partial, float * x, int n, cudaStream_t stream);

// ---- the tensor-core prefill GEMM (gemm_tc.cu) ----
// A TMA descriptor of an f16 activation buffer [rows][cols] (cols a multiple of 64), opaque here so that this header needs no driver types.
struct alignas(64) TensorMap { unsigned char bytes[128]; };
cudaError_t make_activation_map(TensorMap * out, const void * base, int64_t rows, int64_t cols);
// A matrix of `rows` rows of row_bytes bytes (a multiple of 16, 16-byte aligned base) as a 2-D tensor of 16-bit words, copied in boxes of box_rows rows x
// box_bytes bytes (a multiple of 16, at most 512), no swizzle, rows past the end read as zeros.
cudaError_t make_rows_map(TensorMap * out, const void * base, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows);
bool gemm_tc_supported(int dt, const void * W, int64_t N, int64_t K);
// Y[m][n] (+)= X[m] . W[n] (+ bias[n]) for M tokens; X is the f16 buffer behind xmap. With W2: silu(X . W[n]) * (X . W2[n]). Y (f32) and / or Y16 (f16)
// receive the result. *error is set to 2 if a pipeline wait ran out.
// w16_scratch (optional, w16_bytes): room for the matrix (both, for gate/up) as f16 rows; with it and 512 or more tokens the weights are dequantized once
// per call and both operands arrive by TMA.
cudaError_t launch_gemm_tc(int dt, const void * W, const void * W2, const TensorMap * xmap, float * Y, void * Y16, const float * bias, int M, int64_t N, int64_t K,
                           int64_t y_stride, int64_t y16_stride, uint32_t flags, int32_t * error, cudaStream_t stream,
                           void * w16_scratch = nullptr, size_t w16_bytes = 0, int k_splits = 1, int64_t split_stride = 0);
// A product whose tiles would leave most SMs idle (few weight rows against one token tile: a batched decode step) can deal its reduction dimension over
// k_splits blocks per tile: gemm_tc_k_splits says how many (1: do not split), launch_gemm_tc with that k_splits then writes the shares' sums to
// Y + z * split_stride (flags 0, no f16 output), and launch_add_shares adds them onto x in a fixed order, so the result does not depend on timing.
int gemm_tc_k_splits(int dt, int M, int64_t N, int64_t K, bool gate, size_t w16_bytes);
// The same product against weights that already lie in device memory as f16 rows [N][K] (W2_16: the second matrix of a gate / up pair): a decoder that
// runs batched steps keeps such a copy of its matrices, made once with launch_dequant_rows16, instead of dequantizing them in every step.
cudaError_t launch_dequant_rows16(int dt, const void * W, void * out, int64_t rows, int64_t cols, cudaStream_t stream);
int gemm_tc_rows16_k_splits(int M, int64_t N, int64_t K);
cudaError_t launch_gemm_tc_rows16(const void * W16, const void * W2_16, const TensorMap * xmap, float * Y, void * Y16, const float * bias, int M, int64_t N, int64_t K,
                                  int64_t y_stride, int64_t y16_stride, uint32_t flags, int32_t * error, cudaStream_t stream, int k_splits = 1, int64_t split_stride = 0);
cudaError_t launch_add_shares(float * x, const float * shares, int k_splits, int64_t n, int64_t split_stride, cudaStream_t stream);

}  // namespace cuda
}  // namespace dooms
