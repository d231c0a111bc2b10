// C ABI of libvmoe_b200.so. Every function takes raw device pointers and a CUDA stream and
// returns 0 on success or a negative error code (see vmoe_b200/ops/_lib.py for the ctypes
// mirror of these declarations). Nothing here depends on PyTorch.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* vmoe_stream_t;  // cudaStream_t
#define VMOE_API __attribute__((visibility("default")))

// ----------------------------------------------------------------------------- GEMM
// C[b] (M x N) = epilogue( A[b] (M x K) * B[b] (N x K)^T ), bf16 operands, fp32 accumulation
// on tcgen05 tensor cores with TMEM accumulators and TMA-fed shared memory.
//
// Operand storage ("major"):
//   a_mn_major = 0: A stored [M][lda] (K contiguous);  1: A stored [K][lda] (M contiguous)
//   b_mn_major = 0: B stored [N][ldb] (K contiguous);  1: B stored [K][ldb] (N contiguous)
// so that forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run without a transpose.
//
// Epilogue, in this order, per output element v = acc:
//   v += bias[col]                       (bias != NULL; fp32, length N per batch)
//   pre-activation copy to C2            (C2 != NULL; bf16, same layout as C; or gelu'(v)
//                                         when c2_gelu_grad is set, for a cheaper backward)
//   v = gelu_tanh(v)                     (act == 1)
//   v *= gelu_tanh'(gelu_pre[row, col])  (gelu_pre != NULL; bf16, leading dim ldr2)
//   v += residual[row, col]              (residual != NULL; bf16, leading dim ldr)
//   colsum[col] += sum over rows of v    (colsum != NULL; fp32 atomics)
//   C[row, col] = v                      (bf16 or fp32 store, or fp32 atomic add)
struct VmoePushArgs;
typedef struct VmoeGemmArgs {
  const void* A;
  const void* B;
  void* C;
  void* C2;
  const float* bias;
  const void* residual;
  const void* gelu_pre;
  float* colsum;
  const unsigned* a_ready;  // optional per-(batch, m-tile) arrival counters for A rows
  unsigned* status;         // optional device status word (bits: see ptx_sm100.cuh)
  int64_t M, N, K, batch;
  int64_t lda, ldb, ldc, ldr, ldr2;
  int64_t a_batch_stride, b_batch_stride, c_batch_stride, bias_batch_stride, r_batch_stride;
  int32_t a_mn_major, b_mn_major;
  int32_t c_fp32;    // 0: C is bf16, 1: C is fp32
  int32_t c_atomic;  // 1: C += v with fp32 atomics (needs c_fp32)
  int32_t act;       // 0 none, 1 GELU(tanh)
  int32_t split_k;   // >1 splits the K range over CTAs (needs c_atomic)
  uint32_t a_ready_epoch;  // A tile (b, mt) may be loaded once a_ready[...] >= epoch * rows
  int32_t num_sms;   // CTAs to launch at most (0: all SMs of the device)
  int32_t c2_gelu_grad;  // with act == 1: C2 receives gelu'(v) instead of v
  int32_t pre_is_grad;   // gelu_pre already holds gelu'(x): multiply by it as is
  int32_t mt_offset;     // m-tiles are visited starting from this tile (rotation)
  int32_t cta_pair;      // 0: choose by size, 1: one CTA per 128x256 tile, 2: CTA pairs (256x256)
  // Multi-destination bf16 output: when c_multi_count > 0, rows [j * c_multi_rows,
  // (j + 1) * c_multi_rows) of every batch are stored to c_multi[j] (same ldc / batch stride as
  // C, which is then only used for alignment checks). Destinations may be peer-GPU buffers.
  const void* c_multi[8];
  int32_t c_multi_count;
  int64_t c_multi_rows;
  // Fused dispatch: when `push` is set (a VmoePushArgs), the row push (moe_push.cuh) runs inside
  // this launch, in two extra warps of every CTA, while the MMA and epilogue warps consume the
  // A tiles gated by the a_ready counters that the push (of this and of the peer GPUs)
  // advances. Needs the CTA-pair mode and rows that fit the push ring; otherwise the push is
  // launched as a kernel of its own in front of the GEMM (same result).
  const void* push;
  int32_t push_ctas;  // unused (kept for layout compatibility)
  // Completion signal: when signal_count > 0, the last GEMM CTA to finish (all its output
  // stores complete) adds 1, release at system scope, to each signal_flags[i] (device addresses,
  // local or peer). done_counter: a zero-initialised device word private to the caller.
  const void* signal_flags[8];
  int32_t signal_count;
  unsigned* done_counter;
} VmoeGemmArgs;

VMOE_API int vmoe_gemm_bf16(const VmoeGemmArgs* args, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- elementwise
// LayerNorm over the last dim of bf16 x[rows][h] (h % 8 == 0, h <= 2048); gamma/beta fp32 or
// NULL; mean/rstd (fp32 per row) are saved for the backward pass when non-NULL.
VMOE_API int vmoe_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y,
                                float* mean, float* rstd, int64_t rows, int64_t h, float eps,
                                vmoe_stream_t stream);
// dx (bf16) = LayerNorm backward (+ dres if non-NULL); dgamma/dbeta (fp32) are accumulated.
// `scratch` is global memory of vmoe_layernorm_bwd_scratch_bytes(rows, h) bytes that holds the
// per-CTA partial sums of dgamma/dbeta (required when either is non-NULL).
VMOE_API int64_t vmoe_layernorm_bwd_scratch_bytes(int64_t rows, int64_t h);
VMOE_API int vmoe_layernorm_bwd(const void* dy, const void* x, const float* gamma,
                                const float* mean, const float* rstd, const void* dres, void* dx,
                                float* dgamma, float* dbeta, float* scratch, int64_t rows,
                                int64_t h, vmoe_stream_t stream);
// out (bf16 [batch][tokens + has_cls][h]) = concat(cls, emb) + pos: class token (fp32 [h], may
// be NULL = zeros) in row 0 when has_cls, patch embeddings emb (bf16 [batch][tokens][h]) after
// it, position embedding pos (fp32 [tokens + has_cls][h], may be NULL) added to every row.
VMOE_API int vmoe_embed_finalize(const void* emb, const float* cls, const float* pos, void* out,
                                 int64_t batch, int64_t tokens, int64_t h, int has_cls,
                                 vmoe_stream_t stream);

// LayerNorm over short rows (h = 16, 32, 64 or 128) that sit inside a larger tensor as blocks
// of `inner` consecutive rows, the blocks `*_outer` elements apart: row r starts at
// (r / inner) * outer + (r % inner) * h. Used on the q / k slices of a packed QKV projection.
VMOE_API int vmoe_layernorm_fwd_strided(const void* x, const float* gamma, const float* beta,
                                        void* y, float* mean, float* rstd, int64_t rows,
                                        int64_t h, float eps, int64_t inner, int64_t x_outer,
                                        int64_t y_outer, vmoe_stream_t stream);
VMOE_API int vmoe_layernorm_bwd_strided(const void* dy, const void* x, const float* gamma,
                                        const float* mean, const float* rstd, void* dx,
                                        float* dgamma, float* dbeta, float* scratch, int64_t rows,
                                        int64_t h, int64_t inner, int64_t dy_outer,
                                        int64_t x_outer, int64_t dx_outer, vmoe_stream_t stream);

// All-reduce (sum) of the fp32 range [offset, offset + count) of a symmetric gradient buffer
// over `world` ranks with peer loads (two kernels: reduce own slice, gather the others).
// bufs / flags: host arrays of `world` device addresses (gradient buffer base and counter base
// of every rank; counters are uint32 [3][num_ranges], zero-initialised once). `epoch` counts
// calls for this range starting at 1. local_counters: uint32 [2][num_ranges] private to the
// rank, zero-initialised. Before the range is written again the caller must wait until
// counters[2 * num_ranges + range] >= epoch * world (vmoe_wait_counters).
VMOE_API int vmoe_allreduce_range(const uint64_t* bufs, const uint64_t* flags, int32_t world,
                                  int32_t rank, int64_t offset, int64_t count, int32_t range,
                                  int32_t num_ranges, uint32_t epoch, uint32_t* local_counters,
                                  uint32_t* status, int32_t ctas, int64_t limit_cycles,
                                  vmoe_stream_t stream);

// No-allocation variant of vmoe_layernorm_bwd (this entry point has no counterpart in the
// reference, which leaves all memory management to XLA). The partial sums of dgamma / dbeta go
// to a static device array inside the library (3.5 MiB, hidden sizes up to 1024) instead of a
// caller-provided scratch buffer, and the call invokes no allocating routine.
//  * The first call on each device resolves the array's device address (a host-side set-up
//    step); make that call before any stream capture.
//  * All calls on a device share the one array. It keeps the contents of the last call; nothing
//    in it has to be zero on entry, because every launch overwrites the rows it later reads.
//  * Calls that overlap in time on one device (different streams or threads) race on the array;
//    serialise them.
//  * Returns -1 with a message in vmoe_last_error() when h > 1024.
VMOE_API int vmoe_layernorm_bwd_static(const void* dy, const void* x, const float* gamma,
                                       const float* mean, const float* rstd, const void* dres,
                                       void* dx, float* dgamma, float* dbeta, int64_t rows,
                                       int64_t h, vmoe_stream_t stream);
// out[b][n] (fp32) += sum over rows of bf16 x[b][rows][n]; n % 8 == 0.
VMOE_API int vmoe_colsum_bf16(const void* x, float* out, int64_t batch, int64_t rows, int64_t n,
                              vmoe_stream_t stream);
// NHWC images (fp32 or bf16) -> bf16 patch matrix (B*gh*gw, ph*pw*C).
VMOE_API int vmoe_patchify(const void* img, int32_t img_is_bf16, void* out, int64_t b, int64_t hh,
                           int64_t ww, int64_t c, int64_t ph, int64_t pw, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- MoE routing
// Top-K routing plan for `groups` groups of `s` items over `e` experts from softmax gates
// (groups, s, e) fp32. Outputs: expert (groups, s, k), slot (groups, s, k) = position in the
// expert's buffer of that group (>= capacity: dropped), slot_pair (groups, e, capacity) =
// item * k + choice held by each buffer slot, or -1 for an empty slot.
VMOE_API int vmoe_routing_plan(const float* gates, int32_t* expert_out, int32_t* slot_out,
                               int32_t* slot_pair, int64_t groups, int64_t s, int64_t e, int64_t k,
                               int64_t capacity, int32_t batch_priority, vmoe_stream_t stream);
// "Experts choose" plan from softmax gates (groups, s, e) fp32, s <= 4096: every expert takes
// its `capacity` largest gates of each group (ties: lower item first). Outputs: slot
// (groups, s, e) = rank of the item in expert e's order if < capacity, else capacity (not
// taken); slot_pair (groups, e, capacity) = item * e_total + expert (-1: empty slot). These are
// the Top-K tables with K = e choices per item, choice j = expert j.
VMOE_API int vmoe_experts_choose_plan(const float* gates, int32_t* slot_out, int32_t* slot_pair,
                                      int64_t groups, int64_t s, int64_t e, int64_t capacity,
                                      vmoe_stream_t stream);
// Buffer row (g, e, c) at expert_base[e] + (g*C + c)*h  <-  weight * x[g, item] (zeros if the
// slot is empty). expert_base is a device array of e addresses (local or peer memory).
VMOE_API int vmoe_moe_gather_rows(const void* x, const int32_t* slot_pair, const float* weight,
                                  const uint64_t* expert_base, int64_t groups, int64_t s,
                                  int64_t e, int64_t c, int64_t k, int64_t h,
                                  vmoe_stream_t stream);
// out[g, item] = residual + sum_k weight_k * buffer row (expert_k, slot_k); dropped pairs skip.
VMOE_API int vmoe_moe_combine_rows(const uint64_t* expert_base, const int32_t* expert_idx,
                                   const int32_t* slot, const float* weight, const void* residual,
                                   void* out, int64_t groups, int64_t s, int64_t e, int64_t c,
                                   int64_t k, int64_t h, uint32_t* status, vmoe_stream_t stream);
// Backward of combine: dbuf row = gate * dy[item], dgate[pair] = <dy[item], ybuf row>.
VMOE_API int vmoe_moe_combine_bwd(const void* dy, const int32_t* slot_pair, const float* gate,
                                  const uint64_t* ybuf_base, const uint64_t* dbuf_base,
                                  float* dgate, int64_t groups, int64_t s, int64_t e, int64_t c,
                                  int64_t k, int64_t h, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- losses
// kind 0: sigmoid cross-entropy summed over classes; kind 1: softmax cross-entropy with soft
// labels. logits bf16 [rows][ld] (first n columns valid), labels [rows][ld_labels] with
// labels_dtype 0 fp32 / 1 bf16 / 2 uint8. loss fp32 [rows]; dlogits (bf16 [rows][ld], may be
// NULL) = d loss / d logits * grad_scale.
VMOE_API int vmoe_xent(int32_t kind, const void* logits, const void* labels, int32_t labels_dtype,
                       float* loss, void* dlogits, int64_t rows, int64_t n, int64_t ld,
                       int64_t ld_labels, float grad_scale, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- optimizer
// Flat fp32 buffers of n elements (n % 1024 == 0); meta has one {weight_decay, lr_mult,
// grad_scale, pad} float4 per 1024 elements. sums: double[3] = {sum g^2, sum update^2,
// sum p_new^2}; vmoe_grad_sumsq fills sums[0] and vmoe_optimizer_step reads it for the
// global-norm clip (clip_norm > 0) and accumulates sums[1..2]. mode 0 Adam, 1 SGD+momentum.
VMOE_API int vmoe_grad_sumsq(const float* g, const void* meta, int64_t n, double* sums,
                             vmoe_stream_t stream);
VMOE_API int vmoe_optimizer_step(float* p, const float* g, float* m, float* v, void* shadow,
                                 const void* meta, int64_t n, int32_t mode, float lr, float b1,
                                 float b2, float eps, float bc1, float bc2, float momentum,
                                 float clip_norm, float clip_value, float grad_div, double* sums,
                                 vmoe_stream_t stream);

// big_vision Adafactor over a table of tensors (device array of VmoeAdafactorTensor). A tensor
// is (batch, rows, cols) row-major fp32 with its gradient, momentum and optional bf16 shadow;
// `factored` tensors keep the moving averages of the row means (vr: batch x rows) and column
// means (vc: batch x cols) of g^2, others the full second moment v. col_acc (batch x cols, all
// zero between calls) and norm (batch) are scratch. chunk0: first 1024-element chunk of the
// tensor in the update kernel's work list (ascending; update_chunks = total number of chunks);
// finish_first[i]: first block of tensor i in the finish kernel (one block per batch entry of
// every tensor, finish_blocks in total); max_tiles: the largest batch * ceil(rows / 16) of the
// factored tensors (0: none is factored). sums as for vmoe_optimizer_step.
typedef struct VmoeAdafactorTensor {
  float* p;
  const float* g;
  float* mu;
  void* shadow;
  float* vr;
  float* vc;
  float* v;
  float* col_acc;
  float* norm;
  int64_t batch, rows, cols;
  float weight_decay, lr_mult, grad_scale;
  int32_t factored, c_is_largest;
  int64_t chunk0;
} VmoeAdafactorTensor;
VMOE_API int vmoe_adafactor_step(const VmoeAdafactorTensor* table, const int64_t* finish_first,
                                 int32_t num_tensors, int64_t finish_blocks,
                                 int64_t update_chunks, int64_t max_tiles, float decay, float eps,
                                 float momentum, float lr, float clip_norm, float clip_value,
                                 float grad_div, double* sums, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- attention
// Non-causal softmax attention, bf16, head dim D a multiple of 16 up to 80, T queries and Tk keys
// (keys and values of one head must fit shared memory: vmoe_attention_supported). q, k, v, dq, dk,
// dv and out / d_out are addressed as ptr + b*batch + t*tok + h*head (+ d), strides in elements
// and multiples of 8, so q, k and v may point into one packed (B, T, 3, H, D) projection, or q
// into one tensor and k, v into another (cross-attention: Tk and the kv_* / gkv_* strides).
// dropout_p > 0 drops attention weights with a keep mask that is a hash of (seed, batch, head,
// query, key); the backward pass must get the same dropout_p and seed.
typedef struct VmoeAttnArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;          // forward output (input of the backward pass)
  float* lse;         // (B, H, T) log-sum-exp of the scaled scores
  const void* d_out;  // backward only
  void* dq;
  void* dk;
  void* dv;
  unsigned* status;
  int64_t B, H, T, D;
  int64_t q_tok, q_head, q_batch;  // strides of q (and of k, v unless kv_* are set)
  int64_t o_tok, o_head, o_batch;  // strides of out and d_out
  int64_t g_tok, g_head, g_batch;  // strides of dq (and of dk, dv unless gkv_* are set)
  float scale;                     // usually 1 / sqrt(D)
  float dropout_p;                 // 0: no dropout
  int64_t Tk;                      // keys (0: same as T)
  int64_t kv_tok, kv_head, kv_batch;     // strides of k and v (all 0: the q strides)
  int64_t gkv_tok, gkv_head, gkv_batch;  // strides of dk and dv (all 0: the dq strides)
  uint64_t seed;                   // dropout seed
  float* dq_acc;  // backward, when vmoe_attention_bwd_needs_dq_acc: fp32 zeros, B*T*H*D
} VmoeAttnArgs;
VMOE_API int32_t vmoe_attention_supported(int64_t tq, int64_t tk, int64_t d);
VMOE_API int32_t vmoe_attention_bwd_needs_dq_acc(int64_t tq, int64_t d);
VMOE_API int vmoe_attention_fwd(const VmoeAttnArgs* args, vmoe_stream_t stream);
VMOE_API int vmoe_attention_bwd(const VmoeAttnArgs* args, vmoe_stream_t stream);

// ----------------------------------------------------------------------------- expert-parallel P2P
// Gathers the rows routed to every expert and stores them into the owning GPU's row buffer
// (dst_base[e] = address of this rank's block of expert e, possibly peer memory). For every
// 128-row chunk written, the number of rows is added (release, system scope) to the tile
// counters at flag_base[e] (the expert's counters on its owner; tile = buffer row / 128,
// where this rank's block starts at row rank * groups * c). flag_base may be NULL. With
// `weight`, rows are scaled by it and, if ybuf_base/dgate are given, dgate[pair] = <x, ybuf>.
VMOE_API int vmoe_moe_push_rows(const void* x, const int32_t* slot_pair, const float* weight,
                                const uint64_t* dst_base, const uint64_t* flag_base,
                                const uint64_t* ybuf_base, float* dgate, int64_t groups, int64_t s,
                                int64_t e, int64_t c, int64_t k, int64_t h,
                                int64_t experts_per_rank, int64_t ep, int64_t rank,
                                vmoe_stream_t stream);
// The same push with bulk asynchronous copies (global -> shared-memory ring -> owner's buffer),
// one ring per warp. This is the body that vmoe_gemm_bf16 runs in two extra warps of each of
// its CTAs when VmoeGemmArgs.push is set; as a kernel of its own (`ctas` CTAs of 8 warps) it
// serves tests and timing. flag_base[e][tile] counters as for vmoe_moe_push_rows, in steps of
// at most 32 rows. Rows must fit the ring: vmoe_moe_push_bulk_supported(h, with y rows).
typedef struct VmoePushArgs {
  const void* x;
  const int32_t* slot_pair;
  const float* weight;
  const uint64_t* dst_base;
  const uint64_t* flag_base;
  const uint64_t* ybuf_base;
  float* dgate;
  int64_t groups, s, e, c, k, h;
  int64_t experts_per_rank, ep, rank;
} VmoePushArgs;
VMOE_API int32_t vmoe_moe_push_bulk_supported(int64_t h, int32_t with_gate_gradient);
VMOE_API int vmoe_moe_push_rows_bulk(const VmoePushArgs* args, int32_t ctas, uint32_t* status,
                                     vmoe_stream_t stream);
// flags[i] += value for n <= 16 addresses (host array of device addresses, local or peer) in
// one launch, with a system-scope release ordered after all earlier work of the stream.
VMOE_API int vmoe_signal_multi(const uint64_t* flags, int32_t n, uint32_t value,
                               vmoe_stream_t stream);
// *flag += value with a system-scope release, ordered after all earlier work of the stream.
VMOE_API int vmoe_signal(uint32_t* flag, uint32_t value, vmoe_stream_t stream);
// Blocks the stream until counters[i] >= target for all i < n; gives up after limit_cycles
// (0: the library default) and sets the peer-timeout bit in *status.
VMOE_API int vmoe_wait_counters(const uint32_t* counters, int32_t n, uint32_t target,
                                uint32_t* status, int64_t limit_cycles, vmoe_stream_t stream);

// Noisy Top-K router statistics. logits/noise/gates_out: [tokens][E] fp32 (noise NULL = no
// noise, no load loss); sums: [G][4][E] scratch (importance, load, top-1 counts, gate sums);
// losses: [G][3] = importance, load, gshard; coef: [G][3][E] = d loss / d sum, kept for backward.
VMOE_API int vmoe_router_stats_fwd(const float* logits, const float* noise, float* gates_out,
                                   float* sums, float* losses, float* coef, int64_t tokens,
                                   int64_t group_size, int num_experts, float noise_std, int k,
                                   vmoe_stream_t stream);
// d_logits (fp32, may be NULL) and d_logits_bf16 (row stride ld_bf16, may be NULL) from the
// gradients of gates_out (d_gates, may be NULL) and of the three losses (d_losses [G][3]).
VMOE_API int vmoe_router_stats_bwd(const float* logits, const float* noise, const float* d_gates,
                                   const float* d_losses, const float* coef, float* d_logits,
                                   void* d_logits_bf16, int64_t ld_bf16, int64_t tokens,
                                   int64_t group_size, int num_experts, float noise_std, int k,
                                   vmoe_stream_t stream);

// Soft MoE routing weights of `groups` groups of m tokens x s slots (fp32, row-major per group):
// dispatch = softmax over the tokens of each slot, combine = softmax over the slots of each
// token. A group must fit in shared memory: m * s <= vmoe_soft_router_max_group_elements().
VMOE_API int64_t vmoe_soft_router_max_group_elements(void);
VMOE_API int vmoe_soft_router_fwd(const float* logits, float* dispatch, float* combine,
                                  int64_t groups, int32_t m, int32_t s, vmoe_stream_t stream);
// d_logits from the gradients of both weights (either may be NULL).
VMOE_API int vmoe_soft_router_bwd(const float* dispatch, const float* combine,
                                  const float* d_dispatch, const float* d_combine,
                                  float* d_logits, int64_t groups, int32_t m, int32_t s,
                                  vmoe_stream_t stream);

// Mixup: x and out viewed as (lead, batch, inner), fp32 or bf16; weights fp32 (size, lead, batch);
// out[l, b, :] = sum_i weights[i, l, b] * x[l, (b + i) % batch, :], size <= 8.
VMOE_API int vmoe_mixup(const void* x, void* out, const float* weights, int32_t is_bf16,
                        int64_t lead, int64_t batch, int64_t inner, int32_t size,
                        vmoe_stream_t stream);

// Host-side batch assembly (no device work, no state): dst[i] = srcs[i] for n blocks of
// bytes_each bytes, or dst[i][j] = srcs[i][j] * scale + shift from uint8 to float32, spread over
// `threads` threads (0 = one per core, at most 64). Has no counterpart in the reference, whose
// batches are assembled by tf.data.
VMOE_API int vmoe_collate_rows(const void* const* srcs, int64_t n, int64_t bytes_each, void* dst,
                               int32_t threads);
VMOE_API int vmoe_collate_u8_to_f32(const uint8_t* const* srcs, int64_t n, int64_t elems_each,
                                    float* dst, float scale, float shift, int32_t threads);

// Last error text of the calling thread ("" if none).
VMOE_API const char* vmoe_last_error(void);

#ifdef __cplusplus
}
#endif
