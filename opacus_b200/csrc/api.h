// C interface of the sm_100a kernels.  Every function enqueues work on `stream`
// and returns a cudaError_t value (0 = success) for launch/argument errors.
// Pointers are device pointers unless stated otherwise.  `status` points to four
// 32-bit words in device memory, zeroed by the caller; a kernel that had to give
// up on a bounded wait writes a non-zero code there and returns early.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- ghost norms: out_w[n] (+)= scale * <X_n X_n^T, G_n G_n^T>, out_b[n] (+)= scale * sum(G_n G_n^T)
// x: [B, T, d_x] bf16 (or NULL), ids: [B, T] int64 (or NULL; used when x is NULL: X X^T := [id_t == id_s]),
// g: [B, T, d_g] bf16.  scratch: at least dpk_gram_pair_scratch_floats(B, T) floats.
size_t dpk_gram_pair_scratch_floats(int B, int T);
int dpk_gram_pair_norm(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g, float scale,
                       float* scratch, float* out_w, float* out_b, int accumulate, uint32_t* status,
                       cudaStream_t stream);

// The same with distinct left / right operands of each Gram product: x, g are [B, 2 * right_off, d]; rows [0, T) of a
// sample are the left operand, rows [right_off, right_off + T) the right one (right_off a multiple of 128, >= T,
// rows in between zero).  L R^T must be symmetric, as it is for the planes (hi, hi, lo) x (hi, lo, hi) of an fp32
// operand split into bf16 parts stacked along d.
int dpk_gram_pair_norm_lr(const void* x, const int64_t* ids, const void* g, int B, int T, int d_x, int d_g,
                          int right_off, float scale, float* scratch, float* out_w, float* out_b, int accumulate,
                          uint32_t* status, cudaStream_t stream);

// ---- clipped weight gradient: out[M, N] = beta*out + sum_k Gs[k, m] * A[k, n]   (bf16 in, fp32 accumulate)
// gs: [K, M] bf16 row-major, a: [K, N] bf16 row-major, out: [M, N] fp32 or bf16 (out_bf16 != 0).
int dpk_wgrad_tn(const void* gs, const void* a, int K, int M, int N, void* out, int out_bf16, float beta,
                 uint32_t* status, cudaStream_t stream);

// The same product on pairs of SMs (tcgen05 cta_group::2, clusters of two CTAs per 256 x 256 tile, double-buffered
// accumulators): fp32 out, beta in {0, 1} when splits > 1.
int dpk_wgrad2_tn(const void* gs, const void* a, int K, int M, int N, float* out, float beta, int splits,
                  uint32_t* status, cudaStream_t stream);

// Batched / tunable form: gs [batch, K, M], a [batch, K, N], out [batch, M, N]; norm_sq (or NULL) receives
// += ||out[b]||_F^2 per batch entry (fp32 atomics; only without K splitting).  force_* = 0 lets the
// launcher choose tile shape (256x256, 128x256, 128x128) and K split (1, 2, 4, 8).
int dpk_wgrad_tn_ex(const void* gs, const void* a, int K, int M, int N, int batch, void* out, int out_bf16,
                    float beta, float* norm_sq, int force_bm, int force_bn, int force_splits, uint32_t* status,
                    cudaStream_t stream);

// Per-sample (or batch-summed) weight gradient of a 1-d/2-d convolution from channels-last operands, without an
// unfolded input: x [B, H, W, C] bf16, g [B, OH, OW, O] bf16 -> out [B, O, kh, kw, C] (reduce_batch: [O, kh, kw, C],
// fp32, beta in {0, 1}); norm_sq (or NULL) receives += ||out[b]||_F^2; out == NULL computes the norms only.
// C and O must be multiples of 8.
int dpk_conv_psg(const void* x, const void* g, int B, int C, int H, int W, int O, int OH, int OW, int kh, int kw,
                 int sh, int sw, int ph, int pw, int dh, int dw, int reduce_batch, void* out, int out_bf16,
                 float beta, float* norm_sq, uint32_t* status, cudaStream_t stream);

// Cross term of the per-sample gradient norm for a weight tied between an embedding and an output projection:
// out[n] (+)= scale * sum_{t,s} g_h[n, s, ids[n, t]] * <g_e[n, t, :], a_h[n, s, :]>   (g_e, a_h bf16 [B, T, D];
// g_h bf16 or fp32 [B, T, V]).  scratch: 2 * B * ceil(T/128)^2 floats.  D a multiple of 8.
int dpk_tied_cross_norm(const int64_t* ids, const void* g_e, const void* a_h, const void* g_h, int g_h_fp32, int B,
                        int T, int D, int64_t V, float scale, float* scratch, float* out, int accumulate,
                        uint32_t* status, cudaStream_t stream);

// ---- elementwise / reduction kernels
// y[r, :] = bf16(x[r, :] * c[r / rows_per_sample] * scale)
int dpk_scale_rows(const void* x, int x_is_fp32, const float* c, void* y_bf16, int64_t rows, int64_t cols,
                   int64_t rows_per_sample, float scale, cudaStream_t stream);
// fp32 x [rows, cols] (rows = samples * T) -> bf16 y [samples, 3, T, cols]: planes (hi, hi, lo) of x * c[sample] * scale,
// or (hi, lo, hi) when `right`, with hi = bf16(v), lo = bf16(v - hi).  A left and a right operand stacked like this
// along the contraction axis give the fp32 product on the bf16 tensor cores up to a relative 2^-16.
int dpk_split3_rows(const float* x, const float* c, void* y_bf16, int64_t rows, int64_t cols, int64_t T, float scale,
                    int right, cudaStream_t stream);
// ---- ChaCha20 keystream (20 rounds, 64-bit block counter, 64-bit nonce; key8_host: eight host words).
// dpk_chacha_words: n_blocks * 16 raw words.  dpk_chacha_normal: n Gaussians of deviation std by Box-Muller on word
// pairs; draws == 4: element i = std * (sum of the four normals of words [4i, 4i+4)) / 2, draws == 1: the cosine normal
// of words [2i, 2i+2).  `out` 16-byte aligned.
int dpk_chacha_words(uint32_t* out, int64_t n_blocks, const uint32_t* key8_host, uint64_t nonce, uint64_t first_block,
                     cudaStream_t stream);
int dpk_chacha_normal(float* out, int64_t n, const uint32_t* key8_host, uint64_t nonce, uint64_t first_block, float std,
                      int draws, cudaStream_t stream);
// c[n] = min(1, C / (sqrt(max(norm_sq[n], 0)) + 1e-6))
int dpk_clip_factor(const float* norm_sq, float* c, int64_t B, float max_grad_norm, cudaStream_t stream);
// out[n] (+)= sum_j x[n, j]^2    (x: fp32 / bf16 / fp16 by elem_kind 0/1/2)
int dpk_row_norm_sq(const void* x, int elem_kind, int64_t B, int64_t cols, float* out, int accumulate,
                    cudaStream_t stream);
// out[j] = sum_n c[n] * x[n, j]  (out fp32)
int dpk_weighted_sum(const void* x, int elem_kind, const float* c, int64_t B, int64_t cols, float* out,
                     cudaStream_t stream);
// per-sample 2-d input fast path: out_w[n] (+)= scale * |a_n|^2 |g_n|^2, out_b[n] (+)= scale * |g_n|^2
int dpk_outer_norm_sq(const void* a, const void* g, int elem_kind, int64_t B, int64_t d_a, int64_t d_g, float scale,
                      float* out_w, float* out_b, int accumulate, cudaStream_t stream);
// Normalisation layers: per-sample affine gradients from the layer input x and output gradient g.
// kind 0 = LayerNorm, 1 = RMSNorm over the last `d` elements of [B, rows, d];  gw/gb: [B, d] fp32.
// stats_scratch: 2 * B * rows floats of scratch (per-row mean and reciprocal std).
int dpk_norm_lastdim_grad(int kind, const void* x, const void* g, int elem_kind, int64_t B, int64_t rows, int64_t d,
                          float eps, float* stats_scratch, float* gw, float* gb, cudaStream_t stream);
// The same gradients plus their squared norms n2w[n] = ||gw[n]||^2, n2b[n] = ||gb[n]||^2 (+= when accumulate) in
// ONE launch.  tickets ([B] words) must be zero on entry; part: scratch of dpk_norm_lastdim_psg_scratch_floats()
// floats (per-block partial sums, added in a fixed order: the results are reproducible bit for bit).  Covers
// d % 8 == 0, d <= 4096 (d <= 2048 with gb) and 16-byte aligned x / g; returns cudaErrorNotSupported otherwise.
int64_t dpk_norm_lastdim_psg_scratch_floats(int64_t B, int64_t rows, int64_t d, int with_bias);
int dpk_norm_lastdim_psg_fused(int kind, const void* x, const void* g, int elem_kind, int64_t B, int64_t rows,
                               int64_t d, float eps, float* gw, float* gb, float* n2w, float* n2b, int accumulate,
                               unsigned int* tickets, float* part, cudaStream_t stream);
// kind 2 = GroupNorm / InstanceNorm on [B, C, S] with `groups` groups; gw/gb: [B, C] fp32.
int dpk_norm_channel_grad(const void* x, const void* g, int elem_kind, int64_t B, int64_t C, int64_t S, int groups,
                          float eps, float* gw, float* gb, cudaStream_t stream);
// Embedding clipped gradient: out[ids[r], :] += c[r / T] * scale * g[r, :]   (out fp32 [V, D], zeroed by caller)
int dpk_embedding_scatter(const int64_t* ids, const void* g, int elem_kind, const float* c, int64_t rows, int64_t T,
                          int64_t D, int64_t V, int64_t padding_idx, float scale, float* out, cudaStream_t stream);

// ---- fused noise + scale + optimiser update over a table of tensors
struct DpkTensorEntry {
  void* param;         // fp32 or bf16 (param_bf16)
  float* grad;         // in: clipped sum; out: private gradient (noised, scaled)
  float* state0;       // SGD: momentum buffer (or NULL); Adam: exp_avg
  float* state1;       // Adam: exp_avg_sq
  float* master;       // optional fp32 master copy when param is bf16 (or NULL)
  int64_t numel;
  int64_t rng_offset;  // element offset of this tensor in the step's Philox stream
  int32_t param_bf16;
  int32_t pad;
};
struct DpkStepHyper {
  int32_t kind;        // 0 sgd, 1 adam (L2 weight decay), 2 adamw (decoupled)
  int32_t nesterov;
  int32_t first_step;  // SGD momentum buffer not initialised yet
  int32_t pad;
  float lr, momentum, dampening, weight_decay;
  float beta1, beta2, eps, bias_c1, bias_c2_sqrt;  // bias_c1 = 1 - beta1^t, bias_c2_sqrt = sqrt(1 - beta2^t)
  float noise_std, inv_scale;
  uint64_t seed, offset;
};
int dpk_fused_dp_step(const struct DpkTensorEntry* table_dev, int n_tensors, int64_t total_chunks,
                      const int64_t* chunk_prefix_dev, struct DpkStepHyper h, cudaStream_t stream);

// ---- sharded data-parallel step: reduce-scatter + noise + update + all-gather over peer memory
// Pointer arrays are indexed by rank and hold addresses that are valid on THIS GPU (peer mappings of
// symmetric allocations; entry [rank] is local).  grad/param are flat buffers over the whole parameter
// space; master/state0/state1 cover only the slice_len elements of it that this launch updates: the range
// [slice_begin, slice_begin + slice_len) when stripe_len == 0, else slice_len / stripe_len stripes of
// stripe_len elements whose starts are stripe_stride apart, the first at slice_begin (the flat space cut into
// pieces of stripe_stride elements of which every rank owns one stripe).
// flags: at least 32 zero-initialised 32-bit words per rank.  epoch: 1, 2, 3, ... on successive calls.
// grad_mc / param_mc: the same two buffers through the address of an NVLink multicast object that all ranks'
// copies are bound to (NVLS), or NULL: the reduce then uses plain peer loads, the publish plain peer stores.
// segs (device memory, nseg entries, ends ascending, last end >= end of the flat space) gives ranges of the flat
// space their own learning rate and weight decay; nseg <= 1 uses h for everything.
// max_blocks > 0 caps the grid (a launch that shares the GPU with compute-bound kernels).
struct DpkStepSegment {
  int64_t end;
  float lr, weight_decay;
};
struct DpkShardedStep {
  const float* grad[8];
  void* param[8];
  uint32_t* flags[8];
  const float* grad_mc;
  void* param_mc;
  const struct DpkStepSegment* segs;
  int32_t nseg, max_blocks;
  float* master;
  float* state0;
  float* state1;
  int64_t slice_begin, slice_len;
  int64_t stripe_len, stripe_stride;
  // Elements of the flat space at or beyond noise_split draw their noise at counter index + noise_shift
  // (a multiple of 8): tensor-parallel ranks pass distinct shifts for their shards and share the rest.
  int64_t noise_split, noise_shift;
  int32_t world, rank, param_bf16, pad;
  uint32_t epoch, pad2;
  struct DpkStepHyper h;
  uint32_t* status;
};
int dpk_sharded_dp_step(const struct DpkShardedStep* p, cudaStream_t stream);

// Sum of per-rank [n] fp32 vectors over a group of <= 8 ranks through symmetric memory, plus the clip factor
// min(1, max_norm / (sqrt(total) + 1e-6)), identical bits on every rank.  slots[r]: rank r's symmetric buffer of
// 2 * world * capacity floats; flags[r]: rank r's symmetric flag words, of which [flag_base, flag_base + world) are
// used; epoch: 1, 2, 3, ... on successive calls of the same group (all ranks pass the same value).
struct DpkNormAllReduce {
  float* slots[8];
  uint32_t* flags[8];
  const float* sharded;      // [n] partial sums of this rank, or NULL (zeros)
  const float* replicated;   // [n] added once, unreduced, or NULL
  float* total_out;          // [n] or NULL
  float* clip_out;           // [n] or NULL
  // pull != 0: rank r's partial sums already are in slots[r] at (epoch & 1) * world * capacity + r * capacity
  // (accumulated there by earlier kernels on the same stream); `sharded` is ignored and nothing is copied.
  int32_t n, capacity, world, rank, flag_base, pull;
  uint32_t epoch;
  float max_norm;
  uint32_t* status;
};
int dpk_norm_allreduce_clip(const struct DpkNormAllReduce* p, cudaStream_t stream);

// C[M, N] = A[M, K] B[N, K]^T (bf16, K contiguous) alone or fused with a collective over <= 8 NVLink peers:
//   mode 0 plain; mode 1 all-gather of A's rows first; mode 2 all-gather of B's rows first;
//   mode 3 reduce-scatter of C's rows afterwards (out = this rank's M / world rows).
// Gather modes: `a` (mode 1) / `b` (mode 2) is the LOCAL buffer for the whole operand, which the kernel fills
// from shard[r] (rank r's rows, symmetric memory) while it computes; rows must be a multiple of
// world * 128 (mode 1) or world * 256 (mode 2); `ready` = one zero-initialised counter per 128 / 256 rows.
// Mode 3: slots[r] = rank r's symmetric buffer of 2 * M * N bf16; M a multiple of world * 128.
// flags[r]: rank r's symmetric flag words (>= 32, zero-initialised, private to this call site);
// epoch: 1, 2, 3, ... on successive calls with the same buffers.  Modes 1-3 launch cooperatively.
struct DpkTpGemm {
  const void* a;
  const void* b;
  void* out;
  int32_t M, N, K, mode, world, rank, reserved;
  uint32_t epoch;
  const void* shard[8];
  void* slots[8];
  uint32_t* flags[8];
  uint32_t* ready;
  uint32_t* status;
};
int dpk_tp_gemm(const struct DpkTpGemm* p, cudaStream_t stream);

// Token-wise cross entropy from [rows, V] logits (kind: 0 fp32, 1 bf16, 2 fp16).  forward: loss[r], lse[r];
// backward: dlogits = (softmax - onehot) * grad_loss[r] in the logits' precision.  Rows with target ==
// ignore_index give loss 0 / gradient 0.
int dpk_cross_entropy_forward(const void* logits, int kind, const int64_t* target, int64_t rows, int64_t V,
                              int64_t ignore_index, float* loss, float* lse, cudaStream_t stream);
int dpk_cross_entropy_backward(const void* logits, int kind, const int64_t* target, const float* lse,
                               const float* grad_loss, int64_t rows, int64_t V, int64_t ignore_index, void* dlogits,
                               cudaStream_t stream);

// Rotary embedding.  Source / destination are token-major [B, T, H, hd] (flag 0) or head-major [B, H, T, hd]
// (flag 1).  sign = +1 rotates, -1 rotates back (the gradient).  hd a multiple of 16; pointers 16-byte aligned.
int dpk_rope(const void* in, void* out, int kind, int64_t B, int64_t T, int64_t H, int hd, float theta, int src_heads,
             int dst_heads, float sign, cudaStream_t stream);

// SwiGLU: h = silu(gate) * up over n elements (n a multiple of 8, 16-byte aligned), and its gradient.
int dpk_swiglu_forward(const void* gate, const void* up, void* h, int kind, int64_t n, cudaStream_t stream);
int dpk_swiglu_backward(const void* gate, const void* up, const void* dh, void* dgate, void* dup, int kind, int64_t n,
                        cudaStream_t stream);

// Residual add + RMSNorm over [rows, D] (D a multiple of 8, at most 8192; kind 0 fp32 / 1 bf16 / 2 fp16; w has the same
// type).  forward: h = x + delta (delta NULL: h = x and h_out is not written), y = h * rstd * w, rstd[rows] kept.
// backward: dh = (dres or 0) + gradient of the norm with respect to h.
int dpk_add_rmsnorm_forward(const void* x, const void* delta, const void* w, void* h_out, void* y_out, float* rstd_out,
                            int kind, int64_t rows, int64_t D, float eps, cudaStream_t stream);
int dpk_add_rmsnorm_backward(const void* dy, const void* dres, const void* h, const float* rstd, const void* w,
                             void* dh_out, int kind, int64_t rows, int64_t D, cudaStream_t stream);

// Standard normal samples (testing the generator): out[i] for i < n.
int dpk_philox_normal(float* out, int64_t n, uint64_t seed, uint64_t offset, float std, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
