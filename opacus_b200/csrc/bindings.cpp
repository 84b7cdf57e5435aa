// Python bindings (module opacus_b200._C): thin tensor -> pointer marshalling
// around the C interface in api.h.  All work is enqueued on the current torch
// CUDA stream.  A kernel that gives up on a bounded wait records a code in a
// pinned, device-visible status block; every call checks that block first and
// raises if an earlier kernel failed.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <mutex>
#include <sstream>
#include <stdexcept>
#include <vector>

#include "api.h"

namespace {

struct StatusBlock {
  uint32_t* host = nullptr;
  uint32_t* dev = nullptr;
};
StatusBlock g_status[64];
std::mutex g_mu;

// Debug mode (OPACUS_B200_DEBUG=1 or set_debug(true)): every buffer a binding allocates for a kernel to fill starts
// as all-ones bytes, which reads as NaN in fp32 / bf16 / fp16 -- an element a kernel failed to write (a tile missed at
// an odd size, a predicate that is off by one) then shows in the result instead of being whatever the allocator left.
bool g_debug = [] {
  const char* e = getenv("OPACUS_B200_DEBUG");
  return e != nullptr && e[0] != '\0' && e[0] != '0';
}();

at::Tensor poison(at::Tensor t) {
  if (g_debug && t.defined() && t.is_cuda() && t.numel() > 0)
    cudaMemsetAsync(t.data_ptr(), 0xFF, t.nbytes(), at::cuda::getCurrentCUDAStream());
  return t;
}
at::Tensor new_out(at::IntArrayRef sizes, const at::TensorOptions& opt) { return poison(at::empty(sizes, opt)); }
at::Tensor new_out_like(const at::Tensor& t) { return poison(at::empty_like(t)); }

StatusBlock& status_for(int device) {
  std::lock_guard<std::mutex> lock(g_mu);
  StatusBlock& s = g_status[device & 63];
  if (s.host == nullptr) {
    void* h = nullptr;
    TORCH_CHECK(cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess,
                "opacus_b200: cannot allocate the kernel status block");
    memset(h, 0, 64);
    void* d = nullptr;
    TORCH_CHECK(cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess, "opacus_b200: cannot map the kernel status block");
    s.host = static_cast<uint32_t*>(h);
    s.dev = static_cast<uint32_t*>(d);
  }
  return s;
}

// The message below is turned into opacus_b200.utils.errors.CommTimeoutError by the Python wrapper (ops/_cuda.py).
void raise_if_failed(int device) {
  StatusBlock& s = status_for(device);
  const uint32_t code = *reinterpret_cast<volatile uint32_t*>(s.host);
  if (code != 0) {
    const uint32_t blk = s.host[1], d0 = s.host[2], d1 = s.host[3];
    s.host[0] = s.host[1] = s.host[2] = s.host[3] = 0;
    // Formatted with snprintf on purpose: number insertion into a std::ostream (which TORCH_CHECK uses for
    // non-string pieces) crashed in processes that had the CUDA libraries loaded.
    char msg[256];
    snprintf(msg, sizeof(msg),
             "opacus_b200: a kernel gave up on a bounded wait (site %u, code %u, block %u, detail %u/%u); "
             "its results are invalid", code >> 8, code & 0xffu, blk, d0, d1);
    TORCH_CHECK(false, msg);
  }
}

// Error messages are assembled with snprintf and handed to TORCH_CHECK as ONE string: anything else goes through a
// std::ostream inside TORCH_CHECK, and stream formatting crashed in processes that had the CUDA libraries loaded.
void check(int rc, const char* what) {
  if (rc == 0) return;
  char msg[256];
  snprintf(msg, sizeof(msg), "opacus_b200: %s failed: %s", what, cudaGetErrorString(static_cast<cudaError_t>(rc)));
  TORCH_CHECK(false, msg);
}

int elem_kind(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: {
      char msg[128];
      snprintf(msg, sizeof(msg), "opacus_b200: unsupported dtype %s", c10::toString(t.scalar_type()));
      TORCH_CHECK(false, msg);
    }
  }
}

void need_cuda_contig(const at::Tensor& t, const char* name) {
  if (t.is_cuda() && t.is_contiguous()) return;
  char msg[160];
  snprintf(msg, sizeof(msg), "opacus_b200: %s must be a contiguous CUDA tensor", name);
  TORCH_CHECK(false, msg);
}

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// ------------------------------------------------------------------ ghost norms
// x: [B,T,dx] bf16 or None; ids: [B,T] int64 or None; g: [B,T,dg] bf16.
void gram_pair_norm(c10::optional<at::Tensor> x, c10::optional<at::Tensor> ids, at::Tensor g, double scale,
                    at::Tensor scratch, c10::optional<at::Tensor> out_w, c10::optional<at::Tensor> out_b,
                    bool accumulate, int64_t right_off, int64_t logical_T) {
  c10::cuda::CUDAGuard guard(g.device());
  raise_if_failed(g.get_device());
  need_cuda_contig(g, "g");
  TORCH_CHECK(g.dim() == 3 && g.scalar_type() == at::kBFloat16, "g must be [B,T,d] bf16");
  // right_off > 0: tensors are [B, 2 * right_off, d] (left rows, then right rows) and logical_T is the true T
  TORCH_CHECK(right_off == 0 || (g.size(1) == 2 * right_off && logical_T > 0 && logical_T <= right_off),
              "with right_off the operands must have 2 * right_off rows per sample");
  const int B = g.size(0), T = right_off > 0 ? (int)logical_T : (int)g.size(1), dg = g.size(2);
  const int rows_in = g.size(1);
  const void* xp = nullptr;
  int dx = 0;
  if (x.has_value()) {
    need_cuda_contig(*x, "x");
    TORCH_CHECK(x->dim() == 3 && x->scalar_type() == at::kBFloat16 && x->size(0) == B && x->size(1) == rows_in,
                "x must be [B,T,d] bf16");
    xp = x->data_ptr();
    dx = x->size(2);
  }
  const int64_t* idp = nullptr;
  if (ids.has_value()) {
    need_cuda_contig(*ids, "ids");
    TORCH_CHECK(ids->scalar_type() == at::kLong && ids->numel() == (int64_t)B * T, "ids must be [B,T] int64");
    idp = ids->data_ptr<int64_t>();
  }
  TORCH_CHECK(scratch.is_cuda() && scratch.scalar_type() == at::kFloat &&
                  (size_t)scratch.numel() >= dpk_gram_pair_scratch_floats(B, T),
              "scratch too small");
  float* ow = out_w.has_value() ? out_w->data_ptr<float>() : nullptr;
  float* ob = out_b.has_value() ? out_b->data_ptr<float>() : nullptr;
  check(dpk_gram_pair_norm_lr(xp, idp, g.data_ptr(), B, T, dx, dg, (int)right_off, (float)scale,
                              scratch.data_ptr<float>(), ow, ob, accumulate ? 1 : 0, status_for(g.get_device()).dev,
                              stream()),
        "gram_pair_norm");
}

int64_t gram_pair_scratch_floats(int64_t B, int64_t T) { return (int64_t)dpk_gram_pair_scratch_floats(B, T); }

// ------------------------------------------------------------------ clipped weight gradient
void wgrad_tn(at::Tensor gs, at::Tensor a, at::Tensor out, double beta) {
  c10::cuda::CUDAGuard guard(gs.device());
  raise_if_failed(gs.get_device());
  need_cuda_contig(gs, "gs");
  need_cuda_contig(a, "a");
  need_cuda_contig(out, "out");
  TORCH_CHECK(gs.dim() == 2 && a.dim() == 2 && gs.size(0) == a.size(0), "gs [K,M] and a [K,N] expected");
  TORCH_CHECK(gs.scalar_type() == at::kBFloat16 && a.scalar_type() == at::kBFloat16, "bf16 operands expected");
  const int K = gs.size(0), M = gs.size(1), N = a.size(1);
  TORCH_CHECK(out.numel() == (int64_t)M * N, "out must have M*N elements");
  TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16, "out must be fp32 or bf16");
  check(dpk_wgrad_tn(gs.data_ptr(), a.data_ptr(), K, M, N, out.data_ptr(), out.scalar_type() == at::kBFloat16,
                     (float)beta, status_for(gs.get_device()).dev, stream()),
        "wgrad_tn");
}

// The pair-of-SMs form of wgrad_tn (fp32 out only); splits = 0 lets the binding choose.
void wgrad2_tn(at::Tensor gs, at::Tensor a, at::Tensor out, double beta, int64_t splits) {
  c10::cuda::CUDAGuard guard(gs.device());
  raise_if_failed(gs.get_device());
  need_cuda_contig(gs, "gs");
  need_cuda_contig(a, "a");
  need_cuda_contig(out, "out");
  TORCH_CHECK(gs.dim() == 2 && a.dim() == 2 && gs.size(0) == a.size(0), "gs [K,M] and a [K,N] expected");
  TORCH_CHECK(gs.scalar_type() == at::kBFloat16 && a.scalar_type() == at::kBFloat16, "bf16 operands expected");
  const int K = gs.size(0), M = gs.size(1), N = a.size(1);
  TORCH_CHECK(out.numel() == (int64_t)M * N && out.scalar_type() == at::kFloat, "out must be fp32 with M*N elements");
  if (splits <= 0) splits = 1;
  check(dpk_wgrad2_tn(gs.data_ptr(), a.data_ptr(), K, M, N, out.data_ptr<float>(), (float)beta, (int)splits,
                      status_for(gs.get_device()).dev, stream()),
        "wgrad2_tn");
}

// gs [batch, K, M] (or [K, M]), a [batch, K, N] (or [K, N]) bf16; out [batch, M, N]; norm_sq optional fp32 [batch]
void wgrad_tn_ex(at::Tensor gs, at::Tensor a, c10::optional<at::Tensor> out_opt, double beta,
                 c10::optional<at::Tensor> norm_sq, int64_t force_bm, int64_t force_bn, int64_t force_splits) {
  c10::cuda::CUDAGuard guard(gs.device());
  raise_if_failed(gs.get_device());
  need_cuda_contig(gs, "gs");
  need_cuda_contig(a, "a");
  if (out_opt.has_value()) need_cuda_contig(*out_opt, "out");
  TORCH_CHECK(out_opt.has_value() || norm_sq.has_value(), "nothing to compute: neither out nor norm_sq given");
  TORCH_CHECK(gs.scalar_type() == at::kBFloat16 && a.scalar_type() == at::kBFloat16, "bf16 operands expected");
  TORCH_CHECK(gs.dim() == a.dim() && (gs.dim() == 2 || gs.dim() == 3), "gs and a must both be 2-d or 3-d");
  const int batch = gs.dim() == 3 ? gs.size(0) : 1;
  const int K = gs.size(-2), M = gs.size(-1), N = a.size(-1);
  TORCH_CHECK(a.size(-2) == K && (a.dim() == 2 || a.size(0) == batch), "gs and a disagree on batch / K");
  void* out_ptr = nullptr;
  bool out_bf16 = false;
  if (out_opt.has_value()) {
    const at::Tensor& out = *out_opt;
    TORCH_CHECK(out.numel() == (int64_t)batch * M * N, "out must have batch*M*N elements");
    TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16, "out must be fp32 or bf16");
    out_ptr = out.data_ptr();
    out_bf16 = out.scalar_type() == at::kBFloat16;
  }
  float* nsq = nullptr;
  if (norm_sq.has_value()) {
    TORCH_CHECK(norm_sq->is_cuda() && norm_sq->scalar_type() == at::kFloat && norm_sq->numel() == batch, "bad norm_sq");
    nsq = norm_sq->data_ptr<float>();
  }
  check(dpk_wgrad_tn_ex(gs.data_ptr(), a.data_ptr(), K, M, N, batch, out_ptr, out_bf16, (float)beta, nsq,
                        (int)force_bm, (int)force_bn,
                        (int)force_splits, status_for(gs.get_device()).dev, stream()),
        "wgrad_tn_ex");
}

// x [B, H, W, C], g [B, OH, OW, O] bf16 contiguous (channels-last images); conv = {kh, kw, sh, sw, ph, pw, dh, dw};
// out [B, O, kh, kw, C] (or [O, kh, kw, C] fp32 when reduce_batch); norm_sq optional fp32 [B]
void conv_psg(at::Tensor x, at::Tensor g, std::vector<int64_t> conv, bool reduce_batch,
              c10::optional<at::Tensor> out_opt, double beta, c10::optional<at::Tensor> norm_sq) {
  c10::cuda::CUDAGuard guard(x.device());
  raise_if_failed(x.get_device());
  need_cuda_contig(x, "x");
  need_cuda_contig(g, "g");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kBFloat16, "bf16 operands expected");
  TORCH_CHECK(x.dim() == 4 && g.dim() == 4 && x.size(0) == g.size(0), "x [B,H,W,C] and g [B,OH,OW,O] expected");
  TORCH_CHECK(conv.size() == 8, "conv = {kh, kw, sh, sw, ph, pw, dh, dw}");
  TORCH_CHECK(out_opt.has_value() || norm_sq.has_value(), "nothing to compute: neither out nor norm_sq given");
  const int B = x.size(0), H = x.size(1), W = x.size(2), C = x.size(3);
  const int OH = g.size(1), OW = g.size(2), O = g.size(3);
  const int kh = conv[0], kw = conv[1], sh = conv[2], sw = conv[3], ph = conv[4], pw = conv[5], dh = conv[6], dw = conv[7];
  TORCH_CHECK((OH - 1) * sh + (kh - 1) * dh - ph < H + ph && (OW - 1) * sw + (kw - 1) * dw - pw < W + pw,
              "output size does not fit the input for this convolution");
  void* out_ptr = nullptr;
  bool out_bf16 = false;
  if (out_opt.has_value()) {
    const at::Tensor& out = *out_opt;
    need_cuda_contig(out, "out");
    TORCH_CHECK(out.numel() == (int64_t)(reduce_batch ? 1 : B) * O * kh * kw * C, "out has the wrong number of elements");
    TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16, "out must be fp32 or bf16");
    out_ptr = out.data_ptr();
    out_bf16 = out.scalar_type() == at::kBFloat16;
  }
  float* nsq = nullptr;
  if (norm_sq.has_value()) {
    TORCH_CHECK(norm_sq->is_cuda() && norm_sq->scalar_type() == at::kFloat && norm_sq->numel() == B, "bad norm_sq");
    nsq = norm_sq->data_ptr<float>();
  }
  check(dpk_conv_psg(x.data_ptr(), g.data_ptr(), B, C, H, W, O, OH, OW, kh, kw, sh, sw, ph, pw, dh, dw, reduce_batch,
                     out_ptr, out_bf16, (float)beta, nsq, status_for(x.get_device()).dev, stream()),
        "conv_psg");
}

// ids [B, T] int64; g_e, a_h [B, T, D] bf16; g_h [B, T, V] bf16 / fp32 -> out [B] fp32 (added to `total` if given)
at::Tensor tied_cross_norm(at::Tensor ids, at::Tensor g_e, at::Tensor a_h, at::Tensor g_h, double scale,
                           c10::optional<at::Tensor> total) {
  c10::cuda::CUDAGuard guard(g_e.device());
  raise_if_failed(g_e.get_device());
  need_cuda_contig(ids, "ids");
  need_cuda_contig(g_e, "g_e");
  need_cuda_contig(a_h, "a_h");
  need_cuda_contig(g_h, "g_h");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.dim() == 2, "ids must be int64 [B, T]");
  TORCH_CHECK(g_e.scalar_type() == at::kBFloat16 && a_h.scalar_type() == at::kBFloat16, "g_e and a_h must be bf16");
  TORCH_CHECK(g_h.scalar_type() == at::kBFloat16 || g_h.scalar_type() == at::kFloat, "g_h must be bf16 or fp32");
  const int B = ids.size(0), T = ids.size(1);
  TORCH_CHECK(g_e.dim() == 3 && a_h.dim() == 3 && g_h.dim() == 3 && g_e.size(0) == B && g_e.size(1) == T &&
              a_h.size(0) == B && a_h.size(1) == T && g_h.size(0) == B && g_h.size(1) == T &&
              a_h.size(2) == g_e.size(2), "shapes: g_e, a_h [B, T, D], g_h [B, T, V]");
  const int D = g_e.size(2);
  const int64_t V = g_h.size(2);
  const int64_t nT = (T + 127) / 128;
  at::Tensor scratch = new_out({2 * (int64_t)B * nT * nT}, g_e.options().dtype(at::kFloat));
  at::Tensor out;
  int accumulate = 0;
  if (total.has_value()) {
    TORCH_CHECK(total->is_cuda() && total->scalar_type() == at::kFloat && total->is_contiguous() && total->numel() == B,
                "total must be a contiguous fp32 CUDA vector of B elements");
    out = *total;
    accumulate = 1;
  } else {
    out = new_out({B}, g_e.options().dtype(at::kFloat));
  }
  check(dpk_tied_cross_norm(ids.data_ptr<int64_t>(), g_e.data_ptr(), a_h.data_ptr(), g_h.data_ptr(),
                            g_h.scalar_type() == at::kFloat, B, T, D, V, (float)scale, scratch.data_ptr<float>(),
                            out.data_ptr<float>(), accumulate, status_for(g_e.get_device()).dev, stream()),
        "tied_cross_norm");
  return out;
}

at::Tensor scale_rows(at::Tensor x, c10::optional<at::Tensor> c, int64_t rows_per_sample, double scale) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2, "x must be [rows, cols]");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "x must be fp32 or bf16");
  at::Tensor y = new_out(x.sizes(), x.options().dtype(at::kBFloat16));
  const float* cp = nullptr;
  if (c.has_value()) {
    TORCH_CHECK(c->is_cuda() && c->scalar_type() == at::kFloat && c->is_contiguous(), "c must be fp32 CUDA");
    cp = c->data_ptr<float>();
  }
  check(dpk_scale_rows(x.data_ptr(), x.scalar_type() == at::kFloat, cp, y.data_ptr(), x.size(0), x.size(1),
                       rows_per_sample, (float)scale, stream()),
        "scale_rows");
  return y;
}

// x fp32 [rows, cols] -> bf16 [rows / T, 3 * T, cols] (see dpk_split3_rows)
at::Tensor split3_rows(at::Tensor x, c10::optional<at::Tensor> c, int64_t T, double scale, bool right) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.scalar_type() == at::kFloat, "x must be fp32 [rows, cols]");
  TORCH_CHECK(T > 0 && x.size(0) % T == 0 && x.size(1) % 8 == 0, "rows must be a multiple of T and cols of 8");
  at::Tensor y = new_out({x.size(0) / T, 3 * T, x.size(1)}, x.options().dtype(at::kBFloat16));
  const float* cp = nullptr;
  if (c.has_value()) {
    TORCH_CHECK(c->is_cuda() && c->scalar_type() == at::kFloat && c->is_contiguous() && c->numel() == x.size(0) / T,
                "c must be fp32 CUDA, one value per sample");
    cp = c->data_ptr<float>();
  }
  check(dpk_split3_rows(x.data_ptr<float>(), cp, y.data_ptr(), x.size(0), x.size(1), T, (float)scale, right ? 1 : 0,
                        stream()),
        "split3_rows");
  return y;
}

// ChaCha20 keystream words / Gaussians into `out` (see dpk_chacha_words, dpk_chacha_normal); nonce and first block
// are passed as Python ints below 2^64.
void chacha_words(at::Tensor out, std::vector<int64_t> key, py::int_ nonce, py::int_ first_block) {
  c10::cuda::CUDAGuard guard(out.device());
  need_cuda_contig(out, "out");
  TORCH_CHECK(out.scalar_type() == at::kInt && out.numel() % 16 == 0, "out must be int32 with a multiple of 16 elements");
  TORCH_CHECK(key.size() == 8, "key must have eight 32-bit words");
  uint32_t k[8];
  for (int i = 0; i < 8; ++i) k[i] = (uint32_t)key[i];
  check(dpk_chacha_words(reinterpret_cast<uint32_t*>(out.data_ptr<int>()), out.numel() / 16, k,
                         nonce.cast<uint64_t>(), first_block.cast<uint64_t>(), stream()),
        "chacha_words");
}

void chacha_normal(at::Tensor out, std::vector<int64_t> key, py::int_ nonce, py::int_ first_block, double std,
                   int64_t draws) {
  c10::cuda::CUDAGuard guard(out.device());
  need_cuda_contig(out, "out");
  TORCH_CHECK(out.scalar_type() == at::kFloat, "out must be fp32");
  TORCH_CHECK(key.size() == 8, "key must have eight 32-bit words");
  uint32_t k[8];
  for (int i = 0; i < 8; ++i) k[i] = (uint32_t)key[i];
  check(dpk_chacha_normal(out.data_ptr<float>(), out.numel(), k, nonce.cast<uint64_t>(), first_block.cast<uint64_t>(),
                          (float)std, (int)draws, stream()),
        "chacha_normal");
}

at::Tensor clip_factor(at::Tensor n2, double C) {
  c10::cuda::CUDAGuard guard(n2.device());
  need_cuda_contig(n2, "norm_sq");
  TORCH_CHECK(n2.scalar_type() == at::kFloat, "norm_sq must be fp32");
  at::Tensor c = new_out_like(n2);
  check(dpk_clip_factor(n2.data_ptr<float>(), c.data_ptr<float>(), n2.numel(), (float)C, stream()), "clip_factor");
  return c;
}

at::Tensor row_norm_sq(at::Tensor x) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  const int64_t B = x.size(0);
  at::Tensor out = new_out({B}, x.options().dtype(at::kFloat));
  check(dpk_row_norm_sq(x.data_ptr(), elem_kind(x), B, B ? x.numel() / B : 0, out.data_ptr<float>(), 0, stream()),
        "row_norm_sq");
  return out;
}

at::Tensor weighted_sum(at::Tensor x, at::Tensor c, c10::optional<at::Tensor> dest) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  need_cuda_contig(c, "c");
  TORCH_CHECK(c.scalar_type() == at::kFloat && c.numel() == x.size(0), "c must be fp32 [B]");
  const int64_t B = x.size(0), cols = x.numel() / B;
  at::Tensor out;
  if (dest.has_value()) {             // overwritten in place
    TORCH_CHECK(dest->is_cuda() && dest->scalar_type() == at::kFloat && dest->is_contiguous() && dest->numel() == cols,
                "dest must be a contiguous fp32 CUDA tensor with one element per column");
    out = *dest;
  } else {
    out = new_out({cols}, x.options().dtype(at::kFloat));
  }
  check(dpk_weighted_sum(x.data_ptr(), elem_kind(x), c.data_ptr<float>(), B, cols, out.data_ptr<float>(), stream()),
        "weighted_sum");
  return out;
}

void outer_norm_sq(c10::optional<at::Tensor> a, at::Tensor g, double scale, c10::optional<at::Tensor> out_w,
                   c10::optional<at::Tensor> out_b, bool accumulate) {
  c10::cuda::CUDAGuard guard(g.device());
  need_cuda_contig(g, "g");
  const int64_t B = g.size(0);
  const void* ap = nullptr;
  int64_t da = 0;
  if (a.has_value()) {
    need_cuda_contig(*a, "a");
    TORCH_CHECK(a->scalar_type() == g.scalar_type(), "a and g must share a dtype");
    ap = a->data_ptr();
    da = a->numel() / B;
  }
  check(dpk_outer_norm_sq(ap, g.data_ptr(), elem_kind(g), B, da, g.numel() / B, (float)scale,
                          out_w.has_value() ? out_w->data_ptr<float>() : nullptr,
                          out_b.has_value() ? out_b->data_ptr<float>() : nullptr, accumulate, stream()),
        "outer_norm_sq");
}

std::vector<at::Tensor> norm_lastdim_grad(int64_t kind, at::Tensor x, at::Tensor g, int64_t d, double eps,
                                          bool want_w, bool want_b) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  need_cuda_contig(g, "g");
  TORCH_CHECK(x.scalar_type() == g.scalar_type() && x.numel() == g.numel(), "x and g must match");
  const int64_t B = x.size(0), rows = x.numel() / B / d;
  auto opt = x.options().dtype(at::kFloat);
  at::Tensor gw = want_w ? new_out({B, d}, opt) : at::Tensor();
  at::Tensor gb = want_b ? new_out({B, d}, opt) : at::Tensor();
  at::Tensor stats = new_out({B * rows * 2}, opt);
  check(dpk_norm_lastdim_grad((int)kind, x.data_ptr(), g.data_ptr(), elem_kind(x), B, rows, d, (float)eps,
                              stats.data_ptr<float>(), want_w ? gw.data_ptr<float>() : nullptr,
                              want_b ? gb.data_ptr<float>() : nullptr, stream()),
        "norm_lastdim_grad");
  return {gw, gb};
}

// One launch: {gw [B, d], gb [B, d] or undefined, n2w [B], n2b [B] or undefined}; an empty vector when the shape is
// outside what the fused kernel covers (the caller then uses norm_lastdim_grad + row_norm_sq).
std::vector<at::Tensor> norm_lastdim_psg(int64_t kind, at::Tensor x, at::Tensor g, int64_t d, double eps, bool want_b) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  need_cuda_contig(g, "g");
  TORCH_CHECK(x.scalar_type() == g.scalar_type() && x.numel() == g.numel(), "x and g must match");
  const int64_t B = x.size(0), rows = x.numel() / B / d;
  if ((d & 7) || d > 4096 || (want_b && d > 2048) || B > 65535 || B == 0 || rows == 0) return {};
  const int64_t per = B * d;
  at::Tensor gw = new_out({B, d}, x.options().dtype(at::kFloat));
  at::Tensor gb = want_b ? new_out({B, d}, x.options().dtype(at::kFloat)) : at::Tensor();
  // small zeroed block: the two norm vectors and the ticket counters
  at::Tensor small = at::zeros({B * 3}, x.options().dtype(at::kFloat));
  at::Tensor n2w = small.narrow(0, 0, B);
  at::Tensor n2b = want_b ? small.narrow(0, B, B) : at::Tensor();
  unsigned int* tickets = reinterpret_cast<unsigned int*>(small.data_ptr<float>() + 2 * B);
  at::Tensor part = at::empty({dpk_norm_lastdim_psg_scratch_floats(B, rows, d, want_b ? 1 : 0)},
                              x.options().dtype(at::kFloat));
  (void)per;
  const int rc = dpk_norm_lastdim_psg_fused((int)kind, x.data_ptr(), g.data_ptr(), elem_kind(x), B, rows, d, (float)eps,
                                            gw.data_ptr<float>(), want_b ? gb.data_ptr<float>() : nullptr,
                                            n2w.data_ptr<float>(), want_b ? n2b.data_ptr<float>() : nullptr, 0, tickets,
                                            part.data_ptr<float>(), stream());
  if (rc == cudaErrorNotSupported) return {};
  check(rc, "norm_lastdim_psg");
  return {gw, gb, n2w, n2b};
}

std::vector<at::Tensor> norm_channel_grad(at::Tensor x, at::Tensor g, int64_t groups, double eps, bool want_w,
                                          bool want_b) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  need_cuda_contig(g, "g");
  TORCH_CHECK(x.scalar_type() == g.scalar_type() && x.numel() == g.numel() && x.dim() >= 2, "x and g must match");
  const int64_t B = x.size(0), C = x.size(1), S = x.numel() / B / C;
  auto opt = x.options().dtype(at::kFloat);
  at::Tensor gw = want_w ? new_out({B, C}, opt) : at::Tensor();
  at::Tensor gb = want_b ? new_out({B, C}, opt) : at::Tensor();
  check(dpk_norm_channel_grad(x.data_ptr(), g.data_ptr(), elem_kind(x), B, C, S, (int)groups, (float)eps,
                              want_w ? gw.data_ptr<float>() : nullptr, want_b ? gb.data_ptr<float>() : nullptr,
                              stream()),
        "norm_channel_grad");
  return {gw, gb};
}

void embedding_scatter(at::Tensor ids, at::Tensor g, at::Tensor c, int64_t T, int64_t padding_idx, double scale,
                       at::Tensor out) {
  c10::cuda::CUDAGuard guard(g.device());
  need_cuda_contig(ids, "ids");
  need_cuda_contig(g, "g");
  need_cuda_contig(out, "out");
  TORCH_CHECK(ids.scalar_type() == at::kLong && out.scalar_type() == at::kFloat && c.scalar_type() == at::kFloat,
              "ids int64, out fp32, c fp32 expected");
  const int64_t rows = ids.numel(), D = g.numel() / rows, V = out.size(0);
  check(dpk_embedding_scatter(ids.data_ptr<int64_t>(), g.data_ptr(), elem_kind(g), c.data_ptr<float>(), rows, T, D, V,
                              padding_idx, (float)scale, out.data_ptr<float>(), stream()),
        "embedding_scatter");
}

// ------------------------------------------------------------------ fused DP step
// table: uint8 CUDA tensor holding n DpkTensorEntry records; prefix: int64 CUDA [n+1].
void fused_dp_step(at::Tensor table, at::Tensor prefix, int64_t n_tensors, int64_t total_chunks, int64_t kind,
                   bool nesterov, bool first_step, double lr, double momentum, double dampening, double weight_decay,
                   double beta1, double beta2, double eps, double bias_c1, double bias_c2_sqrt, double noise_std,
                   double inv_scale, int64_t seed, int64_t offset) {
  c10::cuda::CUDAGuard guard(table.device());
  raise_if_failed(table.get_device());
  TORCH_CHECK(table.is_cuda() && prefix.is_cuda() && prefix.scalar_type() == at::kLong, "bad table");
  TORCH_CHECK((size_t)table.numel() >= sizeof(DpkTensorEntry) * (size_t)n_tensors, "table too small");
  DpkStepHyper h{};
  h.kind = (int)kind; h.nesterov = nesterov; h.first_step = first_step;
  h.lr = (float)lr; h.momentum = (float)momentum; h.dampening = (float)dampening; h.weight_decay = (float)weight_decay;
  h.beta1 = (float)beta1; h.beta2 = (float)beta2; h.eps = (float)eps; h.bias_c1 = (float)bias_c1;
  h.bias_c2_sqrt = (float)bias_c2_sqrt; h.noise_std = (float)noise_std; h.inv_scale = (float)inv_scale;
  h.seed = (uint64_t)seed; h.offset = (uint64_t)offset;
  check(dpk_fused_dp_step(reinterpret_cast<const DpkTensorEntry*>(table.data_ptr()), (int)n_tensors, total_chunks,
                          prefix.data_ptr<int64_t>(), h, stream()),
        "fused_dp_step");
}

// ------------------------------------------------------------------ sharded DP step over peer memory
void sharded_dp_step(std::vector<int64_t> grad_ptrs, std::vector<int64_t> param_ptrs, std::vector<int64_t> flag_ptrs,
                     at::Tensor master, c10::optional<at::Tensor> state0, c10::optional<at::Tensor> state1,
                     int64_t slice_begin, int64_t slice_len, int64_t rank, bool param_bf16, int64_t epoch,
                     int64_t kind, bool nesterov, bool first_step, double lr, double momentum, double dampening,
                     double weight_decay, double beta1, double beta2, double eps, double bias_c1,
                     double bias_c2_sqrt, double noise_std, double inv_scale, int64_t seed, int64_t offset,
                     int64_t noise_split, int64_t noise_shift, int64_t grad_mc, int64_t param_mc,
                     c10::optional<at::Tensor> segments, int64_t max_blocks, int64_t stripe_len,
                     int64_t stripe_stride) {
  c10::cuda::CUDAGuard guard(master.device());
  raise_if_failed(master.get_device());
  const int world = (int)grad_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)param_ptrs.size() == world && (int)flag_ptrs.size() == world,
              "sharded_dp_step supports 1..8 ranks");
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.numel() >= slice_len, "bad master");
  DpkShardedStep p{};
  for (int r = 0; r < world; ++r) {
    p.grad[r] = reinterpret_cast<const float*>(grad_ptrs[r]);
    p.param[r] = reinterpret_cast<void*>(param_ptrs[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.master = master.data_ptr<float>();
  p.state0 = state0.has_value() ? state0->data_ptr<float>() : nullptr;
  p.state1 = state1.has_value() ? state1->data_ptr<float>() : nullptr;
  p.slice_begin = slice_begin; p.slice_len = slice_len;
  p.grad_mc = reinterpret_cast<const float*>(grad_mc);
  p.param_mc = reinterpret_cast<void*>(param_mc);
  p.max_blocks = (int)max_blocks;
  p.stripe_len = stripe_len; p.stripe_stride = stripe_stride;
  if (segments.has_value()) {
    TORCH_CHECK(segments->is_cuda() && segments->scalar_type() == at::kByte && segments->is_contiguous() &&
                segments->numel() % sizeof(DpkStepSegment) == 0, "segments must be a CUDA byte tensor of DpkStepSegment");
    p.segs = reinterpret_cast<const DpkStepSegment*>(segments->data_ptr());
    p.nseg = (int)(segments->numel() / sizeof(DpkStepSegment));
  }
  TORCH_CHECK(noise_split >= 0 && noise_shift >= 0 && noise_split % 8 == 0 && noise_shift % 8 == 0,
              "noise_split and noise_shift must be non-negative multiples of 8");
  p.noise_split = noise_split; p.noise_shift = noise_shift;
  p.world = world; p.rank = (int)rank; p.param_bf16 = param_bf16 ? 1 : 0;
  p.epoch = (uint32_t)epoch;
  DpkStepHyper& h = p.h;
  h.kind = (int)kind; h.nesterov = nesterov; h.first_step = first_step;
  h.lr = (float)lr; h.momentum = (float)momentum; h.dampening = (float)dampening; h.weight_decay = (float)weight_decay;
  h.beta1 = (float)beta1; h.beta2 = (float)beta2; h.eps = (float)eps; h.bias_c1 = (float)bias_c1;
  h.bias_c2_sqrt = (float)bias_c2_sqrt; h.noise_std = (float)noise_std; h.inv_scale = (float)inv_scale;
  h.seed = (uint64_t)seed; h.offset = (uint64_t)offset;
  p.status = status_for(master.get_device()).dev;
  check(dpk_sharded_dp_step(&p, stream()), "sharded_dp_step");
}

// Peer-memory all-reduce of a [n] fp32 vector + clip factor.  Returns {total, clip}.
std::vector<at::Tensor> norm_allreduce_clip(std::vector<int64_t> slot_ptrs, std::vector<int64_t> flag_ptrs,
                                            c10::optional<at::Tensor> sharded, c10::optional<at::Tensor> replicated,
                                            int64_t n, int64_t capacity, int64_t rank, int64_t flag_base, int64_t epoch,
                                            double max_norm, at::Device device, bool pull) {
  c10::cuda::CUDAGuard guard(device);
  raise_if_failed(device.index());
  const int world = (int)slot_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && (int)flag_ptrs.size() == world, "norm_allreduce_clip supports 1..8 ranks");
  DpkNormAllReduce p{};
  for (int r = 0; r < world; ++r) {
    p.slots[r] = reinterpret_cast<float*>(slot_ptrs[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  auto vec = [&](const c10::optional<at::Tensor>& t, const char* what) -> const float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n, what);
    return t->data_ptr<float>();
  };
  p.sharded = vec(sharded, "sharded must be a contiguous fp32 CUDA vector of n elements");
  p.replicated = vec(replicated, "replicated must be a contiguous fp32 CUDA vector of n elements");
  at::Tensor total = new_out({n}, at::TensorOptions().device(device).dtype(at::kFloat));
  at::Tensor clip = new_out({n}, at::TensorOptions().device(device).dtype(at::kFloat));
  p.total_out = total.data_ptr<float>();
  p.clip_out = clip.data_ptr<float>();
  p.n = (int)n; p.capacity = (int)capacity; p.world = world; p.rank = (int)rank; p.flag_base = (int)flag_base;
  p.epoch = (uint32_t)epoch; p.max_norm = (float)max_norm; p.pull = pull ? 1 : 0;
  p.status = status_for(device.index()).dev;
  check(dpk_norm_allreduce_clip(&p, stream()), "norm_allreduce_clip");
  return {total, clip};
}

// a [M, K], b [N, K] bf16 contiguous; see DpkTpGemm for the modes.  out: [M, N] (modes 0-2) or [M / world, N].
void tp_gemm(at::Tensor a, at::Tensor b, at::Tensor out, int64_t mode, std::vector<int64_t> shard_ptrs,
             std::vector<int64_t> slot_ptrs, std::vector<int64_t> flag_ptrs, c10::optional<at::Tensor> ready,
             int64_t rank, int64_t world, int64_t epoch, int64_t producers) {
  c10::cuda::CUDAGuard guard(a.device());
  raise_if_failed(a.get_device());
  need_cuda_contig(a, "a");
  need_cuda_contig(b, "b");
  need_cuda_contig(out, "out");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
              out.scalar_type() == at::kBFloat16, "bf16 tensors expected");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a [M, K] and b [N, K] expected");
  TORCH_CHECK(world >= 1 && world <= 8, "1..8 ranks");
  DpkTpGemm p{};
  p.a = a.data_ptr(); p.b = b.data_ptr(); p.out = out.data_ptr();
  p.M = (int)a.size(0); p.N = (int)b.size(0); p.K = (int)a.size(1);
  p.mode = (int)mode; p.world = (int)world; p.rank = (int)rank; p.reserved = 0; (void)producers;
  p.epoch = (uint32_t)epoch;
  TORCH_CHECK(out.numel() == (int64_t)(mode == 3 ? p.M / world : p.M) * p.N, "out has the wrong size");
  if (mode != 0) {
    TORCH_CHECK((int64_t)flag_ptrs.size() == world, "one flag pointer per rank");
    for (int r = 0; r < world; ++r) p.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  if (mode == 1 || mode == 2) {
    TORCH_CHECK((int64_t)shard_ptrs.size() == world, "one shard pointer per rank");
    for (int r = 0; r < world; ++r) p.shard[r] = reinterpret_cast<const void*>(shard_ptrs[r]);
    const int64_t units = mode == 1 ? p.M / 128 : p.N / 256;
    TORCH_CHECK(ready.has_value() && ready->is_cuda() && ready->scalar_type() == at::kInt && ready->is_contiguous() &&
                ready->numel() >= units, "ready must be an int32 CUDA vector with one entry per unit");
    p.ready = reinterpret_cast<uint32_t*>(ready->data_ptr<int>());
  }
  if (mode == 3) {
    TORCH_CHECK((int64_t)slot_ptrs.size() == world, "one slot pointer per rank");
    for (int r = 0; r < world; ++r) p.slots[r] = reinterpret_cast<void*>(slot_ptrs[r]);
  }
  p.status = status_for(a.get_device()).dev;
  check(dpk_tp_gemm(&p, stream()), "tp_gemm");
}

// logits [rows, V] (fp32 / bf16 / fp16, contiguous), target int64 [rows] -> {loss fp32 [rows], lse fp32 [rows]}
std::vector<at::Tensor> cross_entropy_forward(at::Tensor logits, at::Tensor target, int64_t ignore_index) {
  c10::cuda::CUDAGuard guard(logits.device());
  need_cuda_contig(logits, "logits");
  need_cuda_contig(target, "target");
  TORCH_CHECK(logits.dim() == 2 && target.dim() == 1 && target.size(0) == logits.size(0), "logits [rows, V], target [rows]");
  TORCH_CHECK(target.scalar_type() == at::kLong, "target must be int64");
  at::Tensor loss = new_out({logits.size(0)}, logits.options().dtype(at::kFloat));
  at::Tensor lse = new_out({logits.size(0)}, logits.options().dtype(at::kFloat));
  check(dpk_cross_entropy_forward(logits.data_ptr(), elem_kind(logits), target.data_ptr<int64_t>(), logits.size(0),
                                  logits.size(1), ignore_index, loss.data_ptr<float>(), lse.data_ptr<float>(), stream()),
        "cross_entropy_forward");
  return {loss, lse};
}

at::Tensor cross_entropy_backward(at::Tensor logits, at::Tensor target, at::Tensor lse, at::Tensor grad_loss,
                                  int64_t ignore_index) {
  c10::cuda::CUDAGuard guard(logits.device());
  need_cuda_contig(logits, "logits");
  need_cuda_contig(target, "target");
  need_cuda_contig(lse, "lse");
  need_cuda_contig(grad_loss, "grad_loss");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && grad_loss.scalar_type() == at::kFloat &&
              lse.numel() == logits.size(0) && grad_loss.numel() == logits.size(0), "lse / grad_loss: fp32 [rows]");
  at::Tensor dx = new_out_like(logits);
  check(dpk_cross_entropy_backward(logits.data_ptr(), elem_kind(logits), target.data_ptr<int64_t>(),
                                   lse.data_ptr<float>(), grad_loss.data_ptr<float>(), logits.size(0), logits.size(1),
                                   ignore_index, dx.data_ptr(), stream()),
        "cross_entropy_backward");
  return dx;
}

// x contiguous 4-d, token-major [B, T, H, hd] or (src_heads) head-major [B, H, T, hd]; returns the rotated tensor
// in token-major or (dst_heads) head-major layout
at::Tensor rope(at::Tensor x, double theta, bool src_heads, bool dst_heads, double sign) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  TORCH_CHECK(x.dim() == 4, "x must be 4-d");
  const int64_t B = x.size(0), hd = x.size(3);
  const int64_t T = src_heads ? x.size(2) : x.size(1), H = src_heads ? x.size(1) : x.size(2);
  at::Tensor out = dst_heads ? new_out({B, H, T, hd}, x.options()) : new_out({B, T, H, hd}, x.options());
  check(dpk_rope(x.data_ptr(), out.data_ptr(), elem_kind(x), B, T, H, (int)hd, (float)theta, src_heads ? 1 : 0,
                 dst_heads ? 1 : 0, (float)sign, stream()),
        "rope");
  return out;
}

at::Tensor swiglu_forward(at::Tensor gate, at::Tensor up) {
  c10::cuda::CUDAGuard guard(gate.device());
  need_cuda_contig(gate, "gate");
  need_cuda_contig(up, "up");
  TORCH_CHECK(gate.sizes() == up.sizes() && gate.scalar_type() == up.scalar_type(), "gate and up must match");
  at::Tensor h = new_out_like(gate);
  check(dpk_swiglu_forward(gate.data_ptr(), up.data_ptr(), h.data_ptr(), elem_kind(gate), gate.numel(), stream()),
        "swiglu_forward");
  return h;
}

std::vector<at::Tensor> swiglu_backward(at::Tensor gate, at::Tensor up, at::Tensor dh) {
  c10::cuda::CUDAGuard guard(gate.device());
  need_cuda_contig(gate, "gate");
  need_cuda_contig(up, "up");
  need_cuda_contig(dh, "dh");
  TORCH_CHECK(gate.sizes() == up.sizes() && gate.sizes() == dh.sizes() && gate.scalar_type() == up.scalar_type() &&
              gate.scalar_type() == dh.scalar_type(), "gate, up and dh must match");
  at::Tensor dg = new_out_like(gate), du = new_out_like(gate);
  check(dpk_swiglu_backward(gate.data_ptr(), up.data_ptr(), dh.data_ptr(), dg.data_ptr(), du.data_ptr(),
                            elem_kind(gate), gate.numel(), stream()),
        "swiglu_backward");
  return {dg, du};
}

// x, delta (optional) [..., D], w [D], same dtype -> {y, h (== x when delta is absent), rstd fp32 [rows]}
std::vector<at::Tensor> add_rmsnorm_forward(at::Tensor x, c10::optional<at::Tensor> delta, at::Tensor w, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  need_cuda_contig(x, "x");
  need_cuda_contig(w, "w");
  const int64_t D = w.numel(), rows = x.numel() / D;
  TORCH_CHECK(x.size(-1) == D && w.scalar_type() == x.scalar_type(), "x [..., D] and w [D] of one dtype expected");
  at::Tensor h = x;
  const void* dp = nullptr;
  void* hp = nullptr;
  if (delta.has_value()) {
    need_cuda_contig(*delta, "delta");
    TORCH_CHECK(delta->sizes() == x.sizes() && delta->scalar_type() == x.scalar_type(), "delta must match x");
    h = new_out_like(x);
    dp = delta->data_ptr();
    hp = h.data_ptr();
  }
  at::Tensor y = new_out_like(x);
  at::Tensor rstd = new_out({rows}, x.options().dtype(at::kFloat));
  check(dpk_add_rmsnorm_forward(x.data_ptr(), dp, w.data_ptr(), hp, y.data_ptr(), rstd.data_ptr<float>(), elem_kind(x),
                                rows, D, (float)eps, stream()),
        "add_rmsnorm_forward");
  return {y, h, rstd};
}

at::Tensor add_rmsnorm_backward(at::Tensor dy, c10::optional<at::Tensor> dres, at::Tensor h, at::Tensor rstd,
                                at::Tensor w) {
  c10::cuda::CUDAGuard guard(dy.device());
  need_cuda_contig(dy, "dy");
  need_cuda_contig(h, "h");
  need_cuda_contig(rstd, "rstd");
  need_cuda_contig(w, "w");
  const int64_t D = w.numel(), rows = h.numel() / D;
  TORCH_CHECK(dy.sizes() == h.sizes() && dy.scalar_type() == h.scalar_type() && w.scalar_type() == h.scalar_type() &&
              rstd.scalar_type() == at::kFloat && rstd.numel() == rows, "dy, h [..., D], w [D], rstd fp32 [rows]");
  const void* rp = nullptr;
  if (dres.has_value()) {
    need_cuda_contig(*dres, "dres");
    TORCH_CHECK(dres->sizes() == h.sizes() && dres->scalar_type() == h.scalar_type(), "dres must match h");
    rp = dres->data_ptr();
  }
  at::Tensor dh = new_out_like(h);
  check(dpk_add_rmsnorm_backward(dy.data_ptr(), rp, h.data_ptr(), rstd.data_ptr<float>(), w.data_ptr(), dh.data_ptr(),
                                 elem_kind(h), rows, D, stream()),
        "add_rmsnorm_backward");
  return dh;
}

at::Tensor philox_normal(int64_t n, int64_t seed, int64_t offset, double std, at::Device device) {
  c10::cuda::CUDAGuard guard(device);
  at::Tensor out = new_out({n}, at::TensorOptions().device(device).dtype(at::kFloat));
  check(dpk_philox_normal(out.data_ptr<float>(), n, (uint64_t)seed, (uint64_t)offset, (float)std, stream()),
        "philox_normal");
  return out;
}

void check_status(int64_t device) { raise_if_failed((int)device); }

// Raises what a timed-out kernel makes the next call raise (host only; for tests of the error path).
void raise_wait_timeout_for_test() { TORCH_CHECK(false, "opacus_b200: a kernel gave up on a bounded wait (test)"); }

int64_t tensor_entry_size() { return (int64_t)sizeof(DpkTensorEntry); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gram_pair_norm", &gram_pair_norm, py::arg("x"), py::arg("ids"), py::arg("g"), py::arg("scale"),
        py::arg("scratch"), py::arg("out_w"), py::arg("out_b"), py::arg("accumulate"), py::arg("right_off") = 0,
        py::arg("logical_T") = 0);
  m.def("gram_pair_scratch_floats", &gram_pair_scratch_floats);
  m.def("wgrad_tn", &wgrad_tn);
  m.def("wgrad_tn_ex", &wgrad_tn_ex);
  m.def("wgrad2_tn", &wgrad2_tn);
  m.def("conv_psg", &conv_psg);
  m.def("tied_cross_norm", &tied_cross_norm);
  m.def("scale_rows", &scale_rows);
  m.def("clip_factor", &clip_factor);
  m.def("split3_rows", &split3_rows);
  m.def("chacha_words", &chacha_words);
  m.def("chacha_normal", &chacha_normal);
  m.def("row_norm_sq", &row_norm_sq);
  m.def("weighted_sum", &weighted_sum, py::arg("x"), py::arg("c"), py::arg("dest") = py::none());
  m.def("outer_norm_sq", &outer_norm_sq);
  m.def("norm_lastdim_grad", &norm_lastdim_grad);
  m.def("norm_channel_grad", &norm_channel_grad);
  m.def("norm_lastdim_psg", &norm_lastdim_psg);
  m.def("embedding_scatter", &embedding_scatter);
  m.def("fused_dp_step", &fused_dp_step);
  m.def("sharded_dp_step", &sharded_dp_step, py::arg("grad_ptrs"), py::arg("param_ptrs"), py::arg("flag_ptrs"),
        py::arg("master"), py::arg("state0"), py::arg("state1"), py::arg("slice_begin"), py::arg("slice_len"),
        py::arg("rank"), py::arg("param_bf16"), py::arg("epoch"), py::arg("kind"), py::arg("nesterov"),
        py::arg("first_step"), py::arg("lr"), py::arg("momentum"), py::arg("dampening"), py::arg("weight_decay"),
        py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("bias_c1"), py::arg("bias_c2_sqrt"),
        py::arg("noise_std"), py::arg("inv_scale"), py::arg("seed"), py::arg("offset"), py::arg("noise_split"),
        py::arg("noise_shift"), py::arg("grad_mc") = 0, py::arg("param_mc") = 0, py::arg("segments") = py::none(),
        py::arg("max_blocks") = 0, py::arg("stripe_len") = 0, py::arg("stripe_stride") = 0);
  m.def("norm_allreduce_clip", &norm_allreduce_clip, py::arg("slot_ptrs"), py::arg("flag_ptrs"), py::arg("sharded"),
        py::arg("replicated"), py::arg("n"), py::arg("capacity"), py::arg("rank"), py::arg("flag_base"),
        py::arg("epoch"), py::arg("max_norm"), py::arg("device"), py::arg("pull") = false);
  m.def("step_segment_size", []() { return (int64_t)sizeof(DpkStepSegment); });
  m.def("tp_gemm", &tp_gemm);
  m.def("cross_entropy_forward", &cross_entropy_forward);
  m.def("cross_entropy_backward", &cross_entropy_backward);
  m.def("rope", &rope);
  m.def("swiglu_forward", &swiglu_forward);
  m.def("swiglu_backward", &swiglu_backward);
  m.def("add_rmsnorm_forward", &add_rmsnorm_forward);
  m.def("add_rmsnorm_backward", &add_rmsnorm_backward);
  m.def("philox_normal", &philox_normal);
  m.def("check_status", &check_status);
  m.def("set_debug", [](bool on) { g_debug = on; });
  m.def("get_debug", []() { return g_debug; });
  m.def("_raise_wait_timeout_for_test", &raise_wait_timeout_for_test);
  m.def("tensor_entry_size", &tensor_entry_size);
}
