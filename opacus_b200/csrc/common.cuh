// Device-side building blocks for the sm_100a kernels of this package:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc / mma / commit / ld),
// shared-memory and instruction descriptors, bounded waits with a status word,
// and a Philox4x32-10 counter-based generator.
//
// Conventions
//  * every spin on an mbarrier is bounded (wall-clock limit read from
//    %globaltimer); on expiry the waiter records where it gave up in a status
//    word in global memory and the kernel unwinds (frees TMEM, returns);
//  * no TMA load uses cluster multicast.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dpk {

// ----------------------------------------------------------------------------- status word
// status[0] : 0 = ok, otherwise (site << 8) | code of the first failure
// status[1] : blockIdx.x of the reporter, status[2..3]: free-form detail
enum : uint32_t { ERR_WAIT_TIMEOUT = 1, ERR_BAD_ARG = 2 };

__device__ __forceinline__ void report_error(uint32_t* status, uint32_t site, uint32_t code, uint32_t d0 = 0,
                                             uint32_t d1 = 0) {
  // `status` may be host-mapped memory: plain stores only (first writer wins approximately).
  if (status != nullptr && *reinterpret_cast<volatile uint32_t*>(status) == 0u) {
    volatile uint32_t* s = status;
    s[1] = blockIdx.x;
    s[2] = d0;
    s[3] = d1;
    s[0] = (site << 8) | code;
  }
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Upper bound for any single wait inside a kernel.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// ----------------------------------------------------------------------------- small helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait.  Returns false after kWaitLimitNs (and records it) or as soon
// as *abort_flag (shared memory) is set by another role of the same CTA.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status, uint32_t site) {
  uint32_t ok;
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_flag) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        report_error(status, site, ERR_WAIT_TIMEOUT, parity, spins);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x,
                                            int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w)
      : "memory");
}

// Tiled store shared -> global (bulk_group completion).  Coordinates must not be negative.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y,
                                             int32_t z, int32_t w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

// Untiled bulk copies (both addresses 16-byte aligned, size a multiple of 16 bytes); never multicast.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gmem_dst)), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() {          // at most N groups still pending (writes complete)
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {     // at most N groups still reading their source
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ----------------------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All previously issued MMAs of this thread arrive on `bar` when complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives
// columns [col, col+32) of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, 128-byte swizzle.
//   bits  0-13 start address >> 4      bits 16-29 leading-dim byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version (1 on sm_100)
//   bits 61-63 layout (2 = 128B swizzle)
// K-major operand (rows of 128 bytes = one swizzle row per MN index):
//   8-row groups are 1024 bytes apart (stride offset); leading offset unused.
// MN-major operand (each K index is a 128-byte row of 64 16-bit MN elements):
//   8-row K groups are 1024 bytes apart (stride offset); successive blocks of
//   64 MN elements are `mn_block_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation.
//   bits 4-5 D format (1 = f32); 7-9 A format; 10-12 B format (0 f16, 1 bf16, 2 tf32)
//   bit 15 A major (1 = MN); bit 16 B major; bits 17-22 N >> 3; bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t M, uint32_t N) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((N >> 3) << 17) | ((M >> 4) << 24);
}

// ----------------------------------------------------------------------------- clip factor
// min(1, C / (sqrt(max(n2, 0)) + 1e-6)) (opacus/optimizers/optimizer.py:452-455), except that a NaN squared norm
// gives NaN: fmaxf / fminf return their non-NaN argument, which would turn "norm unknown" into "do not clip".
__device__ __forceinline__ float clip_factor_of(float n2, float C) {
  if (n2 != n2) return n2;
  return fminf(1.f, C / (sqrtf(fmaxf(n2, 0.f)) + 1e-6f));
}

// ----------------------------------------------------------------------------- flag waits between ranks / blocks
// Epoch flags: a word holds the number of the last step its writer reached.  The high bit tells waiters to give up.
constexpr uint32_t kAbortBit = 0x80000000u;

// Spins until *word >= epoch (wrap-safe) for at most kWaitLimitNs; on expiry records (site, epoch, value seen).
__device__ __forceinline__ bool spin_until_epoch(volatile uint32_t* word, uint32_t epoch, uint32_t* status,
                                                 uint32_t site) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    const uint32_t v = *word;
    if (v & kAbortBit) return false;
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
    if ((++spins & 0xffu) == 0) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        report_error(status, site, ERR_WAIT_TIMEOUT, epoch, v);
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------- Philox4x32-10
struct Philox {
  uint32_t key0, key1;
  __device__ __forceinline__ Philox(uint64_t seed) : key0(static_cast<uint32_t>(seed)), key1(static_cast<uint32_t>(seed >> 32)) {}
  // 128-bit counter = (idx_lo, idx_hi, offset_lo, offset_hi)
  __device__ __forceinline__ uint4 operator()(uint64_t idx, uint64_t offset) const {
    uint4 c = make_uint4(static_cast<uint32_t>(idx), static_cast<uint32_t>(idx >> 32), static_cast<uint32_t>(offset),
                         static_cast<uint32_t>(offset >> 32));
    uint32_t k0 = key0, k1 = key1;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
      uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
      c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    return c;
  }
};

// Two independent N(0,1) from two uniform 32-bit words (Box-Muller).
__device__ __forceinline__ float2 box_muller(uint32_t a, uint32_t b) {
  const float two_pow_m32 = 2.3283064365386963e-10f;
  float u1 = (static_cast<float>(a) + 0.5f) * two_pow_m32;  // (0, 1)
  float u2 = (static_cast<float>(b) + 0.5f) * two_pow_m32;
  // -2 ln(u1) = -(2 ln 2) log2(u1); the hardware log2 has an absolute error near 2^-22, which moves a
  // sample by at most ~1e-3 standard deviations and only for the ~1e-6 of samples with u1 within 1e-6 of 1
  float r = sqrtf(-1.3862943611198906f * __log2f(u1));
  float s, c;
  sincospif(2.0f * u2, &s, &c);
  return make_float2(r * c, r * s);
}

}  // namespace dpk
