// PTX wrappers shared by the TMA-staged kernels: mbarriers with bounded waits and
// 1-D bulk asynchronous copies (cp.async.bulk, the descriptor-free TMA form).
//
// Every wait on an mbarrier is bounded: after about two seconds the CTA sets an
// abort flag, stops waiting (later waits return at once), finishes its barrier
// sequence with meaningless data and raises the device error flag the host can
// read with attnres_b200_error_flag().
#pragma once

#include "common.cuh"

namespace attnres_b200 {

__device__ int g_error_flag = 0;

constexpr int kTmaMinWidth = 256;
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;
constexpr int kSmemPerSm = 220 * 1024;        // left for CTAs after per-CTA reservations
constexpr int kSmemPerCtaMax = 227 * 1024;

// ---------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false (and latches the CTA abort flag) on timeout or
// when another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - start > kWaitTimeoutNs) {
        *abort_flag = 1;
        atomicOr(&g_error_flag, 1);
        return false;
      }
    }
  }
  return true;
}

// Row copy global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

__device__ __forceinline__ void consumer_sync(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
  acc = fmaf(bf16x2_lo(a.x), bf16x2_lo(b.x), acc);
  acc = fmaf(bf16x2_hi(a.x), bf16x2_hi(b.x), acc);
  acc = fmaf(bf16x2_lo(a.y), bf16x2_lo(b.y), acc);
  acc = fmaf(bf16x2_hi(a.y), bf16x2_hi(b.y), acc);
  acc = fmaf(bf16x2_lo(a.z), bf16x2_lo(b.z), acc);
  acc = fmaf(bf16x2_hi(a.z), bf16x2_hi(b.z), acc);
  acc = fmaf(bf16x2_lo(a.w), bf16x2_lo(b.w), acc);
  acc = fmaf(bf16x2_hi(a.w), bf16x2_hi(b.w), acc);
  return acc;
}

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

inline bool tma_shape_ok(int D, int R) {
  return D >= kTmaMinWidth && D % 8 == 0 && (D - R) % 8 == 0;
}

template <typename Kernel>
inline int prepare_kernel(Kernel kernel, uint32_t smem_bytes) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) !=
      cudaSuccess) {
    cudaGetLastError();
    return 9;
  }
  return 0;
}

}  // namespace attnres_b200
