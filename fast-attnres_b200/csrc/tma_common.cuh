// PTX wrappers shared by the TMA-staged kernels: mbarriers with bounded waits and
// 1-D bulk asynchronous copies (cp.async.bulk, the descriptor-free TMA form).
//
// Every wait on an mbarrier is bounded: after about two seconds the CTA sets an
// abort flag, stops waiting (later waits return at once), finishes its barrier
// sequence with meaningless data and raises the device error flag the host can
// read with attnres_b200_error_flag().  The launch itself still returns "ok" (it
// is asynchronous): callers poll the flag at step boundaries.  CTAs of a cluster
// additionally meet at a cluster barrier before they retire.
#pragma once

#include <atomic>

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
// when another thread of the CTA has already given up.  The kernels wait with the
// default limit; the library's self-test passes a short one to run the give-up path.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t limit_ns = kWaitTimeoutNs) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - start > limit_ns) {
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

// Largest dynamic shared-memory size already granted to one kernel instance, per device.
// Every launch function owns a static one, so the attribute is set once per (instance,
// device, size) instead of on every launch.  (cudaDeviceReset discards the attribute
// together with the context; a process that resets a device must reload the library.)
constexpr int kMaxDevices = 64;
struct SmemGrant {
  std::atomic<uint32_t> bytes[kMaxDevices];
};

template <typename Kernel>
inline int prepare_kernel(Kernel kernel, uint32_t smem_bytes, SmemGrant& grant) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return 9;
  }
  const bool cached = device >= 0 && device < kMaxDevices;
  if (cached && grant.bytes[device].load(std::memory_order_acquire) >= smem_bytes) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) !=
      cudaSuccess) {
    cudaGetLastError();
    return 9;
  }
  if (cached) {
    // Monotonic: a concurrent caller that raised the limit further keeps its value.
    uint32_t seen = grant.bytes[device].load(std::memory_order_relaxed);
    while (seen < smem_bytes &&
           !grant.bytes[device].compare_exchange_weak(seen, smem_bytes, std::memory_order_release)) {
    }
  }
  return 0;
}

}  // namespace attnres_b200
