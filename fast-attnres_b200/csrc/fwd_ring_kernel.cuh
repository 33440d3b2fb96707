// TMA-staged forward of the AttnRes read for the aligned layout (feature stride 1,
// 16-byte aligned rows, D and D-R multiples of 8).
//
// A position is owned by a GROUP of G warps (G = 1 for D <= 1024, 2 for 2048,
// 4 for 4096, 8 for 8192); every lane owns four 16-byte chunks of the row, so
// the FP32 accumulator, the query lanes and the current batch all stay in
// registers.  Each group streams its (position, source) rows through its own
// ring of shared-memory stages filled by 1-D bulk asynchronous copies
// (cp.async.bulk + mbarrier complete_tx).  The ring refills itself: as soon as
// the group has moved a batch of two source rows into registers, its leader
// lane issues the copies for the items that will reuse those stages, so a group
// always has `stages` rows in flight without a producer warp or "empty"
// barriers.  Per batch the lanes reduce (sum of squares, dot with the query) of
// both sources with one folded butterfly, the warps of a group meet at a named
// barrier, and every lane folds the batch into its accumulator with an online
// softmax.  Arithmetic on the row uses the packed FP32x2 FMA of sm_100.
//
// The kernel is specialised at compile time on G and on TAIL0, the first of the
// lane's four chunks that lies in the tail key when the boundary D-R falls on a
// multiple of the group width (TAIL0 = 0 is R = D; D = 4096 with R = 1024 is
// TAIL0 = 3), so the common shapes run without per-chunk predicates; those
// instances can also take the row size and the ring depth (eight stages) as
// compile-time constants (template parameter SR), which turns the ring addressing
// into shifts and masks.  TAIL0 = -1 is the
// predicated form for every other aligned shape.  The batch body is instantiated
// for two sources and, for an odd source count, once more for the last one, so no
// per-source "is this source present" test runs in the loop.
#pragma once

#include <type_traits>

#include "tma_common.cuh"

namespace attnres_b200 {

constexpr int kRingChunks = 4;  // 16-byte chunks per lane
constexpr int kRingBatch = 2;   // sources folded per reduction
constexpr int kRingMaxGroupWarps = 8;
constexpr int kRingStaticStages = 8;  // ring depth of the specialised instances

// The next item to consume in a group's ring.  With a compile-time depth of eight stages
// the stage is the low three bits of a running counter and the mbarrier phase the bit
// above them; otherwise stage and phase advance incrementally (no division either way).
template <bool STATIC>
struct RingCursor {
  int at = 0;          // STATIC: item counter modulo 16; otherwise the stage index
  uint32_t phase = 0;  // used by the dynamic form only
  int depth;
  __device__ __forceinline__ explicit RingCursor(int stages) : depth(stages) {}
  __device__ __forceinline__ int stage(int ahead, uint32_t* parity) const {
    if (STATIC) {
      const uint32_t item = (uint32_t)(at + ahead);
      *parity = (item >> 3) & 1u;
      return (int)(item & 7u);
    }
    int st = at + ahead;
    *parity = phase;
    if (st >= depth) {
      st -= depth;
      *parity ^= 1u;
    }
    return st;
  }
  __device__ __forceinline__ void advance(int count) {
    if (STATIC) {
      at = (at + count) & 15;
    } else {
      at += count;
      if (at >= depth) {
        at -= depth;
        phase ^= 1u;
      }
    }
  }
};

struct FwdRingPlan {
  int group_warps;  // G
  int cta_warps;    // 4 or 8
  int stages;       // ring depth per group
  int ctas_per_sm;
  int tail0;        // compile-time tail boundary in chunks-per-lane, or -1
  uint32_t off_bars;
  uint32_t off_part;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

inline bool make_fwd_plan(int S, int D, int R, FwdRingPlan* plan) {
  (void)S;
  if (!tma_shape_ok(D, R)) return false;
  const int chunks = D / 8;
  int need = (chunks + 32 * kRingChunks - 1) / (32 * kRingChunks);
  int G = 1;
  while (G < need) G <<= 1;
  if (G > kRingMaxGroupWarps) return false;
  FwdRingPlan p;
  p.group_warps = G;
  p.cta_warps = G > 4 ? 8 : 4;
  p.ctas_per_sm = p.cta_warps == 4 ? 3 : 1;
  const int lanes = 32 * G, c0 = (D - R) / 8;
  const int groups = p.cta_warps / G;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const uint32_t fixed = 4u * 8u * 8u + 4u * 2u * 2u * kRingBatch * kRingMaxGroupWarps * 4u + 16u + 1024u;
  const uint32_t budget = (uint32_t)kSmemPerSm / (uint32_t)p.ctas_per_sm;
  int stages = (int)((budget - fixed) / ((uint32_t)groups * row_bytes));
  if (stages > 8) stages = 8;
  if (stages < 4) return false;
  p.stages = stages;
  // The specialised instances assume a full row and a ring of exactly eight stages.
  p.tail0 = (chunks == lanes * kRingChunks && c0 % lanes == 0 && stages == kRingStaticStages)
                ? c0 / lanes : -1;
  uint32_t off = (uint32_t)groups * (uint32_t)stages * row_bytes;
  p.off_bars = align_up(off, 8);
  off = p.off_bars + (uint32_t)groups * (uint32_t)stages * 8u;
  p.off_part = align_up(off, 16);
  off = p.off_part + (uint32_t)groups * 2u * 2u * kRingBatch * kRingMaxGroupWarps * 4u;
  p.off_abort = off;
  off += 16;
  p.smem_bytes = off;
  if (p.smem_bytes > (uint32_t)kSmemPerCtaMax) return false;
  *plan = p;
  return true;
}

inline bool tma_fwd_supported(int S, int D, int R) {
  FwdRingPlan plan;
  return make_fwd_plan(S, D, R, &plan);
}

__device__ __forceinline__ void group_sync(int group, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Wait with the polling loop kept out of line: the common case is one try_wait.
__device__ __noinline__ void mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  mbar_wait(bar, parity, abort_flag);
}

__device__ __forceinline__ void mbar_wait_fast(uint64_t* bar, uint32_t parity,
                                               volatile int* abort_flag) {
  if (!mbar_try_wait(bar, parity)) mbar_wait_slow(bar, parity, abort_flag);
}

template <int G, int TAIL0, bool SR, bool LN>
__global__ void __launch_bounds__((G > 4 ? 8 : 4) * 32, G > 4 ? 1 : 3)
fwd_ring_kernel(const __grid_constant__ FwdParams p, const __grid_constant__ FwdRingPlan plan) {
  constexpr int NV = kRingChunks, B = kRingBatch;
  constexpr int WARPS = G > 4 ? 8 : 4;
  constexpr int GROUPS = WARPS / G;
  constexpr int L = G * 32;
  constexpr bool STATIC_TAIL = TAIL0 >= 0;
  static_assert(!SR || STATIC_TAIL, "compile-time ring constants need a full row");
  static_assert(B == 2, "the folded reduction below is written for two sources per batch");
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp / G, wig = warp % G;
  const int gl = wig * 32 + lane;
  const int S = p.S, R = p.R;
  // Full-row instances: width, row size and ring depth are compile-time constants.
  const int D = SR ? L * NV * 8 : p.D;
  const int CH = D / 8, c0 = (D - R) / 8;
  const int nst = SR ? kRingStaticStages : plan.stages;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  unsigned char* ring = smem + (size_t)group * (size_t)nst * row_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + plan.off_bars) + group * nst;
  float4* part_sm = reinterpret_cast<float4*>(smem + plan.off_part) +
                    group * (2 * kRingMaxGroupWarps);  // [2][8] x (ss0, dt0, ss1, dt1)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + plan.off_abort);

  if (tid == 0) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + plan.off_bars);
    for (int i = 0; i < GROUPS * nst; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // The lane's chunks and its query lanes (zero outside the tail key).
  bool in_row[NV], in_tail[NV];
  float2 q2[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = gl + j * L;
    in_row[j] = STATIC_TAIL ? true : c < CH;
    in_tail[j] = STATIC_TAIL ? (j >= TAIL0) : (c < CH && c >= c0);
#pragma unroll
    for (int k = 0; k < 4; ++k) q2[j][k] = make_float2(0.f, 0.f);
    if (in_tail[j]) load_query_chunk(p.query, p.query_stride, c - c0, q2[j]);
  }

  const int64_t total_groups = (int64_t)gridDim.x * GROUPS;
  const int64_t gid = (int64_t)blockIdx.x * GROUPS + group;
  const int64_t my_rows = gid < p.N ? (p.N - gid + total_groups - 1) / total_groups : 0;
  const bool leader = gl == 0;

  // Leader's issue cursor: items are (row, source) pairs in consumption order.
  int64_t rows_to_issue = my_rows;  // rows with at least one source not yet requested
  int in_flight = 0;                // requested, not yet consumed
  int issue_stage = 0;
  int64_t issue_row = gid;
  int issue_s = 0;
  auto issue_one = [&]() {
    mbar_expect_tx(&full_bar[issue_stage], row_bytes);
    bulk_load(ring + (uint32_t)issue_stage * row_bytes,
              p.src.ptr[issue_s] + issue_row * p.src.row_stride[issue_s], row_bytes,
              &full_bar[issue_stage]);
    ++in_flight;
    if (++issue_stage == nst) issue_stage = 0;
    if (++issue_s == S) {
      issue_s = 0;
      issue_row += total_groups;
      --rows_to_issue;
    }
  };
  if (leader) {
    while (rows_to_issue > 0 && in_flight < nst) issue_one();
  }

  RingCursor<SR> cursor(nst);
  int buf = 0;
  const float inv_rank = 1.0f / (float)R;
  for (int64_t row = gid; row < p.N; row += total_groups) {
    float2 acc[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[j][k] = make_float2(0.f, 0.f);
    float run_max = -INFINITY, run_sum = 0.f;

    // One batch of NB (1 or 2) sources starting at source s0.
    auto batch = [&](auto nb_tag, const int s0) {
      constexpr int NB = decltype(nb_tag)::value;
      float2 v2[NB][NV][4];
      float part[2 * B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float2 ss2 = make_float2(0.f, 0.f), dt2 = make_float2(0.f, 0.f);
        if (b < NB) {
          uint32_t phase;
          const int stage = cursor.stage(b, &phase);
          mbar_wait_fast(&full_bar[stage], phase, abort_flag);
          const uint4* vrow = reinterpret_cast<const uint4*>(ring + (uint32_t)stage * row_bytes) + gl;
          uint4 raw[NV];
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            if (in_row[j]) raw[j] = vrow[j * L];
            else raw[j] = make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            float2(&v)[4] = v2[b < NB ? b : 0][j];
            v[0] = make_float2(bf16x2_lo(raw[j].x), bf16x2_hi(raw[j].x));
            v[1] = make_float2(bf16x2_lo(raw[j].y), bf16x2_hi(raw[j].y));
            v[2] = make_float2(bf16x2_lo(raw[j].z), bf16x2_hi(raw[j].z));
            v[3] = make_float2(bf16x2_lo(raw[j].w), bf16x2_hi(raw[j].w));
            if (in_tail[j]) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                ss2 = __ffma2_rn(v[k], v[k], ss2);
                dt2 = __ffma2_rn(v[k], q2[j][k], dt2);
              }
            }
          }
        }
        part[2 * b] = ss2.x + ss2.y;
        part[2 * b + 1] = dt2.x + dt2.y;
      }

      // Folded butterfly over the warp: four values cost 3 + 3 shuffles.  Afterwards
      // lane 0 / 8 / 16 / 24 (and their neighbours) hold the warp total of value 0 / 1 / 2 / 3.
      const bool up16 = (lane & 16) != 0;
      float keep0 = up16 ? part[2] : part[0];
      float keep1 = up16 ? part[3] : part[1];
      keep0 += __shfl_xor_sync(0xffffffffu, up16 ? part[0] : part[2], 16);
      keep1 += __shfl_xor_sync(0xffffffffu, up16 ? part[1] : part[3], 16);
      const bool up8 = (lane & 8) != 0;
      float keep = up8 ? keep1 : keep0;
      keep += __shfl_xor_sync(0xffffffffu, up8 ? keep0 : keep1, 8);
      keep += __shfl_xor_sync(0xffffffffu, keep, 4);
      keep += __shfl_xor_sync(0xffffffffu, keep, 2);
      keep += __shfl_xor_sync(0xffffffffu, keep, 1);
      float tot[2 * B];
      if (G == 1) {
#pragma unroll
        for (int i = 0; i < 2 * B; ++i) tot[i] = __shfl_sync(0xffffffffu, keep, i * 8);
      } else {
        float4* mine = part_sm + buf * kRingMaxGroupWarps;
        if ((lane & 7) == 0) reinterpret_cast<float*>(&mine[wig])[lane >> 3] = keep;
        group_sync(group, L);
#pragma unroll
        for (int i = 0; i < 2 * B; ++i) tot[i] = 0.f;
#pragma unroll
        for (int w = 0; w < G; ++w) {
          const float4 t = mine[w];
          tot[0] += t.x;
          tot[1] += t.y;
          tot[2] += t.z;
          tot[3] += t.w;
        }
      }
      // Every lane of the group has read its chunks of these stages: refill them.
      if (leader) {
        fence_proxy_async();
        in_flight -= NB;
        while (rows_to_issue > 0 && in_flight < nst) issue_one();
      }

      // Online softmax over the batch.
      float z[NB];
      float new_max = run_max;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float inv_rms = rsqrtf(tot[2 * b] * inv_rank + p.eps);
        z[b] = tot[2 * b + 1] * inv_rms * p.scale;
        new_max = fmaxf(new_max, z[b]);
      }
      if (new_max != run_max) {
        const float rescale = __expf(run_max - new_max);
        run_sum *= rescale;
        const float2 r2 = make_float2(rescale, rescale);
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[j][k] = __fmul2_rn(acc[j][k], r2);
        run_max = new_max;
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float w = __expf(z[b] - new_max);
        run_sum += w;
        const float2 w2 = make_float2(w, w);
#pragma unroll
        for (int j = 0; j < NV; ++j)
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[j][k] = __ffma2_rn(w2, v2[b][j][k], acc[j][k]);
        if (leader) p.logits[(int64_t)(s0 + b) * p.N + row] = z[b];
      }
      cursor.advance(NB);
      buf ^= 1;
    };
    int s0 = 0;
    for (; s0 + B <= S; s0 += B) batch(std::integral_constant<int, B>{}, s0);
    if (s0 < S) batch(std::integral_constant<int, 1>{}, s0);

    const float inv_sum = 1.0f / run_sum;
    if (leader) {
      p.stats[row] = run_max;
      p.stats[p.N + row] = inv_sum;
    }
    __nv_bfloat16* orow = p.out + row * p.out_row_stride;
    __nv_bfloat16* rrow = p.out_residual != nullptr ? p.out_residual + row * (int64_t)D : nullptr;
    // out = acc / run_sum: multiply by the reciprocal, then one Newton step on the quotient
    // (o += (acc - o * sum) * inv), which removes the reciprocal's own rounding.
    const float2 i2 = make_float2(inv_sum, inv_sum), nsum2 = make_float2(-run_sum, -run_sum);
    uint32_t hi[NV][4];  // the lane's share of the BF16 output row
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (in_row[j]) {
        uint32_t lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 first = __fmul2_rn(acc[j][k], i2);
          const float2 o = __ffma2_rn(__ffma2_rn(first, nsum2, acc[j][k]), i2, first);
          hi[j][k] = pack_bf16x2(o.x, o.y);
          lo[k] = split_low16x2(o.x, o.y, hi[j][k]);  // what the BF16 rounding dropped
        }
        *reinterpret_cast<uint4*>(orow + (int64_t)(gl + j * L) * 8) =
            make_uint4(hi[j][0], hi[j][1], hi[j][2], hi[j][3]);
        if (rrow != nullptr)
          *reinterpret_cast<uint4*>(rrow + (int64_t)(gl + j * L) * 8) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) hi[j][k] = 0u;
      }
    }

    // Fused LayerNorm of the row just written (from its BF16 values, so the result equals a
    // LayerNorm applied to `out` afterwards): two more reductions over the group, then the
    // normalised row goes out next to the plain one.
    if constexpr (LN) {
      // Sum over the group of one value per lane; every lane gets the total.
      auto group_total = [&](float value) {
        value = warp_sum(value);
        if (G > 1) {
          float* mine = reinterpret_cast<float*>(part_sm + buf * kRingMaxGroupWarps);
          if (lane == 0) mine[wig * 4] = value;
          group_sync(group, L);
          value = 0.f;
#pragma unroll
          for (int w = 0; w < G; ++w) value += mine[w * 4];
          buf ^= 1;
        }
        return value;
      };
      const float inv_width = 1.0f / (float)D;
      float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          sum2 = __fadd2_rn(sum2, make_float2(bf16x2_lo(hi[j][k]), bf16x2_hi(hi[j][k])));
      const float mean = group_total(sum2.x + sum2.y) * inv_width;
      const float2 nmean2 = make_float2(-mean, -mean);
      float2 sq2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (in_row[j]) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 d = __fadd2_rn(make_float2(bf16x2_lo(hi[j][k]), bf16x2_hi(hi[j][k])), nmean2);
            sq2 = __ffma2_rn(d, d, sq2);
          }
        }
      }
      const float rstd = rsqrtf(group_total(sq2.x + sq2.y) * inv_width + p.ln_eps);
      if (leader) {
        p.ln_stats[row] = mean;
        p.ln_stats[p.N + row] = rstd;
      }
      __nv_bfloat16* nrow = p.ln_out + row * (int64_t)D;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (in_row[j]) {
          const int64_t first = (int64_t)(gl + j * L) * 8;
          float w[8], b[8];
          if (p.ln_weight != nullptr) {
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(p.ln_weight + first));
            const float4 w1 = __ldg(reinterpret_cast<const float4*>(p.ln_weight + first) + 1);
            w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
            w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = 1.f;
          }
          if (p.ln_bias != nullptr) {
            const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.ln_bias + first));
            const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.ln_bias + first) + 1);
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
            b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) b[e] = 0.f;
          }
          uint32_t y[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float x0 = (bf16x2_lo(hi[j][k]) - mean) * rstd;
            const float x1 = (bf16x2_hi(hi[j][k]) - mean) * rstd;
            y[k] = pack_bf16x2(fmaf(x0, w[2 * k], b[2 * k]), fmaf(x1, w[2 * k + 1], b[2 * k + 1]));
          }
          *reinterpret_cast<uint4*>(nrow + first) = make_uint4(y[0], y[1], y[2], y[3]);
        }
      }
    }
  }
  // Normal exit: every copy issued was waited for.  After an aborted wait some may still
  // be in flight: hold the CTA (and so its shared memory) for 200 us before retiring.
  if (*abort_flag) {
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) {
    }
  }
}

// Compile-time ring constants (SR), measured on B200 at N = 16384, R = D: eight-warp groups
// +1 %; one-warp groups +4 % at S = 49 and even at S = 9; two-warp groups +6 % at S = 49 but
// -3 % at S = 9; four-warp groups -5 % (D = 4096, S = 49: 6.07 against 6.37 TB/s).  So they are
// used for one- and eight-warp groups, and for two-warp groups from 17 sources up.  The
// instances with the LayerNorm epilogue (LN) are separate so that the plain forward carries
// none of its registers; they use the run-time ring form except for eight-warp groups.
template <int G, int TAIL0, bool SR, bool LN>
inline int launch_fwd_ring_instance(const FwdParams& p, const FwdRingPlan& plan, int grid,
                                    cudaStream_t stream) {
  auto kernel = fwd_ring_kernel<G, TAIL0, SR, LN>;
  static SmemGrant grant;
  if (int st = prepare_kernel(kernel, plan.smem_bytes, grant)) return st;
  kernel<<<grid, plan.cta_warps * 32, plan.smem_bytes, stream>>>(p, plan);
  return cudaGetLastError() == cudaSuccess ? 0 : 9;
}

template <int G, int TAIL0>
inline int launch_fwd_ring(const FwdParams& p, const FwdRingPlan& plan, int grid,
                           cudaStream_t stream) {
  constexpr bool kFull = TAIL0 >= 0;  // full rows always have the eight-stage ring
  if (p.ln_out != nullptr)
    return launch_fwd_ring_instance<G, TAIL0, (G == 8 && kFull), true>(p, plan, grid, stream);
  if constexpr (kFull && (G == 1 || G == 8))
    return launch_fwd_ring_instance<G, TAIL0, true, false>(p, plan, grid, stream);
  if constexpr (kFull && G == 2) {
    if (p.S >= 17) return launch_fwd_ring_instance<G, TAIL0, true, false>(p, plan, grid, stream);
  }
  return launch_fwd_ring_instance<G, TAIL0, false, false>(p, plan, grid, stream);
}

template <int G>
inline int launch_fwd_ring_tail(const FwdParams& p, const FwdRingPlan& plan, int grid,
                                cudaStream_t stream) {
  switch (plan.tail0) {
    case 0: return launch_fwd_ring<G, 0>(p, plan, grid, stream);
    case 1: return launch_fwd_ring<G, 1>(p, plan, grid, stream);
    case 2: return launch_fwd_ring<G, 2>(p, plan, grid, stream);
    case 3: return launch_fwd_ring<G, 3>(p, plan, grid, stream);
    default: return launch_fwd_ring<G, -1>(p, plan, grid, stream);
  }
}

inline int launch_fwd_tma(const FwdParams& p, int sms, cudaStream_t stream) {
  FwdRingPlan plan;
  if (!make_fwd_plan(p.S, p.D, p.R, &plan)) return 9;
  const int groups = plan.cta_warps / plan.group_warps;
  const int64_t wanted = (p.N + groups - 1) / groups;
  const int64_t cap = (int64_t)sms * plan.ctas_per_sm;
  const int grid = (int)(wanted < cap ? wanted : cap);
  switch (plan.group_warps) {
    case 1: return launch_fwd_ring_tail<1>(p, plan, grid, stream);
    case 2: return launch_fwd_ring_tail<2>(p, plan, grid, stream);
    case 4: return launch_fwd_ring_tail<4>(p, plan, grid, stream);
    default: return launch_fwd_ring_tail<8>(p, plan, grid, stream);
  }
}

}  // namespace attnres_b200
