// TMA-staged backward of the AttnRes read for SHORT source lists (S <= 4) in the aligned
// layout (feature stride 1, 16-byte aligned rows, D and D-R multiples of 8).
//
// With few sources a position is small, and the two barriers and the single-warp middle
// section of the staged ("stash") backward dominate.  Here a position is owned by a group
// of G warps, as in the forward ring kernel, and everything about it lives in REGISTERS:
// every lane owns two 16-byte chunks of the row and loads its chunks of the upstream row
// and of all S sources from the group's ring of shared-memory stages (1-D bulk asynchronous
// copies), after which the stages are refilled at once.  The lanes then
//   1. reduce dw_s = v_s . dO and the tail sums of squares of all sources with one folded
//      butterfly (plus one named barrier when the group has more than one warp),
//   2. each form the probabilities, delta and the per-source coefficients themselves from
//      the saved logits (staged one position ahead with cp.async),
//   3. write dV_s = p_s dO + [tail] (ca_s q - cb_s v_s) from the source chunks still in
//      registers and accumulate their dquery lanes across all positions of the group.
// A position therefore costs one barrier, no second read of shared memory and no serial
// section, and the ring keeps `stages` rows in flight whatever the position's size.
//
// Template parameters: G warps per group; SE the exact source count (2..4), or 0 for "any
// count up to four, tested at run time"; FULL: the row is exactly G*32*2 chunks wide (no lane
// holds a chunk beyond the row); TAIL0 >= 0 (needs FULL): chunks j >= TAIL0 of every lane are
// tail chunks, TAIL0 < 0: per-lane predicates.  The exact-count, full-row instances run
// without any per-source or per-chunk test in the position loop.
#pragma once

#include "fwd_ring_kernel.cuh"

namespace attnres_b200 {

constexpr int kBwdRingChunks = 2;     // 16-byte chunks per lane
constexpr int kBwdRingMaxSources = 8;
constexpr int kBwdRingMaxGroupWarps = 16;

struct BwdRingPlan {
  int group_warps;  // G
  int cta_warps;    // max(G, 4)
  int stages;       // ring depth per group, at least S + 1
  int ctas_per_sm;
  int smax;         // compiled bound on S: 4 or 8
  uint32_t off_bars;
  uint32_t off_part;
  uint32_t off_zl;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

inline bool make_bwd_ring_plan(int S, int D, int R, BwdRingPlan* plan) {
  if (!tma_shape_ok(D, R) || S > 4) return false;  // see launch_bwd_ring_smax
  const int chunks = D / 8;
  const int need = (chunks + 32 * kBwdRingChunks - 1) / (32 * kBwdRingChunks);
  int G = 1;
  while (G < need) G <<= 1;
  if (G > kBwdRingMaxGroupWarps) return false;
  BwdRingPlan p;
  p.group_warps = G;
  p.cta_warps = G > 4 ? G : 4;
  p.smax = 4;
  const int groups = p.cta_warps / G;
  const int threads = p.cta_warps * 32;
  const int regs = p.smax == 4 ? 112 : 160;  // the launch bounds below ask for these
  int ctas = 65536 / (threads * regs);
  if (ctas < 1) ctas = 1;
  if (ctas > 4) ctas = 4;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const uint32_t bars = (uint32_t)groups * 24u * 8u;
  const uint32_t part = (uint32_t)groups * 2u * (uint32_t)G * 2u * kBwdRingMaxSources * 4u;
  const uint32_t zl = (uint32_t)groups * 3u * 16u * 4u;
  const uint32_t fixed = bars + part + zl + 16u + 128u;
  int stages = 0;
  while (ctas >= 1) {
    const uint32_t room = (228u * 1024u - (uint32_t)ctas * 1024u) / (uint32_t)ctas;
    const uint32_t usable = room < (uint32_t)kSmemPerCtaMax ? room : (uint32_t)kSmemPerCtaMax;
    stages = usable > fixed ? (int)((usable - fixed) / ((uint32_t)groups * row_bytes)) : 0;
    if (stages >= S + 2) break;
    --ctas;
  }
  if (ctas < 1) return false;
  if (stages > 2 * (S + 1)) stages = 2 * (S + 1);
  if (stages > 24) stages = 24;
  p.stages = stages;
  p.ctas_per_sm = ctas;
  uint32_t off = (uint32_t)groups * (uint32_t)stages * row_bytes;
  p.off_bars = align_up(off, 8);
  off = p.off_bars + bars;
  p.off_part = align_up(off, 16);
  off = p.off_part + part;
  p.off_zl = off;
  off += zl;
  p.off_abort = off;
  off += 16;
  p.smem_bytes = off;
  if (p.smem_bytes > (uint32_t)kSmemPerCtaMax) return false;
  *plan = p;
  return true;
}

inline bool bwd_ring_supported(int S, int D, int R) {
  BwdRingPlan plan;
  return make_bwd_ring_plan(S, D, R, &plan);
}

template <int G, int SE, bool FULL, int TAIL0>
__global__ void __launch_bounds__((G > 4 ? G : 4) * 32, G > 8 ? 1 : G > 4 ? 2 : 4)
bwd_ring_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ BwdRingPlan plan) {
  static_assert(TAIL0 < 0 || FULL, "a compile-time tail boundary needs a full row");
  constexpr int NV = kBwdRingChunks;
  constexpr int WARPS = G > 4 ? G : 4;
  constexpr int GROUPS = WARPS / G;
  constexpr int L = G * 32;
  constexpr int SMAX = SE > 0 ? SE : 4;
  // Values reduced per position: (ss, dw) of every source, padded to a power of two for the
  // folded butterfly.
  constexpr int K = SMAX == 1 ? 2 : SMAX == 2 ? 4 : 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp / G, wig = warp % G;
  const int gl = wig * 32 + lane;
  const int S = SE > 0 ? SE : p.S, D = p.D, R = p.R;
  const int CH = D / 8, c0 = (D - R) / 8, nst = plan.stages;
  const int items = S + 1;  // upstream row, then the sources
  const uint32_t row_bytes = (uint32_t)D * 2u;
  unsigned char* ring = smem + (size_t)group * (size_t)nst * row_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + plan.off_bars) + group * 24;
  float* part_sm = reinterpret_cast<float*>(smem + plan.off_part) +
                   group * (2 * G * 2 * kBwdRingMaxSources);            // [2][G][16]
  float* zl_sm = reinterpret_cast<float*>(smem + plan.off_zl) + group * 48;  // [3][16]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + plan.off_abort);

  if (tid == 0) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + plan.off_bars);
    for (int g = 0; g < GROUPS; ++g)
      for (int i = 0; i < nst; ++i) mbar_init(&bars[g * 24 + i], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  bool in_row_rt[NV], in_tail_rt[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = gl + j * L;
    in_row_rt[j] = c < CH;
    in_tail_rt[j] = in_row_rt[j] && c >= c0;
  }
  // With compile-time j these fold to constants in the specialised instances.
  auto row_ok = [&](int j) { return FULL ? true : in_row_rt[j]; };
  auto tail_ok = [&](int j) { return TAIL0 >= 0 ? j >= TAIL0 : in_tail_rt[j]; };
  float2 q2[NV][4], dq2[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = gl + j * L;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      q2[j][k] = make_float2(0.f, 0.f);
      dq2[j][k] = make_float2(0.f, 0.f);
    }
    if (tail_ok(j)) load_query_chunk(p.query, p.query_stride, c - c0, q2[j]);
  }

  const int64_t total_groups = (int64_t)gridDim.x * GROUPS;
  const int64_t gid = (int64_t)blockIdx.x * GROUPS + group;
  const int64_t my_rows = gid < p.N ? (p.N - gid + total_groups - 1) / total_groups : 0;
  const bool leader = gl == 0;

  // Leader's issue cursor over (row, item) pairs; item 0 is the upstream row.
  int64_t rows_to_issue = my_rows;
  int in_flight = 0, issue_stage = 0, issue_item = 0;
  int64_t issue_row = gid;
  auto issue_one = [&]() {
    const __nv_bfloat16* src =
        issue_item == 0 ? p.grad_out + issue_row * p.go_row_stride
                        : p.src.ptr[issue_item - 1] + issue_row * p.src.row_stride[issue_item - 1];
    mbar_expect_tx(&full_bar[issue_stage], row_bytes);
    bulk_load(ring + (uint32_t)issue_stage * row_bytes, src, row_bytes, &full_bar[issue_stage]);
    ++in_flight;
    if (++issue_stage == nst) issue_stage = 0;
    if (++issue_item == items) {
      issue_item = 0;
      issue_row += total_groups;
      --rows_to_issue;
    }
  };
  if (leader) {
    while (rows_to_issue > 0 && in_flight < nst) issue_one();
  }
  // Saved logits and statistics travel one position ahead: lanes 0..S+1 of the group's first
  // warp copy (logits[0..S), max, 1/sum) of a position into one of THREE small buffers (the
  // buffer written for position r+1 was last read for position r-2, and no warp of the group
  // can still be there once the first warp has passed the barrier of position r-1).
  auto stage_logits = [&](int64_t row, int buffer) {
    if (wig == 0 && lane < S + 2) {
      const float* src = lane < S ? p.logits + (int64_t)lane * p.N + row
                                  : p.stats + (int64_t)(lane - S) * p.N + row;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                       smem_addr(&zl_sm[buffer * 16 + lane])),
                   "l"(src)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (my_rows > 0) stage_logits(gid, 0);

  int use_stage = 0;
  uint32_t use_phase = 0;
  int buf = 0, zbuf = 0;
  const float inv_rank = 1.0f / (float)R;
  for (int64_t row = gid; row < p.N; row += total_groups, buf ^= 1, zbuf = zbuf == 2 ? 0 : zbuf + 1) {
    if (row + total_groups < p.N) {
      stage_logits(row + total_groups, zbuf == 2 ? 0 : zbuf + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }

    // ---- the lane's chunks of the upstream row and of every source, into registers
    uint4 g_raw[NV], v_raw[SMAX][NV];
#pragma unroll
    for (int i = 0; i <= SMAX; ++i) {
      if (i < items) {
        int stage = use_stage + i;
        uint32_t phase = use_phase;
        if (stage >= nst) {
          stage -= nst;
          phase ^= 1u;
        }
        mbar_wait_fast(&full_bar[stage], phase, abort_flag);
        const uint4* src = reinterpret_cast<const uint4*>(ring + (uint32_t)stage * row_bytes) + gl;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const uint4 raw = row_ok(j) ? src[j * L] : make_uint4(0u, 0u, 0u, 0u);
          if (i == 0) g_raw[j] = raw;
          else v_raw[i - 1][j] = raw;
        }
      } else if (i > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) v_raw[i - 1][j] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    float2 g2[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      g2[j][0] = make_float2(bf16x2_lo(g_raw[j].x), bf16x2_hi(g_raw[j].x));
      g2[j][1] = make_float2(bf16x2_lo(g_raw[j].y), bf16x2_hi(g_raw[j].y));
      g2[j][2] = make_float2(bf16x2_lo(g_raw[j].z), bf16x2_hi(g_raw[j].z));
      g2[j][3] = make_float2(bf16x2_lo(g_raw[j].w), bf16x2_hi(g_raw[j].w));
    }

    // ---- per-source partial sums: val[2s] = tail sum of squares, val[2s+1] = v_s . dO
    float val[K];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      float2 ss2 = make_float2(0.f, 0.f), dw2 = make_float2(0.f, 0.f);
      if (s < S) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          float2 v[4];
          v[0] = make_float2(bf16x2_lo(v_raw[s][j].x), bf16x2_hi(v_raw[s][j].x));
          v[1] = make_float2(bf16x2_lo(v_raw[s][j].y), bf16x2_hi(v_raw[s][j].y));
          v[2] = make_float2(bf16x2_lo(v_raw[s][j].z), bf16x2_hi(v_raw[s][j].z));
          v[3] = make_float2(bf16x2_lo(v_raw[s][j].w), bf16x2_hi(v_raw[s][j].w));
#pragma unroll
          for (int k = 0; k < 4; ++k) dw2 = __ffma2_rn(v[k], g2[j][k], dw2);
          if (tail_ok(j)) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ss2 = __ffma2_rn(v[k], v[k], ss2);
          }
        }
      }
      val[2 * s] = ss2.x + ss2.y;
      val[2 * s + 1] = dw2.x + dw2.y;
    }
#pragma unroll
    for (int i = 2 * SMAX; i < K; ++i) val[i] = 0.f;
    // Folded butterfly: each step halves the number of values a lane carries; afterwards
    // lane (i << shift) holds the warp total of value i, for every i < K.
    {
      int offset = 16;
#pragma unroll
      for (int half = K / 2; half >= 1; half /= 2, offset /= 2) {
        const bool upper = (lane & offset) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
          const float send = upper ? val[i] : val[i + half];
          const float keep = upper ? val[i + half] : val[i];
          val[i] = keep + __shfl_xor_sync(0xffffffffu, send, offset);
        }
      }
      for (; offset >= 1; offset /= 2) val[0] += __shfl_xor_sync(0xffffffffu, val[0], offset);
    }
    constexpr int SHIFT = K == 8 ? 2 : K == 4 ? 3 : 4;  // 32 / K lanes share one value
    float tot[K < 4 ? 4 : K];
    if (G == 1) {
#pragma unroll
      for (int i = 0; i < K; ++i) tot[i] = __shfl_sync(0xffffffffu, val[0], i << SHIFT);
    } else {
      float* mine = part_sm + buf * (G * 2 * kBwdRingMaxSources);
      if ((lane & ((1 << SHIFT) - 1)) == 0) mine[wig * (2 * kBwdRingMaxSources) + (lane >> SHIFT)] = val[0];
      group_sync(group, L);
#pragma unroll
      for (int i = 0; i < (K < 4 ? 4 : K); ++i) tot[i] = 0.f;
#pragma unroll
      for (int w = 0; w < G; ++w) {
#pragma unroll
        for (int i = 0; i < K; i += 4) {  // whole float4s; slots beyond K hold stale values
          const float4 t = *reinterpret_cast<const float4*>(&mine[w * (2 * kBwdRingMaxSources) + i]);
          tot[i] += t.x;
          tot[i + 1] += t.y;
          tot[i + 2] += t.z;
          tot[i + 3] += t.w;
        }
      }
    }
    // Every lane of the group holds its chunks in registers: refill the stages.
    if (leader) {
      fence_proxy_async();
      in_flight -= items;
      while (rows_to_issue > 0 && in_flight < nst) issue_one();
    }
    use_stage += items;
    if (use_stage >= nst) {
      use_stage -= nst;
      use_phase ^= 1u;
    }

    // ---- probabilities, delta, coefficients (every lane, from the staged logits)
    const float* zl = zl_sm + zbuf * 16;
    if (G == 1) __syncwarp();  // the staged logits were copied by other lanes of this warp
    const float row_max = zl[S], inv_sum = zl[S + 1];
    float prob[SMAX], delta = 0.f;
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      prob[s] = s < S ? __expf(zl[s] - row_max) * inv_sum : 0.f;
      delta = fmaf(prob[s], tot[2 * s + 1], delta);
    }

    // ---- value gradients from the chunks still in registers, dquery lanes
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      if (s < S) {
        const float ir = rsqrtf(tot[2 * s] * inv_rank + p.eps);
        const float dz = prob[s] * (tot[2 * s + 1] - delta);
        const float ca = ir * p.scale * dz, cb = ir * ir * dz * zl[s] * inv_rank;
        const float2 ps2 = make_float2(prob[s], prob[s]), ca2 = make_float2(ca, ca),
                     ncb2 = make_float2(-cb, -cb);
        __nv_bfloat16* out_row = p.write_dv ? p.grad.ptr[s] + row * p.grad.row_stride[s] : nullptr;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          if (row_ok(j)) {
            float2 dv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) dv[k] = __fmul2_rn(ps2, g2[j][k]);
            if (tail_ok(j)) {
              float2 v[4];
              v[0] = make_float2(bf16x2_lo(v_raw[s][j].x), bf16x2_hi(v_raw[s][j].x));
              v[1] = make_float2(bf16x2_lo(v_raw[s][j].y), bf16x2_hi(v_raw[s][j].y));
              v[2] = make_float2(bf16x2_lo(v_raw[s][j].z), bf16x2_hi(v_raw[s][j].z));
              v[3] = make_float2(bf16x2_lo(v_raw[s][j].w), bf16x2_hi(v_raw[s][j].w));
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                dv[k] = __ffma2_rn(ncb2, v[k], __ffma2_rn(ca2, q2[j][k], dv[k]));
                dq2[j][k] = __ffma2_rn(ca2, v[k], dq2[j][k]);
              }
            }
            if (out_row != nullptr) {
              uint4 packed;
              packed.x = pack_bf16x2(dv[0].x, dv[0].y);
              packed.y = pack_bf16x2(dv[1].x, dv[1].y);
              packed.z = pack_bf16x2(dv[2].x, dv[2].y);
              packed.w = pack_bf16x2(dv[3].x, dv[3].y);
              *reinterpret_cast<uint4*>(out_row + (int64_t)(gl + j * L) * 8) = packed;
            }
          }
        }
      }
    }
  }

  // One partial row per group.
  if (p.dq_partials != nullptr && gid < p.N) {
    float* prow = p.dq_partials + gid * R;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (tail_ok(j)) {
        float4* dst = reinterpret_cast<float4*>(prow + (int64_t)(gl + j * L - c0) * 8);
        dst[0] = make_float4(dq2[j][0].x, dq2[j][0].y, dq2[j][1].x, dq2[j][1].y);
        dst[1] = make_float4(dq2[j][2].x, dq2[j][2].y, dq2[j][3].x, dq2[j][3].y);
      }
    }
  }
  if (*abort_flag) {
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 200000ull) {
    }
  }
}

template <int G, int SE, bool FULL, int TAIL0>
inline int launch_bwd_ring_instance(const BwdParams& p, const BwdRingPlan& plan, int grid,
                                    cudaStream_t stream) {
  auto kernel = bwd_ring_kernel<G, SE, FULL, TAIL0>;
  static SmemGrant grant;
  if (int st = prepare_kernel(kernel, plan.smem_bytes, grant)) return st;
  kernel<<<grid, plan.cta_warps * 32, plan.smem_bytes, stream>>>(p, plan);
  return cudaGetLastError() == cudaSuccess ? 0 : 9;
}

template <int G, int SE>
inline int launch_bwd_ring_tail(const BwdParams& p, const BwdRingPlan& plan, int grid,
                                cudaStream_t stream) {
  if (p.R == p.D) return launch_bwd_ring_instance<G, SE, true, 0>(p, plan, grid, stream);
  return launch_bwd_ring_instance<G, SE, true, -1>(p, plan, grid, stream);
}

// Only lists of up to four sources run here: with five to eight sources in registers the
// kernel measured slower than the staged backward (3.3 vs 3.9 TB/s at S=5, D=4096).  Full
// rows with two or three sources get the exact-count instances (with four the compiler
// interleaves all sources and spills 150 to 380 bytes per thread); everything else the
// run-time form.
template <int G>
inline int launch_bwd_ring_smax(const BwdParams& p, const BwdRingPlan& plan, int grid,
                                cudaStream_t stream) {
  if constexpr (G <= 8) {
    if (p.D / 8 == G * 32 * kBwdRingChunks) {
      if (p.S == 2) return launch_bwd_ring_tail<G, 2>(p, plan, grid, stream);
      if (p.S == 3) return launch_bwd_ring_tail<G, 3>(p, plan, grid, stream);
    }
  }
  return launch_bwd_ring_instance<G, 0, false, -1>(p, plan, grid, stream);
}

// `max_rows` bounds the dquery partial rows (one per group); the count used is returned.
inline int launch_bwd_ring(const BwdParams& p, int sms, int max_rows, int* rows_out,
                           cudaStream_t stream) {
  BwdRingPlan plan;
  if (!make_bwd_ring_plan(p.S, p.D, p.R, &plan)) return 9;
  const int groups = plan.cta_warps / plan.group_warps;
  int64_t grid = (p.N + groups - 1) / groups;
  const int64_t cap = (int64_t)sms * plan.ctas_per_sm;
  if (grid > cap) grid = cap;
  if (grid * groups > max_rows) grid = max_rows / groups;
  // Fewer positions than one CTA has groups: the idle groups write no partial row.
  if (grid < 1 && p.N <= max_rows) grid = 1;
  if (grid < 1) return 9;
  int st;
  switch (plan.group_warps) {
    case 1: st = launch_bwd_ring_smax<1>(p, plan, (int)grid, stream); break;
    case 2: st = launch_bwd_ring_smax<2>(p, plan, (int)grid, stream); break;
    case 4: st = launch_bwd_ring_smax<4>(p, plan, (int)grid, stream); break;
    case 8: st = launch_bwd_ring_smax<8>(p, plan, (int)grid, stream); break;
    default: st = launch_bwd_ring_smax<16>(p, plan, (int)grid, stream); break;
  }
  // Groups beyond N write no partial row; with grid * groups <= N + groups - 1 only the
  // last CTA can have such groups, so count the rows that exist.
  const int64_t written = grid * groups < p.N ? grid * groups : p.N;
  *rows_out = (int)written;
  return st;
}

}  // namespace attnres_b200
