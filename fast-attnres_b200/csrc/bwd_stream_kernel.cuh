// One-pass streaming backward of the AttnRes read for the aligned layout (feature stride 1,
// 16-byte aligned rows, D and D-R multiples of 8).
//
// The staged ("stash") backward needs all S rows of a position in shared memory because
// delta = sum_s p_s (v_s . dO) is only known after every source has been reduced.  When the
// forward also saved its result (the BF16 output and the 16 bits of the FP32 result that its
// rounding dropped, see split_low16x2), delta = sum_d dO_d * result_d is available in full
// FP32 precision BEFORE any source is read, and every source can be finished the moment it
// arrives:
//
//   per position   the group (G warps, four 16-byte chunks per lane, as in the forward ring
//                  kernel) loads dO, out and residual from its ring, keeps dO in registers
//                  and reduces delta;
//   per 2 sources  load the two rows from the ring into registers, reduce
//                  (sum t^2, v . dO) of both with one folded butterfly (plus one named barrier
//                  when G > 1), refill the two stages, then for each of them form
//                  p_s, dz_s, the coefficients, write dV_s and add to the dquery lanes.
//
// Shared memory holds only the ring, so any S fits, three CTAs stay resident per SM and the
// loads of later sources overlap the stores of earlier ones.  The price is 6*D extra bytes per
// position (one more 16-bit row written by the forward, two more read here); which shapes take
// this kernel is decided by attnres_b200_wants_output_residual from measurements.
//
// In accumulate mode (template parameter ACC) the existing gradient row of every source rides
// the ring behind the source row and is added before the store: dsrc[s] += dV_s.
#pragma once

#include "fwd_ring_kernel.cuh"

namespace attnres_b200 {

struct BwdStreamPlan {
  int group_warps;  // G
  int cta_warps;    // 4 or 8
  int stages;       // ring depth per group
  int ctas_per_sm;
  uint32_t off_bars;
  uint32_t off_part;
  uint32_t off_zl;
  uint32_t off_tab;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

constexpr int kStreamLogitSlots = 136;  // S + 2 <= 131 floats, padded

// One entry of the shared-memory copy of the source table.  Indexed reads of the kernel
// parameter block go through the small constant cache; with tens of sources they miss it on
// the path that issues the loads, which is the path that keeps the ring full.  (The gradient
// table stays in the parameter block: its reads are hoisted far ahead of the stores, and a
// shared-memory copy measured slower.)
struct __align__(16) StreamRowRef {
  uint64_t base;       // address of row 0
  int64_t row_stride;  // elements
};

inline bool make_bwd_stream_plan(int S, int D, int R, BwdStreamPlan* plan) {
  if (!tma_shape_ok(D, R)) return false;
  const int chunks = D / 8;
  const int need = (chunks + 32 * kRingChunks - 1) / (32 * kRingChunks);
  int G = 1;
  while (G < need) G <<= 1;
  if (G > kRingMaxGroupWarps) return false;
  BwdStreamPlan p;
  p.group_warps = G;
  p.cta_warps = G > 4 ? 8 : 4;
  p.ctas_per_sm = p.cta_warps == 4 ? 3 : 1;
  const int groups = p.cta_warps / G;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  const uint32_t bars = (uint32_t)groups * 8u * 8u;
  const uint32_t part = (uint32_t)groups * 2u * kRingMaxGroupWarps * 16u;
  const uint32_t zl = (uint32_t)groups * 3u * kStreamLogitSlots * 4u;
  const uint32_t tab = 2u * (uint32_t)S * (uint32_t)sizeof(StreamRowRef);  // sources, gradients
  const uint32_t fixed = bars + part + zl + tab + 16u + 128u;
  const uint32_t room = (228u * 1024u - (uint32_t)p.ctas_per_sm * 1024u) / (uint32_t)p.ctas_per_sm;
  const uint32_t usable = room < (uint32_t)kSmemPerCtaMax ? room : (uint32_t)kSmemPerCtaMax;
  int stages = usable > fixed ? (int)((usable - fixed) / ((uint32_t)groups * row_bytes)) : 0;
  if (stages > 8) stages = 8;
  if (stages < 5) return false;
  p.stages = stages;
  uint32_t off = (uint32_t)groups * (uint32_t)stages * row_bytes;
  p.off_bars = align_up(off, 8);
  off = p.off_bars + bars;
  p.off_part = align_up(off, 16);
  off = p.off_part + part;
  p.off_zl = off;
  off += zl;
  p.off_tab = align_up(off, 16);
  off = p.off_tab + tab;
  p.off_abort = off;
  off += 16;
  p.smem_bytes = off;
  if (p.smem_bytes > (uint32_t)kSmemPerCtaMax) return false;
  *plan = p;
  return true;
}

inline bool bwd_stream_supported(int S, int D, int R) {
  BwdStreamPlan plan;
  return make_bwd_stream_plan(S, D, R, &plan);
}

__device__ __forceinline__ void unpack_pairs(const uint4& raw, float2* f) {
  f[0] = make_float2(bf16x2_lo(raw.x), bf16x2_hi(raw.x));
  f[1] = make_float2(bf16x2_lo(raw.y), bf16x2_hi(raw.y));
  f[2] = make_float2(bf16x2_lo(raw.z), bf16x2_hi(raw.z));
  f[3] = make_float2(bf16x2_lo(raw.w), bf16x2_hi(raw.w));
}

// FULL: the row is exactly G*32*4 chunks wide, so no lane ever holds a chunk beyond the row.
// TAIL0 >= 0 (needs FULL): the query tail starts at a lane-group boundary, chunks j >= TAIL0
// of every lane are tail chunks; TAIL0 < 0: per-lane predicates decide.
// SR (needs FULL): row size and ring depth (eight stages) are compile-time constants.
// ZE: registers of an absent second source are zero-filled (only changes code placement).
// ACC: accumulate.  The existing gradient row of every source travels through the ring right
// behind the source row (2 S + 3 items per position) and is added in FP32 before the one
// rounding to BF16; the four stages of a batch are refilled after the gradients are stored.
template <int G, bool FULL, int TAIL0, bool SR, bool ZE, bool ACC>
__global__ void __launch_bounds__((G > 4 ? 8 : 4) * 32, G > 4 ? 1 : 3)
bwd_stream_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ BwdStreamPlan plan) {
  static_assert(TAIL0 < 0 || FULL, "a compile-time tail boundary needs a full row");
  static_assert(!SR || FULL, "compile-time ring constants need a full row");
  constexpr int NV = kRingChunks, B = 2;
  constexpr int WARPS = G > 4 ? 8 : 4;
  constexpr int GROUPS = WARPS / G;
  constexpr int L = G * 32;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp / G, wig = warp % G;
  const int gl = wig * 32 + lane;
  const int S = p.S, R = p.R;
  // Full-row instances: width, row size and ring depth are compile-time constants.
  const int D = SR ? L * NV * 8 : p.D;
  const int CH = D / 8, c0 = (D - R) / 8;
  const int nst = SR ? kRingStaticStages : plan.stages;
  constexpr int K = ACC ? 2 : 1;  // ring items per source
  const int items = K * S + 3;    // dO, out, residual, then the sources
  const uint32_t row_bytes = (uint32_t)D * 2u;
  unsigned char* ring = smem + (size_t)group * (size_t)nst * row_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + plan.off_bars) + group * 8;
  float4* part_sm = reinterpret_cast<float4*>(smem + plan.off_part) +
                    group * (2 * kRingMaxGroupWarps);  // [2][8] x (ss0, dw0, ss1, dw1)
  float* zl_sm = reinterpret_cast<float*>(smem + plan.off_zl) + group * (3 * kStreamLogitSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + plan.off_abort);
  StreamRowRef* src_tab = reinterpret_cast<StreamRowRef*>(smem + plan.off_tab);
  StreamRowRef* grad_tab = src_tab + S;  // filled and read by the accumulating instances only

  for (int s = tid; s < S; s += WARPS * 32) {
    src_tab[s].base = reinterpret_cast<uint64_t>(p.src.ptr[s]);
    src_tab[s].row_stride = p.src.row_stride[s];
    if (ACC) {
      grad_tab[s].base = reinterpret_cast<uint64_t>(p.grad.ptr[s]);
      grad_tab[s].row_stride = p.grad.row_stride[s];
    }
  }
  if (tid == 0) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + plan.off_bars);
    for (int g = 0; g < GROUPS; ++g)
      for (int i = 0; i < nst; ++i) mbar_init(&bars[g * 8 + i], 1);
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

  int64_t rows_to_issue = my_rows;
  int in_flight = 0, issue_stage = 0, issue_item = 0;
  int64_t issue_row = gid;
  auto issue_one = [&]() {
    const __nv_bfloat16* src;
    if (issue_item == 0) src = p.grad_out + issue_row * p.go_row_stride;
    else if (issue_item == 1) src = p.out_saved + issue_row * (int64_t)D;
    else if (issue_item == 2) src = p.out_residual + issue_row * (int64_t)D;
    else {
      const int k = issue_item - 3;
      const StreamRowRef ref = ACC ? ((k & 1) ? grad_tab[k >> 1] : src_tab[k >> 1]) : src_tab[k];
      src = reinterpret_cast<const __nv_bfloat16*>(ref.base) + issue_row * ref.row_stride;
    }
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
  // Saved logits and statistics travel one position ahead (three buffers, as in the ring
  // backward): the lanes of the group's first warp copy logits[0..S), max, 1/sum.
  auto stage_logits = [&](int64_t row, int buffer) {
    if (wig == 0) {
      for (int i = lane; i < S + 2; i += 32) {
        const float* src = i < S ? p.logits + (int64_t)i * p.N + row
                                 : p.stats + (int64_t)(i - S) * p.N + row;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                         smem_addr(&zl_sm[buffer * kStreamLogitSlots + i])),
                     "l"(src)
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (my_rows > 0) stage_logits(gid, 0);

  RingCursor<SR> cursor(nst);
  int buf = 0, zbuf = 0;
  const float inv_rank = 1.0f / (float)R;

  for (int64_t row = gid; row < p.N; row += total_groups, zbuf = zbuf == 2 ? 0 : zbuf + 1) {
    if (row + total_groups < p.N) {
      stage_logits(row + total_groups, zbuf == 2 ? 0 : zbuf + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }

    // ---- dO into registers; delta = sum_d dO * (the forward's FP32 result)
    float2 g2[NV][4];
    float delta;
    {
      uint32_t phase;
      const int sg = cursor.stage(0, &phase);
      mbar_wait_fast(&full_bar[sg], phase, abort_flag);
      const int so = cursor.stage(1, &phase);
      mbar_wait_fast(&full_bar[so], phase, abort_flag);
      const int sr = cursor.stage(2, &phase);
      mbar_wait_fast(&full_bar[sr], phase, abort_flag);
      const uint4* gp = reinterpret_cast<const uint4*>(ring + (uint32_t)sg * row_bytes) + gl;
      const uint4* op = reinterpret_cast<const uint4*>(ring + (uint32_t)so * row_bytes) + gl;
      const uint4* rp = reinterpret_cast<const uint4*>(ring + (uint32_t)sr * row_bytes) + gl;
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (row_ok(j)) {
          unpack_pairs(gp[j * L], g2[j]);
          const uint4 o = op[j * L], r = rp[j * L];
          acc = __ffma2_rn(g2[j][0], join_low16x2(o.x, r.x), acc);
          acc = __ffma2_rn(g2[j][1], join_low16x2(o.y, r.y), acc);
          acc = __ffma2_rn(g2[j][2], join_low16x2(o.z, r.z), acc);
          acc = __ffma2_rn(g2[j][3], join_low16x2(o.w, r.w), acc);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) g2[j][k] = make_float2(0.f, 0.f);
        }
      }
      float part = warp_sum(acc.x + acc.y);
      if (G > 1) {
        float* mine = reinterpret_cast<float*>(part_sm + buf * kRingMaxGroupWarps);
        if (lane == 0) mine[wig * 4] = part;
        group_sync(group, L);
        part = 0.f;
#pragma unroll
        for (int w = 0; w < G; ++w) part += mine[w * 4];
        buf ^= 1;
      }
      delta = part;
      if (leader) {
        fence_proxy_async();
        in_flight -= 3;
        while (rows_to_issue > 0 && in_flight < nst) issue_one();
      }
      cursor.advance(3);
    }
    const float* zl = zl_sm + zbuf * kStreamLogitSlots;
    if (G == 1) __syncwarp();
    const float row_max = zl[S], inv_sum = zl[S + 1];

    // ---- the sources, two at a time (and a last single one when S is odd)
    // (A compile-time source count per batch lets the compiler interleave both sources and
    // spill; the count stays a run-time value here.)
    auto batch = [&](const int NB, const int s0) {
      uint4 raw[B][NV];
      float part[2 * B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float2 ss2 = make_float2(0.f, 0.f), dw2 = make_float2(0.f, 0.f);
        if (b < NB) {
          uint4(&mine)[NV] = raw[b];
          uint32_t phase;
          const int stage = cursor.stage(b * K, &phase);
          mbar_wait_fast(&full_bar[stage], phase, abort_flag);
          const uint4* vrow = reinterpret_cast<const uint4*>(ring + (uint32_t)stage * row_bytes) + gl;
#pragma unroll
          for (int j = 0; j < NV; ++j) mine[j] = row_ok(j) ? vrow[j * L] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            float2 v[4];
            unpack_pairs(mine[j], v);
#pragma unroll
            for (int k = 0; k < 4; ++k) dw2 = __ffma2_rn(v[k], g2[j][k], dw2);
            if (tail_ok(j)) {
#pragma unroll
              for (int k = 0; k < 4; ++k) ss2 = __ffma2_rn(v[k], v[k], ss2);
            }
          }
        } else if (ZE) {
#pragma unroll
          for (int j = 0; j < NV; ++j) raw[b][j] = make_uint4(0u, 0u, 0u, 0u);
        }
        part[2 * b] = ss2.x + ss2.y;
        part[2 * b + 1] = dw2.x + dw2.y;
      }
      // Folded butterfly over the warp (see the forward ring kernel).
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
      if (!ACC) {
        if (leader) {
          fence_proxy_async();
          in_flight -= NB;
          while (rows_to_issue > 0 && in_flight < nst) issue_one();
        }
        cursor.advance(NB);
      }

      // ---- finish the batch from the chunks still in registers
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (b >= NB) break;
        const int s = s0 + b;
        const float z = zl[s];
        const float prob = __expf(z - row_max) * inv_sum;
        const float ir = rsqrtf(tot[2 * b] * inv_rank + p.eps);
        const float dz = prob * (tot[2 * b + 1] - delta);
        const float ca = ir * p.scale * dz, cb = ir * ir * dz * z * inv_rank;
        const float2 ps2 = make_float2(prob, prob), ca2 = make_float2(ca, ca),
                     ncb2 = make_float2(-cb, -cb);
        __nv_bfloat16* out_row = p.write_dv ? p.grad.ptr[s] + row * p.grad.row_stride[s] : nullptr;
        const uint4* old_row = nullptr;
        if (ACC) {
          uint32_t phase;
          const int stage = cursor.stage(b * K + 1, &phase);
          mbar_wait_fast(&full_bar[stage], phase, abort_flag);
          old_row = reinterpret_cast<const uint4*>(ring + (uint32_t)stage * row_bytes) + gl;
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          if (row_ok(j)) {
            float2 dv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) dv[k] = __fmul2_rn(ps2, g2[j][k]);
            if (tail_ok(j)) {
              float2 v[4];
              unpack_pairs(raw[b][j], v);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                dv[k] = __ffma2_rn(ncb2, v[k], __ffma2_rn(ca2, q2[j][k], dv[k]));
                dq2[j][k] = __ffma2_rn(ca2, v[k], dq2[j][k]);
              }
            }
            if (out_row != nullptr) {
              if (ACC) {
                float2 old[4];
                unpack_pairs(old_row[j * L], old);
#pragma unroll
                for (int k = 0; k < 4; ++k) dv[k] = __fadd2_rn(dv[k], old[k]);
              }
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
      if (ACC) {
        // The old gradient rows were read from the ring during the stores: every lane of the
        // group must be past them before the leader refills the batch's stages.
        if (G > 1) group_sync(group, L);
        else __syncwarp();
        if (leader) {
          fence_proxy_async();
          in_flight -= K * NB;
          while (rows_to_issue > 0 && in_flight < nst) issue_one();
        }
        cursor.advance(K * NB);
      }
      buf ^= 1;
    };
    for (int s0 = 0; s0 < S; s0 += B) batch(S - s0 < B ? S - s0 : B, s0);
  }

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

template <int G, bool FULL, int TAIL0, bool SR, bool ZE, bool ACC>
inline int launch_bwd_stream_variant(const BwdParams& p, const BwdStreamPlan& plan, int grid,
                                     cudaStream_t stream) {
  auto kernel = bwd_stream_kernel<G, FULL, TAIL0, SR, ZE, ACC>;
  static SmemGrant grant;
  if (int st = prepare_kernel(kernel, plan.smem_bytes, grant)) return st;
  kernel<<<grid, plan.cta_warps * 32, plan.smem_bytes, stream>>>(p, plan);
  return cudaGetLastError() == cudaSuccess ? 0 : 9;
}

// Which switches win was measured per group size on B200 (N = 16384, GB/s of algorithmic
// bytes at S = 49, best against worst combination):
//   G = 1 (D = 1024): all three on, 5109 against 3462;   G = 2 (D = 2048): SR alone, 6367 / 5457
//   (SR + ZE, the best before the saved output became an exact FP32 pair, fell to 5578);
//   G = 4 (D = 4096): none, 6336 / 5393 (SR alone costs 14 %);   G = 8 (D = 8192): SR + tail, 6342 / 5489.
// The accumulating instances use the same choice.
template <int G, bool ACC>
inline int launch_bwd_stream_instance(const BwdParams& p, const BwdStreamPlan& plan, int grid,
                                      cudaStream_t stream) {
  const bool full = p.D / 8 == G * 32 * kRingChunks && plan.stages == kRingStaticStages;
  if (!full) return launch_bwd_stream_variant<G, false, -1, false, false, ACC>(p, plan, grid, stream);
  constexpr bool SR = G != 4, ZE = G == 1;
  constexpr int TAIL0 = (G == 1 || G == 8) ? 0 : -1;
  if (TAIL0 == 0 && p.R == p.D)
    return launch_bwd_stream_variant<G, true, TAIL0, SR, ZE, ACC>(p, plan, grid, stream);
  return launch_bwd_stream_variant<G, true, -1, SR, ZE, ACC>(p, plan, grid, stream);
}

template <bool ACC>
inline int launch_bwd_stream_group(const BwdParams& p, const BwdStreamPlan& plan, int grid,
                                   cudaStream_t stream) {
  switch (plan.group_warps) {
    case 1: return launch_bwd_stream_instance<1, ACC>(p, plan, grid, stream);
    case 2: return launch_bwd_stream_instance<2, ACC>(p, plan, grid, stream);
    case 4: return launch_bwd_stream_instance<4, ACC>(p, plan, grid, stream);
    default: return launch_bwd_stream_instance<8, ACC>(p, plan, grid, stream);
  }
}

// `max_rows` bounds the dquery partial rows (one per group); the count used is returned.
inline int launch_bwd_stream(const BwdParams& p, int sms, int max_rows, int* rows_out,
                             cudaStream_t stream) {
  BwdStreamPlan plan;
  if (!make_bwd_stream_plan(p.S, p.D, p.R, &plan)) return 9;
  const int groups = plan.cta_warps / plan.group_warps;
  int64_t grid = (p.N + groups - 1) / groups;
  const int64_t cap = (int64_t)sms * plan.ctas_per_sm;
  if (grid > cap) grid = cap;
  if (grid * groups > max_rows) grid = max_rows / groups;
  // Fewer positions than one CTA has groups: the idle groups write no partial row.
  if (grid < 1 && p.N <= max_rows) grid = 1;
  if (grid < 1) return 9;
  const int st = p.accumulate ? launch_bwd_stream_group<true>(p, plan, (int)grid, stream)
                              : launch_bwd_stream_group<false>(p, plan, (int)grid, stream);
  const int64_t written = grid * groups < p.N ? grid * groups : p.N;
  *rows_out = (int)written;
  return st;
}

}  // namespace attnres_b200
