// TMA-staged backward of the AttnRes read for the aligned layout (feature stride 1,
// 16-byte aligned rows, D and D-R multiples of 8).
//
// Persistent, warp-specialised CTAs.  All S source rows of a position plus its
// upstream row are staged in shared memory by one producer lane issuing 1-D bulk
// asynchronous copies ("stash"), so the position is read from HBM exactly once:
//
//   sweep 1  every warp owns a fixed slice of the row (its upstream lanes stay in
//            registers) and walks the sources dealt to it, reducing
//            dw_s = v_s . dO and the tail sum of squares out of shared memory;
//   middle   warp 0 turns the saved logits into probabilities, forms
//            delta = sum_s p_s dw_s and the three coefficients of every source;
//   sweep 2  every thread owns one or two 16-byte chunks: it re-reads the tail of
//            each source from shared memory, writes
//            dV_s = p_s dO + [tail] (ca_s q - cb_s v_s) and accumulates its lanes
//            of dquery in registers for all positions of the CTA.
//
// A slot is refilled with the next position's source as soon as sweep 2 has
// consumed it.  Row arithmetic uses the packed FP32x2 FMA of sm_100.
#pragma once

#include "tma_common.cuh"

namespace attnres_b200 {

constexpr int kStashSliceChunks = 4;  // chunks of the row a lane covers in sweep 1
constexpr int kStashMaxBuffers = 4;

struct BwdPlan {
  int consumer_warps;
  int row_buffers;  // positions staged at once
  int parts;        // slices of the row in sweep 1 (divides consumer_warps)
  int ctas_per_sm;
  uint32_t row_buffer_bytes;
  uint32_t off_part;
  uint32_t off_coef;
  uint32_t off_bars;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

// 16-byte chunks owned by a consumer thread in sweep 2.
inline int tma_chunks_per_thread(int D) { return D > 4096 ? 2 : 1; }

inline int tma_consumer_warps(int D) {
  const int chunks = D / 8;
  return (chunks + 32 * tma_chunks_per_thread(D) - 1) / (32 * tma_chunks_per_thread(D));
}

// Slices of the row for sweep 1: a divisor of the warp count (so a warp always owns
// the same slice), at most kStashSliceChunks chunks per lane, cheapest by a small
// instruction-count model of (rounds of sources per warp) x (work per source).
inline int stash_parts(int S, int D) {
  const int W = tma_consumer_warps(D), CH = D / 8;
  int best = 0;
  long best_cost = 0;
  for (int np = 1; np <= W; ++np) {
    if (W % np != 0) continue;
    const int iters = (CH + 32 * np - 1) / (32 * np);
    if (iters > kStashSliceChunks) continue;
    const long rounds = ((long)S * np + W - 1) / W;
    const long cost = rounds * (iters * 20L + 24L);
    if (best == 0 || cost < best_cost) {
      best = np;
      best_cost = cost;
    }
  }
  return best;
}

inline bool make_bwd_plan(int S, int D, int R, BwdPlan* plan) {
  if (!tma_shape_ok(D, R)) return false;
  BwdPlan p;
  p.consumer_warps = tma_consumer_warps(D);
  const int W = p.consumer_warps;
  p.parts = stash_parts(S, D);
  if (p.parts < 1) return false;
  p.row_buffer_bytes = (uint32_t)(S + 1) * (uint32_t)D * 2u;
  const uint32_t part_bytes = align_up((uint32_t)S * (uint32_t)p.parts * 2u * 4u, 16);
  const uint32_t coef_bytes = (uint32_t)S * 16u;
  const uint32_t bars_bytes = (uint32_t)kStashMaxBuffers * (uint32_t)(S + 1) * 2u * 8u;
  const uint32_t fixed = part_bytes + coef_bytes + bars_bytes + 16 + 1024;
  const int threads = 32 * (W + 1);
  // Resident CTAs per SM: bounded by threads, by registers (96 per thread, the compiled figure) and, below, by the staged rows.
  const int regs = 96;
  int ctas = 2048 / threads;
  if (ctas > 65536 / (threads * regs)) ctas = 65536 / (threads * regs);
  if (ctas < 1) ctas = 1;
  if (ctas > 6) ctas = 6;
  int buffers = 0;
  while (ctas >= 1) {
    const uint32_t per_cta = (ctas == 1 ? (uint32_t)kSmemPerCtaMax : (uint32_t)kSmemPerSm / ctas);
    buffers = per_cta > fixed ? (int)((per_cta - fixed) / p.row_buffer_bytes) : 0;
    if (buffers >= 1) break;
    --ctas;
  }
  if (ctas < 1 || buffers < 1) return false;
  if (buffers > kStashMaxBuffers) buffers = kStashMaxBuffers;
  p.row_buffers = buffers;
  p.ctas_per_sm = ctas;
  uint32_t off = (uint32_t)buffers * p.row_buffer_bytes;
  p.off_part = off;
  off += part_bytes;
  p.off_coef = off;
  off += coef_bytes;
  p.off_bars = align_up(off, 8);
  off = p.off_bars + bars_bytes;
  p.off_abort = off;
  off += 16;
  p.smem_bytes = off;
  if (p.smem_bytes > (uint32_t)kSmemPerCtaMax) return false;
  *plan = p;
  return true;
}

inline bool tma_bwd_supported(int S, int D, int R) {
  BwdPlan plan;
  return make_bwd_plan(S, D, R, &plan);
}

__device__ __forceinline__ void unpack8_pairs(const uint4& raw, float2* f) {
  f[0] = make_float2(bf16x2_lo(raw.x), bf16x2_hi(raw.x));
  f[1] = make_float2(bf16x2_lo(raw.y), bf16x2_hi(raw.y));
  f[2] = make_float2(bf16x2_lo(raw.z), bf16x2_hi(raw.z));
  f[3] = make_float2(bf16x2_lo(raw.w), bf16x2_hi(raw.w));
}

template <int NV>
__global__ void __launch_bounds__(544)
bwd_tma_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ BwdPlan plan) {
  constexpr int GK = kStashSliceChunks;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = plan.consumer_warps, T = W * 32;
  const int S = p.S, D = p.D, R = p.R;
  const int CH = D / 8, c0 = (D - R) / 8;
  const int NRB = plan.row_buffers, NP = plan.parts, slots = S + 1;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  float* part_sm = reinterpret_cast<float*>(smem + plan.off_part);    // [S][NP][2] (ss, dw)
  float4* coef_sm = reinterpret_cast<float4*>(smem + plan.off_coef);  // [S] (p, ca, cb, -)
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + plan.off_bars);  // [NRB][slots]
  uint64_t* empty_bar = full_bar + NRB * slots;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + plan.off_abort);

  if (tid == 0) {
    for (int i = 0; i < NRB * slots; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], W);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == W) {
    // ---- producer: slot 0 of a row buffer holds the upstream row, slot 1+s source s
    if (lane == 0) {
      uint32_t rb = 0, fill_parity = 1;  // parity of the release that precedes a refill
      bool first_pass = true;
      bool alive = true;
      int issued_slots = 0;
      uint32_t rows_issued = 0;
      for (int64_t row = blockIdx.x; row < p.N && alive; row += gridDim.x) {
        unsigned char* base = smem + (size_t)rb * plan.row_buffer_bytes;
        issued_slots = 0;
        for (int slot = 0; slot < slots; ++slot) {
          uint64_t* fb = &full_bar[rb * slots + slot];
          if (!first_pass && !mbar_wait(&empty_bar[rb * slots + slot], fill_parity, abort_flag)) {
            alive = false;
            break;
          }
          const __nv_bfloat16* src =
              slot == 0 ? p.grad_out + row * p.go_row_stride
                        : p.src.ptr[slot - 1] + row * p.src.row_stride[slot - 1];
          mbar_expect_tx(fb, row_bytes);
          bulk_load(base + (size_t)slot * row_bytes, src, row_bytes, fb);
          ++issued_slots;
        }
        ++rows_issued;
        if (++rb == (uint32_t)NRB) {
          rb = 0;
          if (first_pass) {
            first_pass = false;
            fill_parity = 0;
          } else {
            fill_parity ^= 1u;
          }
        }
      }
      if (!alive) {
        // Copies already issued complete within microseconds; give them a fixed 200 us so
        // none lands after the CTA has retired and its shared memory has a new owner.
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) {
        }
      }
      (void)issued_slots;
      (void)rows_issued;
    }
    return;
  }

  // ---- consumers
  // Sweep-2 ownership: chunk(s) tid (+T), with the matching query lanes and dquery sums.
  int own_chunk[NV];
  float2 q2[NV][4], dq2[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    own_chunk[j] = tid + j * T;
    const bool tail = own_chunk[j] < CH && own_chunk[j] >= c0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = 0.f, hi = 0.f;
      if (tail) {
        const int64_t r = (int64_t)(own_chunk[j] - c0) * 8 + 2 * k;
        lo = __bfloat162float(p.query[r * p.query_stride]);
        hi = __bfloat162float(p.query[(r + 1) * p.query_stride]);
      }
      q2[j][k] = make_float2(lo, hi);
      dq2[j][k] = make_float2(0.f, 0.f);
    }
  }
  // Sweep-1 ownership: slice `my_part` of the row, sources my_first, my_first + step, ...
  const int my_part = warp % NP, my_first = warp / NP, my_step = W / NP;
  constexpr int KS = (kMaxSources + 31) / 32;
  const float inv_rank = 1.0f / (float)R;
  uint32_t rb = 0, parity = 0;
  for (int64_t row = blockIdx.x; row < p.N; row += gridDim.x) {
    const unsigned char* base = smem + (size_t)rb * plan.row_buffer_bytes;
    uint64_t* full_row = &full_bar[rb * slots];
    uint64_t* empty_row = &empty_bar[rb * slots];

    // Saved logits and statistics of this position, fetched early by warp 0.
    float zl[KS], row_max = 0.f, inv_sum = 0.f;
    if (warp == 0) {
      row_max = p.stats[row];
      inv_sum = p.stats[p.N + row];
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int s = lane + 32 * k;
        zl[k] = s < S ? p.logits[(int64_t)s * p.N + row] : 0.f;
      }
    }

    // ---- sweep 1
    mbar_wait(&full_row[0], parity, abort_flag);
    const uint4* grow_sm = reinterpret_cast<const uint4*>(base);
    {
      float2 gs[GK][4];
#pragma unroll
      for (int k = 0; k < GK; ++k) {
        const int c = my_part * 32 + lane + 32 * NP * k;
        if (c < CH) {
          unpack8_pairs(grow_sm[c], gs[k]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) gs[k][e] = make_float2(0.f, 0.f);
        }
      }
      for (int s = my_first; s < S; s += my_step) {
        mbar_wait(&full_row[1 + s], parity, abort_flag);
        const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * row_bytes);
        float2 ss2 = make_float2(0.f, 0.f), dw2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < GK; ++k) {
          const int c = my_part * 32 + lane + 32 * NP * k;
          if (c < CH) {
            float2 v[4];
            unpack8_pairs(vrow[c], v);
#pragma unroll
            for (int e = 0; e < 4; ++e) dw2 = __ffma2_rn(v[e], gs[k][e], dw2);
            if (c >= c0) {
#pragma unroll
              for (int e = 0; e < 4; ++e) ss2 = __ffma2_rn(v[e], v[e], ss2);
            }
          }
        }
        // Folded butterfly: lanes 0-15 end with the warp's sum of squares, 16-31 with dw.
        const float ss = ss2.x + ss2.y, dw = dw2.x + dw2.y;
        const bool up = (lane & 16) != 0;
        float keep = up ? dw : ss;
        keep += __shfl_xor_sync(0xffffffffu, up ? ss : dw, 16);
        keep += __shfl_xor_sync(0xffffffffu, keep, 8);
        keep += __shfl_xor_sync(0xffffffffu, keep, 4);
        keep += __shfl_xor_sync(0xffffffffu, keep, 2);
        keep += __shfl_xor_sync(0xffffffffu, keep, 1);
        if ((lane & 15) == 0) part_sm[(s * NP + my_part) * 2 + (lane >> 4)] = keep;
      }
    }
    consumer_sync(T);

    // ---- delta and the per-source coefficients (warp 0)
    if (warp == 0) {
      float prob[KS], dws[KS], irs[KS];
      float local = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int s = lane + 32 * k;
        prob[k] = dws[k] = irs[k] = 0.f;
        if (s < S) {
          float ss = 0.f, dw = 0.f;
          for (int part = 0; part < NP; ++part) {
            const float2 v = *reinterpret_cast<const float2*>(&part_sm[(s * NP + part) * 2]);
            ss += v.x;
            dw += v.y;
          }
          irs[k] = rsqrtf(ss * inv_rank + p.eps);
          dws[k] = dw;
          prob[k] = __expf(zl[k] - row_max) * inv_sum;
          local = fmaf(prob[k], dw, local);
        }
      }
      const float delta = warp_sum(local);
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int s = lane + 32 * k;
        if (s < S) {
          const float dz = prob[k] * (dws[k] - delta);
          coef_sm[s] = make_float4(prob[k], irs[k] * p.scale * dz,
                                   irs[k] * irs[k] * dz * zl[k] * inv_rank, 0.f);
        }
      }
    }
    consumer_sync(T);

    // ---- sweep 2
    float2 g2[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_chunk[j] < CH) {
        unpack8_pairs(grow_sm[own_chunk[j]], g2[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) g2[j][e] = make_float2(0.f, 0.f);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_row[0]);
    for (int s = 0; s < S; ++s) {
      const float4 cf = coef_sm[s];
      const float2 ps2 = make_float2(cf.x, cf.x), ca2 = make_float2(cf.y, cf.y),
                   ncb2 = make_float2(-cf.z, -cf.z);
      const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * row_bytes);
      __nv_bfloat16* out_row = p.write_dv ? p.grad.ptr[s] + row * p.grad.row_stride[s] : nullptr;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (own_chunk[j] < CH) {
          float2 dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] = __fmul2_rn(ps2, g2[j][e]);
          if (own_chunk[j] >= c0) {
            // Observe the copy's completion in this thread before reading its bytes.
            mbar_wait(&full_row[1 + s], parity, abort_flag);
            float2 v[4];
            unpack8_pairs(vrow[own_chunk[j]], v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              dv[e] = __ffma2_rn(ncb2, v[e], __ffma2_rn(ca2, q2[j][e], dv[e]));
              dq2[j][e] = __ffma2_rn(ca2, v[e], dq2[j][e]);
            }
          }
          if (out_row != nullptr) {
            uint4 packed;
            packed.x = pack_bf16x2(dv[0].x, dv[0].y);
            packed.y = pack_bf16x2(dv[1].x, dv[1].y);
            packed.z = pack_bf16x2(dv[2].x, dv[2].y);
            packed.w = pack_bf16x2(dv[3].x, dv[3].y);
            *reinterpret_cast<uint4*>(out_row + (int64_t)own_chunk[j] * 8) = packed;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_row[1 + s]);
    }
    if (++rb == (uint32_t)NRB) {
      rb = 0;
      parity ^= 1u;
    }
  }

  if (p.dq_partials != nullptr) {
    float* prow = p.dq_partials + (int64_t)blockIdx.x * R;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_chunk[j] < CH && own_chunk[j] >= c0) {
        float4* dst = reinterpret_cast<float4*>(prow + (own_chunk[j] - c0) * 8);
        dst[0] = make_float4(dq2[j][0].x, dq2[j][0].y, dq2[j][1].x, dq2[j][1].y);
        dst[1] = make_float4(dq2[j][2].x, dq2[j][2].y, dq2[j][3].x, dq2[j][3].y);
      }
    }
  }
}

// `max_grid` bounds the grid by the rows of the dquery workspace; the grid used
// is returned so the second-stage reduction sums exactly the rows written.
inline int launch_bwd_tma(const BwdParams& p, int sms, int max_grid, int* grid_out,
                          cudaStream_t stream) {
  BwdPlan plan;
  if (!make_bwd_plan(p.S, p.D, p.R, &plan)) return 9;
  const int threads = 32 * (plan.consumer_warps + 1);
  int64_t cap = (int64_t)sms * plan.ctas_per_sm;
  if (cap > max_grid) cap = max_grid;
  const int grid = (int)(p.N < cap ? p.N : cap);
  if (tma_chunks_per_thread(p.D) == 1) {
    if (int st = prepare_kernel(bwd_tma_kernel<1>, plan.smem_bytes)) return st;
    bwd_tma_kernel<1><<<grid, threads, plan.smem_bytes, stream>>>(p, plan);
  } else {
    if (int st = prepare_kernel(bwd_tma_kernel<2>, plan.smem_bytes)) return st;
    bwd_tma_kernel<2><<<grid, threads, plan.smem_bytes, stream>>>(p, plan);
  }
  *grid_out = grid;
  return cudaGetLastError() == cudaSuccess ? 0 : 9;
}

}  // namespace attnres_b200
