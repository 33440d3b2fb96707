// TMA-staged backward of the AttnRes read for the aligned layout (feature stride 1,
// 16-byte aligned rows, D and D-R multiples of 8).
//
// Persistent, warp-specialised CTAs.  All S source rows of a position plus its
// upstream row are staged in shared memory by one producer lane issuing 1-D bulk
// asynchronous copies ("stash"), so the position is read from HBM exactly once:
// sweep 1 reduces dw_s = v_s . dO and the key norms out of shared memory,
// delta = sum_s p_s dw_s, sweep 2 re-reads the tails from shared memory and
// writes dV.  A slot is refilled with the next position's source as soon as
// sweep 2 has consumed it.
#pragma once

#include "tma_common.cuh"

namespace attnres_b200 {

struct BwdPlan {
  int consumer_warps;
  int row_buffers;  // positions staged at once
  int parts;        // warps per source in sweep 1
  int ctas_per_sm;
  uint32_t row_buffer_bytes;
  uint32_t off_part;
  uint32_t off_coef;
  uint32_t off_bars;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

// NV = 16-byte chunks owned by a consumer thread in the accumulation sweep.
inline int tma_chunks_per_thread(int D) { return D > 4096 ? 2 : 1; }

inline int tma_consumer_warps(int D) {
  const int chunks = D / 8;
  return (chunks + 32 * tma_chunks_per_thread(D) - 1) / (32 * tma_chunks_per_thread(D));
}

inline bool make_bwd_plan(int S, int D, int R, BwdPlan* plan) {
  if (!tma_shape_ok(D, R)) return false;
  BwdPlan p;
  p.consumer_warps = tma_consumer_warps(D);
  const int W = p.consumer_warps;
  const int chunk_groups = (D / 8 + 31) / 32;
  p.parts = W / S;
  if (p.parts > chunk_groups) p.parts = chunk_groups;
  if (p.parts < 1) p.parts = 1;
  p.row_buffer_bytes = (uint32_t)(S + 1) * (uint32_t)D * 2u;
  const uint32_t part_bytes = align_up((uint32_t)S * (uint32_t)p.parts * 2u * 4u, 16);
  const uint32_t coef_bytes = align_up((uint32_t)S * 3u * 4u, 16);
  const int max_buffers = 4;
  const uint32_t bars_bytes = (uint32_t)max_buffers * (uint32_t)(S + 1) * 2u * 8u;
  const uint32_t fixed = part_bytes + coef_bytes + bars_bytes + 16 + 1024;
  const int threads = 32 * (W + 1);
  // Resident CTAs per SM: bounded by threads, by registers (about 72 per thread with one
  // chunk per thread, 100 with two) and, below, by the staged rows.
  const int regs = tma_chunks_per_thread(D) == 1 ? 72 : 100;
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
  if (buffers > max_buffers) buffers = max_buffers;
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

// ---------------------------------------------------------------- backward

template <int NV>
__global__ void __launch_bounds__(544)
bwd_tma_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ BwdPlan plan) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = plan.consumer_warps, T = W * 32;
  const int S = p.S, D = p.D, R = p.R;
  const int CH = D / 8, c0 = (D - R) / 8;
  const int NRB = plan.row_buffers, NP = plan.parts, slots = S + 1;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  float2* part_sm = reinterpret_cast<float2*>(smem + plan.off_part);   // [S][NP] (ss, dw)
  float* coef_sm = reinterpret_cast<float*>(smem + plan.off_coef);     // [S][3]
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
      uint32_t count = 0;  // rows issued
      bool alive = true;
      int issued_slots = 0;
      for (int64_t row = blockIdx.x; row < p.N && alive; row += gridDim.x, ++count) {
        const uint32_t rb = count % NRB, fill = count / NRB;
        unsigned char* base = smem + (size_t)rb * plan.row_buffer_bytes;
        issued_slots = 0;
        for (int slot = 0; slot < slots; ++slot) {
          uint64_t* fb = &full_bar[rb * slots + slot];
          if (fill > 0 && !mbar_wait(&empty_bar[rb * slots + slot], (fill - 1) & 1u, abort_flag)) {
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
      }
      if (!alive) {
        // Bounded wait for the copies of the row that was being issued and the ones before it.
        for (uint32_t back = 0; back < (uint32_t)NRB && back <= count; ++back) {
          const uint32_t c = count - back;
          const int n = back == 0 ? issued_slots : slots;
          for (int slot = 0; slot < n; ++slot) {
            const uint64_t start = global_timer_ns();
            while (!mbar_try_wait(&full_bar[(c % NRB) * slots + slot], (c / NRB) & 1u) &&
                   global_timer_ns() - start < kWaitTimeoutNs / 8) {
            }
          }
        }
      }
    }
    return;
  }

  // ---- consumers
  int own_chunk[NV];
  float q[NV][8], dq[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    own_chunk[j] = tid + j * T;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int d = own_chunk[j] * 8 + e;
      q[j][e] = (own_chunk[j] < CH && own_chunk[j] >= c0)
                    ? __bfloat162float(p.query[(int64_t)(d - (D - R)) * p.query_stride])
                    : 0.f;
      dq[j][e] = 0.f;
    }
  }
  constexpr int KS = (kMaxSources + 31) / 32;
  const float rank_f = (float)R;
  uint32_t count = 0;
  for (int64_t row = blockIdx.x; row < p.N; row += gridDim.x, ++count) {
    const uint32_t rb = count % NRB, parity = (count / NRB) & 1u;
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

    // sweep 1: (source, part) pairs dealt round-robin to the warps
    mbar_wait(&full_row[0], parity, abort_flag);
    const uint4* grow_sm = reinterpret_cast<const uint4*>(base);
    for (int pair = warp; pair < S * NP; pair += W) {
      const int s = pair / NP, part = pair - s * NP;
      mbar_wait(&full_row[1 + s], parity, abort_flag);
      const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * row_bytes);
      float ss = 0.f, dw = 0.f;
      for (int c = part * 32 + lane; c < CH; c += 32 * NP) {
        const uint4 v = vrow[c];
        dw = dot8(v, grow_sm[c], dw);
        if (c >= c0) ss = dot8(v, v, ss);
      }
      ss = warp_sum(ss);
      dw = warp_sum(dw);
      if (lane == 0) part_sm[pair] = make_float2(ss, dw);
    }
    consumer_sync(T);

    // delta and the per-source coefficients (warp 0)
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
            const float2 v = part_sm[s * NP + part];
            ss += v.x;
            dw += v.y;
          }
          irs[k] = rsqrtf(ss / rank_f + p.eps);
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
          coef_sm[3 * s + 0] = prob[k];
          coef_sm[3 * s + 1] = irs[k] * p.scale * dz;
          coef_sm[3 * s + 2] = irs[k] * irs[k] * dz * zl[k] / rank_f;
        }
      }
    }
    consumer_sync(T);

    // sweep 2: dV rows and this thread's share of dquery
    float g[NV][8];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_chunk[j] < CH) {
        unpack8(grow_sm[own_chunk[j]], g[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) g[j][e] = 0.f;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_row[0]);
    for (int s = 0; s < S; ++s) {
      const float ps = coef_sm[3 * s], ca = coef_sm[3 * s + 1], cb = coef_sm[3 * s + 2];
      const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * row_bytes);
      __nv_bfloat16* out_row = p.write_dv ? p.grad.ptr[s] + row * p.grad.row_stride[s] : nullptr;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (own_chunk[j] < CH) {
          float dv[8];
          if (own_chunk[j] >= c0) {
            // Observe the copy's completion in this thread before reading its bytes.
            mbar_wait(&full_row[1 + s], parity, abort_flag);
            float v[8];
            unpack8(vrow[own_chunk[j]], v);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              dv[e] = fmaf(ps, g[j][e], fmaf(ca, q[j][e], -cb * v[e]));
              dq[j][e] = fmaf(ca, v[e], dq[j][e]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) dv[e] = ps * g[j][e];
          }
          if (out_row != nullptr)
            *reinterpret_cast<uint4*>(out_row + (int64_t)own_chunk[j] * 8) = pack8(dv);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_row[1 + s]);
    }
  }

  if (p.dq_partials != nullptr) {
    float* prow = p.dq_partials + (int64_t)blockIdx.x * R;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_chunk[j] < CH && own_chunk[j] >= c0) {
        float4* dst = reinterpret_cast<float4*>(prow + (own_chunk[j] - c0) * 8);
        dst[0] = make_float4(dq[j][0], dq[j][1], dq[j][2], dq[j][3]);
        dst[1] = make_float4(dq[j][4], dq[j][5], dq[j][6], dq[j][7]);
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
