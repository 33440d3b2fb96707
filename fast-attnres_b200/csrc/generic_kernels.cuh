// Layout-generic AttnRes read kernels: any row / feature stride, any width
// 1..8192, any base alignment, 64-bit offsets.  One CTA walks rows; each thread
// owns NJ chunks of VEC consecutive features (VEC = 8 uses 16-byte accesses and
// needs the aligned layout, VEC = 1 is element-wise).  These kernels cover what
// the TMA-staged family does not take and are the cross-check for it.
//
// Equations follow validation/oracle.py:13-19 (forward) and the closed-form
// gradient the reference kernels use (src/attnres/_kernels/fixed_tail.py:606-864).
#pragma once

#include "common.cuh"

namespace attnres_b200 {

// Loads the calling thread's NJ*VEC features of one row as FP32 (zero beyond D).
template <int VEC, int NJ, int T>
__device__ __forceinline__ void load_row(float* dst, const __nv_bfloat16* base,
                                         int64_t feat_stride, int D, int tid) {
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int c = j * T + tid;
    if constexpr (VEC == 8) {
      if (c * 8 < D) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)c * 8));
        unpack8(raw, dst + j * 8);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) dst[j * 8 + e] = 0.f;
      }
    } else {
      const unsigned short* b16 = reinterpret_cast<const unsigned short*>(base);
      dst[j] = (c < D) ? bf16_bits_to_float(__ldg(b16 + (int64_t)c * feat_stride)) : 0.f;
    }
  }
}

// Sums K per-thread values over the CTA.  `scratch` is [2][K][T/32]; the
// caller flips `parity` on every call so consecutive reductions use alternate
// halves and need a single barrier each.  Warps are added in index order.
template <int K, int T>
__device__ __forceinline__ void block_sum(float* vals, float* scratch, int& parity, int tid) {
  constexpr int NW = T / 32;
  const int lane = tid & 31, warp = tid >> 5;
  float* buf = scratch + parity * (K * NW);
#pragma unroll
  for (int k = 0; k < K; ++k) vals[k] = warp_sum(vals[k]);
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < K; ++k) buf[k * NW + warp] = vals[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < K; ++k) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) t += buf[k * NW + w];
    vals[k] = t;
  }
  parity ^= 1;
}

// LN: also write the LayerNorm of the row (FwdParams::ln_out); a separate instance so that
// the plain forward carries none of it.
template <int VEC, int NJ, int T, int B, bool LN>
__global__ void __launch_bounds__(T)
fwd_generic_kernel(const __grid_constant__ FwdParams p) {
  constexpr int NE = VEC * NJ;
  constexpr int NW = T / 32;
  __shared__ float scratch[2 * 2 * B * NW];
  const int tid = threadIdx.x;
  const int D = p.D, S = p.S, tail0 = p.D - p.R;
  const float rank_f = (float)p.R;

  // Query lanes owned by this thread (zero outside the tail), loaded once.
  float q[NE];
  uint32_t tailmask = 0;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const int d = (j * T + tid) * VEC + e;
      const bool in_tail = d < D && d >= tail0;
      q[j * VEC + e] = in_tail ? __bfloat162float(p.query[(int64_t)(d - tail0) * p.query_stride])
                               : 0.f;
      if (in_tail) tailmask |= 1u << (j * VEC + e);
    }
  }

  int parity = 0;
  for (int64_t row = blockIdx.x; row < p.N; row += gridDim.x) {
    float acc[NE];
#pragma unroll
    for (int i = 0; i < NE; ++i) acc[i] = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;

    for (int s0 = 0; s0 < S; s0 += B) {
      float v[B][NE];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int s = s0 + b;
        if (s < S) {
          load_row<VEC, NJ, T>(v[b], p.src.ptr[s] + row * p.src.row_stride[s],
                               p.src.feat_stride[s], D, tid);
        } else {
#pragma unroll
          for (int i = 0; i < NE; ++i) v[b][i] = 0.f;
        }
      }
      // part[2b] = sum of squares over the tail, part[2b+1] = tail . query
      float part[2 * B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float ss = 0.f, dt = 0.f;
#pragma unroll
        for (int i = 0; i < NE; ++i) {
          const float x = v[b][i];
          dt = fmaf(x, q[i], dt);
          if ((tailmask >> i) & 1u) ss = fmaf(x, x, ss);
        }
        part[2 * b] = ss;
        part[2 * b + 1] = dt;
      }
      block_sum<2 * B, T>(part, scratch, parity, tid);

      float z[B];
      float new_max = run_max;
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (s0 + b < S) {
          const float inv_rms = rsqrtf(part[2 * b] / rank_f + p.eps);
          z[b] = part[2 * b + 1] * inv_rms * p.scale;
          new_max = fmaxf(new_max, z[b]);
        } else {
          z[b] = -INFINITY;
        }
      }
      const float rescale = __expf(run_max - new_max);
      run_sum *= rescale;
#pragma unroll
      for (int i = 0; i < NE; ++i) acc[i] *= rescale;
#pragma unroll
      for (int b = 0; b < B; ++b) {
        if (s0 + b < S) {
          const float w = __expf(z[b] - new_max);
          run_sum += w;
#pragma unroll
          for (int i = 0; i < NE; ++i) acc[i] = fmaf(w, v[b][i], acc[i]);
          if (tid == 0) p.logits[(int64_t)(s0 + b) * p.N + row] = z[b];
        }
      }
      run_max = new_max;
    }

    if (tid == 0) {
      p.stats[row] = run_max;
      p.stats[p.N + row] = 1.0f / run_sum;
    }
    __nv_bfloat16* orow = p.out + row * p.out_row_stride;
    __nv_bfloat16* rrow = p.out_residual != nullptr ? p.out_residual + row * (int64_t)D : nullptr;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const int d = (j * T + tid) * VEC + e;
        if (d < D) {
          const float o = acc[j * VEC + e] / run_sum;
          const __nv_bfloat16 hi = __float2bfloat16_rn(o);
          orow[d] = hi;
          if (rrow != nullptr)
            reinterpret_cast<unsigned short*>(rrow)[d] = split_low16(o, __bfloat16_as_ushort(hi));
          if (LN) acc[j * VEC + e] = __bfloat162float(hi);  // kept for the LayerNorm below
        } else if (LN) {
          acc[j * VEC + e] = 0.f;
        }
      }
    }
    // Fused LayerNorm of the BF16 row just written (see FwdParams::ln_out).
    if constexpr (LN) {
      float total[1] = {0.f};
#pragma unroll
      for (int i = 0; i < NE; ++i) total[0] += acc[i];
      block_sum<1, T>(total, scratch, parity, tid);
      const float mean = total[0] / (float)D;
      total[0] = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const int d = (j * T + tid) * VEC + e;
          const float c = acc[j * VEC + e] - mean;
          if (d < D) total[0] = fmaf(c, c, total[0]);
        }
      }
      block_sum<1, T>(total, scratch, parity, tid);
      const float rstd = rsqrtf(total[0] / (float)D + p.ln_eps);
      if (tid == 0) {
        p.ln_stats[row] = mean;
        p.ln_stats[p.N + row] = rstd;
      }
      __nv_bfloat16* nrow = p.ln_out + row * (int64_t)D;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const int d = (j * T + tid) * VEC + e;
          if (d < D) {
            const float w = p.ln_weight != nullptr ? p.ln_weight[d] : 1.f;
            const float b = p.ln_bias != nullptr ? p.ln_bias[d] : 0.f;
            nrow[d] = __float2bfloat16_rn(fmaf((acc[j * VEC + e] - mean) * rstd, w, b));
          }
        }
      }
    }
  }
}

template <int VEC, int NJ, int T, int B>
__global__ void __launch_bounds__(T)
bwd_generic_kernel(const __grid_constant__ BwdParams p) {
  constexpr int NE = VEC * NJ;
  constexpr int NW = T / 32;
  __shared__ float scratch[2 * 2 * B * NW];
  __shared__ float s_dw[kMaxSources];   // sum_d v_s * dO
  __shared__ float s_ir[kMaxSources];   // inverse RMS of the tail key
  __shared__ float c_p[kMaxSources];    // softmax probability
  __shared__ float c_a[kMaxSources];    // inv_rms * scale * dlogit
  __shared__ float c_b[kMaxSources];    // inv_rms^2 * dlogit * logit / R
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int D = p.D, S = p.S, tail0 = p.D - p.R;
  const float rank_f = (float)p.R;

  float q[NE], dq[NE];
  uint32_t tailmask = 0;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const int d = (j * T + tid) * VEC + e;
      const bool in_tail = d < D && d >= tail0;
      q[j * VEC + e] = in_tail ? __bfloat162float(p.query[(int64_t)(d - tail0) * p.query_stride])
                               : 0.f;
      dq[j * VEC + e] = 0.f;
      if (in_tail) tailmask |= 1u << (j * VEC + e);
    }
  }

  int parity = 0;
  for (int64_t row = blockIdx.x; row < p.N; row += gridDim.x) {
    float g[NE];
    load_row<VEC, NJ, T>(g, p.grad_out + row * p.go_row_stride, p.go_feat_stride, D, tid);

    // Sweep 1: per-source dot with the upstream gradient and tail sum of squares.
    for (int s0 = 0; s0 < S; s0 += B) {
      float part[2 * B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const int s = s0 + b;
        float ss = 0.f, dw = 0.f;
        if (s < S) {
          float v[NE];
          load_row<VEC, NJ, T>(v, p.src.ptr[s] + row * p.src.row_stride[s],
                               p.src.feat_stride[s], D, tid);
#pragma unroll
          for (int i = 0; i < NE; ++i) {
            dw = fmaf(v[i], g[i], dw);
            if ((tailmask >> i) & 1u) ss = fmaf(v[i], v[i], ss);
          }
        }
        part[2 * b] = ss;
        part[2 * b + 1] = dw;
      }
      block_sum<2 * B, T>(part, scratch, parity, tid);
      if (tid == 0) {
#pragma unroll
        for (int b = 0; b < B; ++b) {
          if (s0 + b < S) {
            s_ir[s0 + b] = rsqrtf(part[2 * b] / rank_f + p.eps);
            s_dw[s0 + b] = part[2 * b + 1];
          }
        }
      }
    }
    __syncthreads();

    // delta = sum_s p_s * dw_s (equal to sum_d dO*O), then per-source coefficients.
    if (warp == 0) {
      const float row_max = p.stats[row];
      const float inv_sum = p.stats[p.N + row];
      constexpr int KS = (kMaxSources + 31) / 32;
      float prob[KS], zl[KS];
      float local = 0.f;
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int s = lane + 32 * k;
        prob[k] = 0.f;
        zl[k] = 0.f;
        if (s < S) {
          zl[k] = p.logits[(int64_t)s * p.N + row];
          prob[k] = __expf(zl[k] - row_max) * inv_sum;
          local = fmaf(prob[k], s_dw[s], local);
        }
      }
      const float delta = warp_sum(local);
#pragma unroll
      for (int k = 0; k < KS; ++k) {
        const int s = lane + 32 * k;
        if (s < S) {
          const float dz = prob[k] * (s_dw[s] - delta);
          const float ir = s_ir[s];
          c_p[s] = prob[k];
          c_a[s] = ir * p.scale * dz;
          c_b[s] = ir * ir * dz * zl[k] / rank_f;
        }
      }
    }
    __syncthreads();

    // Sweep 2: value gradients and the thread's share of the query gradient.
    for (int s = 0; s < S; ++s) {
      const float ps = c_p[s], ca = c_a[s], cb = c_b[s];
      float v[NE];
      if (tailmask != 0u) {
        load_row<VEC, NJ, T>(v, p.src.ptr[s] + row * p.src.row_stride[s],
                             p.src.feat_stride[s], D, tid);
      } else {
#pragma unroll
        for (int i = 0; i < NE; ++i) v[i] = 0.f;
      }
      float dv[NE];
#pragma unroll
      for (int i = 0; i < NE; ++i) {
        float x = ps * g[i];
        if ((tailmask >> i) & 1u) {
          x += fmaf(ca, q[i], -cb * v[i]);
          dq[i] = fmaf(ca, v[i], dq[i]);
        }
        dv[i] = x;
      }
      if (p.write_dv) {
        __nv_bfloat16* grow = p.grad.ptr[s] + row * p.grad.row_stride[s];
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int c = j * T + tid;
          if constexpr (VEC == 8) {
            if (c * 8 < D) {
              uint4* dst = reinterpret_cast<uint4*>(grow + (int64_t)c * 8);
              if (p.accumulate) {
                float old[8];
                unpack8(*dst, old);
#pragma unroll
                for (int e = 0; e < 8; ++e) dv[j * 8 + e] += old[e];
              }
              *dst = pack8(dv + j * 8);
            }
          } else {
            if (c < D) {
              const float old = p.accumulate ? __bfloat162float(grow[c]) : 0.f;
              grow[c] = __float2bfloat16_rn(dv[j] + old);
            }
          }
        }
      }
    }
  }

  if (p.dq_partials != nullptr) {
    float* prow = p.dq_partials + (int64_t)blockIdx.x * p.R;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const int d = (j * T + tid) * VEC + e;
        if (d < D && d >= tail0) prow[d - tail0] = dq[j * VEC + e];
      }
    }
  }
}

// Backward of the LayerNorm that the fused forward epilogue applies (FwdParams::ln_out), from
// what that forward saved: the BF16 row x (`out`) and (mean, rstd) per row.
//   xhat = (x - mean) * rstd,  gw = g * w,
//   dx   = rstd * (gw - mean_d(gw) - xhat * mean_d(gw * xhat))          -> BF16 [N,D]
//   dw  += g * xhat,  db += g                                            -> per-CTA FP32 partials
// One CTA walks rows; a thread owns the same NJ chunks of eight columns in every row, so its
// weights and its weight / bias gradient sums stay in registers for the whole launch.  The
// partial rows ([gridDim.x, 2 D]: weight gradient, then bias gradient) are summed by
// dq_reduce_kernel in a fixed order.  Needs D % 8 == 0 and 16-byte aligned rows.
struct LayerNormBwdParams {
  const __nv_bfloat16* grad;   // [N,D], row stride grad_row_stride, feature stride 1
  int64_t grad_row_stride;
  const __nv_bfloat16* x;      // [N,D] contiguous: the forward's BF16 output
  const float* stats;          // [2,N]: mean, rstd
  const float* weight;         // [D] or NULL (ones)
  __nv_bfloat16* dx;           // [N,D] contiguous
  float* partials;             // [gridDim.x, 2 D]
  int64_t N;
  int32_t D;
};

// Shared-memory ring of the LayerNorm backward: K stages of B rows.  A thread copies and reads
// back only its own 16-byte chunks (cp.async, no barrier needed for them); lane 0 of every warp
// copies the rows' (mean, rstd) for its warp.
template <int NJ, int T, int B, int K>
struct LayerNormBwdRing {
  static constexpr int kChunks = K * B * 2 * NJ * T;          // uint4 each
  static constexpr int kStats = K * B * 2 * (T / 32);         // float each
  static constexpr uint32_t kBytes = kChunks * 16u + kStats * 4u;
};

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Starts the copies of rows base .. base+B-1 into `stage` and closes the group (also when
// nothing was copied, so that every iteration adds exactly one group).  Rows at or beyond N
// become zeros with rstd = 0: they add nothing to any sum.
template <int NJ, int T, int B, int K>
__device__ __forceinline__ void layer_norm_bwd_issue(const LayerNormBwdParams& p, int64_t base,
                                                     int stage, int tid, uint4* chunks,
                                                     float* stats) {
  constexpr int NW = T / 32;
  const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const int64_t row = base + b;
    const bool valid = row < p.N;
    if (lane == 0) {
      float* dst = stats + ((stage * B + b) * 2) * NW + warp;
      if (valid) {
        cp_async_4(dst, p.stats + row);
        cp_async_4(dst + NW, p.stats + p.N + row);
      } else {
        dst[0] = 0.f;
        dst[NW] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int c = j * T + tid;
      uint4* dst = chunks + (((stage * B + b) * 2) * NJ + j) * T + tid;
      if (valid && c * 8 < p.D) {
        cp_async_16(dst, reinterpret_cast<const uint4*>(p.grad + row * p.grad_row_stride) + c);
        cp_async_16(dst + NJ * T, reinterpret_cast<const uint4*>(p.x + row * (int64_t)p.D) + c);
      } else {
        dst[0] = make_uint4(0u, 0u, 0u, 0u);
        dst[NJ * T] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// B rows per iteration share one CTA-wide reduction, and the rows of the next K-1 iterations
// are on their way into the ring while the current ones are reduced and stored: the kernel is
// bound by how many bytes an SM keeps in flight, not by arithmetic.
template <int NJ, int T, int B, int K>
__global__ void __launch_bounds__(T)
layer_norm_bwd_kernel(const __grid_constant__ LayerNormBwdParams p) {
  constexpr int NW = T / 32;
  using Ring = LayerNormBwdRing<NJ, T, B, K>;
  extern __shared__ __align__(16) unsigned char ring_bytes[];
  uint4* chunks = reinterpret_cast<uint4*>(ring_bytes);
  float* ring_stats = reinterpret_cast<float*>(ring_bytes + Ring::kChunks * 16);
  __shared__ float scratch[2 * 2 * B * NW];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = p.D;
  float w[NJ][8], dw[NJ][8], db[NJ][8];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int c = j * T + tid;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      w[j][e] = (c * 8 < D && p.weight != nullptr) ? p.weight[c * 8 + e] : 1.f;
      dw[j][e] = 0.f;
      db[j][e] = 0.f;
    }
  }
  const float inv_width = 1.0f / (float)D;
  const int64_t stride = (int64_t)gridDim.x * B;
  const int64_t first = (int64_t)blockIdx.x * B;
#pragma unroll
  for (int k = 0; k < K - 1; ++k)
    layer_norm_bwd_issue<NJ, T, B, K>(p, first + k * stride, k, tid, chunks, ring_stats);
  int parity = 0, stage = 0;
  for (int64_t base = first; base < p.N; base += stride) {
    // refills the stage that the previous iteration read (its reads came before that
    // iteration's CTA barrier)
    layer_norm_bwd_issue<NJ, T, B, K>(p, base + (K - 1) * stride, stage == 0 ? K - 1 : stage - 1,
                                      tid, chunks, ring_stats);
    asm volatile("cp.async.wait_group %0;" ::"n"(K - 1) : "memory");
    __syncwarp();
    uint4 gq[B][NJ], xq[B][NJ];
    float mean[B], rstd[B], sums[2 * B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      mean[b] = ring_stats[((stage * B + b) * 2) * NW + warp];
      rstd[b] = ring_stats[((stage * B + b) * 2 + 1) * NW + warp];
      sums[2 * b] = 0.f;
      sums[2 * b + 1] = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const uint4* src = chunks + (((stage * B + b) * 2) * NJ + j) * T + tid;
        gq[b][j] = src[0];
        xq[b][j] = src[NJ * T];
        float g[8], xhat[8];
        unpack8(gq[b][j], g);
        unpack8(xq[b][j], xhat);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xhat[e] = (xhat[e] - mean[b]) * rstd[b];
          const float gw = g[e] * w[j][e];
          sums[2 * b] += gw;
          sums[2 * b + 1] = fmaf(gw, xhat[e], sums[2 * b + 1]);
          dw[j][e] = fmaf(g[e], xhat[e], dw[j][e]);
          db[j][e] += g[e];
        }
      }
    }
    block_sum<2 * B, T>(sums, scratch, parity, tid);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (base + b < p.N) {
        const float mean_gw = sums[2 * b] * inv_width, mean_gwx = sums[2 * b + 1] * inv_width;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
          const int c = j * T + tid;
          if (c * 8 < D) {
            float g[8], xhat[8], dx[8];
            unpack8(gq[b][j], g);
            unpack8(xq[b][j], xhat);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              xhat[e] = (xhat[e] - mean[b]) * rstd[b];
              dx[e] = rstd[b] * (g[e] * w[j][e] - mean_gw - xhat[e] * mean_gwx);
            }
            *(reinterpret_cast<uint4*>(p.dx + (base + b) * (int64_t)D) + c) = pack8(dx);
          }
        }
      }
    }
    stage = stage + 1 == K ? 0 : stage + 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  float* prow = p.partials + (int64_t)blockIdx.x * (2 * D);
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int c = j * T + tid;
    if (c * 8 < D) {
      float4* wdst = reinterpret_cast<float4*>(prow + c * 8);
      float4* bdst = reinterpret_cast<float4*>(prow + D + c * 8);
      wdst[0] = make_float4(dw[j][0], dw[j][1], dw[j][2], dw[j][3]);
      wdst[1] = make_float4(dw[j][4], dw[j][5], dw[j][6], dw[j][7]);
      bdst[0] = make_float4(db[j][0], db[j][1], db[j][2], db[j][3]);
      bdst[1] = make_float4(db[j][4], db[j][5], db[j][6], db[j][7]);
    }
  }
}

// Second stage of the query gradient: column sums of the [rows, R] partials in a fixed
// order, so the result is bit-identical from call to call.  A CTA owns 16 columns (one
// 64-byte segment of every row); its 32 row groups each add every 32nd row, four rows at a
// time into four independent FP64 sums (so several loads are in flight per thread), and the
// groups are then added in index order.  Summing in FP64 means this stage adds no rounding
// of its own: the result is the FP32 rounding of the exact sum of the partials.  The
// reference reduces a [N, R] buffer with ceil(R/32) programs
// (src/attnres/_kernels/fixed_tail.py:875-899).
constexpr int kDqReduceColumns = 16;
constexpr int kDqReduceGroups = 32;

__global__ void __launch_bounds__(kDqReduceColumns * kDqReduceGroups)
dq_reduce_kernel(const float* __restrict__ partials, int rows, int R,
                 __nv_bfloat16* __restrict__ dq_bf16, float* __restrict__ dq_f32) {
  __shared__ double sm[kDqReduceGroups][kDqReduceColumns + 1];
  const int col = threadIdx.x % kDqReduceColumns, grp = threadIdx.x / kDqReduceColumns;
  const int r = blockIdx.x * kDqReduceColumns + col;
  double sum = 0.0;
  if (r < R) {
    const float* column = partials + r;
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    int row = grp;
    for (; row + 3 * kDqReduceGroups < rows; row += 4 * kDqReduceGroups) {
      const float a = column[(int64_t)row * R];
      const float b = column[(int64_t)(row + kDqReduceGroups) * R];
      const float c = column[(int64_t)(row + 2 * kDqReduceGroups) * R];
      const float d = column[(int64_t)(row + 3 * kDqReduceGroups) * R];
      s0 += (double)a;
      s1 += (double)b;
      s2 += (double)c;
      s3 += (double)d;
    }
    for (; row < rows; row += kDqReduceGroups) s0 += (double)column[(int64_t)row * R];
    sum = (s0 + s1) + (s2 + s3);
  }
  sm[grp][col] = sum;
  __syncthreads();
  if (grp == 0 && r < R) {
    double total = 0.0;
#pragma unroll
    for (int k = 0; k < kDqReduceGroups; ++k) total += sm[k][col];
    const float rounded = (float)total;
    if (dq_f32 != nullptr) dq_f32[r] = rounded;
    if (dq_bf16 != nullptr) dq_bf16[r] = __float2bfloat16_rn(rounded);
  }
}

}  // namespace attnres_b200
