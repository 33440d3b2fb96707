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
//
// Two further axes of parallelism keep the kernel applicable and busy:
//
//   cluster   when (S+1) rows of D do not fit one SM's shared memory, a thread-block
//             cluster of C = 2, 4 or 8 CTAs shares the position: CTA r stages and
//             owns columns [r D/C, (r+1) D/C) of every row.  The per-source partial
//             sums of sweep 1 are written into every peer's shared memory
//             (st.shared::cluster) and announced with a remote mbarrier arrive; each
//             CTA then adds the C contributions in rank order, so all of them hold
//             bit-identical coefficients.  Value gradients and dquery lanes are
//             disjoint between the CTAs and need no exchange.
//   groups    when the staged rows leave room for few CTAs per SM and the row is
//             narrow, SG "source groups" of warps share a position in sweep 2
//             (group g takes sources g, g+SG, ...), each with its own dquery sums.
#pragma once

#include "tma_common.cuh"

namespace attnres_b200 {

constexpr int kStashSliceChunks = 4;  // chunks of the row a lane covers in sweep 1
constexpr int kStashMaxBuffers = 4;
constexpr int kStashMaxCluster = 2;  // larger clusters measured slower than the generic kernel
// Registers per thread of the compiled instances, for the occupancy estimate.
inline int stash_regs_per_thread(int threads) { return threads <= 160 ? 100 : threads <= 288 ? 112 : 96; }

struct BwdPlan {
  int cluster;        // C: CTAs sharing one position (1, 2, 4, 8)
  int slice_warps;    // W: warps that cover one CTA's columns in sweep 2
  int source_groups;  // SG
  int row_buffers;    // positions staged at once
  int parts;          // slices of the CTA's columns in sweep 1 (divides W*SG)
  int ctas_per_sm;
  uint32_t slot_bytes;        // one staged row slice
  uint32_t row_buffer_bytes;  // (S+1) slots
  uint32_t off_part;
  uint32_t off_coef;
  uint32_t off_zl;
  uint32_t off_xsum;
  uint32_t off_bars;
  uint32_t off_abort;
  uint32_t smem_bytes;
};

// 16-byte chunks owned by a consumer thread in sweep 2, for a slice of `width` columns.
inline int stash_chunks_per_thread(int width) { return width > 4096 ? 2 : 1; }

inline int stash_slice_warps(int width) {
  const int per_warp = 32 * stash_chunks_per_thread(width);
  return (width / 8 + per_warp - 1) / per_warp;
}

// Slices for sweep 1: a divisor of the warp count (so a warp always owns the same
// slice), at most kStashSliceChunks chunks per lane, cheapest by a small
// instruction-count model of (rounds of sources per warp) x (work per source).
inline int stash_parts(int S, int slice_chunks, int warps) {
  int best = 0;
  long best_cost = 0;
  for (int np = 1; np <= warps; ++np) {
    if (warps % np != 0) continue;
    const int iters = (slice_chunks + 32 * np - 1) / (32 * np);
    if (iters > kStashSliceChunks) continue;
    const long rounds = ((long)S * np + warps - 1) / warps;
    // 20 per chunk and 40 per source visited; a lighter per-source term (24) picked eight
    // parts with a half-empty third round for S = 5, 6 at D = 4096 and measured 4 to 7 % slower.
    const long cost = rounds * (iters * 20L + 40L);
    if (best == 0 || cost < best_cost) {
      best = np;
      best_cost = cost;
    }
  }
  return best;
}

inline bool make_bwd_plan(int S, int D, int R, BwdPlan* plan) {
  if (!tma_shape_ok(D, R)) return false;
  const int CH = D / 8;
  // The smallest cluster that fits wins: the exchange of partial sums between CTAs sits on
  // every position's critical path (measured: a 2-CTA cluster with two CTAs per SM is 20 %
  // slower than one CTA per SM without a cluster on S=25, D=4096).
  for (int C = 1; C <= kStashMaxCluster; C *= 2) {
    if (CH % C != 0) break;
    const int width = D / C;
    if (C > 1 && width < 512) break;
    BwdPlan p;
    p.cluster = C;
    p.slice_warps = stash_slice_warps(width);
    p.slot_bytes = (uint32_t)width * 2u;
    p.row_buffer_bytes = (uint32_t)(S + 1) * p.slot_bytes;
    const int W = p.slice_warps;
    const uint32_t coef_bytes = (uint32_t)S * 16u;
    const uint32_t zl_bytes = align_up((uint32_t)(S + 2) * 4u, 16);
    const uint32_t xsum_bytes = 0u;
    const uint32_t part_copies = C > 1 ? 2u * (uint32_t)C : 1u;
    const uint32_t bars_bytes = (uint32_t)kStashMaxBuffers * (uint32_t)(S + 1) * 2u * 8u + 16u;
    auto fixed_bytes = [&](int parts) {
      return align_up(part_copies * (uint32_t)S * (uint32_t)parts * 8u, 16) + coef_bytes + zl_bytes + xsum_bytes +
             bars_bytes + 16u + 64u;
    };
    // An SM offers 228 KB of shared memory; every resident CTA reserves 1 KB of it.
    auto per_cta_bytes = [](int ctas) {
      const uint32_t share = (228u * 1024u - (uint32_t)ctas * 1024u) / (uint32_t)ctas;
      return share < (uint32_t)kSmemPerCtaMax ? share : (uint32_t)kSmemPerCtaMax;
    };
    // CTAs per SM with one source group, limited by threads, registers and staged rows.
    // More, narrower CTAs beat fewer, wider ones: they overlap each other's phases.
    const int threads = 32 * (W + 1);
    int ctas = 2048 / threads;
    if (ctas > 65536 / (threads * stash_regs_per_thread(threads))) ctas = 65536 / (threads * stash_regs_per_thread(threads));
    if (ctas < 1) ctas = 1;
    if (ctas > 6) ctas = 6;
    if (C > 1 && ctas > 2) ctas = 2;
    int parts = stash_parts(S, CH / C, W);
    if (parts < 1) continue;
    int buffers = 0;
    while (ctas >= 1) {
      const uint32_t room = per_cta_bytes(ctas), fixed = fixed_bytes(parts);
      buffers = room > fixed ? (int)((room - fixed) / p.row_buffer_bytes) : 0;
      if (buffers >= 1) break;
      --ctas;
    }
    if (ctas < 1 || buffers < 1) continue;  // try a larger cluster
    if (buffers > kStashMaxBuffers) buffers = kStashMaxBuffers;
    // Narrow slices with few resident CTAs: let several warp groups share a position.
    int groups = 1;
    while (groups < 4 && groups * 2 <= S && ctas * W * groups * 2 <= 16 &&
           (long)ctas * 32 * (W * groups * 2 + 1) * stash_regs_per_thread(32 * (W * groups * 2 + 1)) <= 65536) {
      const int wider = stash_parts(S, CH / C, W * groups * 2);
      if (wider < 1 || fixed_bytes(wider) + (uint32_t)buffers * p.row_buffer_bytes > per_cta_bytes(ctas))
        break;
      groups *= 2;
      parts = wider;
    }
    p.source_groups = groups;
    p.parts = parts;
    p.row_buffers = buffers;
    p.ctas_per_sm = ctas;
    uint32_t off = (uint32_t)buffers * p.row_buffer_bytes;
    p.off_part = off;
    off += align_up(part_copies * (uint32_t)S * (uint32_t)p.parts * 8u, 16);
    p.off_coef = off;
    off += coef_bytes;
    p.off_zl = off;
    off += zl_bytes;
    p.off_xsum = off;
    off += xsum_bytes;
    p.off_bars = align_up(off, 8);
    off = p.off_bars + bars_bytes;
    p.off_abort = off;
    off += 16;
    p.smem_bytes = off;
    if (p.smem_bytes > (uint32_t)kSmemPerCtaMax) continue;
    *plan = p;
    return true;
  }
  return false;
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

// ---- thread-block cluster helpers (used only when the launch has cluster size > 1)

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Last statement of every thread of a clustered launch: no CTA retires (and hands its shared
// memory to another CTA) while a peer may still store into it or arrive on its barriers.
// Not `.aligned`: of the producer warp only lane 0 is still running when it gets here.
// Every wait before it is bounded, so every thread gets here.
__device__ __forceinline__ void cluster_exit_sync() {
  asm volatile("barrier.cluster.arrive.release;\n"
               "barrier.cluster.wait.acquire;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}

__device__ __forceinline__ void cluster_store_f1(uint32_t remote_addr, float a) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(a) : "memory");
}

__device__ __forceinline__ void cluster_arrive_remote(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait on a barrier that peers of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  if (*abort_flag) return false;
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
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

// CL is the cluster size (1 or 2) and GROUPS says whether source groups are in use; both are
// compile-time so the common single-CTA, single-group case carries none of that code.
// MAXT is the CTA size the instance is compiled for: narrow CTAs may use about 112 registers
// per thread, the 17-warp CTA of a 4096-wide slice is held to 96.
// FULL: R == D and the slice fills the warps exactly, so no chunk needs a predicate.
template <int NV, int CL, bool GROUPS, int MAXT, bool FULL>
__global__ void __launch_bounds__(MAXT, MAXT <= 160 ? 4 : MAXT <= 288 ? 2 : 1)
bwd_tma_kernel(const __grid_constant__ BwdParams p, const __grid_constant__ BwdPlan plan) {
  constexpr int GK = kStashSliceChunks;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int C = CL;
  const int W = plan.slice_warps;
  const int SG = GROUPS ? plan.source_groups : 1;
  const int WT = W * SG, T = WT * 32;
  const int S = p.S, D = p.D, R = p.R;
  const int c0 = (D - R) / 8;            // first tail chunk of the full row
  const int CHs = (D / 8) / C;           // chunks of this CTA's column slice
  const int crank = C > 1 ? (int)cluster_cta_rank() : 0;
  const int chunk_base = crank * CHs;    // global index of the slice's first chunk
  const int64_t position0 = blockIdx.x / C, position_step = gridDim.x / C;
  const int NRB = plan.row_buffers, NP = plan.parts, slots = S + 1;
  const uint32_t slot_bytes = plan.slot_bytes;
  float* part_sm = reinterpret_cast<float*>(smem + plan.off_part);    // [1 or 2][S][C][NP][2] (ss, dw)
  float4* coef_sm = reinterpret_cast<float4*>(smem + plan.off_coef);  // [S] (p, ca, cb, -)
  float* zl_sm = reinterpret_cast<float*>(smem + plan.off_zl);        // [S] logits, max, 1/sum
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + plan.off_bars);  // [NRB][slots]
  uint64_t* empty_bar = full_bar + kStashMaxBuffers * slots;
  uint64_t* xchg_bar = empty_bar + kStashMaxBuffers * slots;  // [2]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + plan.off_abort);

  if (tid == 0) {
    for (int b = 0; b < NRB; ++b) {
      for (int slot = 0; slot < slots; ++slot) {
        mbar_init(&full_bar[b * slots + slot], 1);
        // Slot 0 (upstream row) is read by every warp in sweep 2, source s by group s % SG.
        mbar_init(&empty_bar[b * slots + slot], slot == 0 ? WT : W);
      }
    }
    mbar_init(&xchg_bar[0], C * WT);
    mbar_init(&xchg_bar[1], C * WT);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (C > 1) cluster_sync_all();  // every CTA's barriers exist before anyone arrives remotely

  if (warp == WT) {
    // ---- producer: slot 0 of a row buffer holds the upstream slice, slot 1+s source s
    if (lane == 0) {
      uint32_t rb = 0, fill_parity = 1;  // parity of the release that precedes a refill
      bool first_pass = true, alive = true;
      const int64_t column = (int64_t)chunk_base * 8;
      for (int64_t row = position0; row < p.N && alive; row += position_step) {
        unsigned char* base = smem + (size_t)rb * plan.row_buffer_bytes;
        for (int slot = 0; slot < slots; ++slot) {
          uint64_t* fb = &full_bar[rb * slots + slot];
          if (!first_pass && !mbar_wait(&empty_bar[rb * slots + slot], fill_parity, abort_flag)) {
            alive = false;
            break;
          }
          const __nv_bfloat16* src =
              slot == 0 ? p.grad_out + row * p.go_row_stride
                        : p.src.ptr[slot - 1] + row * p.src.row_stride[slot - 1];
          mbar_expect_tx(fb, slot_bytes);
          bulk_load(base + (size_t)slot * slot_bytes, src + column, slot_bytes, fb);
        }
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
      // The warp's other lanes have exited (exited threads do not count at the barrier).
      if (C > 1) cluster_exit_sync();
    }
    return;
  }

  // ---- consumers
  // Sweep-2 ownership: group `sg` of warps, local chunk(s) wslice*32 + lane (+ W*32).
  const int sg = warp / W, wslice = warp - sg * W;
  int own_chunk[NV];   // local to the CTA's slice
  bool own_valid[NV], own_tail[NV];
  float2 q2[NV][4], dq2[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    own_chunk[j] = wslice * 32 + lane + j * W * 32;
    own_valid[j] = FULL ? true : own_chunk[j] < CHs;
    own_tail[j] = FULL ? true : (own_valid[j] && chunk_base + own_chunk[j] >= c0);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      q2[j][k] = make_float2(0.f, 0.f);
      dq2[j][k] = make_float2(0.f, 0.f);
    }
    if (own_tail[j]) load_query_chunk(p.query, p.query_stride, chunk_base + own_chunk[j] - c0, q2[j]);
  }
  // Sweep-1 ownership: slice `my_part` of the columns, sources my_first, my_first + step, ...
  const int my_part = warp % NP, my_first = warp / NP, my_step = WT / NP;
  const float inv_rank = 1.0f / (float)R;
  uint32_t rb = 0, parity = 0, xchg_count = 0;
  for (int64_t row = position0; row < p.N; row += position_step) {
    const unsigned char* base = smem + (size_t)rb * plan.row_buffer_bytes;
    uint64_t* full_row = &full_bar[rb * slots];
    uint64_t* empty_row = &empty_bar[rb * slots];

    // Saved logits and statistics of this position: warp 0 starts asynchronous 4-byte copies
    // into shared memory now (no registers held, nothing stalls) and reads them after sweep 1.
    if (warp == 0) {
      for (int s = lane; s < S + 2; s += 32) {
        const float* src = s < S ? p.logits + (int64_t)s * p.N + row
                                 : p.stats + (int64_t)(s - S) * p.N + row;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(&zl_sm[s])), "l"(src)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }

    // In a cluster the partial sums alternate between two buffers: a peer may already be
    // writing the next position's sums while this CTA still reads the current ones.
    float* part_row = part_sm + (C > 1 ? (xchg_count & 1u) * (uint32_t)(S * C * NP * 2) : 0u);

    // ---- sweep 1
    mbar_wait(&full_row[0], parity, abort_flag);
    const uint4* grow_sm = reinterpret_cast<const uint4*>(base);
    {
      float2 gs[GK][4];
#pragma unroll
      for (int k = 0; k < GK; ++k) {
        const int c = my_part * 32 + lane + 32 * NP * k;
        if (c < CHs) {
          unpack8_pairs(grow_sm[c], gs[k]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) gs[k][e] = make_float2(0.f, 0.f);
        }
      }
      for (int s = my_first; s < S; s += my_step) {
        mbar_wait(&full_row[1 + s], parity, abort_flag);
        const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * slot_bytes);
        float2 ss2 = make_float2(0.f, 0.f), dw2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < GK; ++k) {
          const int c = my_part * 32 + lane + 32 * NP * k;
          if (c < CHs) {
            float2 v[4];
            unpack8_pairs(vrow[c], v);
#pragma unroll
            for (int e = 0; e < 4; ++e) dw2 = __ffma2_rn(v[e], gs[k][e], dw2);
            if (FULL || chunk_base + c >= c0) {
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
        // Partial sums are laid out [S][C][NP][2]; in a cluster every CTA gets a copy of this
        // CTA's entry straight away, so the exchange overlaps the rest of sweep 1.
        if ((lane & 15) == 0) {
          float* dst = part_row + ((s * C + crank) * NP + my_part) * 2 + (lane >> 4);
          if (C > 1) {
            for (int t = 0; t < C; ++t) cluster_store_f1(cluster_map(smem_addr(dst), (uint32_t)t), keep);
          } else {
            *dst = keep;
          }
        }
      }
    }
    const uint32_t xbuf = xchg_count & 1u, xpar = (xchg_count >> 1) & 1u;
    if (C > 1) {
      // Every warp of every CTA of the cluster announces its partial sums on each CTA's
      // exchange barrier; only warp 0 waits for the full count.
      asm volatile("fence.acq_rel.cluster;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        for (int t = 0; t < C; ++t)
          cluster_arrive_remote(cluster_map(smem_addr(&xchg_bar[xbuf]), (uint32_t)t));
      }
      ++xchg_count;
    } else {
      consumer_sync(T);
    }

    // ---- delta and the per-source coefficients (warp 0; lane l takes sources l, l+32, ...)
    if (warp == 0) {
      asm volatile("cp.async.wait_all;" ::: "memory");
      __syncwarp();
      if (C > 1) mbar_wait_cluster(&xchg_bar[xbuf], xpar, abort_flag);
      const float row_max = zl_sm[S], inv_sum = zl_sm[S + 1];
      float local = 0.f;
      for (int s = lane; s < S; s += 32) {
        float ss = 0.f, dw = 0.f;
        for (int part = 0; part < C * NP; ++part) {  // rank-major: the same order in every CTA
          const float2 v = *reinterpret_cast<const float2*>(&part_row[(s * C * NP + part) * 2]);
          ss += v.x;
          dw += v.y;
        }
        const float z = zl_sm[s];
        const float prob = __expf(z - row_max) * inv_sum;
        coef_sm[s] = make_float4(prob, dw, rsqrtf(ss * inv_rank + p.eps), z);
        local = fmaf(prob, dw, local);
      }
      const float delta = warp_sum(local);
      for (int s = lane; s < S; s += 32) {
        const float4 t = coef_sm[s];  // (p, dw, inv_rms, z) written by this lane above
        const float dz = t.x * (t.y - delta);
        coef_sm[s] = make_float4(t.x, t.z * p.scale * dz, t.z * t.z * dz * t.w * inv_rank, 0.f);
      }
    }
    consumer_sync(T);

    // ---- sweep 2
    float2 g2[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_valid[j]) {
        unpack8_pairs(grow_sm[own_chunk[j]], g2[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) g2[j][e] = make_float2(0.f, 0.f);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_row[0]);
    for (int s = sg; s < S; s += SG) {
      const float4 cf = coef_sm[s];
      const float cp = cf.x, ca = cf.y, cb = cf.z;
      const float2 ps2 = make_float2(cp, cp), ca2 = make_float2(ca, ca), ncb2 = make_float2(-cb, -cb);
      const uint4* vrow = reinterpret_cast<const uint4*>(base + (size_t)(1 + s) * slot_bytes);
      __nv_bfloat16* out_row =
          p.write_dv ? p.grad.ptr[s] + row * p.grad.row_stride[s] + (int64_t)chunk_base * 8 : nullptr;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (own_valid[j]) {
          float2 dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] = __fmul2_rn(ps2, g2[j][e]);
          if (own_tail[j]) {
            // No wait here: in sweep 1 some warp of this CTA observed the completion of every
            // source's copy, and all warps have met at the named barrier since then.
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

  // One partial row per (position stream, source group); each CTA of a cluster writes its
  // own columns of the row.
  if (p.dq_partials != nullptr) {
    float* prow = p.dq_partials + ((int64_t)position0 * SG + sg) * R;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (own_tail[j]) {
        float4* dst = reinterpret_cast<float4*>(prow + (int64_t)(chunk_base + own_chunk[j] - c0) * 8);
        dst[0] = make_float4(dq2[j][0].x, dq2[j][0].y, dq2[j][1].x, dq2[j][1].y);
        dst[1] = make_float4(dq2[j][2].x, dq2[j][2].y, dq2[j][3].x, dq2[j][3].y);
      }
    }
  }
  if (C > 1) cluster_exit_sync();
}

template <int NV, int CL, bool GROUPS, int MAXT, bool FULL>
inline int launch_bwd_stash(const BwdParams& p, const BwdPlan& plan, int grid, int threads,
                            cudaStream_t stream) {
  static SmemGrant grant;
  if (int st = prepare_kernel(bwd_tma_kernel<NV, CL, GROUPS, MAXT, FULL>, plan.smem_bytes, grant))
    return st;
  if (plan.cluster == 1) {
    bwd_tma_kernel<NV, CL, GROUPS, MAXT, FULL><<<grid, threads, plan.smem_bytes, stream>>>(p, plan);
  } else {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)grid, 1, 1);
    config.blockDim = dim3((unsigned)threads, 1, 1);
    config.dynamicSmemBytes = plan.smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = (unsigned)plan.cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, bwd_tma_kernel<NV, CL, GROUPS, MAXT, FULL>, p, plan) != cudaSuccess) {
      cudaGetLastError();
      return 9;
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 9;
}

// `max_rows` bounds the dquery partial rows by the caller's workspace; the number of rows
// written is returned so the second-stage reduction sums exactly those.
inline int launch_bwd_tma(const BwdParams& p, int sms, int max_rows, int* rows_out,
                          cudaStream_t stream) {
  BwdPlan plan;
  if (!make_bwd_plan(p.S, p.D, p.R, &plan)) return 9;
  const int threads = 32 * (plan.slice_warps * plan.source_groups + 1);
  // Position streams: one per CTA (per cluster when C > 1).
  int64_t streams = (int64_t)sms * plan.ctas_per_sm / plan.cluster;
  if (streams > max_rows / plan.source_groups) streams = max_rows / plan.source_groups;
  if (streams > p.N) streams = p.N;
  if (streams < 1) return 9;
  const int grid = (int)streams * plan.cluster;
  const int nv = stash_chunks_per_thread(p.D / plan.cluster);
  const bool groups = plan.source_groups > 1;
  const int slice_chunks = (p.D / 8) / plan.cluster;
  const bool full = p.R == p.D && slice_chunks == 32 * plan.slice_warps * nv;
  int st;
#define ATTNRES_LAUNCH_STASH4(NVV, CLV, MAXT)                                                     \
  st = groups ? (full ? launch_bwd_stash<NVV, CLV, true, MAXT, true>(p, plan, grid, threads, stream)   \
                      : launch_bwd_stash<NVV, CLV, true, MAXT, false>(p, plan, grid, threads, stream)) \
              : (full ? launch_bwd_stash<NVV, CLV, false, MAXT, true>(p, plan, grid, threads, stream)  \
                      : launch_bwd_stash<NVV, CLV, false, MAXT, false>(p, plan, grid, threads, stream))
#define ATTNRES_LAUNCH_STASH(NVV, MAXT)                            \
  if (plan.cluster == 1) { ATTNRES_LAUNCH_STASH4(NVV, 1, MAXT); }   \
  else { ATTNRES_LAUNCH_STASH4(NVV, 2, MAXT); }
  if (nv == 1) {
    if (threads <= 160) { ATTNRES_LAUNCH_STASH(1, 160) }
    else if (threads <= 288) { ATTNRES_LAUNCH_STASH(1, 288) }
    else { ATTNRES_LAUNCH_STASH(1, 544) }
  } else {
    if (threads <= 160) { ATTNRES_LAUNCH_STASH(2, 160) }
    else if (threads <= 288) { ATTNRES_LAUNCH_STASH(2, 288) }
    else { ATTNRES_LAUNCH_STASH(2, 544) }
  }
#undef ATTNRES_LAUNCH_STASH4
#undef ATTNRES_LAUNCH_STASH
  *rows_out = (int)streams * plan.source_groups;
  return st;
}

}  // namespace attnres_b200
