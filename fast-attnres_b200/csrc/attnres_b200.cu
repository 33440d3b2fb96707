// C ABI of the sm_100a AttnRes read kernels (declared in include/attnres_b200.h):
// host-side argument checks, kernel-family selection and launches.
#include "../../include/attnres_b200.h"

#include <cmath>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "generic_kernels.cuh"
#include "fwd_ring_kernel.cuh"
#include "bwd_stash_kernel.cuh"
#include "bwd_ring_kernel.cuh"
#include "bwd_stream_kernel.cuh"

namespace attnres_b200 {
namespace {

int sm_count(int device, int* out) {
  // Queried per call: the attribute lookup is a cached driver read and keeps
  // the library free of mutable global state.
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      sms < 1) {
    cudaGetLastError();
    return ATTNRES_B200_ERR_CUDA;
  }
  *out = sms;
  return ATTNRES_B200_OK;
}

int current_device(int* device) {
  if (cudaGetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return ATTNRES_B200_ERR_CUDA;
  }
  return ATTNRES_B200_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool aligned2(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) == 0; }

int check_shape(int32_t S, int64_t N, int32_t D, int32_t R) {
  if (S < 1 || S > kMaxSources) return ATTNRES_B200_ERR_BAD_SOURCE_COUNT;
  if (D < 1 || D > kMaxWidth) return ATTNRES_B200_ERR_BAD_WIDTH;
  if (R < 1 || R > D) return ATTNRES_B200_ERR_BAD_RANK;
  if (N < 1) return ATTNRES_B200_ERR_BAD_ROWS;
  return ATTNRES_B200_OK;
}

int check_scalars(float eps, float scale) {
  if (!std::isfinite(eps) || eps <= 0.f || !std::isfinite(scale)) return ATTNRES_B200_ERR_BAD_SCALAR;
  return ATTNRES_B200_OK;
}

// Fills the by-value table and reports whether every source allows 16-byte
// accesses along the feature axis.
int fill_sources(SourceTable& t, const void* const* ptrs, const int64_t* rs, const int64_t* fs,
                 int S, int64_t N, bool* vec_ok) {
  bool ok = true;
  for (int s = 0; s < S; ++s) {
    if (ptrs[s] == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
    if (!aligned2(ptrs[s])) return ATTNRES_B200_ERR_MISALIGNED;
    t.ptr[s] = static_cast<const __nv_bfloat16*>(ptrs[s]);
    t.row_stride[s] = rs[s];
    t.feat_stride[s] = fs[s];
    ok = ok && aligned16(ptrs[s]) && fs[s] == 1 && (N == 1 || rs[s] % 8 == 0);
  }
  for (int s = S; s < kMaxSources; ++s) {
    t.ptr[s] = nullptr;
    t.row_stride[s] = 0;
    t.feat_stride[s] = 0;
  }
  *vec_ok = ok;
  return ATTNRES_B200_OK;
}

template <int VEC, int NJ, int T, int B>
int launch_fwd_generic(const FwdParams& p, int grid, cudaStream_t stream) {
  if (p.ln_out != nullptr) fwd_generic_kernel<VEC, NJ, T, B, true><<<grid, T, 0, stream>>>(p);
  else fwd_generic_kernel<VEC, NJ, T, B, false><<<grid, T, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? ATTNRES_B200_OK : ATTNRES_B200_ERR_CUDA;
}

template <int VEC, int NJ, int T, int B>
int launch_bwd_generic(const BwdParams& p, int grid, cudaStream_t stream) {
  bwd_generic_kernel<VEC, NJ, T, B><<<grid, T, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? ATTNRES_B200_OK : ATTNRES_B200_ERR_CUDA;
}

int dispatch_fwd_generic(const FwdParams& p, bool vec, int grid, cudaStream_t st) {
  const int D = p.D;
  if (vec) {
    if (D <= 1024) return launch_fwd_generic<8, 1, 128, 4>(p, grid, st);
    if (D <= 2048) return launch_fwd_generic<8, 1, 256, 4>(p, grid, st);
    if (D <= 4096) return launch_fwd_generic<8, 2, 256, 4>(p, grid, st);
    return launch_fwd_generic<8, 4, 256, 2>(p, grid, st);
  }
  if (D <= 256) return launch_fwd_generic<1, 1, 256, 4>(p, grid, st);
  if (D <= 512) return launch_fwd_generic<1, 2, 256, 4>(p, grid, st);
  if (D <= 1024) return launch_fwd_generic<1, 4, 256, 4>(p, grid, st);
  if (D <= 2048) return launch_fwd_generic<1, 8, 256, 4>(p, grid, st);
  if (D <= 4096) return launch_fwd_generic<1, 16, 256, 4>(p, grid, st);
  return launch_fwd_generic<1, 32, 256, 2>(p, grid, st);
}

int dispatch_bwd_generic(const BwdParams& p, bool vec, int grid, cudaStream_t st) {
  const int D = p.D;
  if (vec) {
    if (D <= 1024) return launch_bwd_generic<8, 1, 128, 4>(p, grid, st);
    if (D <= 2048) return launch_bwd_generic<8, 1, 256, 4>(p, grid, st);
    if (D <= 4096) return launch_bwd_generic<8, 2, 256, 4>(p, grid, st);
    return launch_bwd_generic<8, 4, 256, 2>(p, grid, st);
  }
  if (D <= 256) return launch_bwd_generic<1, 1, 256, 4>(p, grid, st);
  if (D <= 512) return launch_bwd_generic<1, 2, 256, 4>(p, grid, st);
  if (D <= 1024) return launch_bwd_generic<1, 4, 256, 4>(p, grid, st);
  if (D <= 2048) return launch_bwd_generic<1, 8, 256, 4>(p, grid, st);
  if (D <= 4096) return launch_bwd_generic<1, 16, 256, 4>(p, grid, st);
  return launch_bwd_generic<1, 32, 256, 2>(p, grid, st);
}

// Rows of the dquery workspace per SM: one per resident position stream.  Rows of up to 1024
// features are owned by one-warp groups, four to a CTA; twelve rows let the one-pass backward
// keep three CTAs per SM instead of two there (S = 49, D = 1024: 5.11 -> 5.55 TB/s; the staged
// and register-resident kernels run fewer streams and do not change).
inline int workspace_rows_per_sm(int D) { return D <= 1024 ? 12 : 8; }

// The one-pass backward moves 6*D more bytes per position (the forward writes one more 16-bit
// row, which costs it 1/(S+1) of its time; the backward reads two more) and finishes each
// source as it arrives.  Measured on B200 against the two-pass kernels, forward and backward
// together (N = 16384, R = D unless noted):
//   * it wins wherever the staged backward needs a cluster or does not fit (S >= 33 at
//     D = 4096, every long list at D = 8192), and for D <= 2048 wherever a position's staged
//     rows take more than half an SM's shared memory (S >= 33 at D = 2048, S >= 65 at
//     D = 1024): 1.4x to 5x on the backward;
//   * full-width rows with R = D: at D >= 4096 it wins from S = 5 up (backward 5.3 vs 3.9 TB/s
//     at S = 5, 6.3 vs 6.0 at S = 25); at D = 2048 it wins from S = 5 up as well (S = 13:
//     494 vs 524 us, S = 17: 619 vs 645 us, S = 25: 870 vs 887 us for forward + backward);
//   * D = 1024 (one-warp groups, three CTAs per SM): it wins where the staged backward keeps
//     three CTAs or fewer per SM (S = 33: 629 vs 662 us, S = 49: 885 vs 1055 us) and up to
//     twelve sources (S = 5: 137 vs 150 us, S = 9: 209 vs 219 us; S = 13 ties); S = 17 and 25
//     stay with the staged kernel by 2 %; narrower rows (D = 512) stay with it by 20 to 30 %;
//   * up to four sources: the register-resident kernel wins (S = 2, 3: 5.7 vs 4.3 TB/s) or
//     ties once the forward's extra row is counted (S = 4, D = 4096: 388 vs 386 us);
//   * low-rank tails at D = 4096 with a staged backward that fits one SM (S = 16, R = 1024:
//     5.45 vs 5.31 TB/s) and short low-rank lists: the two-pass kernels stay ahead by 3 to 6 %.
bool wants_output_residual(int S, int D, int R) {
  BwdStreamPlan stream;
  if (S <= 4 || !make_bwd_stream_plan(S, D, R, &stream)) return false;
  BwdPlan stash;
  if (!make_bwd_plan(S, D, R, &stash)) return true;
  if (stash.cluster > 1) return true;
  // One position's staged rows take more than half an SM's shared memory: the staged kernel
  // cannot overlap two positions on an SM.  (At D = 4096 it runs one wide CTA per SM by
  // design and holds up until it needs a cluster.)
  const bool one_position_per_sm = (size_t)(S + 1) * (size_t)D * 2u > 114u * 1024u;
  if (D <= 2048 && one_position_per_sm) return true;
  const bool full_row = D / 8 == stream.group_warps * 32 * kRingChunks;
  if (full_row && R == D && D >= 2048) return true;
  return D <= 1024 && (stash.ctas_per_sm <= 3 || (full_row && R == D && S <= 12));
}

// Everything about a backward call that can be judged without touching the device or the
// dquery workspace; shared by both backward entry points so they refuse the same calls with
// the same codes.
int check_backward_args(const void* const* src_ptrs, const int64_t* src_row_stride,
                        const int64_t* src_feat_stride, int32_t S, int64_t N, int32_t D, int32_t R,
                        const void* query, float eps, float scale, const void* grad_out,
                        const float* logits, const float* stats, void* const* dsrc_ptrs,
                        const int64_t* dsrc_row_stride, const void* dq_bf16, const float* dq_f32,
                        uint32_t flags) {
  if (int st = check_shape(S, N, D, R)) return st;
  if (int st = check_scalars(eps, scale)) return st;
  if (flags & ~(ATTNRES_B200_FLAG_FORCE_GENERIC | ATTNRES_B200_FLAG_PREFER_STREAM |
                ATTNRES_B200_FLAG_ACCUMULATE_DV))
    return ATTNRES_B200_ERR_BAD_FLAGS;
  if (!src_ptrs || !src_row_stride || !src_feat_stride || !query || !grad_out || !logits || !stats)
    return ATTNRES_B200_ERR_NULL_POINTER;
  const bool accumulate = (flags & ATTNRES_B200_FLAG_ACCUMULATE_DV) != 0;
  if (accumulate && dsrc_ptrs == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
  const bool want_dq = dq_bf16 != nullptr || dq_f32 != nullptr;
  const bool want_dv = dsrc_ptrs != nullptr;
  if (!want_dq && !want_dv) return ATTNRES_B200_ERR_NOTHING_TO_DO;
  if (want_dv && dsrc_row_stride == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
  if (!aligned2(query) || !aligned2(grad_out) || (dq_bf16 && !aligned2(dq_bf16)))
    return ATTNRES_B200_ERR_MISALIGNED;
  for (int s = 0; s < S; ++s) {
    if (src_ptrs[s] == nullptr || (want_dv && dsrc_ptrs[s] == nullptr))
      return ATTNRES_B200_ERR_NULL_POINTER;
    if (!aligned2(src_ptrs[s]) || (want_dv && !aligned2(dsrc_ptrs[s])))
      return ATTNRES_B200_ERR_MISALIGNED;
  }
  return ATTNRES_B200_OK;
}

// One CTA of one warp: lane 0 announces 32 bytes on a barrier, copies 16 and waits with the
// kernels' bounded wait.  Exercises the give-up path without a fault or a hang.
__global__ void selftest_wait_limit_kernel(const void* scratch16, uint64_t limit_ns) {
  __shared__ __align__(16) unsigned char landing[32];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(&bar, 32u);
    bulk_load(landing, scratch16, 16u, &bar);
    mbar_wait(&bar, 0u, &abort_flag, limit_ns);
    // The 16 bytes that were requested have landed long before the limit; hold the CTA a
    // little all the same, as the kernels do after a wait that ran out.
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 20000ull) {
    }
  }
}

}  // namespace
}  // namespace attnres_b200

using namespace attnres_b200;

extern "C" int attnres_b200_abi_version(void) { return ATTNRES_B200_ABI_VERSION; }

extern "C" const char* attnres_b200_status_string(int status) {
  switch (status) {
    case ATTNRES_B200_OK: return "ok";
    case ATTNRES_B200_ERR_NULL_POINTER: return "a required pointer is NULL";
    case ATTNRES_B200_ERR_BAD_SOURCE_COUNT: return "source count outside 1..129";
    case ATTNRES_B200_ERR_BAD_WIDTH: return "value width outside 1..8192";
    case ATTNRES_B200_ERR_BAD_RANK: return "query rank outside 1..D";
    case ATTNRES_B200_ERR_BAD_ROWS: return "row count must be positive";
    case ATTNRES_B200_ERR_BAD_SCALAR: return "eps must be finite and positive, scale finite";
    case ATTNRES_B200_ERR_MISALIGNED: return "a BF16 pointer is not 2-byte aligned";
    case ATTNRES_B200_ERR_WORKSPACE: return "dquery workspace has too few rows";
    case ATTNRES_B200_ERR_CUDA: return "a CUDA runtime call failed";
    case ATTNRES_B200_ERR_BAD_FLAGS: return "unknown flag bits";
    case ATTNRES_B200_ERR_NOTHING_TO_DO: return "backward needs a value or a query gradient output";
    case ATTNRES_B200_ERR_STATIC_SCRATCH:
      return "shape needs more dquery scratch than the built-in array holds; pass a workspace to "
             "attnres_b200_backward";
    default: return "unknown status";
  }
}

extern "C" const char* attnres_b200_kernel_family(int32_t S, int32_t D, int32_t R,
                                                  int32_t aligned, int32_t backward) {
  if (check_shape(S, 1, D, R) != ATTNRES_B200_OK) return "invalid";
  if (!aligned) return "generic";
  if (backward) {
    // The one-pass kernel counts where the library's own policy asks the forward to save
    // its output (long lists that no staged kernel takes, e.g. S = 129 at D = 8192).
    const bool fast = bwd_ring_supported(S, D, R) || tma_bwd_supported(S, D, R) ||
                      (bwd_stream_supported(S, D, R) && wants_output_residual(S, D, R));
    return fast ? "tma" : "generic";
  }
  return tma_fwd_supported(S, D, R) ? "tma" : "generic";
}

extern "C" int32_t attnres_b200_wants_output_residual(int32_t S, int32_t D, int32_t R) {
  if (check_shape(S, 1, D, R) != ATTNRES_B200_OK) return 0;
  return wants_output_residual(S, D, R) ? 1 : 0;
}

extern "C" int attnres_b200_error_flag(int32_t* flag, int32_t clear) {
  if (flag == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_error_flag, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return ATTNRES_B200_ERR_CUDA;
  }
  *flag = value;
  if (clear && value != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_error_flag, &zero, sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      return ATTNRES_B200_ERR_CUDA;
    }
  }
  return ATTNRES_B200_OK;
}

namespace {

// Optional LayerNorm epilogue of a forward call (all NULL / zero: none).
struct LayerNormArgs {
  const float* weight = nullptr;
  const float* bias = nullptr;
  float eps = 0.f;
  void* out = nullptr;
  float* stats = nullptr;
};

int forward_impl(
    const void* const* src_ptrs, const int64_t* src_row_stride, const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    void* out, int64_t out_row_stride, void* out_residual,
    float* logits, float* stats, const LayerNormArgs& ln,
    uint32_t flags, void* stream) {
  if (int st = check_shape(S, N, D, R)) return st;
  if (int st = check_scalars(eps, scale)) return st;
  if (flags & ~(ATTNRES_B200_FLAG_FORCE_GENERIC | ATTNRES_B200_FLAG_PREFER_STREAM))
    return ATTNRES_B200_ERR_BAD_FLAGS;
  if (!src_ptrs || !src_row_stride || !src_feat_stride || !query || !out || !logits || !stats)
    return ATTNRES_B200_ERR_NULL_POINTER;
  if (!aligned2(query) || !aligned2(out)) return ATTNRES_B200_ERR_MISALIGNED;

  FwdParams p;
  bool vec = false;
  if (int st = fill_sources(p.src, src_ptrs, src_row_stride, src_feat_stride, S, N, &vec)) return st;
  p.S = S;
  p.D = D;
  p.R = R;
  p.N = N;
  p.query = static_cast<const __nv_bfloat16*>(query);
  p.query_stride = query_stride;
  p.eps = eps;
  p.scale = scale;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.out_residual = static_cast<__nv_bfloat16*>(out_residual);
  p.logits = logits;
  p.stats = stats;
  p.ln_weight = ln.weight;
  p.ln_bias = ln.bias;
  p.ln_eps = ln.eps;
  p.ln_out = static_cast<__nv_bfloat16*>(ln.out);
  p.ln_stats = ln.stats;
  vec = vec && D % 8 == 0 && aligned16(out) && (N == 1 || out_row_stride % 8 == 0) &&
        (out_residual == nullptr || aligned16(out_residual)) &&
        (ln.out == nullptr || (aligned16(ln.out) && (ln.weight == nullptr || aligned16(ln.weight)) &&
                               (ln.bias == nullptr || aligned16(ln.bias))));

  int device = 0, sms = 0;
  if (int st = current_device(&device)) return st;
  if (int st = sm_count(device, &sms)) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  if (vec && !(flags & ATTNRES_B200_FLAG_FORCE_GENERIC) && tma_fwd_supported(S, D, R))
    return launch_fwd_tma(p, sms, cs);

  const int64_t cap = (int64_t)sms * 16;
  const int grid = (int)(N < cap ? N : cap);
  return dispatch_fwd_generic(p, vec, grid, cs);
}

}  // namespace

extern "C" int attnres_b200_forward(
    const void* const* src_ptrs, const int64_t* src_row_stride, const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    void* out, int64_t out_row_stride, void* out_residual,
    float* logits, float* stats,
    uint32_t flags, void* stream) {
  return forward_impl(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query, query_stride,
                      eps, scale, out, out_row_stride, out_residual, logits, stats,
                      LayerNormArgs{}, flags, stream);
}

extern "C" int attnres_b200_forward_layer_norm(
    const void* const* src_ptrs, const int64_t* src_row_stride, const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    void* out, int64_t out_row_stride, void* out_residual,
    float* logits, float* stats,
    const float* norm_weight, const float* norm_bias, float norm_eps,
    void* normed_out, float* norm_stats,
    uint32_t flags, void* stream) {
  if (normed_out == nullptr || norm_stats == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
  if (!aligned2(normed_out)) return ATTNRES_B200_ERR_MISALIGNED;
  if (!std::isfinite(norm_eps) || norm_eps < 0.f) return ATTNRES_B200_ERR_BAD_SCALAR;
  LayerNormArgs ln;
  ln.weight = norm_weight;
  ln.bias = norm_bias;
  ln.eps = norm_eps;
  ln.out = normed_out;
  ln.stats = norm_stats;
  return forward_impl(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query, query_stride,
                      eps, scale, out, out_row_stride, out_residual, logits, stats, ln, flags,
                      stream);
}

extern "C" int32_t attnres_b200_dq_workspace_rows(int64_t N, int32_t S, int32_t D, int32_t R,
                                                  int32_t device) {
  if (int st = check_shape(S, N, D, R)) return -st;
  int sms = 0;
  if (int st = sm_count(device, &sms)) return -st;
  const int64_t cap = (int64_t)sms * workspace_rows_per_sm(D);
  return (int32_t)(N < cap ? N : cap);
}

extern "C" int attnres_b200_backward(
    const void* const* src_ptrs, const int64_t* src_row_stride, const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    const void* grad_out, int64_t go_row_stride, int64_t go_feat_stride,
    const float* logits, const float* stats,
    const void* out_saved, const void* out_residual,
    void* const* dsrc_ptrs, const int64_t* dsrc_row_stride,
    float* dq_partials, int32_t dq_partial_rows,
    void* dq_bf16, float* dq_f32,
    uint32_t flags, void* stream) {
  if (int st = check_backward_args(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query, eps,
                                   scale, grad_out, logits, stats, dsrc_ptrs, dsrc_row_stride,
                                   dq_bf16, dq_f32, flags))
    return st;
  const bool accumulate = (flags & ATTNRES_B200_FLAG_ACCUMULATE_DV) != 0;
  const bool want_dq = dq_bf16 != nullptr || dq_f32 != nullptr;
  const bool want_dv = dsrc_ptrs != nullptr;
  if (want_dq && dq_partials == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;

  BwdParams p;
  bool vec = false;
  if (int st = fill_sources(p.src, src_ptrs, src_row_stride, src_feat_stride, S, N, &vec)) return st;
  for (int s = 0; s < kMaxSources; ++s) {
    p.grad.ptr[s] = nullptr;
    p.grad.row_stride[s] = 0;
  }
  if (want_dv) {
    for (int s = 0; s < S; ++s) {
      if (dsrc_ptrs[s] == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
      if (!aligned2(dsrc_ptrs[s])) return ATTNRES_B200_ERR_MISALIGNED;
      p.grad.ptr[s] = static_cast<__nv_bfloat16*>(dsrc_ptrs[s]);
      p.grad.row_stride[s] = dsrc_row_stride[s];
      vec = vec && aligned16(dsrc_ptrs[s]) && (N == 1 || dsrc_row_stride[s] % 8 == 0);
    }
  }
  p.S = S;
  p.D = D;
  p.R = R;
  p.write_dv = want_dv ? 1 : 0;
  p.accumulate = accumulate ? 1 : 0;
  p.N = N;
  p.query = static_cast<const __nv_bfloat16*>(query);
  p.query_stride = query_stride;
  p.eps = eps;
  p.scale = scale;
  p.grad_out = static_cast<const __nv_bfloat16*>(grad_out);
  p.go_row_stride = go_row_stride;
  p.go_feat_stride = go_feat_stride;
  p.logits = logits;
  p.stats = stats;
  p.out_saved = static_cast<const __nv_bfloat16*>(out_saved);
  p.out_residual = static_cast<const __nv_bfloat16*>(out_residual);
  p.dq_partials = want_dq ? dq_partials : nullptr;
  vec = vec && D % 8 == 0 && aligned16(grad_out) && go_feat_stride == 1 &&
        (N == 1 || go_row_stride % 8 == 0) && (!want_dq || aligned16(dq_partials));

  int device = 0, sms = 0;
  if (int st = current_device(&device)) return st;
  if (int st = sm_count(device, &sms)) return st;
  const int64_t cap = (int64_t)sms * workspace_rows_per_sm(D);
  const int max_rows = (int)(N < cap ? N : cap);
  if (want_dq && dq_partial_rows < max_rows) return ATTNRES_B200_ERR_WORKSPACE;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);

  int grid = max_rows;
  int st = ATTNRES_B200_ERR_CUDA;
  if (vec && !(flags & ATTNRES_B200_FLAG_FORCE_GENERIC)) {
    // Short source lists keep the whole position in registers; long ones stream through a
    // ring when the forward saved its output; the rest stage the position in shared memory.
    const bool have_saved = out_saved != nullptr && out_residual != nullptr &&
                            aligned16(out_saved) && aligned16(out_residual);
    if (have_saved && bwd_stream_supported(S, D, R) &&
        (accumulate || (flags & ATTNRES_B200_FLAG_PREFER_STREAM) || wants_output_residual(S, D, R)))
      st = launch_bwd_stream(p, sms, max_rows, &grid, cs);
    // Only the one-pass and the generic kernels accumulate.
    if (st != ATTNRES_B200_OK && !accumulate && bwd_ring_supported(S, D, R))
      st = launch_bwd_ring(p, sms, max_rows, &grid, cs);
    if (st != ATTNRES_B200_OK && !accumulate && tma_bwd_supported(S, D, R))
      st = launch_bwd_tma(p, sms, max_rows, &grid, cs);
  }
  if (st != ATTNRES_B200_OK) {
    // Not eligible, or the launch was refused (for example a cluster shape this device
    // cannot co-schedule): the layout-generic kernel takes any input.
    grid = max_rows;
    st = dispatch_bwd_generic(p, vec, grid, cs);
  }
  if (st != ATTNRES_B200_OK) return st;
  if (want_dq) {
    dq_reduce_kernel<<<(R + kDqReduceColumns - 1) / kDqReduceColumns,
                       kDqReduceColumns * kDqReduceGroups, 0, cs>>>(
        dq_partials, grid, R, static_cast<__nv_bfloat16*>(dq_bf16), dq_f32);
    if (cudaGetLastError() != cudaSuccess) return ATTNRES_B200_ERR_CUDA;
  }
  return ATTNRES_B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward without a caller workspace: the dquery partials go to a fixed device array.

namespace {

// The only device memory the library owns.  In host code this name is a host-side handle,
// not a device address; static_scratch_address() below asks the runtime for the address.
static __device__ __align__(256) float g_static_dq_scratch[ATTNRES_B200_STATIC_SCRATCH_FLOATS];

std::mutex g_static_scratch_mutex;
float* g_static_scratch_address[kMaxDevices] = {};

// Device address of the array on the CURRENT device, looked up once per device.
int static_scratch_address(int device, float** out) {
  if (device < 0 || device >= kMaxDevices) return ATTNRES_B200_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    float* address = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_dq_scratch) != cudaSuccess ||
        address == nullptr) {
      cudaGetLastError();
      return ATTNRES_B200_ERR_CUDA;
    }
    g_static_scratch_address[device] = address;
  }
  *out = g_static_scratch_address[device];
  return ATTNRES_B200_OK;
}

}  // namespace

extern "C" int attnres_b200_backward_static_scratch(
    const void* const* src_ptrs, const int64_t* src_row_stride, const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    const void* grad_out, int64_t go_row_stride, int64_t go_feat_stride,
    const float* logits, const float* stats,
    const void* out_saved, const void* out_residual,
    void* const* dsrc_ptrs, const int64_t* dsrc_row_stride,
    void* dq_bf16, float* dq_f32,
    uint32_t flags, void* stream) {
  if (int st = check_backward_args(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query, eps,
                                   scale, grad_out, logits, stats, dsrc_ptrs, dsrc_row_stride,
                                   dq_bf16, dq_f32, flags))
    return st;
  if (dq_bf16 == nullptr && dq_f32 == nullptr)  // value gradients only: no scratch involved
    return attnres_b200_backward(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query,
                                 query_stride, eps, scale, grad_out, go_row_stride, go_feat_stride,
                                 logits, stats, out_saved, out_residual, dsrc_ptrs, dsrc_row_stride,
                                 nullptr, 0, nullptr, nullptr, flags, stream);
  int device = 0;
  if (int st = current_device(&device)) return st;
  const int32_t rows = attnres_b200_dq_workspace_rows(N, S, D, R, device);
  if (rows < 0) return -rows;
  if ((int64_t)rows * R > (int64_t)ATTNRES_B200_STATIC_SCRATCH_FLOATS)
    return ATTNRES_B200_ERR_STATIC_SCRATCH;
  float* scratch = nullptr;
  if (int st = static_scratch_address(device, &scratch)) return st;
  // Every element of scratch[0 : grid*R] that the second stage sums is written by the first
  // stage of this same call, so stale contents from earlier calls are never read.
  return attnres_b200_backward(src_ptrs, src_row_stride, src_feat_stride, S, N, D, R, query,
                               query_stride, eps, scale, grad_out, go_row_stride, go_feat_stride,
                               logits, stats, out_saved, out_residual, dsrc_ptrs, dsrc_row_stride,
                               scratch, rows, dq_bf16,
                               dq_f32, flags, stream);
}

extern "C" int attnres_b200_selftest_wait_limit(const void* scratch16, uint64_t limit_ns,
                                                void* stream) {
  if (scratch16 == nullptr) return ATTNRES_B200_ERR_NULL_POINTER;
  if (!aligned16(scratch16)) return ATTNRES_B200_ERR_MISALIGNED;
  if (limit_ns < 1000ull || limit_ns > 100000000ull) return ATTNRES_B200_ERR_BAD_SCALAR;
  selftest_wait_limit_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(scratch16, limit_ns);
  return cudaGetLastError() == cudaSuccess ? ATTNRES_B200_OK : ATTNRES_B200_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// Backward of the fused LayerNorm epilogue.

namespace {
// Instance per width class, from timing the candidates on 16 384-row inputs: rows per
// iteration (B), ring stages (K), and the CTAs an SM holds (registers and ring bytes).
struct LayerNormBwdPlan {
  int rows_per_iteration;
  int ctas_per_sm;
};

inline LayerNormBwdPlan layer_norm_bwd_plan(int D) {
  if (D <= 1024) return {2, 6};   // <2, 64, 2, 4>
  if (D <= 2048) return {2, 3};   // <2, 128, 2, 2>
  if (D <= 4096) return {2, 2};   // <4, 128, 2, 2>
  return {1, 1};                  // <4, 256, 1, 3>
}

inline int layer_norm_bwd_grid(int64_t N, int D, int sms) {
  const LayerNormBwdPlan plan = layer_norm_bwd_plan(D);
  const int64_t iterations = (N + plan.rows_per_iteration - 1) / plan.rows_per_iteration;
  const int64_t cap = (int64_t)sms * plan.ctas_per_sm;
  return (int)(iterations < cap ? iterations : cap);
}

template <int NJ, int T, int B, int K>
int launch_layer_norm_bwd(const LayerNormBwdParams& p, int grid, cudaStream_t stream) {
  static SmemGrant grant;
  constexpr uint32_t smem = LayerNormBwdRing<NJ, T, B, K>::kBytes;
  if (int st = prepare_kernel(layer_norm_bwd_kernel<NJ, T, B, K>, smem, grant)) return st;
  layer_norm_bwd_kernel<NJ, T, B, K><<<grid, T, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? ATTNRES_B200_OK : ATTNRES_B200_ERR_CUDA;
}
}  // namespace

extern "C" int32_t attnres_b200_layer_norm_workspace_rows(int64_t N, int32_t D, int32_t device) {
  if (D < 1 || D > kMaxWidth) return -ATTNRES_B200_ERR_BAD_WIDTH;
  if (N < 1) return -ATTNRES_B200_ERR_BAD_ROWS;
  int sms = 0;
  if (int st = sm_count(device, &sms)) return -st;
  return layer_norm_bwd_grid(N, D, sms);
}

extern "C" int attnres_b200_layer_norm_backward(
    const void* grad_normed, int64_t grad_row_stride, const void* out, const float* norm_stats,
    const float* norm_weight, int64_t N, int32_t D,
    void* grad_out, float* partials, int32_t partial_rows, float* grad_weight_bias,
    void* stream) {
  if (D < 1 || D > kMaxWidth) return ATTNRES_B200_ERR_BAD_WIDTH;
  if (N < 1) return ATTNRES_B200_ERR_BAD_ROWS;
  if (!grad_normed || !out || !norm_stats || !grad_out || !partials || !grad_weight_bias)
    return ATTNRES_B200_ERR_NULL_POINTER;
  // 16-byte accesses along the rows; other layouts are the caller's to handle.
  if (D % 8 != 0 || !aligned16(grad_normed) || !aligned16(out) || !aligned16(grad_out) ||
      !aligned16(partials) || (N > 1 && grad_row_stride % 8 != 0))
    return ATTNRES_B200_ERR_MISALIGNED;
  int device = 0, sms = 0;
  if (int st = current_device(&device)) return st;
  if (int st = sm_count(device, &sms)) return st;
  const int grid = layer_norm_bwd_grid(N, D, sms);
  if (partial_rows < grid) return ATTNRES_B200_ERR_WORKSPACE;
  LayerNormBwdParams p;
  p.grad = static_cast<const __nv_bfloat16*>(grad_normed);
  p.grad_row_stride = grad_row_stride;
  p.x = static_cast<const __nv_bfloat16*>(out);
  p.stats = norm_stats;
  p.weight = norm_weight;
  p.dx = static_cast<__nv_bfloat16*>(grad_out);
  p.partials = partials;
  p.N = N;
  p.D = D;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  int st;
  if (D <= 1024) st = launch_layer_norm_bwd<2, 64, 2, 4>(p, grid, cs);
  else if (D <= 2048) st = launch_layer_norm_bwd<2, 128, 2, 2>(p, grid, cs);
  else if (D <= 4096) st = launch_layer_norm_bwd<4, 128, 2, 2>(p, grid, cs);
  else st = launch_layer_norm_bwd<4, 256, 1, 3>(p, grid, cs);
  if (st != ATTNRES_B200_OK) return st;
  const int columns = 2 * D;
  dq_reduce_kernel<<<(columns + kDqReduceColumns - 1) / kDqReduceColumns,
                     kDqReduceColumns * kDqReduceGroups, 0, cs>>>(partials, grid, columns, nullptr,
                                                                  grad_weight_bias);
  return cudaGetLastError() == cudaSuccess ? ATTNRES_B200_OK : ATTNRES_B200_ERR_CUDA;
}
