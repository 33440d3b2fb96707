// Shared definitions for the sm_100a AttnRes read kernels: the by-value source
// tables, kernel parameter blocks and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace attnres_b200 {

constexpr int kMaxSources = 129;  // src/attnres/_sources.py:12
constexpr int kMaxWidth = 8192;   // src/attnres/_sources.py:13

// One record per source, passed BY VALUE inside the kernel parameter block
// (3 096 bytes).  The reference selects the source pointer with a chain of
// `tl.where` over a tuple of tensor arguments
// (src/attnres/_kernels/fla_full_sources.py:253-282); a parameter-space table
// needs no device allocation, no host-to-device copy and is frozen into a CUDA
// graph node at capture time.
struct SourceTable {
  const __nv_bfloat16* ptr[kMaxSources];
  int64_t row_stride[kMaxSources];   // elements
  int64_t feat_stride[kMaxSources];  // elements
};

// Per-source gradient outputs: rows of D contiguous BF16 values.
struct GradTable {
  __nv_bfloat16* ptr[kMaxSources];
  int64_t row_stride[kMaxSources];  // elements
};

struct FwdParams {
  SourceTable src;
  int32_t S;
  int32_t D;
  int32_t R;
  int64_t N;
  const __nv_bfloat16* query;
  int64_t query_stride;
  float eps;
  float scale;
  __nv_bfloat16* out;
  int64_t out_row_stride;
  // Optional 16-bit [N,D] (contiguous): the part of the FP32 result that the BF16 rounding of
  // `out` dropped (split_low16x2 below), so out + residual is the FP32 result.  NULL skips it.
  __nv_bfloat16* out_residual;
  float* logits;  // [S,N]
  float* stats;   // [2,N]: max, 1/denominator
  // Optional fused epilogue: LayerNorm over the D features of the BF16-rounded output row,
  // ln_out = (out - mean) * rstd * ln_weight + ln_bias, written as BF16 [N,D] (contiguous)
  // together with (mean, rstd) per row.  NULL `ln_out` disables it; NULL weight / bias mean
  // ones / zeros.
  const float* ln_weight;  // [D]
  const float* ln_bias;    // [D]
  float ln_eps;
  __nv_bfloat16* ln_out;
  float* ln_stats;  // [2,N]: mean, 1/sqrt(var + ln_eps)
};

struct BwdParams {
  SourceTable src;
  GradTable grad;
  int32_t S;
  int32_t D;
  int32_t R;
  int32_t write_dv;  // 0: skip the value-gradient stores
  int32_t accumulate;  // 1: add to the existing value-gradient rows instead of overwriting
  int64_t N;
  const __nv_bfloat16* query;
  int64_t query_stride;
  float eps;
  float scale;
  const __nv_bfloat16* grad_out;
  int64_t go_row_stride;
  int64_t go_feat_stride;
  const float* logits;
  const float* stats;
  // Optional: the forward's BF16 output and its 16-bit residual (both [N,D] contiguous),
  // together the forward's FP32 result.  With them delta = sum_d dO * result is known before
  // any source is read, which lets the streaming backward finish every source in one pass.
  const __nv_bfloat16* out_saved;
  const __nv_bfloat16* out_residual;
  float* dq_partials;  // [gridDim.x, R]
};

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// The two BF16 halves of a packed 32-bit word (element 0 is the low half).
__device__ __forceinline__ float bf16x2_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The saved output.  The forward rounds its FP32 result to BF16 (`out`) and, when asked, also
// keeps what the rounding dropped, as one unsigned 16-bit integer per element (offset binary):
//     low = float_bits(result) - (bf16_bits(out) << 16) + 0x8000          (in 0 .. 0x10000)
// Round-to-nearest moves the upper half of the FP32 pattern by at most one step, so the value
// fits 16 bits except for the tie that rounds DOWN to even (0x10000), which is stored as
// 0xffff (one FP32 ulp off, one element in 2^17).  The backward gets the FP32 result back by
// placing the two halves side by side and subtracting 0x8000, so `out` + `low` is a full FP32
// copy of the output in the space of two BF16 rows.  (The reference saves a separate FP32
// copy, src/attnres/_kernels/fixed_tail.py:917-919.)
//
// Packed form: `hi` holds two BF16 outputs, the returned word their two 16-bit remainders.
__device__ __forceinline__ uint32_t split_low16x2(float x0, float x1, uint32_t hi) {
  const uint32_t d0 = min(__float_as_uint(x0) - (hi << 16) + 0x8000u, 0xffffu);
  const uint32_t d1 = min(__float_as_uint(x1) - (hi & 0xffff0000u) + 0x8000u, 0xffffu);
  return __byte_perm(d0, d1, 0x5410);
}

__device__ __forceinline__ unsigned short split_low16(float x, unsigned short hi) {
  return (unsigned short)min(__float_as_uint(x) - ((uint32_t)hi << 16) + 0x8000u, 0xffffu);
}

// Inverse of split_low16x2: the two FP32 results from the packed BF16 pair and remainders.
__device__ __forceinline__ float2 join_low16x2(uint32_t hi, uint32_t low) {
  return make_float2(__uint_as_float(__byte_perm(low, hi, 0x5410) - 0x8000u),
                     __uint_as_float(__byte_perm(low, hi, 0x7632) - 0x8000u));
}

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  f[0] = bf16x2_lo(raw.x);
  f[1] = bf16x2_hi(raw.x);
  f[2] = bf16x2_lo(raw.y);
  f[3] = bf16x2_hi(raw.y);
  f[4] = bf16x2_lo(raw.z);
  f[5] = bf16x2_hi(raw.z);
  f[6] = bf16x2_lo(raw.w);
  f[7] = bf16x2_hi(raw.w);
}

__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 r;
  r.x = pack_bf16x2(f[0], f[1]);
  r.y = pack_bf16x2(f[2], f[3]);
  r.z = pack_bf16x2(f[4], f[5]);
  r.w = pack_bf16x2(f[6], f[7]);
  return r;
}

// The eight query values of tail chunk `chunk` (elements 8*chunk .. 8*chunk+7) as four FP32
// pairs: one 16-byte load when the query is contiguous and aligned, element loads otherwise.
__device__ __forceinline__ void load_query_chunk(const __nv_bfloat16* query, int64_t stride,
                                                 int chunk, float2* q) {
  if (stride == 1 && (reinterpret_cast<uintptr_t>(query) & 15u) == 0) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(query) + chunk);
    q[0] = make_float2(bf16x2_lo(raw.x), bf16x2_hi(raw.x));
    q[1] = make_float2(bf16x2_lo(raw.y), bf16x2_hi(raw.y));
    q[2] = make_float2(bf16x2_lo(raw.z), bf16x2_hi(raw.z));
    q[3] = make_float2(bf16x2_lo(raw.w), bf16x2_hi(raw.w));
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t r = (int64_t)chunk * 8 + 2 * k;
      q[k] = make_float2(__bfloat162float(query[r * stride]), __bfloat162float(query[(r + 1) * stride]));
    }
  }
}

// Butterfly sum: every lane ends with the same value, in an order that depends
// only on the lane layout (so results are reproducible run to run).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace attnres_b200
