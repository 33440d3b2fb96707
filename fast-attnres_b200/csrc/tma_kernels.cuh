#pragma once
#include "common.cuh"
namespace attnres_b200 {
inline bool tma_fwd_supported(int, int, int) { return false; }
inline bool tma_bwd_supported(int, int, int) { return false; }
inline int launch_fwd_tma(const FwdParams&, int, cudaStream_t) { return 9; }
inline int launch_bwd_tma(const BwdParams&, int, int, int*, cudaStream_t) { return 9; }
}
