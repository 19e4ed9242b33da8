// Constants and helpers shared by the tcgen05 attention kernels (forward: kernels_att_tc.cu,
// backward: kernels_att_bwd_tc.cu).
#pragma once
#include "kernels.cuh"
#include "gemm.cuh"
#include "fast_types.cuh"
#include <cuda.h>

namespace ts2 {

static constexpr int TC_BM = 128;  // node rows per CTA
static constexpr int TC_BN = 64;   // keys per tile
static constexpr int TC_HD = 128;  // head width
static constexpr int Q_BYTES = TC_BM * TC_HD * 2;   // 32 KB: two 128-byte-wide atoms of 128 rows
static constexpr int KV_BYTES = TC_BN * TC_HD * 2;  // 16 KB: two atoms of 64 rows
static constexpr int P_BYTES = TC_BM * TC_BN * 2;   // 16 KB: one atom of 128 rows

// dK and dV together (kernels_att_bwd_kv_tc.cu); meta: the packed per-node records of att_pack_meta_kernel
int attention_backward_kv_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float4 *meta,
                             int Tpad, const int *rev_first, const int *rev_last, int T, int H, float slope, void *dk, void *dv,
                             bool out16);

__host__ __device__ inline float att_dot_scale_tc() { return sqrtf(1.0f / 128) * (0.5f / 0.693147f) * 1.0f; }


} // namespace ts2
