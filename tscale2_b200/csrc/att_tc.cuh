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

__host__ __device__ inline float att_dot_scale_tc() { return sqrtf(1.0f / 128) * (0.5f / 0.693147f) * 1.0f; }

#ifdef __CUDACC__
// barrier of the two warps that share TMEM lane quarter q (ids 2..5; compile-time ids keep the CTA at 6 barriers)
__device__ __forceinline__ void pair_barrier(int q)
{
    switch (q) {
    case 0: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 5, 64;" ::: "memory"); break;
    }
}
#endif

} // namespace ts2
