// Shared helpers: error handling, launch accounting, small PTX wrappers for
// sm_100a (mbarrier, TMA, tcgen05).  Everything here is internal to the library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>
#include <cstdio>
#include <string>
#include <atomic>
#include "../../include/ts2_b200.h"

namespace ts2 {

// ---- host side ---------------------------------------------------------------
extern thread_local std::string g_last_error;
extern std::atomic<long long> g_launch_count;

int fail(int code, const char *fmt, ...);

#define TS2_CUDA(expr)                                                                            \
    do {                                                                                          \
        cudaError_t _e = (expr);                                                                  \
        if (_e != cudaSuccess)                                                                    \
            return ts2::fail(TS2_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                             __FILE__, __LINE__);                                                 \
    } while (0)

#define TS2_CHECK_LAUNCH()                                                                  \
    do {                                                                                    \
        ts2::g_launch_count.fetch_add(1, std::memory_order_relaxed);                        \
        cudaError_t _e = cudaGetLastError();                                                \
        if (_e != cudaSuccess)                                                              \
            return ts2::fail(TS2_ERR_CUDA, "kernel launch failed: %s (%s:%d)",             \
                             cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

int sm_count(int device);
// blocks of `threads` threads (no dynamic shared memory) of this kernel that one SM holds at once (>= 1)
int resident_blocks(int device, const void *kernel, int threads);

// A word in device memory that kernels OR error bits into instead of trapping
// or spinning forever; read by the host after synchronizing.
int32_t *device_status_word(int device);
#define TS2_STATUS_WAIT_TIMEOUT 1
#define TS2_STATUS_BAD_ARG 2
// the word ts2_gemm_dw_noalloc's kernels use instead (a static __device__ variable: that entry point may not call
// cudaMalloc, which device_status_word() does on first use); null until that entry point has run on the device
int32_t *static_status_word_if_ready(int device);
// After the caller has synchronized: reads both status words of the device, clears the ones that were set and
// returns TS2_OK or TS2_ERR_DEVICE_STATUS (with the message set).  Allocates nothing.
int collect_device_status(int device);

// ---- device side -------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}

// Bounded wait: gives up after ~1.5e9 clocks or as soon as another thread of
// the CTA has raised *abort_flag; a give-up raises the flag itself.  No wait in
// this library spins without a limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag)
{
    if (mbar_try_wait(bar, parity))
        return true;
    long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((it & 63) == 63) {
            if (*abort_flag)
                return false;
            if (clock64() - t0 > 1500000000ll) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// 2-D tiled TMA load, no multicast: every CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, uint32_t bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}
// 2-D tiled TMA store shared -> global (rows / columns outside the tensor are clipped), bulk-group completion
__device__ __forceinline__ void tma_store_2d(const void *tmap, uint32_t src, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
// untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}
// untiled bulk copy shared -> global (bulk-group completion), same alignment rules
__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// tcgen05 ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row
// (lane base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns (e.g. 16 packed fp16 values per row)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor of tcgen05.mma (sm_100 format, 128-byte swizzle)
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
// D[tmem] (+)= A[smem] . B[smem], fp16 / bf16 operands, fp32 accumulate, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: the A operand (128 rows x 16 fp16, row = lane, two values per 32-bit column)
// is read from tensor memory, so a tile produced by the compute warps needs neither shared memory nor a proxy fence
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Four MMAs along K issued as one block by one thread: the descriptors advance by a_step / b_step (in 16-byte
// units) in their low word, which holds the start address (shared-memory addresses stay below 2^18, so the
// sum never carries out of the field).  The first MMA accumulates iff acc_first, the others always.
__device__ __forceinline__ void umma_f16_x4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc_first,
                                            uint32_t a_step, uint32_t b_step)
{
    asm volatile("{\n\t.reg .pred p, t;\n\t.reg .b32 alo, ahi, blo, bhi;\n\t.reg .b64 da, db;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\tsetp.eq.b32 t, %4, %4;\n\t"
                 "mov.b64 {alo, ahi}, %1;\n\tmov.b64 {blo, bhi}, %2;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
                 "add.u32 alo, alo, %5;\n\tadd.u32 blo, blo, %6;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t"
                 "add.u32 alo, alo, %5;\n\tadd.u32 blo, blo, %6;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t"
                 "add.u32 alo, alo, %5;\n\tadd.u32 blo, blo, %6;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, t;\n\t}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc_first), "r"(a_step), "r"(b_step)
                 : "memory");
}
// instruction descriptor for kind::f16: fp32 accumulator, fp16 operands, M = 128
__host__ __device__ constexpr uint32_t umma_idesc_f16(int n, bool a_mn, bool b_mn)
{
    return (1u << 4) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

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

// fp32 pair -> packed fp16 pair (lo in the low half), round to nearest even; a magnitude above 65504 saturates to
// +-65504 instead of becoming an infinity.  Every fp16 store of the library goes through this: one infinity in a
// gradient (the keys every later node attends to collect gradients of many thousand) turns into NaN at the next
// difference and then into a NaN loss.  Same single cvt instruction as the plain conversion.
__device__ __forceinline__ __half2 sat_half2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return *(__half2 *)&r;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

#endif // __CUDACC__
} // namespace ts2
