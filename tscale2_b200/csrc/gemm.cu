// Persistent warp-specialised tcgen05 GEMM for sm_100a.
//
//   warp 0      : TMA producer — cp.async.bulk.tensor (no multicast) into a ring of
//                 128B-swizzled shared-memory stages, completion on mbarriers
//   warp 1      : allocates TMEM, issues tcgen05.mma (one elected thread), releases
//                 stages and publishes accumulators with tcgen05.commit
//   warps 2..9  : epilogue — tcgen05.ld the fp32/int32 accumulator (128 lanes x BN
//                 columns; two warps per lane quarter, half of the columns each) out of
//                 TMEM, apply scales, convert, stage 32-row blocks in shared memory and
//                 write them with TMA stores (direct stores for the accumulate form)
// Two TMEM accumulators (2 x BN columns) let the epilogue of one tile overlap the
// main loop of the next.  Work units are (tile, K-split); partial tiles of split
// units go to an fp32 workspace and are combined by reduce_splitk_kernel in a fixed
// order (deterministic, no atomics).
//
// It replaces the mma.sync kernels of the reference: Fp8MatMul
// (src/lib/cuda/cuda_fp8.cuh:123-228), Int8MatMulKernel* (src/lib/cuda/cuda_i8.cuh:157-320),
// Fp16MatMul (src/lib/cuda/cuda_fp16.cuh:49-164), and, because the dW operands are read
// token-major through MN-major shared-memory descriptors, also the per-step transposes
// (src/gpt/compute/matmul_fwdbwd.cuh:149-162,169-280).
#include "gemm.cuh"
#include "fast_types.cuh"
#include <cuda.h>
#include <vector>
#include <type_traits>
#include <mutex>

namespace ts2 {

static constexpr int BM = 128;
static constexpr int STAGE_ROW_BYTES = 128; // one swizzle row
static constexpr int NUM_THREADS = 320; // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)
static constexpr int NUM_THREADS_GATED = 576; // the gated-activation epilogue does more per element: 16 epilogue warps

struct GemmParams {
    int M, N;
    int m_tiles, n_tiles, splits;
    int n_fast;        // tile order: consecutive tiles walk N first (the CTAs of a wave share A rows) or M first (share B rows)
    int k_blocks;      // total K blocks (one block = one pipeline stage)
    int kb_per_split;
    uint32_t idesc;
    void *C;
    long long ldc;
    float alpha;
    const float *dyn_scale, *dyn_scale2, *row_scale, *col_scale, *c_in;
    int out_kind;
    float *workspace;
    int32_t *status;
    // dynamic unit scheduler: {next unit, finished CTAs}, both zero between launches (the last CTA to finish resets
    // them); null: unit i of CTA b is b + i * gridDim.x
    int *sched = nullptr;
    // grouped forms (mixture-of-experts): 0 none; 1 every 128-row M tile belongs to one group (tile_group[m_tile],
    // negative: skip) and reads B rows [group * group_rows_b + n]; 2 the K range of a unit is the row segment of
    // its group (group_kptr[g] .. group_kptr[g+1], multiples of the K block) and C moves by c_group_stride per group
    int group_mode, groups;
    const int *tile_group;
    int group_rows_b;
    const int *group_kptr;
    long long c_group_stride;
    int bk;
    int tma_store; // the epilogue stages 32-row blocks in shared memory and writes them with TMA (tmC)
    // gated-activation form (see Epilogue in gemm.cuh): a tile is 128 "wide" columns [nt * 128, +128) and the 128
    // "gate" columns pair_stride further on
    int pair_stride = 0;
    void *act_out = nullptr;
    long long act_ld = 0;
    float *act_scale = nullptr;
    float act_mult = 1.f;
    int act_kind = 0; // format of act_out: 0 e4m3, 1 fp16, 2 int8
};

struct Unit {
    int m0, n0, nt, kb0, kb1, b_row_off;
    long long c_off;
};

// Tile index -> tile coordinates.  The CTAs of a wave work on consecutive tiles, so the fast index decides which
// operand they share through L2: the host picks the order that streams the larger operand from HBM once and
// re-reads the smaller one (which stays in L2).
__device__ __forceinline__ void tile_coords(const GemmParams &p, int tile, int &mt, int &nt)
{
    if (p.n_fast) {
        nt = tile % p.n_tiles;
        mt = tile / p.n_tiles;
    } else {
        mt = tile % p.m_tiles;
        nt = tile / p.m_tiles;
    }
}

// identical in the three roles, so that they agree on which units exist
__device__ __forceinline__ bool decode_unit(const GemmParams &p, int u, int bn, Unit &t)
{
    const int tiles = p.m_tiles * p.n_tiles;
    t.b_row_off = 0;
    t.c_off = 0;
    if (p.group_mode == 2) {
        const int g = u / tiles, tile = u - g * tiles;
        t.m0 = (tile % p.m_tiles) * BM;
        t.n0 = (tile / p.m_tiles) * bn;
        t.kb0 = __ldg(p.group_kptr + g) / p.bk;
        t.kb1 = __ldg(p.group_kptr + g + 1) / p.bk;
        t.c_off = (long long)g * p.c_group_stride;
        return t.kb1 > t.kb0;
    }
    const int tile = u / p.splits, split = u - tile * p.splits;
    int mt, nt;
    tile_coords(p, tile, mt, nt);
    t.m0 = mt * BM;
    t.n0 = nt * (p.pair_stride ? bn / 2 : bn);
    t.nt = nt;
    t.kb0 = split * p.kb_per_split;
    t.kb1 = min(p.k_blocks, t.kb0 + p.kb_per_split);
    if (p.group_mode == 1) {
        const int g = __ldg(p.tile_group + mt);
        if (g < 0)
            return false;
        t.b_row_off = g * p.group_rows_b;
    }
    return true;
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= 1ull << 46; // descriptor version of sm_100
    d |= 2ull << 61; // 128-byte swizzle
    return d;
}

template <int MMA>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (MMA == 0) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                     : "memory");
    } else if constexpr (MMA == 1) {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                     : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                     "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                     : "memory");
    }
}

template <int BN>
struct SmemLayout {
    static constexpr int A_BYTES = BM * STAGE_ROW_BYTES;
    static constexpr int B_BYTES = BN * STAGE_ROW_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int STAGING_OFFSET = BAR_OFFSET + 1024;     // epilogue staging: 8 warps x 4 KB
    static constexpr int TOTAL = STAGING_OFFSET + 4 * 2 * 4096 + 1024; // + alignment slack
};

// ES: element size in bytes; MMA: 0 = f8f6f4, 1 = f16 (fp16/bf16), 2 = i8; MN: operand layout
// GATED: the gated-activation epilogue (Epilogue::pair_stride) is compiled in; a separate instantiation keeps its
// registers out of the plain kernels
template <int BN, int ES, int MMA, bool MN, bool GATED = false>
__global__ void __launch_bounds__(GATED ? NUM_THREADS_GATED : NUM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const GemmParams p)
{
    using L = SmemLayout<BN>;
    constexpr int STAGES = L::STAGES;
    constexpr int ELEMS_PER_ROW = STAGE_ROW_BYTES / ES; // elements in one 128-byte swizzle row
    constexpr int UMMA_K = 32 / ES;                     // elements per MMA along K
    constexpr int K_STEPS = 4;                          // MMAs per stage
    constexpr int BK = MN ? (UMMA_K * K_STEPS) : ELEMS_PER_ROW; // K elements per stage (equal in both layouts)
    constexpr uint32_t TMEM_COLS = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = (uint64_t *)(smem + L::BAR_OFFSET);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), tfull0 = smem_u32(bars + 2 * STAGES),
                   tempty0 = smem_u32(bars + 2 * STAGES + 2), drain = smem_u32(bars + 2 * STAGES + 4);
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 5);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    // Unit ring: the producer draws the CTA's next unit (from a global counter, so that a CTA that starts late or runs
    // beside another kernel simply takes fewer units) and hands its number to the MMA thread and the epilogue warps
    // through RING shared-memory slots: rfull (1 arrival: the producer), rempty (the MMA thread + every epilogue warp).
    constexpr int RING = 8;
    constexpr int EPI_WARPS = GATED ? 16 : 8;
    uint64_t *rbars = (uint64_t *)(smem + L::BAR_OFFSET + 256);
    const uint32_t rfull0 = smem_u32(rbars), rempty0 = smem_u32(rbars + RING);
    volatile int *unit_ring = (volatile int *)(rbars + 2 * RING);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < RING; ++s) {
            mbar_init(rfull0 + 8 * s, 1);
            mbar_init(rempty0 + 8 * s, 1 + EPI_WARPS);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, EPI_WARPS); // one arrival per epilogue warp
        }
        mbar_init(drain, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles = p.m_tiles * p.n_tiles;
    const int units = p.group_mode == 2 ? tiles * p.groups : tiles * p.splits;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int issued = 0;
            bool ok = true;
            int rslot = 0, seq = 0;
            uint32_t rphase = 0;
            // Two instances of the loop, so that the number drawn from the counter is not merged with the static one
            // right after the draw: the atomic takes about a microsecond to answer, and its result must not be touched
            // before the top of the next iteration, a whole unit's copies later.
            auto producer_loop = [&](auto dynamic_tag) {
            constexpr bool DYNAMIC = decltype(dynamic_tag)::value;
            auto draw = [&]() -> int {
                if constexpr (DYNAMIC) {
                    int v;
                    asm volatile("atom.global.add.s32 %0, [%1], 1;" : "=r"(v) : "l"(p.sched) : "memory");
                    return v;
                } else {
                    return (int)blockIdx.x + (seq++) * (int)gridDim.x;
                }
            };
            int next_u = draw();
            while (ok) {
                const int u = next_u;
                if (!mbar_wait(rempty0 + 8 * rslot, rphase ^ 1, abort_flag)) {
                    ok = false;
                    break;
                }
                unit_ring[rslot] = u < units ? u : -1;
                mbar_arrive(rfull0 + 8 * rslot); // release: the slot's number is visible to whoever sees the arrival
                if (++rslot == RING) {
                    rslot = 0;
                    rphase ^= 1;
                }
                if (u >= units)
                    break;
                next_u = draw(); // the counter's latency hides behind this unit's copies
                Unit un;
                if (!decode_unit(p, u, BN, un))
                    continue;
                const int m0 = un.m0, n0 = un.n0 + un.b_row_off, kb0 = un.kb0, kb1 = un.kb1;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_arrive_expect_tx(fb, L::STAGE_BYTES);
                    const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES), sb = sa + L::A_BYTES;
                    const int k0 = kb * BK;
                    if constexpr (!MN) {
                        tma_load_2d(sa, &tmA, fb, k0, m0);
                        if (GATED) { // two boxes of BN / 2 rows: wide rows, gate rows
                            tma_load_2d(sb, &tmB, fb, k0, n0);
                            tma_load_2d(sb + (BN / 2) * STAGE_ROW_BYTES, &tmB, fb, k0, p.pair_stride + n0);
                        } else {
                            tma_load_2d(sb, &tmB, fb, k0, n0);
                        }
                    } else {
                        // one box per 128-byte atom along M / N, each BK rows of the token-major operand
#pragma unroll
                        for (int j = 0; j < BM / ELEMS_PER_ROW; ++j)
                            tma_load_2d(sa + j * BK * STAGE_ROW_BYTES, &tmA, fb, m0 + j * ELEMS_PER_ROW, k0);
#pragma unroll
                        for (int j = 0; j < BN / ELEMS_PER_ROW; ++j)
                            tma_load_2d(sb + j * BK * STAGE_ROW_BYTES, &tmB, fb, n0 + j * ELEMS_PER_ROW, k0);
                    }
                    ++issued;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            };
            if (p.sched)
                producer_loop(std::true_type());
            else
                producer_loop(std::false_type());
            if (!ok) {
                // abort path: wait (bounded) for the copies still in flight before the CTA gives its
                // shared memory back.  The last min(issued, STAGES) stages may have pending copies.
                int s = stage;
                uint32_t ph = phase;
                for (int i = 0; i < min(issued, STAGES); ++i) {
                    if (--s < 0) {
                        s = STAGES - 1;
                        ph ^= 1;
                    }
                    long long t0 = clock64();
                    while (!mbar_try_wait(full0 + 8 * s, ph) && clock64() - t0 < 200000000ll) {
                    }
                }
            }
            // every CTA passes here exactly once, after its last draw: the last one leaves the counters at zero for the
            // next launch that uses them
            if (p.sched && atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
                p.sched[0] = 0;
                p.sched[1] = 0;
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            int rslot = 0;
            uint32_t rphase = 0;
            while (ok) {
                if (!mbar_wait(rfull0 + 8 * rslot, rphase, abort_flag))
                    break;
                const int u = unit_ring[rslot];
                mbar_arrive(rempty0 + 8 * rslot);
                if (++rslot == RING) {
                    rslot = 0;
                    rphase ^= 1;
                }
                if (u < 0)
                    break;
                Unit un;
                if (!decode_unit(p, u, BN, un))
                    continue;
                const int kb0 = un.kb0, kb1 = un.kb1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag))
                    break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES), sb = sa + L::A_BYTES;
                    uint64_t adesc, bdesc;
                    uint32_t step;
                    if constexpr (!MN) {
                        adesc = make_smem_desc(sa, 16, 1024);
                        bdesc = make_smem_desc(sb, 16, 1024);
                        step = (UMMA_K * ES) >> 4; // 32 bytes along the swizzle row
                    } else {
                        adesc = make_smem_desc(sa, BK * STAGE_ROW_BYTES, 1024);
                        bdesc = make_smem_desc(sb, BK * STAGE_ROW_BYTES, 1024);
                        step = (UMMA_K * STAGE_ROW_BYTES) >> 4; // UMMA_K token rows
                    }
#pragma unroll
                    for (int k = 0; k < K_STEPS; ++k)
                        umma<MMA>(tmem_d, adesc + (uint64_t)(k * step), bdesc + (uint64_t)(k * step), p.idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * stage);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok)
                    tc_commit(tfull0 + 8 * acc);
                acc ^= 1;
                if (acc == 0)
                    acc_phase ^= 1;
            }
            // every MMA issued so far has completed once this commit arrives
            tc_commit(drain);
            long long t0 = clock64();
            while (!mbar_try_wait(drain, 0) && clock64() - t0 < 1500000000ll) {
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quarter = warp & 3; // TMEM lanes this warp may read: [32*quarter, +32)
        float alpha = p.alpha;
        if (p.dyn_scale)
            alpha *= __ldg(p.dyn_scale);
        if (p.dyn_scale2)
            alpha *= __ldg(p.dyn_scale2);
        int acc = 0;
        uint32_t acc_phase = 0;
        // the two warps of a quarter split the tile's columns: warps 2-5 take the first half, 6-9 the second
        const int half = (warp - 2) >> 2;
        constexpr int CHUNKS = BN / 32;
        const int c_begin = half * (CHUNKS / 2), c_end = c_begin + CHUNKS / 2;
        uint8_t *const stg_warp = smem + L::STAGING_OFFSET + (warp - 2) * 4096;
        const bool out16 = p.out_kind == TS2_OUT_F16 || p.out_kind == TS2_OUT_BF16;
        int rslot = 0;
        uint32_t rphase = 0;
        for (;;) {
            if (!__all_sync(0xffffffffu, mbar_wait(rfull0 + 8 * rslot, rphase, abort_flag)))
                break;
            const int u = unit_ring[rslot];
            __syncwarp(); // every lane has read the slot before the warp gives it back
            if (lane == 0)
                mbar_arrive(rempty0 + 8 * rslot);
            if (++rslot == RING) {
                rslot = 0;
                rphase ^= 1;
            }
            if (u < 0)
                break;
            Unit un;
            if (!decode_unit(p, u, BN, un))
                continue;
            const int m0 = un.m0, n0 = un.n0;
            uint8_t *const Cg = (uint8_t *)p.C + un.c_off * ((p.out_kind == TS2_OUT_F32 || p.out_kind == TS2_OUT_F32_ADD) ? 4 : 2);
            const float *const Cin = p.c_in + un.c_off;
            if (p.out_kind == TS2_OUT_F32_ADD && p.splits == 1) {
                // the residual input of this tile is known long before its accumulator is: pull this thread's 128-byte
                // pieces into L2 while the main loop runs, so that the loads below do not pay the HBM latency per chunk
                const long long prow = m0 + quarter * 32 + lane;
                if (prow < p.M) {
                    for (int c = c_begin; c < c_end; ++c)
                        if (n0 + c * 32 < p.N)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(Cin + prow * p.ldc + n0 + c * 32));
                }
            }
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag))
                break;
            tc_fence_after();
            const int row_in_tile = quarter * 32 + lane;
            const long long row = m0 + row_in_tile;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            float rs = 1.f;
            if (p.splits == 1 && p.row_scale && row < p.M)
                rs = __ldg(p.row_scale + row);
            rs *= alpha;
            if constexpr (GATED) {
                // Gated-activation form.  TMEM columns [0, 128) hold the wide tile, [128, 256) the gate tile.  Sixteen
                // epilogue warps, four per lane quarter: warp part j takes wide columns [32 j, +32) and the gate columns
                // under them, and reads the other 96 wide columns once more for the sum of squares of the whole
                // 128-wide tile (cheaper than an exchange between warps, and no barrier a failed wait could break).
                const int part = (warp - 2) >> 2;
                const int wcol = n0 + part * 32, gcol = p.pair_stride + wcol; // first wide / gate column of this warp
                uint8_t *const blk = smem + L::STAGING_OFFSET + (warp - 2) * 2048;
                auto scaled32 = [&](int chunk, int col, float *v) { // 32 accumulator columns -> scaled values
                    uint32_t r[32];
                    tmem_ld32(taddr + chunk * 32, r);
                    tmem_ld_wait();
                    auto acc = [&](int i) { return (MMA == 2) ? (float)(int)r[i] : __uint_as_float(r[i]); };
                    if (p.col_scale) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 cs = __ldg((const float4 *)(p.col_scale + col) + i);
                            v[4 * i] = acc(4 * i) * rs * cs.x, v[4 * i + 1] = acc(4 * i + 1) * rs * cs.y;
                            v[4 * i + 2] = acc(4 * i + 2) * rs * cs.z, v[4 * i + 3] = acc(4 * i + 3) * rs * cs.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            v[i] = acc(i) * rs;
                    }
                };
                // 32 fp16 columns -> the warp's staging block -> TMA store (rows >= M, columns >= N clipped)
                auto stage_store16 = [&](const float *v, int col) {
                    uint8_t *srow = blk + lane * 64;
                    const int sw = (lane >> 1) & 3;
                    if (lane == 0)
                        bulk_wait_read<0>(); // the previous store has read the block
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 h0 = sat_half2(v[8 * i], v[8 * i + 1]), h1 = sat_half2(v[8 * i + 2], v[8 * i + 3]),
                                h2 = sat_half2(v[8 * i + 4], v[8 * i + 5]), h3 = sat_half2(v[8 * i + 6], v[8 * i + 7]);
                        *(uint4 *)(srow + ((i ^ sw) << 4)) = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (col < p.N)
                            tma_store_2d(&tmC, smem_u32(blk), col, m0 + quarter * 32);
                        bulk_commit();
                    }
                };
                float wv[32], sum2 = 0.f;
                scaled32(part, wcol, wv);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    sum2 = fmaf(wv[i], wv[i], sum2);
#pragma unroll 1
                for (int oc = 1; oc < 4; ++oc) {
                    const int ch = (part + oc) & 3;
                    float ov[32];
                    scaled32(ch, n0 + ch * 32, ov);
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        s4[i & 3] = fmaf(ov[i], ov[i], s4[i & 3]);
                    sum2 += (s4[0] + s4[1]) + (s4[2] + s4[3]);
                }
                const float tscale = tile_scale(sum2);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    wv[i] *= tscale;
                if (part == 0 && row < p.M)
                    p.act_scale[row * p.n_tiles + un.nt] = tscale;
                stage_store16(wv, wcol);
                float gv[32];
                scaled32(4 + part, gcol, gv);
                stage_store16(gv, gcol);
                if (row < p.M) {
                    const size_t aidx = (size_t)row * p.act_ld + wcol;
                    if (p.act_kind == 2) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            Fast<2>::store4(p.act_out, aidx + 4 * i,
                                            make_float4(lolu_mult(gv[4 * i]) * wv[4 * i] * p.act_mult, lolu_mult(gv[4 * i + 1]) * wv[4 * i + 1] * p.act_mult,
                                                        lolu_mult(gv[4 * i + 2]) * wv[4 * i + 2] * p.act_mult,
                                                        lolu_mult(gv[4 * i + 3]) * wv[4 * i + 3] * p.act_mult));
                    } else if (p.act_kind == 1) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            Fast<1>::store4(p.act_out, aidx + 4 * i,
                                            make_float4(lolu_mult(gv[4 * i]) * wv[4 * i] * p.act_mult, lolu_mult(gv[4 * i + 1]) * wv[4 * i + 1] * p.act_mult,
                                                        lolu_mult(gv[4 * i + 2]) * wv[4 * i + 2] * p.act_mult,
                                                        lolu_mult(gv[4 * i + 3]) * wv[4 * i + 3] * p.act_mult));
                    } else {
                        // sigmoid(2 g) = 0.5 + 0.5 tanh(g): one MUFU op; its 2^-11 error is far below the e4m3 step
                        const float hm = 0.5f * p.act_mult;
                        auto gated = [&](int e) {
                            float th;
                            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(gv[e]));
                            return fmaf(th, hm, hm) * wv[e];
                        };
#pragma unroll
                        for (int j = 0; j < 2; ++j) { // 16 e4m3 bytes per store
                            uint32_t w4[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int e = 16 * j + 4 * i;
                                __nv_fp8x4_e4m3 pk(make_float4(gated(e), gated(e + 1), gated(e + 2), gated(e + 3)));
                                w4[i] = pk.__x;
                            }
                            *(uint4 *)((uint8_t *)p.act_out + aidx + 16 * j) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(tempty0 + 8 * acc);
                acc ^= 1;
                if (acc == 0)
                    acc_phase ^= 1;
                continue;
            }
#pragma unroll 1
            for (int c = c_begin; c < c_end; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                tmem_ld_wait();
                const int col = n0 + c * 32;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    v[i] = (MMA == 2) ? (float)(int)r[i] : __uint_as_float(r[i]);
                if (p.splits > 1) {
                    float4 *dst = (float4 *)(p.workspace + ((size_t)u * BM + row_in_tile) * BN + c * 32);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    continue;
                }
                if (p.tma_store) {
                    // coalesced path: the warp's 32 rows x 128 bytes go through a swizzled staging block and one TMA
                    // store; 16-bit outputs fill a block with two 32-column chunks.  Rows >= M and columns >= N are
                    // clipped by the TMA unit.
                    if (col < p.N) {
                        if (p.col_scale) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float4 cs = __ldg((const float4 *)(p.col_scale + col) + i);
                                v[4 * i] *= cs.x * rs;
                                v[4 * i + 1] *= cs.y * rs;
                                v[4 * i + 2] *= cs.z * rs;
                                v[4 * i + 3] *= cs.w * rs;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                v[i] *= rs;
                        }
                        if (p.out_kind == TS2_OUT_F32_ADD && row < p.M) {
                            // accumulate form: the residual input comes by plain loads (this thread's 128-byte piece of
                            // its row, prefetched into L2 above); the sum leaves through the staging blocks like a plain
                            // output, so that HBM sees whole lines instead of 16-byte pieces of 32 rows per store
                            const float4 *src = (const float4 *)(Cin + row * p.ldc + col);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float4 o = src[i];
                                v[4 * i] += o.x, v[4 * i + 1] += o.y, v[4 * i + 2] += o.z, v[4 * i + 3] += o.w;
                            }
                        }
                    }
                    // Two 2 KB blocks per warp (32 rows x 64 bytes, 64-byte swizzle: 16-byte chunk j of row r sits at
                    // j ^ ((r >> 1) & 3)), used in turn: before a block is refilled, all bulk groups but the most recent
                    // one must have read their source, i.e. the store that last used this block.  A group is committed
                    // for every fill, also when the store itself is clipped away, so that this count stays right.
                    const int sw = (lane >> 1) & 3;
                    if (out16) {
                        uint8_t *blk = stg_warp + (c & 1) * 2048, *srow = blk + lane * 64;
                        if (lane == 0)
                            bulk_wait_read<1>();
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 pk;
                            if (p.out_kind == TS2_OUT_F16) {
                                __half2 h0 = sat_half2(v[8 * i], v[8 * i + 1]), h1 = sat_half2(v[8 * i + 2], v[8 * i + 3]),
                                        h2 = sat_half2(v[8 * i + 4], v[8 * i + 5]), h3 = sat_half2(v[8 * i + 6], v[8 * i + 7]);
                                pk = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                            } else {
                                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]),
                                               h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]),
                                               h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]),
                                               h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                                pk = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                            }
                            *(uint4 *)(srow + ((i ^ sw) << 4)) = pk;
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            if (col < p.N)
                                tma_store_2d(&tmC, smem_u32(blk), col, m0 + quarter * 32);
                            bulk_commit();
                        }
                    } else {
#pragma unroll
                        for (int hb = 0; hb < 2; ++hb) { // 16 fp32 columns per block
                            uint8_t *blk = stg_warp + hb * 2048, *srow = blk + lane * 64;
                            if (lane == 0)
                                bulk_wait_read<1>();
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                *(float4 *)(srow + ((i ^ sw) << 4)) =
                                    make_float4(v[16 * hb + 4 * i], v[16 * hb + 4 * i + 1], v[16 * hb + 4 * i + 2], v[16 * hb + 4 * i + 3]);
                            fence_proxy_async();
                            __syncwarp();
                            if (lane == 0) {
                                if (col + 16 * hb < p.N)
                                    tma_store_2d(&tmC, smem_u32(blk), col + 16 * hb, m0 + quarter * 32);
                                bulk_commit();
                            }
                        }
                    }
                    continue;
                }
                if (row >= p.M || col >= p.N)
                    continue;
                if (p.col_scale) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 cs = __ldg((const float4 *)(p.col_scale + col) + i);
                        v[4 * i] *= cs.x * rs;
                        v[4 * i + 1] *= cs.y * rs;
                        v[4 * i + 2] *= cs.z * rs;
                        v[4 * i + 3] *= cs.w * rs;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        v[i] *= rs;
                }
                if (p.out_kind == TS2_OUT_F32 || p.out_kind == TS2_OUT_F32_ADD) {
                    float4 *dst = (float4 *)((float *)Cg + row * p.ldc + col);
                    if (p.out_kind == TS2_OUT_F32_ADD) {
                        const float4 *src = (const float4 *)(Cin + row * p.ldc + col);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float4 o = src[i];
                            dst[i] = make_float4(o.x + v[4 * i], o.y + v[4 * i + 1], o.z + v[4 * i + 2], o.w + v[4 * i + 3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                } else if (p.out_kind == TS2_OUT_F16) {
                    uint4 *dst = (uint4 *)((__half *)Cg + row * p.ldc + col);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 h0 = sat_half2(v[8 * i], v[8 * i + 1]), h1 = sat_half2(v[8 * i + 2], v[8 * i + 3]),
                                h2 = sat_half2(v[8 * i + 4], v[8 * i + 5]), h3 = sat_half2(v[8 * i + 6], v[8 * i + 7]);
                        dst[i] = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                    }
                } else {
                    uint4 *dst = (uint4 *)((__nv_bfloat16 *)Cg + row * p.ldc + col);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]),
                                       h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]),
                                       h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]),
                                       h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                        dst[i] = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(tempty0 + 8 * acc);
            acc ^= 1;
            if (acc == 0)
                acc_phase ^= 1;
        }
        if (p.tma_store && lane == 0)
            bulk_wait_read<0>(); // the staging blocks must outlive the stores that read them
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && *abort_flag)
        atomicOr(p.status, TS2_STATUS_WAIT_TIMEOUT);
}

// Sums the K-split partial tiles in split order and applies the epilogue.
template <int BN>
__global__ void reduce_splitk_kernel(const GemmParams p)
{
    const int tiles = p.m_tiles * p.n_tiles;
    const int vec_per_tile = BM * BN / 4;
    const long long total = (long long)tiles * vec_per_tile;
    float alpha = p.alpha;
    if (p.dyn_scale)
        alpha *= __ldg(p.dyn_scale);
    if (p.dyn_scale2)
        alpha *= __ldg(p.dyn_scale2);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int tile = (int)(i / vec_per_tile), e = (int)(i % vec_per_tile);
        const int r = e / (BN / 4), c = (e % (BN / 4)) * 4;
        int mt, nt;
        tile_coords(p, tile, mt, nt);
        const long long row = (long long)mt * BM + r;
        const int col = nt * BN + c;
        if (row >= p.M || col >= p.N)
            continue;
        float4 s = make_float4(0, 0, 0, 0);
        for (int sp = 0; sp < p.splits; ++sp) {
            float4 v = *(const float4 *)(p.workspace + ((size_t)(tile * p.splits + sp) * BM + r) * BN + c);
            s.x += v.x;
            s.y += v.y;
            s.z += v.z;
            s.w += v.w;
        }
        float rs = alpha * (p.row_scale ? __ldg(p.row_scale + row) : 1.f);
        float4 cs = p.col_scale ? __ldg((const float4 *)(p.col_scale + col)) : make_float4(1, 1, 1, 1);
        s.x *= rs * cs.x;
        s.y *= rs * cs.y;
        s.z *= rs * cs.z;
        s.w *= rs * cs.w;
        if (p.out_kind == TS2_OUT_F32) {
            *(float4 *)((float *)p.C + row * p.ldc + col) = s;
        } else if (p.out_kind == TS2_OUT_F32_ADD) {
            float4 *d = (float4 *)((float *)p.C + row * p.ldc + col);
            float4 o = *(const float4 *)(p.c_in + row * p.ldc + col);
            *d = make_float4(o.x + s.x, o.y + s.y, o.z + s.z, o.w + s.w);
        } else if (p.out_kind == TS2_OUT_F16) {
            __half2 a = sat_half2(s.x, s.y), b = sat_half2(s.z, s.w);
            *(uint2 *)((__half *)p.C + row * p.ldc + col) = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
        } else {
            __nv_bfloat162 a = __floats2bfloat162_rn(s.x, s.y), b = __floats2bfloat162_rn(s.z, s.w);
            *(uint2 *)((__nv_bfloat16 *)p.C + row * p.ldc + col) = make_uint2(*(uint32_t *)&a, *(uint32_t *)&b);
        }
    }
}

// ---------------------------------------------------------------------------------
// host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// 2-D map over a row-major [rows][ld] array of es-byte elements; box = row_bytes (128 or 64, swizzled alike) x box_rows
static int make_tmap(CUtensorMap *tm, const void *base, int es, int64_t inner, int64_t rows, int64_t ld, int box_rows,
                     int row_bytes = STAGE_ROW_BYTES)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn)
        return fail(TS2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)base & 15) || ((ld * es) & 15))
        return fail(TS2_ERR_INVALID_ARG, "operand base and row pitch must be multiples of 16 bytes");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(ld * es)};
    cuuint32_t box[2] = {(cuuint32_t)(row_bytes / es), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = (es == 1) ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (es == 2) ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    CUresult r = fn(tm, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TS2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return TS2_OK;
}

int make_tensor_map(::CUtensorMap_st *tm, const void *base, int es, int64_t inner, int64_t rows, int64_t ld, int box_rows)
{
    return make_tmap(tm, base, es, inner, rows, ld, box_rows);
}

static int elem_size(int kind) { return (kind == KIND_F16 || kind == KIND_BF16) ? 2 : 1; }

static uint32_t instr_desc(int kind, bool mn, int bn)
{
    uint32_t c_fmt, ab_fmt;
    switch (kind) {
    case KIND_E4M3: c_fmt = 1; ab_fmt = 0; break; // f32 accumulate, e4m3
    case KIND_F16: c_fmt = 1; ab_fmt = 0; break;  // f16
    case KIND_BF16: c_fmt = 1; ab_fmt = 1; break; // bf16
    default: c_fmt = 2; ab_fmt = 1; break;        // s32 accumulate, s8
    }
    uint32_t d = 0;
    d |= c_fmt << 4;
    d |= ab_fmt << 7;
    d |= ab_fmt << 10;
    d |= (mn ? 1u : 0u) << 15; // A is MN-major
    d |= (mn ? 1u : 0u) << 16; // B is MN-major
    d |= (uint32_t)(bn >> 3) << 17;
    d |= (uint32_t)(BM >> 4) << 24;
    return d;
}

static int pick_bn(int64_t N) { return (N % 256 == 0 || N > 1024) ? 256 : 128; }

struct Plan {
    int bn, m_tiles, n_tiles, k_blocks, splits, kb_per_split, grid;
};

static Plan make_plan(int device, int kind, bool mn, int64_t M, int64_t N, int64_t K, int group_mode = 0, int groups = 1)
{
    Plan pl;
    const int es = elem_size(kind);
    const int bk = STAGE_ROW_BYTES / es;
    pl.bn = pick_bn(N);
    pl.m_tiles = (int)ceil_div(M, BM);
    pl.n_tiles = (int)ceil_div(N, pl.bn);
    pl.k_blocks = (int)ceil_div(K, bk);
    const int sms = sm_count(device);
    const int tiles = std::max(1, pl.m_tiles * pl.n_tiles); // an empty problem is rejected by gemm(); keep the arithmetic defined
    int splits = 1;
    if (group_mode == 0 && tiles * 2 <= sms) { // fewer than half the SMs would have work: split K
        splits = sms / tiles;
        splits = std::min(splits, std::max(1, pl.k_blocks / 8)); // keep at least 8 K blocks per unit
    }
    pl.kb_per_split = std::max(1, (int)ceil_div(pl.k_blocks, splits));
    pl.splits = std::max(1, (int)ceil_div(pl.k_blocks, pl.kb_per_split));
    pl.grid = std::min(sms, tiles * pl.splits * (group_mode == 2 ? std::max(1, groups) : 1));
    return pl;
}

int gemm_splits(int device, int kind, bool mn, int64_t M, int64_t N, int64_t K) { return make_plan(device, kind, mn, M, N, K).splits; }

size_t gemm_workspace_bytes(int device, int kind, bool mn, int64_t M, int64_t N, int64_t K)
{
    Plan pl = make_plan(device, kind, mn, M, N, K);
    if (pl.splits == 1)
        return 0;
    return (size_t)pl.m_tiles * pl.n_tiles * pl.splits * BM * pl.bn * sizeof(float);
}

// Counters of the dynamic unit scheduler: SCHED_SLOTS pairs {next unit, finished CTAs} per device, zero between
// launches (the kernel's last CTA resets its pair).  Launches take the pairs in turn, so two launches share one only
// if SCHED_SLOTS others were issued between them while the first is still running.
static constexpr int SCHED_SLOTS = 1024;
static int *sched_counters(int device)
{
    static int *base[16] = {};
    static std::mutex mu;
    static std::atomic<unsigned> serial{0};
    {
        std::lock_guard<std::mutex> lk(mu);
        int *&b = base[device & 15];
        if (!b) {
            if (cudaMalloc(&b, SCHED_SLOTS * 2 * sizeof(int)) != cudaSuccess) {
                b = nullptr;
                return nullptr;
            }
            cudaMemset(b, 0, SCHED_SLOTS * 2 * sizeof(int));
        }
    }
    return base[device & 15] + 2 * (serial.fetch_add(1, std::memory_order_relaxed) % SCHED_SLOTS);
}

static std::atomic<int> g_reserved_sms{0};
void gemm_reserve_sms(int n) { g_reserved_sms.store(std::max(0, n), std::memory_order_relaxed); }

// ---- timing ----------------------------------------------------------------------
static std::mutex g_time_mu;
static bool g_time_on = false;
struct TimedLaunch {
    cudaEvent_t a, b;
    double flops, bytes;
    int tag;
};
static double g_tag_ms[GEMM_TAGS] = {}, g_tag_flops[GEMM_TAGS] = {};
static long long g_tag_launches[GEMM_TAGS] = {};
static std::vector<TimedLaunch> g_timed;
static std::vector<cudaEvent_t> g_event_pool;
static double g_ms_total = 0, g_flops_total = 0, g_bytes_total = 0;
static long long g_timed_launches = 0;

void gemm_timing_enable(bool on)
{
    std::lock_guard<std::mutex> lk(g_time_mu);
    g_time_on = on;
}

static void timing_collect_locked()
{
    for (auto &t : g_timed) {
        if (cudaEventSynchronize(t.b) == cudaSuccess) {
            float ms = 0;
            if (cudaEventElapsedTime(&ms, t.a, t.b) == cudaSuccess) {
                g_ms_total += ms;
                g_flops_total += t.flops;
                g_bytes_total += t.bytes;
                ++g_timed_launches;
                const int tag = t.tag >= 0 && t.tag < GEMM_TAGS ? t.tag : 0;
                g_tag_ms[tag] += ms;
                g_tag_flops[tag] += t.flops;
                ++g_tag_launches[tag];
            }
        }
        g_event_pool.push_back(t.a);
        g_event_pool.push_back(t.b);
    }
    g_timed.clear();
}

void gemm_timing_get(bool reset, double *ms_total, long long *launches, double *flops_total, double *bytes_total)
{
    std::lock_guard<std::mutex> lk(g_time_mu);
    timing_collect_locked();
    if (ms_total)
        *ms_total = g_ms_total;
    if (launches)
        *launches = g_timed_launches;
    if (flops_total)
        *flops_total = g_flops_total;
    if (bytes_total)
        *bytes_total = g_bytes_total;
    if (reset) {
        g_ms_total = g_flops_total = g_bytes_total = 0;
        g_timed_launches = 0;
        for (int i = 0; i < GEMM_TAGS; ++i) {
            g_tag_ms[i] = g_tag_flops[i] = 0;
            g_tag_launches[i] = 0;
        }
    }
}

void gemm_timing_get_tag(int tag, double *ms_total, long long *launches, double *flops_total)
{
    std::lock_guard<std::mutex> lk(g_time_mu);
    timing_collect_locked();
    const int t = tag >= 0 && tag < GEMM_TAGS ? tag : 0;
    if (ms_total)
        *ms_total = g_tag_ms[t];
    if (launches)
        *launches = g_tag_launches[t];
    if (flops_total)
        *flops_total = g_tag_flops[t];
}

static cudaEvent_t pooled_event()
{
    if (!g_event_pool.empty()) {
        cudaEvent_t e = g_event_pool.back();
        g_event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

template <int BN, int ES, int MMA, bool MN, bool GATED = false>
static int launch(const GemmArgs &a, const Plan &pl, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmC,
                  const GemmParams &p)
{
    auto kern = gemm_kernel<BN, ES, MMA, MN, GATED>;
    static bool configured[16] = {};
    if (!configured[a.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::TOTAL));
        configured[a.device & 15] = true;
    }
    // SMs left to kernels that run beside this one (the data-parallel exchange): a persistent CTA that finds its SM
    // taken starts only when another CTA of the grid has finished all of its units, which can double the launch's time
    const int grid = std::max(1, std::min(pl.grid, sm_count(a.device) - g_reserved_sms.load(std::memory_order_relaxed)));
    kern<<<grid, GATED ? NUM_THREADS_GATED : NUM_THREADS, SmemLayout<BN>::TOTAL, a.stream>>>(tmA, tmB, tmC, p);
    TS2_CHECK_LAUNCH();
    if (pl.splits > 1) {
        const long long total = (long long)pl.m_tiles * pl.n_tiles * BM * BN / 4;
        int blocks = (int)std::min<long long>(ceil_div(total, 256), 4 * sm_count(a.device));
        reduce_splitk_kernel<BN><<<blocks, 256, 0, a.stream>>>(p);
        TS2_CHECK_LAUNCH();
    }
    return TS2_OK;
}

int gemm(const GemmArgs &a)
{
    if (a.M <= 0 || a.N <= 0 || a.K <= 0)
        return fail(TS2_ERR_INVALID_ARG, "gemm: empty problem (M=%lld N=%lld K=%lld)", (long long)a.M, (long long)a.N, (long long)a.K);
    if (a.N % 32)
        return fail(TS2_ERR_INVALID_ARG, "gemm: N must be a multiple of 32 (N=%lld)", (long long)a.N);
    if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || a.K >= (1ll << 31))
        return fail(TS2_ERR_TOO_LARGE, "gemm: dimension exceeds 2^31");
    const int es = elem_size(a.kind);
    const int out_es = (a.epi.out_kind == TS2_OUT_F32 || a.epi.out_kind == TS2_OUT_F32_ADD) ? 4 : 2;
    if (((uintptr_t)a.C & 15) || ((a.ldc * out_es) & 15))
        return fail(TS2_ERR_INVALID_ARG, "gemm: output base and pitch must be multiples of 16 bytes");
    if (a.epi.col_scale && ((uintptr_t)a.epi.col_scale & 15))
        return fail(TS2_ERR_INVALID_ARG, "gemm: col_scale must be 16-byte aligned");
    TS2_CUDA(cudaSetDevice(a.device));
    if (a.group_mode == 1 && (a.mn_major || !a.tile_group || a.group_rows_b <= 0 || a.groups <= 0))
        return fail(TS2_ERR_INVALID_ARG, "gemm: bad row-grouped arguments");
    if (a.group_mode == 2 && (!a.mn_major || !a.group_kptr || a.groups <= 0))
        return fail(TS2_ERR_INVALID_ARG, "gemm: bad K-grouped arguments");
    const bool paired = a.epi.pair_stride != 0;
    if (paired && (a.mn_major || a.group_mode || a.epi.out_kind != TS2_OUT_F16 || a.N != 2 * a.epi.pair_stride ||
                   a.epi.pair_stride % 128 || !a.epi.act_out || !a.epi.act_scale || a.epi.act_ld < a.epi.pair_stride ||
                   a.epi.act_kind < 0 || a.epi.act_kind > 2 || (a.epi.act_ld * (a.epi.act_kind == 1 ? 2 : 1)) % 16 ||
                   ((uintptr_t)a.epi.act_out & 15)))
        return fail(TS2_ERR_INVALID_ARG, "gemm: bad gated-activation arguments");
    Plan pl = make_plan(a.device, a.kind, a.mn_major, a.M, a.N, a.K, a.group_mode, a.groups);
    if (paired) { // one tile = 128 wide + 128 gate columns, never split along K (the epilogue needs whole sums)
        if (pl.bn != 256)
            return fail(TS2_ERR_UNSUPPORTED, "gemm: the gated-activation form needs 256-column tiles");
        pl.n_tiles = (int)(a.epi.pair_stride / 128);
        pl.splits = 1;
        pl.kb_per_split = pl.k_blocks;
        pl.grid = std::min(sm_count(a.device), pl.m_tiles * pl.n_tiles);
    }
    if (pl.splits > 1) {
        size_t need = (size_t)pl.m_tiles * pl.n_tiles * pl.splits * BM * pl.bn * sizeof(float);
        if (!a.workspace || a.workspace_bytes < need)
            return fail(TS2_ERR_INVALID_ARG, "gemm: split-K needs %zu workspace bytes, got %zu", need, a.workspace_bytes);
    }
    CUtensorMap tmA, tmB;
    const int bk = STAGE_ROW_BYTES / es;
    int rc;
    if (!a.mn_major) {
        if ((rc = make_tmap(&tmA, a.A, es, a.K, a.M, a.lda, BM)) != TS2_OK)
            return rc;
        if ((rc = make_tmap(&tmB, a.B, es, a.K, a.group_mode == 1 ? a.N * a.groups : a.N, a.ldb, paired ? pl.bn / 2 : pl.bn)) != TS2_OK)
            return rc;
    } else {
        if ((rc = make_tmap(&tmA, a.A, es, a.M, a.K, a.lda, bk)) != TS2_OK)
            return rc;
        if ((rc = make_tmap(&tmB, a.B, es, a.N, a.K, a.ldb, bk)) != TS2_OK)
            return rc;
    }
    GemmParams p;
    p.M = (int)a.M;
    p.N = (int)a.N;
    p.m_tiles = pl.m_tiles;
    p.n_tiles = pl.n_tiles;
    p.n_fast = a.M > a.N ? 1 : 0; // operand bytes are M x K and N x K of the same element size
    p.splits = pl.splits;
    p.k_blocks = pl.k_blocks;
    p.kb_per_split = pl.kb_per_split;
    p.idesc = instr_desc(a.kind, a.mn_major, pl.bn);
    p.C = a.C;
    p.ldc = a.ldc;
    p.alpha = a.epi.alpha;
    p.dyn_scale = a.epi.dyn_scale;
    p.dyn_scale2 = a.epi.dyn_scale2;
    p.row_scale = a.epi.row_scale;
    p.col_scale = a.epi.col_scale;
    p.c_in = a.epi.c_in ? a.epi.c_in : (const float *)a.C;
    p.out_kind = a.epi.out_kind;
    p.workspace = (float *)a.workspace;
    p.status = device_status_word(a.device);
    if (!p.status)
        return fail(TS2_ERR_CUDA, "gemm: no device status word");
    // Units are assigned statically by default (CTA b takes units b, b + grid, ...).  Drawing them from a global counter
    // (TS2_GEMM_DYNAMIC_UNITS=1) keeps a CTA that starts late, because a communication kernel holds its SM, from
    // stretching the launch, but measured 6 - 10 % slower on the contractions of a whole step, more than it saves.
    static const bool dynamic_units = getenv("TS2_GEMM_DYNAMIC_UNITS") != nullptr;
    p.sched = dynamic_units ? sched_counters(a.device) : nullptr;
    if (dynamic_units && !p.sched)
        return fail(TS2_ERR_CUDA, "gemm: no scheduler counters");
    p.group_mode = a.group_mode;
    p.groups = a.groups;
    p.tile_group = a.tile_group;
    p.group_rows_b = a.group_rows_b;
    p.group_kptr = a.group_kptr;
    p.c_group_stride = a.c_group_stride;
    p.bk = bk;
    p.pair_stride = (int)a.epi.pair_stride;
    p.act_out = a.epi.act_out;
    p.act_ld = a.epi.act_ld;
    p.act_scale = a.epi.act_scale;
    p.act_mult = a.epi.act_mult;
    p.act_kind = a.epi.act_kind;
    // coalesced TMA-store epilogue (the accumulate form adds its residual input first; split units go to the workspace;
    // per-group C offsets of mode 2 are not expressible as one 2-D map)
    CUtensorMap tmC = tmA;
    p.tma_store = 0;
    if (pl.splits == 1 && a.group_mode != 2) {
        if ((rc = make_tmap(&tmC, a.C, out_es, a.N, a.M, a.ldc, 32, 64)) != TS2_OK)
            return rc;
        p.tma_store = 1;
    }

    cudaEvent_t ea = nullptr, eb = nullptr;
    bool timed;
    {
        std::lock_guard<std::mutex> lk(g_time_mu);
        timed = g_time_on;
        if (timed) {
            ea = pooled_event();
            eb = pooled_event();
        }
    }
    if (timed)
        cudaEventRecord(ea, a.stream);

    const int mma = (a.kind == KIND_E4M3) ? 0 : (a.kind == KIND_I8 ? 2 : 1);
#define TS2_GEMM_CASE(BN_, ES_, MMA_, MN_)                                   \
    if (pl.bn == BN_ && es == ES_ && mma == MMA_ && a.mn_major == MN_)       \
        rc = launch<BN_, ES_, MMA_, MN_>(a, pl, tmA, tmB, tmC, p);
    rc = TS2_ERR_UNSUPPORTED;
    if (paired) {
        if (es == 1 && mma == 0)
            rc = launch<256, 1, 0, false, true>(a, pl, tmA, tmB, tmC, p);
        else if (es == 2 && mma == 1)
            rc = launch<256, 2, 1, false, true>(a, pl, tmA, tmB, tmC, p);
        else if (es == 1 && mma == 2)
            rc = launch<256, 1, 2, false, true>(a, pl, tmA, tmB, tmC, p);
    } else {
    TS2_GEMM_CASE(256, 1, 0, false)
    TS2_GEMM_CASE(128, 1, 0, false)
    TS2_GEMM_CASE(256, 1, 0, true)
    TS2_GEMM_CASE(128, 1, 0, true)
    TS2_GEMM_CASE(256, 2, 1, false)
    TS2_GEMM_CASE(128, 2, 1, false)
    TS2_GEMM_CASE(256, 2, 1, true)
    TS2_GEMM_CASE(128, 2, 1, true)
    TS2_GEMM_CASE(256, 1, 2, false)
    TS2_GEMM_CASE(128, 1, 2, false)
    TS2_GEMM_CASE(256, 1, 2, true)
    TS2_GEMM_CASE(128, 1, 2, true)
    }
#undef TS2_GEMM_CASE
    if (rc == TS2_ERR_UNSUPPORTED)
        return fail(rc, "gemm: unsupported configuration");
    if (timed) {
        cudaEventRecord(eb, a.stream);
        std::lock_guard<std::mutex> lk(g_time_mu);
        // algorithmic bytes: both operands once, the output once, the residual input of the accumulate form once
        const double mn = (double)a.M * (double)a.N;
        const double bytes = ((double)a.M + (double)a.N) * (double)a.K * es + mn * out_es + (a.epi.out_kind == TS2_OUT_F32_ADD ? mn * 4 : 0);
        g_timed.push_back({ea, eb, 2.0 * mn * (double)a.K, bytes, a.tag});
    }
    return rc;
}

// ---------------------------------------------------------------------------------
// dW contraction for callers that may not allocate.
//
// Some hosts hand every byte of device memory to their own pools when they start (the trainer this
// library plugs into does) or run a steady-state loop in which cudaMalloc's device-wide
// synchronisation would stall their other streams; for them a kernel whose scratch has to be
// cudaMalloc'ed by someone is unusable.  This variant of ts2_gemm_dw keeps the split-K scratch in
// a fixed array inside the library image instead.
static constexpr size_t STATIC_SCRATCH_BYTES = 16u << 20; // 16 MiB, resident on every GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
static __device__ int g_static_status; // bit 0: a bounded wait in the kernel gave up

struct StaticScratch {
    bool ready = false;
    float *scratch = nullptr; // device address of g_static_scratch on this device
    int32_t *status = nullptr;
};
static StaticScratch g_static[16];
static std::mutex g_static_mu;

// set-up, once per device, with that device current: in host code the array's name is only a handle; the address a
// kernel can use comes from cudaGetSymbolAddress
static int static_setup(int device, StaticScratch *out)
{
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticScratch &slot = g_static[device];
    if (!slot.ready) {
        void *p = nullptr, *q = nullptr;
        TS2_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        TS2_CUDA(cudaGetSymbolAddress(&q, g_static_status));
        slot.scratch = (float *)p;
        slot.status = (int32_t *)q;
        slot.ready = true;
    }
    *out = slot;
    return TS2_OK;
}

// one CTA waits, with the library's bounded wait, on a barrier nothing arrives at, gives up after the limit and
// raises the time-out bit of the given status word (the way a contraction kernel reports a wait that ran out)
__global__ void static_status_selftest_kernel(int32_t *status)
{
    __shared__ uint64_t bar;
    __shared__ int abort_s;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_s = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(smem_u32(&bar), 0, &abort_s))
        atomicOr(status, TS2_STATUS_WAIT_TIMEOUT);
}

// The status word of the no-allocation entry point on this device, or null while that entry point has not run
// there (then nothing can have been OR-ed into it).  Never allocates and never triggers the symbol look-up.
int32_t *static_status_word_if_ready(int device)
{
    if (device < 0 || device >= 16)
        return nullptr;
    std::lock_guard<std::mutex> lk(g_static_mu);
    return g_static[device].ready ? g_static[device].status : nullptr;
}

} // namespace ts2

using namespace ts2;

extern "C" int ts2_gemm_dw_noalloc(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                                   const void *dY, const void *X, void *dW, float alpha)
{
    const int kind = prec == TS2_PREC_FP8 ? KIND_E4M3 : prec == TS2_PREC_F16 ? KIND_F16 : prec == TS2_PREC_INT8 ? KIND_I8 : -1;
    if (kind < 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: unknown precision %d", prec);
    if (T <= 0 || in_dim <= 0 || out_dim <= 0 || !dY || !X || !dW)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: empty problem or null pointer");
    if (in_dim % 32)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: in_dim must be a multiple of 32 (got %lld)", (long long)in_dim);
    if (out_kind != TS2_OUT_F32 && out_kind != TS2_OUT_F32_ADD)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: the gradient is fp32 (TS2_OUT_F32 or TS2_OUT_F32_ADD)");
    if (T >= (1ll << 31) || in_dim >= (1ll << 31) || out_dim >= (1ll << 31))
        return fail(TS2_ERR_TOO_LARGE, "ts2_gemm_dw_noalloc: dimension exceeds 2^31");
    if (((uintptr_t)dW & 15) || ((in_dim * 4) & 15))
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: output base and pitch must be multiples of 16 bytes");
    if (device < 0 || device >= 16)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_noalloc: device %d out of range", device);
    TS2_CUDA(cudaSetDevice(device));
    StaticScratch st;
    int rc = static_setup(device, &st);
    if (rc != TS2_OK)
        return rc;
    const Plan pl = make_plan(device, kind, true, out_dim, in_dim, T);
    const size_t need = pl.splits > 1 ? (size_t)pl.m_tiles * pl.n_tiles * pl.splits * BM * pl.bn * sizeof(float) : 0;
    if (need > STATIC_SCRATCH_BYTES)
        return fail(TS2_ERR_TOO_LARGE,
                    "ts2_gemm_dw_noalloc: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                    "use ts2_gemm_dw with a caller-provided workspace",
                    need, STATIC_SCRATCH_BYTES);
    const int es = elem_size(kind), bk = STAGE_ROW_BYTES / es;
    CUtensorMap tmA, tmB;
    if ((rc = make_tmap(&tmA, dY, es, out_dim, T, out_dim, bk)) != TS2_OK)
        return rc;
    if ((rc = make_tmap(&tmB, X, es, in_dim, T, in_dim, bk)) != TS2_OK)
        return rc;
    GemmParams p;
    p.M = (int)out_dim;
    p.N = (int)in_dim;
    p.m_tiles = pl.m_tiles;
    p.n_tiles = pl.n_tiles;
    p.n_fast = out_dim > in_dim ? 1 : 0;
    p.splits = pl.splits;
    p.k_blocks = pl.k_blocks;
    p.kb_per_split = pl.kb_per_split;
    p.idesc = instr_desc(kind, true, pl.bn);
    p.C = dW;
    p.ldc = in_dim;
    p.alpha = alpha;
    p.dyn_scale = p.dyn_scale2 = p.row_scale = p.col_scale = nullptr;
    p.c_in = (const float *)dW;
    p.out_kind = out_kind;
    // every (tile, split) unit overwrites its whole partial tile before the reduction reads it, so
    // nothing in the scratch has to start at zero; the status word is only ever OR-ed into
    p.workspace = st.scratch;
    p.status = st.status;
    p.group_mode = 0;
    p.groups = 1;
    p.tile_group = nullptr;
    p.group_rows_b = 0;
    p.group_kptr = nullptr;
    p.c_group_stride = 0;
    p.bk = bk;
    p.tma_store = 0;
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    const int mma = (kind == KIND_E4M3) ? 0 : (kind == KIND_I8 ? 2 : 1);
    rc = TS2_ERR_UNSUPPORTED;
#define TS2_NOALLOC_CASE(BN_, ES_, MMA_)             \
    if (pl.bn == BN_ && es == ES_ && mma == MMA_)    \
        rc = launch<BN_, ES_, MMA_, true>(a, pl, tmA, tmB, tmA, p);
    TS2_NOALLOC_CASE(256, 1, 0)
    TS2_NOALLOC_CASE(128, 1, 0)
    TS2_NOALLOC_CASE(256, 2, 1)
    TS2_NOALLOC_CASE(128, 2, 1)
    TS2_NOALLOC_CASE(256, 1, 2)
    TS2_NOALLOC_CASE(128, 1, 2)
#undef TS2_NOALLOC_CASE
    if (rc == TS2_ERR_UNSUPPORTED)
        return fail(rc, "ts2_gemm_dw_noalloc: unsupported configuration");
    return rc;
}

// Self-test of the status path of ts2_gemm_dw_noalloc: the same bounded wait as ts2_selftest_wait_limit, reported
// through the static status word that entry point's kernels use.  Allocates nothing.
extern "C" int ts2_selftest_wait_limit_noalloc(int device)
{
    if (device < 0 || device >= 16)
        return fail(TS2_ERR_INVALID_ARG, "ts2_selftest_wait_limit_noalloc: device %d out of range", device);
    TS2_CUDA(cudaSetDevice(device));
    StaticScratch st;
    int rc = static_setup(device, &st);
    if (rc != TS2_OK)
        return rc;
    static_status_selftest_kernel<<<1, 32>>>(st.status);
    TS2_CHECK_LAUNCH();
    TS2_CUDA(cudaDeviceSynchronize());
    return collect_device_status(device);
}
