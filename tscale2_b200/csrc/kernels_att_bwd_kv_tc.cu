// tcgen05 attention backward, dK and dV from one kernel (head width 128, sm_100a).  Same math, inputs and outputs
// as the dK / dV modes of kernels_att_bwd_tc.cu (references: src/gpt/compute/layer_att_reference.h:41-212,
// gpu_att_fp16.cu / .cuh), which recompute the same S = K . Q^T twice and stream Q and dO twice.
//
// A CTA owns 128 resident keys (K and V rows) and streams 64-node tiles of Q and dO:
//   S^T  = K . Q^T,  dP^T = V . dO^T          128 x 64 each, fp32, into one of TWO S / dP buffer pairs in TMEM
//   compute: P^T = 2^(S^T ds - lse) masked;  Gv = P^T;  Gk = P^T (dP^T - dscale) c2        fp16, back into TMEM
//   dV += Gv . dO,  dK += Gk . Q               128 x 128 each, G as the TMEM A operand, streamed tile MN-major
// TMEM (512 columns): pair 0 = S [0,64) dP [64,128); dK [128,256); dV [256,384); pair 1 = S [384,448) dP [448,512).
// With two S / dP pairs the issuer queues the products of tile j+1 before it waits for the compute warps of tile
// j, so the tensor pipe works while they compute.  G goes where the thread's own S / dP values were (same lane,
// own columns); at that time no MMA writes into that 128-column group (the next tile's products go to the other
// pair, the accumulators are other groups), and the pair is overwritten only after the MMAs that read it are complete
// (pair_free).  20 warps: TMA producer, two MMA issuers (first products; accumulating products), 1 idle, 16 compute
// (four per TMEM lane quarter, 16 of the tile's 64 columns each).  Every wait is bounded; a give-up raises the status
// word.
#include "att_tc.cuh"

namespace ts2 {

static constexpr int KV_THREADS = 128 + 512;
static constexpr int KV_STAGES = 4;
static constexpr int KV_META_BYTES = TC_BN * 16;
static constexpr int KV_STAGE_BYTES = 2 * KV_BYTES; // Q tile + dO tile, 64 rows each
static constexpr int KV_RES_BYTES = 2 * Q_BYTES;    // K block + V block, 128 rows each
static constexpr int KV_STAGE_OFF = KV_RES_BYTES;
static constexpr int KV_META_OFF = KV_STAGE_OFF + KV_STAGES * KV_STAGE_BYTES;
static constexpr int KV_BAR_OFF = KV_META_OFF + KV_STAGES * KV_META_BYTES;
static constexpr int KV_SMEM = KV_BAR_OFF + 256;
static_assert(KV_SMEM <= 232448, "shared memory budget");

struct AttBwdKvParams {
    int T, H, Tpad;
    float slope;
    const int *rev_first, *rev_last;
    const float4 *meta; // [H][Tpad]: {-lse, -dscale * c2, span start, span length} per node
    void *dk, *dv;      // fp32 or fp16 [T][128 H]
    int32_t *status;
};

// OUT16: the gradients are written as fp16 (what the engine feeds its next kernel with) instead of fp32
template <bool OUT16>
__global__ void __launch_bounds__(KV_THREADS, 1)
    att_bwd_kv_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                         const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, const AttBwdKvParams p)
{
    extern __shared__ __align__(1024) uint8_t att_kv_smem[];
    uint8_t *smem = att_kv_smem;
    if (smem_u32(smem) & 1023) { // the swizzled tiles need a 1024-byte aligned base; refuse instead of computing garbage
        if (threadIdx.x == 0)
            atomicOr(p.status, TS2_STATUS_BAD_ARG);
        return;
    }
    const uint32_t sK = smem_u32(smem), sV = sK + Q_BYTES, sStage = sK + KV_STAGE_OFF, sMeta = sK + KV_META_OFF;
    uint64_t *bars = (uint64_t *)(smem + KV_BAR_OFF);
    // res_full, st_full[4], st_empty[4], s_full[2], pair_free[2], g_full[2], all_done.  Everything that is handed over
    // once per tile has one barrier per S / dP pair: the next phase of a pair's barrier belongs to the tile two further
    // on, which cannot start before the waiter of this phase has acted, so a parity test can never miss a phase.
    const uint32_t res_full = smem_u32(bars), st_full0 = smem_u32(bars + 1), st_empty0 = smem_u32(bars + 5), s_full0 = smem_u32(bars + 9),
                   pair_free0 = smem_u32(bars + 11), g_full0 = smem_u32(bars + 13), all_done = smem_u32(bars + 15);
    uint32_t *tmem_slot = (uint32_t *)(bars + 16);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    int *rng = (int *)(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = p.T, H = p.H, h = blockIdx.y, r0 = blockIdx.x * TC_BM;

    // range of nodes that see any of this block's keys
    if (threadIdx.x == 0) {
        rng[0] = 0x7fffffff;
        rng[1] = -1;
    }
    __syncthreads();
    if (threadIdx.x < TC_BM && r0 + (int)threadIdx.x < T) {
        const int a = p.rev_first[r0 + threadIdx.x], e = p.rev_last[r0 + threadIdx.x];
        if (e >= a) {
            atomicMin(&rng[0], a);
            atomicMax(&rng[1], e);
        }
    }
    if (threadIdx.x == 0) {
        mbar_init(res_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(st_full0 + 8 * s, 1);
            mbar_init(st_empty0 + 8 * s, 1);
        }
        mbar_init(s_full0, 1);
        mbar_init(s_full0 + 8, 1);
        mbar_init(g_full0, 512);
        mbar_init(g_full0 + 8, 512);
        mbar_init(pair_free0, 1);
        mbar_init(pair_free0 + 8, 1);
        mbar_init(all_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmDO);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tDK = tmem_base + 128, tDV = tmem_base + 256;
    const int tile0 = rng[1] >= rng[0] ? rng[0] / TC_BN : 0;
    const int n = rng[1] >= rng[0] ? rng[1] / TC_BN - tile0 + 1 : 0;
    const int col0 = h * TC_HD;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && n > 0) {
            mbar_arrive_expect_tx(res_full, KV_RES_BYTES);
            tma_load_2d(sK, &tmK, res_full, col0, r0);
            tma_load_2d(sK + Q_BYTES / 2, &tmK, res_full, col0 + 64, r0);
            tma_load_2d(sV, &tmV, res_full, col0, r0);
            tma_load_2d(sV + Q_BYTES / 2, &tmV, res_full, col0 + 64, r0);
            for (int j = 0; j < n; ++j) {
                const int st = j % KV_STAGES, row = (tile0 + j) * TC_BN;
                if (!mbar_wait(st_empty0 + 8 * st, ((j / KV_STAGES) & 1) ^ 1, abort_flag))
                    break;
                const uint32_t fb = st_full0 + 8 * st;
                mbar_arrive_expect_tx(fb, KV_STAGE_BYTES + KV_META_BYTES);
                const uint32_t dq = sStage + st * KV_STAGE_BYTES, dd = dq + KV_BYTES;
                tma_load_2d(dq, &tmQ, fb, col0, row);
                tma_load_2d(dq + KV_BYTES / 2, &tmQ, fb, col0 + 64, row);
                tma_load_2d(dd, &tmDO, fb, col0, row);
                tma_load_2d(dd + KV_BYTES / 2, &tmDO, fb, col0 + 64, row);
                bulk_load(sMeta + st * KV_META_BYTES, p.meta + (size_t)h * p.Tpad + row, KV_META_BYTES, fb);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer A: S^T and dP^T ----------------
        // Two issuing threads on two schedulers.  A thread is held for about as long as the MMAs it issues run, and
        // while the compute warps are busy its instructions wait for issue slots; with one thread for all four products
        // of a tile the tensor pipe stood idle for more than half of every tile.  This one runs one tile ahead with the
        // first products; issuer B (warp 2) follows the compute warps with the accumulating ones.
        if (lane == 0 && n > 0) {
            constexpr uint32_t idesc_s = umma_idesc_f16(TC_BN, false, false);
            const uint64_t dK = umma_smem_desc(sK, 16, 1024), dV = umma_smem_desc(sV, 16, 1024);
            bool ok = mbar_wait(res_full, 0, abort_flag);
            for (int jj = 0; jj < n && ok; ++jj) { // S^T and dP^T of tile jj into pair jj & 1
                // the pair held G of tile jj - 2: the MMAs that read it must be complete before these write there.  A
                // barrier per pair, so that its next phase cannot complete before this thread has issued tile jj
                if (jj >= 2 && !mbar_wait(pair_free0 + 8 * (jj & 1), ((jj - 2) >> 1) & 1, abort_flag))
                    break;
                const int st = jj % KV_STAGES;
                if (!mbar_wait(st_full0 + 8 * st, (jj / KV_STAGES) & 1, abort_flag))
                    break;
                tc_fence_after();
                const uint32_t bq = sStage + st * KV_STAGE_BYTES, bd = bq + KV_BYTES;
                const uint64_t dQ = umma_smem_desc(bq, 16, 1024), dD = umma_smem_desc(bd, 16, 1024);
                const uint32_t tS = tmem_base + ((jj & 1) ? 384 : 0), tDP = tS + TC_BN;
                // 8 steps of 16 head dims; operands are two 64-dim atoms each
                umma_f16_x4(tS, dK, dQ, idesc_s, 0u, 2u, 2u);
                umma_f16_x4(tS, dK + (Q_BYTES / 2 >> 4), dQ + (KV_BYTES / 2 >> 4), idesc_s, 1u, 2u, 2u);
                umma_f16_x4(tDP, dV, dD, idesc_s, 0u, 2u, 2u);
                umma_f16_x4(tDP, dV + (Q_BYTES / 2 >> 4), dD + (KV_BYTES / 2 >> 4), idesc_s, 1u, 2u, 2u);
                tc_commit(s_full0 + 8 * (jj & 1));
            }
        }
    } else if (warp == 2) {
        // ------------------------------ MMA issuer B: dV and dK -------------------
        if (lane == 0 && n > 0) {
            constexpr uint32_t idesc_acc = umma_idesc_f16(TC_HD, false, true);
            for (int j = 0; j < n; ++j) {
                const int st = j % KV_STAGES;
                if (!mbar_wait(g_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag) ||
                    !mbar_wait(st_full0 + 8 * st, (j / KV_STAGES) & 1, abort_flag))
                    break;
                tc_fence_after();
                // dV += Gv . dO, dK += Gk . Q: 4 steps of 16 nodes; G from tensor memory (part kk of the compute warps
                // left its 16 nodes as 8 columns of fp16 pairs at column 16 kk of the S / dP block), the streamed
                // tile read MN-major (its 128 columns are the output columns), 16 rows = 2048 bytes per step
                const uint32_t bq = sStage + st * KV_STAGE_BYTES, bd = bq + KV_BYTES;
                const uint64_t dQm = umma_smem_desc(bq, KV_BYTES / 2, 1024), dDm = umma_smem_desc(bd, KV_BYTES / 2, 1024);
                const uint32_t tS = tmem_base + ((j & 1) ? 384 : 0), tDP = tS + TC_BN;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f16_ts(tDV, tS + 16 * kk, dDm + (uint64_t)(kk * 128), idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f16_ts(tDK, tDP + 16 * kk, dQm + (uint64_t)(kk * 128), idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(pair_free0 + 8 * (j & 1));
                tc_commit(st_empty0 + 8 * st);
                if (j == n - 1)
                    tc_commit(all_done); // a barrier of its own for the epilogue
            }
        }
    } else if (warp >= 4) {
        // ------------------------------ compute warps -----------------------------
        const int quarter = warp & 3, part = (warp - 4) >> 2;
        const int row = quarter * 32 + lane;
        const int rr = r0 + row; // key of this thread
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float ds = att_dot_scale_tc(), c2 = ds * 0.693147f, slope = p.slope;
        bool ok = true;
        for (int j = 0; j < n; ++j) {
            // s_full says the products are done; the tile's per-node records came with the same stage by a bulk copy, and
            // the threads that read them observe that stage's barrier themselves (it has long completed: the issuer
            // waited for it before the products), which is what orders the copy's writes before these reads
            ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag) &&
                                             mbar_wait(st_full0 + 8 * (j % KV_STAGES), (j / KV_STAGES) & 1, abort_flag));
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t tS = tmem_base + ((j & 1) ? 384 : 0) + lane_addr + part * 16, tDP = tS + TC_BN;
            const int c0 = (tile0 + j) * TC_BN + part * 16; // first node of this thread's columns
            const float4 *mt = (const float4 *)(smem + KV_META_OFF + (j % KV_STAGES) * KV_META_BYTES) + part * 16;
            uint32_t rs[16], rp[16];
            tmem_ld16(tS, rs);
            tmem_ld16(tDP, rp);
            tmem_ld_wait();
            uint32_t gv[8], gk[8];
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                float w2[2], g2[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float4 m = mt[i + e];
                    float off = m.x;
                    if (slope != 0.f)
                        off -= slope * (float)(c0 + i + e - rr);
                    const bool valid = (unsigned)(rr - __float_as_int(m.z)) <= (unsigned)__float_as_int(m.w);
                    float w;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(fmaf(__uint_as_float(rs[i + e]), ds, off)));
                    w = valid ? w : 0.f;
                    w2[e] = w;
                    g2[e] = w * fmaf(__uint_as_float(rp[i + e]), c2, m.y);
                }
                const __half2 hv = sat_half2(w2[0], w2[1]), hk = sat_half2(g2[0], g2[1]);
                gv[i >> 1] = *(const uint32_t *)&hv;
                gk[i >> 1] = *(const uint32_t *)&hk;
            }
            // Gv / Gk go where this thread's own S / dP values were (its lane, the first 8 of its 16 columns)
            tmem_st8(tS, gv);
            tmem_st8(tDP, gk);
            tmem_st_wait();
            tc_fence_before();
            // 512 arrivals per tile on the pair's barrier.  No thread can arrive for tile j + 2 (same barrier) before this
            // phase is complete: S of tile j + 2 is written only after the MMAs that read this tile's G have finished.
            mbar_arrive(g_full0 + 8 * (j & 1));
        }
        // epilogue: both accumulators -> fp32 outputs.  A warp's 32 rows x 32 columns go through a 4 KB block of the
        // (now idle) stage area, rows of 128 bytes with the 128-byte swizzle (16-byte chunk c of row r at c ^ (r & 7)),
        // and one TMA store each: direct stores would write 16 bytes into each of 32 different lines per instruction.
        // Rows past T are clipped by the TMA unit.
        if (n > 0 && ok)
            ok = mbar_wait(all_done, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if constexpr (OUT16) {
            // fp16: parts 0, 1 take the two 64-column halves of dK, parts 2, 3 those of dV: 32 rows x 128 bytes per warp
            const int which = part >> 1, hc = part & 1;
            uint8_t *blk = smem + KV_STAGE_OFF + (warp - 4) * 4096, *srow = blk + lane * 128;
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t r[32];
                if (n > 0 && ok) {
                    tmem_ld32((which ? tDV : tDK) + lane_addr + hc * 64 + cc * 32, r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        r[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 h0 = sat_half2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])),
                                  h1 = sat_half2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])),
                                  h2 = sat_half2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])),
                                  h3 = sat_half2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                    *(uint4 *)(srow + (((cc * 4 + i) ^ (lane & 7)) << 4)) =
                        make_uint4(*(const uint32_t *)&h0, *(const uint32_t *)&h1, *(const uint32_t *)&h2, *(const uint32_t *)&h3);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(which ? (const void *)&tmDV : (const void *)&tmDK, smem_u32(blk), col0 + hc * 64, r0 + quarter * 32);
                bulk_commit();
            }
        } else
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            uint32_t r[32];
            if (n > 0 && ok) {
                tmem_ld32((which ? tDV : tDK) + lane_addr + part * 32, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = 0u;
            }
            uint8_t *blk = smem + KV_STAGE_OFF + ((warp - 4) * 2 + which) * 4096, *srow = blk + lane * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *(uint4 *)(srow + ((i ^ (lane & 7)) << 4)) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(which ? (const void *)&tmDV : (const void *)&tmDK, smem_u32(blk), col0 + part * 32, r0 + quarter * 32);
                bulk_commit();
            }
        }
        if (lane == 0)
            bulk_wait_read<0>(); // shared memory must outlive the stores that read it
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, 512);
    if (threadIdx.x == 0 && *abort_flag)
        atomicOr(p.status, TS2_STATUS_WAIT_TIMEOUT);
}

int attention_backward_kv_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float4 *meta,
                             int Tpad, const int *rev_first, const int *rev_last, int T, int H, float slope, void *dk, void *dv,
                             bool out16)
{
    static bool configured[16] = {};
    if (!configured[c.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(att_bwd_kv_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM));
        TS2_CUDA(cudaFuncSetAttribute(att_bwd_kv_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM));
        configured[c.device & 15] = true;
    }
    const int Q = H * TC_HD;
    CUtensorMap tK, tV, tQ, tDO, tDK, tDV;
    int rc;
    if ((rc = make_tensor_map(&tK, k, 2, Q, T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tV, v, 2, Q, T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tQ, q, 2, Q, T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tDO, dout, 2, Q, T, Q, TC_BN)) != TS2_OK)
        return rc;
    // outputs: boxes of 128 bytes (32 fp32 or 64 fp16 columns) x 32 rows
    if ((rc = make_tensor_map(&tDK, dk, out16 ? 2 : 4, Q, T, Q, 32)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tDV, dv, out16 ? 2 : 4, Q, T, Q, 32)) != TS2_OK)
        return rc;
    AttBwdKvParams p;
    p.T = T;
    p.H = H;
    p.Tpad = Tpad;
    p.slope = slope;
    p.rev_first = rev_first;
    p.rev_last = rev_last;
    p.meta = meta;
    p.dk = dk;
    p.dv = dv;
    p.status = device_status_word(c.device);
    if (!p.status)
        return fail(TS2_ERR_CUDA, "attention: no device status word");
    dim3 grid((unsigned)ceil_div(T, TC_BM), (unsigned)H);
    if (out16)
        att_bwd_kv_tc_kernel<true><<<grid, KV_THREADS, KV_SMEM, c.stream>>>(tK, tV, tQ, tDO, tDK, tDV, p);
    else
        att_bwd_kv_tc_kernel<false><<<grid, KV_THREADS, KV_SMEM, c.stream>>>(tK, tV, tQ, tDO, tDK, tDV, p);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
