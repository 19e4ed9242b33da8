// tcgen05 formulation of the attention core for head width 128 (sm_100a): the two contractions
// of every (128-row block, 64-wide tile) pair run on the 5th-generation tensor cores with their
// accumulators in TMEM; operands arrive by TMA (no multicast) in 128-byte-swizzled tiles.
// Same math and the same inputs / outputs as kernels_att_mma.cu (see there for the references
// into src/gpt/compute/layer_att_reference.h and gpu_att_fp16.cu).
//
// Forward, one CTA per (128 nodes, head), 320 threads:
//   warp 0     TMA producer: Q block once, then K and V tiles through two 2-stage rings (a K stage is
//              free again as soon as its S product is done, long before the V stage of the same tile)
//   warp 1     TMEM owner and MMA issuer: S = Q . K^T (128 x 64, fp32, two buffers in TMEM, so the
//              product of tile j+1 runs while tile j is in the softmax), later O += P . V
//   warps 2-9  softmax: two warps per TMEM lane quarter, thread = (node row, 32 of the tile's 64 keys);
//              the pair agrees on the row maximum through shared memory (rounded up to bf16, so both
//              use the same reference), writes P (fp16) into a swizzled K-major shared-memory tile
//              for the second MMA and rescales O in TMEM only when a row's maximum grew by more
//              than 8 (2^8 headroom in fp16 P and fp32 sums), which keeps tcgen05.ld/st of O off
//              the common path
// The zero "sink" vector of the reference is the initial state m = 0, l = 1.
// Two CTAs fit an SM (112 KB shared memory, 256 TMEM columns each), so one CTA's softmax overlaps
// the other's MMAs.  Every wait is bounded (see mbar_wait); a give-up raises the status word.
#include "att_tc.cuh"

namespace ts2 {

static constexpr int TC_THREADS = 320;
// 112 KB of tiles + 128 B of barriers + 512 B of exchange slots: two CTAs per SM (2 x (115328 + 1024 reserved) <= 228 KB)
static constexpr int FWD_XCH_OFF = Q_BYTES + 2 * 2 * KV_BYTES + P_BYTES + 128; // row maxima of the two column halves, bf16
static constexpr int FWD_SMEM = FWD_XCH_OFF + 2 * TC_BM * 2;

struct AttTcParams {
    int T, H;
    float slope;
    const int *span_start, *span_finish;
    __half *o;
    float *lse;
    int32_t *status;
};

__global__ void __launch_bounds__(TC_THREADS, 2)
    att_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const AttTcParams p)
{
    extern __shared__ __align__(1024) uint8_t att_tc_smem[];
    uint8_t *smem = att_tc_smem;
    if (smem_u32(smem) & 1023) { // the swizzled tiles need a 1024-byte aligned base; refuse instead of computing garbage
        if (threadIdx.x == 0)
            atomicOr(p.status, TS2_STATUS_BAD_ARG);
        return;
    }
    const uint32_t sQ = smem_u32(smem), sK = sQ + Q_BYTES, sV = sK + 2 * KV_BYTES, sP = sV + 2 * KV_BYTES;
    uint64_t *bars = (uint64_t *)(smem + Q_BYTES + 4 * KV_BYTES + P_BYTES);
    const uint32_t q_full = smem_u32(bars), k_full0 = smem_u32(bars + 1), k_empty0 = smem_u32(bars + 3), v_full0 = smem_u32(bars + 5),
                   v_empty0 = smem_u32(bars + 7), s_full0 = smem_u32(bars + 9), p_full = smem_u32(bars + 11), o_ready = smem_u32(bars + 12);
    uint32_t *tmem_slot = (uint32_t *)(bars + 13);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    int &s_lo = *(int *)(tmem_slot + 2), &s_hi = *(int *)(tmem_slot + 3);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = p.T, H = p.H, h = blockIdx.y, t0 = blockIdx.x * TC_BM;

    // key range of the block: [min start, max finish] over its rows
    {
        if (threadIdx.x == 0) {
            s_lo = 0x7fffffff;
            s_hi = -1;
        }
        __syncthreads();
        if (threadIdx.x < TC_BM && t0 + (int)threadIdx.x < T) {
            const int st = p.span_start[t0 + threadIdx.x], fi = p.span_finish[t0 + threadIdx.x];
            if (fi >= st) {
                atomicMin(&s_lo, st);
                atomicMax(&s_hi, fi);
            }
        }
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full0 + 8 * s, 1);
            mbar_init(k_empty0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1);
            mbar_init(v_empty0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1);
        }
        mbar_init(p_full, 256);
        mbar_init(o_ready, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 2 * TC_BN; // S buffers at columns 0 and 64
    const int lo = s_lo, hi = s_hi;
    const int tile0 = hi >= lo ? lo / TC_BN : 0, tile1 = hi >= lo ? hi / TC_BN : -1; // no keys: no tiles
    const int col0 = h * TC_HD;

    const int n_tiles = tile1 - tile0 + 1;
    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            mbar_arrive_expect_tx(q_full, Q_BYTES);
            tma_load_2d(sQ, &tmQ, q_full, col0, t0);
            tma_load_2d(sQ + Q_BYTES / 2, &tmQ, q_full, col0 + 64, t0);
            // order of need: K(0), then for every tile K(j+1) before V(j)
            bool ok = true;
            for (int j = -1; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    const int jj = j + 1, st = jj & 1;
                    if (!(ok = mbar_wait(k_empty0 + 8 * st, ((jj >> 1) & 1) ^ 1, abort_flag)))
                        break;
                    const uint32_t fb = k_full0 + 8 * st, dk = sK + st * KV_BYTES;
                    mbar_arrive_expect_tx(fb, KV_BYTES);
                    tma_load_2d(dk, &tmK, fb, col0, (tile0 + jj) * TC_BN);
                    tma_load_2d(dk + KV_BYTES / 2, &tmK, fb, col0 + 64, (tile0 + jj) * TC_BN);
                }
                if (j >= 0) {
                    const int st = j & 1;
                    if (!(ok = mbar_wait(v_empty0 + 8 * st, ((j >> 1) & 1) ^ 1, abort_flag)))
                        break;
                    const uint32_t fb = v_full0 + 8 * st, dv = sV + st * KV_BYTES;
                    mbar_arrive_expect_tx(fb, KV_BYTES);
                    tma_load_2d(dv, &tmV, fb, col0, (tile0 + j) * TC_BN);
                    tma_load_2d(dv + KV_BYTES / 2, &tmV, fb, col0 + 64, (tile0 + j) * TC_BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(TC_BN, false, false);
            constexpr uint32_t idesc_pv = umma_idesc_f16(TC_HD, false, true);
            // descriptors differ from these bases only in the 16-byte-granular start address (the low field; shared
            // memory addresses stay below 2^18, so adding to it never carries into the next field)
            const uint64_t dq = umma_smem_desc(sQ, 16, 1024), dk = umma_smem_desc(sK, 16, 1024), dp = umma_smem_desc(sP, 16, 1024),
                           dv = umma_smem_desc(sV, KV_BYTES / 2, 1024);
            auto issue_qk = [&](int jj) { // S[jj & 1] = Q . K(jj)^T: 8 steps of 16 head dims; two 64-dim atoms per operand
                const uint64_t kb = dk + (uint64_t)((jj & 1) * (KV_BYTES >> 4));
                const uint32_t d = tmem_S + (jj & 1) * TC_BN;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_f16(d, dq + (uint64_t)(((k >> 2) * (Q_BYTES / 2) + (k & 3) * 32) >> 4),
                             kb + (uint64_t)(((k >> 2) * (KV_BYTES / 2) + (k & 3) * 32) >> 4), idesc_qk, k > 0 ? 1u : 0u);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(k_full0, 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
                tc_commit(s_full0);
                tc_commit(k_empty0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                if (j + 1 < n_tiles) {
                    // the S buffer of tile j+1 was last read by the softmax of tile j-1, which has arrived at p_full
                    const int sn = (j + 1) & 1;
                    if (!mbar_wait(k_full0 + 8 * sn, ((j + 1) >> 1) & 1, abort_flag))
                        break;
                    tc_fence_after();
                    issue_qk(j + 1);
                    tc_commit(s_full0 + 8 * sn);
                    tc_commit(k_empty0 + 8 * sn);
                }
                if (!mbar_wait(p_full, j & 1, abort_flag) || !mbar_wait(v_full0 + 8 * st, (j >> 1) & 1, abort_flag))
                    break;
                tc_fence_after();
                // O += P . V: 4 steps of 16 keys; V tile is MN-major for this product (dims contiguous)
                const uint64_t vb = dv + (uint64_t)(st * (KV_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem_O, dp + (uint64_t)(k * 2), vb + (uint64_t)(k * 128), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                tc_commit(v_empty0 + 8 * st);
                tc_commit(o_ready);
            }
        }
    } else {
        // ------------------------------ softmax warps -----------------------------
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane, t = t0 + row;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int st_row = t < T ? p.span_start[t] : 0, fi_row = t < T ? p.span_finish[t] : -1;
        const float ds = att_dot_scale_tc(), slope = p.slope;
        __nv_bfloat16 *xch = (__nv_bfloat16 *)(smem + FWD_XCH_OFF); // [half][row]
        float m_used = 0.f, l = half == 0 ? 1.f : 0.f; // the zero vector of weight 2^-m, counted once per row
        bool ok = true;
        for (int tile = tile0, j = 0; tile <= tile1; ++tile, ++j) {
            // after a failed wait a warp keeps walking the loop, because its partner counts on one pair barrier per
            // tile, but touches neither TMEM nor the P tile any more
            if (ok)
                ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * (j & 1), (j >> 1) & 1, abort_flag));
            // S is double-buffered, so a warp that is done with tile j - 1 may find this tile's S ready before a slower
            // warp has finished tile j - 1.  It goes on only when all 256 threads have arrived at p_full for that tile:
            // then its partner has read the exchange slot it is about to rewrite, and its own arrival below cannot be
            // counted for the previous phase.  (The phase cannot have completed without this thread's own arrival, so
            // the parity test is unambiguous.)
            if (ok && j > 0)
                ok = __all_sync(0xffffffffu, mbar_wait(p_full, (j - 1) & 1, abort_flag));
            tc_fence_after();
            float s[32];
            if (ok) {
                uint32_t r0[32];
                tmem_ld32(tmem_S + lane_addr + (j & 1) * TC_BN + half * 32, r0);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    s[i] = __uint_as_float(r0[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    s[i] = 0.f;
            }
            const int key0 = tile * TC_BN + half * 32;
            // four independent chains keep the warps busy
            float mx4[4] = {m_used, m_used, m_used, m_used};
            const bool inside = key0 >= st_row && key0 + 31 <= fi_row; // all 32 keys visible from this row
            const bool plain = slope == 0.f && inside; // then s stays the raw product and the scale rides in the exponent's fma
            if (plain) {
                float r4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r4[i & 3] = fmaxf(r4[i & 3], s[i]);
                mx4[0] = fmaxf(m_used, fmaxf(fmaxf(r4[0], r4[1]), fmaxf(r4[2], r4[3])) * ds);
            } else {
                const float base = slope * (float)(t - key0);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + i;
                    float x = fmaf(s[i], ds, fmaf(slope, (float)i, -base));
                    x = (key >= st_row && key <= fi_row) ? x : -INFINITY;
                    s[i] = x;
                    mx4[i & 3] = fmaxf(mx4[i & 3], x);
                }
            }
            // agree on the row maximum with the warp that holds the other 32 keys; rounding up to bf16 makes the
            // exchanged value the reference both use (a reference above the true maximum only makes P smaller).
            // The slot is free: every thread has arrived at p_full for the previous tile (waited for above), which each
            // does after reading its partner's slot.
            const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            xch[half * TC_BM + row] = mine;
            pair_barrier(quarter);
            const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(xch[(half ^ 1) * TC_BM + row]));
            // rescale only when some row of the warp outgrew its reference maximum by more than 8
            const bool need = mx > m_used + 8.f;
            const bool warp_need = __any_sync(0xffffffffu, need);
            float rs = 1.f;
            if (need) {
                rs = exp2f(m_used - mx);
                m_used = mx;
                l *= rs;
            }
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            const float es = plain ? ds : 1.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float pv;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pv) : "f"(fmaf(s[i], es, -m_used)));
                s[i] = pv;
                sum4[i & 3] += pv;
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // the previous P . V must have finished before P is overwritten or O is touched
            if (ok && j > 0)
                ok = __all_sync(0xffffffffu, mbar_wait(o_ready, (j - 1) & 1, abort_flag));
            if (!ok)
                continue;
            tc_fence_after();
            if (warp_need && j > 0) {
#pragma unroll 1
                for (int c = 2 * half; c < 2 * half + 2; ++c) { // each warp of the pair rescales 64 of the 128 columns
                    uint32_t r[32];
                    tmem_ld32(tmem_O + lane_addr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        r[i] = __float_as_uint(__uint_as_float(r[i]) * rs);
                    tmem_st32(tmem_O + lane_addr + c * 32, r);
                }
                tmem_st_wait();
            }
            // P row -> swizzled K-major tile: 8 chunks of 8 halves, chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)
            {
                uint8_t *prow = smem + Q_BYTES + 4 * KV_BYTES + row * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    __half2 h0 = sat_half2(s[8 * c], s[8 * c + 1]), h1 = sat_half2(s[8 * c + 2], s[8 * c + 3]),
                            h2 = sat_half2(s[8 * c + 4], s[8 * c + 5]), h3 = sat_half2(s[8 * c + 6], s[8 * c + 7]);
                    *(uint4 *)(prow + (((half * 4 + c) ^ (row & 7)) << 4)) =
                        make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                }
            }
            fence_proxy_async(); // generic-proxy writes of P become visible to the tensor core's async proxy
            tc_fence_before();
            mbar_arrive(p_full);
        }
        // epilogue: O / l and lse
        if (n_tiles > 0 && ok)
            ok = mbar_wait(o_ready, (n_tiles - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        // row sum = the two halves' partial sums (same reference maximum); the P tile is free by now (all threads
        // of the pair are past the last tile when they reach the barrier) and lends its first 1 KB for the exchange
        float *lx = (float *)(smem + Q_BYTES + 4 * KV_BYTES);
        lx[half * TC_BM + row] = l;
        pair_barrier(quarter);
        l += lx[(half ^ 1) * TC_BM + row];
        const float inv = 1.f / l;
        // A warp's 32 rows x 64 fp16 columns go through a 4 KB block of the Q tile (idle now: every MMA is complete),
        // rows of 128 bytes with the 128-byte swizzle (16-byte chunk c of row r at c ^ (r & 7)), and one TMA store:
        // direct stores would write 16 bytes into each of 32 different lines per instruction.  Rows past T are clipped.
        uint8_t *blk = smem + (warp - 2) * 4096, *srow = blk + lane * 128;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
            const int c = 2 * half + cc;
            uint32_t r[32];
            if (n_tiles > 0 && ok) {
                tmem_ld32(tmem_O + lane_addr + c * 32, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 h0 = sat_half2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv),
                        h1 = sat_half2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv),
                        h2 = sat_half2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv),
                        h3 = sat_half2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
                *(uint4 *)(srow + (((cc * 4 + i) ^ (lane & 7)) << 4)) = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(&tmO, smem_u32(blk), h * TC_HD + half * 64, t0 + quarter * 32);
            bulk_commit();
            bulk_wait_read<0>(); // shared memory must outlive the store that reads it
        }
        if (t < T && half == 0)
            p.lse[(size_t)t * H + h] = m_used + log2f(l);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        tmem_dealloc(tmem_base, 256);
    if (threadIdx.x == 0 && *abort_flag)
        atomicOr(p.status, TS2_STATUS_WAIT_TIMEOUT);
}

int attention_forward_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                         int T, int H, float slope, __half *o, float *lse)
{
    static bool configured[16] = {};
    if (!configured[c.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(att_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        configured[c.device & 15] = true;
    }
    const int Q = H * TC_HD;
    CUtensorMap tmQ, tmK, tmV, tmO;
    int rc;
    if ((rc = make_tensor_map(&tmQ, q, 2, Q, T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tmK, k, 2, Q, T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tmV, v, 2, Q, T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tmO, o, 2, Q, T, Q, 32)) != TS2_OK) // output: boxes of 64 fp16 columns x 32 rows
        return rc;
    AttTcParams p;
    p.T = T;
    p.H = H;
    p.slope = slope;
    p.span_start = span_start;
    p.span_finish = span_finish;
    p.o = o;
    p.lse = lse;
    p.status = device_status_word(c.device);
    if (!p.status)
        return fail(TS2_ERR_CUDA, "attention: no device status word");
    dim3 grid((unsigned)ceil_div(T, TC_BM), (unsigned)H);
    att_fwd_tc_kernel<<<grid, TC_THREADS, FWD_SMEM, c.stream>>>(tmQ, tmK, tmV, tmO, p);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
