// tcgen05 formulation of the attention core for head width 128 (sm_100a): the two contractions
// of every (128-row block, 64-wide tile) pair run on the 5th-generation tensor cores with their
// accumulators in TMEM; operands arrive by TMA (no multicast) in 128-byte-swizzled tiles.
// Same math and the same inputs / outputs as kernels_att_mma.cu (see there for the references
// into src/gpt/compute/layer_att_reference.h and gpu_att_fp16.cu).
//
// Forward, one CTA per (128 nodes, head), 192 threads:
//   warp 0     TMA producer: Q block once, then K / V tiles through a 2-stage ring
//   warp 1     TMEM owner and MMA issuer: S = Q . K^T (128 x 64, fp32 in TMEM), later O += P . V
//   warps 2-5  softmax: thread = node row (TMEM lane), so row maximum and row sum are thread-local;
//              writes P (fp16) into a swizzled K-major shared-memory tile for the second MMA and
//              rescales O in TMEM only when a row's maximum grew by more than 8 (2^8 headroom in
//              fp16 P and fp32 sums), which keeps tcgen05.ld/st of O off the common path
// The zero "sink" vector of the reference is the initial state m = 0, l = 1.
// Two CTAs fit an SM (112 KB shared memory, 256 TMEM columns each), so one CTA's softmax overlaps
// the other's MMAs.  Every wait is bounded (see mbar_wait); a give-up raises the status word.
#include "kernels.cuh"
#include "gemm.cuh"
#include "fast_types.cuh"
#include <cuda.h>

namespace ts2 {

static constexpr int TC_BM = 128;  // node rows per CTA
static constexpr int TC_BN = 64;   // keys per tile
static constexpr int TC_HD = 128;  // head width
static constexpr int TC_THREADS = 192;
static constexpr int Q_BYTES = TC_BM * TC_HD * 2;   // 32 KB: two 128-byte-wide atoms of 128 rows
static constexpr int KV_BYTES = TC_BN * TC_HD * 2;  // 16 KB: two atoms of 64 rows
static constexpr int P_BYTES = TC_BM * TC_BN * 2;   // 16 KB: one atom of 128 rows
// 112 KB of tiles + 128 B of barriers: two CTAs per SM (2 x (114816 + 1024 reserved) <= 228 KB)
static constexpr int FWD_SMEM = Q_BYTES + 2 * 2 * KV_BYTES + P_BYTES + 128;

__host__ __device__ inline float att_dot_scale_tc() { return sqrtf(1.0f / 128) * (0.5f / 0.693147f) * 1.0f; }

struct AttTcParams {
    int T, H;
    float slope;
    const int *span_start, *span_finish;
    __half *o;
    float *lse;
    int32_t *status;
};

__global__ void __launch_bounds__(TC_THREADS)
    att_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const AttTcParams p)
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
    const uint32_t q_full = smem_u32(bars), kv_full0 = smem_u32(bars + 1), kv_empty0 = smem_u32(bars + 3), s_full = smem_u32(bars + 5),
                   p_full = smem_u32(bars + 6), o_ready = smem_u32(bars + 7);
    uint32_t *tmem_slot = (uint32_t *)(bars + 8);
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
            mbar_init(kv_full0 + 8 * s, 1);
            mbar_init(kv_empty0 + 8 * s, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_full, 128);
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
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + TC_BN;
    const int lo = s_lo, hi = s_hi;
    const int tile0 = hi >= lo ? lo / TC_BN : 0, tile1 = hi >= lo ? hi / TC_BN : -1; // no keys: no tiles
    const int col0 = h * TC_HD;

    if (warp == 0) {
        if (lane == 0 && tile1 >= tile0) {
            mbar_arrive_expect_tx(q_full, Q_BYTES);
            tma_load_2d(sQ, &tmQ, q_full, col0, t0);
            tma_load_2d(sQ + Q_BYTES / 2, &tmQ, q_full, col0 + 64, t0);
            for (int tile = tile0, j = 0; tile <= tile1; ++tile, ++j) {
                const int st = j & 1;
                if (!mbar_wait(kv_empty0 + 8 * st, ((j >> 1) & 1) ^ 1, abort_flag))
                    break;
                const uint32_t fb = kv_full0 + 8 * st;
                mbar_arrive_expect_tx(fb, 2 * KV_BYTES);
                const uint32_t dk = sK + st * KV_BYTES, dv = sV + st * KV_BYTES;
                tma_load_2d(dk, &tmK, fb, col0, tile * TC_BN);
                tma_load_2d(dk + KV_BYTES / 2, &tmK, fb, col0 + 64, tile * TC_BN);
                tma_load_2d(dv, &tmV, fb, col0, tile * TC_BN);
                tma_load_2d(dv + KV_BYTES / 2, &tmV, fb, col0 + 64, tile * TC_BN);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && tile1 >= tile0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(TC_BN, false, false);
            constexpr uint32_t idesc_pv = umma_idesc_f16(TC_HD, false, true);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            for (int tile = tile0, j = 0; tile <= tile1 && ok; ++tile, ++j) {
                const int st = j & 1;
                if (!mbar_wait(kv_full0 + 8 * st, (j >> 1) & 1, abort_flag))
                    break;
                tc_fence_after();
                // S = Q . K^T: 8 steps of 16 head dims; Q and K tiles are two 64-dim atoms each
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t a = umma_smem_desc(sQ + (k >> 2) * (Q_BYTES / 2) + (k & 3) * 32, 16, 1024);
                    const uint64_t b = umma_smem_desc(sK + st * KV_BYTES + (k >> 2) * (KV_BYTES / 2) + (k & 3) * 32, 16, 1024);
                    umma_f16(tmem_S, a, b, idesc_qk, k > 0 ? 1u : 0u);
                }
                tc_commit(s_full);
                if (!mbar_wait(p_full, j & 1, abort_flag))
                    break;
                tc_fence_after();
                // O += P . V: 4 steps of 16 keys; V tile is MN-major for this product (dims contiguous)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t a = umma_smem_desc(sP + k * 32, 16, 1024);
                    const uint64_t b = umma_smem_desc(sV + st * KV_BYTES + k * 16 * 128, KV_BYTES / 2, 1024);
                    umma_f16(tmem_O, a, b, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(kv_empty0 + 8 * st);
                tc_commit(o_ready);
            }
        }
    } else {
        // ------------------------------ softmax warps -----------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane, t = t0 + row;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int st_row = t < T ? p.span_start[t] : 0, fi_row = t < T ? p.span_finish[t] : -1;
        const float ds = att_dot_scale_tc(), slope = p.slope;
        float m_used = 0.f, l = 1.f; // the zero vector of weight 2^-m
        bool ok = true;
        for (int tile = tile0, j = 0; tile <= tile1; ++tile, ++j) {
            if (!mbar_wait(s_full, j & 1, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();
            float s[TC_BN];
            {
                uint32_t r0[32], r1[32];
                tmem_ld32(tmem_S + lane_addr, r0);
                tmem_ld32(tmem_S + lane_addr + 32, r1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    s[i] = __uint_as_float(r0[i]);
                    s[32 + i] = __uint_as_float(r1[i]);
                }
            }
            const int key0 = tile * TC_BN;
            // four independent chains keep the single warp per scheduler busy
            float mx4[4] = {m_used, m_used, m_used, m_used};
            const bool inside = key0 >= st_row && key0 + TC_BN - 1 <= fi_row; // whole tile visible from this row
            if (slope == 0.f && inside) {
#pragma unroll
                for (int i = 0; i < TC_BN; ++i) {
                    s[i] *= ds;
                    mx4[i & 3] = fmaxf(mx4[i & 3], s[i]);
                }
            } else {
                const float base = slope * (float)(t - key0);
#pragma unroll
                for (int i = 0; i < TC_BN; ++i) {
                    const int key = key0 + i;
                    float x = fmaf(s[i], ds, fmaf(slope, (float)i, -base));
                    x = (key >= st_row && key <= fi_row) ? x : -INFINITY;
                    s[i] = x;
                    mx4[i & 3] = fmaxf(mx4[i & 3], x);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
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
#pragma unroll
            for (int i = 0; i < TC_BN; ++i) {
                float pv;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pv) : "f"(s[i] - m_used));
                s[i] = pv;
                sum4[i & 3] += pv;
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // the previous P . V must have finished before P is overwritten or O is touched
            if (j > 0 && !mbar_wait(o_ready, (j - 1) & 1, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (warp_need && j > 0) {
#pragma unroll 1
                for (int c = 0; c < TC_HD / 32; ++c) {
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
                for (int c = 0; c < 8; ++c) {
                    __half2 h0 = __floats2half2_rn(s[8 * c], s[8 * c + 1]), h1 = __floats2half2_rn(s[8 * c + 2], s[8 * c + 3]),
                            h2 = __floats2half2_rn(s[8 * c + 4], s[8 * c + 5]), h3 = __floats2half2_rn(s[8 * c + 6], s[8 * c + 7]);
                    *(uint4 *)(prow + ((c ^ (row & 7)) << 4)) = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                }
            }
            fence_proxy_async(); // generic-proxy writes of P become visible to the tensor core's async proxy
            tc_fence_before();
            mbar_arrive(p_full);
        }
        // epilogue: O / l and lse
        const int n_tiles = tile1 - tile0 + 1;
        if (n_tiles > 0 && ok)
            ok = mbar_wait(o_ready, (n_tiles - 1) & 1, abort_flag);
        tc_fence_after();
        const float inv = 1.f / l;
        __half *dst = p.o + (size_t)t * (H * TC_HD) + h * TC_HD;
#pragma unroll 1
        for (int c = 0; c < TC_HD / 32; ++c) {
            uint32_t r[32];
            if (n_tiles > 0 && ok) {
                tmem_ld32(tmem_O + lane_addr + c * 32, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = 0u;
            }
            if (t < T) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __half2 h0 = __floats2half2_rn(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv),
                            h1 = __floats2half2_rn(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv),
                            h2 = __floats2half2_rn(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv),
                            h3 = __floats2half2_rn(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv);
                    *(uint4 *)(dst + c * 32 + i * 8) = make_uint4(*(uint32_t *)&h0, *(uint32_t *)&h1, *(uint32_t *)&h2, *(uint32_t *)&h3);
                }
            }
        }
        if (t < T)
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
    CUtensorMap tmQ, tmK, tmV;
    int rc;
    if ((rc = make_tensor_map(&tmQ, q, 2, Q, T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tmK, k, 2, Q, T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tmV, v, 2, Q, T, Q, TC_BN)) != TS2_OK)
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
    att_fwd_tc_kernel<<<grid, TC_THREADS, FWD_SMEM, c.stream>>>(tmQ, tmK, tmV, p);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
