// tcgen05 attention backward for head width 128 (sm_100a): dQ, the packing of the per-node records, and the entry
// point of the backward pass (dK and dV come from kernels_att_bwd_kv_tc.cu).  Same math, inputs and outputs as the
// mma.sync formulation in kernels_att_mma.cu (see there for the references into
// src/gpt/compute/layer_att_reference.h and gpu_att_fp16.cu).
//
// dQ: a CTA owns 256 resident nodes (Q and dO rows) as two blocks of 128, and streams 64-key tiles of K and V once
// for both blocks (half the L2 traffic of one block per CTA):
//   first MMAs   S = Q . K^T  and  dP = dO . V^T               128 x 64 each, fp32 in TMEM
//   compute      G = P (dP - dscale) c2                        fp16, left in TMEM in place of the dP values
//   second MMA   dQ += G . K                                   128 x 128 in TMEM, G the TMEM A operand, K read MN-major
// Each block has its own MMA issuer thread, its own 8 compute warps (two per TMEM lane quarter, 32 of the tile's 64
// keys each) and its own 256 TMEM columns.  20 warps: TMA producer, 2 MMA issuers, 1 idle, 16 compute.  (One block per
// CTA with two S / dP pairs, the structure of the dK / dV kernel, was measured slower here: twice the CTAs and twice
// the streamed bytes.)  Every wait is bounded (see mbar_wait); a give-up raises the status word.
#include "att_tc.cuh"
#include <mutex>

namespace ts2 {

static constexpr int BW_ROWS = 2 * TC_BM;
static constexpr int BW_THREADS = 128 + 2 * 256;

struct AttBwdParams {
    int T, H;
    float slope;
    const int *span_start, *span_finish;
    const float *lse, *dscale;
    void *out; // dq: fp32 or fp16 [T][128 H]
    int32_t *status;
};

struct BwdLayout {
    static constexpr int STAGES = 3;
    static constexpr int A1_OFF = 0;
    static constexpr int A2_OFF = A1_OFF + 2 * Q_BYTES;
    static constexpr int RES_BYTES = 4 * Q_BYTES; // Q and dO of both blocks
    static constexpr int STAGE_OFF = RES_BYTES;
    static constexpr int STAGE_BYTES = 2 * KV_BYTES;
    static constexpr int BAR_OFF = STAGE_OFF + STAGES * STAGE_BYTES;
    static constexpr int SMEM = BAR_OFF + 256;
};
static_assert(BwdLayout::SMEM <= 232448, "shared memory budget");

// {-lse, -dscale * c2, start, finish - start} per (head, node); nodes past T and nodes with an empty span get a
// start no key index reaches
__global__ void att_pack_meta_kernel(const float *__restrict__ lse, const float *__restrict__ dscale, const int *__restrict__ span_start,
                                     const int *__restrict__ span_finish, int T, int Tpad, int H, float c2, float4 *__restrict__ meta)
{
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= Tpad * H)
        return;
    const int h = idx / Tpad, t = idx - h * Tpad;
    float4 m = make_float4(0.f, 0.f, __int_as_float(0x40000000), __int_as_float(0));
    if (t < T) {
        const int st = span_start[t], fi = span_finish[t];
        if (fi >= st)
            m = make_float4(-lse[(size_t)t * H + h], -dscale[(size_t)t * H + h] * c2, __int_as_float(st), __int_as_float(fi - st));
    }
    meta[idx] = m;
}

// OUT16: dQ is written as fp16 (what the engine feeds its next kernel with) instead of fp32
template <bool OUT16>
__global__ void __launch_bounds__(BW_THREADS, 1)
    att_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmA2,
                      const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmB2,
                      const __grid_constant__ CUtensorMap tmOut, const AttBwdParams p)
{
    using L = BwdLayout;
    constexpr int STAGES = L::STAGES;
    extern __shared__ __align__(1024) uint8_t att_bwd_smem[];
    uint8_t *smem = att_bwd_smem;
    if (smem_u32(smem) & 1023) { // the swizzled tiles need a 1024-byte aligned base; refuse instead of computing garbage
        if (threadIdx.x == 0)
            atomicOr(p.status, TS2_STATUS_BAD_ARG);
        return;
    }
    const uint32_t sA1 = smem_u32(smem) + L::A1_OFF, sA2 = smem_u32(smem) + L::A2_OFF, sStage = smem_u32(smem) + L::STAGE_OFF;
    uint64_t *bars = (uint64_t *)(smem + L::BAR_OFF);
    const uint32_t res_full = smem_u32(bars), st_full0 = smem_u32(bars + 1), st_empty0 = smem_u32(bars + 4), s_full0 = smem_u32(bars + 7),
                   g_full0 = smem_u32(bars + 9), acc_ready0 = smem_u32(bars + 11);
    uint32_t *tmem_slot = (uint32_t *)(bars + 13);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    int *rng = (int *)(tmem_slot + 2); // lo, hi of block 0; lo, hi of block 1

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = p.T, H = p.H, h = blockIdx.y, r0 = blockIdx.x * BW_ROWS;

    // range of streamed rows each block has to visit
    if (threadIdx.x < 4)
        rng[threadIdx.x] = (threadIdx.x & 1) ? -1 : 0x7fffffff;
    __syncthreads();
    if (threadIdx.x < BW_ROWS && r0 + (int)threadIdx.x < T) {
        const int r = r0 + threadIdx.x, b = threadIdx.x >> 7;
        const int a = p.span_start[r], e = p.span_finish[r];
        if (e >= a) {
            atomicMin(&rng[2 * b], a);
            atomicMax(&rng[2 * b + 1], e);
        }
    }
    if (threadIdx.x == 0) {
        mbar_init(res_full, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(st_full0 + 8 * s, 1);
            mbar_init(st_empty0 + 8 * s, 2); // both MMA issuers release a stage
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full0 + 8 * b, 1);
            mbar_init(g_full0 + 8 * b, 256);
            mbar_init(acc_ready0 + 8 * b, 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA1);
        prefetch_tmap(&tmB1);
        prefetch_tmap(&tmB2);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // tile ranges: per block [tlo, thi] (empty: tlo > thi), and their union [u0, u0 + n)
    const bool any0 = rng[1] >= rng[0], any1 = rng[3] >= rng[2];
    const int tlo0 = any0 ? rng[0] / TC_BN : 0x3fffffff, thi0 = any0 ? rng[1] / TC_BN : -1;
    const int tlo1 = any1 ? rng[2] / TC_BN : 0x3fffffff, thi1 = any1 ? rng[3] / TC_BN : -1;
    const int u0 = min(tlo0, tlo1), u1 = max(thi0, thi1);
    const int n = u1 >= u0 ? u1 - u0 + 1 : 0;
    const int col0 = h * TC_HD;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && n > 0) {
            mbar_arrive_expect_tx(res_full, L::RES_BYTES);
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                tma_load_2d(sA1 + b * Q_BYTES, &tmA1, res_full, col0, r0 + b * TC_BM);
                tma_load_2d(sA1 + b * Q_BYTES + Q_BYTES / 2, &tmA1, res_full, col0 + 64, r0 + b * TC_BM);
                tma_load_2d(sA2 + b * Q_BYTES, &tmA2, res_full, col0, r0 + b * TC_BM);
                tma_load_2d(sA2 + b * Q_BYTES + Q_BYTES / 2, &tmA2, res_full, col0 + 64, r0 + b * TC_BM);
            }
            for (int j = 0; j < n; ++j) {
                const int st = j % STAGES, row = (u0 + j) * TC_BN;
                if (!mbar_wait(st_empty0 + 8 * st, ((j / STAGES) & 1) ^ 1, abort_flag))
                    break;
                const uint32_t fb = st_full0 + 8 * st;
                mbar_arrive_expect_tx(fb, L::STAGE_BYTES);
                const uint32_t d1 = sStage + st * L::STAGE_BYTES, d2 = d1 + KV_BYTES;
                tma_load_2d(d1, &tmB1, fb, col0, row);
                tma_load_2d(d1 + KV_BYTES / 2, &tmB1, fb, col0 + 64, row);
                tma_load_2d(d2, &tmB2, fb, col0, row);
                tma_load_2d(d2 + KV_BYTES / 2, &tmB2, fb, col0 + 64, row);
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------ MMA issuer of block b ---------------------
        if (lane == 0 && n > 0) {
            const int b = warp - 1, my_lo = b ? tlo1 : tlo0, my_hi = b ? thi1 : thi0;
            constexpr uint32_t idesc_s = umma_idesc_f16(TC_BN, false, false);
            constexpr uint32_t idesc_acc = umma_idesc_f16(TC_HD, false, true);
            const uint32_t tS = tmem_base + b * 256, tDP = tS + TC_BN, tACC = tS + 2 * TC_BN;
            const uint64_t dA1 = umma_smem_desc(sA1 + b * Q_BYTES, 16, 1024), dA2 = umma_smem_desc(sA2 + b * Q_BYTES, 16, 1024);
            const uint32_t s_full = s_full0 + 8 * b, g_full = g_full0 + 8 * b, acc_ready = acc_ready0 + 8 * b;
            bool ok = mbar_wait(res_full, 0, abort_flag);
            // The two blocks run the same cycle (first products, compute, accumulating product); started together they stay
            // in step, the tensor pipe idle while both compute and the compute warps idle while both multiply.  Block 1
            // therefore starts when block 0's first products are done (block 0 then computes), after which the shared
            // tensor pipe keeps the two out of phase.
            if (ok && b == 1 && any0)
                ok = mbar_wait(s_full0, 0, abort_flag);
            int k = 0; // tiles of this block so far
            for (int j = 0; j < n && ok; ++j) {
                const int st = j % STAGES, tile = u0 + j;
                // also a block that skips the tile waits for it, so that it never runs a ring phase ahead
                if (!mbar_wait(st_full0 + 8 * st, (j / STAGES) & 1, abort_flag))
                    break;
                if (tile >= my_lo && tile <= my_hi) {
                    tc_fence_after();
                    const uint32_t b1 = sStage + st * L::STAGE_BYTES, b2 = b1 + KV_BYTES;
                    const uint64_t dB1 = umma_smem_desc(b1, 16, 1024), dB2 = umma_smem_desc(b2, 16, 1024);
                    // 8 steps of 16 head dims; operands are two 64-dim atoms each
                    umma_f16_x4(tS, dA1, dB1, idesc_s, 0u, 2u, 2u);
                    umma_f16_x4(tS, dA1 + (Q_BYTES / 2 >> 4), dB1 + (KV_BYTES / 2 >> 4), idesc_s, 1u, 2u, 2u);
                    // the dP columns still hold G of the previous tile, the A operand of its second MMA: that MMA must be
                    // complete before these may write there (it was issued eight MMAs ago, so this wait is normally over
                    // before it starts)
                    if (k > 0 && !mbar_wait(acc_ready, (k - 1) & 1, abort_flag))
                        break;
                    umma_f16_x4(tDP, dA2, dB2, idesc_s, 0u, 2u, 2u);
                    umma_f16_x4(tDP, dA2 + (Q_BYTES / 2 >> 4), dB2 + (KV_BYTES / 2 >> 4), idesc_s, 1u, 2u, 2u);
                    tc_commit(s_full);
                    if (!mbar_wait(g_full, k & 1, abort_flag))
                        break;
                    tc_fence_after();
                    // dQ += G . K: 4 steps of 16 keys.  G is read from tensor memory, where the compute warps left it in the dP
                    // columns (in place of the dP values they consumed): fp16 pairs, keys 0-15 in columns 0-7, 16-31 in
                    // 8-15, 32-47 in 32-39, 48-63 in 40-47.  The K tile is read MN-major (its 128 columns are the output
                    // columns), 16 rows = 2048 bytes per step.
                    const uint64_t dB = umma_smem_desc(b1, KV_BYTES / 2, 1024);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_f16_ts(tACC, tDP + (kk >> 1) * 32 + (kk & 1) * 8, dB + (uint64_t)(kk * 128), idesc_acc, (k > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(acc_ready);
                    ++k;
                }
                tc_commit(st_empty0 + 8 * st);
            }
        }
    } else if (warp >= 4) {
        // ------------------------------ compute warps of block b ------------------
        const int b = (warp - 4) >> 3, half = ((warp - 4) & 7) >> 2, quarter = warp & 3;
        const int my_lo = b ? tlo1 : tlo0, my_hi = b ? thi1 : thi0;
        const int row = quarter * 32 + lane;
        const int rr = r0 + b * TC_BM + row; // node of this thread
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t tS = tmem_base + b * 256 + lane_addr + half * 32, tDP = tS + TC_BN, tACC = tmem_base + b * 256 + 2 * TC_BN + lane_addr;
        const uint32_t s_full = s_full0 + 8 * b, g_full = g_full0 + 8 * b, acc_ready = acc_ready0 + 8 * b;
        const float ds = att_dot_scale_tc(), c2 = ds * 0.693147f, slope = p.slope;
        int st_row = 0, len_row = -1;
        float nlse_row = 0.f, ndc_row = 0.f;
        if (rr < T) {
            st_row = p.span_start[rr];
            len_row = p.span_finish[rr] - st_row;
            nlse_row = -p.lse[(size_t)rr * H + h];
            ndc_row = -p.dscale[(size_t)rr * H + h] * c2;
        }
        bool ok = true;
        int k = 0;
        for (int j = 0; j < n; ++j) {
            const int tile = u0 + j;
            if (tile < my_lo || tile > my_hi)
                continue;
            // s_full also says that the previous second MMA of this block is done with G: its issuer commits in order
            ok = __all_sync(0xffffffffu, mbar_wait(s_full, k & 1, abort_flag));
            if (!ok)
                break;
            tc_fence_after();
            const int c0 = tile * TC_BN + half * 32; // first key of this thread's columns
            // two passes of 16 columns: few enough live registers that the compiler can interleave the per-element
            // chains (fma -> ex2 -> select -> fma -> multiply -> convert)
#pragma unroll
            for (int q16 = 0; q16 < 2; ++q16) {
                uint32_t rs[16], rp[16];
                tmem_ld16(tS + q16 * 16, rs);
                tmem_ld16(tDP + q16 * 16, rp);
                tmem_ld_wait();
                float g[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int c = c0 + q16 * 16 + i;
                    float off = nlse_row;
                    const bool valid = (unsigned)(c - st_row) <= (unsigned)len_row && len_row >= 0;
                    if (slope != 0.f)
                        off -= slope * (float)(rr - c);
                    float w;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(fmaf(__uint_as_float(rs[i]), ds, off)));
                    w = valid ? w : 0.f;
                    g[i] = w * fmaf(__uint_as_float(rp[i]), c2, ndc_row);
                }
                // G goes where this thread's dP values were (its own lane, its own columns): 16 fp16 values = 8 columns
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __half2 hv = sat_half2(g[2 * i], g[2 * i + 1]);
                    packed[i] = *(const uint32_t *)&hv;
                }
                tmem_st8(tDP + q16 * 8, packed);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(g_full);
            ++k;
        }
        // epilogue: this thread's 64 columns of the accumulator row -> fp32 output
        if (k > 0 && ok)
            ok = mbar_wait(acc_ready, (k - 1) & 1, abort_flag);
        // the staging blocks below lie in the resident tile, which the producer fills for both blocks whenever the CTA
        // has any tile: a block without tiles of its own must see that copy landed before it writes there
        if (n > 0 && ok)
            ok = mbar_wait(res_full, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        // A warp's 32 rows x 32 columns go through a 4 KB block of the block's own resident A1 tile (idle now: every MMA
        // of this block is complete), rows of 128 bytes with the 128-byte swizzle (16-byte chunk c of row r at
        // c ^ (r & 7)), and one TMA store: direct stores would write 16 bytes into each of 32 different lines per
        // instruction.  Rows past T are clipped by the TMA unit.
        uint8_t *blk = smem + L::A1_OFF + b * Q_BYTES + ((warp - 4) & 7) * 4096, *srow = blk + lane * 128;
        if constexpr (OUT16) { // this warp's 64 columns as fp16: one block of 32 rows x 128 bytes, one store
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t r[32];
                if (k > 0 && ok) {
                    tmem_ld32(tACC + (2 * half + cc) * 32, r);
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
                tma_store_2d(&tmOut, smem_u32(blk), col0 + half * 64, r0 + b * TC_BM + quarter * 32);
                bulk_commit();
            }
        } else
#pragma unroll 1
        for (int c = 2 * half; c < 2 * half + 2; ++c) {
            uint32_t r[32];
            if (k > 0 && ok) {
                tmem_ld32(tACC + c * 32, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    r[i] = 0u;
            }
            if (lane == 0)
                bulk_wait_read<0>(); // the previous store has read the block
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i)
                *(uint4 *)(srow + ((i ^ (lane & 7)) << 4)) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(&tmOut, smem_u32(blk), col0 + c * 32, r0 + b * TC_BM + quarter * 32);
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

// a1 = Q, a2 = dO (resident), b1 = K, b2 = V (streamed)
static int launch_bwd_dq(const Ctx &c, const __half *a1, const __half *a2, const __half *b1, const __half *b2, const AttBwdParams &p,
                         bool out16)
{
    auto kern = out16 ? att_bwd_dq_tc_kernel<true> : att_bwd_dq_tc_kernel<false>;
    static bool configured[16] = {};
    if (!configured[c.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(att_bwd_dq_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdLayout::SMEM));
        TS2_CUDA(cudaFuncSetAttribute(att_bwd_dq_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdLayout::SMEM));
        configured[c.device & 15] = true;
    }
    const int Q = p.H * TC_HD;
    CUtensorMap tA1, tA2, tB1, tB2, tOut;
    int rc;
    if ((rc = make_tensor_map(&tA1, a1, 2, Q, p.T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tA2, a2, 2, Q, p.T, Q, TC_BM)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tB1, b1, 2, Q, p.T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tB2, b2, 2, Q, p.T, Q, TC_BN)) != TS2_OK)
        return rc;
    if ((rc = make_tensor_map(&tOut, p.out, out16 ? 2 : 4, Q, p.T, Q, 32)) != TS2_OK) // boxes of 128 bytes x 32 rows
        return rc;
    dim3 grid((unsigned)ceil_div(p.T, BW_ROWS), (unsigned)p.H);
    kern<<<grid, BW_THREADS, BwdLayout::SMEM, c.stream>>>(tA1, tA2, tB1, tB2, tOut, p);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// per-device buffer of the packed per-node quantities, grown on demand (never inside a steady-state step:
// the node count of a model is fixed)
static int meta_buffer(int device, size_t bytes, float4 **out)
{
    static std::mutex mu;
    static float4 *buf[16] = {};
    static size_t cap[16] = {};
    std::lock_guard<std::mutex> lock(mu);
    const int d = device & 15;
    if (cap[d] < bytes) {
        if (buf[d]) {
            TS2_CUDA(cudaDeviceSynchronize());
            TS2_CUDA(cudaFree(buf[d]));
            buf[d] = nullptr;
            cap[d] = 0;
        }
        TS2_CUDA(cudaMalloc(&buf[d], bytes));
        cap[d] = bytes;
    }
    *out = buf[d];
    return TS2_OK;
}

int attention_backward_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                          const float *dscale, const int *span_start, const int *span_finish, const int *rev_first, const int *rev_last,
                          int T, int H, float slope, void *dq, void *dk, void *dv, bool grads16)
{
    AttBwdParams p;
    p.T = T;
    p.H = H;
    const int Tpad = (int)ceil_div(T, TC_BN) * TC_BN;
    p.slope = slope;
    p.span_start = span_start;
    p.span_finish = span_finish;
    p.lse = lse;
    p.dscale = dscale;
    p.status = device_status_word(c.device);
    if (!p.status)
        return fail(TS2_ERR_CUDA, "attention: no device status word");
    int rc;
    float4 *meta = nullptr;
    if ((rc = meta_buffer(c.device, (size_t)Tpad * H * sizeof(float4), &meta)) != TS2_OK)
        return rc;
    {
        const int total = Tpad * H;
        att_pack_meta_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, c.stream>>>(lse, dscale, span_start, span_finish, T, Tpad, H,
                                                                                  att_dot_scale_tc() * 0.693147f, meta);
        TS2_CHECK_LAUNCH();
    }
    p.out = dq;
    if ((rc = launch_bwd_dq(c, q, dout, k, v, p, grads16)) != TS2_OK)
        return rc;
    // dK and dV from one kernel that shares S and the streamed tiles (kernels_att_bwd_kv_tc.cu)
    return attention_backward_kv_tc(c, q, k, v, dout, meta, Tpad, rev_first, rev_last, T, H, slope, dk, dv, grads16);
}

} // namespace ts2
