// Tensor-core formulation of the attention core (forward, dQ, dK/dV) for head width 128
// over one inclusive key span per node.  Same math as kernels_att.cu (which follows
// ComputeValLookup / GradQ / GradK, src/gpt/compute/layer_att_reference.h:41-212) and the
// same role as the reference's Fp16Att / Fp16AttGradQ / Fp16AttGradKV
// (src/gpt/compute/gpu_att_fp16.cu:41-215, gpu_att_fp16.cuh:60-358), organised differently:
// 64-row blocks against 64-wide tiles of the other side, fp16 mma.sync m16n8k16 with fp32
// accumulation, cp.async double buffering of the streamed tiles, 16-byte xor-swizzled
// shared-memory rows read with ldmatrix, online base-2 softmax with the zero "sink" vector
// folded into the initial state (m = 0, l = 1).
//
// A block's key range is [min start, max finish] of its rows; the per-element mask
// start[row] <= key <= finish[row] does the rest, so any one-span-per-node graph is handled.
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int BLK = 64;           // rows per block and per streamed tile
static constexpr int HD = 128;           // head width
static constexpr int TILE_BYTES = BLK * HD * 2;
static constexpr int ATT_THREADS = 128;

__host__ __device__ inline float att_dot_scale_mma() { return sqrtf(1.0f / 128) * (0.5f / 0.693147f) * 1.0f; }

// ---- small PTX wrappers ----------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid)
{
    const int sz = valid ? 16 : 0; // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b)
{
    __half2 h = sat_half2(a, b);
    return *(uint32_t *)&h;
}

// shared-memory tile [64 rows][128 halves]: row pitch 256 B, 16-byte chunk c of row r stored at c ^ (r & 7)
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) { return base + row * 256 + ((chunk ^ (row & 7)) << 4); }

// rows [row0, row0+64) x head h of a [T][Q] fp16 array -> tile; rows outside [0, T) are zero
__device__ __forceinline__ void load_tile(uint32_t base, const __half *__restrict__ src, int row0, int T, int Q, int h)
{
#pragma unroll
    for (int i = 0; i < (BLK * 16) / ATT_THREADS; ++i) {
        const int idx = threadIdx.x + i * ATT_THREADS;
        const int r = idx >> 4, c = idx & 15;
        const int row = row0 + r;
        const bool ok = row >= 0 && row < T;
        const __half *p = src + (size_t)(ok ? row : 0) * Q + h * HD + c * 8;
        cp_async16(tile_addr(base, r, c), p, ok);
    }
}

// A fragments (16 rows x 16 k) of a row-major tile: rows r0.., k block kb (16 halves)
__device__ __forceinline__ void load_a(uint32_t base, int r0, int kb, uint32_t (&a)[4])
{
    const int lane = threadIdx.x & 31;
    ldsm_x4(tile_addr(base, r0 + (lane & 15), kb * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
}
// B fragments for X . Y^T with Y row-major [n][k]: two n-tiles (16 rows of Y starting at n0), k block kb.
// b[0], b[1]: n-tile n0..n0+7; b[2], b[3]: n-tile n0+8..n0+15
__device__ __forceinline__ void load_b_nt(uint32_t base, int n0, int kb, uint32_t (&b)[4])
{
    const int lane = threadIdx.x & 31;
    ldsm_x4(tile_addr(base, n0 + (lane & 7) + ((lane >> 4) << 3), kb * 2 + ((lane >> 3) & 1)), b[0], b[1], b[2], b[3]);
}
// B fragments for X . Y with Y row-major [k][n]: k block k0..k0+15 (rows of Y), two n-tiles (16 columns from nb*16)
__device__ __forceinline__ void load_b_nn(uint32_t base, int k0, int nb, uint32_t (&b)[4])
{
    const int lane = threadIdx.x & 31;
    ldsm_x4_t(tile_addr(base, k0 + (lane & 7) + (((lane >> 3) & 1) << 3), nb * 2 + (lane >> 4)), b[0], b[1], b[2], b[3]);
}

// block-wide min/max of per-row span bounds -> tile range to visit
__device__ __forceinline__ void block_range(int lo, int hi, int *s_lo, int *s_hi, int &out_lo, int &out_hi)
{
    if (threadIdx.x == 0) {
        *s_lo = 0x7fffffff;
        *s_hi = -1;
    }
    __syncthreads();
    if (hi >= lo) {
        atomicMin(s_lo, lo);
        atomicMax(s_hi, hi);
    }
    __syncthreads();
    out_lo = *s_lo;
    out_hi = *s_hi;
}

// S (16 x 64 per warp) = A-tile rows [r0, r0+16) . B-tile^T, both [64][128] row-major tiles
__device__ __forceinline__ void gemm_nt_16x64(uint32_t a_base, int r0, uint32_t b_base, float (&s)[8][4])
{
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            s[nt][i] = 0.f;
#pragma unroll
    for (int kb = 0; kb < HD / 16; ++kb) {
        uint32_t a[4];
        load_a(a_base, r0, kb, a);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            uint32_t b[4];
            load_b_nt(b_base, np * 16, kb, b);
            mma16816(s[2 * np], a, b[0], b[1]);
            mma16816(s[2 * np + 1], a, b[2], b[3]);
        }
    }
}

// acc (16 x 128 per warp) += P (16 x 64, fp16 A fragments built from s) . B-tile ([64][128] row-major)
__device__ __forceinline__ void gemm_nn_16x128(const float (&s)[8][4], uint32_t b_base, float (&acc)[16][4])
{
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
        uint32_t a[4];
        a[0] = pack_half2(s[2 * kb][0], s[2 * kb][1]);
        a[1] = pack_half2(s[2 * kb][2], s[2 * kb][3]);
        a[2] = pack_half2(s[2 * kb + 1][0], s[2 * kb + 1][1]);
        a[3] = pack_half2(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            uint32_t b[4];
            load_b_nn(b_base, kb * 16, nb, b);
            mma16816(acc[2 * nb], a, b[0], b[1]);
            mma16816(acc[2 * nb + 1], a, b[2], b[3]);
        }
    }
}

// ---------------------------------------------------------------------------------------
// forward: grid (query blocks, heads)
__global__ void __launch_bounds__(ATT_THREADS)
    att_fwd_mma_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                       const int *__restrict__ span_start, const int *__restrict__ span_finish, int T, int H, float slope,
                       __half *__restrict__ o, float *__restrict__ lse)
{
    extern __shared__ __align__(1024) uint8_t att_smem[];
    __shared__ int s_lo, s_hi;
    const uint32_t sQ = smem_u32(att_smem), sK = sQ + TILE_BYTES, sV = sK + 2 * TILE_BYTES; // K and V double-buffered
    const int Q = H * HD, h = blockIdx.y, t0 = blockIdx.x * BLK;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float ds = att_dot_scale_mma();

    // per-thread rows: t0 + warp*16 + lane/4 (+8)
    const int r_lo = warp * 16 + (lane >> 2);
    int st[2], fi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int t = t0 + r_lo + 8 * i;
        st[i] = t < T ? span_start[t] : 0;
        fi[i] = t < T ? span_finish[t] : -1;
    }
    int lo, hi;
    {
        // every row of the block contributes once: threads with lane%4 == 0 own rows r_lo and r_lo+8
        int mylo = 0x7fffffff, myhi = -1;
        if ((lane & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (fi[i] >= st[i]) {
                    mylo = min(mylo, st[i]);
                    myhi = max(myhi, fi[i]);
                }
        }
        block_range(mylo, myhi, &s_lo, &s_hi, lo, hi);
    }
    float m[2] = {0.f, 0.f}, l[2] = {1.f, 1.f};
    float acc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            acc[n][i] = 0.f;

    if (hi >= lo) {
        const int tile0 = lo / BLK, tile1 = hi / BLK;
        load_tile(sQ, q, t0, T, Q, h);
        load_tile(sK, k, tile0 * BLK, T, Q, h);
        load_tile(sV, v, tile0 * BLK, T, Q, h);
        cp_async_commit();
        for (int tile = tile0; tile <= tile1; ++tile) {
            const int buf = (tile - tile0) & 1;
            if (tile < tile1) {
                load_tile(sK + (buf ^ 1) * TILE_BYTES, k, (tile + 1) * BLK, T, Q, h);
                load_tile(sV + (buf ^ 1) * TILE_BYTES, v, (tile + 1) * BLK, T, Q, h);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            float s[8][4];
            gemm_nt_16x64(sQ, warp * 16, sK + buf * TILE_BYTES, s);
            // scale, ALiBi, mask, running maximum
            const int key0 = tile * BLK + (lane & 3) * 2;
            float mx[2] = {m[0], m[1]};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1, key = key0 + nt * 8 + (i & 1);
                    float x = s[nt][i] * ds - slope * (float)(t0 + r_lo + 8 * rr - key);
                    x = (key >= st[rr] && key <= fi[rr]) ? x : -INFINITY;
                    s[nt][i] = x;
                    mx[rr] = fmaxf(mx[rr], x);
                }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            }
            float rs[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                rs[rr] = exp2f(m[rr] - mx[rr]);
                m[rr] = mx[rr];
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float p = exp2f(s[nt][i] - m[i >> 1]);
                    s[nt][i] = p;
                    sum[i >> 1] += p;
                }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 1);
                sum[rr] += __shfl_xor_sync(0xffffffffu, sum[rr], 2);
                l[rr] = l[rr] * rs[rr] + sum[rr];
            }
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                acc[n][0] *= rs[0];
                acc[n][1] *= rs[0];
                acc[n][2] *= rs[1];
                acc[n][3] *= rs[1];
            }
            gemm_nn_16x128(s, sV + buf * TILE_BYTES, acc);
            __syncthreads();
        }
    }
    // epilogue
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int t = t0 + r_lo + 8 * rr;
        if (t >= T)
            continue;
        const float inv = 1.f / l[rr];
        __half *dst = o + (size_t)t * Q + h * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < 16; ++n)
            *(__half2 *)(dst + n * 8) = sat_half2(acc[n][2 * rr] * inv, acc[n][2 * rr + 1] * inv);
        if ((lane & 3) == 0)
            lse[(size_t)t * H + h] = m[rr] + log2f(l[rr]);
    }
}

// ---------------------------------------------------------------------------------------
// dQ: grid (query blocks, heads); streams K/V tiles
__global__ void __launch_bounds__(ATT_THREADS)
    att_dq_mma_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                      const __half *__restrict__ dout, const float *__restrict__ lse, const float *__restrict__ dscale,
                      const int *__restrict__ span_start, const int *__restrict__ span_finish, int T, int H, float slope,
                      float *__restrict__ dq)
{
    extern __shared__ __align__(1024) uint8_t att_smem[];
    __shared__ int s_lo, s_hi;
    const uint32_t sQ = smem_u32(att_smem), sDO = sQ + TILE_BYTES, sK = sDO + TILE_BYTES, sV = sK + 2 * TILE_BYTES;
    const int Q = H * HD, h = blockIdx.y, t0 = blockIdx.x * BLK;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float ds = att_dot_scale_mma(), c2 = ds * 0.693147f;
    const int r_lo = warp * 16 + (lane >> 2);
    int st[2], fi[2];
    float ls[2], dsc[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int t = t0 + r_lo + 8 * i;
        st[i] = t < T ? span_start[t] : 0;
        fi[i] = t < T ? span_finish[t] : -1;
        ls[i] = t < T ? lse[(size_t)t * H + h] : 0.f;
        dsc[i] = t < T ? dscale[(size_t)t * H + h] : 0.f;
    }
    int lo, hi;
    {
        int mylo = 0x7fffffff, myhi = -1;
        if ((lane & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (fi[i] >= st[i]) {
                    mylo = min(mylo, st[i]);
                    myhi = max(myhi, fi[i]);
                }
        }
        block_range(mylo, myhi, &s_lo, &s_hi, lo, hi);
    }
    float acc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            acc[n][i] = 0.f;
    if (hi >= lo) {
        const int tile0 = lo / BLK, tile1 = hi / BLK;
        load_tile(sQ, q, t0, T, Q, h);
        load_tile(sDO, dout, t0, T, Q, h);
        load_tile(sK, k, tile0 * BLK, T, Q, h);
        load_tile(sV, v, tile0 * BLK, T, Q, h);
        cp_async_commit();
        for (int tile = tile0; tile <= tile1; ++tile) {
            const int buf = (tile - tile0) & 1;
            if (tile < tile1) {
                load_tile(sK + (buf ^ 1) * TILE_BYTES, k, (tile + 1) * BLK, T, Q, h);
                load_tile(sV + (buf ^ 1) * TILE_BYTES, v, (tile + 1) * BLK, T, Q, h);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            float s[8][4], dp[8][4];
            gemm_nt_16x64(sQ, warp * 16, sK + buf * TILE_BYTES, s);
            gemm_nt_16x64(sDO, warp * 16, sV + buf * TILE_BYTES, dp);
            const int key0 = tile * BLK + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1, key = key0 + nt * 8 + (i & 1);
                    const float x = s[nt][i] * ds - slope * (float)(t0 + r_lo + 8 * rr - key);
                    const float w = (key >= st[rr] && key <= fi[rr]) ? exp2f(x - ls[rr]) : 0.f;
                    s[nt][i] = w * (dp[nt][i] - dsc[rr]) * c2; // dDot
                }
            gemm_nn_16x128(s, sK + buf * TILE_BYTES, acc);
            __syncthreads();
        }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int t = t0 + r_lo + 8 * rr;
        if (t >= T)
            continue;
        float *dst = dq + (size_t)t * Q + h * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < 16; ++n)
            *(float2 *)(dst + n * 8) = make_float2(acc[n][2 * rr], acc[n][2 * rr + 1]);
    }
}

// ---------------------------------------------------------------------------------------
// dK, dV: grid (key blocks, heads); streams Q/dO tiles of the nodes that attend to the block
__global__ void __launch_bounds__(ATT_THREADS)
    att_dkv_mma_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                       const __half *__restrict__ dout, const float *__restrict__ lse, const float *__restrict__ dscale,
                       const int *__restrict__ span_start, const int *__restrict__ span_finish, const int *__restrict__ rev_first,
                       const int *__restrict__ rev_last, int T, int H, float slope, float *__restrict__ dk, float *__restrict__ dv)
{
    extern __shared__ __align__(1024) uint8_t att_smem[];
    __shared__ int s_lo, s_hi;
    __shared__ int s_st[2][BLK], s_fi[2][BLK];
    __shared__ float s_lse[2][BLK], s_dsc[2][BLK];
    const uint32_t sK = smem_u32(att_smem), sV = sK + TILE_BYTES, sQ = sV + TILE_BYTES, sDO = sQ + 2 * TILE_BYTES;
    const int Q = H * HD, h = blockIdx.y, k0 = blockIdx.x * BLK;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float ds = att_dot_scale_mma(), c2 = ds * 0.693147f;
    const int r_lo = warp * 16 + (lane >> 2); // key rows of this thread: k0 + r_lo (+8)
    int lo, hi;
    {
        int mylo = 0x7fffffff, myhi = -1;
        if (threadIdx.x < BLK) {
            const int key = k0 + threadIdx.x;
            if (key < T) {
                mylo = rev_first[key];
                myhi = rev_last[key];
            }
        }
        block_range(mylo, myhi, &s_lo, &s_hi, lo, hi);
    }
    float ak[16][4], av[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            ak[n][i] = av[n][i] = 0.f;

    auto load_meta = [&](int buf, int row0) {
        if (threadIdx.x < BLK) {
            const int t = row0 + threadIdx.x;
            const bool ok = t < T;
            s_st[buf][threadIdx.x] = ok ? span_start[t] : 0;
            s_fi[buf][threadIdx.x] = ok ? span_finish[t] : -1;
            s_lse[buf][threadIdx.x] = ok ? lse[(size_t)t * H + h] : 0.f;
            s_dsc[buf][threadIdx.x] = ok ? dscale[(size_t)t * H + h] : 0.f;
        }
    };

    if (hi >= lo) {
        const int tile0 = lo / BLK, tile1 = hi / BLK;
        load_tile(sK, k, k0, T, Q, h);
        load_tile(sV, v, k0, T, Q, h);
        load_tile(sQ, q, tile0 * BLK, T, Q, h);
        load_tile(sDO, dout, tile0 * BLK, T, Q, h);
        cp_async_commit();
        load_meta(0, tile0 * BLK);
        for (int tile = tile0; tile <= tile1; ++tile) {
            const int buf = (tile - tile0) & 1;
            if (tile < tile1) {
                load_tile(sQ + (buf ^ 1) * TILE_BYTES, q, (tile + 1) * BLK, T, Q, h);
                load_tile(sDO + (buf ^ 1) * TILE_BYTES, dout, (tile + 1) * BLK, T, Q, h);
                cp_async_commit();
                load_meta(buf ^ 1, (tile + 1) * BLK);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            // transposed problem: rows = keys of this block, columns = the tile's nodes
            float s[8][4], dp[8][4];
            gemm_nt_16x64(sK, warp * 16, sQ + buf * TILE_BYTES, s);
            gemm_nt_16x64(sV, warp * 16, sDO + buf * TILE_BYTES, dp);
            const int col0 = (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = col0 + nt * 8 + (i & 1);
                    const int key = k0 + r_lo + 8 * (i >> 1);
                    const int t = tile * BLK + c;
                    const float x = s[nt][i] * ds - slope * (float)(t - key);
                    const float w = (key >= s_st[buf][c] && key <= s_fi[buf][c]) ? exp2f(x - s_lse[buf][c]) : 0.f;
                    s[nt][i] = w;
                    dp[nt][i] = w * (dp[nt][i] - s_dsc[buf][c]) * c2;
                }
            gemm_nn_16x128(s, sDO + buf * TILE_BYTES, av);
            gemm_nn_16x128(dp, sQ + buf * TILE_BYTES, ak);
            __syncthreads();
        }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int key = k0 + r_lo + 8 * rr;
        if (key >= T)
            continue;
        float *dkp = dk + (size_t)key * Q + h * HD + (lane & 3) * 2;
        float *dvp = dv + (size_t)key * Q + h * HD + (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            *(float2 *)(dkp + n * 8) = make_float2(ak[n][2 * rr], ak[n][2 * rr + 1]);
            *(float2 *)(dvp + n * 8) = make_float2(av[n][2 * rr], av[n][2 * rr + 1]);
        }
    }
}

// ---------------------------------------------------------------------------------------
static int configure_att(int device)
{
    static bool done[16] = {};
    if (!done[device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(att_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 5 * TILE_BYTES));
        TS2_CUDA(cudaFuncSetAttribute(att_dq_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * TILE_BYTES));
        TS2_CUDA(cudaFuncSetAttribute(att_dkv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * TILE_BYTES));
        done[device & 15] = true;
    }
    return TS2_OK;
}

int attention_forward_mma(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                          int T, int H, float slope, __half *o, float *lse)
{
    int rc = configure_att(c.device);
    if (rc != TS2_OK)
        return rc;
    dim3 grid((unsigned)ceil_div(T, BLK), (unsigned)H);
    att_fwd_mma_kernel<<<grid, ATT_THREADS, 5 * TILE_BYTES, c.stream>>>(q, k, v, span_start, span_finish, T, H, slope, o, lse);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int attention_backward_mma(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                           const float *dscale, const int *span_start, const int *span_finish, const int *rev_first,
                           const int *rev_last, int T, int H, float slope, float *dq, float *dk, float *dv)
{
    int rc = configure_att(c.device);
    if (rc != TS2_OK)
        return rc;
    dim3 grid((unsigned)ceil_div(T, BLK), (unsigned)H);
    att_dq_mma_kernel<<<grid, ATT_THREADS, 6 * TILE_BYTES, c.stream>>>(q, k, v, dout, lse, dscale, span_start, span_finish, T, H, slope, dq);
    TS2_CHECK_LAUNCH();
    att_dkv_mma_kernel<<<grid, ATT_THREADS, 6 * TILE_BYTES, c.stream>>>(q, k, v, dout, lse, dscale, span_start, span_finish, rev_first,
                                                                        rev_last, T, H, slope, dk, dv);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
