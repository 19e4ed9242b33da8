// Bandwidth-bound kernels of the training step: embedding, tile normalisation and
// its backward, gradient cast/scale, LoLU activations and their backward, softmax
// cross-entropy.  One warp owns one 128-wide tile of one row (a lane holds four
// consecutive elements: 16-byte accesses for fp32, 8 for fp16, 4 for e4m3) and
// strides over (row, tile) pairs; reductions are warp shuffles.
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int WARPS = 8;
static constexpr int THREADS = WARPS * 32;

static int grid_for(const Ctx &c, long long warp_items)
{
    long long blocks = ceil_div(warp_items, WARPS);
    long long cap = (long long)sm_count(c.device) * 8;
    return (int)std::max<long long>(1, std::min(blocks, cap));
}

// for the grid-stride kernels that carry most of the bytes: exactly the blocks that are resident at once.  With a
// fixed 8 blocks per SM a kernel that fits 5 (48 registers) ran a second, partly filled wave at a fraction of the
// bandwidth.
template <typename K>
static int grid_for(const Ctx &c, K kernel, long long warp_items)
{
    long long blocks = ceil_div(warp_items, WARPS);
    long long cap = (long long)sm_count(c.device) * resident_blocks(c.device, (const void *)kernel, THREADS);
    return (int)std::max<long long>(1, std::min(blocks, cap));
}

// R items per warp and iteration: all loads of the R items are issued before any of them is
// consumed, which keeps enough bytes in flight per SM to approach HBM bandwidth
#define WARP_BATCH_LOOP(total, R)                                                                          \
    const int lane = threadIdx.x & 31;                                                                     \
    const unsigned wstride = gridDim.x * WARPS, total_items = (unsigned)(total);                          \
    for (unsigned base = blockIdx.x * WARPS + (threadIdx.x >> 5); base < total_items; base += wstride * (R))

#define WARP_ITEM_LOOP(total) \
    const int lane = threadIdx.x & 31; \
    for (unsigned item = blockIdx.x * WARPS + (threadIdx.x >> 5), total_items = (unsigned)(total); item < total_items; \
         item += gridDim.x * WARPS)

// ---------------------------------------------------------------------------------
__global__ void embed_forward_kernel(const __half *__restrict__ embed, const float *__restrict__ sko,
                                     const uint32_t *__restrict__ label_arr, const uint32_t *__restrict__ label_ptr, int T, int D,
                                     float *__restrict__ state)
{
    const int tiles = D / TILE;
    const float scale = __ldg(sko) * (1.f / 32);
    WARP_ITEM_LOOP((long long)T * tiles)
    {
        const int t = (int)(item / tiles), off = (int)(item % tiles) * TILE + lane * 4;
        float4 acc = make_float4(0, 0, 0, 0);
        for (uint32_t k = label_ptr[t]; k < label_ptr[t + 1]; ++k) {
            uint32_t label = label_arr[k];
            float w = (label & TS2_LABEL_NEGATIVE) ? -1.f : 1.f;
            label &= TS2_LABEL_MASK;
            float4 e = load_half4(embed + (size_t)label * D + off);
            // the CPU path adds (q * scale) * w label by label
            acc.x += (e.x * scale) * w;
            acc.y += (e.y * scale) * w;
            acc.z += (e.z * scale) * w;
            acc.w += (e.w * scale) * w;
        }
        *(float4 *)(state + (size_t)t * D + off) = acc;
    }
}

int embed_forward(const Ctx &c, const __half *embed, const float *sko, const uint32_t *label_arr, const uint32_t *label_ptr, int T,
                  int D, float *state)
{
    embed_forward_kernel<<<grid_for(c, (long long)T * (D / TILE)), THREADS, 0, c.stream>>>(embed, sko, label_arr, label_ptr, T, D, state);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
template <int FT>
__global__ void tilenorm_forward_kernel(const float *__restrict__ x, int T, int D, float s_act, void *__restrict__ n_fast,
                                        __half *__restrict__ n16)
{
    const int tiles = D / TILE;
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        float4 v[R];
        size_t idx[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            idx[r] = ok[r] ? (size_t)(item / tiles) * D + (item % tiles) * TILE + lane * 4 : 0;
            v[r] = ok[r] ? *(const float4 *)(x + idx[r]) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const float scale = tile_scale(warp_sum(dot4(v[r], v[r])));
            const float4 nv = scale4(v[r], scale);
            Fast<FT>::store4(n_fast, idx[r], scale4(nv, s_act));
            if (n16)
                store_half4(n16 + idx[r], nv);
        }
    }
}

int tilenorm_forward(const Ctx &c, const float *x, int T, int D, void *n_fast, __half *n16)
{
    const int grid = c.ft == 0   ? grid_for(c, tilenorm_forward_kernel<0>, (long long)T * (D / TILE))
                     : c.ft == 1 ? grid_for(c, tilenorm_forward_kernel<1>, (long long)T * (D / TILE))
                                 : grid_for(c, tilenorm_forward_kernel<2>, (long long)T * (D / TILE));
    if (c.ft == 0)
        tilenorm_forward_kernel<0><<<grid, THREADS, 0, c.stream>>>(x, T, D, c.s_act, n_fast, n16);
    else if (c.ft == 1)
        tilenorm_forward_kernel<1><<<grid, THREADS, 0, c.stream>>>(x, T, D, c.s_act, n_fast, n16);
    else
        tilenorm_forward_kernel<2><<<grid, THREADS, 0, c.stream>>>(x, T, D, c.s_act, n_fast, n16);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

__global__ void tilenorm_backward_kernel(const float *__restrict__ x, const float *__restrict__ dn, const float *__restrict__ dyn,
                                         float dn_alpha, int T, int D, float *__restrict__ g, int add, unsigned *__restrict__ absmax,
                                         unsigned *__restrict__ health, unsigned step_no)
{
    const int tiles = D / TILE;
    const float a = dn_alpha * (dyn ? __ldg(dyn) : 1.f);
    float local_max = 0.f;
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        float4 xv[R], dv[R], o[R];
        size_t idx[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            idx[r] = ok[r] ? (size_t)(item / tiles) * D + (item % tiles) * TILE + lane * 4 : 0;
            xv[r] = ok[r] ? *(const float4 *)(x + idx[r]) : make_float4(0, 0, 0, 0);
            dv[r] = ok[r] ? *(const float4 *)(dn + idx[r]) : make_float4(0, 0, 0, 0);
            o[r] = (ok[r] && add) ? *(const float4 *)(g + idx[r]) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const float4 d = scale4(dv[r], a);
            const float sum2 = warp_sum(dot4(xv[r], xv[r]));
            const float dp = warp_sum(dot4(xv[r], d));
            float4 res = make_float4(0, 0, 0, 0);
            if (sum2 != 0.f) {
                const float sigma = dp / sum2, scale = sqrtf(128.f / sum2);
                res = make_float4(scale * (d.x - xv[r].x * sigma), scale * (d.y - xv[r].y * sigma), scale * (d.z - xv[r].z * sigma),
                                  scale * (d.w - xv[r].w * sigma));
            }
            res = make_float4(o[r].x + res.x, o[r].y + res.y, o[r].z + res.z, o[r].w + res.w);
            *(float4 *)(g + idx[r]) = res;
            local_max = fmaxf(local_max, fmaxf(fmaxf(fabsf(res.x), fabsf(res.y)), fmaxf(fabsf(res.z), fabsf(res.w))));
            // fmaxf drops a NaN operand: a NaN anywhere in the row piece turns the running maximum into inf instead
            if (!(res.x == res.x && res.y == res.y && res.z == res.z && res.w == res.w))
                local_max = INFINITY;
        }
    }
    if (absmax) {
        __shared__ float block_max[WARPS];
        local_max = warp_max(local_max);
        if ((threadIdx.x & 31) == 0)
            block_max[threadIdx.x >> 5] = local_max;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.f;
            for (int i = 0; i < WARPS; ++i)
                m = fmaxf(m, block_max[i]);
            if (m == m && m < 3.0e38f) // NaN / inf never become the scale reference
                atomicMax(absmax, __float_as_uint(m));
            else if (health)
                atomicCAS(health, 0u, step_no); // the first step at which this boundary's gradient was not finite
        }
    }
}

int tilenorm_backward(const Ctx &c, const float *x, const float *dn, const float *dyn, float dn_alpha, int T, int D, float *g, bool add,
                      unsigned *absmax, unsigned *health, unsigned step_no)
{
    tilenorm_backward_kernel<<<grid_for(c, tilenorm_backward_kernel, (long long)T * (D / TILE)), THREADS, 0, c.stream>>>(
        x, dn, dyn, dn_alpha, T, D, g, add ? 1 : 0, absmax, health, step_no);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// power-of-two multiplier that brings max|g| just below `target`
__device__ __forceinline__ float grad_mult(unsigned absmax_bits, float target)
{
    const float m = __uint_as_float(absmax_bits);
    if (!(m > 0.f))
        return 1.f;
    float e = floorf(log2f(target / m));
    e = fminf(fmaxf(e, -100.f), 100.f);
    return exp2f(e);
}

template <int FT>
__global__ void cast_grad_kernel(const float *__restrict__ g, size_t n4, const unsigned *__restrict__ absmax, void *__restrict__ out,
                                 float *__restrict__ ginv, float f_static, const float *__restrict__ sko, float *__restrict__ fscale)
{
    const float mult = grad_mult(*absmax, 128.f);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        *ginv = 1.f / mult;
        if (fscale)
            *fscale = f_static * (sko ? *sko : 1.f) / mult;
    }
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += stride * 4) {
        float4 v[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            v[r] = (i0 + r * stride < n4) ? *(const float4 *)(g + (i0 + r * stride) * 4) : make_float4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (i0 + r * stride < n4)
                Fast<FT>::store4(out, (i0 + r * stride) * 4, scale4(v[r], mult));
    }
}

int cast_grad(const Ctx &c, const float *g, size_t n, const unsigned *absmax, void *g_fast, float *ginv, float f_static, const float *sko,
              float *fscale)
{
    const size_t n4 = n / 4;
    const int per_sm = resident_blocks(c.device, c.ft == 0 ? (const void *)cast_grad_kernel<0> : (const void *)cast_grad_kernel<1>, THREADS);
    const int grid = (int)std::min<size_t>(ceil_div(n4, THREADS), (size_t)sm_count(c.device) * per_sm);
    if (c.ft == 0)
        cast_grad_kernel<0><<<grid, THREADS, 0, c.stream>>>(g, n4, absmax, g_fast, ginv, f_static, sko, fscale);
    else
        cast_grad_kernel<1><<<grid, THREADS, 0, c.stream>>>(g, n4, absmax, g_fast, ginv, f_static, sko, fscale);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// Row quantization to int8 with the reference's stochastic rounding (NormalizeVecsRowMaxKernel,
// src/gpt/compute/row_scale.cuh:12-43, TCudaRngLCG, src/lib/cuda/cuda_util.cuh:538-559): one warp per row;
// scale = max|x| / 127; lane h owns the elements h, h + 32, h + 64, ... and draws one uniform number per element, in
// that order, from a linear congruential generator seeded with (bits of x[h], bits of x[0], row); q = round to
// nearest even, saturating, of x / scale + u - 0.5.  x = src * mult, mult a power of two (so the scaling is exact).
// The quantized row goes through a shared-memory row so that it leaves in 16-byte pieces.  Optionally also writes x as
// fp16 (the operand of the fp16 dW contraction).  SRC: float or __half.
struct RowQuantLCG {
    uint32_t state;
    __device__ RowQuantLCG(uint32_t a, uint32_t b, uint32_t c) { state = a * 0x398bf183u + b * 0x1affc3dfu + c * 0x9023a049u; }
    __device__ float uniform()
    {
        state = state * 0x448e3079u + 0xc484ef10u;
        return (float)state * (1.0f / 4294967296.0f);
    }
};

template <typename SRC>
__device__ __forceinline__ float rq_load(const SRC *p, size_t i);
template <>
__device__ __forceinline__ float rq_load<float>(const float *p, size_t i)
{
    return p[i];
}
template <>
__device__ __forceinline__ float rq_load<__half>(const __half *p, size_t i)
{
    return __half2float(p[i]);
}

template <typename SRC>
__global__ void rowquant_i8_kernel(const SRC *__restrict__ src, int T, int D, const unsigned *__restrict__ absmax, float target,
                                   int8_t *__restrict__ q, float *__restrict__ row_scale, __half *__restrict__ x16,
                                   float *__restrict__ ginv, float f_static, const float *__restrict__ sko, float *__restrict__ fscale)
{
    extern __shared__ int8_t rq_rows[]; // [WARPS][D]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const float mult = absmax ? grad_mult(*absmax, target) : 1.f;
    if (blockIdx.x == 0 && threadIdx.x == 0 && ginv) {
        *ginv = 1.f / mult;
        if (fscale)
            *fscale = f_static * (sko ? *sko : 1.f) / mult;
    }
    int8_t *row_s = rq_rows + (size_t)wid * D;
    for (int t = blockIdx.x * WARPS + wid; t < T; t += gridDim.x * WARPS) {
        const SRC *row = src + (size_t)t * D;
        float mx = 0.f;
        for (int d = lane; d < D; d += 32)
            mx = fmaxf(mx, fabsf(rq_load<SRC>(row, d) * mult));
        mx = warp_max(mx);
        float scale = 0.f;
        if (mx > 0.f) {
            scale = mx / 127;
            const float inv = 1 / scale;
            RowQuantLCG rng(__float_as_uint(rq_load<SRC>(row, lane) * mult), __float_as_uint(rq_load<SRC>(row, 0) * mult), (uint32_t)t);
            for (int d = lane; d < D; d += 32) {
                const float x = rq_load<SRC>(row, d) * mult;
                row_s[d] = (int8_t)sat_i8(__fsub_rn(__fmaf_rn(x, inv, rng.uniform()), 0.5f));
                if (x16)
                    x16[(size_t)t * D + d] = __float2half_rn(x);
            }
        } else {
            for (int d = lane; d < D; d += 32) {
                row_s[d] = 0;
                if (x16)
                    x16[(size_t)t * D + d] = __float2half_rn(0.f);
            }
        }
        __syncwarp();
        for (int i = lane; i < D / 16; i += 32)
            *(uint4 *)(q + (size_t)t * D + 16 * i) = *(const uint4 *)(row_s + 16 * i);
        if (lane == 0)
            row_scale[t] = scale;
        __syncwarp();
    }
}

template <typename SRC>
static int rowquant_launch(const Ctx &c, const SRC *src, int T, int D, const unsigned *absmax, int8_t *q, float *row_scale, __half *x16,
                           float *ginv, float f_static, const float *sko, float *fscale)
{
    if (D % 128 || D > 16384)
        return fail(TS2_ERR_INVALID_ARG, "rowquant: row length %d must be a multiple of 128 up to 16384", D);
    auto kern = rowquant_i8_kernel<SRC>;
    const size_t smem = (size_t)WARPS * D;
    static bool configured[16] = {};
    if (smem > 48 * 1024 && !configured[c.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(rowquant_i8_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * 16384));
        TS2_CUDA(cudaFuncSetAttribute(rowquant_i8_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * 16384));
        configured[c.device & 15] = true;
    }
    const int grid = (int)std::max<long long>(1, std::min<long long>(ceil_div(T, WARPS), (long long)sm_count(c.device) * 4));
    kern<<<grid, THREADS, smem, c.stream>>>(src, T, D, absmax, 128.f, q, row_scale, x16, ginv, f_static, sko, fscale);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int rowquant_grad(const Ctx &c, const float *g, int T, int D, const unsigned *absmax, int8_t *q, float *row_scale, __half *g16, float *ginv,
                  float f_static, const float *sko, float *fscale)
{
    return rowquant_launch<float>(c, g, T, D, absmax, q, row_scale, g16, ginv, f_static, sko, fscale);
}

int rowquant_half(const Ctx &c, const __half *x, int T, int D, int8_t *q, float *row_scale)
{
    return rowquant_launch<__half>(c, x, T, D, nullptr, q, row_scale, nullptr, nullptr, 1.f, nullptr, nullptr);
}

__global__ void i8_to_half_kernel(const char4 *__restrict__ src, size_t n4, uint2 *__restrict__ dst)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const char4 v = src[i];
        const __half2 a = __floats2half2_rn((float)v.x, (float)v.y), b = __floats2half2_rn((float)v.z, (float)v.w);
        dst[i] = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
    }
}

int i8_to_half(const Ctx &c, const void *src, size_t n, __half *dst)
{
    const size_t n4 = n / 4;
    const int grid = (int)std::max<size_t>(1, std::min<size_t>(ceil_div(n4, 256 * 4), (size_t)sm_count(c.device) * 8));
    i8_to_half_kernel<<<grid, 256, 0, c.stream>>>((const char4 *)src, n4, (uint2 *)dst);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// (the forward FFN activation lives in the contraction's gated epilogue, gemm.cu)
template <int FT>
__global__ void ffn_act_backward_kernel(const __half *__restrict__ drg, const __half *__restrict__ wg, const __half *__restrict__ what,
                                        int what_ld, const float *__restrict__ wscale, int T, int F, void *__restrict__ d2)
{
    const int tiles = F / TILE;
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        float4 g[R], gate[R], wn[R];
        float scale[R];
        size_t t[R];
        int off[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            const int tile = ok[r] ? (int)(item % tiles) : 0;
            off[r] = tile * TILE + lane * 4;
            g[r] = ok[r] ? load_half4(drg + t[r] * F + off[r]) : make_float4(0, 0, 0, 0);
            gate[r] = ok[r] ? load_half4(wg + t[r] * 2 * F + F + off[r]) : make_float4(0, 0, 0, 0);
            wn[r] = ok[r] ? load_half4(what + t[r] * what_ld + off[r]) : make_float4(0, 0, 0, 0);
            scale[r] = ok[r] ? wscale[t[r] * tiles + tile] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const float4 m = make_float4(lolu_mult_ft<FT>(gate[r].x), lolu_mult_ft<FT>(gate[r].y), lolu_mult_ft<FT>(gate[r].z), lolu_mult_ft<FT>(gate[r].w));
            const float4 dgate = make_float4(g[r].x * wn[r].x * m.x * (1 - m.x) * 2.f, g[r].y * wn[r].y * m.y * (1 - m.y) * 2.f,
                                             g[r].z * wn[r].z * m.z * (1 - m.z) * 2.f, g[r].w * wn[r].w * m.w * (1 - m.w) * 2.f);
            const float4 dwn = make_float4(g[r].x * m.x, g[r].y * m.y, g[r].z * m.z, g[r].w * m.w);
            // tile-norm backward expressed with the normalized vector: scale * (d - wn * (wn . d) / 128)
            const float proj = warp_sum(dot4(wn[r], dwn)) * (1.f / 128);
            const float sc = scale[r];
            const float4 dwide = make_float4(sc * (dwn.x - wn[r].x * proj), sc * (dwn.y - wn[r].y * proj), sc * (dwn.z - wn[r].z * proj),
                                             sc * (dwn.w - wn[r].w * proj));
            Fast<FT>::store4(d2, t[r] * 2 * F + off[r], dwide);
            Fast<FT>::store4(d2, t[r] * 2 * F + F + off[r], dgate);
        }
    }
}

// The e4m3 pipeline's form of the kernel above in packed fp16 (see fast_types.cuh): same loads and stores, a third of
// the instructions.  The sum over the tile is accumulated in fp32.
__global__ void ffn_act_backward_e4m3_kernel(const __half *__restrict__ drg, const __half *__restrict__ wg, const __half *__restrict__ what,
                                             int what_ld, const float *__restrict__ wscale, int T, int F, uint8_t *__restrict__ d2)
{
    const int tiles = F / TILE;
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        uint2 g[R], gate[R], wn[R];
        float scale[R];
        size_t t[R];
        int off[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            const int tile = ok[r] ? (int)(item % tiles) : 0;
            off[r] = tile * TILE + lane * 4;
            const uint2 z = make_uint2(0u, 0u);
            g[r] = ok[r] ? *(const uint2 *)(drg + t[r] * F + off[r]) : z;
            gate[r] = ok[r] ? *(const uint2 *)(wg + t[r] * 2 * F + F + off[r]) : z;
            wn[r] = ok[r] ? *(const uint2 *)(what + t[r] * what_ld + off[r]) : z;
            scale[r] = ok[r] ? wscale[t[r] * tiles + tile] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const __half2 one = __float2half2_rn(1.f), two = __float2half2_rn(2.f);
            const __half2 g0 = h2_from_bits(g[r].x), g1 = h2_from_bits(g[r].y), w0 = h2_from_bits(wn[r].x), w1 = h2_from_bits(wn[r].y);
            const __half2 m0 = lolu_mult_h2(h2_from_bits(gate[r].x)), m1 = lolu_mult_h2(h2_from_bits(gate[r].y));
            // d gate = g wn m (1 - m) 2: the bounded factors first, the gradient last
            const __half2 dg0 = __hmul2(g0, __hmul2(w0, __hmul2(__hmul2(m0, two), __hsub2(one, m0))));
            const __half2 dg1 = __hmul2(g1, __hmul2(w1, __hmul2(__hmul2(m1, two), __hsub2(one, m1))));
            const __half2 dw0 = __hmul2(g0, m0), dw1 = __hmul2(g1, m1); // gradient of the normalized wide values
            // tile-norm backward expressed with the normalized vector: scale * (d - wn * (wn . d) / 128)
            const float2 p0 = __half22float2(__hmul2(w0, dw0)), p1 = __half22float2(__hmul2(w1, dw1));
            const float proj = warp_sum((p0.x + p0.y) + (p1.x + p1.y)) * (1.f / 128);
            const __half2 nproj = __float2half2_rn(-proj), sc = __float2half2_rn(scale[r]);
            const __half2 dx0 = __hmul2(sc, __hfma2(w0, nproj, dw0)), dx1 = __hmul2(sc, __hfma2(w1, nproj, dw1));
            *(uint32_t *)(d2 + t[r] * 2 * F + off[r]) = e4m3x4_from_h2(dx0, dx1);
            *(uint32_t *)(d2 + t[r] * 2 * F + F + off[r]) = e4m3x4_from_h2(dg0, dg1);
        }
    }
}

int ffn_act_backward(const Ctx &c, const __half *drg, const __half *wg, const __half *what, int what_ld, const float *wscale, int T, int F,
                     void *d2)
{
    if (c.ft == 0) {
        ffn_act_backward_e4m3_kernel<<<grid_for(c, ffn_act_backward_e4m3_kernel, (long long)T * (F / TILE)), THREADS, 0, c.stream>>>(
            drg, wg, what, what_ld, wscale, T, F, (uint8_t *)d2);
        TS2_CHECK_LAUNCH();
        return TS2_OK;
    }
    const int grid = c.ft == 0 ? grid_for(c, ffn_act_backward_kernel<0>, (long long)T * (F / TILE))
                               : grid_for(c, ffn_act_backward_kernel<1>, (long long)T * (F / TILE));
    if (c.ft == 0)
        ffn_act_backward_kernel<0><<<grid, THREADS, 0, c.stream>>>(drg, wg, what, what_ld, wscale, T, F, d2);
    else
        ffn_act_backward_kernel<1><<<grid, THREADS, 0, c.stream>>>(drg, wg, what, what_ld, wscale, T, F, d2);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
template <int FT>
__global__ void att_gate_forward_kernel(const __half *__restrict__ qkvg, const __half *__restrict__ o, int T, int Q, float s_act,
                                        void *__restrict__ rg)
{
    const int tiles = Q / TILE;
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        float4 gate[R], ov[R];
        size_t t[R];
        int off[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            off[r] = (ok[r] ? (int)(item % tiles) : 0) * TILE + lane * 4;
            gate[r] = ok[r] ? load_half4(qkvg + t[r] * 4 * Q + 3 * Q + off[r]) : make_float4(0, 0, 0, 0);
            ov[r] = ok[r] ? load_half4(o + t[r] * Q + off[r]) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const float4 res = make_float4(lolu_mult_ft<FT>(gate[r].x) * ov[r].x, lolu_mult_ft<FT>(gate[r].y) * ov[r].y,
                                           lolu_mult_ft<FT>(gate[r].z) * ov[r].z, lolu_mult_ft<FT>(gate[r].w) * ov[r].w);
            Fast<FT>::store4(rg, t[r] * Q + off[r], scale4(res, s_act));
        }
    }
}

__global__ void att_gate_forward_e4m3_kernel(const __half *__restrict__ qkvg, const __half *__restrict__ o, int T, int Q, float s_act,
                                             uint8_t *__restrict__ rg)
{
    const int tiles = Q / TILE;
    constexpr int R = 4;
    const __half2 sa = __float2half2_rn(s_act);
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        uint2 gate[R], ov[R];
        size_t t[R];
        int off[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            off[r] = (ok[r] ? (int)(item % tiles) : 0) * TILE + lane * 4;
            const uint2 z = make_uint2(0u, 0u);
            gate[r] = ok[r] ? *(const uint2 *)(qkvg + t[r] * 4 * Q + 3 * Q + off[r]) : z;
            ov[r] = ok[r] ? *(const uint2 *)(o + t[r] * Q + off[r]) : z;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const __half2 r0 = __hmul2(__hmul2(lolu_mult_h2(h2_from_bits(gate[r].x)), h2_from_bits(ov[r].x)), sa);
            const __half2 r1 = __hmul2(__hmul2(lolu_mult_h2(h2_from_bits(gate[r].y)), h2_from_bits(ov[r].y)), sa);
            *(uint32_t *)(rg + t[r] * Q + off[r]) = e4m3x4_from_h2(r0, r1);
        }
    }
}

int att_gate_forward(const Ctx &c, const __half *qkvg, const __half *o, int T, int Q, void *rg)
{
    if (c.ft == 0) {
        att_gate_forward_e4m3_kernel<<<grid_for(c, att_gate_forward_e4m3_kernel, (long long)T * (Q / TILE)), THREADS, 0, c.stream>>>(
            qkvg, o, T, Q, c.s_act, (uint8_t *)rg);
        TS2_CHECK_LAUNCH();
        return TS2_OK;
    }
    const int grid = c.ft == 0   ? grid_for(c, att_gate_forward_kernel<0>, (long long)T * (Q / TILE))
                     : c.ft == 1 ? grid_for(c, att_gate_forward_kernel<1>, (long long)T * (Q / TILE))
                                 : grid_for(c, att_gate_forward_kernel<2>, (long long)T * (Q / TILE));
    if (c.ft == 0)
        att_gate_forward_kernel<0><<<grid, THREADS, 0, c.stream>>>(qkvg, o, T, Q, c.s_act, rg);
    else if (c.ft == 1)
        att_gate_forward_kernel<1><<<grid, THREADS, 0, c.stream>>>(qkvg, o, T, Q, c.s_act, rg);
    else
        att_gate_forward_kernel<2><<<grid, THREADS, 0, c.stream>>>(qkvg, o, T, Q, c.s_act, rg);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

template <int FT>
__global__ void att_gate_backward_kernel(const __half *__restrict__ drg, const __half *__restrict__ qkvg, const __half *__restrict__ o,
                                         int T, int Q, void *__restrict__ d4, __half *__restrict__ dout, float *__restrict__ dscale)
{
    const int tiles = Q / TILE; // = heads
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        float4 g[R], gate[R], ov[R];
        size_t t[R];
        int h[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            h[r] = ok[r] ? (int)(item % tiles) : 0;
            const int off = h[r] * TILE + lane * 4;
            g[r] = ok[r] ? load_half4(drg + t[r] * Q + off) : make_float4(0, 0, 0, 0);
            gate[r] = ok[r] ? load_half4(qkvg + t[r] * 4 * Q + 3 * Q + off) : make_float4(0, 0, 0, 0);
            ov[r] = ok[r] ? load_half4(o + t[r] * Q + off) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const int off = h[r] * TILE + lane * 4;
            const float4 m = make_float4(lolu_mult_ft<FT>(gate[r].x), lolu_mult_ft<FT>(gate[r].y), lolu_mult_ft<FT>(gate[r].z), lolu_mult_ft<FT>(gate[r].w));
            const float4 dgate = make_float4(g[r].x * ov[r].x * m.x * (1 - m.x) * 2.f, g[r].y * ov[r].y * m.y * (1 - m.y) * 2.f,
                                             g[r].z * ov[r].z * m.z * (1 - m.z) * 2.f, g[r].w * ov[r].w * m.w * (1 - m.w) * 2.f);
            const float4 dov = make_float4(g[r].x * m.x, g[r].y * m.y, g[r].z * m.z, g[r].w * m.w);
            Fast<FT>::store4(d4, t[r] * 4 * Q + 3 * Q + off, dgate);
            store_half4(dout + t[r] * Q + off, dov);
            const float ds = warp_sum(dot4(dov, ov[r]));
            if (lane == 0)
                dscale[t[r] * tiles + h[r]] = ds;
        }
    }
}

__global__ void att_gate_backward_e4m3_kernel(const __half *__restrict__ drg, const __half *__restrict__ qkvg, const __half *__restrict__ o,
                                              int T, int Q, uint8_t *__restrict__ d4, __half *__restrict__ dout, float *__restrict__ dscale)
{
    const int tiles = Q / TILE; // = heads
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * tiles, R)
    {
        uint2 g[R], gate[R], ov[R];
        size_t t[R];
        int h[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / tiles : 0;
            h[r] = ok[r] ? (int)(item % tiles) : 0;
            const int off = h[r] * TILE + lane * 4;
            const uint2 z = make_uint2(0u, 0u);
            g[r] = ok[r] ? *(const uint2 *)(drg + t[r] * Q + off) : z;
            gate[r] = ok[r] ? *(const uint2 *)(qkvg + t[r] * 4 * Q + 3 * Q + off) : z;
            ov[r] = ok[r] ? *(const uint2 *)(o + t[r] * Q + off) : z;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const int off = h[r] * TILE + lane * 4;
            const __half2 one = __float2half2_rn(1.f), two = __float2half2_rn(2.f);
            const __half2 g0 = h2_from_bits(g[r].x), g1 = h2_from_bits(g[r].y), o0 = h2_from_bits(ov[r].x), o1 = h2_from_bits(ov[r].y);
            const __half2 m0 = lolu_mult_h2(h2_from_bits(gate[r].x)), m1 = lolu_mult_h2(h2_from_bits(gate[r].y));
            const __half2 dg0 = __hmul2(g0, __hmul2(o0, __hmul2(__hmul2(m0, two), __hsub2(one, m0))));
            const __half2 dg1 = __hmul2(g1, __hmul2(o1, __hmul2(__hmul2(m1, two), __hsub2(one, m1))));
            const __half2 do0 = __hmul2(g0, m0), do1 = __hmul2(g1, m1);
            *(uint32_t *)(d4 + t[r] * 4 * Q + 3 * Q + off) = e4m3x4_from_h2(dg0, dg1);
            *(uint2 *)(dout + t[r] * Q + off) = make_uint2(bits_from_h2(do0), bits_from_h2(do1));
            // dscale from the fp16 values the attention kernels will read
            const float2 a0 = __half22float2(do0), a1 = __half22float2(do1), b0 = __half22float2(o0), b1 = __half22float2(o1);
            const float ds = warp_sum(fmaf(a0.x, b0.x, a0.y * b0.y) + fmaf(a1.x, b1.x, a1.y * b1.y));
            if (lane == 0)
                dscale[t[r] * tiles + h[r]] = ds;
        }
    }
}

int att_gate_backward(const Ctx &c, const __half *drg, const __half *qkvg, const __half *o, int T, int Q, void *d4, __half *dout,
                      float *dscale)
{
    if (c.ft == 0) {
        att_gate_backward_e4m3_kernel<<<grid_for(c, att_gate_backward_e4m3_kernel, (long long)T * (Q / TILE)), THREADS, 0, c.stream>>>(
            drg, qkvg, o, T, Q, (uint8_t *)d4, dout, dscale);
        TS2_CHECK_LAUNCH();
        return TS2_OK;
    }
    const int grid = c.ft == 0 ? grid_for(c, att_gate_backward_kernel<0>, (long long)T * (Q / TILE))
                               : grid_for(c, att_gate_backward_kernel<1>, (long long)T * (Q / TILE));
    if (c.ft == 0)
        att_gate_backward_kernel<0><<<grid, THREADS, 0, c.stream>>>(drg, qkvg, o, T, Q, d4, dout, dscale);
    else
        att_gate_backward_kernel<1><<<grid, THREADS, 0, c.stream>>>(drg, qkvg, o, T, Q, d4, dout, dscale);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// One block per row; the row of fp16 logits is staged in shared memory, read once
// from HBM and overwritten once with the gradient.  Three passes over the staged row,
// all in 16-byte vectors: maximum; e = 2^(x + bias - max) with its fp32 sum, e kept in
// place as fp16; gradient (onehot - e / sum) * gscale.  One exponential per logit.
__global__ void __launch_bounds__(512, 2)
    softmax_ce_kernel(__half *__restrict__ logits, int rows, int V, const float *__restrict__ bias, const int *__restrict__ target,
                      float gscale, float *__restrict__ logp_sum, int write_grad)
{
    extern __shared__ uint4 row_s4[];
    __shared__ float red[32];
    __shared__ float x_tgt_s;
    const int tid = threadIdx.x, nthr = blockDim.x, nvec = V / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        uint4 *src = (uint4 *)(logits + (size_t)row * V);
        const int tgt = target[row];
        if (tgt < 0) {
            if (write_grad)
                for (int i = tid; i < nvec; i += nthr)
                    src[i] = make_uint4(0, 0, 0, 0);
            continue;
        }
        float mx = 0.f; // the reference starts the maximum at 0 and takes it over the logits without bias
        for (int i0 = tid; i0 < nvec; i0 += nthr * 4) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                raw[u] = (i0 + u * nthr < nvec) ? src[i0 + u * nthr] : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u * nthr >= nvec)
                    continue;
                row_s4[i0 + u * nthr] = raw[u];
                const __half2 *h = (const __half2 *)&raw[u];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = __half22float2(h[j]);
                    mx = fmaxf(mx, fmaxf(f.x, f.y));
                }
            }
        }
        mx = warp_max(mx);
        if ((tid & 31) == 0)
            red[tid >> 5] = mx;
        __syncthreads();
        mx = 0.f;
        for (int i = 0; i < nthr / 32; ++i)
            mx = fmaxf(mx, red[i]);
        __syncthreads();
        float sum0 = 0.f, sum1 = 0.f;
        for (int i = tid; i < nvec; i += nthr) { // every thread revisits the vectors it staged itself
            uint4 raw = row_s4[i];
            __half2 *h = (__half2 *)&raw;
            float bv[8];
            if (bias) {
                const float4 b0 = __ldg((const float4 *)(bias + 8 * i)), b1 = __ldg((const float4 *)(bias + 8 * i) + 1);
                bv[0] = b0.x, bv[1] = b0.y, bv[2] = b0.z, bv[3] = b0.w, bv[4] = b1.x, bv[5] = b1.y, bv[6] = b1.z, bv[7] = b1.w;
            }
            const int trel = tgt - 8 * i; // position of the target inside this vector, if 0..7
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                const float x0 = f.x + (bias ? bv[2 * j] : 0.f), x1 = f.y + (bias ? bv[2 * j + 1] : 0.f);
                if (trel == 2 * j)
                    x_tgt_s = x0;
                if (trel == 2 * j + 1)
                    x_tgt_s = x1;
                float e0, e1;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0 - mx));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1 - mx));
                sum0 += e0;
                sum1 += e1;
                h[j] = sat_half2(e0, e1);
            }
            row_s4[i] = raw;
        }
        float sum = warp_sum(sum0 + sum1);
        if ((tid & 31) == 0)
            red[tid >> 5] = sum;
        __syncthreads();
        sum = 0.f;
        for (int i = 0; i < nthr / 32; ++i)
            sum += red[i];
        const float inv = 1.f / sum;
        if (tid == 0)
            atomicAdd(logp_sum, (x_tgt_s - mx) * 0.69314718f - logf(sum));
        if (write_grad) {
            const float ninv = -inv * gscale;
            for (int i = tid; i < nvec; i += nthr) {
                uint4 raw = row_s4[i];
                __half2 *h = (__half2 *)&raw;
                const int trel = tgt - 8 * i;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 e = __half22float2(h[j]);
                    h[j] = sat_half2(fmaf(e.x, ninv, trel == 2 * j ? gscale : 0.f), fmaf(e.y, ninv, trel == 2 * j + 1 ? gscale : 0.f));
                }
                src[i] = raw;
            }
        }
        __syncthreads();
    }
}

// The same three passes with the row traffic taken off the threads: one block per SM keeps two rows in shared memory;
// while it works on one, the next arrives by a bulk copy (mbarrier completion) and the previous one leaves by a bulk
// store, so HBM stays busy through the compute passes.  Used when two rows fit (vocabulary up to ~56 k).
__global__ void __launch_bounds__(1024, 1)
    softmax_ce_pipe_kernel(__half *__restrict__ logits, int rows, int V, const float *__restrict__ bias, const int *__restrict__ target,
                           float gscale, float *__restrict__ logp_sum, int write_grad, int32_t *status)
{
    extern __shared__ __align__(128) uint8_t sm_rows[];
    __shared__ float red[32];
    __shared__ float x_tgt_s;
    __shared__ uint64_t full_bar[2];
    __shared__ int abort_s;
    const int tid = threadIdx.x, nthr = blockDim.x, nvec = V / 8;
    const uint32_t row_bytes = (uint32_t)V * 2;
    const uint32_t buf_bytes = (row_bytes + 127) & ~127u;
    if (tid == 0) {
        mbar_init(smem_u32(&full_bar[0]), 1);
        mbar_init(smem_u32(&full_bar[1]), 1);
        abort_s = 0;
        fence_barrier_init();
    }
    __syncthreads();
    volatile int *abort_flag = &abort_s;
    const int first = blockIdx.x, step = gridDim.x;
    if (tid == 0 && first < rows) {
        mbar_arrive_expect_tx(smem_u32(&full_bar[0]), row_bytes);
        bulk_load(smem_u32(sm_rows), logits + (size_t)first * V, row_bytes, smem_u32(&full_bar[0]));
    }
    int it = 0;
    for (int row = first; row < rows; row += step, ++it) {
        const int b = it & 1;
        uint4 *row_s4 = (uint4 *)(sm_rows + (size_t)b * buf_bytes);
        uint4 *dst = (uint4 *)(logits + (size_t)row * V);
        const int tgt = target[row];
        const bool ok = mbar_wait(smem_u32(&full_bar[b]), (it >> 1) & 1, abort_flag);
        if (!__syncthreads_and(ok))
            break;
        float mx = 0.f; // the reference starts the maximum at 0 and takes it over the logits without bias
        if (tgt >= 0) {
            __half2 m2 = __float2half2_rn(0.f); // the values are fp16: their maximum is exact in packed fp16 arithmetic
            for (int i = tid; i < nvec; i += nthr) {
                const uint4 raw = row_s4[i];
                const __half2 *h = (const __half2 *)&raw;
                m2 = __hmax2(m2, __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3])));
            }
            mx = fmaxf(__low2float(m2), __high2float(m2));
        }
        // the other buffer: its row left by a bulk store at the end of the previous iteration, which has had the pass
        // above to read shared memory; once it has, the next row may come in
        if (tid == 0 && row + step < rows) {
            bulk_wait_read<0>();
            mbar_arrive_expect_tx(smem_u32(&full_bar[b ^ 1]), row_bytes);
            bulk_load(smem_u32(sm_rows + (size_t)(b ^ 1) * buf_bytes), logits + (size_t)(row + step) * V, row_bytes, smem_u32(&full_bar[b ^ 1]));
        }
        if (tgt < 0) { // no target: zero gradient
            if (write_grad) {
                for (int i = tid; i < nvec; i += nthr)
                    row_s4[i] = make_uint4(0, 0, 0, 0);
                fence_proxy_async();
                __syncthreads();
                if (tid == 0) {
                    bulk_store(dst, smem_u32(row_s4), row_bytes);
                    bulk_commit();
                }
            }
            continue;
        }
        mx = warp_max(mx);
        if ((tid & 31) == 0)
            red[tid >> 5] = mx;
        __syncthreads();
        mx = warp_max((tid & 31) < nthr / 32 ? red[tid & 31] : 0.f); // at most 32 warps: one partial per lane
        __syncthreads();
        float sum0 = 0.f, sum1 = 0.f;
        // the bias vector (4 bytes per logit, as many bytes as two rows) comes from L2 every row: the loads of the next
        // vector are issued before this one's arithmetic
        float4 nb0 = make_float4(0, 0, 0, 0), nb1 = nb0;
        if (bias && tid < nvec)
            nb0 = __ldg((const float4 *)(bias + 8 * tid)), nb1 = __ldg((const float4 *)(bias + 8 * tid) + 1);
        for (int i = tid; i < nvec; i += nthr) {
            uint4 raw = row_s4[i];
            __half2 *h = (__half2 *)&raw;
            float bv[8];
            if (bias) {
                const float4 b0 = nb0, b1 = nb1;
                if (i + nthr < nvec)
                    nb0 = __ldg((const float4 *)(bias + 8 * (i + nthr))), nb1 = __ldg((const float4 *)(bias + 8 * (i + nthr)) + 1);
                bv[0] = b0.x, bv[1] = b0.y, bv[2] = b0.z, bv[3] = b0.w, bv[4] = b1.x, bv[5] = b1.y, bv[6] = b1.z, bv[7] = b1.w;
            }
            if (i == (tgt >> 3)) { // the vector that holds the target's logit: keep it before it is overwritten
                const int kk = tgt & 7;
                const uint32_t wsel = (kk >> 1) == 0 ? raw.x : (kk >> 1) == 1 ? raw.y : (kk >> 1) == 2 ? raw.z : raw.w;
                const __half_raw hr = {(unsigned short)((kk & 1) ? (wsel >> 16) : (wsel & 0xffffu))};
                x_tgt_s = __half2float(__half(hr)) + (bias ? __ldg(bias + tgt) : 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                const float x0 = f.x + (bias ? bv[2 * j] : 0.f), x1 = f.y + (bias ? bv[2 * j + 1] : 0.f);
                float e0, e1;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(x0 - mx));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(x1 - mx));
                sum0 += e0;
                sum1 += e1;
                h[j] = sat_half2(e0, e1);
            }
            row_s4[i] = raw;
        }
        float sum = warp_sum(sum0 + sum1);
        if ((tid & 31) == 0)
            red[tid >> 5] = sum;
        __syncthreads();
        sum = warp_sum((tid & 31) < nthr / 32 ? red[tid & 31] : 0.f);
        const float inv = 1.f / sum;
        if (tid == 0)
            atomicAdd(logp_sum, (x_tgt_s - mx) * 0.69314718f - logf(sum));
        if (write_grad) {
            const float ninv = -inv * gscale;
            for (int i = tid; i < nvec; i += nthr) { // every thread revisits the vectors it wrote itself
                uint4 raw = row_s4[i];
                __half2 *h = (__half2 *)&raw;
                float gt = 0.f; // gradient of the target's logit, computed in fp32 from the same e before it is replaced
                if (i == (tgt >> 3)) {
                    const int kk = tgt & 7;
                    const uint32_t wsel = (kk >> 1) == 0 ? raw.x : (kk >> 1) == 1 ? raw.y : (kk >> 1) == 2 ? raw.z : raw.w;
                    const __half_raw hr = {(unsigned short)((kk & 1) ? (wsel >> 16) : (wsel & 0xffffu))};
                    gt = fmaf(__half2float(__half(hr)), ninv, gscale);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 e = __half22float2(h[j]);
                    h[j] = sat_half2(e.x * ninv, e.y * ninv);
                }
                if (i == (tgt >> 3)) {
                    const int kk = tgt & 7;
                    const unsigned short gb = __half_as_ushort(__float2half_rn(gt));
                    auto patch = [&](uint32_t w, int idx) {
                        return (kk >> 1) != idx ? w : (kk & 1) ? ((w & 0x0000ffffu) | ((uint32_t)gb << 16)) : ((w & 0xffff0000u) | gb);
                    };
                    raw.x = patch(raw.x, 0), raw.y = patch(raw.y, 1), raw.z = patch(raw.z, 2), raw.w = patch(raw.w, 3);
                }
                row_s4[i] = raw;
            }
            fence_proxy_async(); // the bulk store reads shared memory through the async proxy
            __syncthreads();
            if (tid == 0) {
                bulk_store(dst, smem_u32(row_s4), row_bytes);
                bulk_commit();
            }
        } else {
            // the sum pass wrote e back into this buffer through the generic proxy and the next bulk copy into it goes
            // through the async proxy: order them (the gradient path above has the same fence before its store)
            fence_proxy_async();
            __syncthreads(); // red[] and x_tgt_s are reused by the next row
        }
    }
    if (tid == 0) {
        bulk_wait_read<0>(); // shared memory must outlive the stores that read it
        if (abort_s)
            atomicOr(status, TS2_STATUS_WAIT_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------
// Debug trace: order-independent checksum (sum of the 32-bit words as a 64-bit integer, so equal buffers give equal
// sums whatever the thread order), the number of non-finite elements and the largest finite magnitude of a buffer.
// kind 0: raw words, 1: fp32, 2: fp16 pairs.  out[0] += sum, out[1] += non-finite count, out[2] = max(out[2], bits
// of the largest finite |x| as fp32).
__global__ void checksum_kernel(const uint32_t *__restrict__ p, size_t nwords, int kind, unsigned long long *__restrict__ out)
{
    unsigned long long sum = 0, bad = 0;
    float mx = 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t w = p[i];
        sum += w;
        if (kind == 1) {
            if ((w & 0x7f800000u) == 0x7f800000u)
                ++bad;
            else
                mx = fmaxf(mx, fabsf(__uint_as_float(w)));
        } else if (kind == 2) {
            const float2 f = __half22float2(*(const __half2 *)&w);
            if ((w & 0x7c00u) == 0x7c00u)
                ++bad;
            else
                mx = fmaxf(mx, fabsf(f.x));
            if ((w & 0x7c000000u) == 0x7c000000u)
                ++bad;
            else
                mx = fmaxf(mx, fabsf(f.y));
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        bad += __shfl_xor_sync(0xffffffffu, bad, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(out, sum);
        if (bad)
            atomicAdd(out + 1, bad);
        if (mx > 0.f)
            atomicMax(out + 2, (unsigned long long)__float_as_uint(mx));
    }
}

int checksum(const Ctx &c, const void *p, size_t bytes, int kind, unsigned long long *out)
{
    const size_t nwords = bytes / 4;
    const int grid = (int)std::max<size_t>(1, std::min<size_t>(ceil_div(nwords, 256 * 8), (size_t)sm_count(c.device) * 8));
    checksum_kernel<<<grid, 256, 0, c.stream>>>((const uint32_t *)p, nwords, kind, out);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int softmax_ce(const Ctx &c, __half *logits, int rows, int V, const float *bias, const int *target, float gscale, float *logp_sum,
               bool write_grad)
{
    if (V % 8)
        return fail(TS2_ERR_INVALID_ARG, "softmax_ce: vocabulary must be a multiple of 8");
    const size_t two_rows = 2 * (((size_t)V * sizeof(__half) + 127) & ~(size_t)127);
    if (two_rows <= 224 * 1024) {
        static bool configured_pipe[16] = {};
        if (!configured_pipe[c.device & 15]) {
            TS2_CUDA(cudaFuncSetAttribute(softmax_ce_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
            configured_pipe[c.device & 15] = true;
        }
        int32_t *status = device_status_word(c.device);
        if (!status)
            return fail(TS2_ERR_CUDA, "softmax_ce: no device status word");
        const int grid = std::min(rows, sm_count(c.device));
        softmax_ce_pipe_kernel<<<grid, 1024, two_rows, c.stream>>>(logits, rows, V, bias, target, gscale, logp_sum, write_grad ? 1 : 0, status);
        TS2_CHECK_LAUNCH();
        return TS2_OK;
    }
    const size_t smem = (size_t)V * sizeof(__half);
    static bool configured[16] = {};
    if (smem > 48 * 1024 && !configured[c.device & 15]) {
        TS2_CUDA(cudaFuncSetAttribute(softmax_ce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[c.device & 15] = true;
    }
    if (smem > 200 * 1024)
        return fail(TS2_ERR_TOO_LARGE, "softmax_ce: vocabulary %d does not fit the shared-memory row buffer", V);
    const int grid = std::min(rows, sm_count(c.device) * 2);
    softmax_ce_kernel<<<grid, 512, smem, c.stream>>>(logits, rows, V, bias, target, gscale, logp_sum, write_grad ? 1 : 0);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
