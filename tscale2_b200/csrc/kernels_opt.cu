// Gradient apply and weight requantisation: the arithmetic of the reference's MatrixRowSum2Kernel,
// UpdateGlobalRowDisp, AddGradientKernel (src/gpt/matrix/agpu_cuda.cu:32-134) and ConvertMatrixKernel
// (src/gpt/matrix/agpu_cuda.cuh:63-101), restructured from one chain of launches per matrix into a few launches
// over flat buffers that hold every matrix, so that a data-parallel rank can own any contiguous part of them.
// The requantiser's output is also copied transposed for the dX contractions, so no per-step transpose remains.
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int WARPS = 8;
static constexpr int THREADS = WARPS * 32;

__global__ void fill_vector_kernel(float *dst, int n, float value, const float *dyn, int reciprocal)
{
    float v = value;
    if (dyn)
        v = reciprocal ? value / *dyn : value * *dyn;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        dst[i] = v;
}

// ---------------------------------------------------------------------------------
// Flat, sharded form of the optimizer and the requantiser.  All matrices live in flat buffers (weights, momentum,
// gradient) in matrix order, grouped into buckets (embedding, final layer, one per layer).  A rank owns one
// contiguous element range of every bucket (the whole bucket without data parallelism); OptSeg describes the part
// of one matrix that falls into such a range.  Work items are (segment, row) pairs: one warp per row part, so every
// per-row sum has a fixed order and nothing needs atomics.  Per-row results go to vectors indexed by a global row
// number (rows of all matrices in matrix order); rows cut by a range boundary are completed by the data-parallel
// sum of those vectors.  This replaces the per-matrix chains MatrixRowSum2Kernel -> UpdateGlobalRowDisp ->
// AddGradientKernel -> ConvertMatrixKernel of the reference (agpu_cuda.cu:32-134, agpu_cuda.cuh:63-101) by five
// launches per step over everything a rank owns.

// binary search: the segment that holds work item `item`
__device__ __forceinline__ int find_seg(const OptSeg *__restrict__ segs, int nseg, int item)
{
    int lo = 0, hi = nseg - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (segs[mid].item0 <= item)
            lo = mid;
        else
            hi = mid - 1;
    }
    return lo;
}

// columns [c0, c1) of row r of the segment's matrix that belong to the range
__device__ __forceinline__ void seg_row_cols(const OptSeg &sg, int r, long long &base, int &c0, int &c1)
{
    const long long row_begin = (long long)r * sg.x;
    c0 = (int)(max(row_begin, sg.a) - row_begin);
    c1 = (int)(min(row_begin + sg.x, sg.b) - row_begin);
    base = sg.flat_off + row_begin;
}

__global__ void opt_row_sum2_kernel(const OptSeg *__restrict__ segs, int nseg, int nitems, const float *__restrict__ grad,
                                    float *__restrict__ rowsum)
{
    const int lane = threadIdx.x & 31;
    for (int item = blockIdx.x * WARPS + (threadIdx.x >> 5); item < nitems; item += gridDim.x * WARPS) {
        const OptSeg sg = segs[find_seg(segs, nseg, item)];
        const int r = sg.row0 + (item - sg.item0);
        long long base;
        int c0, c1;
        seg_row_cols(sg, r, base, c0, c1);
        const float4 *src = (const float4 *)(grad + base);
        float s = 0.f;
        for (int i = c0 / 4 + lane; i < c1 / 4; i += 32) {
            const float4 v = src[i];
            s += dot4(v, v);
        }
        s = warp_sum(s);
        if (lane == 0)
            rowsum[sg.grow0 + r] = s;
    }
}

// one block per matrix: dispersion EMA -> row scale for every row of the matrix (UpdateGlobalRowDisp)
__global__ void opt_disp_kernel(const OptMat *__restrict__ mats, const float *__restrict__ rowsum, float disp_decay,
                                float *__restrict__ row_scale)
{
    __shared__ float red[32];
    __shared__ float bcast;
    const OptMat mt = mats[blockIdx.x];
    const float *sum2 = rowsum + mt.grow0;
    float *rs_out = row_scale + mt.grow0;
    const long long step = mt.y / mt.row_disp_size;
    const float sw = *mt.sum_weight * disp_decay + 1.f;
    const float norm = 1.f / sw;
    if (step == 1) {
        for (long long r = threadIdx.x; r < mt.y; r += blockDim.x) {
            const float rd = mt.row_disp[r] * disp_decay + sum2[r] / (float)mt.x;
            mt.row_disp[r] = rd;
            const float d = rd * norm;
            rs_out[r] = d > 0.f ? 1.f / sqrtf(d) : 0.f;
        }
    } else {
        for (int b = 0; b < mt.row_disp_size; ++b) {
            float s = 0.f;
            for (long long k = threadIdx.x; k < step; k += blockDim.x)
                s += sum2[b * step + k];
            s = warp_sum(s);
            if ((threadIdx.x & 31) == 0)
                red[threadIdx.x >> 5] = s;
            __syncthreads();
            if (threadIdx.x == 0) {
                float tot = 0.f;
                for (int i = 0; i < (int)blockDim.x / 32; ++i)
                    tot += red[i];
                const float rd = mt.row_disp[b] * disp_decay + tot / ((float)mt.x * (float)step);
                mt.row_disp[b] = rd;
                const float d = rd * norm;
                bcast = d > 0.f ? 1.f / sqrtf(d) : 0.f;
            }
            __syncthreads();
            const float rs = bcast;
            for (long long k = threadIdx.x; k < step; k += blockDim.x)
                rs_out[b * step + k] = rs;
            __syncthreads();
        }
    }
    __syncthreads();
    if (threadIdx.x == 0)
        *mt.sum_weight = sw;
}

// AddGradientKernel on the rows of the range (UPDATE) and the sum of squares of the (new) weights per row part
template <bool UPDATE>
__global__ void opt_update_kernel(const OptSeg *__restrict__ segs, int nseg, int nitems, const float *__restrict__ grad,
                                  const float *__restrict__ row_scale, ts2_training_step step, float *__restrict__ avg,
                                  float *__restrict__ w, double *__restrict__ roww2)
{
    const int lane = threadIdx.x & 31;
    for (int item = blockIdx.x * WARPS + (threadIdx.x >> 5); item < nitems; item += gridDim.x * WARPS) {
        const OptSeg sg = segs[find_seg(segs, nseg, item)];
        const int r = sg.row0 + (item - sg.item0);
        long long base;
        int c0, c1;
        seg_row_cols(sg, r, base, c0, c1);
        float4 *ww = (float4 *)(w + base);
        double s = 0.0;
        if (UPDATE) {
            const float rs = row_scale[sg.grow0 + r];
            const float step_mult = step.rate * sqrtf(sg.sparsity);
            const float shrink = 1.f - step_mult * step.l2reg;
            const float beta1 = step.beta1, w0 = step.weight0, w1 = step.weight1;
            const float4 *g = (const float4 *)(grad + base);
            float4 *a = (float4 *)(avg + base);
            for (int i = c0 / 4 + lane; i < c1 / 4; i += 32) {
                const float4 d = scale4(g[i], rs);
                const float4 oa = a[i], ow = ww[i];
                float4 na, nw;
#define TS2_UPD(f)                                         \
    na.f = oa.f * beta1 + d.f * (1.f - beta1);             \
    nw.f = ow.f * shrink + (na.f * w1 + d.f * w0) * step_mult;
                TS2_UPD(x)
                TS2_UPD(y)
                TS2_UPD(z)
                TS2_UPD(w)
#undef TS2_UPD
                a[i] = na;
                ww[i] = nw;
                s += (double)nw.x * nw.x + (double)nw.y * nw.y + (double)nw.z * nw.z + (double)nw.w * nw.w;
            }
        } else {
            for (int i = c0 / 4 + lane; i < c1 / 4; i += 32) {
                const float4 v = ww[i];
                s += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
            }
        }
        for (int o = 16; o > 0; o >>= 1)
            s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0)
            roww2[sg.grow0 + r] = s;
    }
}

// one block per matrix: sko = sqrt(sum of squares / (x y)), rows summed in a fixed order
__global__ void opt_sko_kernel(const OptMat *__restrict__ mats, const double *__restrict__ roww2, float *__restrict__ skos)
{
    __shared__ double red[32];
    const OptMat mt = mats[blockIdx.x];
    double s = 0.0;
    for (long long r = threadIdx.x; r < mt.y; r += blockDim.x)
        s += roww2[mt.grow0 + r];
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < (int)blockDim.x / 32; ++i)
            tot += red[i];
        skos[blockIdx.x] = sqrtf((float)tot / (float)(mt.x * mt.y));
    }
}

// ConvertMatrixKernel on the rows of the range: q = enc(w * 32 / sko) into the matrix's row-major quantized copy
__global__ void opt_quant_kernel(const OptSeg *__restrict__ segs, int nseg, int nitems, const float *__restrict__ w,
                                 const float *__restrict__ skos)
{
    const int lane = threadIdx.x & 31;
    for (int item = blockIdx.x * WARPS + (threadIdx.x >> 5); item < nitems; item += gridDim.x * WARPS) {
        const OptSeg sg = segs[find_seg(segs, nseg, item)];
        const int r = sg.row0 + (item - sg.item0);
        long long base;
        int c0, c1;
        seg_row_cols(sg, r, base, c0, c1);
        const float sko = skos[sg.mat];
        const float mult = (sko == 0.f) ? 0.f : (1.f / (sko * (1.f / 32)));
        const float4 *src = (const float4 *)(w + base);
        uint8_t *dst = sg.qbase + (size_t)r * sg.x * sg.qsize;
        for (int i = c0 / 4 + lane; i < c1 / 4; i += 32) {
            const float4 v = scale4(src[i], mult);
            if (sg.qkind == 2) { // int8: nearest even, saturating (PackFloatToInt8, src/gpt/model_params/sse_utils.h:56-78)
                *(uint32_t *)(dst + 4 * (size_t)i) = sat_i8(v.x) | (sat_i8(v.y) << 8) | (sat_i8(v.z) << 16) | (sat_i8(v.w) << 24);
            } else if (sg.qkind == 0) {
                const uint32_t pk = (uint32_t)encode_e4m3_weight(v.x) | ((uint32_t)encode_e4m3_weight(v.y) << 8) |
                                    ((uint32_t)encode_e4m3_weight(v.z) << 16) | ((uint32_t)encode_e4m3_weight(v.w) << 24);
                *(uint32_t *)(dst + 4 * (size_t)i) = pk;
            } else {
                const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y), h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
                *(uint2 *)(dst + 8 * (size_t)i) =
                    make_uint2((uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16),
                               (uint32_t)__half_as_ushort(h2) | ((uint32_t)__half_as_ushort(h3) << 16));
            }
        }
    }
}

static int opt_grid(const Ctx &c, int nitems)
{
    return (int)std::max<long long>(1, std::min<long long>(ceil_div(nitems, WARPS), (long long)sm_count(c.device) * 8));
}

int opt_row_sum2(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *grad, float *rowsum)
{
    if (nitems <= 0)
        return TS2_OK;
    opt_row_sum2_kernel<<<opt_grid(c, nitems), THREADS, 0, c.stream>>>(segs, nseg, nitems, grad, rowsum);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int opt_disp(const Ctx &c, const OptMat *mats, int n_mats, const float *rowsum, float disp_decay, float *row_scale)
{
    opt_disp_kernel<<<n_mats, 1024, 0, c.stream>>>(mats, rowsum, disp_decay, row_scale);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int opt_update(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *grad, const float *row_scale,
               const ts2_training_step *step, float *avg, float *w, double *roww2)
{
    if (nitems <= 0)
        return TS2_OK;
    if (step)
        opt_update_kernel<true><<<opt_grid(c, nitems), THREADS, 0, c.stream>>>(segs, nseg, nitems, grad, row_scale, *step, avg, w, roww2);
    else
        opt_update_kernel<false><<<opt_grid(c, nitems), THREADS, 0, c.stream>>>(segs, nseg, nitems, nullptr, nullptr, ts2_training_step(),
                                                                                 nullptr, w, roww2);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int opt_sko(const Ctx &c, const OptMat *mats, int n_mats, const double *roww2, float *skos)
{
    opt_sko_kernel<<<n_mats, 1024, 0, c.stream>>>(mats, roww2, skos);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int opt_quantize(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *w, const float *skos)
{
    if (nitems <= 0)
        return TS2_OK;
    opt_quant_kernel<<<opt_grid(c, nitems), THREADS, 0, c.stream>>>(segs, nseg, nitems, w, skos);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// Copy of a block of already quantized values (ES bytes per element) into another row-major place and / or its
// transpose: 32x32 tiles, both sides coalesced.  TH: the transposed copy holds the value widened to fp16 (1: from e4m3,
// 2: from int8), 0: copied as it is.
template <int ES, int TH>
__global__ void qcopy_kernel(const void *__restrict__ src, long long x, long long y, long long ld_src, void *__restrict__ dst,
                             long long ld, void *__restrict__ dstT, long long ldT)
{
    using QT = typename std::conditional<ES == 1, uint8_t, uint16_t>::type;
    using TT = typename std::conditional<TH != 0, uint16_t, QT>::type;
    __shared__ QT tile[32][33];
    const long long x0 = (long long)blockIdx.x * 32, y0 = (long long)blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const long long yy = y0 + r, xx = x0 + threadIdx.x;
        QT qv = QT();
        if (yy < y && xx < x) {
            qv = ((const QT *)src)[yy * ld_src + xx];
            if (dst)
                ((QT *)dst)[yy * ld + xx] = qv;
        }
        tile[r][threadIdx.x] = qv;
    }
    if (!dstT)
        return;
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const long long xx = x0 + r, yy = y0 + threadIdx.x;
        if (xx < x && yy < y) {
            const QT qv = tile[threadIdx.x][r];
            if constexpr (TH == 1 && ES == 1) {
                __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)qv, __NV_E4M3);
                ((uint16_t *)dstT)[xx * ldT + yy] = h2.x;
            } else if constexpr (TH == 2 && ES == 1) {
                ((uint16_t *)dstT)[xx * ldT + yy] = __half_as_ushort(__float2half_rn((float)(int8_t)qv));
            } else {
                ((TT *)dstT)[xx * ldT + yy] = qv;
            }
        }
    }
}

int qcopy_block(const Ctx &c, const void *src, int64_t x, int64_t y, int64_t ld_src, int elem_size, void *dst, int64_t ld, void *dstT,
                int64_t ldT, int transposed_as_half)
{
    dim3 g((unsigned)ceil_div(x, 32), (unsigned)ceil_div(y, 32)), b(32, 8);
    if (elem_size == 1 && transposed_as_half == 1)
        qcopy_kernel<1, 1><<<g, b, 0, c.stream>>>(src, x, y, ld_src, dst, ld, dstT, ldT);
    else if (elem_size == 1 && transposed_as_half == 2)
        qcopy_kernel<1, 2><<<g, b, 0, c.stream>>>(src, x, y, ld_src, dst, ld, dstT, ldT);
    else if (elem_size == 1)
        qcopy_kernel<1, 0><<<g, b, 0, c.stream>>>(src, x, y, ld_src, dst, ld, dstT, ldT);
    else
        qcopy_kernel<2, 0><<<g, b, 0, c.stream>>>(src, x, y, ld_src, dst, ld, dstT, ldT);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// the scale vectors of one dense layer from its matrix scales (skos of the layer's matrices, in matrix order):
// forward column scales a (x sko_k for the K block of an attention layer), dW row scales 1 / sko for the matrices
// that are followed by a normalisation (Q, K, V; Expand), 1 elsewhere
__global__ void layer_scales_kernel(float *__restrict__ fwd_col, float *__restrict__ bwd_row, int W, int ncat, int is_att, float a,
                                    const float *__restrict__ skos)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ncat * W; i += gridDim.x * blockDim.x) {
        const int j = i / W;
        fwd_col[i] = (is_att && j == 1) ? a * skos[1] : a;
        const bool scaled = is_att ? j < 3 : j == 0;
        bwd_row[i] = scaled ? 1.f / skos[j] : 1.f;
    }
}

int layer_scales(const Ctx &c, float *fwd_col, float *bwd_row, int W, int ncat, bool is_att, float a, const float *skos)
{
    layer_scales_kernel<<<std::max(1, std::min(64, (ncat * W + 255) / 256)), 256, 0, c.stream>>>(fwd_col, bwd_row, W, ncat, is_att ? 1 : 0,
                                                                                              a, skos);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int fill_vector(const Ctx &c, float *dst, int n, float value, const float *dyn, bool reciprocal_dyn)
{
    fill_vector_kernel<<<std::max(1, std::min(64, (n + 255) / 256)), 256, 0, c.stream>>>(dst, n, value, dyn, reciprocal_dyn ? 1 : 0);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
