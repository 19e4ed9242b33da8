// Gradient apply and weight requantisation for one matrix: the reference's
// MatrixRowSum2Kernel, UpdateGlobalRowDisp, AddGradientKernel (src/gpt/matrix/agpu_cuda.cu:32-134)
// and ConvertMatrixKernel (src/gpt/matrix/agpu_cuda.cuh:63-101).  The requantiser also writes
// the transposed copy that the dX contraction reads, so no per-step transpose remains.
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int WARPS = 8;
static constexpr int THREADS = WARPS * 32;

__global__ void row_sum2_kernel(const float *__restrict__ m, long long x, long long y, float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    for (long long row = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5); row < y; row += (long long)gridDim.x * WARPS) {
        const float4 *src = (const float4 *)(m + row * x);
        float s = 0.f;
        for (long long i = lane; i < x / 4; i += 32) {
            float4 v = src[i];
            s += dot4(v, v);
        }
        s = warp_sum(s);
        if (lane == 0)
            out[row] = s;
    }
}

// single block: dispersion EMA per row block -> row scale (UpdateGlobalRowDisp)
__global__ void update_row_disp_kernel(long long x, long long y, int row_disp_size, const float *__restrict__ sum2,
                                       float disp_decay, float *__restrict__ sum_weight, float *__restrict__ row_disp,
                                       float *__restrict__ row_scale)
{
    __shared__ float red[32];
    __shared__ float bcast;
    const long long step = y / row_disp_size;
    const float sw = *sum_weight * disp_decay + 1.f;
    const float norm = 1.f / sw;
    if (step == 1) {
        for (long long r = threadIdx.x; r < y; r += blockDim.x) {
            const float rd = row_disp[r] * disp_decay + sum2[r] / (float)x;
            row_disp[r] = rd;
            const float d = rd * norm;
            row_scale[r] = d > 0.f ? 1.f / sqrtf(d) : 0.f;
        }
    } else {
        for (int b = 0; b < row_disp_size; ++b) {
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
                const float rd = row_disp[b] * disp_decay + tot / ((float)x * (float)step);
                row_disp[b] = rd;
                const float d = rd * norm;
                bcast = d > 0.f ? 1.f / sqrtf(d) : 0.f;
            }
            __syncthreads();
            const float rs = bcast;
            for (long long k = threadIdx.x; k < step; k += blockDim.x)
                row_scale[b * step + k] = rs;
            __syncthreads();
        }
    }
    __syncthreads();
    if (threadIdx.x == 0)
        *sum_weight = sw;
}

__global__ void add_gradient_kernel(long long x, long long y, const float *__restrict__ grad, const float *__restrict__ row_scale,
                                    float step_mult, float shrink, float beta1, float w0, float w1, float *__restrict__ avg,
                                    float *__restrict__ w)
{
    const int lane = threadIdx.x & 31;
    for (long long row = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5); row < y; row += (long long)gridDim.x * WARPS) {
        const float rs = row_scale[row];
        const float4 *g = (const float4 *)(grad + row * x);
        float4 *a = (float4 *)(avg + row * x), *ww = (float4 *)(w + row * x);
        for (long long i = lane; i < x / 4; i += 32) {
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
        }
    }
}

int apply_gradient(const Ctx &c, const OptMatrix &m, const ts2_training_step &step)
{
    if (m.x % 4 || m.row_disp_size <= 0 || m.y % m.row_disp_size)
        return fail(TS2_ERR_INVALID_ARG, "apply_gradient: bad shape");
    const int grid = (int)std::max<long long>(1, std::min<long long>(ceil_div(m.y, WARPS), (long long)sm_count(c.device) * 8));
    row_sum2_kernel<<<grid, THREADS, 0, c.stream>>>(m.grad, m.x, m.y, m.row_sum2);
    TS2_CHECK_LAUNCH();
    update_row_disp_kernel<<<1, 1024, 0, c.stream>>>(m.x, m.y, m.row_disp_size, m.row_sum2, step.disp_decay, m.sum_weight, m.row_disp,
                                                     m.row_scale);
    TS2_CHECK_LAUNCH();
    const float step_mult = step.rate * sqrtf(m.sparsity);
    const float shrink = 1.f - step_mult * step.l2reg;
    add_gradient_kernel<<<grid, THREADS, 0, c.stream>>>(m.x, m.y, m.grad, m.row_scale, step_mult, shrink, step.beta1, step.weight0,
                                                        step.weight1, m.avg_grad, m.w);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// requantisation: sko = sqrt(sum w^2 / (x*y)) (double accumulation), q = enc(w * 32 / sko)

__global__ void row_sum2_double_kernel(const float *__restrict__ m, long long x, long long y, double *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    for (long long row = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5); row < y; row += (long long)gridDim.x * WARPS) {
        const float *src = m + row * x;
        double s = 0.0;
        for (long long i = lane; i < x; i += 32)
            s += (double)src[i] * (double)src[i];
        for (int o = 16; o > 0; o >>= 1)
            s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0)
            out[row] = s;
    }
}

__global__ void sko_kernel(const double *__restrict__ row_sum2, long long x, long long y, float *__restrict__ sko_out)
{
    __shared__ double red[32];
    double s = 0.0;
    for (long long r = threadIdx.x; r < y; r += blockDim.x)
        s += row_sum2[r];
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < (int)blockDim.x / 32; ++i)
            tot += red[i];
        *sko_out = sqrtf((float)tot / (float)(x * y));
    }
}

// 32x32 tiles: coalesced reads of w, coalesced writes of both the row-major and the transposed copy
// TH: the transposed copy holds the quantized value widened to fp16 (exact for e4m3)
template <int FT, bool TH>
__global__ void convert_kernel(const float *__restrict__ w, long long x, long long y, const float *__restrict__ sko_ptr,
                               void *__restrict__ dst, long long ld, void *__restrict__ dstT, long long ldT)
{
    using QT = typename std::conditional<FT == 0, uint8_t, __half>::type;
    using TT = typename std::conditional<TH, __half, QT>::type;
    __shared__ QT tile[32][33];
    const float sko = *sko_ptr;
    const float discr = sko * (1.f / 32);
    const float mult = (sko == 0.f) ? 0.f : (1.f / discr);
    const long long x0 = (long long)blockIdx.x * 32, y0 = (long long)blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const long long yy = y0 + r, xx = x0 + threadIdx.x;
        QT qv = QT();
        if (yy < y && xx < x) {
            const float v = w[yy * x + xx] * mult;
            if constexpr (FT == 0)
                qv = encode_e4m3_weight(v);
            else
                qv = __float2half_rn(v);
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
            if constexpr (TH && FT == 0) {
                __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)qv, __NV_E4M3);
                ((__half *)dstT)[xx * ldT + yy] = __ushort_as_half(h2.x);
            } else {
                ((TT *)dstT)[xx * ldT + yy] = qv;
            }
        }
    }
}

int matrix_sko(const Ctx &c, const float *w, int64_t x, int64_t y, float *sko_out, float *scratch)
{
    // scratch holds y doubles
    const int grid = (int)std::max<long long>(1, std::min<long long>(ceil_div(y, WARPS), (long long)sm_count(c.device) * 8));
    row_sum2_double_kernel<<<grid, THREADS, 0, c.stream>>>(w, x, y, (double *)scratch);
    TS2_CHECK_LAUNCH();
    sko_kernel<<<1, 1024, 0, c.stream>>>((const double *)scratch, x, y, sko_out);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int requantize(const Ctx &c, const float *w, int64_t x, int64_t y, int quant, void *dst, int64_t ld, void *dstT, int64_t ldT,
               float *sko_out, float *scratch, bool transposed_as_half)
{
    int rc = matrix_sko(c, w, x, y, sko_out, scratch);
    if (rc != TS2_OK)
        return rc;
    return convert_block(c, w, x, y, quant, dst, ld, dstT, ldT, sko_out, transposed_as_half);
}

int convert_block(const Ctx &c, const float *w, int64_t x, int64_t y, int quant, void *dst, int64_t ld, void *dstT, int64_t ldT,
                  const float *sko_out, bool transposed_as_half)
{
    dim3 g((unsigned)ceil_div(x, 32), (unsigned)ceil_div(y, 32)), b(32, 8);
    if (quant == 0 && transposed_as_half)
        convert_kernel<0, true><<<g, b, 0, c.stream>>>(w, x, y, sko_out, dst, ld, dstT, ldT);
    else if (quant == 0)
        convert_kernel<0, false><<<g, b, 0, c.stream>>>(w, x, y, sko_out, dst, ld, dstT, ldT);
    else
        convert_kernel<1, false><<<g, b, 0, c.stream>>>(w, x, y, sko_out, dst, ld, dstT, ldT);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

__global__ void fill_vector_kernel(float *dst, int n, float value, const float *dyn, int reciprocal)
{
    float v = value;
    if (dyn)
        v = reciprocal ? value / *dyn : value * *dyn;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        dst[i] = v;
}

int fill_vector(const Ctx &c, float *dst, int n, float value, const float *dyn, bool reciprocal_dyn)
{
    fill_vector_kernel<<<std::max(1, std::min(64, (n + 255) / 256)), 256, 0, c.stream>>>(dst, n, value, dyn, reciprocal_dyn ? 1 : 0);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
