// extern "C" operator-level entry points of include/ts2_b200.h (device helpers and
// the contraction kernels).  Plain pointers and sizes only.
#include "gemm.cuh"
#include "kernels.cuh"
#include <vector>

namespace ts2 {
const char *global_error();

}
using namespace ts2;

static int kind_of(int prec)
{
    switch (prec) {
    case TS2_PREC_FP8: return KIND_E4M3;
    case TS2_PREC_F16: return KIND_F16;
    case TS2_PREC_INT8: return KIND_I8;
    default: return -1;
    }
}

extern "C" {

int ts2_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess)
        return 0;
    return n;
}

int ts2_dev_alloc(int device, size_t bytes, void **ptr)
{
    if (!ptr)
        return fail(TS2_ERR_INVALID_ARG, "ts2_dev_alloc: null out pointer");
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaMalloc(ptr, bytes ? bytes : 16));
    return TS2_OK;
}

int ts2_dev_free(int device, void *ptr)
{
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaFree(ptr));
    return TS2_OK;
}

int ts2_dev_upload(int device, void *dst, const void *host_src, size_t bytes)
{
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaMemcpy(dst, host_src, bytes, cudaMemcpyHostToDevice));
    return TS2_OK;
}

int ts2_dev_download(int device, void *host_dst, const void *src, size_t bytes)
{
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_dev_memset(int device, void *dst, int value, size_t bytes)
{
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaMemset(dst, value, bytes));
    return TS2_OK;
}

// Synchronizes the device and reports (and clears) the status word that kernels OR
// error bits into when a bounded wait gives up.
int ts2_dev_sync(int device)
{
    TS2_CUDA(cudaSetDevice(device));
    TS2_CUDA(cudaDeviceSynchronize());
    return collect_device_status(device);
}

// One CTA waits, with the library's bounded wait, on an mbarrier nothing ever arrives at: the wait gives up after its
// limit (about 1.5e9 clocks, under a second), the kernel ORs the time-out bit into the status word and returns.
__global__ void wait_limit_selftest_kernel(int32_t *status)
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

int ts2_selftest_wait_limit(int device)
{
    TS2_CUDA(cudaSetDevice(device));
    int32_t *w = device_status_word(device);
    if (!w)
        return fail(TS2_ERR_CUDA, "no device status word");
    wait_limit_selftest_kernel<<<1, 32>>>(w);
    TS2_CHECK_LAUNCH();
    return ts2_dev_sync(device);
}

int ts2_gemm_tn(int device, void *stream, int prec, int out_kind, int64_t M, int64_t N, int64_t K, const void *A,
                int64_t lda, const void *B, int64_t ldb, void *C, int64_t ldc, float alpha, const float *row_scale,
                const float *col_scale)
{
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    a.kind = kind_of(prec);
    if (a.kind < 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_tn: unknown precision %d", prec);
    a.mn_major = false;
    a.M = M, a.N = N, a.K = K;
    a.A = A, a.lda = lda, a.B = B, a.ldb = ldb, a.C = C, a.ldc = ldc;
    a.epi.alpha = alpha;
    a.epi.row_scale = row_scale;
    a.epi.col_scale = col_scale;
    a.epi.out_kind = out_kind;
    if (gemm_splits(device, a.kind, false, M, N, K) > 1) {
        // few output tiles and a long K: the scheduler splits K and needs scratch for the partial
        // tiles; this entry point takes it from the stream-ordered allocator for the call.
        size_t need = gemm_workspace_bytes(device, a.kind, false, M, N, K);
        void *ws = nullptr;
        TS2_CUDA(cudaSetDevice(device));
        TS2_CUDA(cudaMallocAsync(&ws, need, a.stream));
        a.workspace = ws;
        a.workspace_bytes = need;
        int rc = gemm(a);
        cudaFreeAsync(ws, a.stream);
        return rc;
    }
    return gemm(a);
}

int ts2_gemm_dx(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                const void *dY, const void *Wt, void *dX, float alpha, const float *row_scale,
                const float *col_scale)
{
    return ts2_gemm_tn(device, stream, prec, out_kind, T, in_dim, out_dim, dY, out_dim, Wt, out_dim, dX, in_dim, alpha, row_scale,
                       col_scale);
}

size_t ts2_gemm_dw_workspace_bytes(int64_t T, int64_t in_dim, int64_t out_dim)
{
    int dev = 0;
    cudaGetDevice(&dev);
    // element size does not change the tiling of M x N; K blocks differ (128 vs 64 tokens), take the larger
    size_t a = gemm_workspace_bytes(dev, KIND_E4M3, true, out_dim, in_dim, T);
    size_t b = gemm_workspace_bytes(dev, KIND_F16, true, out_dim, in_dim, T);
    return a > b ? a : b;
}

int ts2_gemm_dw(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                const void *dY, const void *X, void *dW, float alpha, void *workspace, size_t workspace_bytes)
{
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    a.kind = kind_of(prec);
    if (a.kind < 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw: unknown precision %d", prec);
    a.mn_major = true;
    a.M = out_dim, a.N = in_dim, a.K = T;
    a.A = dY, a.lda = out_dim, a.B = X, a.ldb = in_dim, a.C = dW, a.ldc = in_dim;
    a.epi.alpha = alpha;
    a.epi.out_kind = out_kind;
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    return gemm(a);
}

int ts2_gemm_dw_scaled(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                       const void *dY, const void *X, void *dW, float alpha, const float *row_scale, const float *col_scale,
                       void *workspace, size_t workspace_bytes)
{
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    a.kind = kind_of(prec);
    if (a.kind < 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_scaled: unknown precision %d", prec);
    a.mn_major = true;
    a.M = out_dim, a.N = in_dim, a.K = T;
    a.A = dY, a.lda = out_dim, a.B = X, a.ldb = in_dim, a.C = dW, a.ldc = in_dim;
    a.epi.alpha = alpha;
    a.epi.row_scale = row_scale;
    a.epi.col_scale = col_scale;
    a.epi.out_kind = out_kind;
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    return gemm(a);
}

// grouped contractions of the mixture-of-experts layers (device pointers; tables on the device)
int ts2_gemm_tn_grouped(int device, void *stream, int prec, int out_kind, int64_t rows, int64_t N, int64_t K, const void *A,
                        const void *B, void *C, float alpha, int groups, const int32_t *tile_group)
{
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    a.kind = kind_of(prec);
    if (a.kind < 0 || groups <= 0 || !tile_group)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_tn_grouped: bad arguments");
    a.M = rows, a.N = N, a.K = K;
    a.A = A, a.lda = K, a.B = B, a.ldb = K, a.C = C, a.ldc = N;
    a.epi.alpha = alpha;
    a.epi.out_kind = out_kind;
    a.group_mode = 1;
    a.groups = groups;
    a.tile_group = tile_group;
    a.group_rows_b = (int)N;
    return gemm(a);
}

int ts2_gemm_dw_grouped(int device, void *stream, int prec, int out_kind, int64_t rows, int64_t in_dim, int64_t out_dim,
                        const void *dY, const void *X, void *dW, float alpha, int groups, const int32_t *seg_ptr)
{
    GemmArgs a;
    a.device = device;
    a.stream = (cudaStream_t)stream;
    a.kind = kind_of(prec);
    if (a.kind < 0 || groups <= 0 || !seg_ptr)
        return fail(TS2_ERR_INVALID_ARG, "ts2_gemm_dw_grouped: bad arguments");
    a.mn_major = true;
    a.M = out_dim, a.N = in_dim, a.K = rows;
    a.A = dY, a.lda = out_dim, a.B = X, a.ldb = in_dim, a.C = dW, a.ldc = in_dim;
    a.epi.alpha = alpha;
    a.epi.out_kind = out_kind;
    a.group_mode = 2;
    a.groups = groups;
    a.group_kptr = seg_ptr;
    a.c_group_stride = out_dim * in_dim;
    return gemm(a);
}

// CpuMoe on the device: logits host [T][E] -> ids host [T][k], weights host [T][k]
int ts2_moe_route(int device, const float *logits, int T, int expert_count, int selected, int32_t *ids, float *weights)
{
    if (!logits || !ids || !weights || T <= 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_moe_route: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    float *dl = nullptr, *dw = nullptr;
    int *di = nullptr;
    TS2_CUDA(cudaMalloc(&dl, (size_t)T * expert_count * 4));
    TS2_CUDA(cudaMalloc(&dw, (size_t)T * selected * 4));
    TS2_CUDA(cudaMalloc(&di, (size_t)T * selected * 4));
    TS2_CUDA(cudaMemcpy(dl, logits, (size_t)T * expert_count * 4, cudaMemcpyHostToDevice));
    Ctx c;
    c.device = device;
    int rc = moe_route(c, dl, expert_count, T, expert_count, selected, di, dw);
    if (rc == TS2_OK) {
        cudaMemcpy(ids, di, (size_t)T * selected * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(weights, dw, (size_t)T * selected * 4, cudaMemcpyDeviceToHost);
    }
    cudaFree(dl);
    cudaFree(dw);
    cudaFree(di);
    return rc;
}

// ---- the bandwidth-bound gradient kernels, one call each (device pointers) ----------------------------------------
static Ctx op_ctx(int device, void *stream, int prec)
{
    Ctx c;
    c.device = device;
    c.stream = (cudaStream_t)stream;
    c.ft = prec == TS2_PREC_FP8 ? 0 : prec == TS2_PREC_F16 ? 1 : 2;
    c.s_act = c.ft == 0 ? 16.f : c.ft == 1 ? 1.f : 24.f;
    return c;
}

int ts2_op_tilenorm_backward(int device, void *stream, const float *x, const float *dn, const float *dyn_scale, int T, int D,
                             float *g, int add, uint32_t *absmax_bits)
{
    if (!x || !dn || !g || T <= 0 || D <= 0 || D % 128)
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_tilenorm_backward: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    return tilenorm_backward(op_ctx(device, stream, TS2_PREC_F16), x, dn, dyn_scale, 1.f, T, D, g, add != 0, absmax_bits);
}

int ts2_op_cast_grad(int device, void *stream, int prec, const float *g, int64_t n, const uint32_t *absmax_bits, void *g_fast,
                     float *ginv)
{
    if (!g || !absmax_bits || !g_fast || !ginv || n <= 0 || n % 4 || (prec != TS2_PREC_FP8 && prec != TS2_PREC_F16))
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_cast_grad: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    return cast_grad(op_ctx(device, stream, prec), g, (size_t)n, absmax_bits, g_fast, ginv, 1.f, nullptr, nullptr);
}

int ts2_op_ffn_act_backward(int device, void *stream, int prec, const void *drg, const void *wide_gate, const float *wscale, int T,
                            int F, void *d_wide_gate)
{
    if (!drg || !wide_gate || !wscale || !d_wide_gate || T <= 0 || F <= 0 || F % 128 || (prec != TS2_PREC_FP8 && prec != TS2_PREC_F16))
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_ffn_act_backward: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    return ffn_act_backward(op_ctx(device, stream, prec), (const __half *)drg, (const __half *)wide_gate, (const __half *)wide_gate,
                            2 * F, wscale, T, F, d_wide_gate);
}

int ts2_op_att_gate_backward(int device, void *stream, int prec, const void *drg, const void *qkvg, const void *o, int T, int Q,
                             void *d4, void *dout, float *dscale)
{
    if (!drg || !qkvg || !o || !d4 || !dout || !dscale || T <= 0 || Q <= 0 || Q % 128 || (prec != TS2_PREC_FP8 && prec != TS2_PREC_F16))
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_att_gate_backward: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    return att_gate_backward(op_ctx(device, stream, prec), (const __half *)drg, (const __half *)qkvg, (const __half *)o, T, Q, d4,
                             (__half *)dout, dscale);
}

int ts2_op_rowquant_i8(int device, void *stream, const float *x, int T, int D, int8_t *q, float *row_scale)
{
    if (!x || !q || !row_scale || T <= 0 || D <= 0)
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_rowquant_i8: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    return rowquant_grad(op_ctx(device, stream, TS2_PREC_INT8), x, T, D, nullptr, q, row_scale, nullptr, nullptr, 1.f, nullptr, nullptr);
}

// attention core on device arrays; span_start / span_finish are host arrays of T ints
int ts2_attention_forward(int device, void *stream, int variant, const void *q, const void *k, const void *v, const int32_t *span_start,
                          const int32_t *span_finish, int T, int head_count, float alibi_slope, void *o, float *lse)
{
    if (T <= 0 || head_count <= 0 || !q || !k || !v || !o || !lse || !span_start || !span_finish)
        return fail(TS2_ERR_INVALID_ARG, "ts2_attention_forward: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    int *d = nullptr;
    TS2_CUDA(cudaMalloc(&d, (size_t)T * 8));
    TS2_CUDA(cudaMemcpy(d, span_start, (size_t)T * 4, cudaMemcpyHostToDevice));
    TS2_CUDA(cudaMemcpy(d + T, span_finish, (size_t)T * 4, cudaMemcpyHostToDevice));
    Ctx c;
    c.device = device;
    c.stream = (cudaStream_t)stream;
    int rc = variant == 2 ? attention_forward_tc(c, (const __half *)q, (const __half *)k, (const __half *)v, d, d + T, T, head_count,
                                                 alibi_slope, (__half *)o, lse)
             : variant == 0 ? attention_forward_mma(c, (const __half *)q, (const __half *)k, (const __half *)v, d, d + T, T, head_count,
                                                    alibi_slope, (__half *)o, lse)
                            : attention_forward_rowwise(c, (const __half *)q, (const __half *)k, (const __half *)v, d, d + T, T, head_count,
                                                      alibi_slope, (__half *)o, lse);
    cudaStreamSynchronize(c.stream);
    cudaFree(d);
    return rc;
}

int ts2_attention_backward(int device, void *stream, int variant, const void *q, const void *k, const void *v, const void *dout,
                           const float *lse, const float *dscale, const int32_t *span_start, const int32_t *span_finish, int T,
                           int head_count, float alibi_slope, void *dq, void *dk, void *dv)
{
    if (T <= 0 || head_count <= 0 || !q || !k || !v || !dout || !lse || !dscale || !span_start || !span_finish || !dq || !dk || !dv)
        return fail(TS2_ERR_INVALID_ARG, "ts2_attention_backward: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    int *d = nullptr; // start | finish | rev_first | rev_last | scan scratch (2T)
    TS2_CUDA(cudaMalloc(&d, (4 * (size_t)T + batch_scan_tmp_elems(T)) * 4));
    TS2_CUDA(cudaMemcpy(d, span_start, (size_t)T * 4, cudaMemcpyHostToDevice));
    TS2_CUDA(cudaMemcpy(d + T, span_finish, (size_t)T * 4, cudaMemcpyHostToDevice));
    Ctx c;
    c.device = device;
    c.stream = (cudaStream_t)stream;
    if (int rc0 = batch_reverse_ranges(c, d, d + T, T, d + 4 * (size_t)T, d + 2 * (size_t)T, d + 3 * (size_t)T)) {
        cudaFree(d);
        return rc0;
    }
    const __half *Q = (const __half *)q, *K = (const __half *)k, *V = (const __half *)v, *DO = (const __half *)dout;
    float *fq = (float *)dq, *fk = (float *)dk, *fv = (float *)dv;
    int rc = variant == 2 || variant == 3
                 ? attention_backward_tc(c, Q, K, V, DO, lse, dscale, d, d + T, d + 2 * T, d + 3 * T, T, head_count, alibi_slope, dq, dk, dv,
                                         variant == 3)
             : variant == 0 ? attention_backward_mma(c, Q, K, V, DO, lse, dscale, d, d + T, d + 2 * T, d + 3 * T, T, head_count, alibi_slope,
                                                   fq, fk, fv)
                          : attention_backward_rowwise(c, Q, K, V, DO, lse, dscale, d, d + T, d + 2 * T, d + 3 * T, T, head_count,
                                                       alibi_slope, fq, fk, fv);
    cudaStreamSynchronize(c.stream);
    cudaFree(d);
    return rc;
}

int ts2_op_attention_reverse_ranges(int device, void *stream, const int32_t *span_start, const int32_t *span_finish, int T,
                                    int32_t *rev_first, int32_t *rev_last)
{
    if (T <= 0 || !span_start || !span_finish || !rev_first || !rev_last)
        return fail(TS2_ERR_INVALID_ARG, "ts2_op_attention_reverse_ranges: bad arguments");
    TS2_CUDA(cudaSetDevice(device));
    int *d = nullptr;
    TS2_CUDA(cudaMalloc(&d, (4 * (size_t)T + batch_scan_tmp_elems(T)) * 4));
    TS2_CUDA(cudaMemcpy(d, span_start, (size_t)T * 4, cudaMemcpyHostToDevice));
    TS2_CUDA(cudaMemcpy(d + T, span_finish, (size_t)T * 4, cudaMemcpyHostToDevice));
    Ctx c;
    c.device = device;
    c.stream = (cudaStream_t)stream;
    int rc = batch_reverse_ranges(c, d, d + T, T, d + 4 * (size_t)T, d + 2 * (size_t)T, d + 3 * (size_t)T);
    if (rc == TS2_OK && cudaStreamSynchronize(c.stream) != cudaSuccess)
        rc = fail(TS2_ERR_CUDA, "ts2_op_attention_reverse_ranges: the stream failed");
    if (rc == TS2_OK) {
        cudaMemcpy(rev_first, d + 2 * (size_t)T, (size_t)T * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(rev_last, d + 3 * (size_t)T, (size_t)T * 4, cudaMemcpyDeviceToHost);
    }
    cudaFree(d);
    return rc;
}

} // extern "C"
