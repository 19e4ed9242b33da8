// extern "C" operator-level entry points of include/ts2_b200.h (device helpers and
// the contraction kernels).  Plain pointers and sizes only.
#include "gemm.cuh"

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
    int32_t *w = device_status_word(device);
    if (w) {
        int32_t v = 0;
        TS2_CUDA(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
        if (v) {
            cudaMemset(w, 0, sizeof(v));
            return fail(TS2_ERR_DEVICE_STATUS, "device status word = 0x%x (bit0: a bounded wait in a kernel timed out)", v);
        }
    }
    return TS2_OK;
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

} // extern "C"
