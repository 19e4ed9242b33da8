// TEST INFRASTRUCTURE — the reference's OWN host-side optimizer step, THostModelMatrix::AddDelta
// (src/gpt/matrix/host_matrix.cpp:123-157, with TMatrixDeltaAddCtx :25-86), compiled from the reference's sources where
// they lie (oracle/Makefile, target opt) and driven through a C entry point, so that the restated optimizer of the
// oracle (ts2o_apply_gradient) is checked against the reference's code and not only against itself.
//
// AddDelta takes the gradient as a TModelMatrixHalfDelta (fp16 values times one power-of-two scale per row, plus the
// row's sum of squares; src/gpt/matrix/delta.h:22-45).  The driver builds that form from an fp32 gradient and returns
// the gradient as the reference then sees it (TModelMatrixHalfDelta::GetAllData), which is what the caller feeds to
// the restatement.
//
// The reference keeps its host matrices in memory obtained from its CUDA allocator (cuMemCreate, cuda_memory.cpp);
// this build replaces the four allocation entry points of src/lib/cuda/cuda_memory.h by plain aligned host memory so
// that the code runs on a machine without a GPU.  Nothing else of the reference is replaced.
#include <gpt/matrix/host_matrix.h>
#include <immintrin.h>
#include <cstdlib>
#include <cstring>

namespace NCuda
{
char *CudaHugeAlloc(yint sz) { return (char *)aligned_alloc(128, (size_t)((sz + 127) / 128 * 128)); }
void CudaHugeFree(void *p) { free(p); }
char *CudaHugeHostAlloc(yint sz) { return (char *)aligned_alloc(128, (size_t)((sz + 127) / 128 * 128)); }
void CudaHugeHostFree(void *p) { free(p); }
}

extern "C" int ts2ref_add_delta(float *weights, float *avrg, const float *grad, long long x_size, long long y_size, float *row_disp,
                                long long row_disp_size, float *sum_weight, float sparsity, float rate, float l2reg, float beta1,
                                float weight0, float weight1, float disp_decay, float *grad_seen, float *sum2_out)
{
    if (x_size % 8 || row_disp_size <= 0 || y_size % row_disp_size)
        return -1;
    TModelMatrix mm;
    mm.SetSizes(x_size, y_size, row_disp_size, sparsity);
    for (yint y = 0; y < y_size; ++y) {
        memcpy(&mm.GetMatrix()[y][0], weights + y * x_size, (size_t)x_size * 4);
        memcpy(&mm.GetGrad1()[y][0], avrg + y * x_size, (size_t)x_size * 4);
    }
    TVector<float> rd(row_disp, row_disp + row_disp_size);
    mm.SetRowDisp(*sum_weight, rd);

    THostModelMatrix host;
    host.Create(x_size, y_size, sparsity);
    host.SetData(mm);

    TModelMatrixHalfDelta delta;
    delta.Init(x_size, y_size);
    for (yint y = 0; y < y_size; ++y) {
        const float *g = grad + y * x_size;
        float mx = 0;
        for (yint x = 0; x < x_size; ++x)
            mx = fmaxf(mx, fabsf(g[x]));
        TModelMatrixHalfDelta::TRow &row = delta.Rows[y];
        row.Scale = 0;
        row.Sum2 = 0;
        if (mx == 0)
            continue;
        int e = 0;
        frexpf(mx, &e); // mx = f * 2^e, f in [0.5, 1): values / 2^e stay below 1
        const float scale = ldexpf(1.f, e);
        fp16 *dst = delta.GetRow(y);
        float sum2 = 0;
        for (yint x = 0; x < x_size; ++x) {
            dst[x] = _cvtss_sh(g[x] / scale, 0);
            const float v = _cvtsh_ss(dst[x]);
            sum2 += v * v;
        }
        row.Scale = scale;
        row.Sum2 = sum2 * scale * scale;
    }
    if (grad_seen) {
        TArray2D<float> seen;
        delta.GetAllData(&seen);
        for (yint y = 0; y < y_size; ++y)
            memcpy(grad_seen + y * x_size, &seen[y][0], (size_t)x_size * 4);
    }

    TTrainingStep step;
    step.Rate = rate;
    step.L2Reg = l2reg;
    step.Beta1 = beta1;
    step.Weight0 = weight0;
    step.Weight1 = weight1;
    step.DispDecay = disp_decay;
    host.AddDelta(delta, step);

    TModelMatrix res;
    host.GetData(&res);
    for (yint y = 0; y < y_size; ++y) {
        memcpy(weights + y * x_size, &res.GetMatrix()[y][0], (size_t)x_size * 4);
        memcpy(avrg + y * x_size, &res.GetGrad1()[y][0], (size_t)x_size * 4);
    }
    for (yint i = 0; i < row_disp_size; ++i)
        row_disp[i] = res.GetRowDisp()[i];
    *sum_weight = res.GetSumWeight();
    if (sum2_out)
        *sum2_out = host.GetSum2();
    return 0;
}
