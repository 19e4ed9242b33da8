// Tensor-core contraction for sm_100a: C[M][N] = epilogue(sum_k A(m,k) * B(n,k)).
// One persistent, warp-specialised kernel (gemm.cu) serves the forward, dX and dW
// contractions of the training step.
#pragma once
#include "common.cuh"
struct CUtensorMap_st;

namespace ts2 {

enum GemmKind { KIND_E4M3 = 0, KIND_F16 = 1, KIND_I8 = 2, KIND_BF16 = 3 };

struct Epilogue {
    float alpha = 1.f;
    const float *dyn_scale = nullptr;  // device scalar multiplied in (loss-scale bookkeeping)
    const float *dyn_scale2 = nullptr; // second device scalar
    const float *row_scale = nullptr;  // [M] device
    const float *col_scale = nullptr;  // [N] device
    const float *c_in = nullptr;       // TS2_OUT_F32_ADD: C = c_in + result (same pitch as C); null: in place
    int out_kind = TS2_OUT_F32;
    // Gated-activation form (FFN expansion, K-major fp16 output only): B holds two row blocks, "wide" rows [0, pair_stride)
    // and "gate" rows [pair_stride, 2 pair_stride), N = 2 pair_stride.  A tile covers 128 columns of each, and the
    // epilogue applies the 128-wide tile normalisation to the wide half, stores the normalised wide and the raw gate
    // values as fp16 in C (same columns as the plain form), the tile scale in act_scale[M][pair_stride / 128] and
    // act_mult * sigmoid(2 gate) * normalised wide in act_out[M][act_ld] (act_kind 0: e4m3 bytes, 1: fp16, 2: int8).
    int64_t pair_stride = 0;
    void *act_out = nullptr;
    int64_t act_ld = 0;
    float *act_scale = nullptr;
    float act_mult = 1.f;
    int act_kind = 0;
};

struct GemmArgs {
    int device = 0;
    cudaStream_t stream = nullptr;
    int kind = KIND_E4M3;
    // false: A is [M][lda], B is [N][ldb], K contiguous (forward and dX)
    // true : A is [K][lda] with M contiguous, B is [K][ldb] with N contiguous (dW: both operands token-major)
    bool mn_major = false;
    int64_t M = 0, N = 0, K = 0;
    const void *A = nullptr;
    int64_t lda = 0;
    const void *B = nullptr;
    int64_t ldb = 0;
    void *C = nullptr;
    int64_t ldc = 0;
    Epilogue epi;
    // grouped forms for mixture-of-experts layers (see GemmParams in gemm.cu)
    int group_mode = 0; // 1: B rows chosen per 128-row M tile (tile_group), N = rows of B per group; 2: K segment per group
    int groups = 0;
    const int *tile_group = nullptr; // device, one entry per M tile, negative = skip the tile
    int group_rows_b = 0;
    const int *group_kptr = nullptr; // device, groups + 1 row offsets (multiples of 128)
    int64_t c_group_stride = 0;      // elements of C between groups (mode 2)
    int tag = 0;               // class of the launch for the timing statistics (GEMM_TAG_*)
    void *workspace = nullptr; // split-K partial tiles (fp32); needed when gemm_splits() > 1
    size_t workspace_bytes = 0;
};

// number of K splits the scheduler will use for this shape (1 = no workspace needed)
int gemm_splits(int device, int kind, bool mn_major, int64_t M, int64_t N, int64_t K);
size_t gemm_workspace_bytes(int device, int kind, bool mn_major, int64_t M, int64_t N, int64_t K);
int gemm(const GemmArgs &a);

// 2-D TMA descriptor over a row-major [rows][ld] array of es-byte elements: box = 128 bytes x box_rows, 128-byte swizzle,
// out-of-range elements read as zero
int make_tensor_map(::CUtensorMap_st *tm, const void *base, int es, int64_t inner, int64_t rows, int64_t ld, int box_rows);

// SMs the contraction's persistent grid leaves free (for communication kernels that run beside it); process-wide
void gemm_reserve_sms(int n);

// classes of launches the timing statistics keep apart: other (operator-level calls), forward, dX and dW of the layers
// in the engine's operand format, and the final layer's three contractions (logits in the operand format, dX and dW fp16)
enum { GEMM_TAG_OTHER = 0, GEMM_TAG_FWD = 1, GEMM_TAG_DX = 2, GEMM_TAG_DW = 3, GEMM_TAG_FINAL = 4, GEMM_TAGS = 5 };
void gemm_timing_get_tag(int tag, double *ms_total, long long *launches, double *flops_total);

// accumulated device time of the contraction kernel (enabled by gemm_timing_enable)
void gemm_timing_enable(bool on);
void gemm_timing_get(bool reset, double *ms_total, long long *launches, double *flops_total, double *bytes_total = nullptr);

} // namespace ts2
