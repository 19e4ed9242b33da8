/* TEST INFRASTRUCTURE — C interface of the CPU oracle (see prim.h).
 * Built twice from the same driver: libts2_oracle.so (restated primitives)
 * and _ref/libts2_oracle_ref.so (the reference's own compiled primitives). */
#ifndef TS2_ORACLE_H
#define TS2_ORACLE_H
#include "../include/ts2_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* how the contractions see the weights (TFastModelFloat, cfg_precision.h:21-46) */
#define TS2O_QUANT_I8 0
#define TS2O_QUANT_E4M3 1
#define TS2O_QUANT_HALF 2
#define TS2O_QUANT_NONE 3 /* fp32 master weights, no quantization */

typedef struct ts2o_outputs {
    float **grads;      /* n_mats pointers ([y][x] fp32), entries may be NULL */
    float *states;      /* (layer_count+1) * T * dim, or NULL */
    float *state_grads; /* (layer_count+1) * T * dim, or NULL; [d] = gradient w.r.t. the state entering layer d */
    float *target_prob; /* target_count floats, or NULL */
    double score;       /* mean log p(target), natural log (ComputeScore) */
    double seconds;     /* wall time of forward+backward */
} ts2o_outputs;

const char *ts2o_backend(void);

/* 0 (default): activations and gradients stay fp32, the reference's CPU path.  1: the four operand tensors of the
 * layer contractions (normalized state, gated activation, state gradient, first-contraction output gradients) are
 * rounded to e4m3 at the points and scales the B200 engine's fp8 pipeline rounds them (dense ATT / FFN layers; the
 * reference's GPU path does the same with TNormStateFloat / TFastGradientFloat = e4m3, cfg_precision.h:28-35).
 * 2: the same for the engine's int8 pipeline: normalized state and gated activation as int8 at 24 x their value, the
 * gradient operand of every dX product quantized per token row to int8 (nearest), the dW products from the unquantized
 * gradients.  Used to separate the engine's own error from the error of the number format.  Process-wide switch. */
void ts2o_set_activation_quant(int mode);
/* row quantization to int8 with stochastic rounding, the operand form of the reference's int8 backward contractions
 * (NormalizeVecsRowMaxKernel, src/gpt/compute/row_scale.cuh:12-43) */
void ts2o_rowquant_i8(const float *x, int T, int D, int8_t *q, float *row_scale);
/* the rounding that mode applies: fp32 -> nearest e4m3 value (ties to even, subnormals, saturation at 448) */
void ts2o_round_e4m3(const float *src, int64_t n, float *dst);

/* one forward + backward of TComputeContext::ComputeBackprop
 * (src/gpt/compute/cpu_transformer.cpp:128-198) */
int ts2o_backprop(const ts2_model_descr *descr, const ts2_matrix_view *mats, int n_mats, const float *bias,
                  const ts2_batch_nodes *nodes, int weight_quant, ts2o_outputs *out);

/* TQuantizedMatrix::Convert + GetFastFloatData (src/gpt/matrix/quant.h:42-79):
 * q[y][x] as bytes (i8 / e4m3) or halves, deq = values the CPU path computes with */
int ts2o_quantize_matrix(const float *w, int64_t x_size, int64_t y_size, int quant, int no_scale, void *q_out, float *deq_out,
                         float *sko_out);

/* the scalar element encoders behind ts2o_quantize_matrix: dst[i] = encode(src[i] * mult);
 * and the reference's e4m3 decoder (ConvertE4toFloat, src/util/fp8.h:4-22) */
void ts2o_encode(const float *src, int64_t n, int quant, float mult, void *dst);
float ts2o_decode_e4m3(uint8_t x);

/* ApplyGradientImpl (src/gpt/matrix/agpu_cuda.cuh:484-524) with the kernels
 * of src/gpt/matrix/agpu_cuda.cu:32-134: updates weights, avg_grad, row_disp,
 * sum_weight in place from the fp32 gradient. */
int ts2o_apply_gradient(float *weights, float *avg_grad, const float *grad, int64_t x_size, int64_t y_size, float *row_disp,
                        int64_t row_disp_size, float *sum_weight, float sparsity, const ts2_training_step *step);

/* primitives, for op-level parity tests (row-major fp32) */
void ts2o_mul_forward(const float *x, const float *w, float *y, int T, int in_dim, int out_dim);
void ts2o_mul_backward_accum(float *dx, const float *w, const float *dy, int T, int in_dim, int out_dim);
void ts2o_sum_rank_one(const float *x, const float *dy, float *delta, int T, int in_dim, int out_dim);
void ts2o_normalize_state(const float *state, float *out, int T, int dim, int head_count);
void ts2o_normalize_state_backward(const float *state, const float *dnorm, float *grad, int T, int dim, int head_count);
void ts2o_lolu(const float *gate, const float *vals, float *out, int64_t n);
void ts2o_backprop_lolu(const float *gate, const float *vals, const float *grad, float *dgate, float *dvals, int64_t n);
void ts2o_rope(float *p, int T, int dim, int head_dim, float dir);
/* attention forward + backward for one layer; q,k post-rope, v normalized.
 * att: one CSR span list.  outputs may be NULL. */
void ts2o_attention(const float *q, const float *k, const float *v, int T, int head_count, float alibi_slope,
                    const ts2_attention_info *att, float *val_lookup, float *sum_weight, float *max_dp,
                    const float *d_val_lookup, float *dq, float *dk, float *dv);
/* CpuMoe / CpuBackpropMoe (src/gpt/compute/layer_moe.cu:287-360) */
void ts2o_moe_select(const float *logits, float *weights, int T, int expert_count, int selected);
void ts2o_moe_select_backward(const float *weights, float *dmoe, int T, int expert_count);

#ifdef __cplusplus
}
#endif
#endif
