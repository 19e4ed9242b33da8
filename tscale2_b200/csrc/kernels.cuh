// Launchers of the bandwidth-bound kernels of the training step (kernels_*.cu).
// All pointers are device pointers; every launcher returns TS2_OK or an error code.
// FT (fast type) selects the operand format of the contractions: 0 = e4m3 bytes,
// 1 = fp16.
#pragma once
#include "common.cuh"

namespace ts2 {

constexpr int TILE = 128; // STATE_NORM_TILE / MM_TILE / head dim of the reference

struct Ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int ft = 0;         // 0 e4m3, 1 fp16, 2 int8
    float s_act = 16.f; // quantization scale of normalized activations (1 for fp16)
};

// ---- kernels_elem.cu ---------------------------------------------------------------
// state0[t] = sum over the node's labels of +-E[label] * (sko/32)   (ComputeEmbedding, cpu_transformer.cpp:66-90)
int embed_forward(const Ctx &c, const __half *embed, const float *sko, const uint32_t *label_arr, const uint32_t *label_ptr, int T,
                  int D, float *state);

// ---- kernels_batch.cu: batch preparation on the device -------------------------------
// codes of the batch status record {code, where, detail, detail}; 0 = the batch was well formed
enum {
    BATCH_OK = 0,
    BATCH_BAD_SPAN_PTR = 1,  // where = node
    BATCH_MULTI_SPAN = 2,    // where = node, detail = spans
    BATCH_BAD_SPAN = 3,      // where = node, details = start, finish
    BATCH_BAD_TARGET = 4,    // where = target entry, details = node, id
    BATCH_DUP_TARGET = 5,    // where = node
    BATCH_BAD_LABEL_PTR = 6, // where = node
    BATCH_BAD_LABEL = 7,     // where = entry of label_arr, details = label, node
};
// per-node span tables from the CSR form (at most one span per node), and per key the range [rev_first, rev_last] of
// nodes that may attend to it ((T, -1) = none; a superset, the kernels test each node's own span).
// scan_tmp: batch_scan_tmp_elems(T) ints.
size_t batch_scan_tmp_elems(int T);
int batch_span_tables(const Ctx &c, const int *span_ptr, const int *csr_start, const int *csr_finish, int T, int n_spans, int *start,
                      int *finish, int *scan_tmp, int *rev_first, int *rev_last, int *status);
int batch_reverse_ranges(const Ctx &c, const int *start, const int *finish, int T, int *scan_tmp, int *rev_first, int *rev_last);
// target[t] = id of the node's target or -1
int batch_targets(const Ctx &c, const int *node, const int *id, int n, int T, int V, int *target, int *status);
// inverse label index (TLabelInverseIndex, gpu_embedding.cuh:10-76): the entries (label, node | sign bit) of the batch
// sorted by label, nodes of one label in node order
struct LabelIndex {
    uint32_t *key[2] = {nullptr, nullptr}, *val[2] = {nullptr, nullptr}; // capacity label_cap each
    uint32_t *hist = nullptr;                                            // label_index_hist_elems(label_cap)
    float *partial = nullptr;                                            // label_index_partial_elems(label_cap, D)
    uint32_t n = 0;
    int sorted = 0; // which of key[] / val[] holds the sorted entries
};
size_t label_index_hist_elems(size_t label_cap);
size_t label_index_partial_elems(size_t label_cap, int D);
// validates label_arr / label_ptr in place (bad labels become label 0, label_ptr is clamped to n_labels) and writes the
// unsorted entries of ix; label_index_sort orders them (a stable radix sort, 8 bits per pass)
int label_index_entries(const Ctx &c, uint32_t *label_arr, uint32_t *label_ptr, int T, uint32_t n_labels, uint32_t label_count,
                        LabelIndex &ix, int *status);
int label_index_sort(const Ctx &c, uint32_t label_count, LabelIndex &ix);
// dE[label] += sum over the label's nodes, in node order, of +-g[node]   (embedding delta, cpu_transformer.cpp:176-196;
// BackpropEmbeddings over the inverse index, gpu_embedding.cuh).  One writer per row: no atomics, a fixed order.
int embed_backward_indexed(const Ctx &c, const float *g, const LabelIndex &ix, int D, float *dE);

// n = tilenorm(x) quantized (NormalizeState with 128-wide tiles, cpu_util.cpp:72-99); n16 optional fp16 copy
int tilenorm_forward(const Ctx &c, const float *x, int T, int D, void *n_fast, __half *n16);

// g_out = (add ? g_in : 0) + tilenorm_bwd(x, dn * (*dyn))   (NormalizeStateBackward, cpu_util.cpp:102-134;
// BackpropLayerNormalize, gpu_layer_norm.cuh:89-115).  absmax: running max |g_out| as float bits.
// health (optional): set to step_no by the first call whose g_out holds a NaN or an infinity (0 = never happened).
int tilenorm_backward(const Ctx &c, const float *x, const float *dn, const float *dyn, float dn_alpha, int T, int D, float *g, bool add,
                      unsigned *absmax, unsigned *health = nullptr, unsigned step_no = 0);

// g_fast = g * mult, mult = largest power of two with max|g| * mult <= target; ginv = 1/mult;
// fscale = f_static * (*sko) * ginv   (ScaleGrad / ComputeGradMult, gpu_grad_scale.cuh:33-62)
int cast_grad(const Ctx &c, const float *g, size_t n, const unsigned *absmax, void *g_fast, float *ginv, float f_static, const float *sko,
              float *fscale);

// int8 pipeline: row quantization with the reference's stochastic rounding (NormalizeVecsRowMaxKernel,
// row_scale.cuh:12-43): q[t][d] int8, row_scale[t] = max|x[t]| / 127.
//  rowquant_grad: x = g * 2^k (2^k from the running abs-max as in cast_grad; also writes ginv, fscale and, optionally,
//                 x as fp16 for the fp16 dW contraction);  rowquant_half: x = an fp16 tensor as it is.
int rowquant_grad(const Ctx &c, const float *g, int T, int D, const unsigned *absmax, int8_t *q, float *row_scale, __half *g16, float *ginv,
                  float f_static, const float *sko, float *fscale);
int rowquant_half(const Ctx &c, const __half *x, int T, int D, int8_t *q, float *row_scale);
// int8 values widened to fp16 (exact), n a multiple of 4
int i8_to_half(const Ctx &c, const void *src, size_t n, __half *dst);

// FFN activation (LoLU + tile-norm of the wide vector), TFFLayer::ComputeForward layer_ffn.cu:190-211.
// wg: [T][2F] fp16 = [wide | gate]; what: normalized wide fp16 [T][F]; wscale [T][F/128]; rg fast [T][F]
// BackpropLoLU + NormalizeStateBackward of the wide vector (layer_ffn.cu:232-236): d2 fast [T][2F] = [dwide | dgate]
// what: normalised wide values, row pitch what_ld (the wide half of wg when the contraction's epilogue wrote them there)
int ffn_act_backward(const Ctx &c, const __half *drg, const __half *wg, const __half *what, int what_ld, const float *wscale, int T, int F,
                     void *d2);

// attention gate: rg = sigmoid(2 gate) * o  (LoLU, cpu_util.cpp:139-168); gate inside qkvg [T][4Q] at column 3Q
int att_gate_forward(const Ctx &c, const __half *qkvg, const __half *o, int T, int Q, void *rg);
// dgate -> d4[:, 3Q:4Q] (fast), do (fp16) and dScale[t][h] = sum do*o  (BackpropLoLU + ComputeDScale)
int att_gate_backward(const Ctx &c, const __half *drg, const __half *qkvg, const __half *o, int T, int Q, void *d4, __half *dout,
                      float *dscale);

// debug trace: out[0] += sum of the buffer's 32-bit words (as a 64-bit integer), out[1] += its non-finite elements,
// out[2] = max(out[2], fp32 bits of the largest finite magnitude)   (kind 0: words only, 1: fp32, 2: fp16)
int checksum(const Ctx &c, const void *p, size_t bytes, int kind, unsigned long long *out);

// softmax cross-entropy over base-2 logits (SoftMax, cpu_transformer.cpp:12-37; gradient :146-159):
// logits fp16 [rows][V] are replaced by (onehot - p) * gscale; logp_sum += log p(target) (natural log).
int softmax_ce(const Ctx &c, __half *logits, int rows, int V, const float *bias, const int *target, float gscale, float *logp_sum,
               bool write_grad);

// ---- kernels_att.cu ----------------------------------------------------------------
// qkvg [T][4Q] fp16 -> q = rope(tilenorm_h(Q)), k = rope(K), v = tilenorm_h(V), each [T][Q] fp16;
// qscale, vscale [T][H]   (TAttLayer::ComputeForward, layer_att.cu:384-394)
int att_post_forward(const Ctx &c, const __half *qkvg, const float *rope, int T, int H, __half *q, __half *k, __half *v, float *qscale,
                     float *vscale);
// inverse of the above for gradients (layer_att.cu:464-470): writes d4[:, 0:3Q] (fast)
// grads16: dq, dk, dv are fp16 (the tcgen05 attention kernels' engine form) instead of fp32
int att_post_backward(const Ctx &c, const void *dq, const void *dk, const void *dv, bool grads16, const __half *q, const __half *v,
                      const float *qscale, const float *vscale, const float *rope, const float *sko_k, int T, int H, void *d4);
int fill_rope(const Ctx &c, float *rope, int T);

// attention over one span per node (ComputeValLookup / GradQ / GradK, layer_att_reference.h:41-212)
// o [T][Q] fp16, lse [T][H] = maxDP + log2(sumWeight); dq, dk, dv fp32, or fp16 with grads16
int attention_forward(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                      int T, int H, float slope, __half *o, float *lse);
int attention_backward(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                       const float *dscale, const int *span_start, const int *span_finish, const int *rev_first, const int *rev_last,
                       int T, int H, float slope, void *dq, void *dk, void *dv, bool grads16 = false);

// the two formulations behind attention_forward / attention_backward
int attention_forward_mma(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                          int T, int H, float slope, __half *o, float *lse);
int attention_backward_mma(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                           const float *dscale, const int *span_start, const int *span_finish, const int *rev_first,
                           const int *rev_last, int T, int H, float slope, float *dq, float *dk, float *dv);
int attention_forward_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                         int T, int H, float slope, __half *o, float *lse);
int attention_backward_tc(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                          const float *dscale, const int *span_start, const int *span_finish, const int *rev_first, const int *rev_last,
                          int T, int H, float slope, void *dq, void *dk, void *dv, bool grads16 = false);
int attention_forward_rowwise(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start,
                              const int *span_finish, int T, int H, float slope, __half *o, float *lse);
int attention_backward_rowwise(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                               const float *dscale, const int *span_start, const int *span_finish, const int *rev_first,
                               const int *rev_last, int T, int H, float slope, float *dq, float *dk, float *dv);
// host: for every key the range [first, last] of nodes whose span may contain it (a superset; kernels re-check)

// ---- kernels_moe.cu ----------------------------------------------------------------
// CpuMoe (layer_moe.cu:287-328): ids[T][k] and weights[T][k] from router logits [T][ld]
int moe_route(const Ctx &c, const float *logits, int ld, int T, int E, int k, int *ids, float *weights);
// expert-sorted slot tables (segments padded to 128 rows): seg_ptr[E+1], tile_group[max_rows/128] (-1: unused),
// slot_of[T*k], token_of[max_rows] (-1: unused), weight_of[max_rows]; scratch: hist and block_base, ceil(T/256)*E ints each
int moe_build_slots(const Ctx &c, const int *ids, const float *weights, int T, int k, int E, int max_rows, int *hist_scratch,
                    int *block_base_scratch, int *seg_ptr, int *tile_group, int *slot_of, int *token_of, float *weight_of, int *counts = nullptr);
// expert-parallel row space (rows received for the experts a rank owns): tables from the segment offsets seg[E + 1] and
// the rows with data valid[E]; zeroing of the padding rows of a received buffer
int moe_ep_tables(const Ctx &c, const int *seg, const int *valid, int E, int max_rows, int *tile_group, int *token_of);
int moe_zero_pad_rows(const Ctx &c, void *buf, int row_bytes, const int *seg, const int *valid, int E);
// row blocks pulled from other ranks' buffers over peer memory (bases[peer], plain loads) into `local`:
// moves[i] = {peer, row on the sender side, row on the owner side, rows}; to_owner: sender rows -> owner rows
int moe_pull_rows(const Ctx &c, const int4 *moves, int n_moves, uint8_t *const *bases, void *local, int row_bytes, bool to_owner,
                  long long total_bytes);
int moe_gather_rows(const Ctx &c, const void *src, const int *token_of, int rows, int row_bytes, void *dst);
int moe_act_forward(const Ctx &c, const __half *cat, const int *token_of, const float *weight_of, int rows, int X, __half *what,
                    float *wscale, void *rg);
int moe_act_backward(const Ctx &c, const __half *drg, const __half *cat, const __half *what, const float *wscale, const int *token_of,
                     const float *weight_of, int rows, int X, void *dcat, float *dmoe_part);
// out[t] = (in ? in[t] : out[t]) + sum_j y[slot_of[t*k+j]]
int moe_combine(const Ctx &c, const float *y, const int *slot_of, int T, int k, int D, const float *in, float *out);
int moe_combine_half(const Ctx &c, const __half *y, const int *slot_of, int T, int k, int D, const float *in, float *out);
int moe_router_backward(const Ctx &c, const float *dmoe_part, int tiles, const int *ids, const float *weights, const int *slot_of, int T,
                        int k, int E, int ld, void *dl);

// ---- kernels_opt.cu ----------------------------------------------------------------
int fill_vector(const Ctx &c, float *dst, int n, float value, const float *dyn, bool reciprocal_dyn);

// ---- flat, sharded optimizer + requantiser (kernels_opt.cu) -------------------------
// the part [a, b) (elements inside the matrix, multiples of 4) of one matrix that a rank owns
struct OptSeg {
    long long flat_off; // element offset of the matrix in the flat weight / momentum / gradient buffers
    long long a, b;
    int x, y;
    int row0, nrows; // rows that intersect [a, b)
    int grow0;       // global row number of the matrix's row 0
    int item0;       // work items (rows) of the segments before this one
    int mat;         // matrix index
    int qsize;       // bytes per quantized element
    int qkind;       // its format: 0 e4m3, 1 fp16, 2 int8
    uint8_t *qbase;  // row-major quantized copy of the matrix
    float sparsity;
};
struct OptMat {
    long long x, y;
    int row_disp_size, grow0;
    float *row_disp, *sum_weight;
};
int opt_row_sum2(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *grad, float *rowsum);
int opt_disp(const Ctx &c, const OptMat *mats, int n_mats, const float *rowsum, float disp_decay, float *row_scale);
// step == nullptr: no update, only the per-row sums of squares of the weights
int opt_update(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *grad, const float *row_scale,
               const ts2_training_step *step, float *avg, float *w, double *roww2);
int opt_sko(const Ctx &c, const OptMat *mats, int n_mats, const double *roww2, float *skos);
int opt_quantize(const Ctx &c, const OptSeg *segs, int nseg, int nitems, const float *w, const float *skos);
// copy / transposed copy of quantized values; dst or dstT may be null; transposed_as_half: 0 no, 1 e4m3 -> fp16, 2 int8 -> fp16
int qcopy_block(const Ctx &c, const void *src, int64_t x, int64_t y, int64_t ld_src, int elem_size, void *dst, int64_t ld, void *dstT,
                int64_t ldT, int transposed_as_half);
int layer_scales(const Ctx &c, float *fwd_col, float *bwd_row, int W, int ncat, bool is_att, float a, const float *skos);

} // namespace ts2
