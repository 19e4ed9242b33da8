/*
 * ts2_b200.h — C ABI of the B200 (sm_100a) training-backward engine.
 *
 * The library behind this header replaces the compute backend that the
 * TScale2 trainer reaches through IModel / IModelInstance
 * (src/gpt/compute/model.h:22-56) and the factory CreateLocalTransformer
 * (src/gpt/compute/model.h:141).  Everything is plain pointers and sizes; all
 * host arrays are caller-owned and are copied before the call returns.
 *
 * Conventions
 *  - every matrix is row-major fp32 [y_size = out][x_size = in], the shapes
 *    and the order are those of TModelDescr::EnumLayerMatrices
 *    (src/gpt/model_params/model_dim.h:219-258): index 0 = embedding
 *    [label_count][dim], 1 = final layer [output_token_count][dim], then for
 *    each layer in order its matrices (ATT: Q,K,V,Gate,Combiner; FFN:
 *    Expand,Gate,Contract; MOE: Expand,Gate,Contract,Select).
 *  - "gradient" is the ascent direction the reference back-propagates
 *    (onehot - p, src/gpt/compute/cpu_transformer.cpp:146-156); the optimizer
 *    adds rate * normalized gradient.
 *  - every function returns TS2_OK or a negative error code; nothing aborts
 *    (the reference aborts through Y_VERIFY; return codes are the one
 *    deliberate difference).  ts2_last_error() gives the message.
 *  - there is no CPU fallback: without a CUDA device ts2_create fails with
 *    TS2_ERR_NO_DEVICE.
 */
#ifndef TS2_B200_H
#define TS2_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS2_OK 0
#define TS2_ERR_INVALID_ARG (-1)
#define TS2_ERR_NO_DEVICE (-2)
#define TS2_ERR_CUDA (-3)
#define TS2_ERR_UNSUPPORTED (-4)
#define TS2_ERR_TOO_LARGE (-5)
#define TS2_ERR_TIMEOUT (-6)
#define TS2_ERR_COMM (-7)
#define TS2_ERR_DEVICE_STATUS (-8)

/* ELayerType, src/gpt/model_params/model_dim.h:56-61 */
#define TS2_LAYER_ATT 0
#define TS2_LAYER_ATT_3LIN 1 /* RNN variant: rejected with TS2_ERR_UNSUPPORTED */
#define TS2_LAYER_FFN 2
#define TS2_LAYER_MOE 3

/* subset of the MPF_* model flags that changes the backward pass,
 * src/gpt/model_params/model_dim.h:35-53 */
#define TS2_MPF_DISABLE_TUNE_EMBED 0x8ull
#define TS2_MPF_DISABLE_TUNE_FINAL_LAYER 0x4000ull
#define TS2_MPF_DISABLE_TUNE_LAYERS 0x8000ull

/* arithmetic of the contractions; the reference selects this at compile time
 * in src/gpt/compute/cfg_precision.h:18-46 */
#define TS2_PREC_FP8 0  /* e4m3 operands, fp32 accumulate (reference "fp8 matmul" block) */
#define TS2_PREC_F16 1  /* fp16 operands, fp32 accumulate (reference "fp16 matmul" block) */
#define TS2_PREC_INT8 2 /* int8 operands, int32 accumulate (reference "int8 matmul" block, its default); the engine
                         * runs forward and dX contractions in int8 with per-row gradient scales, dW in fp16 */

/* ts2_backprop add_to_model; EAddToModel, src/gpt/matrix/base_host.h:20-23 */
#define TS2_GRADIENT_ACCUMULATE 0
#define TS2_GRADIENT_APPLY 1

#define TS2_LABEL_NEGATIVE 0x80000000u /* src/gpt/att/nodes_batch.h:6 */
#define TS2_LABEL_MASK 0x7fffffffu

/* TModelDescr::TLayerParams, src/gpt/model_params/model_dim.h:159-168 */
typedef struct ts2_layer_params {
    int32_t layer_type;
    float alibi_slope;
    int32_t attention_type_id;
} ts2_layer_params;

/* TModelDims + TModelDescr, src/gpt/model_params/model_dim.h:118-180.
 * q_dim and tt_dim must be 128 (cfg_precision.h:79-80), dim a multiple of 128. */
typedef struct ts2_model_descr {
    int32_t dim;
    int32_t q_dim;
    int32_t tt_dim;
    int32_t head_count;
    int32_t ffn_tiles; /* FFN width = 128 * ffn_tiles */
    int32_t expert_dim;
    int32_t moe_expert_count;
    int32_t moe_selected;
    int32_t label_count;        /* embedding rows */
    int32_t output_token_count; /* final layer rows (vocabulary) */
    int32_t attention_type_count;
    int32_t layer_count;
    const ts2_layer_params *layers;
    uint64_t flags;
    int32_t precision; /* TS2_PREC_FP8, TS2_PREC_F16 or TS2_PREC_INT8 (dense layers only) */
    int32_t reserved;
} ts2_model_descr;

typedef struct ts2_matrix_view {
    float *data;    /* row-major, row stride = x_size */
    int64_t x_size; /* input width */
    int64_t y_size; /* output width */
} ts2_matrix_view;

/* TAttentionInfo, src/gpt/att/att.h:22-49: CSR list of inclusive [start,finish]
 * spans per node.  The engine accepts at most one span per node, which is what
 * the trainer generates (src/gpt/att/sliding_window.cpp:113-118,213-224). */
typedef struct ts2_attention_info {
    const int32_t *span_start;
    const int32_t *span_finish;
    const int32_t *span_ptr; /* node_count + 1 */
} ts2_attention_info;

/* TBatchNodes, src/gpt/att/nodes_batch.h:36-49 */
typedef struct ts2_batch_nodes {
    int32_t node_count;
    const uint32_t *label_arr; /* top bit = negative sign */
    const uint32_t *label_ptr; /* node_count + 1 */
    int32_t target_count;
    const int32_t *target_node;
    const int32_t *target_id;
    int32_t attention_type_count;
    const ts2_attention_info *att;
} ts2_batch_nodes;

/* TTrainingStep, src/gpt/train_config/train_step.h:4-26 */
typedef struct ts2_training_step {
    float rate;
    float l2reg;
    float beta1;
    float weight0;
    float weight1;
    float disp_decay;
} ts2_training_step;

typedef struct ts2_model ts2_model;

/* ------------------------------------------------------------------------- */
/* model life cycle: CreateLocalTransformer, src/gpt/compute/model.cu:257-264 */

/* Number of matrices (2 + per-layer) and their shapes for a description. */
int ts2_matrix_count(const ts2_model_descr *descr);
int ts2_matrix_shape(const ts2_model_descr *descr, int index, int64_t *x_size, int64_t *y_size);

/* mats: fp32 master weights in the order above; bias: output_token_count floats
 * (may be NULL = zeros).  device: CUDA ordinal this process drives (one process
 * per GPU).  max_nodes: capacity in nodes (tokens) per step. */
int ts2_create(const ts2_model_descr *descr, const ts2_matrix_view *mats, int n_mats, const float *bias,
               int device, int max_nodes, ts2_model **out);
void ts2_destroy(ts2_model *m);
const char *ts2_last_error(const ts2_model *m); /* m may be NULL: last create error */

/* IModelInstance::GetNodes + Init(INIT_BACKPROP), src/gpt/compute/model.h:32-35;
 * TSinlgeComputeContext::Init, src/gpt/compute/gpu_transformer.cu:526-566 */
int ts2_set_batch(ts2_model *m, const ts2_batch_nodes *nodes);
/* What the reference derives from a batch on the host before a step (span tables of TNodesBatch / GroupAttention,
 * src/gpt/att/att.h:125-211; TLabelInverseIndex::BuildInverseIndex, src/gpt/compute/gpu_embedding.cuh:38-75) is
 * derived on the device here: ts2_set_batch copies the arrays as they are and checks only counts and capacities.
 * Every element is validated on the device; a malformed element (label or target out of range, a node with more than
 * one span or target, a span outside the batch, a label_ptr / span_ptr that is not a CSR offset array) is replaced by a
 * harmless one and reported by the next ts2_wait (or any other call that waits) as TS2_ERR_INVALID_ARG /
 * TS2_ERR_UNSUPPORTED with the first offending element in ts2_last_error; the step that used the batch is then
 * meaningless but has touched nothing outside its buffers.
 *
 * The derived tables of the current batch, for tests (each pointer may be NULL; node_count ints each):
 * span_start / span_finish: the node's span or (0, -1); rev_first / rev_last: per key the range of nodes that may
 * attend to it, (node_count, -1) if none - a superset, kernels test each node's own span; target: id or -1. */
int ts2_get_batch_tables(ts2_model *m, int attention_type, int32_t *span_start, int32_t *span_finish, int32_t *rev_first,
                         int32_t *rev_last, int32_t *target);
/* The inverse label index of the current batch: all (label, node) entries sorted by label, the nodes of one label in
 * the order of label_arr (= node order); bit 31 of a node entry is TS2_LABEL_NEGATIVE of that occurrence.  The
 * embedding gradient sums a label's nodes in this order, so it does not depend on the schedule. */
int ts2_get_label_index(ts2_model *m, uint32_t *labels, uint32_t *nodes, int64_t capacity, int64_t *count);

/* IModel::Backprop, src/gpt/compute/model.h:53 — asynchronous: enqueues the
 * forward pass, the backward pass and (TS2_GRADIENT_APPLY) the gradient
 * reduction + optimizer + requantization. */
int ts2_backprop(ts2_model *m, const ts2_training_step *step, int add_to_model);
/* IModel::WaitAllCompute, src/gpt/compute/model.h:54 — bounded wait */
int ts2_wait(ts2_model *m);
/* IModelInstance::ComputeScore, src/gpt/compute/model.h:39: mean log p(target) (natural log) */
int ts2_forward_score(ts2_model *m, float *out_score);
/* IModel::GetAvrgTrainErr, src/gpt/compute/model.h:55: mean -log p(target) of the last backprop */
int ts2_avg_train_err(ts2_model *m, float *out_err);

/* IModel::GetParams / SetParams, src/gpt/compute/model.h:48-49.  what selects
 * the per-matrix tensor: master weights, momentum (Grad1), or the raw fp32
 * weight gradient of the last ts2_backprop (the tap the parity tests read:
 * the tensor the reference hands to HostApplyDelta,
 * src/gpt/compute/cpu_util.h:86-95). */
#define TS2_PARAM_WEIGHTS 0
#define TS2_PARAM_MOMENTUM 1
#define TS2_PARAM_GRADIENT 2
int ts2_get_params(ts2_model *m, int what, ts2_matrix_view *mats_out, int n_mats);
int ts2_set_params(ts2_model *m, int what, const ts2_matrix_view *mats, int n_mats);
/* RowDisp / SumWeight of a matrix (TModelMatrix, src/gpt/model_params/model_matrix.h:61-70) */
int ts2_get_row_disp(ts2_model *m, int index, float *row_disp, int64_t n, float *sum_weight);
/* the other direction, for resuming from a model file (TModelMatrix::SetRowDisp, model_matrix.h:85-89) */
int ts2_set_row_disp(ts2_model *m, int index, const float *row_disp, int64_t n, float sum_weight);
/* quantized weights as the contractions see them: bytes (e4m3) or halves,
 * [y][x], and the per-matrix scale sko (src/gpt/matrix/agpu_cuda.cuh:63-101) */
int ts2_get_fast_weights(ts2_model *m, int index, void *dst, int64_t dst_bytes, float *matrix_scale);

/* debugging / parity taps: fp32 residual state entering layer `layer`
 * (layer == layer_count: after the last layer) and the state gradient at the
 * same boundary captured during the last ts2_backprop (enabled by
 * ts2_set_debug_taps before the call; costs one copy per layer). */
int ts2_set_debug_taps(ts2_model *m, int enable);
/* raw copy of an internal per-layer buffer after the last step, for tests: "rg", "dcat", "cat16", "n_fast",
 * "n_rows", "logits", "ids", "weights", "slot_of", "token_of", "seg_ptr", "moe_g", "drg", "capture" (the caller knows the layout) */
int ts2_debug_read(ts2_model *m, const char *name, int layer, void *dst, int64_t bytes);
int ts2_get_state_tap(ts2_model *m, int layer, int gradient, float *dst, int64_t n_floats);

/* Step health (no reference counterpart; the reference's trainer only sees a NaN in the averaged training error,
 * src/gpt/train/train_ctx.cpp:11-31).  first_bad_step[b], b = 0 .. layer_count, is the number (1 = the first
 * ts2_backprop of this model) of the first step whose state gradient at layer boundary b held a NaN or an infinity,
 * 0 if that never happened; the flag rides on the abs-max reduction of the norm-backward kernel, so it costs
 * nothing per step.  reset clears the flags.  steps_so_far (optional) receives the step counter. */
int ts2_get_step_health(ts2_model *m, int reset, uint32_t *first_bad_step, int n_boundaries, int64_t *steps_so_far);
/* training error (mean -log p(target), as ts2_avg_train_err) of the last n ts2_backprop calls, oldest first, n <= 256:
 * every step's loss can be checked after a timed loop without a device read inside it */
int ts2_get_loss_history(ts2_model *m, float *out_err, int n);
/* drops an accumulated, not yet applied gradient: the next ts2_backprop starts from zero (the reference reaches the
 * same state by applying with a zero rate; used by the repeatability tests) */
int ts2_discard_gradient(ts2_model *m);
/* Debug trace (no reference counterpart), off by default.  When enabled, every ts2_backprop records for each
 * intermediate buffer of the step, in stream order, an order-independent checksum (the sum of its 32-bit words as a
 * 64-bit integer), the number of non-finite elements and the largest finite magnitude (max_abs, optional; 0 for byte
 * buffers); one extra read pass per buffer.  Two steps from the same
 * state must give the same checksums for every buffer (the embedding gradient, summed with float atomics, has no
 * record).  ts2_get_debug_trace returns the number of records of the last step in *count and fills up to `capacity`
 * entries; ts2_debug_trace_name gives a record's name ("dq[3]" = buffer dq of layer 3). */
int ts2_set_debug_trace(ts2_model *m, int enable);
int ts2_get_debug_trace(ts2_model *m, uint64_t *sums, uint64_t *nonfinite, float *max_abs, int capacity, int *count);
/* with the trace enabled: the buffer behind the record called record_name (NULL or "": none) is also copied aside
 * during the step, up to max_bytes, and can be read back with ts2_debug_read(m, "capture", 0, dst, bytes) */
int ts2_set_debug_capture(ts2_model *m, const char *record_name, int64_t max_bytes);
const char *ts2_debug_trace_name(ts2_model *m, int index);

/* ------------------------------------------------------------------------- */
/* data-parallel gradient reduction; replaces TMultiDeviceReducer::AllReduce,
 * src/lib/cuda/multi_device_buf.cu:193-265, called from
 * TAgpuCudaModelMatrix::ApplyGradientImpl, src/gpt/matrix/agpu_cuda.cuh:484-500, by reduce-scatter -> sharded
 * optimizer -> all-gather of the quantized weights (NCCL).  One process per GPU; rank 0 creates the 128-byte id and
 * the host shares it.  world_size must divide 256.  After ts2_comm_init the fp32 master weights and momentum of a rank
 * are current only in the parts it owns; ts2_get_params / ts2_set_params bring them up to date first with an
 * all-gather, so every rank must make those calls together (in the same order), like ts2_backprop.  The gradient tap
 * (TS2_PARAM_GRADIENT) after an applied step holds the summed gradient in the rank's own parts and the rank's local
 * gradient elsewhere. */
/* Layout of the data-parallel exchange, computable without a device.  The engine keeps weights, momentum and gradient
 * in flat fp32 buffers: the matrices in the order above, grouped into buckets (embedding; final layer; one per layer,
 * but one per matrix in a mixture-of-experts layer, so that a rank's part of an expert matrix is whole experts)
 * whose lengths are padded to a multiple of 1024 elements.  With world_size ranks, rank r owns elements
 * [bucket_offset[b] + r * bucket_elems[b] / world_size, + bucket_elems[b] / world_size) of every bucket b: a step
 * reduce-scatters each bucket's gradient onto those parts (as soon as the backward pass has written the bucket),
 * every rank runs the optimizer and the requantiser on its parts only (per-row sums of squares are completed by a
 * small all-reduce), and the quantized bytes are all-gathered.  Returns the number of buckets; fills up to
 * max_buckets entries of the bucket arrays and, if matrix_offset is given, the n_mats matrix offsets (elements). */
int ts2_dp_layout(const ts2_model_descr *descr, int64_t *matrix_offset, int n_mats, int64_t *bucket_offset, int64_t *bucket_elems,
                  int32_t *bucket_first_matrix, int max_buckets);
#define TS2_COMM_ID_BYTES 128
int ts2_comm_unique_id(uint8_t id[TS2_COMM_ID_BYTES]);
int ts2_comm_init(ts2_model *m, int rank, int world_size, const uint8_t id[TS2_COMM_ID_BYTES]);
/* Expert parallelism for the mixture-of-experts layers, on top of the data-parallel exchange (after ts2_comm_init, all
 * ranks, expert_count divisible by the world size): rank r computes experts [r E / N, (r + 1) E / N) for the rows of
 * ALL ranks.  Each rank sorts its (token, choice) rows by expert as before; per layer the ranks exchange their
 * per-expert row counts, then the rows themselves travel to the experts' owners and the results back (ncclSend /
 * ncclRecv blocks in expert order on a communicator of their own); the backward pass sends the state gradient rows
 * the same way and returns the routing-weight gradients and the input gradients.  The weight gradient of an expert
 * arises complete on its owner.  The counts are read on the host once per layer and step.  The reference splits
 * experts over the devices of a device group that all see the same tokens (GetExpertSpan / AllGatherMoe / ReduceMoe,
 * src/gpt/compute/layer_moe.cu:52-66,170,231); with one process per GPU and different tokens on every rank that becomes
 * this exchange.  capacity_factor (1 .. world size; 0 = the default, min(world size, 4)): a rank can receive up to that many times its own
 * number of rows; a step that needs more fails on every rank with TS2_ERR_TOO_LARGE.
 * The rows travel through the library's own copy kernel over peer memory: the staging buffers of all ranks are mapped
 * into every process with CUDA IPC (one node), a 4-byte all-reduce is the barrier before each copy; where a buffer
 * cannot be mapped, or with TS2_EP_EXCHANGE=nccl, all ranks use ncclSend / ncclRecv on the same blocks instead.
 * In the e4m3 pipeline the experts' results return as fp16 rows, in the fp16 pipeline as fp32.
 * The three expert matrices of a layer are buckets of their own (ts2_dp_layout) whose r-th part is rank r's experts:
 * they are neither reduce-scattered nor all-gathered any more.
 * After this call ts2_forward_score is a collective call like ts2_backprop (every forward pass exchanges rows), and
 * ts2_destroy must be called by all ranks (it meets the others once more before the mapped buffers are freed). */
int ts2_set_expert_parallel(ts2_model *m, float capacity_factor);
/* Measurement hook: device time (events around every row exchange on the compute stream), bytes this rank sent to
 * other ranks and number of exchanges since the last call; enable switches the recording on or off from now on. */
int ts2_get_exchange_ms(ts2_model *m, int enable, float *ms, double *bytes_sent, int *exchanges);
/* The plan of one layer's exchange, as every rank computes it from all ranks' per-expert row counts
 * counts[world_size][expert_count] (host arithmetic only; no device needed).  own_seg[E + 1]: this rank's own
 * expert-sorted layout (segments padded to 128 rows); x_seg[E + 1], x_valid[E]: the layout of the rows it receives for
 * its experts; moves: n_out blocks this rank sends then n_in blocks it receives, each {peer, first row in the
 * sender's own layout (-1 for a remote sender), first row in the owner's layout, rows}; max_x_rows: the largest
 * received layout of any rank. */
int ts2_moe_exchange_plan(int world_size, int rank, int expert_count, const int32_t *counts, int32_t *own_seg, int32_t *x_seg,
                          int32_t *x_valid, int32_t *moves, int max_moves, int32_t *n_out, int32_t *n_in, int32_t *max_x_rows);

/* counters for the bench: kernels of this library launched since the last reset */
int64_t ts2_launch_count(ts2_model *m, int reset);
/* device time of the last ts2_backprop in ms (CUDA events on the engine's stream) */
int ts2_last_step_ms(ts2_model *m, float *ms);
/* a CUDA-event bracket on the engine's stream around any number of calls: ts2_timer_begin
 * records the first event, ts2_timer_end records the second, waits for it and returns the
 * elapsed device time in ms */
int ts2_timer_begin(ts2_model *m);
int ts2_timer_end(ts2_model *m, float *ms);
/* average duration (ms) and launch count of the contraction kernel over the
 * steps since the last reset, measured with CUDA events on the engine's stream
 * when profiling is enabled (adds a pair of events per launch) */
int ts2_set_kernel_timing(ts2_model *m, int enable);
int ts2_get_kernel_timing(ts2_model *m, int reset, double *gemm_ms_total, int64_t *gemm_launches, double *gemm_flops_total);
/* the same totals for one class of launches (read before a resetting ts2_get_kernel_timing): 0 operator-level calls,
 * 1 forward contractions of the layers, 2 their dX contractions, 3 their dW contractions, 4 the final layer's three
 * (logits, dX and dW in fp16).  No reference counterpart (measurement). */
#define TS2_GEMM_CLASS_OTHER 0
#define TS2_GEMM_CLASS_FORWARD 1
#define TS2_GEMM_CLASS_DX 2
#define TS2_GEMM_CLASS_DW 3
#define TS2_GEMM_CLASS_FINAL 4
int ts2_get_kernel_timing_class(ts2_model *m, int cls, double *gemm_ms_total, int64_t *gemm_launches, double *gemm_flops_total);
/* algorithmic bytes (both operands once, output once, residual input once) of the contraction launches timed
 * since the last reset; read it before ts2_get_kernel_timing(reset = 1).  No reference counterpart (measurement). */
int ts2_get_kernel_bytes(ts2_model *m, double *gemm_bytes_total);

/* ------------------------------------------------------------------------- */
/* operator-level entry points (device pointers unless named host_*); these
 * are the pieces ts2_backprop is built from, exported for the parity tests
 * and micro-benchmarks.  stream is a cudaStream_t passed as void*. */

int ts2_device_count(void);
int ts2_dev_alloc(int device, size_t bytes, void **ptr);
int ts2_dev_free(int device, void *ptr);
int ts2_dev_upload(int device, void *dst, const void *host_src, size_t bytes);
int ts2_dev_download(int device, void *host_dst, const void *src, size_t bytes);
int ts2_dev_memset(int device, void *dst, int value, size_t bytes);
int ts2_dev_sync(int device);
/* Self-test of the bounded waits (no reference counterpart): launches one CTA that waits on a barrier nothing arrives
 * at.  The wait gives up after its limit (under a second), the kernel sets the time-out bit of the device status word
 * and returns; the call reports it like ts2_dev_sync: TS2_ERR_DEVICE_STATUS is the expected result, and the context
 * stays usable (nothing traps, nothing spins without a limit). */
int ts2_selftest_wait_limit(int device);

/* C[M][N] (+)= alpha * A[M][K] · B[N][K]^T — both operands K-contiguous.
 * Replaces Fp8MatMul / Int8MatMul / Fp16MatMul (src/lib/cuda/cuda_fp8.cuh:123-228,
 * cuda_i8.cuh:157-260, cuda_fp16.cuh:49-164).  prec: TS2_PREC_*; out_kind:
 * TS2_OUT_*; row_scale[M] / col_scale[N] optional fp32 factors applied in the
 * epilogue (TStoreScaled, Int8MatMulKernelRowScale).  M, N, K multiples of 128
 * (MM_TILE, src/lib/cuda/cuda_matmul.cuh:10). */
#define TS2_OUT_F32 0
#define TS2_OUT_F32_ADD 1 /* C += result */
#define TS2_OUT_F16 2
#define TS2_OUT_BF16 3
int ts2_gemm_tn(int device, void *stream, int prec, int out_kind, int64_t M, int64_t N, int64_t K, const void *A,
                int64_t lda, const void *B, int64_t ldb, void *C, int64_t ldc, float alpha, const float *row_scale,
                const float *col_scale);

/* dX = dY[T][out] · W[out][in]  (MulBackwardWithAccum without the accumulate,
 * src/gpt/compute/cpu_util.cpp:30-47; TMatMulBuffers::Backprop,
 * src/gpt/compute/layer_cuda_base.cuh:238-250).  Wt is W stored transposed
 * [in][out] as the requantizer keeps it. */
int ts2_gemm_dx(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                const void *dY, const void *Wt, void *dX, float alpha, const float *row_scale,
                const float *col_scale);

/* dW[out][in] (+)= alpha * dY[T][out]^T · X[T][in]  (SumRankOne,
 * src/gpt/compute/cpu_util.cpp:50-67; TMatMulBuffers::BackpropDelta,
 * src/gpt/compute/matmul_fwdbwd.cuh:149-162).  Both operands are token-major;
 * the contraction dimension T is split over the SMs and the partial tiles are
 * reduced through `workspace` (ts2_gemm_dw_workspace_bytes). */
size_t ts2_gemm_dw_workspace_bytes(int64_t T, int64_t in_dim, int64_t out_dim);
int ts2_gemm_dw(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                const void *dY, const void *X, void *dW, float alpha, void *workspace, size_t workspace_bytes);

/* ts2_gemm_dw with the per-row / per-column fp32 factors of the epilogue (row_scale[out_dim], col_scale[in_dim], either may
 * be NULL): the dW side of the reference's scaled stores (TStoreScaled, src/lib/cuda/cuda_matmul.cuh). */
int ts2_gemm_dw_scaled(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                       const void *dY, const void *X, void *dW, float alpha, const float *row_scale, const float *col_scale,
                       void *workspace, size_t workspace_bytes);

/* The same contraction as ts2_gemm_dw for callers that must not allocate device memory — a host
 * whose own pools took all of it at start-up, or a loop that cannot afford cudaMalloc's device-wide
 * synchronisation.  (No counterpart in the reference: its kernels get scratch from the trainer's
 * pool allocator.)  The split-K scratch is a fixed 16 MiB array inside the library image, present on
 * every GPU that loads the library; a shape whose partial tiles need more is refused with
 * TS2_ERR_TOO_LARGE and belongs to ts2_gemm_dw.  The call runs no cudaMalloc / cudaFree and no
 * allocating library routine.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) and sets the kernel's shared-memory attribute; make that first call
 * before any stream capture.  All calls share the one array and it keeps whatever the last call
 * left there (nothing needs to start at zero: each partial tile is fully rewritten before it is
 * read), so two calls that overlap on the GPU — different streams, or different host threads —
 * race; serialise them on one stream.  A bounded wait that gives up inside its kernels is reported by the next
 * ts2_dev_sync / ts2_wait as TS2_ERR_DEVICE_STATUS, like everywhere else.  out_kind: TS2_OUT_F32 or TS2_OUT_F32_ADD. */
int ts2_gemm_dw_noalloc(int device, void *stream, int prec, int out_kind, int64_t T, int64_t in_dim, int64_t out_dim,
                        const void *dY, const void *X, void *dW, float alpha);
/* Self-test of that entry point's error path (no counterpart in the reference).  Its kernels report a bounded wait
 * that ran out in a status word of their own, a static device variable, because the library's ordinary status word is
 * cudaMalloc'ed on first use; ts2_dev_sync and ts2_wait read and clear both words.  This call makes a wait run out
 * the allowed way (one CTA, a barrier nothing arrives at, under a second) against that word and returns what
 * ts2_dev_sync then reports: TS2_ERR_DEVICE_STATUS is the expected result and the context stays usable. */
int ts2_selftest_wait_limit_noalloc(int device);

/* Grouped forms of the two contractions for expert-sorted rows (the reference's grouped mma.sync
 * GEMMs with GridZ = experts, src/gpt/compute/moe_matmul.cuh:255-291).  Rows are sorted by expert and each
 * expert's segment is padded to a multiple of 128 rows.
 *   ts2_gemm_tn_grouped: C[rows][N] = alpha * A[rows][K] . B[g][N][K]^T where g = tile_group[row / 128]
 *     (device int array, negative: the tile is skipped and its C rows are left untouched);
 *   ts2_gemm_dw_grouped: dW[g][out][in] (+)= alpha * dY[seg]^T . X[seg] over the rows
 *     seg = [seg_ptr[g], seg_ptr[g+1]) (device int array of groups + 1 multiples of 128; empty segments
 *     leave dW[g] untouched). */
int ts2_gemm_tn_grouped(int device, void *stream, int prec, int out_kind, int64_t rows, int64_t N, int64_t K, const void *A,
                        const void *B, void *C, float alpha, int groups, const int32_t *tile_group);
int ts2_gemm_dw_grouped(int device, void *stream, int prec, int out_kind, int64_t rows, int64_t in_dim, int64_t out_dim,
                        const void *dY, const void *X, void *dW, float alpha, int groups, const int32_t *seg_ptr);

/* The bandwidth-bound gradient kernels, one call each (device pointers), exported for operator-level parity tests.
 *  - ts2_op_tilenorm_backward: g = (add ? g : 0) + NormalizeStateBackward(x, dn * (*dyn_scale or 1)) over 128-wide tiles
 *    (src/gpt/compute/cpu_util.cpp:102-134; BackpropLayerNormalize, src/gpt/compute/gpu_layer_norm.cuh:89-115), and the
 *    running maximum of |g| as float bits (absmax_bits, optional; the caller zeroes it);
 *  - ts2_op_cast_grad: g_fast = g * 2^k in the operand format (e4m3 bytes or fp16), 2^k the largest power of two with
 *    max|g| * 2^k <= 128 taken from *absmax_bits, *ginv = 2^-k (ScaleGrad / ComputeGradMult,
 *    src/gpt/compute/gpu_grad_scale.cuh:33-62);
 *  - ts2_op_ffn_act_backward: wide_gate fp16 [T][2F] = [tile-normalized wide | gate], wscale [T][F/128] the tiles' norm
 *    factors, drg fp16 [T][F] -> d_wide_gate [T][2F] = [d wide | d gate] in the operand format (BackpropLoLU +
 *    NormalizeStateBackward of the wide vector, src/gpt/compute/layer_ffn.cu:232-236; BackpropRowTileNormalizeLoLU,
 *    src/gpt/compute/gpu_lolu.cuh:108-173);
 *  - ts2_op_att_gate_backward: qkvg fp16 [T][4Q] (gate in columns [3Q, 4Q)), o fp16 [T][Q], drg fp16 [T][Q] ->
 *    d4[:, 3Q:4Q] = d gate (operand format, row pitch 4Q), dout fp16 [T][Q], dscale[T][Q/128] = sum(dout * o) per head
 *    (BackpropLoLUdScale, src/gpt/compute/gpu_lolu.cuh:72-106). */
int ts2_op_tilenorm_backward(int device, void *stream, const float *x, const float *dn, const float *dyn_scale, int T, int D,
                             float *g, int add, uint32_t *absmax_bits);
int ts2_op_cast_grad(int device, void *stream, int prec, const float *g, int64_t n, const uint32_t *absmax_bits, void *g_fast,
                     float *ginv);
int ts2_op_ffn_act_backward(int device, void *stream, int prec, const void *drg, const void *wide_gate, const float *wscale, int T,
                            int F, void *d_wide_gate);
int ts2_op_att_gate_backward(int device, void *stream, int prec, const void *drg, const void *qkvg, const void *o, int T, int Q,
                             void *d4, void *dout, float *dscale);
/* Row quantization of the int8 pipeline's gradient operands (NormalizeVecsRowMaxKernel with TCudaRngLCG,
 * src/gpt/compute/row_scale.cuh:12-43, src/lib/cuda/cuda_util.cuh:538-559): x fp32 [T][D] on the device, D a multiple
 * of 128; row_scale[t] = max|x[t]| / 127; q[t][d] = the int8 nearest (ties to even, saturating) to
 * x[t][d] / row_scale[t] + u - 0.5, u in [0, 1) drawn for row t by lane h = d mod 32 as its (d / 32 + 1)-th number from
 * state = bits(x[t][h]) * 0x398bf183 + bits(x[t][0]) * 0x1affc3df + t * 0x9023a049, state = state * 0x448e3079 +
 * 0xc484ef10, u = state * 2^-32.  Bit-exact with that definition. */
int ts2_op_rowquant_i8(int device, void *stream, const float *x, int T, int D, int8_t *q, float *row_scale);
/* Per key the range of nodes whose span may hold it, computed on the device as ts2_set_batch does (prefix maximum
 * of the span ends, suffix minimum of the span starts, two binary searches per key).  Host arrays of T ints; nodes
 * without a span have finish < start.  Any spans are allowed, monotone or not. */
int ts2_op_attention_reverse_ranges(int device, void *stream, const int32_t *span_start, const int32_t *span_finish, int T,
                                    int32_t *rev_first, int32_t *rev_last);

/* Expert selection of a mixture-of-experts layer (CpuMoe, src/gpt/compute/layer_moe.cu:287-328;
 * MoeCalcSampleExpertLists, src/gpt/compute/moe_kernels.cu:54-104): the `selected` largest logits per
 * node (lowest index wins ties), weights exp((l - lmax)/2) scaled to L2 norm sqrt(expert_count).
 * Host arrays: logits [T][expert_count] -> ids [T][selected], weights [T][selected]. */
int ts2_moe_route(int device, const float *logits, int T, int expert_count, int selected, int32_t *ids, float *weights);

/* Attention core of one layer over one inclusive key span per node (span_finish < span_start: none):
 * ComputeValLookup / GradQ / GradK, src/gpt/compute/layer_att_reference.h:41-212; Fp16Att,
 * Fp16AttGradQ, Fp16AttGradKV, src/gpt/compute/gpu_att_fp16.cu:41-215, gpu_att_fp16.cuh:60-358.
 * q (normalized, rotated), k (rotated), v (normalized), o, dout: fp16 [T][128*head_count] on the
 * device; lse[T][head_count] = maxDP + log2(sumWeight); dscale[T][head_count] = sum(dout * o);
 * dq, dk, dv fp32 [T][128*head_count]; span arrays are host arrays.  variant 2: tcgen05 kernels;
 * 3 (backward only): the same kernels with dq, dk, dv written as fp16, the form the engine runs
 * (its next kernel reads them once); 0: mma.sync kernels; 1: warp-per-row fp32 formulation (0 and
 * 1 are second opinions for the tests). */
int ts2_attention_forward(int device, void *stream, int variant, const void *q, const void *k, const void *v,
                          const int32_t *span_start, const int32_t *span_finish, int T, int head_count, float alibi_slope,
                          void *o, float *lse);
int ts2_attention_backward(int device, void *stream, int variant, const void *q, const void *k, const void *v, const void *dout,
                           const float *lse, const float *dscale, const int32_t *span_start, const int32_t *span_finish, int T,
                           int head_count, float alibi_slope, void *dq, void *dk, void *dv);

#ifdef __cplusplus
}
#endif
#endif
