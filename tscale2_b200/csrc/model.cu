// The training-step engine behind the model-level C ABI: what the reference builds in
// TSinlgeComputeContext (src/gpt/compute/gpu_transformer.cu:94-502) — forward pass, final
// layer, per-layer backward, gradient hand-off, optimizer, requantisation — laid out
// for one B200:
//   * every activation the backward pass needs is kept (the reference keeps only the
//     normalized state and re-runs each layer's forward inside backward,
//     layer_ffn.cu:53-67,83-113; 180 GB of HBM makes that trade unnecessary);
//   * the Q/K/V/Gate matrices (and Expand/Gate of an FFN) are stored concatenated, with a
//     transposed copy written by the requantiser, so a layer is 6 contractions
//     (2 forward, 2 dX, 2 dW) and no transposes;
//   * weight gradients accumulate in one flat fp32 buffer (matrix order of the C ABI), which
//     is also the message of the data-parallel all-reduce.
// Scale bookkeeping follows the CPU formulas of the reference (cpu_util.cpp, layer_att.cu:368-482,
// layer_ffn.cu:190-248); see the comments at each contraction.
#include "gemm.cuh"
#include "kernels.cuh"
#include <nccl.h>
#include <vector>
#include <cmath>
#include <cstring>
#include <algorithm>
#include <chrono>
#include <thread>

namespace ts2 {
const char *global_error();

static const float LOG2F = 0.693147f; // LOG2, model_dim.h:16

struct Matrix {
    int64_t x = 0, y = 0;
    int row_disp_size = 1;
    float sparsity = 1.f;
    float *w = nullptr, *avg = nullptr, *grad = nullptr; // grad points into the flat buffer
    float *row_disp = nullptr, *sum_weight = nullptr, *sko = nullptr;
    size_t offset = 0; // element offset in the flat buffers
};

// Expert-parallel exchange of one mixture-of-experts layer, computed on the host from every rank's per-expert row counts.
// Own rows are sorted by expert (segments padded to 128 rows), so the rows for one destination expert are one block.
struct EpPlan {
    struct Move {
        int peer;      // the other rank (this rank: a local copy)
        int own_row;   // first row in this rank's own expert-sorted layout
        int x_row;     // first row in the owner's layout
        int rows;
    };
    std::vector<Move> out;  // blocks of own rows that go to the experts' owners (x_row: in the owner's layout)
    std::vector<Move> in;   // blocks this rank receives for its experts (own_row: in the sender's layout)
    std::vector<int> x_seg, x_valid; // [E + 1], [E]: segments of the received rows, empty for other ranks' experts
    int x_rows = 0;                  // rows of the received layout, a multiple of 128
};

struct Layer {
    int type = 0;
    float slope = 0;
    int att_type = 0;
    int mat0 = 0;   // index of the first matrix
    int wide = 0;   // Q (attention) or F (ffn)
    int ncat = 0;   // 4 (attention) or 2 (ffn)
    // quantized weights
    void *Wcat = nullptr, *WcatT = nullptr; // [ncat*wide][D], [D][ncat*wide]
    void *Wc = nullptr, *WcT = nullptr;     // [D][wide], [wide][D]
    float *fwd_col = nullptr;               // [ncat*wide] forward column scales
    float *bwd_row = nullptr;               // [ncat*wide] dW row scales
    // saved activations
    void *n_fast = nullptr;                 // [T][D]
    __half *cat16 = nullptr;                // [T][ncat*wide]: Q|K|V|Gate or wide|gate
    __half *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr; // attention
    float *qscale = nullptr, *vscale = nullptr, *lse = nullptr;
    __half *what = nullptr;                 // ffn: normalized wide
    float *wscale = nullptr;
    void *rg = nullptr;                     // [T][wide]  (MoE: [rows][X])
    // mixture of experts: wide = expert width X, ncat = 2; quantized weights are per expert:
    // Wcat [E][2X][D], WcatT [E][D][2X], Wc [E][D][X], WcT [E][X][D]; select matrix padded to epad rows / columns
    void *Wsel = nullptr, *WselT = nullptr; // [epad][D], [D][epad]
    float *bwd_row_e = nullptr;             // [X] 1 / sko of the expand matrix
    void *n_rows = nullptr;                 // [rows][D] gathered normalized state
    float *logits = nullptr;                // [T][epad]
    int *ids = nullptr, *slot_of = nullptr, *token_of = nullptr, *tile_group = nullptr, *seg_ptr = nullptr;
    float *weights = nullptr, *weight_of = nullptr;
    // expert parallel: the tables above describe this rank's own (token, choice) rows; the rows the rank computes (received
    // for the experts it owns) have tables of their own, and a plan of the exchange kept from the forward pass
    int *x_token_of = nullptr, *x_tile_group = nullptr, *x_seg = nullptr, *x_valid = nullptr;
    float *x_weight_of = nullptr;
    int4 *d_moves = nullptr; // plan.out then plan.in as {peer, sender row, owner row, rows}
    EpPlan plan;
};

// A bucket is a run of matrices that is contiguous in the flat buffers: the embedding, the final layer, one per layer.
// It is the unit of the data-parallel exchange: its gradient is reduce-scattered as soon as the backward pass has
// written it, every rank updates and requantises one contiguous 1 / world part of it, and the quantized bytes are
// all-gathered.  Its length is padded to a multiple of BUCKET_PAD elements so that it divides evenly.
static constexpr size_t BUCKET_PAD = 1024;
struct Bucket {
    size_t off = 0, elems = 0; // element offset / padded length in the flat buffers
    int mat0 = 0, mat1 = 0;    // matrices [mat0, mat1)
    int qsize = 1;             // bytes per quantized element
    uint8_t *qflat = nullptr;  // row-major quantized copies of the bucket's matrices, in flat order (elems * qsize bytes)
    // one expert matrix of a mixture-of-experts layer ([E x rows][cols]: an expert is a row range, so the r-th of N parts
    // of the bucket is exactly the experts of rank r)
    bool expert_matrix = false;
    bool owner_only = false; // expert parallel: the owner holds the complete gradient of its part, nothing is exchanged
};

struct BatchDev {
    // one host-to-device copy per batch brings the raw CSR arrays into `raw`; label_arr / label_ptr point into it,
    // everything else is derived on the device (kernels_batch.cu)
    uint32_t *raw = nullptr;
    size_t raw_cap = 0; // elements, also the size of one pinned staging slot
    uint32_t *label_arr = nullptr, *label_ptr = nullptr;
    uint32_t n_labels = 0;
    int *target = nullptr;
    std::vector<int *> span_start, span_finish, rev_first, rev_last;
    int *scan_tmp = nullptr; // batch_scan_tmp_elems(max_nodes)
    int *status = nullptr;   // {code, where, detail, detail}: the first malformed element seen since it was last reported
    LabelIndex ix;
    bool ix_sorted = false;
    size_t label_cap = 0;
    int node_count = 0, target_count = 0;
    // two pinned staging slots: the next batch is written while the copy of the previous one may still be queued
    cudaEvent_t slot_ev[2] = {nullptr, nullptr};
    bool slot_used[2] = {false, false};
    int next_slot = 0;
};

} // namespace ts2

using namespace ts2;

struct ts2_model {
    ts2_model_descr descr;
    std::vector<ts2_layer_params> layer_params;
    int device = 0, max_nodes = 0;
    int D = 0, H = 0, Q = 0, F = 0, V = 0, L = 0;
    int ft = 0;
    int kind = KIND_E4M3;
    float s_act = 16.f;
    cudaStream_t stream = nullptr, comm_stream = nullptr;
    // flat, sharded optimizer (kernels_opt.cu): buckets, per-row vectors over all matrices, segment tables for the
    // whole model (requantisation at creation / ts2_set_params) and for this rank's parts (training steps)
    std::vector<Bucket> buckets;
    std::vector<int> mat_bucket, mat_grow0;
    size_t flat_elems = 0;
    int n_rows_total = 0;
    float *rowsum = nullptr, *row_scale = nullptr; // [n_rows_total]
    double *roww2 = nullptr;                       // [n_rows_total]
    OptMat *d_optmats = nullptr;
    OptSeg *d_segs_full = nullptr, *d_segs_shard = nullptr;
    int nseg_full = 0, nitems_full = 0, nseg_shard = 0, nitems_shard = 0;
    bool master_stale = false; // data parallel: the fp32 weights / momentum outside this rank's parts are out of date
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr, ev_grads = nullptr, ev_reduced = nullptr, ev_t0 = nullptr, ev_t1 = nullptr;
    std::string error;
    std::vector<void *> allocs;
    std::vector<Matrix> mats;
    std::vector<Layer> layers;
    size_t total_params = 0;
    float *w_flat = nullptr, *avg_flat = nullptr, *grad_flat = nullptr;
    float *skos = nullptr; // [n_mats]
    float *bias = nullptr;
    bool has_bias = false; // a model created without a bias vector skips the loads (the buffer then holds zeros)
    __half *embed16 = nullptr;
    void *Wf = nullptr;      // [V][D] fast
    __half *WfT16 = nullptr; // [D][V]
    // activations
    std::vector<float *> states; // L+1
    float *g = nullptr, *dn = nullptr;
    void *g_fast = nullptr;
    void *nF_fast = nullptr;
    __half *nF16 = nullptr;
    __half *logits = nullptr;
    int chunk = 0;
    __half *drg = nullptr, *dout = nullptr;
    void *dcat = nullptr;
    float *dscale = nullptr;
    __half *dq = nullptr, *dk = nullptr, *dv = nullptr; // attention gradients, fp16 between the attention core and its post-kernel
    // int8 pipeline: the gradient operands of the dX contractions are row-quantized int8 (+ one fp32 scale per row), the
    // dW contractions read fp16: the state gradient and the first-contraction output gradients as fp16, and the int8
    // activations widened to fp16
    __half *g16 = nullptr, *dcat16 = nullptr, *x16 = nullptr;
    float *g_rs = nullptr, *dcat_rs = nullptr;
    float *rope = nullptr;
    // mixture-of-experts scratch shared by the layers
    int E = 0, K = 0, X = 0, epad = 0, moe_rows = 0;
    float *moe_y = nullptr, *dmoe_part = nullptr;
    void *moe_g = nullptr, *moe_dl = nullptr;
    int *moe_hist = nullptr, *moe_base = nullptr;
    // expert parallel (ts2_set_expert_parallel): rank r owns experts [r E / world, (r + 1) E / world)
    bool ep = false;
    int x_cap = 0;                                    // capacity of the received layout in rows
    void *own_rows = nullptr, *own_g = nullptr;       // staging in this rank's own layout: gathered rows going out
    float *own_y = nullptr, *own_part = nullptr;      // and results coming back
    int *cnt_own = nullptr, *cnt_all = nullptr;       // [E], [world][E] row counts per expert
    int *h_cnt = nullptr;                             // pinned copy of cnt_all
    ncclComm_t comm_x = nullptr;                      // communicator of the row exchanges (a split of comm)
    // exchange over peer memory: the staging buffers of every rank mapped into this process (CUDA IPC); tables of the
    // N base pointers per buffer on the device; a 4-byte all-reduce on comm_x is the barrier between "written" and "read"
    enum { PB_OWN_ROWS, PB_OWN_G, PB_OWN_W, PB_MOE_Y, PB_PART, PB_COUNT };
    bool x_peer = false;
    std::vector<void *> ipc_opened;
    uint8_t **d_peer = nullptr; // [PB_COUNT][world]
    float *own_w = nullptr;     // routing weights of the own rows, staged for the owners
    int *x_flag = nullptr;
    // device time of the exchanges (events around each one, summed by ts2_get_exchange_ms); off unless asked for
    bool x_timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> x_events;
    size_t x_events_used = 0;
    double x_bytes = 0; // bytes this rank sent to other ranks since the last read
    unsigned *absmax = nullptr; // [L+2]
    float *ginv = nullptr, *fscale = nullptr, *logp = nullptr;
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    int64_t max_rows = 0;
    BatchDev batch;
    void *pinned = nullptr;
    size_t pinned_bytes = 0;
    int *h_batch_status = nullptr; // pinned copy of batch.status, refreshed by every ts2_set_batch
    bool grads_dirty = false; // the flat gradient holds an accumulated, not yet applied gradient
    bool reduce_in_backward = false; // this backward pass is followed by apply(): all-reduce every layer's gradient as soon as it is complete
    int gemm_tag = 0; // class of the contractions being queued (timing statistics)
    bool debug_taps = false;
    float *grad_taps = nullptr;
    // step health: health[b] = number of the first step whose state gradient at layer boundary b held a NaN or an
    // infinity (0: never); the training error of the last LOSS_RING steps (sum of log p, one slot per step)
    static constexpr int LOSS_RING = 256;
    unsigned *health = nullptr; // [L + 1]
    float *logp_ring = nullptr; // [LOSS_RING]
    int ring_targets[LOSS_RING] = {};
    unsigned step_no = 0;       // steps (ts2_backprop calls) so far
    // debug trace: checksum + non-finite count of every intermediate buffer of the step (off by default)
    static constexpr int TRACE_MAX = 1024;
    bool trace_on = false;
    unsigned long long *trace_dev = nullptr; // [TRACE_MAX][4]: checksum, non-finite count, max |x| bits, unused
    std::vector<std::string> trace_names;
    std::string capture_name; // trace record whose buffer is also copied aside ("dk[18]"), for ts2_debug_read("capture")
    void *capture_buf = nullptr;
    size_t capture_cap = 0, capture_bytes = 0;
    float last_ms = 0;
    bool timing_valid = false;
    int last_targets = 0;
    // data parallel
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

namespace {

int mfail(ts2_model *m, int code)
{
    if (m)
        m->error = g_last_error;
    return code;
}

#define M_TRY(expr)                 \
    do {                            \
        int _rc = (expr);           \
        if (_rc != TS2_OK)          \
            return mfail(m, _rc);   \
    } while (0)

template <class T>
int dalloc(ts2_model *m, T **p, size_t count)
{
    void *q = nullptr;
    size_t bytes = std::max<size_t>(count * sizeof(T), 256);
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess)
        return fail(TS2_ERR_CUDA, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    m->allocs.push_back(q);
    *p = (T *)q;
    return TS2_OK;
}

// replaces a device buffer by a larger one (contents are not kept); the device must be idle
template <class T>
int regrow(ts2_model *m, T **p, size_t count)
{
    if (*p) {
        auto it = std::find(m->allocs.begin(), m->allocs.end(), (void *)*p);
        if (it != m->allocs.end())
            m->allocs.erase(it);
        cudaFree((void *)*p);
        *p = nullptr;
    }
    return dalloc(m, p, count);
}

int layer_matrix_count(int type) { return type == TS2_LAYER_ATT ? 5 : type == TS2_LAYER_FFN ? 3 : type == TS2_LAYER_MOE ? 4 : -1; }

Ctx ctx_of(ts2_model *m)
{
    Ctx c;
    c.device = m->device;
    c.stream = m->stream;
    c.ft = m->ft;
    c.s_act = m->s_act;
    return c;
}

size_t fast_size(const ts2_model *m) { return m->ft == 1 ? 2 : 1; }

// C = epilogue(A[M][K] . B[N][K]^T), K contiguous in both
int gemm_tn(ts2_model *m, int kind, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda, const void *B, int64_t ldb, void *C,
            int64_t ldc, const Epilogue &epi)
{
    GemmArgs a;
    a.device = m->device;
    a.stream = m->stream;
    a.kind = kind;
    a.mn_major = false;
    a.M = M, a.N = N, a.K = K;
    a.A = A, a.lda = lda, a.B = B, a.ldb = ldb, a.C = C, a.ldc = ldc;
    a.epi = epi;
    a.tag = m->gemm_tag;
    a.workspace = m->workspace;
    a.workspace_bytes = m->workspace_bytes;
    return gemm(a);
}

// dW[Mo][Ni] = epilogue(dY[T][Mo]^T . X[T][Ni]), both token-major
int gemm_dw(ts2_model *m, int kind, int64_t Mo, int64_t Ni, int64_t T, const void *dY, int64_t ldy, const void *X, int64_t ldx, float *dW,
            const Epilogue &epi)
{
    GemmArgs a;
    a.device = m->device;
    a.stream = m->stream;
    a.kind = kind;
    a.mn_major = true;
    a.M = Mo, a.N = Ni, a.K = T;
    a.A = dY, a.lda = ldy, a.B = X, a.ldb = ldx, a.C = dW, a.ldc = Ni;
    a.epi = epi;
    a.tag = m->gemm_tag == GEMM_TAG_FINAL ? GEMM_TAG_FINAL : GEMM_TAG_DW;
    a.workspace = m->workspace;
    a.workspace_bytes = m->workspace_bytes;
    return gemm(a);
}

// rows of A are expert-sorted: every 128-row tile reads the weights of its expert (B has E * N rows)
int gemm_rows_grouped(ts2_model *m, const Layer &ly, int64_t rows, int64_t N, int64_t K, const void *A, int64_t lda, const void *B,
                      int64_t ldb, void *C, int64_t ldc, const Epilogue &epi)
{
    GemmArgs a;
    a.device = m->device;
    a.stream = m->stream;
    a.kind = m->kind;
    a.mn_major = false;
    a.M = rows, a.N = N, a.K = K;
    a.A = A, a.lda = lda, a.B = B, a.ldb = ldb, a.C = C, a.ldc = ldc;
    a.epi = epi;
    a.tag = m->gemm_tag;
    a.group_mode = 1;
    a.groups = m->E;
    a.tile_group = m->ep ? ly.x_tile_group : ly.tile_group;
    a.group_rows_b = (int)N;
    return gemm(a);
}

// per-expert weight gradients: dW_e[Mo][Ni] = dY_e^T . X_e over the rows of expert e's segment
int gemm_k_grouped(ts2_model *m, const Layer &ly, int64_t Mo, int64_t Ni, int64_t rows, const void *dY, int64_t ldy, const void *X,
                   int64_t ldx, float *dW, int64_t stride, const Epilogue &epi)
{
    GemmArgs a;
    a.device = m->device;
    a.stream = m->stream;
    a.kind = m->kind;
    a.mn_major = true;
    a.M = Mo, a.N = Ni, a.K = rows;
    a.A = dY, a.lda = ldy, a.B = X, a.ldb = ldx, a.C = dW, a.ldc = Ni;
    a.epi = epi;
    a.tag = GEMM_TAG_DW;
    a.group_mode = 2;
    a.groups = m->E;
    a.group_kptr = m->ep ? ly.x_seg : ly.seg_ptr;
    a.c_group_stride = stride;
    return gemm(a);
}

int validate(const ts2_model_descr *d)
{
    if (!d)
        return fail(TS2_ERR_INVALID_ARG, "null model description");
    if (d->dim <= 0 || d->dim % 128)
        return fail(TS2_ERR_INVALID_ARG, "dim must be a positive multiple of 128 (got %d)", d->dim);
    if (d->q_dim != 128 || d->tt_dim != 128)
        return fail(TS2_ERR_UNSUPPORTED, "q_dim and tt_dim must be 128 (got %d, %d)", d->q_dim, d->tt_dim);
    if (d->head_count <= 0 || d->ffn_tiles < 0 || d->layer_count < 0 || (d->layer_count && !d->layers))
        return fail(TS2_ERR_INVALID_ARG, "bad head / ffn / layer counts");
    if (d->label_count <= 0 || d->output_token_count <= 0 || d->output_token_count % 32)
        return fail(TS2_ERR_INVALID_ARG, "label_count must be positive and output_token_count a positive multiple of 32");
    // flags that change the compute path in ways this backend does not implement (model_dim.h:40,51-52): per-node
    // sample vectors added to the embedding (MPF_SAMPLE_EMBED_VECTORS, cpu_transformer.cpp:93-99), the RNN variants
    if (d->flags & (0x10ull | 0x10000ull | 0x20000ull))
        return fail(TS2_ERR_UNSUPPORTED, "model flags 0x%llx: MPF_SAMPLE_EMBED_VECTORS / MPF_RNN / MPF_RNN_CROSS are not supported",
                    (unsigned long long)d->flags);
    if (d->precision != TS2_PREC_FP8 && d->precision != TS2_PREC_F16 && d->precision != TS2_PREC_INT8)
        return fail(TS2_ERR_UNSUPPORTED, "precision must be TS2_PREC_FP8, TS2_PREC_F16 or TS2_PREC_INT8");
    for (int l = 0; l < d->layer_count; ++l) {
        int t = d->layers[l].layer_type;
        if (t == TS2_LAYER_MOE) {
            if (d->precision == TS2_PREC_INT8)
                return fail(TS2_ERR_UNSUPPORTED, "layer %d: mixture-of-experts layers are not available with TS2_PREC_INT8", l);
            if (d->moe_expert_count < 1 || d->moe_expert_count > 128 || d->moe_selected < 1 || d->moe_selected > 8 ||
                d->moe_selected > d->moe_expert_count || d->expert_dim <= 0 || d->expert_dim % 128)
                return fail(TS2_ERR_UNSUPPORTED,
                            "layer %d: MoE needs 1..128 experts, 1..8 selected, expert_dim a multiple of 128 (got %d, %d, %d)", l,
                            d->moe_expert_count, d->moe_selected, d->expert_dim);
            continue;
        }
        if (t != TS2_LAYER_ATT && t != TS2_LAYER_FFN)
            return fail(TS2_ERR_UNSUPPORTED, "layer %d: unsupported layer type %d", l, t);
        if (t == TS2_LAYER_FFN && d->ffn_tiles <= 0)
            return fail(TS2_ERR_INVALID_ARG, "ffn layer with ffn_tiles = 0");
        if (t == TS2_LAYER_ATT && (d->layers[l].attention_type_id < 0 || d->layers[l].attention_type_id >= d->attention_type_count))
            return fail(TS2_ERR_INVALID_ARG, "layer %d: attention_type_id out of range", l);
    }
    return TS2_OK;
}

void shapes_of(const ts2_model_descr *d, std::vector<std::pair<int64_t, int64_t>> *out) // (x, y)
{
    const int64_t D = d->dim, Q = (int64_t)d->q_dim * d->head_count, TT = (int64_t)d->tt_dim * d->head_count, F = 128ll * d->ffn_tiles;
    out->clear();
    out->push_back({D, d->label_count});
    out->push_back({D, d->output_token_count});
    for (int l = 0; l < d->layer_count; ++l) {
        switch (d->layers[l].layer_type) {
        case TS2_LAYER_ATT:
            out->push_back({D, Q});
            out->push_back({D, Q});
            out->push_back({D, TT});
            out->push_back({D, TT});
            out->push_back({TT, D});
            break;
        case TS2_LAYER_FFN:
            out->push_back({D, F});
            out->push_back({D, F});
            out->push_back({F, D});
            break;
        case TS2_LAYER_MOE: {
            const int64_t xp = d->expert_dim, e = d->moe_expert_count;
            out->push_back({D, xp * e});
            out->push_back({D, xp * e});
            out->push_back({xp, D * e});
            out->push_back({D, e});
            break;
        }
        default:
            break;
        }
    }
}

// Layout of the flat parameter buffers: the matrices in C-ABI order, grouped into buckets (embedding, final layer, one
// per layer), every bucket padded to BUCKET_PAD elements
void layout_buckets(const ts2_model_descr *d, const std::vector<std::pair<int64_t, int64_t>> &shapes, std::vector<Bucket> *buckets,
                    std::vector<size_t> *mat_off, std::vector<int> *mat_bucket)
{
    const int n_mats = (int)shapes.size();
    // buckets: embedding, final layer, one per layer; a mixture-of-experts layer has one per matrix (expand, gate,
    // contract, select)
    std::vector<int> first = {0, 1};
    std::vector<bool> expert = {false, false};
    int mi = 2;
    for (int l = 0; l < d->layer_count; ++l) {
        const int n = layer_matrix_count(d->layers[l].layer_type);
        if (d->layers[l].layer_type == TS2_LAYER_MOE) {
            for (int j = 0; j < n; ++j) {
                first.push_back(mi + j);
                expert.push_back(j < 3);
            }
        } else {
            first.push_back(mi);
            expert.push_back(false);
        }
        mi += n;
    }
    first.push_back(n_mats);
    buckets->assign(first.size() - 1, Bucket());
    for (size_t b = 0; b + 1 < first.size(); ++b)
        (*buckets)[b].expert_matrix = expert[b];
    mat_off->assign(n_mats, 0);
    mat_bucket->assign(n_mats, 0);
    size_t off = 0;
    for (size_t b = 0; b + 1 < first.size(); ++b) {
        Bucket &bk = (*buckets)[b];
        bk.mat0 = first[b];
        bk.mat1 = first[b + 1];
        bk.off = off;
        for (int i = bk.mat0; i < bk.mat1; ++i) {
            (*mat_off)[i] = off;
            (*mat_bucket)[i] = (int)b;
            off += (size_t)shapes[i].first * shapes[i].second;
        }
        off = (off + BUCKET_PAD - 1) / BUCKET_PAD * BUCKET_PAD;
        bk.elems = off - bk.off;
    }
}

// ---- optimizer + requantisation over the flat buffers -------------------------------------------------------
// the parts of the matrices that rank `rank` of `world` owns: one contiguous 1 / world part of every bucket
void build_segments(const ts2_model *m, int world, int rank, std::vector<OptSeg> *segs, int *nitems)
{
    segs->clear();
    int items = 0;
    for (const Bucket &bk : m->buckets) {
        const size_t part = bk.elems / world, lo = bk.off + part * rank, hi = lo + part;
        for (int i = bk.mat0; i < bk.mat1; ++i) {
            const Matrix &mt = m->mats[i];
            const size_t m_lo = mt.offset, m_hi = mt.offset + (size_t)mt.x * mt.y;
            const size_t a = std::max(lo, m_lo), b = std::min(hi, m_hi);
            if (b <= a)
                continue;
            OptSeg sg;
            sg.flat_off = (long long)mt.offset;
            sg.a = (long long)(a - m_lo);
            sg.b = (long long)(b - m_lo);
            sg.x = (int)mt.x;
            sg.y = (int)mt.y;
            sg.row0 = (int)(sg.a / mt.x);
            sg.nrows = (int)((sg.b - 1) / mt.x) - sg.row0 + 1;
            sg.grow0 = m->mat_grow0[i];
            sg.item0 = items;
            sg.mat = i;
            sg.qsize = bk.qsize;
            sg.qkind = bk.qsize == 2 ? 1 : (m->ft == 2 ? 2 : 0);
            sg.qbase = bk.qflat + (mt.offset - bk.off) * bk.qsize;
            sg.sparsity = mt.sparsity;
            items += sg.nrows;
            segs->push_back(sg);
        }
    }
    *nitems = items;
}

int upload_segments(ts2_model *m, const std::vector<OptSeg> &segs, OptSeg **dst)
{
    if (!*dst)
        M_TRY(dalloc(m, dst, m->mats.size() + 2 * m->buckets.size() + 4)); // a part cuts at most two matrices more per bucket
    TS2_CUDA(cudaMemcpyAsync(*dst, segs.data(), segs.size() * sizeof(OptSeg), cudaMemcpyHostToDevice, m->stream));
    TS2_CUDA(cudaStreamSynchronize(m->stream)); // the host vector may go away
    return TS2_OK;
}

#define M_NCCL(expr)                                                                              \
    do {                                                                                          \
        ncclResult_t _r = (expr);                                                                 \
        if (_r != ncclSuccess)                                                                    \
            return mfail(m, fail(TS2_ERR_COMM, "%s failed: %s", #expr, ncclGetErrorString(_r))); \
    } while (0)

// ---- expert parallel ------------------------------------------------------------------------------------------
// The plan of one layer's exchange from all ranks' per-expert row counts cnt[world][E] (pure host arithmetic; every rank
// computes the same numbers).  Returns the largest received layout over all ranks in *max_x_rows.
void ep_plan(int world, int rank, int E, const int *cnt, EpPlan *p, int *max_x_rows)
{
    const int per = E / world;
    auto pad = [](int n) { return (n + 127) / 128 * 128; };
    std::vector<int> own_seg(E + 1, 0), total(E, 0), before(E, 0), owner_seg(E, 0);
    std::vector<int> seg_of((size_t)world * (E + 1), 0); // every rank's own expert-sorted layout
    for (int s = 0; s < world; ++s)
        for (int e = 0; e < E; ++e)
            seg_of[(size_t)s * (E + 1) + e + 1] = seg_of[(size_t)s * (E + 1) + e] + pad(cnt[s * E + e]);
    for (int e = 0; e < E; ++e) {
        own_seg[e + 1] = own_seg[e] + pad(cnt[rank * E + e]);
        for (int s = 0; s < world; ++s) {
            if (s == rank)
                before[e] = total[e];
            total[e] += cnt[s * E + e];
        }
    }
    *max_x_rows = 0;
    for (int o = 0; o < world; ++o) {
        int pos = 0;
        for (int e = o * per; e < (o + 1) * per; ++e) {
            owner_seg[e] = pos;
            pos += pad(total[e]);
        }
        *max_x_rows = std::max(*max_x_rows, pos);
    }
    p->out.clear();
    p->in.clear();
    p->x_seg.assign(E + 1, 0);
    p->x_valid.assign(E, 0);
    int pos = 0;
    for (int e = 0; e < E; ++e) {
        const int owner = e / per;
        p->x_seg[e] = pos;
        if (cnt[rank * E + e])
            p->out.push_back({owner, own_seg[e], owner_seg[e] + before[e], cnt[rank * E + e]});
        if (owner != rank)
            continue;
        int off = 0;
        for (int s = 0; s < world; ++s) {
            const int n = cnt[s * E + e];
            if (n)
                p->in.push_back({s, seg_of[(size_t)s * (E + 1) + e], pos + off, n});
            off += n;
        }
        p->x_valid[e] = off;
        pos += pad(off);
    }
    p->x_seg[E] = pos;
    p->x_rows = pos;
}

// counts of all ranks -> plan, tables of the received layout.  Waits for the device (the counts come from this step's
// routing): once per mixture-of-experts layer in the forward pass; the backward pass reuses the plan.
// The exchanges use a communicator of their own (comm_x) on the compute stream - they are on the critical path anyway -
// so that they do not queue behind the gradient reduce-scatters of the communication stream.
int ep_prepare(ts2_model *m, Layer &ly)
{
    const int E = m->E, N = m->world;
    M_NCCL(ncclAllGather(m->cnt_own, m->cnt_all, E, ncclInt32, m->comm_x, m->stream));
    TS2_CUDA(cudaMemcpyAsync(m->h_cnt, m->cnt_all, (size_t)N * E * 4, cudaMemcpyDeviceToHost, m->stream));
    TS2_CUDA(cudaStreamSynchronize(m->stream));
    int max_x = 0;
    ep_plan(N, m->rank, E, m->h_cnt, &ly.plan, &max_x);
    if (max_x > m->x_cap) // every rank sees the same counts and takes the same decision
        return fail(TS2_ERR_TOO_LARGE,
                    "expert parallel: one rank would receive %d rows, the capacity is %d (ts2_set_expert_parallel with a larger factor)",
                    max_x, m->x_cap);
    TS2_CUDA(cudaMemcpyAsync(ly.x_seg, ly.plan.x_seg.data(), (size_t)(E + 1) * 4, cudaMemcpyHostToDevice, m->stream));
    TS2_CUDA(cudaMemcpyAsync(ly.x_valid, ly.plan.x_valid.data(), (size_t)E * 4, cudaMemcpyHostToDevice, m->stream));
    if (ly.plan.x_rows)
        M_TRY(moe_ep_tables(ctx_of(m), ly.x_seg, ly.x_valid, E, ly.plan.x_rows, ly.x_tile_group, ly.x_token_of));
    if (m->x_peer) {
        const size_t n = ly.plan.out.size() + ly.plan.in.size();
        static_assert(sizeof(EpPlan::Move) == sizeof(int4), "moves are uploaded as they are");
        if (!ly.plan.out.empty())
            TS2_CUDA(cudaMemcpyAsync(ly.d_moves, ly.plan.out.data(), ly.plan.out.size() * sizeof(int4), cudaMemcpyHostToDevice, m->stream));
        if (!ly.plan.in.empty())
            TS2_CUDA(cudaMemcpyAsync(ly.d_moves + ly.plan.out.size(), ly.plan.in.data(), ly.plan.in.size() * sizeof(int4),
                                     cudaMemcpyHostToDevice, m->stream));
        (void)n;
    }
    return TS2_OK;
}

// The same exchange with this library's own copy kernel over peer memory: after a barrier (all ranks have written their
// side) the rank that needs a block pulls it from the other rank's buffer.  which_remote: the table of the buffer the
// blocks are read from (the senders' staging buffer on the way to the owners, the owners' result buffer on the way
// back); the barrier of the next exchange also tells that every rank is done reading this one's sources.
int ep_exchange_peer(ts2_model *m, const Layer &ly, bool to_owner, int which_remote, void *local, size_t row_bytes, bool zero_pads,
                     bool barrier = true)
{
    const EpPlan &p = ly.plan;
    cudaStream_t cs = m->stream;
    std::pair<cudaEvent_t, cudaEvent_t> *ev = nullptr;
    if (m->x_timing) {
        if (m->x_events_used == m->x_events.size()) {
            std::pair<cudaEvent_t, cudaEvent_t> e;
            TS2_CUDA(cudaEventCreate(&e.first));
            TS2_CUDA(cudaEventCreate(&e.second));
            m->x_events.push_back(e);
        }
        ev = &m->x_events[m->x_events_used++];
    }
    static const bool copy_only = getenv("TS2_EP_TIME_COPY_ONLY") != nullptr; // leave the barrier out of the timed part
    if (ev && !copy_only)
        TS2_CUDA(cudaEventRecord(ev->first, cs));
    if (barrier)
        M_NCCL(ncclAllReduce(m->x_flag, m->x_flag, 1, ncclInt32, ncclMax, m->comm_x, cs));
    if (ev && copy_only)
        TS2_CUDA(cudaEventRecord(ev->first, cs));
    // on the way to the owners this rank pulls what it receives (plan.in); on the way back what it sent (plan.out)
    const std::vector<EpPlan::Move> &list = to_owner ? p.in : p.out;
    const int4 *moves = ly.d_moves + (to_owner ? p.out.size() : 0);
    long long bytes = 0;
    for (const EpPlan::Move &mv : list) {
        bytes += (long long)mv.rows * (long long)row_bytes;
        if (m->x_timing && mv.peer != m->rank)
            m->x_bytes += (double)mv.rows * row_bytes; // received = sent, by symmetry of the roles
    }
    M_TRY(moe_pull_rows(ctx_of(m), moves, (int)list.size(), m->d_peer + (size_t)which_remote * m->world, local, (int)row_bytes, to_owner,
                        bytes));
    if (ev)
        TS2_CUDA(cudaEventRecord(ev->second, cs));
    if (to_owner && zero_pads && p.x_rows)
        M_TRY(moe_zero_pad_rows(ctx_of(m), local, (int)row_bytes, ly.x_seg, ly.x_valid, m->E));
    return TS2_OK;
}

// to_owner: rows of `own` (this rank's expert-sorted layout) go to the experts' owners, which place them in `x`
// (their received layout); otherwise the way back.  Blocks travel in expert order between every pair of ranks, so
// sends and receives pair up.
int ep_exchange(ts2_model *m, const Layer &ly, bool to_owner, void *own, void *x, size_t row_bytes, bool zero_pads)
{
    const EpPlan &p = ly.plan;
    cudaStream_t cs = m->stream;
    uint8_t *o = (uint8_t *)own, *xx = (uint8_t *)x;
    std::pair<cudaEvent_t, cudaEvent_t> *ev = nullptr;
    if (m->x_timing) {
        if (m->x_events_used == m->x_events.size()) {
            std::pair<cudaEvent_t, cudaEvent_t> e;
            TS2_CUDA(cudaEventCreate(&e.first));
            TS2_CUDA(cudaEventCreate(&e.second));
            m->x_events.push_back(e);
        }
        ev = &m->x_events[m->x_events_used++];
        TS2_CUDA(cudaEventRecord(ev->first, cs));
        for (const EpPlan::Move &mv : to_owner ? p.out : p.in)
            if (mv.peer != m->rank)
                m->x_bytes += (double)mv.rows * row_bytes;
    }
    for (const EpPlan::Move &mv : p.in)
        if (mv.peer == m->rank) {
            uint8_t *a = o + (size_t)mv.own_row * row_bytes, *b = xx + (size_t)mv.x_row * row_bytes;
            TS2_CUDA(cudaMemcpyAsync(to_owner ? b : a, to_owner ? a : b, (size_t)mv.rows * row_bytes, cudaMemcpyDeviceToDevice, cs));
        }
    M_NCCL(ncclGroupStart());
    for (const EpPlan::Move &mv : p.out) {
        if (mv.peer == m->rank)
            continue;
        uint8_t *a = o + (size_t)mv.own_row * row_bytes;
        if (to_owner)
            M_NCCL(ncclSend(a, (size_t)mv.rows * row_bytes, ncclUint8, mv.peer, m->comm_x, cs));
        else
            M_NCCL(ncclRecv(a, (size_t)mv.rows * row_bytes, ncclUint8, mv.peer, m->comm_x, cs));
    }
    for (const EpPlan::Move &mv : p.in) {
        if (mv.peer == m->rank)
            continue;
        uint8_t *b = xx + (size_t)mv.x_row * row_bytes;
        if (to_owner)
            M_NCCL(ncclRecv(b, (size_t)mv.rows * row_bytes, ncclUint8, mv.peer, m->comm_x, cs));
        else
            M_NCCL(ncclSend(b, (size_t)mv.rows * row_bytes, ncclUint8, mv.peer, m->comm_x, cs));
    }
    M_NCCL(ncclGroupEnd());
    if (ev)
        TS2_CUDA(cudaEventRecord(ev->second, cs));
    if (to_owner && zero_pads && p.x_rows)
        M_TRY(moe_zero_pad_rows(ctx_of(m), x, (int)row_bytes, ly.x_seg, ly.x_valid, m->E));
    return TS2_OK;
}

// transposed copies, per-expert layouts and scale vectors from the row-major quantized matrices and their scales
int post_quantize(ts2_model *m)
{
    Ctx c = ctx_of(m);
    const int D = m->D;
    const size_t fs = fast_size(m);
    // final layer: fp16 transposed copy of the same quantized values for the dX contraction
    M_TRY(qcopy_block(c, m->Wf, D, m->V, D, (int)fs, nullptr, 0, m->WfT16, m->V, m->ft == 0 ? 1 : m->ft == 2 ? 2 : 0));
    const float a = sqrtf(1.0f / D) / (m->s_act * 32.f);
    for (Layer &ly : m->layers) {
        const int W = ly.wide, n = ly.ncat;
        auto qsrc = [&](int mat) {
            const Bucket &bk = m->buckets[m->mat_bucket[mat]];
            return bk.qflat + (m->mats[mat].offset - bk.off) * fs;
        };
        if (ly.type == TS2_LAYER_MOE) {
            // the flat order keeps each matrix whole ([E X][D] expand, gate; [E D][X] contract); the contractions want
            // the blocks of one expert together: Wcat [E][2X][D], WcatT [E][D][2X], Wc [E][D][X], WcT [E][X][D]
            const int E = m->E, X = m->X;
            for (int e = 0; e < E; ++e) {
                uint8_t *cat = (uint8_t *)ly.Wcat + (size_t)e * 2 * X * D * fs, *catT = (uint8_t *)ly.WcatT + (size_t)e * D * 2 * X * fs;
                M_TRY(qcopy_block(c, qsrc(ly.mat0) + (size_t)e * X * D * fs, D, X, D, (int)fs, cat, D, catT, 2 * X, 0));
                M_TRY(qcopy_block(c, qsrc(ly.mat0 + 1) + (size_t)e * X * D * fs, D, X, D, (int)fs, cat + (size_t)X * D * fs, D,
                                  catT + (size_t)X * fs, 2 * X, 0));
                M_TRY(qcopy_block(c, qsrc(ly.mat0 + 2) + (size_t)e * D * X * fs, X, D, X, (int)fs, (uint8_t *)ly.Wc + (size_t)e * D * X * fs, X,
                                  (uint8_t *)ly.WcT + (size_t)e * X * D * fs, D, 0));
            }
            M_TRY(qcopy_block(c, qsrc(ly.mat0 + 3), D, E, D, (int)fs, ly.Wsel, D, ly.WselT, m->epad, 0));
            M_TRY(fill_vector(c, ly.fwd_col, 2 * X, a, nullptr, false));
            M_TRY(fill_vector(c, ly.bwd_row_e, X, 1.f, m->mats[ly.mat0].sko, true));
            continue;
        }
        // the concatenated block [n W][D] transposes in one pass: its row blocks become the column blocks of WcatT
        M_TRY(qcopy_block(c, ly.Wcat, D, (int64_t)n * W, D, (int)fs, nullptr, 0, ly.WcatT, (int64_t)n * W, 0));
        M_TRY(qcopy_block(c, ly.Wc, W, D, W, (int)fs, nullptr, 0, ly.WcT, D, 0));
        // forward column scales: matrices followed by a normalisation (Q, V, Expand) and the gates use the unit-RMS
        // matrix q/32 (GetDataNoScale), K carries its matrix scale; dW rows of Q, K, V / Expand are divided by theirs
        M_TRY(layer_scales(c, ly.fwd_col, ly.bwd_row, W, n, ly.type == TS2_LAYER_ATT, a, m->skos + ly.mat0));
    }
    return TS2_OK;
}

// Requantisation of the whole model on this rank alone (creation, ts2_set_params): matrix scales, quantized copies
int requantize_all(ts2_model *m)
{
    Ctx c = ctx_of(m);
    M_TRY(opt_update(c, m->d_segs_full, m->nseg_full, m->nitems_full, nullptr, nullptr, nullptr, nullptr, m->w_flat, m->roww2));
    M_TRY(opt_sko(c, m->d_optmats, (int)m->mats.size(), m->roww2, m->skos));
    M_TRY(opt_quantize(c, m->d_segs_full, m->nseg_full, m->nitems_full, m->w_flat, m->skos));
    M_TRY(post_quantize(m));
    return TS2_OK;
}

int build_model(ts2_model *m, const ts2_matrix_view *mats, int n_mats, const float *bias)
{
    const ts2_model_descr &d = m->descr;
    m->D = d.dim;
    m->H = d.head_count;
    m->Q = 128 * d.head_count;
    m->F = 128 * d.ffn_tiles;
    m->V = d.output_token_count;
    m->L = d.layer_count;
    // operand format of the contractions: e4m3 with activations at 16 x their unit-rms value; fp16; int8 with activations at
    // 24 x (the reference's STATE_VEC_SCALE / FFN_VEC_SCALE / V_VEC_SCALE = 1 / 24, cfg_precision.h:72-77)
    m->ft = d.precision == TS2_PREC_FP8 ? 0 : d.precision == TS2_PREC_F16 ? 1 : 2;
    m->kind = m->ft == 0 ? KIND_E4M3 : m->ft == 1 ? KIND_F16 : KIND_I8;
    m->s_act = m->ft == 0 ? 16.f : m->ft == 1 ? 1.f : 24.f;
    m->E = d.moe_expert_count;
    m->K = d.moe_selected;
    m->X = d.expert_dim;
    m->epad = (m->E + 31) / 32 * 32;
    m->moe_rows = (m->K * m->max_nodes + 127) / 128 * 128 + 128 * m->E;
    const int D = m->D, T = m->max_nodes, L = m->L;
    const size_t fs = fast_size(m);

    std::vector<std::pair<int64_t, int64_t>> shapes;
    shapes_of(&d, &shapes);
    if ((int)shapes.size() != n_mats)
        return fail(TS2_ERR_INVALID_ARG, "expected %d matrices, got %d", (int)shapes.size(), n_mats);
    m->mats.resize(n_mats);
    std::vector<size_t> mat_off;
    layout_buckets(&d, shapes, &m->buckets, &mat_off, &m->mat_bucket);
    m->buckets[0].qsize = 2; // the embedding is always fp16 (TEmbedFloat, cfg_precision.h:62)
    for (size_t b = 1; b < m->buckets.size(); ++b)
        m->buckets[b].qsize = (int)fs;
    m->mat_grow0.assign(n_mats, 0);
    size_t params = 0;
    int rows = 0;
    for (int i = 0; i < n_mats; ++i) {
        if (!mats[i].data || mats[i].x_size != shapes[i].first || mats[i].y_size != shapes[i].second)
            return fail(TS2_ERR_INVALID_ARG, "matrix %d: expected [%lld][%lld], got [%lld][%lld]", i, (long long)shapes[i].second,
                        (long long)shapes[i].first, (long long)mats[i].y_size, (long long)mats[i].x_size);
        Matrix &mt = m->mats[i];
        mt.x = shapes[i].first;
        mt.y = shapes[i].second;
        mt.row_disp_size = (i < 2) ? (int)mt.y : 1; // per-row dispersion for embedding and final layer (model_params.cpp:150-151)
        mt.offset = mat_off[i];
        params += (size_t)mt.x * mt.y;
        m->mat_grow0[i] = rows;
        rows += (int)mt.y;
        m->max_rows = std::max(m->max_rows, mt.y);
    }
    const size_t off = m->buckets.back().off + m->buckets.back().elems;
    m->total_params = params;
    m->flat_elems = off;
    m->n_rows_total = rows;
    M_TRY(dalloc(m, &m->w_flat, off));
    M_TRY(dalloc(m, &m->avg_flat, off));
    M_TRY(dalloc(m, &m->grad_flat, off));
    M_TRY(dalloc(m, &m->skos, n_mats));
    M_TRY(dalloc(m, &m->rowsum, (size_t)rows));
    M_TRY(dalloc(m, &m->row_scale, (size_t)rows));
    M_TRY(dalloc(m, &m->roww2, (size_t)rows));
    TS2_CUDA(cudaMemsetAsync(m->w_flat, 0, off * 4, m->stream));
    TS2_CUDA(cudaMemsetAsync(m->avg_flat, 0, off * 4, m->stream));
    TS2_CUDA(cudaMemsetAsync(m->grad_flat, 0, off * 4, m->stream));
    for (Bucket &bk : m->buckets) {
        M_TRY(dalloc(m, &bk.qflat, bk.elems * bk.qsize));
        TS2_CUDA(cudaMemsetAsync(bk.qflat, 0, bk.elems * bk.qsize, m->stream));
    }
    auto qptr = [&](int mat) {
        const Bucket &bk = m->buckets[m->mat_bucket[mat]];
        return bk.qflat + (m->mats[mat].offset - bk.off) * bk.qsize;
    };
    for (int i = 0; i < n_mats; ++i) {
        Matrix &mt = m->mats[i];
        mt.w = m->w_flat + mt.offset;
        mt.avg = m->avg_flat + mt.offset;
        mt.grad = m->grad_flat + mt.offset;
        mt.sko = m->skos + i;
        M_TRY(dalloc(m, &mt.row_disp, mt.row_disp_size + 1));
        mt.sum_weight = mt.row_disp + mt.row_disp_size;
        TS2_CUDA(cudaMemsetAsync(mt.row_disp, 0, (mt.row_disp_size + 1) * 4, m->stream));
        TS2_CUDA(cudaMemcpyAsync(mt.w, mats[i].data, (size_t)mt.x * mt.y * 4, cudaMemcpyHostToDevice, m->stream));
    }
    M_TRY(dalloc(m, &m->bias, m->V));
    m->has_bias = bias != nullptr;
    if (bias)
        TS2_CUDA(cudaMemcpyAsync(m->bias, bias, (size_t)m->V * 4, cudaMemcpyHostToDevice, m->stream));
    else
        TS2_CUDA(cudaMemsetAsync(m->bias, 0, (size_t)m->V * 4, m->stream));

    // quantized weights: the row-major copies of the embedding, the final layer and the dense layers' matrices are
    // the buckets' quantized buffers themselves (the requantiser and the data-parallel all-gather write them in place)
    m->embed16 = (__half *)qptr(0);
    m->Wf = qptr(1);
    M_TRY(dalloc(m, &m->WfT16, (size_t)m->V * D));
    m->layers.resize(L);
    int mi = 2;
    int max_wide = m->Q, max_cat = 4 * m->Q;
    bool has_moe = false;
    for (int l = 0; l < L; ++l) {
        Layer &ly = m->layers[l];
        ly.type = d.layers[l].layer_type;
        ly.slope = d.layers[l].alibi_slope;
        ly.att_type = d.layers[l].attention_type_id;
        ly.mat0 = mi;
        mi += layer_matrix_count(ly.type);
        ly.wide = ly.type == TS2_LAYER_ATT ? m->Q : (ly.type == TS2_LAYER_FFN ? m->F : m->X);
        ly.ncat = ly.type == TS2_LAYER_ATT ? 4 : 2;
        if (ly.type == TS2_LAYER_MOE) {
            has_moe = true;
            const size_t E = m->E, X = m->X, R = m->moe_rows;
            // an expert sees the fraction selected / experts of the tokens: the reference scales the step of the expert
            // matrices by the square root of it (moeFraction, EnumLayerMatrices, model_dim.h:230,252-254; host_matrix.cpp:40)
            for (int j = 0; j < 3; ++j)
                m->mats[ly.mat0 + j].sparsity = (float)m->K / (float)m->E;
            M_TRY(dalloc(m, (uint8_t **)&ly.Wcat, E * 2 * X * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.WcatT, E * 2 * X * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.Wc, E * X * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.WcT, E * X * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.Wsel, (size_t)m->epad * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.WselT, (size_t)m->epad * D * fs));
            TS2_CUDA(cudaMemsetAsync(ly.Wsel, 0, (size_t)m->epad * D * fs, m->stream));
            TS2_CUDA(cudaMemsetAsync(ly.WselT, 0, (size_t)m->epad * D * fs, m->stream));
            M_TRY(dalloc(m, &ly.fwd_col, 2 * X));
            M_TRY(dalloc(m, &ly.bwd_row_e, X));
            M_TRY(dalloc(m, (uint8_t **)&ly.n_fast, (size_t)T * D * fs));
            M_TRY(dalloc(m, (uint8_t **)&ly.n_rows, R * D * fs));
            M_TRY(dalloc(m, &ly.cat16, R * 2 * X));
            M_TRY(dalloc(m, &ly.what, R * X));
            M_TRY(dalloc(m, &ly.wscale, R * (X / 128)));
            M_TRY(dalloc(m, (uint8_t **)&ly.rg, R * X * fs));
            M_TRY(dalloc(m, &ly.logits, (size_t)T * m->epad));
            M_TRY(dalloc(m, &ly.ids, (size_t)T * m->K));
            M_TRY(dalloc(m, &ly.weights, (size_t)T * m->K));
            M_TRY(dalloc(m, &ly.slot_of, (size_t)T * m->K));
            M_TRY(dalloc(m, &ly.token_of, R));
            M_TRY(dalloc(m, &ly.weight_of, R));
            M_TRY(dalloc(m, &ly.tile_group, R / 128));
            M_TRY(dalloc(m, &ly.seg_ptr, E + 1));
            continue;
        }
        max_wide = std::max(max_wide, ly.wide);
        max_cat = std::max(max_cat, ly.ncat * ly.wide);
        const size_t W = ly.wide, C = (size_t)ly.ncat * ly.wide;
        ly.Wcat = qptr(ly.mat0); // the ncat matrices are consecutive in the flat order: together they are [C][D]
        ly.Wc = qptr(ly.mat0 + ly.ncat);
        M_TRY(dalloc(m, (uint8_t **)&ly.WcatT, C * D * fs));
        M_TRY(dalloc(m, (uint8_t **)&ly.WcT, W * D * fs));
        M_TRY(dalloc(m, &ly.fwd_col, C));
        M_TRY(dalloc(m, &ly.bwd_row, C));
        M_TRY(dalloc(m, (uint8_t **)&ly.n_fast, (size_t)T * D * fs));
        M_TRY(dalloc(m, &ly.cat16, (size_t)T * C));
        M_TRY(dalloc(m, (uint8_t **)&ly.rg, (size_t)T * W * fs));
        if (ly.type == TS2_LAYER_ATT) {
            M_TRY(dalloc(m, &ly.q, (size_t)T * W));
            M_TRY(dalloc(m, &ly.k, (size_t)T * W));
            M_TRY(dalloc(m, &ly.v, (size_t)T * W));
            M_TRY(dalloc(m, &ly.o, (size_t)T * W));
            M_TRY(dalloc(m, &ly.qscale, (size_t)T * m->H));
            M_TRY(dalloc(m, &ly.vscale, (size_t)T * m->H));
            M_TRY(dalloc(m, &ly.lse, (size_t)T * m->H));
        } else {
            M_TRY(dalloc(m, &ly.wscale, (size_t)T * (W / 128)));
        }
    }
    // activations
    m->states.resize(L + 1);
    for (int l = 0; l <= L; ++l)
        M_TRY(dalloc(m, &m->states[l], (size_t)T * D));
    M_TRY(dalloc(m, &m->g, (size_t)T * D));
    M_TRY(dalloc(m, &m->dn, (size_t)T * D));
    M_TRY(dalloc(m, (uint8_t **)&m->g_fast, (size_t)T * D * fs));
    M_TRY(dalloc(m, (uint8_t **)&m->nF_fast, (size_t)T * D * fs));
    M_TRY(dalloc(m, &m->nF16, (size_t)T * D));
    // the final layer is processed in chunks of nodes so that its logits stay a few hundred MB
    {
        // Memory bound: logits of a chunk <= 512 MB of fp16.  Within it the chunk is sized so that the dX contraction of the
        // final layer ([chunk][D] from K = V, 128 x 256 tiles) is one full wave of the SMs: its time per wave is set by K,
        // so a chunk of 41 tile rows x 3 (123 of 148 SMs at dim 768) cost as much as one of 49 x 3.
        const int by_memory = std::max(128, (int)((size_t)(1u << 28) / (size_t)m->V) / 128 * 128);
        const int n_tiles = (D + 255) / 256, sms = sm_count(m->device);
        const int wave_rows = std::max(1, sms / n_tiles) * 128;
        int chunk = wave_rows;
        while (chunk + wave_rows <= by_memory * 5 / 4) // whole waves while the buffer stays within 25 % of the bound
            chunk += wave_rows;
        m->chunk = std::min(T, chunk);
    }
    M_TRY(dalloc(m, &m->logits, (size_t)m->chunk * m->V));
    size_t drg_elems = (size_t)T * max_wide, dcat_elems = (size_t)T * max_cat;
    if (has_moe) {
        const size_t R = m->moe_rows, X = m->X;
        drg_elems = std::max(drg_elems, R * X);
        dcat_elems = std::max(dcat_elems, R * 2 * X);
        M_TRY(dalloc(m, &m->moe_y, R * D));
        M_TRY(dalloc(m, (uint8_t **)&m->moe_g, R * D * fs));
        M_TRY(dalloc(m, &m->dmoe_part, R * (X / 128)));
        M_TRY(dalloc(m, (uint8_t **)&m->moe_dl, (size_t)T * m->epad * fs));
        const size_t nb = (size_t)(T + 255) / 256 * m->E;
        M_TRY(dalloc(m, &m->moe_hist, nb));
        M_TRY(dalloc(m, &m->moe_base, nb));
    }
    M_TRY(dalloc(m, &m->drg, drg_elems));
    M_TRY(dalloc(m, &m->dout, (size_t)T * m->Q));
    M_TRY(dalloc(m, (uint8_t **)&m->dcat, dcat_elems * fs));
    if (m->ft == 2) {
        M_TRY(dalloc(m, &m->g16, (size_t)T * D));
        M_TRY(dalloc(m, &m->dcat16, dcat_elems));
        M_TRY(dalloc(m, &m->x16, (size_t)T * std::max(max_wide, D)));
        M_TRY(dalloc(m, &m->g_rs, (size_t)T));
        M_TRY(dalloc(m, &m->dcat_rs, (size_t)T));
    }
    M_TRY(dalloc(m, &m->dscale, (size_t)T * m->H));
    M_TRY(dalloc(m, &m->dq, (size_t)T * m->Q));
    M_TRY(dalloc(m, &m->dk, (size_t)T * m->Q));
    M_TRY(dalloc(m, &m->dv, (size_t)T * m->Q));
    M_TRY(dalloc(m, &m->rope, (size_t)T * 128));
    M_TRY(dalloc(m, &m->absmax, L + 2));
    M_TRY(dalloc(m, &m->ginv, 4));
    m->fscale = m->ginv + 1;
    M_TRY(dalloc(m, &m->health, L + 1));
    TS2_CUDA(cudaMemsetAsync(m->health, 0, (L + 1) * 4, m->stream));
    M_TRY(dalloc(m, &m->logp_ring, ts2_model::LOSS_RING + 1)); // the last slot serves ts2_forward_score
    TS2_CUDA(cudaMemsetAsync(m->logp_ring, 0, (ts2_model::LOSS_RING + 1) * 4, m->stream));
    m->logp = m->logp_ring;
    // batch
    BatchDev &b = m->batch;
    b.label_cap = (size_t)T * 4;
    M_TRY(dalloc(m, &b.target, (size_t)T));
    const int na = std::max(1, d.attention_type_count);
    // labels, label_ptr, per attention type span_ptr + starts + finishes, target nodes + ids; each rounded up to 16 bytes
    b.raw_cap = b.label_cap + ((size_t)T + 4) + (size_t)na * 3 * ((size_t)T + 4) + 2 * ((size_t)T + 4);
    M_TRY(dalloc(m, &b.raw, b.raw_cap));
    b.label_arr = b.raw;
    b.label_ptr = b.raw;
    b.span_start.resize(na);
    b.span_finish.resize(na);
    b.rev_first.resize(na);
    b.rev_last.resize(na);
    for (int a = 0; a < na; ++a) {
        M_TRY(dalloc(m, &b.span_start[a], (size_t)T));
        M_TRY(dalloc(m, &b.span_finish[a], (size_t)T));
        M_TRY(dalloc(m, &b.rev_first[a], (size_t)T));
        M_TRY(dalloc(m, &b.rev_last[a], (size_t)T));
    }
    M_TRY(dalloc(m, &b.scan_tmp, batch_scan_tmp_elems(T)));
    M_TRY(dalloc(m, &b.status, 4));
    TS2_CUDA(cudaMemsetAsync(b.status, 0, 16, m->stream));
    for (int i = 0; i < 2; ++i) {
        M_TRY(dalloc(m, &b.ix.key[i], b.label_cap));
        M_TRY(dalloc(m, &b.ix.val[i], b.label_cap));
    }
    M_TRY(dalloc(m, &b.ix.hist, label_index_hist_elems(b.label_cap)));
    M_TRY(dalloc(m, &b.ix.partial, label_index_partial_elems(b.label_cap, D)));
    m->pinned_bytes = 2 * b.raw_cap * 4 + 16;
    TS2_CUDA(cudaMallocHost(&m->pinned, m->pinned_bytes));
    m->h_batch_status = (int *)((uint32_t *)m->pinned + 2 * b.raw_cap);
    memset(m->h_batch_status, 0, 16);
    for (int i = 0; i < 2; ++i)
        TS2_CUDA(cudaEventCreateWithFlags(&b.slot_ev[i], cudaEventDisableTiming));

    // split-K scratch: the largest request of any dW contraction of this model
    size_t ws = 0;
    for (Layer &ly : m->layers) {
        if (ly.type == TS2_LAYER_MOE)
            continue; // the grouped contractions never split K
        for (int kind : {m->kind, (int)KIND_F16}) { // the int8 pipeline runs its dW contractions in fp16
            ws = std::max(ws, gemm_workspace_bytes(m->device, kind, true, (int64_t)ly.ncat * ly.wide, D, T));
            ws = std::max(ws, gemm_workspace_bytes(m->device, kind, true, D, ly.wide, T));
        }
    }
    ws = std::max(ws, gemm_workspace_bytes(m->device, KIND_F16, true, m->V, D, m->chunk));
    ws = std::max(ws, gemm_workspace_bytes(m->device, KIND_F16, true, m->V, D, 128));
    // forward / dX contractions with few tiles (tiny models) may split as well
    ws = std::max<size_t>(ws, (size_t)sm_count(m->device) * 128 * 256 * 4 * 2);
    M_TRY(dalloc(m, (uint8_t **)&m->workspace, ws));
    m->workspace_bytes = ws;

    Ctx c = ctx_of(m);
    M_TRY(fill_rope(c, m->rope, T));
    // tables of the flat optimizer
    {
        std::vector<OptMat> om(n_mats);
        for (int i = 0; i < n_mats; ++i) {
            om[i].x = m->mats[i].x;
            om[i].y = m->mats[i].y;
            om[i].row_disp_size = m->mats[i].row_disp_size;
            om[i].grow0 = m->mat_grow0[i];
            om[i].row_disp = m->mats[i].row_disp;
            om[i].sum_weight = m->mats[i].sum_weight;
        }
        M_TRY(dalloc(m, &m->d_optmats, (size_t)n_mats));
        TS2_CUDA(cudaMemcpyAsync(m->d_optmats, om.data(), om.size() * sizeof(OptMat), cudaMemcpyHostToDevice, m->stream));
        TS2_CUDA(cudaStreamSynchronize(m->stream));
        std::vector<OptSeg> segs;
        build_segments(m, 1, 0, &segs, &m->nitems_full);
        m->nseg_full = (int)segs.size();
        M_TRY(upload_segments(m, segs, &m->d_segs_full));
        // without data parallelism this rank's parts are everything
        m->d_segs_shard = m->d_segs_full;
        m->nseg_shard = m->nseg_full;
        m->nitems_shard = m->nitems_full;
    }
    M_TRY(requantize_all(m));
    TS2_CUDA(cudaStreamSynchronize(m->stream));
    return TS2_OK;
}

// debug trace record (no-op unless enabled): checksum and non-finite count of a buffer as the stream sees it here
enum { TR_RAW = 0, TR_F32 = 1, TR_F16 = 2 };
int trace(ts2_model *m, const char *name, int layer, const void *p, size_t bytes, int kind)
{
    if (!m->trace_on || (int)m->trace_names.size() >= ts2_model::TRACE_MAX)
        return TS2_OK;
    const size_t idx = m->trace_names.size();
    m->trace_names.push_back(layer >= 0 ? std::string(name) + "[" + std::to_string(layer) + "]" : std::string(name));
    if (!m->capture_name.empty() && m->trace_names.back() == m->capture_name && bytes <= m->capture_cap) {
        TS2_CUDA(cudaMemcpyAsync(m->capture_buf, p, bytes, cudaMemcpyDeviceToDevice, m->stream));
        m->capture_bytes = bytes;
    }
    return checksum(ctx_of(m), p, bytes, kind, m->trace_dev + 4 * idx);
}
#define TRACE(name, layer, p, bytes, kind) M_TRY(trace(m, name, layer, p, bytes, kind))

// ---- forward -------------------------------------------------------------------------
int forward(ts2_model *m)
{
    Ctx c = ctx_of(m);
    const int T = m->batch.node_count, D = m->D, H = m->H;
    const BatchDev &b = m->batch;
    const size_t fsz = fast_size(m);
    m->gemm_tag = GEMM_TAG_FWD;
    M_TRY(embed_forward(c, m->embed16, m->mats[0].sko, b.label_arr, b.label_ptr, T, D, m->states[0]));
    TRACE("state", 0, m->states[0], (size_t)T * D * 4, TR_F32);
    for (int l = 0; l < m->L; ++l) {
        Layer &ly = m->layers[l];
        const int W = ly.wide, C = ly.ncat * W;
        M_TRY(tilenorm_forward(c, m->states[l], T, D, ly.n_fast, nullptr));
        TRACE("n_fast", l, ly.n_fast, (size_t)T * D * fsz, fsz == 2 ? TR_F16 : TR_RAW);
        if (ly.type == TS2_LAYER_MOE) {
            // TMoELayer::ComputeForward, layer_moe.cu:459-486, on expert-sorted rows
            const int E = m->E, K = m->K, X = m->X, rows = (K * T + 127) / 128 * 128 + 128 * E;
            const size_t fs = fast_size(m);
            Epilogue es;
            es.alpha = sqrtf(1.0f / D) / (m->s_act * 32.f); // select matrix is used without its scale
            es.out_kind = TS2_OUT_F32;
            M_TRY(gemm_tn(m, m->kind, T, m->epad, D, ly.n_fast, D, ly.Wsel, D, ly.logits, m->epad, es));
            M_TRY(moe_route(c, ly.logits, m->epad, T, E, K, ly.ids, ly.weights));
            M_TRY(moe_build_slots(c, ly.ids, ly.weights, T, K, E, rows, m->moe_hist, m->moe_base, ly.seg_ptr, ly.tile_group, ly.slot_of,
                                  ly.token_of, ly.weight_of, m->ep ? m->cnt_own : nullptr));
            // xrows: the rows this rank computes - its own (token, choice) rows, or, expert parallel, the rows of all
            // ranks for the experts it owns
            int xrows = rows;
            const int *x_token_of = ly.token_of;
            const float *x_weight_of = ly.weight_of;
            if (m->ep) {
                M_TRY(moe_gather_rows(c, ly.n_fast, ly.token_of, rows, (int)(D * fs), m->own_rows));
                M_TRY(ep_prepare(m, ly));
                xrows = ly.plan.x_rows;
                x_token_of = ly.x_token_of;
                x_weight_of = ly.x_weight_of;
                if (m->x_peer) {
                    TS2_CUDA(cudaMemcpyAsync(m->own_w, ly.weight_of, (size_t)rows * 4, cudaMemcpyDeviceToDevice, m->stream));
                    M_TRY(ep_exchange_peer(m, ly, true, ts2_model::PB_OWN_ROWS, ly.n_rows, D * fs, true));
                    M_TRY(ep_exchange_peer(m, ly, true, ts2_model::PB_OWN_W, ly.x_weight_of, 4, false, false));
                } else {
                    M_TRY(ep_exchange(m, ly, true, m->own_rows, ly.n_rows, D * fs, true));
                    M_TRY(ep_exchange(m, ly, true, ly.weight_of, ly.x_weight_of, 4, false));
                }
            } else {
                M_TRY(moe_gather_rows(c, ly.n_fast, ly.token_of, rows, (int)(D * fs), ly.n_rows));
            }
            Epilogue e1;
            e1.col_scale = ly.fwd_col;
            e1.out_kind = TS2_OUT_F16;
            // the contract matrix is [D][E*X] for the CPU path: its dot scale is sqrt(1 / (E*X))
            Epilogue e2;
            e2.alpha = sqrtf(1.0f / ((float)E * X)) / (m->s_act * 32.f);
            e2.dyn_scale = m->mats[ly.mat0 + 2].sko;
            // expert parallel, e4m3 pipeline: the results travel back as fp16 (half the bytes of the largest message).  The
            // fp16 pipeline keeps fp32: a perturbation of 1e-4 of the states flips the expert choice of borderline tokens
            // in the layers above, and that pipeline is the one held to the single-process result.
            const bool y16 = m->ep && m->ft == 0;
            e2.out_kind = y16 ? TS2_OUT_F16 : TS2_OUT_F32;
            if (xrows) {
                M_TRY(gemm_rows_grouped(m, ly, xrows, 2 * X, D, ly.n_rows, D, ly.Wcat, D, ly.cat16, 2 * X, e1));
                M_TRY(moe_act_forward(c, ly.cat16, x_token_of, x_weight_of, xrows, X, ly.what, ly.wscale, ly.rg));
                M_TRY(gemm_rows_grouped(m, ly, xrows, D, X, ly.rg, X, ly.Wc, X, m->moe_y, D, e2));
            }
            if (m->ep) {
                const size_t yb = (size_t)D * (y16 ? 2 : 4);
                if (m->x_peer)
                    M_TRY(ep_exchange_peer(m, ly, false, ts2_model::PB_MOE_Y, m->own_y, yb, false));
                else
                    M_TRY(ep_exchange(m, ly, false, m->own_y, m->moe_y, yb, false));
                if (y16)
                    M_TRY(moe_combine_half(c, (const __half *)m->own_y, ly.slot_of, T, K, D, m->states[l], m->states[l + 1]));
                else
                    M_TRY(moe_combine(c, m->own_y, ly.slot_of, T, K, D, m->states[l], m->states[l + 1]));
            } else {
                M_TRY(moe_combine(c, m->moe_y, ly.slot_of, T, K, D, m->states[l], m->states[l + 1]));
            }
            TRACE("state", l + 1, m->states[l + 1], (size_t)T * D * 4, TR_F32);
            continue;
        }
        // [Q|K|V|Gate] or [wide|gate] = n . Wcat^T * sqrt(1/D)   (MulForward, cpu_util.cpp:7-27)
        Epilogue e1;
        e1.col_scale = ly.fwd_col;
        e1.out_kind = TS2_OUT_F16;
        if (ly.type != TS2_LAYER_ATT) {
            // FFN: the contraction's epilogue normalises the wide tiles, applies the gate and writes rg itself
            // (LoLU of the reference: sigmoid(2 gate) * tilenorm(wide)); cat16 then holds [normalised wide | gate]
            e1.pair_stride = W;
            e1.col_scale = nullptr; // both matrices are used without their scale: the uniform factor rides in alpha
            e1.alpha = sqrtf(1.0f / D) / (m->s_act * 32.f);
            e1.act_out = ly.rg;
            e1.act_ld = W;
            e1.act_scale = ly.wscale;
            e1.act_mult = m->s_act;
            e1.act_kind = m->ft;
        }
        M_TRY(gemm_tn(m, m->kind, T, C, D, ly.n_fast, D, ly.Wcat, D, ly.cat16, C, e1));
        TRACE("cat16", l, ly.cat16, (size_t)T * C * 2, TR_F16);
        if (ly.type == TS2_LAYER_ATT) {
            M_TRY(att_post_forward(c, ly.cat16, m->rope, T, H, ly.q, ly.k, ly.v, ly.qscale, ly.vscale));
            TRACE("q", l, ly.q, (size_t)T * W * 2, TR_F16);
            TRACE("k", l, ly.k, (size_t)T * W * 2, TR_F16);
            TRACE("v", l, ly.v, (size_t)T * W * 2, TR_F16);
            M_TRY(attention_forward(c, ly.q, ly.k, ly.v, b.span_start[ly.att_type], b.span_finish[ly.att_type], T, H, ly.slope, ly.o, ly.lse));
            TRACE("att_o", l, ly.o, (size_t)T * W * 2, TR_F16);
            TRACE("att_lse", l, ly.lse, (size_t)T * H * 4, TR_F32);
            M_TRY(att_gate_forward(c, ly.cat16, ly.o, T, W, ly.rg));
        } else {
            TRACE("wscale", l, ly.wscale, (size_t)T * (W / 128) * 4, TR_F32);
        }
        TRACE("rg", l, ly.rg, (size_t)T * W * fsz, fsz == 2 ? TR_F16 : TR_RAW);
        // state_out = state_in + rg . Wc^T * sqrt(1/wide) with Wc = q * sko / 32
        Epilogue e2;
        e2.alpha = sqrtf(1.0f / W) / (m->s_act * 32.f);
        e2.dyn_scale = m->mats[ly.mat0 + ly.ncat].sko;
        e2.out_kind = TS2_OUT_F32_ADD;
        e2.c_in = m->states[l];
        M_TRY(gemm_tn(m, m->kind, T, D, W, ly.rg, W, ly.Wc, W, m->states[l + 1], D, e2));
        TRACE("state", l + 1, m->states[l + 1], (size_t)T * D * 4, TR_F32);
    }
    M_TRY(tilenorm_forward(c, m->states[m->L], T, D, m->nF_fast, m->nF16));
    TRACE("nF16", -1, m->nF16, (size_t)T * D * 2, TR_F16);
    return TS2_OK;
}

// logits of nodes [r0, r0+rows) -> softmax; with backward: dnF rows and the final-layer gradient
int final_layer(ts2_model *m, bool backward)
{
    Ctx c = ctx_of(m);
    const int T = m->batch.node_count, D = m->D, V = m->V;
    const size_t fs = fast_size(m);
    const float gscale = 1024.f;                           // keeps p ~ 1/V inside the fp16 normal range
    const float gs = (1.f / LOG2F) * LOG2F;                // CalcFinalLayerMult() * LOG2, cpu_transformer.cpp:159
    const bool tune_final = !(m->descr.flags & TS2_MPF_DISABLE_TUNE_FINAL_LAYER);
    m->gemm_tag = GEMM_TAG_FINAL;
    TS2_CUDA(cudaMemsetAsync(m->logp, 0, 4, m->stream));
    for (int r0 = 0; r0 < T; r0 += m->chunk) {
        const int rows = std::min(m->chunk, T - r0);
        Epilogue e;
        e.alpha = sqrtf(1.0f / D) / (m->s_act * 32.f) * (1.f / LOG2F); // MulForward scale * CalcFinalLayerMult()
        e.dyn_scale = m->mats[1].sko;
        e.out_kind = TS2_OUT_F16;
        M_TRY(gemm_tn(m, m->kind, rows, V, D, (const uint8_t *)m->nF_fast + (size_t)r0 * D * fs, D, m->Wf, D, m->logits, V, e));
        TRACE("logits", r0 / m->chunk, m->logits, (size_t)rows * V * 2, TR_F16);
        M_TRY(softmax_ce(c, m->logits, rows, V, m->has_bias ? m->bias : nullptr, m->batch.target + r0, gscale, m->logp, backward));
        if (!backward)
            continue;
        TRACE("dlogits", r0 / m->chunk, m->logits, (size_t)rows * V * 2, TR_F16);
        // dnF = g . Wf * sqrt(1/D)   (MulBackwardWithAccum, cpu_transformer.cpp:163)
        Epilogue ex;
        ex.alpha = sqrtf(1.0f / D) / 32.f * gs / gscale;
        ex.dyn_scale = m->mats[1].sko;
        ex.out_kind = TS2_OUT_F32;
        M_TRY(gemm_tn(m, KIND_F16, rows, D, V, m->logits, V, m->WfT16, V, m->dn + (size_t)r0 * D, D, ex));
        TRACE("dnF", r0 / m->chunk, m->dn + (size_t)r0 * D, (size_t)rows * D * 4, TR_F32);
        if (tune_final) {
            // dWf += g^T . nF   (SumRankOne, cpu_transformer.cpp:168)
            Epilogue ew;
            ew.alpha = gs / gscale;
            ew.out_kind = TS2_OUT_F32_ADD;
            M_TRY(gemm_dw(m, KIND_F16, V, D, rows, m->logits, V, m->nF16 + (size_t)r0 * D, D, m->mats[1].grad, ew));
        }
    }
    if (backward && tune_final)
        TRACE("dW_final", -1, m->mats[1].grad, (size_t)V * D * 4, TR_F32);
    return TS2_OK;
}

int tap_gradient(ts2_model *m, int boundary)
{
    if (!m->debug_taps)
        return TS2_OK;
    const size_t n = (size_t)m->batch.node_count * m->D;
    TS2_CUDA(cudaMemcpyAsync(m->grad_taps + (size_t)boundary * m->max_nodes * m->D, m->g, n * 4, cudaMemcpyDeviceToDevice, m->stream));
    return TS2_OK;
}

// data-parallel sum of the gradient of the bucket that starts at matrix m0, on the communication stream, ordered
// after what the main stream has queued so far; the backward pass goes on meanwhile.  Reduce-scatter: every rank
// receives the sum for the 1 / world part of the bucket it will update (in place: the part sits where it was).
// gradients of the matrices [m0, m1) (whole buckets) are complete: reduce-scatter their buckets
static int reduce_matrices(ts2_model *m, int m0, int m1)
{
    if (!m->reduce_in_backward)
        return TS2_OK;
    TS2_CUDA(cudaEventRecord(m->ev_grads, m->stream));
    TS2_CUDA(cudaStreamWaitEvent(m->comm_stream, m->ev_grads, 0));
    for (int b = m->mat_bucket[m0]; b < (int)m->buckets.size() && m->buckets[b].mat0 < m1; ++b) {
        const Bucket &bk = m->buckets[b];
        if (bk.owner_only)
            continue; // expert parallel: this rank's part is its own experts, whose gradient arose here in full
        const size_t part = bk.elems / m->world;
        M_NCCL(ncclReduceScatter(m->grad_flat + bk.off, m->grad_flat + bk.off + part * m->rank, part, ncclFloat, ncclSum, m->comm,
                                 m->comm_stream));
    }
    return TS2_OK;
}

// Backward pass of one dense layer in the int8 pipeline (the reference's default build: FWD / BWD_MATMUL_TYPE =
// MATMUL_INT8, cfg_precision.h:21-26).  Same chain as the e4m3 / fp16 pipelines with these differences:
//  * the gradient operand of each dX contraction is quantized per row to int8 with the reference's stochastic rounding
//    (NormalizeVecsRowMaxKernel, row_scale.cuh:12-43) and its row scale is applied in the contraction's epilogue
//    (Int8MatMulKernelRowScale, src/lib/cuda/cuda_i8.cuh:200-260);
//  * the dW contractions run in fp16 on the unquantized gradients and the int8 activations widened to fp16: their
//    contraction index is the token, so a per-token scale cannot leave through the epilogue; the reference sorts the
//    tokens by scale and rescales its int32 accumulator every 128 tokens (cuda_i8.cuh:264-320), which has no cheap
//    form on a TMEM accumulator; fp16 operands are more exact than that and cost the tensor rate of that third;
//  * the element-wise gradient kernels are the fp16 pipeline's.
int backward_dense_int8(ts2_model *m, int l)
{
    Ctx c = ctx_of(m), c16 = c;
    c16.ft = 1;
    const int T = m->batch.node_count, D = m->D, H = m->H;
    const BatchDev &b = m->batch;
    const bool tune_layers = !(m->descr.flags & TS2_MPF_DISABLE_TUNE_LAYERS);
    Layer &ly = m->layers[l];
    const int W = ly.wide, C = ly.ncat * W;
    Matrix &mc = m->mats[ly.mat0 + ly.ncat];
    M_TRY(rowquant_grad(c, m->g, T, D, m->absmax + l + 1, (int8_t *)m->g_fast, m->g_rs, m->g16, m->ginv, sqrtf((float)D / (float)W), mc.sko,
                        m->fscale));
    TRACE("g_fast", l, m->g_fast, (size_t)T * D, TR_RAW);
    Epilogue e3;
    e3.alpha = 1.f / (32.f * sqrtf((float)D));
    e3.row_scale = m->g_rs;
    e3.out_kind = TS2_OUT_F16;
    M_TRY(gemm_tn(m, KIND_I8, T, W, D, m->g_fast, D, ly.WcT, D, m->drg, W, e3));
    TRACE("drg", l, m->drg, (size_t)T * W * 2, TR_F16);
    if (tune_layers) {
        M_TRY(i8_to_half(c, ly.rg, (size_t)T * W, m->x16));
        Epilogue e6;
        e6.alpha = 1.f / m->s_act;
        e6.dyn_scale = m->ginv;
        e6.out_kind = TS2_OUT_F32_ADD;
        M_TRY(gemm_dw(m, KIND_F16, D, W, T, m->g16, D, m->x16, W, mc.grad, e6));
        TRACE("dW_c", l, mc.grad, (size_t)D * W * 4, TR_F32);
    }
    if (ly.type == TS2_LAYER_ATT) {
        M_TRY(att_gate_backward(c16, m->drg, ly.cat16, ly.o, T, W, m->dcat16, m->dout, m->dscale));
        M_TRY(attention_backward(c, ly.q, ly.k, ly.v, m->dout, ly.lse, m->dscale, b.span_start[ly.att_type], b.span_finish[ly.att_type],
                                 b.rev_first[ly.att_type], b.rev_last[ly.att_type], T, H, ly.slope, m->dq, m->dk, m->dv, true));
        M_TRY(att_post_backward(c16, m->dq, m->dk, m->dv, true, ly.q, ly.v, ly.qscale, ly.vscale, m->rope, m->mats[ly.mat0 + 1].sko, T, H,
                                m->dcat16));
    } else {
        M_TRY(ffn_act_backward(c16, m->drg, ly.cat16, ly.cat16, 2 * W, ly.wscale, T, W, m->dcat16));
    }
    TRACE("dcat16", l, m->dcat16, (size_t)T * C * 2, TR_F16);
    M_TRY(rowquant_half(c, m->dcat16, T, C, (int8_t *)m->dcat, m->dcat_rs));
    Epilogue e4;
    e4.alpha = sqrtf(1.0f / D) / 32.f;
    e4.row_scale = m->dcat_rs;
    e4.out_kind = TS2_OUT_F32;
    M_TRY(gemm_tn(m, KIND_I8, T, D, C, m->dcat, C, ly.WcatT, C, m->dn, D, e4));
    TRACE("dn", l, m->dn, (size_t)T * D * 4, TR_F32);
    if (tune_layers) {
        M_TRY(i8_to_half(c, ly.n_fast, (size_t)T * D, m->x16));
        Epilogue e5;
        e5.alpha = 1.f / m->s_act;
        e5.dyn_scale = m->fscale;
        e5.row_scale = ly.bwd_row;
        e5.out_kind = TS2_OUT_F32_ADD;
        M_TRY(gemm_dw(m, KIND_F16, C, D, T, m->dcat16, C, m->x16, D, m->mats[ly.mat0].grad, e5));
        TRACE("dW_cat", l, m->mats[ly.mat0].grad, (size_t)C * D * 4, TR_F32);
    }
    return TS2_OK;
}

int backward(ts2_model *m)
{
    Ctx c = ctx_of(m);
    const int T = m->batch.node_count, D = m->D, H = m->H, L = m->L;
    const BatchDev &b = m->batch;
    const bool tune_layers = !(m->descr.flags & TS2_MPF_DISABLE_TUNE_LAYERS);
    TS2_CUDA(cudaMemsetAsync(m->absmax, 0, (L + 2) * 4, m->stream));
    M_TRY(final_layer(m, true));
    m->gemm_tag = GEMM_TAG_DX;
    M_TRY(reduce_matrices(m, 1, 2));
    M_TRY(tilenorm_backward(c, m->states[L], m->dn, nullptr, 1.f, T, D, m->g, false, m->absmax + L, m->health + L, m->step_no));
    TRACE("g", L, m->g, (size_t)T * D * 4, TR_F32);
    M_TRY(tap_gradient(m, L));
    const size_t fsz = fast_size(m);
    for (int l = L - 1; l >= 0; --l) {
        Layer &ly = m->layers[l];
        const int W = ly.wide, C = ly.ncat * W;
        Matrix &mc = m->mats[ly.mat0 + ly.ncat];
        if (ly.type == TS2_LAYER_MOE) {
            // TMoELayer::ComputeBackward, layer_moe.cu:488-537, on expert-sorted rows
            const int E = m->E, K = m->K, X = m->X, rows = (K * T + 127) / 128 * 128 + 128 * E;
            const size_t fs = fast_size(m);
            if (m->ep) // rows of all ranks meet in one contraction: one power-of-two gradient scale for all of them
                M_NCCL(ncclAllReduce(m->absmax + l + 1, m->absmax + l + 1, 1, ncclUint32, ncclMax, m->comm_x, m->stream));
            M_TRY(cast_grad(c, m->g, (size_t)T * D, m->absmax + l + 1, m->g_fast, m->ginv, sqrtf((float)D / ((float)E * X)), mc.sko,
                            m->fscale));
            const int xrows = m->ep ? ly.plan.x_rows : rows;
            const int *x_token_of = m->ep ? ly.x_token_of : ly.token_of;
            const float *x_weight_of = m->ep ? ly.x_weight_of : ly.weight_of;
            if (m->ep) {
                M_TRY(moe_gather_rows(c, m->g_fast, ly.token_of, rows, (int)(D * fs), m->own_g));
                if (m->x_peer)
                    M_TRY(ep_exchange_peer(m, ly, true, ts2_model::PB_OWN_G, m->moe_g, D * fs, true));
                else
                    M_TRY(ep_exchange(m, ly, true, m->own_g, m->moe_g, D * fs, true));
            } else {
                M_TRY(moe_gather_rows(c, m->g_fast, ly.token_of, rows, (int)(D * fs), m->moe_g));
            }
            Epilogue e3;
            e3.alpha = 1.f / (32.f * sqrtf((float)D));
            e3.out_kind = TS2_OUT_F16;
            if (xrows) {
                M_TRY(gemm_rows_grouped(m, ly, xrows, X, D, m->moe_g, D, ly.WcT, D, m->drg, X, e3));
                if (tune_layers) {
                    Epilogue e6;
                    e6.alpha = 1.f / m->s_act;
                    e6.dyn_scale = m->ginv;
                    e6.out_kind = TS2_OUT_F32_ADD;
                    M_TRY(gemm_k_grouped(m, ly, D, X, xrows, m->moe_g, D, ly.rg, X, mc.grad, (int64_t)D * X, e6));
                }
                M_TRY(moe_act_backward(c, m->drg, ly.cat16, ly.what, ly.wscale, x_token_of, x_weight_of, xrows, X, m->dcat, m->dmoe_part));
            }
            const float *part_own = m->dmoe_part;
            if (m->ep) {
                if (m->x_peer)
                    M_TRY(ep_exchange_peer(m, ly, false, ts2_model::PB_PART, m->own_part, (size_t)(X / 128) * 4, false));
                else
                    M_TRY(ep_exchange(m, ly, false, m->own_part, m->dmoe_part, (size_t)(X / 128) * 4, false));
                part_own = m->own_part;
            }
            M_TRY(moe_router_backward(c, part_own, X / 128, ly.ids, ly.weights, ly.slot_of, T, K, E, m->epad, m->moe_dl));
            // router: dn = dl . Sel * sqrt(1/D) (scale-free matrix), dW_sel = dl^T . n
            Epilogue er;
            er.alpha = sqrtf(1.0f / D) / 32.f;
            er.out_kind = TS2_OUT_F32;
            M_TRY(gemm_tn(m, m->kind, T, D, m->epad, m->moe_dl, m->epad, ly.WselT, m->epad, m->dn, D, er));
            if (tune_layers) {
                Epilogue ew;
                ew.alpha = 1.f / m->s_act;
                ew.dyn_scale = m->fscale;
                ew.out_kind = TS2_OUT_F32_ADD;
                M_TRY(gemm_dw(m, m->kind, E, D, T, m->moe_dl, m->epad, ly.n_fast, D, m->mats[ly.mat0 + 3].grad, ew));
            }
            Epilogue e4;
            e4.alpha = sqrtf(1.0f / D) / 32.f;
            const bool y16 = m->ep && m->ft == 0;
            e4.out_kind = y16 ? TS2_OUT_F16 : TS2_OUT_F32;
            if (xrows)
                M_TRY(gemm_rows_grouped(m, ly, xrows, D, 2 * X, m->dcat, 2 * X, ly.WcatT, 2 * X, m->moe_y, D, e4));
            if (m->ep) {
                const size_t yb = (size_t)D * (y16 ? 2 : 4);
                if (m->x_peer)
                    M_TRY(ep_exchange_peer(m, ly, false, ts2_model::PB_MOE_Y, m->own_y, yb, false));
                else
                    M_TRY(ep_exchange(m, ly, false, m->own_y, m->moe_y, yb, false));
                if (y16)
                    M_TRY(moe_combine_half(c, (const __half *)m->own_y, ly.slot_of, T, K, D, nullptr, m->dn));
                else
                    M_TRY(moe_combine(c, m->own_y, ly.slot_of, T, K, D, nullptr, m->dn));
            } else {
                M_TRY(moe_combine(c, m->moe_y, ly.slot_of, T, K, D, nullptr, m->dn));
            }
            if (tune_layers && xrows) {
                Epilogue e5;
                e5.alpha = 1.f / m->s_act;
                e5.dyn_scale = m->fscale;
                e5.out_kind = TS2_OUT_F32_ADD;
                Epilogue e5e = e5;
                e5e.row_scale = ly.bwd_row_e; // expand is followed by a normalisation: rows divided by its matrix scale
                M_TRY(gemm_k_grouped(m, ly, X, D, xrows, m->dcat, 2 * X, ly.n_rows, D, m->mats[ly.mat0].grad, (int64_t)X * D, e5e));
                M_TRY(gemm_k_grouped(m, ly, X, D, xrows, (const uint8_t *)m->dcat + (size_t)X * fs, 2 * X, ly.n_rows, D,
                                     m->mats[ly.mat0 + 1].grad, (int64_t)X * D, e5));
            }
            M_TRY(reduce_matrices(m, ly.mat0, l + 1 < L ? m->layers[l + 1].mat0 : (int)m->mats.size()));
            M_TRY(tilenorm_backward(c, m->states[l], m->dn, m->fscale, 1.f, T, D, m->g, true, m->absmax + l, m->health + l, m->step_no));
            TRACE("g", l, m->g, (size_t)T * D * 4, TR_F32);
            M_TRY(tap_gradient(m, l));
            continue;
        }
        if (m->ft == 2) {
            M_TRY(backward_dense_int8(m, l));
        } else {
        // g_fast = g * 2^k; fscale = sqrt(D/W) * sko_c / 2^k turns the scale-free intermediate gradients
        // below into true ones
        M_TRY(cast_grad(c, m->g, (size_t)T * D, m->absmax + l + 1, m->g_fast, m->ginv, sqrtf((float)D / (float)W), mc.sko, m->fscale));
        // drg (scale-free) = g_fast . (q_c/32) / sqrt(D): the true value is drg * fscale
        // (MulBackwardWithAccum with the contract / combiner matrix)
        Epilogue e3;
        e3.alpha = 1.f / (32.f * sqrtf((float)D));
        e3.out_kind = TS2_OUT_F16;
        TRACE("g_fast", l, m->g_fast, (size_t)T * D * fsz, fsz == 2 ? TR_F16 : TR_RAW);
        M_TRY(gemm_tn(m, m->kind, T, W, D, m->g_fast, D, ly.WcT, D, m->drg, W, e3));
        TRACE("drg", l, m->drg, (size_t)T * W * 2, TR_F16);
        if (tune_layers) {
            // dWc = g^T . rg   (SumRankOne)
            Epilogue e6;
            e6.alpha = 1.f / m->s_act;
            e6.dyn_scale = m->ginv;
            e6.out_kind = TS2_OUT_F32_ADD;
            M_TRY(gemm_dw(m, m->kind, D, W, T, m->g_fast, D, ly.rg, W, mc.grad, e6));
            TRACE("dW_c", l, mc.grad, (size_t)D * W * 4, TR_F32);
        }
        if (ly.type == TS2_LAYER_ATT) {
            M_TRY(att_gate_backward(c, m->drg, ly.cat16, ly.o, T, W, m->dcat, m->dout, m->dscale));
            TRACE("dout", l, m->dout, (size_t)T * W * 2, TR_F16);
            TRACE("dscale", l, m->dscale, (size_t)T * H * 4, TR_F32);
            M_TRY(attention_backward(c, ly.q, ly.k, ly.v, m->dout, ly.lse, m->dscale, b.span_start[ly.att_type], b.span_finish[ly.att_type],
                                     b.rev_first[ly.att_type], b.rev_last[ly.att_type], T, H, ly.slope, m->dq, m->dk, m->dv, true));
            TRACE("dq", l, m->dq, (size_t)T * W * 2, TR_F16);
            TRACE("dk", l, m->dk, (size_t)T * W * 2, TR_F16);
            TRACE("dv", l, m->dv, (size_t)T * W * 2, TR_F16);
            M_TRY(att_post_backward(c, m->dq, m->dk, m->dv, true, ly.q, ly.v, ly.qscale, ly.vscale, m->rope, m->mats[ly.mat0 + 1].sko, T, H,
                                    m->dcat));
        } else {
            M_TRY(ffn_act_backward(c, m->drg, ly.cat16, ly.cat16, 2 * W, ly.wscale, T, W, m->dcat));
        }
        TRACE("dcat", l, m->dcat, (size_t)T * C * fsz, fsz == 2 ? TR_F16 : TR_RAW);
        // dn (scale-free) = dcat . (q_cat/32) * sqrt(1/D)
        Epilogue e4;
        e4.alpha = sqrtf(1.0f / D) / 32.f;
        e4.out_kind = TS2_OUT_F32;
        M_TRY(gemm_tn(m, m->kind, T, D, C, m->dcat, C, ly.WcatT, C, m->dn, D, e4));
        TRACE("dn", l, m->dn, (size_t)T * D * 4, TR_F32);
        if (tune_layers) {
            // dWcat = dcat^T . n * fscale, rows of matrices that are followed by a normalisation divided by sko
            Epilogue e5;
            e5.alpha = 1.f / m->s_act;
            e5.dyn_scale = m->fscale;
            e5.row_scale = ly.bwd_row;
            e5.out_kind = TS2_OUT_F32_ADD;
            M_TRY(gemm_dw(m, m->kind, C, D, T, m->dcat, C, ly.n_fast, D, m->mats[ly.mat0].grad, e5));
            TRACE("dW_cat", l, m->mats[ly.mat0].grad, (size_t)C * D * 4, TR_F32);
        }
        }
        M_TRY(reduce_matrices(m, ly.mat0, l + 1 < L ? m->layers[l + 1].mat0 : (int)m->mats.size()));
        M_TRY(tilenorm_backward(c, m->states[l], m->dn, m->fscale, 1.f, T, D, m->g, true, m->absmax + l, m->health + l, m->step_no));
        TRACE("g", l, m->g, (size_t)T * D * 4, TR_F32);
        M_TRY(tap_gradient(m, l));
    }
    if (!(m->descr.flags & TS2_MPF_DISABLE_TUNE_EMBED))
        if (!m->batch.ix_sorted) {
            M_TRY(label_index_sort(c, (uint32_t)m->descr.label_count, m->batch.ix));
            m->batch.ix_sorted = true;
        }
        M_TRY(embed_backward_indexed(c, m->g, b.ix, D, m->mats[0].grad));
    M_TRY(reduce_matrices(m, 0, 1));
    return TS2_OK;
}

// Optimizer + requantisation of this rank's parts (everything without data parallelism).  Per-row sums of squares
// of gradient and weights go to vectors over all rows of all matrices; with data parallelism those vectors are summed
// over the ranks (1 MB and 2 MB), which completes the rows a part boundary cuts and gives every rank the matrix-level
// sums; the quantized bytes are then all-gathered (a quarter of the fp32 bytes an all-reduce design moves twice).
int apply(ts2_model *m, const ts2_training_step *step)
{
    Ctx c = ctx_of(m);
    const bool dp = m->comm && m->world > 1;
    const int n_mats = (int)m->mats.size();
    if (dp) {
        if (!m->reduce_in_backward) { // gradients accumulated by calls that did not apply: exchange them now
            m->reduce_in_backward = true;
            for (const Bucket &bk : m->buckets)
                M_TRY(reduce_matrices(m, bk.mat0, bk.mat1));
            m->reduce_in_backward = false;
        }
        TS2_CUDA(cudaEventRecord(m->ev_reduced, m->comm_stream));
        TS2_CUDA(cudaStreamWaitEvent(m->stream, m->ev_reduced, 0));
        TS2_CUDA(cudaMemsetAsync(m->rowsum, 0, (size_t)m->n_rows_total * 4, m->stream));
        TS2_CUDA(cudaMemsetAsync(m->roww2, 0, (size_t)m->n_rows_total * 8, m->stream));
    }
    M_TRY(opt_row_sum2(c, m->d_segs_shard, m->nseg_shard, m->nitems_shard, m->grad_flat, m->rowsum));
    if (dp)
        M_NCCL(ncclAllReduce(m->rowsum, m->rowsum, (size_t)m->n_rows_total, ncclFloat, ncclSum, m->comm, m->stream));
    M_TRY(opt_disp(c, m->d_optmats, n_mats, m->rowsum, step->disp_decay, m->row_scale));
    M_TRY(opt_update(c, m->d_segs_shard, m->nseg_shard, m->nitems_shard, m->grad_flat, m->row_scale, step, m->avg_flat, m->w_flat,
                     m->roww2));
    if (dp)
        M_NCCL(ncclAllReduce(m->roww2, m->roww2, (size_t)m->n_rows_total, ncclDouble, ncclSum, m->comm, m->stream));
    M_TRY(opt_sko(c, m->d_optmats, n_mats, m->roww2, m->skos));
    M_TRY(opt_quantize(c, m->d_segs_shard, m->nseg_shard, m->nitems_shard, m->w_flat, m->skos));
    if (dp) {
        M_NCCL(ncclGroupStart());
        for (const Bucket &bk : m->buckets) {
            if (bk.owner_only)
                continue; // a rank only reads the quantized weights of its own experts
            const size_t part = bk.elems / m->world * bk.qsize;
            ncclResult_t r = ncclAllGather(bk.qflat + part * m->rank, bk.qflat, part, ncclUint8, m->comm, m->stream);
            if (r != ncclSuccess) {
                ncclGroupEnd();
                return mfail(m, fail(TS2_ERR_COMM, "ncclAllGather failed: %s", ncclGetErrorString(r)));
            }
        }
        M_NCCL(ncclGroupEnd());
        m->master_stale = true;
    }
    M_TRY(post_quantize(m));
    return TS2_OK;
}

// data parallel: brings the fp32 weights and momentum of the other ranks' parts up to date (all ranks must call)
int sync_master(ts2_model *m)
{
    if (!m->master_stale)
        return TS2_OK;
    M_NCCL(ncclGroupStart());
    for (const Bucket &bk : m->buckets) {
        const size_t part = bk.elems / m->world;
        for (float *flat : {m->w_flat, m->avg_flat}) {
            ncclResult_t r = ncclAllGather(flat + bk.off + part * m->rank, flat + bk.off, part, ncclFloat, m->comm, m->stream);
            if (r != ncclSuccess) {
                ncclGroupEnd();
                return mfail(m, fail(TS2_ERR_COMM, "ncclAllGather failed: %s", ncclGetErrorString(r)));
            }
        }
    }
    M_NCCL(ncclGroupEnd());
    m->master_stale = false;
    return TS2_OK;
}

// ts2_set_batch: the raw CSR arrays of the batch go to the device in one copy; the per-node tables are derived and
// every element is validated there (kernels_batch.cu).  The host checks only what it can without a loop over the batch.
int stage_batch(ts2_model *m, const ts2_batch_nodes *nd)
{
    const int T = nd->node_count;
    if (T <= 0 || T > m->max_nodes)
        return fail(T > m->max_nodes ? TS2_ERR_TOO_LARGE : TS2_ERR_INVALID_ARG, "node_count %d outside (0, %d]", T, m->max_nodes);
    if (!nd->label_ptr || (nd->label_ptr[T] && !nd->label_arr))
        return fail(TS2_ERR_INVALID_ARG, "null label arrays");
    const size_t n_labels = nd->label_ptr[T];
    BatchDev &b = m->batch;
    if (n_labels > b.label_cap)
        return fail(TS2_ERR_TOO_LARGE, "%zu labels exceed the capacity %zu", n_labels, b.label_cap);
    const int na = m->descr.attention_type_count;
    if (nd->attention_type_count < na)
        return fail(TS2_ERR_INVALID_ARG, "batch has %d attention types, the model needs %d", nd->attention_type_count, na);
    const int n_targets = nd->target_count;
    if (n_targets < 0 || (n_targets && (!nd->target_node || !nd->target_id)))
        return fail(TS2_ERR_INVALID_ARG, "bad target arrays");
    if (n_targets > T)
        return fail(TS2_ERR_UNSUPPORTED, "%d targets for %d nodes: at most one target per node is supported", n_targets, T);
    for (int a = 0; a < na; ++a) {
        const ts2_attention_info &ai = nd->att[a];
        if (!ai.span_ptr)
            return fail(TS2_ERR_INVALID_ARG, "attention type %d: null span_ptr", a);
        const int n_spans = ai.span_ptr[T];
        if (n_spans < 0 || (n_spans && (!ai.span_start || !ai.span_finish)))
            return fail(TS2_ERR_INVALID_ARG, "attention type %d: bad span arrays", a);
        if (n_spans > T)
            return fail(TS2_ERR_UNSUPPORTED, "attention type %d: %d spans for %d nodes; at most one span per node is supported", a,
                        n_spans, T);
    }
    const int slot = b.next_slot;
    b.next_slot ^= 1;
    if (b.slot_used[slot])
        TS2_CUDA(cudaEventSynchronize(b.slot_ev[slot])); // the copy that last read this slot
    uint32_t *h = (uint32_t *)m->pinned + (size_t)slot * b.raw_cap;
    size_t used = 0;
    auto put = [&](const void *src, size_t n) {
        const size_t at = used;
        if (n)
            memcpy(h + at, src, n * 4);
        used += (n + 3) & ~(size_t)3;
        return at;
    };
    const size_t o_labels = put(nd->label_arr, n_labels), o_label_ptr = put(nd->label_ptr, (size_t)T + 1);
    std::vector<size_t> o_ptr(na), o_start(na), o_finish(na);
    std::vector<int> n_spans(na);
    for (int a = 0; a < na; ++a) {
        const ts2_attention_info &ai = nd->att[a];
        n_spans[a] = ai.span_ptr[T];
        o_ptr[a] = put(ai.span_ptr, (size_t)T + 1);
        o_start[a] = put(ai.span_start, n_spans[a]);
        o_finish[a] = put(ai.span_finish, n_spans[a]);
    }
    const size_t o_tnode = put(nd->target_node, n_targets), o_tid = put(nd->target_id, n_targets);
    cudaStream_t s = m->stream;
    TS2_CUDA(cudaMemcpyAsync(b.raw, h, used * 4, cudaMemcpyHostToDevice, s));
    TS2_CUDA(cudaEventRecord(b.slot_ev[slot], s));
    b.slot_used[slot] = true;
    Ctx c = ctx_of(m);
    b.label_arr = b.raw + o_labels;
    b.label_ptr = b.raw + o_label_ptr;
    b.n_labels = (uint32_t)n_labels;
    b.ix_sorted = false;
    M_TRY(label_index_entries(c, b.label_arr, b.label_ptr, T, b.n_labels, (uint32_t)m->descr.label_count, b.ix, b.status));
    for (int a = 0; a < na; ++a)
        M_TRY(batch_span_tables(c, (const int *)b.raw + o_ptr[a], (const int *)b.raw + o_start[a], (const int *)b.raw + o_finish[a], T,
                                n_spans[a], b.span_start[a], b.span_finish[a], b.scan_tmp, b.rev_first[a], b.rev_last[a], b.status));
    M_TRY(batch_targets(c, (const int *)b.raw + o_tnode, (const int *)b.raw + o_tid, n_targets, T, m->V, b.target, b.status));
    TS2_CUDA(cudaMemcpyAsync(m->h_batch_status, b.status, 16, cudaMemcpyDeviceToHost, s));
    b.node_count = T;
    b.target_count = n_targets;
    return TS2_OK;
}

// what the device found wrong with a batch, if anything; clears the record
int report_batch_status(ts2_model *m)
{
    int *h = m->h_batch_status;
    if (!h || h[0] == BATCH_OK)
        return TS2_OK;
    const int code = h[0], where = h[1], d0 = h[2], d1 = h[3];
    h[0] = BATCH_OK;
    cudaMemsetAsync(m->batch.status, 0, 16, m->stream);
    switch (code) {
    case BATCH_BAD_SPAN_PTR:
        return fail(TS2_ERR_INVALID_ARG, "batch: span_ptr of node %d is malformed (offset %d, count %d)", where, d0, d1);
    case BATCH_MULTI_SPAN:
        return fail(TS2_ERR_UNSUPPORTED, "batch: node %d has %d attention spans; at most one is supported", where, d0);
    case BATCH_BAD_SPAN:
        return fail(TS2_ERR_INVALID_ARG, "batch: node %d: span [%d, %d] out of range", where, d0, d1);
    case BATCH_BAD_TARGET:
        return fail(TS2_ERR_INVALID_ARG, "batch: target %d: node %d / id %d out of range", where, d0, d1);
    case BATCH_DUP_TARGET:
        return fail(TS2_ERR_UNSUPPORTED, "batch: node %d has more than one target", where);
    case BATCH_BAD_LABEL_PTR:
        return fail(TS2_ERR_INVALID_ARG, "batch: label_ptr of node %d is malformed (%d, %d)", where, d0, d1);
    case BATCH_BAD_LABEL:
        return fail(TS2_ERR_INVALID_ARG, "batch: label %d (entry %d, node %d) out of range", d0, where, d1);
    }
    return fail(TS2_ERR_INVALID_ARG, "batch: malformed (code %d)", code);
}

int wait_stream(ts2_model *m)
{
    // bounded wait: poll the stream for up to 120 s of wall time, then report a timeout
    cudaError_t e;
    const auto t0 = std::chrono::steady_clock::now();
    while ((e = cudaStreamQuery(m->stream)) == cudaErrorNotReady) {
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > 120.0)
            return fail(TS2_ERR_TIMEOUT, "the device did not finish within 120 s");
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > 0.002)
            std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (e != cudaSuccess)
        return fail(TS2_ERR_CUDA, "stream failed: %s", cudaGetErrorString(e));
    M_TRY(collect_device_status(m->device));
    return report_batch_status(m);
}

} // namespace

// ---------------------------------------------------------------------------------------
extern "C" {

int ts2_matrix_count(const ts2_model_descr *descr)
{
    int rc = validate(descr);
    if (rc != TS2_OK)
        return rc;
    std::vector<std::pair<int64_t, int64_t>> s;
    shapes_of(descr, &s);
    return (int)s.size();
}

int ts2_matrix_shape(const ts2_model_descr *descr, int index, int64_t *x_size, int64_t *y_size)
{
    int rc = validate(descr);
    if (rc != TS2_OK)
        return rc;
    std::vector<std::pair<int64_t, int64_t>> s;
    shapes_of(descr, &s);
    if (index < 0 || index >= (int)s.size() || !x_size || !y_size)
        return fail(TS2_ERR_INVALID_ARG, "matrix index %d out of range", index);
    *x_size = s[index].first;
    *y_size = s[index].second;
    return TS2_OK;
}

int ts2_create(const ts2_model_descr *descr, const ts2_matrix_view *mats, int n_mats, const float *bias, int device, int max_nodes,
               ts2_model **out)
{
    if (!out)
        return fail(TS2_ERR_INVALID_ARG, "null out pointer");
    *out = nullptr;
    int rc = validate(descr);
    if (rc != TS2_OK)
        return rc;
    if (!mats || max_nodes <= 0)
        return fail(TS2_ERR_INVALID_ARG, "null matrices or max_nodes <= 0");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        return fail(TS2_ERR_NO_DEVICE, "no CUDA device: this library has no CPU fallback");
    if (device < 0 || device >= n_dev)
        return fail(TS2_ERR_INVALID_ARG, "device %d out of range (%d devices)", device, n_dev);
    cudaDeviceProp prop;
    TS2_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(TS2_ERR_NO_DEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only", device, prop.major, prop.minor);
    TS2_CUDA(cudaSetDevice(device));
    ts2_model *m = new ts2_model();
    m->descr = *descr;
    m->layer_params.assign(descr->layers, descr->layers + descr->layer_count);
    m->descr.layers = m->layer_params.data();
    m->device = device;
    m->max_nodes = (max_nodes + 127) / 128 * 128;
    cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
    cudaStreamCreateWithFlags(&m->comm_stream, cudaStreamNonBlocking);
    cudaEventCreate(&m->ev_start);
    cudaEventCreate(&m->ev_stop);
    cudaEventCreate(&m->ev_t0);
    cudaEventCreate(&m->ev_t1);
    cudaEventCreateWithFlags(&m->ev_grads, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&m->ev_reduced, cudaEventDisableTiming);
    rc = build_model(m, mats, n_mats, bias);
    if (rc != TS2_OK) {
        ts2_destroy(m);
        return rc;
    }
    *out = m;
    return TS2_OK;
}

void ts2_destroy(ts2_model *m)
{
    if (!m)
        return;
    cudaSetDevice(m->device);
    cudaDeviceSynchronize();
    if (m->x_peer && m->comm_x) {
        // other ranks may still be reading this rank's exchange buffers: meet them once more before anything is freed
        // (bounded: a rank that is gone must not keep this one here)
        if (ncclAllReduce(m->x_flag, m->x_flag, 1, ncclInt32, ncclMax, m->comm_x, m->stream) == ncclSuccess) {
            const auto t0 = std::chrono::steady_clock::now();
            while (cudaStreamQuery(m->stream) == cudaErrorNotReady &&
                   std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < 10.0)
                std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
    }
    for (void *p : m->ipc_opened)
        cudaIpcCloseMemHandle(p);
    if (m->comm_x)
        ncclCommDestroy(m->comm_x);
    if (m->comm)
        ncclCommDestroy(m->comm);
    if (m->h_cnt)
        cudaFreeHost(m->h_cnt);
    for (auto &e : m->x_events) {
        cudaEventDestroy(e.first);
        cudaEventDestroy(e.second);
    }
    for (void *p : m->allocs)
        cudaFree(p);
    if (m->pinned)
        cudaFreeHost(m->pinned);
    for (cudaEvent_t e : m->batch.slot_ev)
        if (e)
            cudaEventDestroy(e);
    if (m->ev_start)
        cudaEventDestroy(m->ev_start);
    if (m->ev_stop)
        cudaEventDestroy(m->ev_stop);
    if (m->ev_t0)
        cudaEventDestroy(m->ev_t0);
    if (m->ev_t1)
        cudaEventDestroy(m->ev_t1);
    if (m->ev_grads)
        cudaEventDestroy(m->ev_grads);
    if (m->ev_reduced)
        cudaEventDestroy(m->ev_reduced);
    if (m->stream)
        cudaStreamDestroy(m->stream);
    if (m->comm_stream)
        cudaStreamDestroy(m->comm_stream);
    delete m;
}

const char *ts2_last_error(const ts2_model *m)
{
    if (m && !m->error.empty())
        return m->error.c_str();
    return global_error();
}

int ts2_set_batch(ts2_model *m, const ts2_batch_nodes *nodes)
{
    if (!m || !nodes)
        return fail(TS2_ERR_INVALID_ARG, "null argument");
    TS2_CUDA(cudaSetDevice(m->device));
    // the staging buffer is reused: the previous copy must have left it
    M_TRY(wait_stream(m));
    M_TRY(stage_batch(m, nodes));
    return TS2_OK;
}

int ts2_backprop(ts2_model *m, const ts2_training_step *step, int add_to_model)
{
    if (!m || !step)
        return fail(TS2_ERR_INVALID_ARG, "null argument");
    if (m->batch.node_count <= 0)
        return mfail(m, fail(TS2_ERR_INVALID_ARG, "ts2_backprop before ts2_set_batch"));
    TS2_CUDA(cudaSetDevice(m->device));
    TS2_CUDA(cudaEventRecord(m->ev_start, m->stream));
    ++m->step_no;
    m->logp = m->logp_ring + m->step_no % ts2_model::LOSS_RING; // final_layer() clears and fills this step's slot
    m->ring_targets[m->step_no % ts2_model::LOSS_RING] = m->batch.target_count;
    if (m->trace_on) {
        m->trace_names.clear();
        TS2_CUDA(cudaMemsetAsync(m->trace_dev, 0, (size_t)ts2_model::TRACE_MAX * 32, m->stream));
    }
    if (!m->grads_dirty)
        TS2_CUDA(cudaMemsetAsync(m->grad_flat, 0, m->flat_elems * 4, m->stream));
    M_TRY(forward(m));
    // an accumulated gradient of earlier calls sits in the same buffer: the per-layer sums below then cover it too
    m->reduce_in_backward = add_to_model == TS2_GRADIENT_APPLY && m->comm && m->world > 1;
    const int brc = backward(m);
    m->reduce_in_backward = false;
    if (brc != TS2_OK)
        return brc;
    m->grads_dirty = true;
    m->last_targets = m->batch.target_count;
    if (add_to_model == TS2_GRADIENT_APPLY) {
        m->reduce_in_backward = m->comm && m->world > 1; // tells apply() that the exchanges are already queued
        const int arc = apply(m, step);
        m->reduce_in_backward = false;
        if (arc != TS2_OK)
            return arc;
        m->grads_dirty = false;
    }
    TS2_CUDA(cudaEventRecord(m->ev_stop, m->stream));
    m->timing_valid = true;
    return TS2_OK;
}

int ts2_wait(ts2_model *m)
{
    if (!m)
        return fail(TS2_ERR_INVALID_ARG, "null model");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    return TS2_OK;
}

int ts2_forward_score(ts2_model *m, float *out_score)
{
    if (!m || !out_score)
        return fail(TS2_ERR_INVALID_ARG, "null argument");
    if (m->batch.node_count <= 0)
        return mfail(m, fail(TS2_ERR_INVALID_ARG, "ts2_forward_score before ts2_set_batch"));
    TS2_CUDA(cudaSetDevice(m->device));
    const bool tr = m->trace_on;
    m->trace_on = false;
    float *const step_slot = m->logp;
    m->logp = m->logp_ring + ts2_model::LOSS_RING; // the last training step's slot stays readable
    int rc = forward(m);
    if (rc == TS2_OK)
        rc = final_layer(m, false);
    float *const score_slot = m->logp;
    m->logp = step_slot;
    m->trace_on = tr;
    if (rc != TS2_OK)
        return rc;
    M_TRY(wait_stream(m));
    float s = 0;
    TS2_CUDA(cudaMemcpy(&s, score_slot, 4, cudaMemcpyDeviceToHost));
    *out_score = m->batch.target_count ? s / m->batch.target_count : 0.f;
    return TS2_OK;
}

int ts2_avg_train_err(ts2_model *m, float *out_err)
{
    if (!m || !out_err)
        return fail(TS2_ERR_INVALID_ARG, "null argument");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    float s = 0;
    TS2_CUDA(cudaMemcpy(&s, m->logp, 4, cudaMemcpyDeviceToHost));
    *out_err = m->last_targets ? -s / m->last_targets : 0.f;
    return TS2_OK;
}

int ts2_get_params(ts2_model *m, int what, ts2_matrix_view *mats_out, int n_mats)
{
    if (!m || !mats_out || n_mats != (int)m->mats.size())
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_get_params");
    TS2_CUDA(cudaSetDevice(m->device));
    if (what != TS2_PARAM_GRADIENT)
        M_TRY(sync_master(m));
    M_TRY(wait_stream(m));
    for (int i = 0; i < n_mats; ++i) {
        Matrix &mt = m->mats[i];
        if (!mats_out[i].data)
            continue;
        if (mats_out[i].x_size != mt.x || mats_out[i].y_size != mt.y)
            return mfail(m, fail(TS2_ERR_INVALID_ARG, "matrix %d: shape mismatch", i));
        const float *src = what == TS2_PARAM_WEIGHTS ? mt.w : what == TS2_PARAM_MOMENTUM ? mt.avg : mt.grad;
        TS2_CUDA(cudaMemcpy(mats_out[i].data, src, (size_t)mt.x * mt.y * 4, cudaMemcpyDeviceToHost));
    }
    return TS2_OK;
}

int ts2_set_params(ts2_model *m, int what, const ts2_matrix_view *mats, int n_mats)
{
    if (!m || !mats || n_mats != (int)m->mats.size() || what == TS2_PARAM_GRADIENT)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_set_params");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(sync_master(m)); // a partial update must land on current values
    M_TRY(wait_stream(m));
    for (int i = 0; i < n_mats; ++i) {
        Matrix &mt = m->mats[i];
        if (!mats[i].data)
            continue;
        if (mats[i].x_size != mt.x || mats[i].y_size != mt.y)
            return mfail(m, fail(TS2_ERR_INVALID_ARG, "matrix %d: shape mismatch", i));
        TS2_CUDA(cudaMemcpy(what == TS2_PARAM_WEIGHTS ? mt.w : mt.avg, mats[i].data, (size_t)mt.x * mt.y * 4, cudaMemcpyHostToDevice));
    }
    if (what == TS2_PARAM_WEIGHTS) {
        M_TRY(requantize_all(m));
        M_TRY(wait_stream(m));
    }
    return TS2_OK;
}

int ts2_get_batch_tables(ts2_model *m, int attention_type, int32_t *span_start, int32_t *span_finish, int32_t *rev_first,
                         int32_t *rev_last, int32_t *target)
{
    if (!m)
        return TS2_ERR_INVALID_ARG;
    const BatchDev &b = m->batch;
    if (b.node_count <= 0)
        return fail(TS2_ERR_INVALID_ARG, "no batch was set");
    if (attention_type < 0 || attention_type >= (int)b.span_start.size())
        return fail(TS2_ERR_INVALID_ARG, "attention type %d out of range", attention_type);
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    const size_t bytes = (size_t)b.node_count * 4;
    const int a = attention_type;
    const std::pair<int32_t *, const int *> out[] = {{span_start, b.span_start[a]}, {span_finish, b.span_finish[a]},
                                                     {rev_first, b.rev_first[a]},   {rev_last, b.rev_last[a]},
                                                     {target, b.target}};
    for (const auto &o : out)
        if (o.first)
            TS2_CUDA(cudaMemcpy(o.first, o.second, bytes, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_get_label_index(ts2_model *m, uint32_t *labels, uint32_t *nodes, int64_t capacity, int64_t *count)
{
    if (!m || !count)
        return TS2_ERR_INVALID_ARG;
    BatchDev &b = m->batch;
    if (b.node_count <= 0)
        return fail(TS2_ERR_INVALID_ARG, "no batch was set");
    *count = b.n_labels;
    if ((int64_t)b.n_labels > capacity || (b.n_labels && (!labels || !nodes)))
        return fail(TS2_ERR_TOO_LARGE, "%u entries, capacity %lld", b.n_labels, (long long)capacity);
    TS2_CUDA(cudaSetDevice(m->device));
    if (!b.ix_sorted) {
        M_TRY(label_index_sort(ctx_of(m), (uint32_t)m->descr.label_count, b.ix));
        b.ix_sorted = true;
    }
    M_TRY(wait_stream(m));
    if (b.n_labels) {
        TS2_CUDA(cudaMemcpy(labels, b.ix.key[b.ix.sorted], (size_t)b.n_labels * 4, cudaMemcpyDeviceToHost));
        TS2_CUDA(cudaMemcpy(nodes, b.ix.val[b.ix.sorted], (size_t)b.n_labels * 4, cudaMemcpyDeviceToHost));
    }
    return TS2_OK;
}

int ts2_get_row_disp(ts2_model *m, int index, float *row_disp, int64_t n, float *sum_weight)
{
    if (!m || index < 0 || index >= (int)m->mats.size())
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_get_row_disp");
    Matrix &mt = m->mats[index];
    if (n != mt.row_disp_size)
        return fail(TS2_ERR_INVALID_ARG, "matrix %d has %d dispersion entries, caller passed %lld", index, mt.row_disp_size, (long long)n);
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    if (row_disp)
        TS2_CUDA(cudaMemcpy(row_disp, mt.row_disp, (size_t)n * 4, cudaMemcpyDeviceToHost));
    if (sum_weight)
        TS2_CUDA(cudaMemcpy(sum_weight, mt.sum_weight, 4, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_set_row_disp(ts2_model *m, int index, const float *row_disp, int64_t n, float sum_weight)
{
    if (!m || index < 0 || index >= (int)m->mats.size() || !row_disp)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_set_row_disp");
    Matrix &mt = m->mats[index];
    if (n != mt.row_disp_size)
        return fail(TS2_ERR_INVALID_ARG, "matrix %d has %d dispersion entries, caller passed %lld", index, mt.row_disp_size, (long long)n);
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    TS2_CUDA(cudaMemcpy(mt.row_disp, row_disp, (size_t)n * 4, cudaMemcpyHostToDevice));
    TS2_CUDA(cudaMemcpy(mt.sum_weight, &sum_weight, 4, cudaMemcpyHostToDevice));
    return TS2_OK;
}

int ts2_get_fast_weights(ts2_model *m, int index, void *dst, int64_t dst_bytes, float *matrix_scale)
{
    if (!m || index < 0 || index >= (int)m->mats.size() || !dst)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_get_fast_weights");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    Matrix &mt = m->mats[index];
    const void *src = nullptr;
    size_t es = fast_size(m);
    if (index == 0) {
        src = m->embed16;
        es = 2;
    } else if (index == 1) {
        src = m->Wf;
    } else {
        for (Layer &ly : m->layers) {
            const int j = index - ly.mat0;
            if (ly.type == TS2_LAYER_MOE || j < 0 || j > ly.ncat)
                continue; // expert matrices are stored per expert, not in matrix order
            src = j < ly.ncat ? (const void *)((const uint8_t *)ly.Wcat + (size_t)j * ly.wide * m->D * es) : ly.Wc;
            break;
        }
    }
    const size_t bytes = (size_t)mt.x * mt.y * es;
    if (!src || dst_bytes < (int64_t)bytes)
        return fail(TS2_ERR_INVALID_ARG, "ts2_get_fast_weights: need %zu bytes", bytes);
    TS2_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    if (matrix_scale)
        TS2_CUDA(cudaMemcpy(matrix_scale, mt.sko, 4, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_set_debug_taps(ts2_model *m, int enable)
{
    if (!m)
        return fail(TS2_ERR_INVALID_ARG, "null model");
    TS2_CUDA(cudaSetDevice(m->device));
    if (enable && !m->grad_taps)
        M_TRY(dalloc(m, &m->grad_taps, (size_t)(m->L + 1) * m->max_nodes * m->D));
    m->debug_taps = enable != 0;
    return TS2_OK;
}

int ts2_get_state_tap(ts2_model *m, int layer, int gradient, float *dst, int64_t n_floats)
{
    if (!m || !dst || layer < 0 || layer > m->L)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_get_state_tap");
    const size_t n = (size_t)m->batch.node_count * m->D;
    if ((size_t)n_floats < n)
        return fail(TS2_ERR_INVALID_ARG, "tap needs %zu floats", n);
    if (gradient && !m->grad_taps)
        return fail(TS2_ERR_INVALID_ARG, "gradient taps were not enabled before the step");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    const float *src = gradient ? m->grad_taps + (size_t)layer * m->max_nodes * m->D : m->states[layer];
    TS2_CUDA(cudaMemcpy(dst, src, n * 4, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_debug_read(ts2_model *m, const char *name, int layer, void *dst, int64_t bytes)
{
    if (!m || !name || !dst || layer < 0 || layer >= m->L)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_debug_read");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    const Layer &ly = m->layers[layer];
    const std::string n = name;
    const void *src = n == "rg" ? ly.rg : n == "dcat" ? m->dcat : n == "token_of" ? (const void *)ly.token_of
                      : n == "seg_ptr" ? (const void *)ly.seg_ptr : n == "slot_of" ? (const void *)ly.slot_of
                      : n == "ids" ? (const void *)ly.ids : n == "weights" ? (const void *)ly.weights
                      : n == "cat16" ? (const void *)ly.cat16 : n == "n_fast" ? ly.n_fast : n == "n_rows" ? ly.n_rows
                      : n == "logits" ? (const void *)ly.logits : n == "moe_g" ? m->moe_g : n == "drg" ? (const void *)m->drg
                      : n == "weight_of" ? (const void *)ly.weight_of : n == "x_seg" ? (const void *)ly.x_seg
                      : n == "x_valid" ? (const void *)ly.x_valid : n == "x_token_of" ? (const void *)ly.x_token_of
                      : n == "x_weight_of" ? (const void *)ly.x_weight_of : n == "x_tile_group" ? (const void *)ly.x_tile_group
                      : n == "own_rows" ? (const void *)m->own_rows : n == "own_y" ? (const void *)m->own_y
                      : n == "moe_y" ? (const void *)m->moe_y
                      : n == "capture" && (size_t)bytes <= m->capture_bytes ? m->capture_buf : nullptr;
    if (!src)
        return fail(TS2_ERR_INVALID_ARG, "ts2_debug_read: unknown or absent buffer '%s'", name);
    TS2_CUDA(cudaMemcpy(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost));
    return TS2_OK;
}

int ts2_discard_gradient(ts2_model *m)
{
    if (!m)
        return fail(TS2_ERR_INVALID_ARG, "null model");
    m->grads_dirty = false; // the next ts2_backprop clears the flat gradient before it accumulates
    return TS2_OK;
}

int ts2_get_step_health(ts2_model *m, int reset, uint32_t *first_bad_step, int n_boundaries, int64_t *steps_so_far)
{
    if (!m || !first_bad_step || n_boundaries != m->L + 1)
        return fail(TS2_ERR_INVALID_ARG, "ts2_get_step_health: pass layer_count + 1 entries");
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    TS2_CUDA(cudaMemcpy(first_bad_step, m->health, (size_t)(m->L + 1) * 4, cudaMemcpyDeviceToHost));
    if (reset)
        TS2_CUDA(cudaMemset(m->health, 0, (size_t)(m->L + 1) * 4));
    if (steps_so_far)
        *steps_so_far = m->step_no;
    return TS2_OK;
}

int ts2_get_loss_history(ts2_model *m, float *out_err, int n)
{
    if (!m || !out_err || n < 0 || n > ts2_model::LOSS_RING || (unsigned)n > m->step_no)
        return fail(TS2_ERR_INVALID_ARG, "ts2_get_loss_history: n must be in [0, min(%d, steps so far)]", ts2_model::LOSS_RING);
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    float ring[ts2_model::LOSS_RING];
    TS2_CUDA(cudaMemcpy(ring, m->logp_ring, sizeof(ring), cudaMemcpyDeviceToHost));
    for (int i = 0; i < n; ++i) { // oldest first
        const unsigned step = m->step_no - (unsigned)(n - 1 - i), slot = step % ts2_model::LOSS_RING;
        out_err[i] = m->ring_targets[slot] ? -ring[slot] / m->ring_targets[slot] : 0.f;
    }
    return TS2_OK;
}

int ts2_set_debug_trace(ts2_model *m, int enable)
{
    if (!m)
        return fail(TS2_ERR_INVALID_ARG, "null model");
    TS2_CUDA(cudaSetDevice(m->device));
    if (enable && !m->trace_dev)
        M_TRY(dalloc(m, &m->trace_dev, (size_t)ts2_model::TRACE_MAX * 4));
    m->trace_on = enable != 0;
    if (!enable)
        m->trace_names.clear();
    return TS2_OK;
}

int ts2_set_debug_capture(ts2_model *m, const char *record_name, int64_t max_bytes)
{
    if (!m || max_bytes < 0)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_set_debug_capture");
    TS2_CUDA(cudaSetDevice(m->device));
    m->capture_name = record_name ? record_name : "";
    m->capture_bytes = 0;
    if (!m->capture_name.empty() && (size_t)max_bytes > m->capture_cap) {
        M_TRY(dalloc(m, (uint8_t **)&m->capture_buf, (size_t)max_bytes)); // an earlier, smaller buffer stays with the model
        m->capture_cap = (size_t)max_bytes;
    }
    return TS2_OK;
}

int ts2_get_debug_trace(ts2_model *m, uint64_t *sums, uint64_t *nonfinite, float *max_abs, int capacity, int *count)
{
    if (!m || !count || capacity < 0 || (capacity && (!sums || !nonfinite)))
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_get_debug_trace");
    const int n = (int)m->trace_names.size();
    *count = n;
    if (!capacity || !n)
        return TS2_OK;
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    std::vector<unsigned long long> host((size_t)n * 4);
    TS2_CUDA(cudaMemcpy(host.data(), m->trace_dev, host.size() * 8, cudaMemcpyDeviceToHost));
    for (int i = 0; i < std::min(n, capacity); ++i) {
        sums[i] = host[4 * i];
        nonfinite[i] = host[4 * i + 1];
        if (max_abs) {
            const uint32_t bits = (uint32_t)host[4 * i + 2];
            memcpy(max_abs + i, &bits, 4);
        }
    }
    return TS2_OK;
}

const char *ts2_debug_trace_name(ts2_model *m, int index)
{
    if (!m || index < 0 || index >= (int)m->trace_names.size())
        return "";
    return m->trace_names[index].c_str();
}

int ts2_dp_layout(const ts2_model_descr *descr, int64_t *matrix_offset, int n_mats, int64_t *bucket_offset, int64_t *bucket_elems,
                  int32_t *bucket_first_matrix, int max_buckets)
{
    int rc = validate(descr);
    if (rc != TS2_OK)
        return rc;
    std::vector<std::pair<int64_t, int64_t>> shapes;
    shapes_of(descr, &shapes);
    std::vector<Bucket> buckets;
    std::vector<size_t> mat_off;
    std::vector<int> mat_bucket;
    layout_buckets(descr, shapes, &buckets, &mat_off, &mat_bucket);
    if (matrix_offset) {
        if (n_mats != (int)shapes.size())
            return fail(TS2_ERR_INVALID_ARG, "ts2_dp_layout: expected %d matrices, got %d", (int)shapes.size(), n_mats);
        for (int i = 0; i < n_mats; ++i)
            matrix_offset[i] = (int64_t)mat_off[i];
    }
    for (int b = 0; b < std::min((int)buckets.size(), max_buckets); ++b) {
        if (bucket_offset)
            bucket_offset[b] = (int64_t)buckets[b].off;
        if (bucket_elems)
            bucket_elems[b] = (int64_t)buckets[b].elems;
        if (bucket_first_matrix)
            bucket_first_matrix[b] = buckets[b].mat0;
    }
    return (int)buckets.size();
}

int ts2_comm_unique_id(uint8_t id[TS2_COMM_ID_BYTES])
{
    static_assert(sizeof(ncclUniqueId) <= TS2_COMM_ID_BYTES, "id buffer too small");
    if (!id)
        return fail(TS2_ERR_INVALID_ARG, "null id");
    ncclUniqueId u;
    ncclResult_t r = ncclGetUniqueId(&u);
    if (r != ncclSuccess)
        return fail(TS2_ERR_COMM, "ncclGetUniqueId failed: %s", ncclGetErrorString(r));
    memset(id, 0, TS2_COMM_ID_BYTES);
    memcpy(id, &u, sizeof(u));
    return TS2_OK;
}

int ts2_comm_init(ts2_model *m, int rank, int world_size, const uint8_t id[TS2_COMM_ID_BYTES])
{
    if (!m || !id || world_size < 1 || rank < 0 || rank >= world_size)
        return fail(TS2_ERR_INVALID_ARG, "bad arguments to ts2_comm_init");
    if (m->comm)
        return fail(TS2_ERR_INVALID_ARG, "communicator already initialised");
    TS2_CUDA(cudaSetDevice(m->device));
    m->rank = rank;
    m->world = world_size;
    if (world_size == 1)
        return TS2_OK;
    if (BUCKET_PAD % (4 * (size_t)world_size))
        return fail(TS2_ERR_UNSUPPORTED, "world size %d: every rank's part of a bucket must be a multiple of 4 elements (world sizes that divide %zu)",
                    world_size, BUCKET_PAD / 4);
    ncclUniqueId u;
    memcpy(&u, id, sizeof(u));
    // The exchanges run beside the backward pass, whose contractions are persistent kernels sized to every SM, and a
    // communication CTA does not fit beside a contraction CTA (shared memory).  Measured on two B200s (step time against
    // one GPU's on the same box): a cap of 4 CTAs +5.1 %, 8 +2.8 %, 16 +2.1 %, 32 +0.9 %, NCCL's own choice +1.5 %: short
    // exchanges on many SMs disturb the contractions less than long ones on few, so the default is no cap
    // (TS2_NCCL_MAX_CTAS sets one).
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    int max_ctas = 0;
    if (const char *e = getenv("TS2_NCCL_MAX_CTAS"))
        max_ctas = atoi(e);
    if (max_ctas > 0) {
        cfg.maxCTAs = max_ctas;
        cfg.minCTAs = std::min(cfg.maxCTAs, 1);
    }
    ncclResult_t r = ncclCommInitRankConfig(&m->comm, world_size, u, rank, &cfg);
    if (r != ncclSuccess) {
        m->comm = nullptr;
        return mfail(m, fail(TS2_ERR_COMM, "ncclCommInitRankConfig failed: %s", ncclGetErrorString(r)));
    }
    // Leaving SMs free for the exchanges instead (TS2_GEMM_RESERVE_SMS, default 0) measured slower: +7 % with 8 SMs.
    if (const char *e = getenv("TS2_GEMM_RESERVE_SMS"))
        gemm_reserve_sms(atoi(e));
    std::vector<OptSeg> segs;
    build_segments(m, world_size, rank, &segs, &m->nitems_shard);
    m->nseg_shard = (int)segs.size();
    m->d_segs_shard = nullptr;
    M_TRY(upload_segments(m, segs, &m->d_segs_shard));
    return TS2_OK;
}

// Maps the exchange buffers of every other rank into this process (CUDA IPC handles travel through an all-gather) and
// puts the base pointers, this rank's own among them, in a device table.  All ranks agree on the outcome: where any
// rank cannot map a buffer, every rank keeps the ncclSend / ncclRecv exchange (TS2_EP_EXCHANGE=nccl asks for that).
static int ep_map_peers(ts2_model *m)
{
    const int N = m->world, NB = ts2_model::PB_COUNT;
    void *local[NB] = {m->own_rows, m->own_g, m->own_w, m->moe_y, m->dmoe_part};
    const char *mode = getenv("TS2_EP_EXCHANGE");
    int ok = !(mode && std::string(mode) == "nccl");
    std::vector<cudaIpcMemHandle_t> all((size_t)N * NB);
    cudaIpcMemHandle_t mine[NB];
    memset(mine, 0, sizeof(mine));
    for (int k = 0; k < NB && ok; ++k)
        if (cudaIpcGetMemHandle(&mine[k], local[k]) != cudaSuccess) {
            cudaGetLastError();
            ok = 0;
        }
    uint8_t *d_h = nullptr;
    const size_t hb = sizeof(mine);
    M_TRY(dalloc(m, &d_h, hb * (N + 1) + 16));
    TS2_CUDA(cudaMemcpy(d_h + hb * N, mine, hb, cudaMemcpyHostToDevice));
    M_NCCL(ncclAllGather(d_h + hb * N, d_h, hb, ncclUint8, m->comm_x, m->stream));
    int *d_ok = (int *)(d_h + hb * (N + 1));
    TS2_CUDA(cudaMemcpyAsync(d_ok, &ok, 4, cudaMemcpyHostToDevice, m->stream));
    M_NCCL(ncclAllReduce(d_ok, d_ok, 1, ncclInt32, ncclMin, m->comm_x, m->stream));
    TS2_CUDA(cudaStreamSynchronize(m->stream));
    TS2_CUDA(cudaMemcpy(all.data(), d_h, hb * N, cudaMemcpyDeviceToHost));
    TS2_CUDA(cudaMemcpy(&ok, d_ok, 4, cudaMemcpyDeviceToHost));
    std::vector<uint8_t *> table((size_t)NB * N, nullptr);
    for (int r = 0; r < N && ok; ++r)
        for (int k = 0; k < NB && ok; ++k) {
            if (r == m->rank) {
                table[(size_t)k * N + r] = (uint8_t *)local[k];
                continue;
            }
            void *ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, all[(size_t)r * NB + k], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                ok = 0;
                break;
            }
            m->ipc_opened.push_back(ptr);
            table[(size_t)k * N + r] = (uint8_t *)ptr;
        }
    // every rank must have opened everything
    TS2_CUDA(cudaMemcpyAsync(d_ok, &ok, 4, cudaMemcpyHostToDevice, m->stream));
    M_NCCL(ncclAllReduce(d_ok, d_ok, 1, ncclInt32, ncclMin, m->comm_x, m->stream));
    TS2_CUDA(cudaStreamSynchronize(m->stream));
    TS2_CUDA(cudaMemcpy(&ok, d_ok, 4, cudaMemcpyDeviceToHost));
    if (ok) {
        M_TRY(dalloc(m, &m->d_peer, (size_t)NB * N));
        TS2_CUDA(cudaMemcpy(m->d_peer, table.data(), table.size() * sizeof(uint8_t *), cudaMemcpyHostToDevice));
    }
    m->x_peer = ok != 0;
    return TS2_OK;
}

int ts2_set_expert_parallel(ts2_model *m, float capacity_factor)
{
    if (!m)
        return TS2_ERR_INVALID_ARG;
    if (!m->comm || m->world < 2)
        return fail(TS2_ERR_INVALID_ARG, "expert parallel needs ts2_comm_init with more than one rank first");
    if (m->ep)
        return fail(TS2_ERR_INVALID_ARG, "expert parallel is already on");
    if (m->E == 0 || m->moe_rows == 0)
        return fail(TS2_ERR_INVALID_ARG, "the model has no mixture-of-experts layer");
    if (m->E % m->world)
        return fail(TS2_ERR_UNSUPPORTED, "%d experts do not divide over %d ranks", m->E, m->world);
    if (!(capacity_factor >= 1.f) || capacity_factor > (float)m->world)
        capacity_factor = std::min(4.f, (float)m->world); // a router without a balancing term sent 2.9x to one of 4 ranks
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(sync_master(m));
    TS2_CUDA(cudaDeviceSynchronize());
    ncclResult_t r = ncclCommSplit(m->comm, 0, m->rank, &m->comm_x, nullptr);
    if (r != ncclSuccess) {
        m->comm_x = nullptr;
        return mfail(m, fail(TS2_ERR_COMM, "ncclCommSplit failed: %s", ncclGetErrorString(r)));
    }
    // received layout: a rank's share of all (token, choice) rows times the factor, plus the padding of its experts
    const size_t own = (size_t)m->K * m->max_nodes;
    const size_t R = ((size_t)(capacity_factor * (double)own) + 127) / 128 * 128 + 128 * (size_t)(m->E / m->world);
    m->x_cap = (int)R;
    const size_t D = m->D, X = m->X, fs = fast_size(m), T = m->max_nodes;
    for (Layer &ly : m->layers) {
        if (ly.type != TS2_LAYER_MOE)
            continue;
        M_TRY(regrow(m, (uint8_t **)&ly.n_rows, R * D * fs));
        M_TRY(regrow(m, &ly.cat16, R * 2 * X));
        M_TRY(regrow(m, &ly.what, R * X));
        M_TRY(regrow(m, &ly.wscale, R * (X / 128)));
        M_TRY(regrow(m, (uint8_t **)&ly.rg, R * X * fs));
        M_TRY(dalloc(m, &ly.x_token_of, R));
        M_TRY(dalloc(m, &ly.x_weight_of, R));
        M_TRY(dalloc(m, &ly.x_tile_group, R / 128));
        M_TRY(dalloc(m, &ly.x_seg, (size_t)m->E + 1));
        M_TRY(dalloc(m, &ly.x_valid, (size_t)m->E));
    }
    size_t max_wide = 0, max_cat = 0;
    for (const Layer &ly : m->layers)
        if (ly.type != TS2_LAYER_MOE) {
            max_wide = std::max<size_t>(max_wide, ly.wide);
            max_cat = std::max<size_t>(max_cat, (size_t)ly.ncat * ly.wide);
        }
    M_TRY(regrow(m, &m->moe_y, R * D));
    M_TRY(regrow(m, (uint8_t **)&m->moe_g, R * D * fs));
    M_TRY(regrow(m, &m->dmoe_part, R * (X / 128)));
    M_TRY(regrow(m, &m->drg, std::max(T * max_wide, R * X)));
    M_TRY(regrow(m, (uint8_t **)&m->dcat, std::max(T * max_cat, R * 2 * X) * fs));
    const size_t own_rows = m->moe_rows;
    M_TRY(dalloc(m, (uint8_t **)&m->own_rows, own_rows * D * fs));
    M_TRY(dalloc(m, (uint8_t **)&m->own_g, own_rows * D * fs));
    M_TRY(dalloc(m, &m->own_y, own_rows * D));
    M_TRY(dalloc(m, &m->own_part, own_rows * (X / 128)));
    M_TRY(dalloc(m, &m->cnt_own, (size_t)m->E));
    M_TRY(dalloc(m, &m->cnt_all, (size_t)m->E * m->world));
    TS2_CUDA(cudaMallocHost(&m->h_cnt, (size_t)m->E * m->world * 4));
    M_TRY(dalloc(m, &m->own_w, own_rows));
    M_TRY(dalloc(m, &m->x_flag, 1));
    TS2_CUDA(cudaMemset(m->x_flag, 0, 4));
    for (Layer &ly : m->layers)
        if (ly.type == TS2_LAYER_MOE)
            M_TRY(dalloc(m, &ly.d_moves, (size_t)m->E * (m->world + 1)));
    M_TRY(ep_map_peers(m));
    // the expert matrices stop travelling: rank r's part of such a bucket is the rows of its experts (no padding, whole
    // experts per part), their gradient arises there in full and only that rank reads their quantized weights
    for (Bucket &bk : m->buckets) {
        if (!bk.expert_matrix)
            continue;
        const Matrix &mt = m->mats[bk.mat0];
        const size_t per_expert = (size_t)mt.x * mt.y / m->E;
        bk.owner_only = bk.mat1 == bk.mat0 + 1 && bk.elems == (size_t)mt.x * mt.y && (bk.elems / m->world) % per_expert == 0;
    }
    m->ep = true;
    return TS2_OK;
}

int ts2_get_exchange_ms(ts2_model *m, int enable, float *ms, double *bytes_sent, int *exchanges)
{
    if (!m)
        return TS2_ERR_INVALID_ARG;
    TS2_CUDA(cudaSetDevice(m->device));
    M_TRY(wait_stream(m));
    float total = 0.f;
    for (size_t i = 0; i < m->x_events_used; ++i) {
        float t = 0.f;
        TS2_CUDA(cudaEventElapsedTime(&t, m->x_events[i].first, m->x_events[i].second));
        total += t;
    }
    if (ms)
        *ms = total;
    if (bytes_sent)
        *bytes_sent = m->x_bytes;
    if (exchanges)
        *exchanges = (int)m->x_events_used;
    m->x_events_used = 0;
    m->x_bytes = 0;
    m->x_timing = enable != 0;
    return TS2_OK;
}

int ts2_moe_exchange_plan(int world_size, int rank, int expert_count, const int32_t *counts, int32_t *own_seg, int32_t *x_seg,
                          int32_t *x_valid, int32_t *moves, int max_moves, int32_t *n_out, int32_t *n_in, int32_t *max_x_rows)
{
    if (world_size < 1 || rank < 0 || rank >= world_size || expert_count < 1 || expert_count % world_size || !counts || !own_seg || !x_seg ||
        !x_valid || !moves || !n_out || !n_in || !max_x_rows)
        return fail(TS2_ERR_INVALID_ARG, "ts2_moe_exchange_plan: bad arguments");
    EpPlan p;
    int mx = 0;
    ep_plan(world_size, rank, expert_count, counts, &p, &mx);
    if ((int)(p.out.size() + p.in.size()) > max_moves)
        return fail(TS2_ERR_TOO_LARGE, "ts2_moe_exchange_plan: %zu moves, room for %d", p.out.size() + p.in.size(), max_moves);
    own_seg[0] = 0;
    for (int e = 0; e < expert_count; ++e)
        own_seg[e + 1] = own_seg[e] + (counts[rank * expert_count + e] + 127) / 128 * 128;
    memcpy(x_seg, p.x_seg.data(), (size_t)(expert_count + 1) * 4);
    memcpy(x_valid, p.x_valid.data(), (size_t)expert_count * 4);
    int k = 0;
    for (const auto *list : {&p.out, &p.in})
        for (const EpPlan::Move &mv : *list) {
            moves[4 * k + 0] = mv.peer;
            moves[4 * k + 1] = mv.own_row;
            moves[4 * k + 2] = mv.x_row;
            moves[4 * k + 3] = mv.rows;
            ++k;
        }
    *n_out = (int)p.out.size();
    *n_in = (int)p.in.size();
    *max_x_rows = mx;
    return TS2_OK;
}

int64_t ts2_launch_count(ts2_model *, int reset)
{
    long long v = reset ? g_launch_count.exchange(0) : g_launch_count.load();
    return v;
}

int ts2_last_step_ms(ts2_model *m, float *ms)
{
    if (!m || !ms || !m->timing_valid)
        return fail(TS2_ERR_INVALID_ARG, "no timed step");
    TS2_CUDA(cudaSetDevice(m->device));
    TS2_CUDA(cudaEventSynchronize(m->ev_stop));
    TS2_CUDA(cudaEventElapsedTime(ms, m->ev_start, m->ev_stop));
    return TS2_OK;
}

int ts2_timer_begin(ts2_model *m)
{
    if (!m)
        return fail(TS2_ERR_INVALID_ARG, "null model");
    TS2_CUDA(cudaSetDevice(m->device));
    TS2_CUDA(cudaEventRecord(m->ev_t0, m->stream));
    return TS2_OK;
}

int ts2_timer_end(ts2_model *m, float *ms)
{
    if (!m || !ms)
        return fail(TS2_ERR_INVALID_ARG, "null argument");
    TS2_CUDA(cudaSetDevice(m->device));
    TS2_CUDA(cudaEventRecord(m->ev_t1, m->stream));
    M_TRY(wait_stream(m));
    TS2_CUDA(cudaEventElapsedTime(ms, m->ev_t0, m->ev_t1));
    return TS2_OK;
}

int ts2_set_kernel_timing(ts2_model *, int enable)
{
    gemm_timing_enable(enable != 0);
    return TS2_OK;
}

int ts2_get_kernel_bytes(ts2_model *, double *gemm_bytes_total)
{
    gemm_timing_get(false, nullptr, nullptr, nullptr, gemm_bytes_total);
    return TS2_OK;
}

int ts2_get_kernel_timing_class(ts2_model *, int cls, double *gemm_ms_total, int64_t *gemm_launches, double *gemm_flops_total)
{
    if (cls < 0 || cls >= GEMM_TAGS)
        return fail(TS2_ERR_INVALID_ARG, "ts2_get_kernel_timing_class: class %d outside [0, %d)", cls, (int)GEMM_TAGS);
    long long n = 0;
    gemm_timing_get_tag(cls, gemm_ms_total, &n, gemm_flops_total);
    if (gemm_launches)
        *gemm_launches = n;
    return TS2_OK;
}

int ts2_get_kernel_timing(ts2_model *, int reset, double *gemm_ms_total, int64_t *gemm_launches, double *gemm_flops_total)
{
    long long n = 0;
    gemm_timing_get(reset != 0, gemm_ms_total, &n, gemm_flops_total);
    if (gemm_launches)
        *gemm_launches = n;
    return TS2_OK;
}

} // extern "C"
