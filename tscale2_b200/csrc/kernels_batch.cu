// Batch preparation on the device: what the reference derives from a batch on one host thread before each step
// (attention span tables, TNodesBatch / GroupAttention, src/gpt/att/att.h:125-211; the inverse label index of the
// embedding gradient, TLabelInverseIndex, src/gpt/compute/gpu_embedding.cuh:10-76) is computed here from the raw CSR
// arrays of the batch, which arrive in one host-to-device copy.
//
//  * per-node span tables and, per key, the range of nodes that may attend to it (prefix maximum of the span ends,
//    suffix minimum of the span starts, two binary searches per key);
//  * the target table;
//  * the inverse label index: entries (label, node) sorted by label with a stable 8-bit LSD radix sort, so that the
//    nodes of one label appear in node order, and an embedding gradient that sums them in that fixed order - no float
//    atomics, the result does not depend on the schedule.
//
// Every element of the inputs is validated here as well.  A bad element is replaced by a harmless one (label 0, no
// span, no target) so that the kernels that follow stay inside their buffers, and the first one is recorded in a
// status record that the host reads when it next waits for the stream.
#include "kernels.cuh"

namespace ts2 {
namespace {

constexpr int BP_THREADS = 256;
constexpr int BP_WARPS = BP_THREADS / 32;

__device__ __forceinline__ void batch_fail(int *status, int code, int where, int a, int b)
{
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = where;
        status[2] = a;
        status[3] = b;
    }
}

// ---- spans ---------------------------------------------------------------------------
__global__ void span_expand_kernel(const int *__restrict__ span_ptr, const int *__restrict__ csr_start, const int *__restrict__ csr_finish,
                                   int T, int n_spans, int *__restrict__ start, int *__restrict__ finish, int *status)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T)
        return;
    const int p0 = span_ptr[t], n = span_ptr[t + 1] - p0;
    int s = 0, f = -1;
    if (n < 0 || p0 < 0 || p0 + n > n_spans) {
        batch_fail(status, BATCH_BAD_SPAN_PTR, t, p0, n);
    } else if (n > 1) {
        batch_fail(status, BATCH_MULTI_SPAN, t, n, 0);
    } else if (n == 1) {
        s = csr_start[p0];
        f = csr_finish[p0];
        if (s < 0 || f >= T || f < s) {
            batch_fail(status, BATCH_BAD_SPAN, t, s, f);
            s = 0;
            f = -1;
        }
    }
    start[t] = s;
    finish[t] = f;
}

// run_max[t] = max of finish[0..t], suf_min[t] = min of start[t..T) over the nodes that have a span (-1 / T where none
// has).  Two launches over blocks of 1024 nodes: the blocks' own maxima and minima first, then each block scans its
// nodes starting from what the blocks before (after) it hold.
__global__ void __launch_bounds__(1024) span_block_reduce_kernel(const int *__restrict__ start, const int *__restrict__ finish, int T,
                                                                 int *__restrict__ blk_max, int *__restrict__ blk_min)
{
    __shared__ int s_max[32], s_min[32];
    const int t = blockIdx.x * 1024 + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int mx = -1, mn = T;
    if (t < T) {
        const int s = start[t], f = finish[t];
        if (f >= s) {
            mx = f;
            mn = s;
        }
    }
    for (int d = 16; d; d >>= 1) {
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
        mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, d));
    }
    if (lane == 0) {
        s_max[warp] = mx;
        s_min[warp] = mn;
    }
    __syncthreads();
    if (warp == 0) {
        mx = s_max[lane];
        mn = s_min[lane];
        for (int d = 16; d; d >>= 1) {
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, d));
        }
        if (lane == 0) {
            blk_max[blockIdx.x] = mx;
            blk_min[blockIdx.x] = mn;
        }
    }
}

__global__ void __launch_bounds__(1024) span_scan_kernel(const int *__restrict__ start, const int *__restrict__ finish, int T,
                                                         const int *__restrict__ blk_max, const int *__restrict__ blk_min,
                                                         int *__restrict__ run_max, int *__restrict__ suf_min)
{
    __shared__ int s_max[32], s_min[32];
    const int t = blockIdx.x * 1024 + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int mx = -1, mn = T;
    if (t < T) {
        const int s = start[t], f = finish[t];
        if (f >= s) {
            mx = f;
            mn = s;
        }
    }
    // inside the warp: inclusive prefix maximum, inclusive suffix minimum
    for (int d = 1; d < 32; d <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, mx, d), b = __shfl_down_sync(0xffffffffu, mn, d);
        if (lane >= d)
            mx = max(mx, a);
        if (lane + d < 32)
            mn = min(mn, b);
    }
    if (lane == 31)
        s_max[warp] = mx;
    if (lane == 0)
        s_min[warp] = mn;
    __syncthreads();
    // what the earlier warps and blocks hold (the later ones for the minimum)
    int before = -1, after = T;
    for (int w = 0; w < warp; ++w)
        before = max(before, s_max[w]);
    for (int w = warp + 1; w < 32; ++w)
        after = min(after, s_min[w]);
    for (int bb = lane; bb < (int)blockIdx.x; bb += 32)
        before = max(before, blk_max[bb]);
    for (int bb = blockIdx.x + 1 + lane; bb < (int)gridDim.x; bb += 32)
        after = min(after, blk_min[bb]);
    for (int d = 16; d; d >>= 1) {
        before = max(before, __shfl_xor_sync(0xffffffffu, before, d));
        after = min(after, __shfl_xor_sync(0xffffffffu, after, d));
    }
    if (t < T) {
        run_max[t] = max(mx, before);
        suf_min[t] = min(mn, after);
    }
}

// nodes that may attend to key `to`: none before the first node whose running maximum of span ends reaches `to`, none
// after the last node whose suffix minimum of span starts is at most `to`.  (T, -1) when there is none.
__global__ void span_reverse_kernel(const int *__restrict__ run_max, const int *__restrict__ suf_min, int T, int *__restrict__ rev_first,
                                    int *__restrict__ rev_last)
{
    const int to = blockIdx.x * blockDim.x + threadIdx.x;
    if (to >= T)
        return;
    int lo = 0, hi = T; // first t with run_max[t] >= to
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (run_max[mid] >= to)
            hi = mid;
        else
            lo = mid + 1;
    }
    const int first = lo;
    lo = 0, hi = T; // first t with suf_min[t] > to
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (suf_min[mid] > to)
            hi = mid;
        else
            lo = mid + 1;
    }
    const int last = lo - 1;
    const bool any = first <= last;
    rev_first[to] = any ? first : T;
    rev_last[to] = any ? last : -1;
}

// ---- targets -------------------------------------------------------------------------
__global__ void target_scatter_kernel(const int *__restrict__ node, const int *__restrict__ id, int n, int T, int V, int *__restrict__ target,
                                      int *status)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int t = node[i], v = id[i];
    if (t < 0 || t >= T || v < 0 || v >= V) {
        batch_fail(status, BATCH_BAD_TARGET, i, t, v);
        return;
    }
    if (atomicExch(&target[t], v) != -1)
        batch_fail(status, BATCH_DUP_TARGET, t, v, 0);
}

// ---- labels --------------------------------------------------------------------------
// validates label_ptr / label_arr in place and writes the (label, node | sign) entries of the inverse index
__global__ void label_entries_kernel(uint32_t *__restrict__ label_arr, uint32_t *__restrict__ label_ptr, int T, uint32_t n_labels,
                                     uint32_t label_count, uint32_t *__restrict__ key, uint32_t *__restrict__ val, int *status)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T)
        return;
    uint32_t p0 = label_ptr[t], p1 = label_ptr[t + 1];
    if (p0 > p1 || p1 > n_labels) {
        batch_fail(status, BATCH_BAD_LABEL_PTR, t, (int)p0, (int)p1);
        p0 = min(p0, n_labels);
        p1 = min(max(p1, p0), n_labels);
    }
    for (uint32_t k = p0; k < p1; ++k) {
        const uint32_t raw = label_arr[k];
        uint32_t label = raw & TS2_LABEL_MASK;
        if (label >= label_count) {
            batch_fail(status, BATCH_BAD_LABEL, (int)k, (int)label, t);
            label = 0;
            label_arr[k] = raw & TS2_LABEL_NEGATIVE;
        }
        key[k] = label;
        val[k] = (uint32_t)t | (raw & TS2_LABEL_NEGATIVE);
    }
}

// label_ptr clamped to n_labels (second pass: the loops `for k in [ptr[t], ptr[t+1])` of the embedding kernels then
// stay inside label_arr whatever the input held)
__global__ void label_ptr_clamp_kernel(uint32_t *__restrict__ label_ptr, int T, uint32_t n_labels)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t <= T)
        label_ptr[t] = min(label_ptr[t], n_labels);
}

// One pass of a stable least-significant-digit radix sort, 8 bits per pass, 256 entries per block.
//   COUNT: hist[digit * nblocks + block] = entries of the block with that digit
//   !COUNT: hist holds the exclusive scan of those counts; entries go to hist[..] + rank inside the block
template <bool COUNT>
__global__ void __launch_bounds__(BP_THREADS) radix_pass_kernel(const uint32_t *__restrict__ key_in, const uint32_t *__restrict__ val_in,
                                                                uint32_t n, int shift, uint32_t *__restrict__ hist, uint32_t nblocks,
                                                                uint32_t *__restrict__ key_out, uint32_t *__restrict__ val_out)
{
    __shared__ uint32_t cnt[BP_WARPS][256];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < BP_WARPS * 256; i += BP_THREADS)
        (&cnt[0][0])[i] = 0;
    __syncthreads();
    const uint32_t k = blockIdx.x * BP_THREADS + tid;
    const bool live = k < n;
    const uint32_t kv = live ? key_in[k] : 0;
    const uint32_t digit = live ? (kv >> shift) & 255u : 256u; // 256: the padding threads of the last block
    const unsigned peers = __match_any_sync(0xffffffffu, digit);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1));
    if (live && rank_in_warp == 0)
        cnt[warp][digit] = __popc(peers);
    __syncthreads();
    if (COUNT) {
        uint32_t sum = 0;
#pragma unroll
        for (int w = 0; w < BP_WARPS; ++w)
            sum += cnt[w][tid];
        hist[(size_t)tid * nblocks + blockIdx.x] = sum;
    } else if (live) {
        uint32_t before = 0;
        for (int w = 0; w < warp; ++w)
            before += cnt[w][digit];
        const uint32_t dst = hist[(size_t)digit * nblocks + blockIdx.x] + before + rank_in_warp;
        key_out[dst] = kv;
        val_out[dst] = val_in[k];
    }
}

// exclusive scan of `total` counters in place, blocks of 1024: the blocks' sums first, then each block scans its
// counters on top of the sums of the blocks before it
__global__ void __launch_bounds__(1024) scan_block_sums_kernel(const uint32_t *__restrict__ x, uint32_t total, uint32_t *__restrict__ blk_sum)
{
    __shared__ uint32_t s_sum[32];
    const uint32_t i = blockIdx.x * 1024 + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t v = i < total ? x[i] : 0;
    for (int d = 16; d; d >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0)
        s_sum[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = s_sum[lane];
        for (int d = 16; d; d >>= 1)
            v += __shfl_xor_sync(0xffffffffu, v, d);
        if (lane == 0)
            blk_sum[blockIdx.x] = v;
    }
}

__global__ void __launch_bounds__(1024) exclusive_scan_kernel(uint32_t *__restrict__ x, uint32_t total, const uint32_t *__restrict__ blk_sum)
{
    __shared__ uint32_t s_sum[32];
    const uint32_t i = blockIdx.x * 1024 + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t own = i < total ? x[i] : 0;
    uint32_t v = own;
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d)
            v += a;
    }
    if (lane == 31)
        s_sum[warp] = v;
    __syncthreads();
    uint32_t before = 0;
    for (int w = 0; w < warp; ++w)
        before += s_sum[w];
    uint32_t carry = 0;
    for (uint32_t bb = lane; bb < blockIdx.x; bb += 32)
        carry += blk_sum[bb];
    for (int d = 16; d; d >>= 1)
        carry += __shfl_xor_sync(0xffffffffu, carry, d);
    if (i < total)
        x[i] = carry + before + v - own;
}

// ---- embedding gradient through the inverse index ----------------------------------------
// The sorted entries are cut into chunks of EMB_CHUNK; one warp walks one chunk for one 128-wide tile of the state and
// sums the runs of equal labels in entry order.  A run that lies inside its chunk is added to its row of dE by that
// warp alone.  A run that crosses a chunk border leaves partial sums (slot 1: the run leaves the chunk at its end and
// did not enter it at the start; slot 0: the run entered at the start), which embed_chain_kernel adds up chunk by chunk.
constexpr int EMB_CHUNK = 64;

__device__ __forceinline__ void add4(float4 &a, const float4 &g, float w)
{
    a.x += g.x * w;
    a.y += g.y * w;
    a.z += g.z * w;
    a.w += g.w * w;
}

__device__ __forceinline__ void accumulate_row(float *row, const float4 &a)
{
    float4 v = *(float4 *)row;
    v.x += a.x;
    v.y += a.y;
    v.z += a.z;
    v.w += a.w;
    *(float4 *)row = v;
}

__global__ void __launch_bounds__(BP_THREADS) embed_runs_kernel(const float *__restrict__ g, const uint32_t *__restrict__ key,
                                                                const uint32_t *__restrict__ val, uint32_t n, int D,
                                                                float *__restrict__ dE, float *__restrict__ partial)
{
    const int tiles = D / TILE, lane = threadIdx.x & 31;
    const uint32_t nchunks = (n + EMB_CHUNK - 1) / EMB_CHUNK;
    const unsigned long long items = (unsigned long long)nchunks * tiles;
    for (unsigned long long item = blockIdx.x * BP_WARPS + (threadIdx.x >> 5); item < items; item += (unsigned long long)gridDim.x * BP_WARPS) {
        const uint32_t c = (uint32_t)(item / tiles);
        const int off = (int)(item % tiles) * TILE + lane * 4;
        const uint32_t k0 = c * EMB_CHUNK, k1 = min(n, k0 + EMB_CHUNK);
        const bool entered = k0 > 0 && key[k0 - 1] == key[k0]; // the first run began in an earlier chunk
        uint32_t run_label = key[k0];
        bool first_run = true;
        float4 acc = make_float4(0, 0, 0, 0);
        for (uint32_t kb = k0; kb < k1; kb += 32) {
            const uint32_t kk = kb + lane;
            const uint32_t my_key = kk < k1 ? key[kk] : 0, my_val = kk < k1 ? val[kk] : 0;
            const int cnt = (int)min(32u, k1 - kb);
            for (int j0 = 0; j0 < cnt; j0 += 4) {
                float4 gv[4];
                uint32_t lab[4];
                float w[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = min(j0 + u, cnt - 1);
                    lab[u] = __shfl_sync(0xffffffffu, my_key, j);
                    const uint32_t v = __shfl_sync(0xffffffffu, my_val, j);
                    w[u] = (v & TS2_LABEL_NEGATIVE) ? -1.f : 1.f;
                    gv[u] = *(const float4 *)(g + (size_t)(v & TS2_LABEL_MASK) * D + off);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (j0 + u >= cnt)
                        break;
                    if (lab[u] != run_label) {
                        // the run ended inside the chunk
                        if (first_run && entered)
                            *(float4 *)(partial + ((size_t)c * 2 + 0) * D + off) = acc;
                        else
                            accumulate_row(dE + (size_t)run_label * D + off, acc);
                        acc = make_float4(0, 0, 0, 0);
                        run_label = lab[u];
                        first_run = false;
                    }
                    add4(acc, gv[u], w[u]);
                }
            }
        }
        const bool leaves = k1 < n && key[k1] == run_label;
        if (first_run && entered)
            *(float4 *)(partial + ((size_t)c * 2 + 0) * D + off) = acc;
        else if (leaves)
            *(float4 *)(partial + ((size_t)c * 2 + 1) * D + off) = acc;
        else
            accumulate_row(dE + (size_t)run_label * D + off, acc);
    }
}

__global__ void __launch_bounds__(BP_THREADS) embed_chain_kernel(const uint32_t *__restrict__ key, uint32_t n, int D,
                                                                 const float *__restrict__ partial, float *__restrict__ dE)
{
    const int tiles = D / TILE, lane = threadIdx.x & 31;
    const uint32_t nchunks = (n + EMB_CHUNK - 1) / EMB_CHUNK;
    const unsigned long long items = (unsigned long long)nchunks * tiles;
    for (unsigned long long item = blockIdx.x * BP_WARPS + (threadIdx.x >> 5); item < items; item += (unsigned long long)gridDim.x * BP_WARPS) {
        const uint32_t c = (uint32_t)(item / tiles);
        const int off = (int)(item % tiles) * TILE + lane * 4;
        const uint32_t k0 = c * EMB_CHUNK, k1 = min(n, k0 + EMB_CHUNK);
        if (k1 >= n)
            continue;
        const uint32_t label = key[k1 - 1];
        if (key[k1] != label)
            continue; // nothing leaves this chunk
        if (k0 > 0 && key[k0 - 1] == label && key[k0] == label)
            continue; // the run that leaves also entered: an earlier chunk heads the chain
        float4 sum = *(const float4 *)(partial + ((size_t)c * 2 + 1) * D + off);
        for (uint32_t cc = c + 1; cc < nchunks; ++cc) {
            const float4 p = *(const float4 *)(partial + ((size_t)cc * 2 + 0) * D + off);
            sum.x += p.x;
            sum.y += p.y;
            sum.z += p.z;
            sum.w += p.w;
            const uint32_t e1 = min(n, (cc + 1) * EMB_CHUNK);
            if (!(key[e1 - 1] == label && e1 < n && key[e1] == label))
                break;
        }
        accumulate_row(dE + (size_t)label * D + off, sum);
    }
}

int blocks_for(long long n)
{
    return (int)std::max<long long>(1, (n + BP_THREADS - 1) / BP_THREADS);
}

} // namespace

int batch_span_tables(const Ctx &c, const int *span_ptr, const int *csr_start, const int *csr_finish, int T, int n_spans, int *start,
                      int *finish, int *scan_tmp, int *rev_first, int *rev_last, int *status)
{
    span_expand_kernel<<<blocks_for(T), BP_THREADS, 0, c.stream>>>(span_ptr, csr_start, csr_finish, T, n_spans, start, finish, status);
    TS2_CHECK_LAUNCH();
    return batch_reverse_ranges(c, start, finish, T, scan_tmp, rev_first, rev_last);
}

int batch_reverse_ranges(const Ctx &c, const int *start, const int *finish, int T, int *scan_tmp, int *rev_first, int *rev_last)
{
    const int nb = (T + 1023) / 1024;
    int *blk = scan_tmp + 2 * (size_t)T;
    span_block_reduce_kernel<<<nb, 1024, 0, c.stream>>>(start, finish, T, blk, blk + nb);
    TS2_CHECK_LAUNCH();
    span_scan_kernel<<<nb, 1024, 0, c.stream>>>(start, finish, T, blk, blk + nb, scan_tmp, scan_tmp + T);
    TS2_CHECK_LAUNCH();
    span_reverse_kernel<<<blocks_for(T), BP_THREADS, 0, c.stream>>>(scan_tmp, scan_tmp + T, T, rev_first, rev_last);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int batch_targets(const Ctx &c, const int *node, const int *id, int n, int T, int V, int *target, int *status)
{
    TS2_CUDA(cudaMemsetAsync(target, 0xff, (size_t)T * 4, c.stream));
    if (n > 0) {
        target_scatter_kernel<<<blocks_for(n), BP_THREADS, 0, c.stream>>>(node, id, n, T, V, target, status);
        TS2_CHECK_LAUNCH();
    }
    return TS2_OK;
}

size_t batch_scan_tmp_elems(int T)
{
    return 2 * (size_t)T + 2 * (((size_t)T + 1023) / 1024);
}

size_t label_index_hist_elems(size_t label_cap)
{
    const size_t counters = 256 * ((label_cap + BP_THREADS - 1) / BP_THREADS);
    return counters + (counters + 1023) / 1024; // and the block sums of their scan
}

size_t label_index_partial_elems(size_t label_cap, int D)
{
    return ((label_cap + EMB_CHUNK - 1) / EMB_CHUNK) * 2 * (size_t)D;
}

int label_index_entries(const Ctx &c, uint32_t *label_arr, uint32_t *label_ptr, int T, uint32_t n_labels, uint32_t label_count,
                        LabelIndex &ix, int *status)
{
    ix.n = n_labels;
    ix.sorted = 0;
    if (n_labels) {
        // entries that no node owns (a label_ptr with gaps) must still be valid: label 0 of node 0
        TS2_CUDA(cudaMemsetAsync(ix.key[0], 0, (size_t)n_labels * 4, c.stream));
        TS2_CUDA(cudaMemsetAsync(ix.val[0], 0, (size_t)n_labels * 4, c.stream));
    }
    label_entries_kernel<<<blocks_for(T), BP_THREADS, 0, c.stream>>>(label_arr, label_ptr, T, n_labels, label_count, ix.key[0], ix.val[0],
                                                                     status);
    TS2_CHECK_LAUNCH();
    label_ptr_clamp_kernel<<<blocks_for(T + 1), BP_THREADS, 0, c.stream>>>(label_ptr, T, n_labels);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int label_index_sort(const Ctx &c, uint32_t label_count, LabelIndex &ix)
{
    if (ix.n == 0)
        return TS2_OK;
    int bits = 1;
    while (bits < 31 && (1u << bits) < label_count)
        ++bits;
    const uint32_t nblocks = (ix.n + BP_THREADS - 1) / BP_THREADS;
    int cur = 0;
    for (int shift = 0; shift < bits; shift += 8) {
        const int out = cur ^ 1;
        radix_pass_kernel<true><<<nblocks, BP_THREADS, 0, c.stream>>>(ix.key[cur], ix.val[cur], ix.n, shift, ix.hist, nblocks, nullptr,
                                                                     nullptr);
        TS2_CHECK_LAUNCH();
        const uint32_t total = 256 * nblocks, nb = (total + 1023) / 1024;
        scan_block_sums_kernel<<<nb, 1024, 0, c.stream>>>(ix.hist, total, ix.hist + total);
        TS2_CHECK_LAUNCH();
        exclusive_scan_kernel<<<nb, 1024, 0, c.stream>>>(ix.hist, total, ix.hist + total);
        TS2_CHECK_LAUNCH();
        radix_pass_kernel<false><<<nblocks, BP_THREADS, 0, c.stream>>>(ix.key[cur], ix.val[cur], ix.n, shift, ix.hist, nblocks, ix.key[out],
                                                                      ix.val[out]);
        TS2_CHECK_LAUNCH();
        cur = out;
    }
    ix.sorted = cur;
    return TS2_OK;
}

int embed_backward_indexed(const Ctx &c, const float *g, const LabelIndex &ix, int D, float *dE)
{
    if (ix.n == 0)
        return TS2_OK;
    const uint32_t nchunks = (ix.n + EMB_CHUNK - 1) / EMB_CHUNK;
    const long long items = (long long)nchunks * (D / TILE);
    const int grid = (int)std::max<long long>(1, std::min<long long>((items + BP_WARPS - 1) / BP_WARPS, (long long)sm_count(c.device) * 8));
    embed_runs_kernel<<<grid, BP_THREADS, 0, c.stream>>>(g, ix.key[ix.sorted], ix.val[ix.sorted], ix.n, D, dE, ix.partial);
    TS2_CHECK_LAUNCH();
    embed_chain_kernel<<<grid, BP_THREADS, 0, c.stream>>>(ix.key[ix.sorted], ix.n, D, ix.partial, dE);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
