// Mixture-of-experts kernels: routing (top-k, weights), the token -> expert-sorted slot tables,
// row gathers, activation forward / backward for expert-sorted rows, expert combine forward /
// backward, router gradient.  Math follows the reference's CPU path: CpuMoe, CpuBackpropMoe,
// ScaleExperts, BackpropScaleExperts (src/gpt/compute/layer_moe.cu:287-404); the roles are those of
// MoeCalcSampleExpertLists, GroupPerExpertLists, FillXpTables, MoeGroupSamples, MatrixLoLUmoe,
// CombineExperts, BackpropRowTileNormalizeLoLUmoe, BackpropMoeKernel
// (src/gpt/compute/moe_kernels.cu:54-355, moe_kernels.cuh:14-177).
//
// Slots: every (token, choice) pair gets one row in an expert-sorted buffer; an expert's segment is
// padded to a multiple of 128 rows so that every 128-row tile of a contraction belongs to one expert.
// Slot order inside a segment is token order (stable), so the tables are deterministic.
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int WARPS = 8;
static constexpr int THREADS = WARPS * 32;
static constexpr int ROUTE_BLOCK = 256; // tokens per block in the slot assignment

static int grid_for(const Ctx &c, long long warp_items)
{
    long long blocks = ceil_div(warp_items, WARPS);
    long long cap = (long long)sm_count(c.device) * 8;
    return (int)std::max<long long>(1, std::min(blocks, cap));
}

#define WARP_ITEM_LOOP(total)                                                                                              \
    const int lane = threadIdx.x & 31;                                                                                     \
    for (unsigned item = blockIdx.x * WARPS + (threadIdx.x >> 5), total_items = (unsigned)(total); item < total_items;     \
         item += gridDim.x * WARPS)

// ---------------------------------------------------------------------------------------
// top-k by repeated arg-max (lowest index wins ties), weights exp((l - lmax)/2) scaled to L2 norm sqrt(E)
__global__ void moe_route_kernel(const float *__restrict__ logits, int ld, int T, int E, int k, int *__restrict__ ids,
                                 float *__restrict__ weights)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T)
        return;
    const float *l = logits + (size_t)t * ld;
    float max_val = -1e10f;
    for (int x = 0; x < E; ++x)
        max_val = fmaxf(max_val, l[x]);
    unsigned long long taken_lo = 0, taken_hi = 0; // up to 128 experts
    float w[8];
    float sum2 = 0.f;
    for (int z = 0; z < k; ++z) {
        float top = -1e10f;
        int top_idx = 0;
        for (int x = 0; x < E; ++x) {
            const bool taken = x < 64 ? (taken_lo >> x) & 1 : (taken_hi >> (x - 64)) & 1;
            const float v = taken ? -1e10f : l[x];
            if (v > top) {
                top = v;
                top_idx = x;
            }
        }
        if (top_idx < 64)
            taken_lo |= 1ull << top_idx;
        else
            taken_hi |= 1ull << (top_idx - 64);
        const float wz = expf((top - max_val) * 0.5f); // MOE_SCALE
        ids[(size_t)t * k + z] = top_idx;
        w[z] = wz;
        sum2 += wz * wz;
    }
    const float scale = sqrtf((float)E) * sqrtf(1.f / sum2);
    for (int z = 0; z < k; ++z)
        weights[(size_t)t * k + z] = w[z] * scale;
}

int moe_route(const Ctx &c, const float *logits, int ld, int T, int E, int k, int *ids, float *weights)
{
    if (k < 1 || k > 8 || E < k || E > 128)
        return fail(TS2_ERR_UNSUPPORTED, "moe_route: need 1 <= selected <= 8 and selected <= experts <= 128 (got %d of %d)", k, E);
    moe_route_kernel<<<(T + 127) / 128, 128, 0, c.stream>>>(logits, ld, T, E, k, ids, weights);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// slot tables in three steps: per-block histograms, one-block scan, in-order assignment
__global__ void moe_count_kernel(const int *__restrict__ ids, int n_pairs, int k, int E, int *__restrict__ hist)
{
    extern __shared__ int sh[];
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        sh[e] = 0;
    __syncthreads();
    const int p0 = blockIdx.x * ROUTE_BLOCK * k, p1 = min(n_pairs, p0 + ROUTE_BLOCK * k);
    for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x)
        atomicAdd(&sh[ids[p]], 1);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        hist[blockIdx.x * E + e] = sh[e];
}

// seg_ptr[e]: first row of expert e's segment (multiples of 128); block_base[b][e]: first slot of block b in it;
// tile_group[tile]: expert of each 128-row tile, -1 beyond the used rows; token_of / weight_of reset for all rows
__global__ void moe_scan_kernel(const int *__restrict__ hist, int n_blocks, int E, int max_rows, int *__restrict__ seg_ptr,
                                int *__restrict__ block_base, int *__restrict__ tile_group, int *__restrict__ token_of,
                                int *__restrict__ counts)
{
    __shared__ int total[128], start[129];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int b = 0; b < n_blocks; ++b) {
            block_base[b * E + e] = run; // relative for now
            run += hist[b * E + e];
        }
        total[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int pos = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = pos;
            pos += (total[e] + 127) / 128 * 128;
        }
        start[E] = pos;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x)
        seg_ptr[e] = start[e];
    if (counts)
        for (int e = threadIdx.x; e < E; e += blockDim.x)
            counts[e] = total[e];
    for (int i = threadIdx.x; i < n_blocks * E; i += blockDim.x)
        block_base[i] += start[i % E];
    for (int tile = threadIdx.x; tile < max_rows / 128; tile += blockDim.x) {
        const int row = tile * 128;
        int g = -1;
        for (int e = 0; e < E; ++e)
            if (row >= start[e] && row < start[e + 1])
                g = e;
        tile_group[tile] = g;
    }
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x)
        token_of[r] = -1;
}

__global__ void moe_assign_kernel(const int *__restrict__ ids, const float *__restrict__ weights, int n_pairs, int k, int E,
                                  const int *__restrict__ block_base, int *__restrict__ slot_of, int *__restrict__ token_of,
                                  float *__restrict__ weight_of)
{
    // thread e walks the block's (token, choice) pairs in order and hands out expert e's slots
    const int p0 = blockIdx.x * ROUTE_BLOCK * k, p1 = min(n_pairs, p0 + ROUTE_BLOCK * k);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int next = block_base[blockIdx.x * E + e];
        for (int p = p0; p < p1; ++p) {
            if (ids[p] != e)
                continue;
            slot_of[p] = next;
            token_of[next] = p / k;
            weight_of[next] = weights[p];
            ++next;
        }
    }
}

int moe_build_slots(const Ctx &c, const int *ids, const float *weights, int T, int k, int E, int max_rows, int *hist_scratch,
                    int *block_base_scratch, int *seg_ptr, int *tile_group, int *slot_of, int *token_of, float *weight_of, int *counts)
{
    const int n_pairs = T * k, n_blocks = (T + ROUTE_BLOCK - 1) / ROUTE_BLOCK;
    moe_count_kernel<<<n_blocks, 256, E * sizeof(int), c.stream>>>(ids, n_pairs, k, E, hist_scratch);
    TS2_CHECK_LAUNCH();
    moe_scan_kernel<<<1, 1024, 0, c.stream>>>(hist_scratch, n_blocks, E, max_rows, seg_ptr, block_base_scratch, tile_group, token_of,
                                               counts);
    TS2_CHECK_LAUNCH();
    moe_assign_kernel<<<n_blocks, 128, 0, c.stream>>>(ids, weights, n_pairs, k, E, block_base_scratch, slot_of, token_of, weight_of);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// Expert-parallel row space: the rows a rank received for the experts it owns.  seg[e] .. seg[e + 1] is expert e's
// segment (multiples of 128, empty for experts of other ranks), valid[e] of its rows hold data.
//  tile_group[tile] = expert of each 128-row tile (-1 beyond the used rows); token_of[row] = 0 for a row with data, -1
//  for padding (the activation kernels only test its sign).
__global__ void moe_ep_tables_kernel(const int *__restrict__ seg, const int *__restrict__ valid, int E, int max_rows,
                                     int *__restrict__ tile_group, int *__restrict__ token_of)
{
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= max_rows)
        return;
    int g = -1, used = 0;
    for (int e = 0; e < E; ++e)
        if (r >= seg[e] && r < seg[e + 1]) {
            g = e;
            used = r - seg[e] < valid[e];
        }
    token_of[r] = used ? 0 : -1;
    if ((r & 127) == 0)
        tile_group[r >> 7] = g;
}

int moe_ep_tables(const Ctx &c, const int *seg, const int *valid, int E, int max_rows, int *tile_group, int *token_of)
{
    moe_ep_tables_kernel<<<(max_rows + 255) / 256, 256, 0, c.stream>>>(seg, valid, E, max_rows, tile_group, token_of);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// zeroes the padding rows of a received buffer (a contraction over an expert's segment reads them)
__global__ void moe_zero_pad_rows_kernel(uint8_t *__restrict__ buf, int row_bytes, const int *__restrict__ seg, const int *__restrict__ valid)
{
    const int e = blockIdx.x;
    const int r0 = seg[e] + valid[e], r1 = seg[e + 1];
    const long long chunks = (long long)(r1 - r0) * (row_bytes / 16);
    uint4 *dst = (uint4 *)(buf + (size_t)r0 * row_bytes);
    for (long long i = threadIdx.x; i < chunks; i += blockDim.x)
        dst[i] = make_uint4(0, 0, 0, 0);
}

int moe_zero_pad_rows(const Ctx &c, void *buf, int row_bytes, const int *seg, const int *valid, int E)
{
    if (row_bytes % 16)
        return fail(TS2_ERR_INVALID_ARG, "moe_zero_pad_rows: row size must be a multiple of 16 bytes");
    moe_zero_pad_rows_kernel<<<E, 256, 0, c.stream>>>((uint8_t *)buf, row_bytes, seg, valid);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// Row exchange between ranks over peer memory (NVLink): each block of rows is pulled by the rank that needs it with
// plain loads from the other rank's buffer (mapped through CUDA IPC; this rank's own buffer is in the same table, so
// local blocks go the same way).  moves[i] = {peer, row in the sender-side layout, row in the owner-side layout, rows};
// to_owner: source = bases[peer] + sender row, destination = local + owner row; otherwise the other way round.
// A CTA takes chunks of 32 KB; V = bytes per access (16, or 4 for rows that are not multiples of 16 bytes).
constexpr int PULL_CHUNK = 32768;
constexpr int PULL_MAX_MOVES = 256;

template <int V>
__global__ void __launch_bounds__(256) moe_pull_rows_kernel(const int4 *__restrict__ moves, int n_moves, uint8_t *const *__restrict__ bases,
                                                            uint8_t *__restrict__ local, int row_bytes, int to_owner)
{
    __shared__ int first_chunk[PULL_MAX_MOVES + 1];
    using VT = typename std::conditional<V == 16, uint4, uint32_t>::type;
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < n_moves; ++i) {
            first_chunk[i] = run;
            run += (int)(((long long)moves[i].w * row_bytes + PULL_CHUNK - 1) / PULL_CHUNK);
        }
        first_chunk[n_moves] = run;
    }
    __syncthreads();
    const int total = first_chunk[n_moves];
    for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
        int lo = 0, hi = n_moves; // the move this chunk belongs to: last i with first_chunk[i] <= chunk
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (first_chunk[mid] <= chunk)
                lo = mid;
            else
                hi = mid;
        }
        const int4 mv = moves[lo];
        const long long bytes = (long long)mv.w * row_bytes, off = (long long)(chunk - first_chunk[lo]) * PULL_CHUNK;
        const int n = (int)(min((long long)PULL_CHUNK, bytes - off) / V);
        const long long src_row = to_owner ? mv.y : mv.z, dst_row = to_owner ? mv.z : mv.y;
        const VT *src = (const VT *)(bases[mv.x] + src_row * row_bytes + off);
        VT *dst = (VT *)(local + dst_row * row_bytes + off);
        int i = threadIdx.x;
        for (; i + 3 * 256 < n; i += 4 * 256) { // four loads in flight per thread
            const VT a = src[i], b = src[i + 256], c = src[i + 512], d = src[i + 768];
            dst[i] = a;
            dst[i + 256] = b;
            dst[i + 512] = c;
            dst[i + 768] = d;
        }
        for (; i < n; i += 256)
            dst[i] = src[i];
    }
}

int moe_pull_rows(const Ctx &c, const int4 *moves, int n_moves, uint8_t *const *bases, void *local, int row_bytes, bool to_owner,
                  long long total_bytes)
{
    if (n_moves <= 0)
        return TS2_OK;
    if (n_moves > PULL_MAX_MOVES || row_bytes % 4)
        return fail(TS2_ERR_INVALID_ARG, "moe_pull_rows: %d moves (at most %d), rows of %d bytes", n_moves, PULL_MAX_MOVES, row_bytes);
    const long long chunks = total_bytes / PULL_CHUNK + n_moves;
    const int grid = (int)std::max<long long>(1, std::min<long long>(chunks, (long long)sm_count(c.device) * 8));
    if (row_bytes % 16 == 0)
        moe_pull_rows_kernel<16><<<grid, 256, 0, c.stream>>>(moves, n_moves, bases, (uint8_t *)local, row_bytes, to_owner ? 1 : 0);
    else
        moe_pull_rows_kernel<4><<<grid, 256, 0, c.stream>>>(moves, n_moves, bases, (uint8_t *)local, row_bytes, to_owner ? 1 : 0);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// dst[s] = src[token_of[s]] (zeros for unused slots); rows of row_bytes (multiple of 16)
__global__ void moe_gather_rows_kernel(const uint8_t *__restrict__ src, const int *__restrict__ token_of, int rows, int row_bytes,
                                       uint8_t *__restrict__ dst)
{
    const int chunks = row_bytes / 16;
    const long long total = (long long)rows * chunks;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int s = (int)(i / chunks), ch = (int)(i % chunks);
        const int t = token_of[s];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t >= 0)
            v = *(const uint4 *)(src + (size_t)t * row_bytes + (size_t)ch * 16);
        *(uint4 *)(dst + (size_t)s * row_bytes + (size_t)ch * 16) = v;
    }
}

int moe_gather_rows(const Ctx &c, const void *src, const int *token_of, int rows, int row_bytes, void *dst)
{
    if (row_bytes % 16)
        return fail(TS2_ERR_INVALID_ARG, "moe_gather_rows: row size must be a multiple of 16 bytes");
    const long long total = (long long)rows * (row_bytes / 16);
    const int grid = (int)std::min<long long>(ceil_div(total, 256), (long long)sm_count(c.device) * 8);
    moe_gather_rows_kernel<<<std::max(grid, 1), 256, 0, c.stream>>>((const uint8_t *)src, token_of, rows, row_bytes, (uint8_t *)dst);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// cat [rows][2X] fp16 = [wide | gate] per slot -> what (normalized wide), wscale, rg = LoLU(gate, what) * weight_of[slot]
template <int FT>
__global__ void moe_act_forward_kernel(const __half *__restrict__ cat, const int *__restrict__ token_of,
                                       const float *__restrict__ weight_of, int rows, int X, float s_act, __half *__restrict__ what,
                                       float *__restrict__ wscale, void *__restrict__ rg)
{
    const int tiles = X / TILE;
    WARP_ITEM_LOOP((long long)rows * tiles)
    {
        const size_t s = item / tiles;
        const int tile = item % tiles, off = tile * TILE + lane * 4;
        if (token_of[s] < 0) {
            Fast<FT>::zero4(rg, s * X + off); // (the fp8x4 constructor mis-packs a constant zero vector)
            continue;
        }
        const float4 wide = load_half4(cat + s * 2 * X + off), gate = load_half4(cat + s * 2 * X + X + off);
        const float scale = tile_scale(warp_sum(dot4(wide, wide)));
        const float4 wn = scale4(wide, scale);
        store_half4(what + s * X + off, wn);
        if (lane == 0)
            wscale[s * tiles + tile] = scale;
        const float w = weight_of[s] * s_act;
        Fast<FT>::store4(rg, s * X + off,
                         make_float4(lolu_mult(gate.x) * wn.x * w, lolu_mult(gate.y) * wn.y * w, lolu_mult(gate.z) * wn.z * w,
                                     lolu_mult(gate.w) * wn.w * w));
    }
}

int moe_act_forward(const Ctx &c, const __half *cat, const int *token_of, const float *weight_of, int rows, int X, __half *what,
                    float *wscale, void *rg)
{
    const int grid = grid_for(c, (long long)rows * (X / TILE));
    if (c.ft == 0)
        moe_act_forward_kernel<0><<<grid, THREADS, 0, c.stream>>>(cat, token_of, weight_of, rows, X, c.s_act, what, wscale, rg);
    else
        moe_act_forward_kernel<1><<<grid, THREADS, 0, c.stream>>>(cat, token_of, weight_of, rows, X, c.s_act, what, wscale, rg);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// drg [rows][X] fp16 (gradient of the weighted rg) -> dcat [rows][2X] = [dwide | dgate], dmoe_part[rows][X/128] =
// per-tile sums of rgSrc * drg (the gradient of the routing weight, BackpropScaleExperts)
template <int FT>
__global__ void moe_act_backward_kernel(const __half *__restrict__ drg, const __half *__restrict__ cat, const __half *__restrict__ what,
                                        const float *__restrict__ wscale, const int *__restrict__ token_of,
                                        const float *__restrict__ weight_of, int rows, int X, void *__restrict__ dcat,
                                        float *__restrict__ dmoe_part)
{
    const int tiles = X / TILE;
    WARP_ITEM_LOOP((long long)rows * tiles)
    {
        const size_t s = item / tiles;
        const int tile = item % tiles, off = tile * TILE + lane * 4;
        if (token_of[s] < 0) {
            Fast<FT>::zero4(dcat, s * 2 * X + off);
            Fast<FT>::zero4(dcat, s * 2 * X + X + off);
            if (lane == 0)
                dmoe_part[s * tiles + tile] = 0.f;
            continue;
        }
        const float4 g0 = load_half4(drg + s * X + off), gate = load_half4(cat + s * 2 * X + X + off), wn = load_half4(what + s * X + off);
        const float sc = wscale[s * tiles + tile], w = weight_of[s];
        const float4 m = make_float4(lolu_mult(gate.x), lolu_mult(gate.y), lolu_mult(gate.z), lolu_mult(gate.w));
        // gradient of the routing weight: sum over the expert's columns of rgSrc * drg
        const float part = warp_sum(m.x * wn.x * g0.x + m.y * wn.y * g0.y + m.z * wn.z * g0.z + m.w * wn.w * g0.w);
        if (lane == 0)
            dmoe_part[s * tiles + tile] = part;
        const float4 g = scale4(g0, w); // gradient of the unweighted rgSrc
        const float4 dgate = make_float4(g.x * wn.x * m.x * (1 - m.x) * 2.f, g.y * wn.y * m.y * (1 - m.y) * 2.f,
                                         g.z * wn.z * m.z * (1 - m.z) * 2.f, g.w * wn.w * m.w * (1 - m.w) * 2.f);
        const float4 dwn = make_float4(g.x * m.x, g.y * m.y, g.z * m.z, g.w * m.w);
        const float proj = warp_sum(dot4(wn, dwn)) * (1.f / 128);
        Fast<FT>::store4(dcat, s * 2 * X + off,
                         make_float4(sc * (dwn.x - wn.x * proj), sc * (dwn.y - wn.y * proj), sc * (dwn.z - wn.z * proj),
                                     sc * (dwn.w - wn.w * proj)));
        Fast<FT>::store4(dcat, s * 2 * X + X + off, dgate);
    }
}

int moe_act_backward(const Ctx &c, const __half *drg, const __half *cat, const __half *what, const float *wscale, const int *token_of,
                     const float *weight_of, int rows, int X, void *dcat, float *dmoe_part)
{
    const int grid = grid_for(c, (long long)rows * (X / TILE));
    if (c.ft == 0)
        moe_act_backward_kernel<0><<<grid, THREADS, 0, c.stream>>>(drg, cat, what, wscale, token_of, weight_of, rows, X, dcat, dmoe_part);
    else
        moe_act_backward_kernel<1><<<grid, THREADS, 0, c.stream>>>(drg, cat, what, wscale, token_of, weight_of, rows, X, dcat, dmoe_part);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// out[t] = (in ? in[t] : out[t]) + sum over the token's choices of y[slot]   (fp32 rows of width D)
__global__ void moe_combine_kernel(const float *__restrict__ y, const int *__restrict__ slot_of, int T, int k, int D,
                                   const float *__restrict__ in, float *__restrict__ out)
{
    const int tiles = D / TILE;
    WARP_ITEM_LOOP((long long)T * tiles)
    {
        const size_t t = item / tiles;
        const int off = (item % tiles) * TILE + lane * 4;
        float4 acc = *(const float4 *)((in ? in : out) + t * D + off);
        for (int j = 0; j < k; ++j) {
            const float4 v = *(const float4 *)(y + (size_t)slot_of[t * k + j] * D + off);
            acc = make_float4(acc.x + v.x, acc.y + v.y, acc.z + v.z, acc.w + v.w);
        }
        *(float4 *)(out + t * D + off) = acc;
    }
}

// the same sum over fp16 rows (expert parallel: results come back from the experts' owners as fp16)
__global__ void moe_combine_half_kernel(const __half *__restrict__ y, const int *__restrict__ slot_of, int T, int k, int D,
                                        const float *__restrict__ in, float *__restrict__ out)
{
    const int tiles = D / TILE;
    WARP_ITEM_LOOP((long long)T * tiles)
    {
        const size_t t = item / tiles;
        const int off = (item % tiles) * TILE + lane * 4;
        float4 acc = *(const float4 *)((in ? in : out) + t * D + off);
        for (int j = 0; j < k; ++j) {
            const float4 v = load_half4(y + (size_t)slot_of[t * k + j] * D + off);
            acc = make_float4(acc.x + v.x, acc.y + v.y, acc.z + v.z, acc.w + v.w);
        }
        *(float4 *)(out + t * D + off) = acc;
    }
}

int moe_combine_half(const Ctx &c, const __half *y, const int *slot_of, int T, int k, int D, const float *in, float *out)
{
    moe_combine_half_kernel<<<grid_for(c, (long long)T * (D / TILE)), THREADS, 0, c.stream>>>(y, slot_of, T, k, D, in, out);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int moe_combine(const Ctx &c, const float *y, const int *slot_of, int T, int k, int D, const float *in, float *out)
{
    moe_combine_kernel<<<grid_for(c, (long long)T * (D / TILE)), THREADS, 0, c.stream>>>(y, slot_of, T, k, D, in, out);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------------
// router gradient (CpuBackpropMoe): with w~ = w / sqrt(E), g~ = dw * sqrt(E): dl = (w~ g~ - w~^2 sum(w~ g~)) / 2
// on the selected experts, 0 elsewhere; dl rows have pitch ld (padding zeroed)
template <int FT>
__global__ void moe_router_backward_kernel(const float *__restrict__ dmoe_part, int tiles, const int *__restrict__ ids,
                                           const float *__restrict__ weights, const int *__restrict__ slot_of, int T, int k, int E,
                                           int ld, void *__restrict__ dl)
{
    using QT = typename std::conditional<FT == 0, __nv_fp8_e4m3, __half>::type;
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T)
        return;
    QT *row = (QT *)dl + (size_t)t * ld;
    for (int x = 0; x < ld; ++x)
        row[x] = QT(0.f);
    const float root = sqrtf((float)E);
    float wt[8], gt[8], avrg = 0.f;
    for (int j = 0; j < k; ++j) {
        const int s = slot_of[(size_t)t * k + j];
        float d = 0.f;
        for (int i = 0; i < tiles; ++i)
            d += dmoe_part[(size_t)s * tiles + i];
        wt[j] = weights[(size_t)t * k + j] / root;
        gt[j] = d * root;
        avrg += wt[j] * gt[j];
    }
    for (int j = 0; j < k; ++j)
        row[ids[(size_t)t * k + j]] = QT((wt[j] * gt[j] - wt[j] * wt[j] * avrg) * 0.5f);
}

int moe_router_backward(const Ctx &c, const float *dmoe_part, int tiles, const int *ids, const float *weights, const int *slot_of, int T,
                        int k, int E, int ld, void *dl)
{
    if (c.ft == 0)
        moe_router_backward_kernel<0><<<(T + 127) / 128, 128, 0, c.stream>>>(dmoe_part, tiles, ids, weights, slot_of, T, k, E, ld, dl);
    else
        moe_router_backward_kernel<1><<<(T + 127) / 128, 128, 0, c.stream>>>(dmoe_part, tiles, ids, weights, slot_of, T, k, E, ld, dl);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

} // namespace ts2
