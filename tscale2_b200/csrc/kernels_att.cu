// Attention part of the training step: per-head normalisation + RoPE of Q/K/V and
// their backward, and the attention core over one inclusive key span per node
// (ComputeValLookup / GradQ / GradK, src/gpt/compute/layer_att_reference.h:41-212):
//   dp(from,to) = q_from . k_to * sqrt(1/128) * 0.5/ln2 - slope * (from - to)
//   weights 2^(dp - maxDP) with maxDP >= 0 and an extra zero vector of weight 2^-maxDP.
// This file holds the warp-per-row formulation (fp32 math, coalesced 8-byte loads), kept as an
// independent second formulation for the tests; the engine runs the tcgen05 kernels of
// kernels_att_tc.cu (kernels_att_mma.cu holds an mma.sync formulation, also kept for the tests).
#include "kernels.cuh"
#include "fast_types.cuh"

namespace ts2 {

static constexpr int WARPS = 8;
static constexpr int THREADS = WARPS * 32;

static int grid_for(const Ctx &c, long long warp_items)
{
    long long blocks = ceil_div(warp_items, WARPS);
    long long cap = (long long)sm_count(c.device) * 8;
    return (int)std::max<long long>(1, std::min(blocks, cap));
}

// for the grid-stride kernels that carry most of the bytes: exactly the blocks that are resident at once.  With a
// fixed 8 blocks per SM a kernel that fits 5 (48 registers) ran a second, partly filled wave at a fraction of the
// bandwidth.
template <typename K>
static int grid_for(const Ctx &c, K kernel, long long warp_items)
{
    long long blocks = ceil_div(warp_items, WARPS);
    long long cap = (long long)sm_count(c.device) * resident_blocks(c.device, (const void *)kernel, THREADS);
    return (int)std::max<long long>(1, std::min(blocks, cap));
}

#define WARP_BATCH_LOOP(total, R)                                                             \
    const int lane = threadIdx.x & 31;                                                        \
    const unsigned wstride = gridDim.x * WARPS, total_items = (unsigned)(total);             \
    for (unsigned base = blockIdx.x * WARPS + (threadIdx.x >> 5); base < total_items; base += wstride * (R))

#define WARP_ITEM_LOOP(total) \
    const int lane = threadIdx.x & 31; \
    for (unsigned item = blockIdx.x * WARPS + (threadIdx.x >> 5), total_items = (unsigned)(total); item < total_items; \
         item += gridDim.x * WARPS)

// AttDotScale = CalcDotScale(128) * ATT_DOTPRODUCT_SCALE / LOG2 (layer_att_reference.h:30-33)
__host__ __device__ inline float att_dot_scale() { return sqrtf(1.0f / 128) * (0.5f / 0.693147f) * 1.0f; }

// rope[t][2i] = cos(t * theta^(-2i/128)), rope[t][2i+1] = sin(...)   (TRopeComputer, src/gpt/att/rope.cpp:4-24)
__global__ void fill_rope_kernel(float *__restrict__ rope, int T)
{
    const long long total = (long long)T * 64;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / 64), k = (int)(i % 64);
        const float freq = (float)exp(-log(500000.0) * (k * 2. / 128));
        const float angle = (float)t * freq;
        rope[(size_t)t * 128 + 2 * k] = (float)cos((double)angle);
        rope[(size_t)t * 128 + 2 * k + 1] = (float)sin((double)angle);
    }
}

int fill_rope(const Ctx &c, float *rope, int T)
{
    fill_rope_kernel<<<std::max(1, std::min(T, 1024)), 64, 0, c.stream>>>(rope, T);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

__device__ __forceinline__ float4 rope_apply(float4 v, float4 cs, float dir)
{
    // pairs (0,1) and (2,3) of the lane's four elements; cs = (cos0, sin0, cos1, sin1)
    const float s0 = cs.y * dir, s1 = cs.w * dir;
    return make_float4(v.x * cs.x - v.y * s0, v.x * s0 + v.y * cs.x, v.z * cs.z - v.w * s1, v.z * s1 + v.w * cs.z);
}

__global__ void att_post_forward_kernel(const __half *__restrict__ qkvg, const float *__restrict__ rope, int T, int H,
                                        __half *__restrict__ q, __half *__restrict__ k, __half *__restrict__ v,
                                        float *__restrict__ qscale, float *__restrict__ vscale)
{
    const int Q = H * TILE;
    constexpr int R = 2; // two (node, head) items in flight per warp
    WARP_BATCH_LOOP((long long)T * H, R)
    {
        float4 qs[R], ks[R], vs[R], cs[R];
        size_t t[R];
        int h[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / H : 0;
            h[r] = ok[r] ? (int)(item % H) : 0;
            const __half *src = qkvg + t[r] * 4 * Q + h[r] * TILE + lane * 4;
            qs[r] = ok[r] ? load_half4(src) : make_float4(0, 0, 0, 0);
            ks[r] = ok[r] ? load_half4(src + Q) : make_float4(0, 0, 0, 0);
            vs[r] = ok[r] ? load_half4(src + 2 * Q) : make_float4(0, 0, 0, 0);
            cs[r] = ok[r] ? *(const float4 *)(rope + t[r] * 128 + lane * 4) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            const int off = h[r] * TILE + lane * 4;
            const float sq = tile_scale(warp_sum(dot4(qs[r], qs[r]))), sv = tile_scale(warp_sum(dot4(vs[r], vs[r])));
            store_half4(q + t[r] * Q + off, rope_apply(scale4(qs[r], sq), cs[r], 1.f));
            store_half4(k + t[r] * Q + off, rope_apply(ks[r], cs[r], 1.f));
            store_half4(v + t[r] * Q + off, scale4(vs[r], sv));
            if (lane == 0) {
                qscale[t[r] * H + h[r]] = sq;
                vscale[t[r] * H + h[r]] = sv;
            }
        }
    }
}

int att_post_forward(const Ctx &c, const __half *qkvg, const float *rope, int T, int H, __half *q, __half *k, __half *v, float *qscale,
                     float *vscale)
{
    att_post_forward_kernel<<<grid_for(c, att_post_forward_kernel, (long long)T * H), THREADS, 0, c.stream>>>(qkvg, rope, T, H, q, k, v, qscale, vscale);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// GT: type of the incoming gradients (float or __half)
template <typename GT>
__device__ __forceinline__ float4 load_grad4(const GT *p);
template <>
__device__ __forceinline__ float4 load_grad4<float>(const float *p)
{
    return *(const float4 *)p;
}
template <>
__device__ __forceinline__ float4 load_grad4<__half>(const __half *p)
{
    return load_half4(p);
}

template <int FT, typename GT>
__global__ void att_post_backward_kernel(const GT *__restrict__ dq, const GT *__restrict__ dk, const GT *__restrict__ dv,
                                         const __half *__restrict__ q, const __half *__restrict__ v, const float *__restrict__ qscale,
                                         const float *__restrict__ vscale, const float *__restrict__ rope,
                                         const float *__restrict__ sko_k, int T, int H, void *__restrict__ d4)
{
    const int Q = H * TILE;
    const float kfold = __ldg(sko_k);
    constexpr int R = 2;
    WARP_BATCH_LOOP((long long)T * H, R)
    {
        float4 cs[R], qv[R], gq[R], gk[R], vv[R], gv[R];
        float sq[R], sv[R];
        size_t t[R];
        int off[R];
        bool ok[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned item = base + r * wstride;
            ok[r] = item < total_items;
            t[r] = ok[r] ? item / H : 0;
            const int h = ok[r] ? (int)(item % H) : 0;
            off[r] = h * TILE + lane * 4;
            const float4 z = make_float4(0, 0, 0, 0);
            cs[r] = ok[r] ? *(const float4 *)(rope + t[r] * 128 + lane * 4) : z;
            qv[r] = ok[r] ? load_half4(q + t[r] * Q + off[r]) : z;
            gq[r] = ok[r] ? load_grad4<GT>(dq + t[r] * Q + off[r]) : z;
            gk[r] = ok[r] ? load_grad4<GT>(dk + t[r] * Q + off[r]) : z;
            vv[r] = ok[r] ? load_half4(v + t[r] * Q + off[r]) : z;
            gv[r] = ok[r] ? load_grad4<GT>(dv + t[r] * Q + off[r]) : z;
            sq[r] = ok[r] ? qscale[t[r] * H + h] : 0.f;
            sv[r] = ok[r] ? vscale[t[r] * H + h] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (!ok[r])
                continue;
            // q: tile-norm backward in the rotated frame (the rotation is orthogonal), then rotate back
            const float pq = warp_sum(dot4(qv[r], gq[r])) * (1.f / 128);
            const float4 rq = rope_apply(
                make_float4(gq[r].x - qv[r].x * pq, gq[r].y - qv[r].y * pq, gq[r].z - qv[r].z * pq, gq[r].w - qv[r].w * pq), cs[r], -1.f);
            Fast<FT>::store4(d4, t[r] * 4 * Q + off[r], scale4(rq, sq[r]));
            // k: rotate back; the matrix scale of K is folded in here so that the 4-way dX contraction
            // can use scale-free weights for every block
            Fast<FT>::store4(d4, t[r] * 4 * Q + Q + off[r], scale4(rope_apply(gk[r], cs[r], -1.f), kfold));
            // v: tile-norm backward
            const float pv = warp_sum(dot4(vv[r], gv[r])) * (1.f / 128);
            Fast<FT>::store4(d4, t[r] * 4 * Q + 2 * Q + off[r],
                             make_float4(sv[r] * (gv[r].x - vv[r].x * pv), sv[r] * (gv[r].y - vv[r].y * pv),
                                         sv[r] * (gv[r].z - vv[r].z * pv), sv[r] * (gv[r].w - vv[r].w * pv)));
        }
    }
}

int att_post_backward(const Ctx &c, const void *dq, const void *dk, const void *dv, bool grads16, const __half *q, const __half *v,
                      const float *qscale, const float *vscale, const float *rope, const float *sko_k, int T, int H, void *d4)
{
#define TS2_POST_BWD(FT_, GT_)                                                                                          \
    att_post_backward_kernel<FT_, GT_><<<grid_for(c, att_post_backward_kernel<FT_, GT_>, (long long)T * H), THREADS, 0, \
                                         c.stream>>>((const GT_ *)dq, (const GT_ *)dk, (const GT_ *)dv, q, v, qscale, vscale, \
                                                     rope, sko_k, T, H, d4)
    if (c.ft == 0 && grads16)
        TS2_POST_BWD(0, __half);
    else if (c.ft == 0)
        TS2_POST_BWD(0, float);
    else if (grads16)
        TS2_POST_BWD(1, __half);
    else
        TS2_POST_BWD(1, float);
#undef TS2_POST_BWD
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

// ---------------------------------------------------------------------------------
// attention core, one warp per (node, head)

__global__ void attention_forward_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                                         const int *__restrict__ span_start, const int *__restrict__ span_finish, int T, int H,
                                         float slope, __half *__restrict__ o, float *__restrict__ lse)
{
    const int Q = H * TILE;
    const float ds = att_dot_scale();
    WARP_ITEM_LOOP((long long)T * H)
    {
        const int t = (int)(item / H), h = (int)(item % H), off = h * TILE + lane * 4;
        const float4 qv = load_half4(q + (size_t)t * Q + off);
        float m = 0.f, S = 1.f; // running maximum (never below 0) and sum, including the zero vector of weight 2^-m
        float4 acc = make_float4(0, 0, 0, 0);
        const int s0 = span_start[t], s1 = span_finish[t];
        for (int to = s0; to <= s1; ++to) {
            const float4 kv = load_half4(k + (size_t)to * Q + off);
            const float dp = warp_sum(dot4(qv, kv)) * ds - slope * (float)(t - to);
            if (dp > m) {
                const float r = exp2f(m - dp);
                S *= r;
                acc = scale4(acc, r);
                m = dp;
            }
            const float w = exp2f(dp - m);
            S += w;
            acc = axpy4(w, load_half4(v + (size_t)to * Q + off), acc);
        }
        store_half4(o + (size_t)t * Q + off, scale4(acc, 1.f / S));
        if (lane == 0)
            lse[(size_t)t * H + h] = m + log2f(S);
    }
}

int attention_forward_rowwise(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start,
                              const int *span_finish, int T, int H, float slope, __half *o, float *lse)
{
    attention_forward_kernel<<<grid_for(c, (long long)T * H), THREADS, 0, c.stream>>>(q, k, v, span_start, span_finish, T, H, slope, o, lse);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

__global__ void attention_dq_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                                    const __half *__restrict__ dout, const float *__restrict__ lse, const float *__restrict__ dscale,
                                    const int *__restrict__ span_start, const int *__restrict__ span_finish, int T, int H, float slope,
                                    float *__restrict__ dq)
{
    const int Q = H * TILE;
    const float ds = att_dot_scale(), c2 = ds * 0.693147f;
    WARP_ITEM_LOOP((long long)T * H)
    {
        const int t = (int)(item / H), h = (int)(item % H), off = h * TILE + lane * 4;
        const float4 qv = load_half4(q + (size_t)t * Q + off), dov = load_half4(dout + (size_t)t * Q + off);
        const float l = lse[(size_t)t * H + h], dsc = dscale[(size_t)t * H + h];
        float4 acc = make_float4(0, 0, 0, 0);
        const int s0 = span_start[t], s1 = span_finish[t];
        for (int to = s0; to <= s1; ++to) {
            const float4 kv = load_half4(k + (size_t)to * Q + off), vv = load_half4(v + (size_t)to * Q + off);
            const float dp = warp_sum(dot4(qv, kv)) * ds - slope * (float)(t - to);
            const float w = exp2f(dp - l);
            const float dW = warp_sum(dot4(dov, vv));
            acc = axpy4(w * (dW - dsc) * c2, kv, acc);
        }
        *(float4 *)(dq + (size_t)t * Q + off) = acc;
    }
}

__global__ void attention_dkv_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                                     const __half *__restrict__ dout, const float *__restrict__ lse, const float *__restrict__ dscale,
                                     const int *__restrict__ span_start, const int *__restrict__ span_finish,
                                     const int *__restrict__ rev_first, const int *__restrict__ rev_last, int T, int H, float slope,
                                     float *__restrict__ dk, float *__restrict__ dv)
{
    const int Q = H * TILE;
    const float ds = att_dot_scale(), c2 = ds * 0.693147f;
    WARP_ITEM_LOOP((long long)T * H)
    {
        const int to = (int)(item / H), h = (int)(item % H), off = h * TILE + lane * 4;
        const float4 kv = load_half4(k + (size_t)to * Q + off), vv = load_half4(v + (size_t)to * Q + off);
        float4 ak = make_float4(0, 0, 0, 0), av = make_float4(0, 0, 0, 0);
        const int f0 = rev_first[to], f1 = rev_last[to];
        for (int t = f0; t <= f1; ++t) {
            if (span_start[t] > to || span_finish[t] < to)
                continue;
            const float4 qv = load_half4(q + (size_t)t * Q + off), dov = load_half4(dout + (size_t)t * Q + off);
            const float dp = warp_sum(dot4(qv, kv)) * ds - slope * (float)(t - to);
            const float w = exp2f(dp - lse[(size_t)t * H + h]);
            const float dW = warp_sum(dot4(dov, vv));
            ak = axpy4(w * (dW - dscale[(size_t)t * H + h]) * c2, qv, ak);
            av = axpy4(w, dov, av);
        }
        *(float4 *)(dk + (size_t)to * Q + off) = ak;
        *(float4 *)(dv + (size_t)to * Q + off) = av;
    }
}

int attention_backward_rowwise(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                               const float *dscale, const int *span_start, const int *span_finish, const int *rev_first,
                               const int *rev_last, int T, int H, float slope, float *dq, float *dk, float *dv)
{
    const int grid = grid_for(c, (long long)T * H);
    attention_dq_kernel<<<grid, THREADS, 0, c.stream>>>(q, k, v, dout, lse, dscale, span_start, span_finish, T, H, slope, dq);
    TS2_CHECK_LAUNCH();
    attention_dkv_kernel<<<grid, THREADS, 0, c.stream>>>(q, k, v, dout, lse, dscale, span_start, span_finish, rev_first, rev_last, T, H,
                                                         slope, dk, dv);
    TS2_CHECK_LAUNCH();
    return TS2_OK;
}

int attention_forward(const Ctx &c, const __half *q, const __half *k, const __half *v, const int *span_start, const int *span_finish,
                      int T, int H, float slope, __half *o, float *lse)
{
    return attention_forward_tc(c, q, k, v, span_start, span_finish, T, H, slope, o, lse);
}

int attention_backward(const Ctx &c, const __half *q, const __half *k, const __half *v, const __half *dout, const float *lse,
                       const float *dscale, const int *span_start, const int *span_finish, const int *rev_first, const int *rev_last,
                       int T, int H, float slope, void *dq, void *dk, void *dv, bool grads16)
{
    return attention_backward_tc(c, q, k, v, dout, lse, dscale, span_start, span_finish, rev_first, rev_last, T, H, slope, dq, dk, dv,
                                 grads16);
}

} // namespace ts2
