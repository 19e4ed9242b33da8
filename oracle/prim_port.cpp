// TEST INFRASTRUCTURE — restatement of the reference CPU primitives in plain
// C++.  Summation order follows the reference loops so that results agree
// with prim_ref.cpp to rounding; OpenMP only splits loops whose iterations
// write disjoint outputs (OMP_NUM_THREADS=1 gives the scalar reference timing).  See prim.h for the citations.
#include "prim.h"
#include <cmath>
#include <cstring>
#include <algorithm>

namespace ts2o {
namespace prim {

static const float kLog2 = 0.693147f;          // LOG2, model_dim.h:16
static const float kAttDotProductScale = 0.5f; // ATT_DOTPRODUCT_SCALE, model_dim.h:18
static const float kLoluScale = 2.f;           // LOLU_SCALE, model_dim.h:21

const char *BackendName() { return "port"; }

static inline float DotScale(int n) { return sqrtf(1.0f / n); } // CalcDotScale, model_dim.h:23

Mat MulForward(const Mat &x, const Mat &w)
{
    const int T = x.rows, in = x.cols, out = w.rows;
    Mat y(T, out);
    const float s = DotScale(in);
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float *xr = x.row(t);
        float *yr = y.row(t);
        for (int o = 0; o < out; ++o) {
            const float *wr = w.row(o);
            float acc = 0;
            for (int i = 0; i < in; ++i)
                acc += xr[i] * wr[i];
            yr[o] = acc * s;
        }
    }
    return y;
}

void MulBackwardWithAccum(Mat *dx, const Mat &w, const Mat &dy)
{
    const int T = dy.rows, in = w.cols, out = dy.cols;
    const float s = DotScale(in);
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float *g = dy.row(t);
        float *d = dx->row(t);
        for (int i = 0; i < in; ++i) {
            float acc = 0;
            for (int o = 0; o < out; ++o)
                acc += g[o] * w.v[(size_t)o * in + i];
            d[i] += acc * s;
        }
    }
}

void SumRankOne(const Mat &x, Mat *delta, const Mat &dy)
{
    const int T = x.rows, in = x.cols, out = dy.cols;
    delta->resize(out, in);
#pragma omp parallel for schedule(static)
    for (int o = 0; o < out; ++o) {
        float *dr = delta->row(o);
        for (int i = 0; i < in; ++i) {
            float acc = 0;
            for (int t = 0; t < T; ++t)
                acc += dy.v[(size_t)t * out + o] * x.v[(size_t)t * in + i];
            dr[i] += acc;
        }
    }
}

Mat NormalizeState(const Mat &state, int headCount)
{
    const int T = state.rows, dim = state.cols, hd = dim / headCount;
    Mat res(T, dim);
    for (int t = 0; t < T; ++t) {
        for (int h = 0; h < headCount; ++h) {
            const float *src = state.row(t) + h * hd;
            float *dst = res.row(t) + h * hd;
            float sum2 = 0;
            for (int i = 0; i < hd; ++i)
                sum2 += src[i] * src[i];
            if (sum2 == 0) {
                for (int i = 0; i < hd; ++i)
                    dst[i] = 0;
            } else {
                float scale = sqrt(hd / sum2);
                for (int i = 0; i < hd; ++i)
                    dst[i] = src[i] * scale;
            }
        }
    }
    return res;
}

void NormalizeStateBackward(const Mat &state, int headCount, const Mat &dnorm, Mat *grad)
{
    const int T = state.rows, dim = state.cols, hd = dim / headCount;
    if (grad->rows != T || grad->cols != dim)
        grad->resize(T, dim);
    for (int t = 0; t < T; ++t) {
        for (int h = 0; h < headCount; ++h) {
            const float *src = state.row(t) + h * hd;
            const float *g = dnorm.row(t) + h * hd;
            float *dst = grad->row(t) + h * hd;
            float sum2 = 0, dp = 0;
            for (int i = 0; i < hd; ++i) {
                sum2 += src[i] * src[i];
                dp += src[i] * g[i];
            }
            if (sum2 == 0) {
                for (int i = 0; i < hd; ++i)
                    dst[i] = 0;
            } else {
                float sigma = dp / sum2;
                float scale = sqrt(hd / sum2);
                for (int i = 0; i < hd; ++i)
                    dst[i] = scale * (g[i] - src[i] * sigma);
            }
        }
    }
}

static inline float LoluMult(float gate)
{
    float arg = gate * kLoluScale;
    if (arg < -20)
        return 0;
    if (arg > 20)
        return 1;
    float w = expf(arg);
    return w / (1 + w);
}

void LoLU(const Mat &gate, const Mat &vals, Mat *out)
{
    out->resize(vals.rows, vals.cols);
    for (size_t i = 0; i < vals.v.size(); ++i)
        out->v[i] = LoluMult(gate.v[i]) * vals.v[i];
}

void BackpropLoLU(const Mat &gate, const Mat &vals, const Mat &grad, Mat *gradGate, Mat *gradVals)
{
    gradGate->resize(vals.rows, vals.cols);
    gradVals->resize(vals.rows, vals.cols);
    for (size_t i = 0; i < vals.v.size(); ++i) {
        float m = LoluMult(gate.v[i]);
        gradGate->v[i] = grad.v[i] * vals.v[i] * m * (1 - m) * kLoluScale;
        gradVals->v[i] = grad.v[i] * m;
    }
}

void FillRopeBuf(Mat *rope, int width, int len)
{
    const float theta = 500000;
    std::vector<float> freq;
    for (int k = 0; k < width / 2; ++k)
        freq.push_back(exp(-log(theta) * (k * 2. / width)));
    rope->resize(len, width);
    for (int t = 0; t < len; ++t) {
        float *buf = rope->row(t);
        for (int k = 0; k < width; k += 2) {
            float angle = t * freq[k / 2];
            buf[k] = cos(angle);
            buf[k + 1] = sin(angle);
        }
    }
}

void ApplyRope(const Mat &rope, float dir, Mat *p)
{
    const int hs = rope.cols;
    for (int t = 0; t < p->rows; ++t) {
        const float *rb = rope.row(t);
        float *vec = p->row(t);
        for (int off = 0; off < p->cols; off += hs) {
            for (int k = 0; k < hs; k += 2) {
                float c = rb[k], s = rb[k + 1] * dir;
                float a = vec[off + k], b = vec[off + k + 1];
                vec[off + k] = a * c - b * s;
                vec[off + k + 1] = a * s + b * c;
            }
        }
    }
}

AttInfo TransposeAttention(const AttInfo &att)
{
    AttInfo res;
    if (att.ptr.size() <= 1)
        return res;
    const int n = (int)att.ptr.size() - 1;
    std::vector<std::vector<std::pair<int, int>>> rev(n);
    for (int from = 0; from < n; ++from) {
        for (int s = att.ptr[from]; s < att.ptr[from + 1]; ++s) {
            for (int to = att.start[s]; to <= att.finish[s]; ++to) {
                auto &dst = rev[to];
                if (!dst.empty() && dst.back().second == from - 1)
                    dst.back().second = from;
                else
                    dst.push_back({from, from});
            }
        }
    }
    res.ptr.push_back(0);
    for (int to = 0; to < n; ++to) {
        for (auto &sp : rev[to]) {
            res.start.push_back(sp.first);
            res.finish.push_back(sp.second);
        }
        res.ptr.push_back((int)res.start.size());
    }
    return res;
}

void Attention::Init(int headCount_, int qDim_, int ttDim_, float alibiSlope_)
{
    headCount = headCount_;
    qDim = qDim_;
    ttDim = ttDim_;
    alibiSlope = alibiSlope_;
    dotScale = DotScale(qDim) * (kAttDotProductScale / kLog2) * 1.0f;
}

static inline float CalcDP(const Attention &a, const Mat &q, const Mat &k, int qOff, int from, int to)
{
    const float *qr = q.row(from) + qOff, *kr = k.row(to) + qOff;
    float sum = 0;
    for (int x = 0; x < a.qDim; ++x)
        sum += qr[x] * kr[x];
    float dp = sum * a.dotScale;
    dp += -(a.alibiSlope) * (from - to);
    return dp;
}

void Attention::ComputeValLookup(const Mat &q, const Mat &k, const Mat &v, const AttInfo &att, Mat *valLookup)
{
    const int len = q.rows;
    valLookup->resize(len, ttDim * headCount);
    sumWeight.resize(headCount, len);
    maxDP.resize(headCount, len);
    for (int head = 0; head < headCount; ++head) {
        const int qOff = head * qDim, ttOff = head * ttDim;
#pragma omp parallel for schedule(dynamic, 16)
        for (int from = 0; from < len; ++from) {
            std::vector<float> acc(ttDim);
            float mx = 0;
            for (int s = att.ptr[from]; s < att.ptr[from + 1]; ++s)
                for (int to = att.start[s]; to <= att.finish[s]; ++to)
                    mx = fmaxf(mx, CalcDP(*this, q, k, qOff, from, to));
            float sw = exp2(-mx); // zero vector of weight 1
            std::fill(acc.begin(), acc.end(), 0.f);
            for (int s = att.ptr[from]; s < att.ptr[from + 1]; ++s) {
                for (int to = att.start[s]; to <= att.finish[s]; ++to) {
                    float dp = CalcDP(*this, q, k, qOff, from, to);
                    float w = exp2(dp - mx);
                    sw += w;
                    const float *vr = v.row(to) + ttOff;
                    for (int x = 0; x < ttDim; ++x)
                        acc[x] += w * vr[x];
                }
            }
            sumWeight.row(head)[from] = sw;
            maxDP.row(head)[from] = mx;
            float inv = 1 / sw;
            float *dst = valLookup->row(from) + ttOff;
            for (int x = 0; x < ttDim; ++x)
                dst[x] = acc[x] * inv;
        }
    }
}

static inline float CalcDDot(const Attention &a, const Mat &v, const Mat &dVal, const Mat &dScale, int head, int ttOff, int from,
                             int to, float dp, float mx, float sw)
{
    float w = exp2(dp - mx) / sw;
    const float *dv = dVal.row(from) + ttOff, *vr = v.row(to) + ttOff;
    float dW = 0;
    for (int x = 0; x < a.ttDim; ++x)
        dW += dv[x] * vr[x];
    float ds = dScale.row(head)[from];
    return w * (dW - ds) * a.dotScale * kLog2;
}

void Attention::GradQ(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &att, Mat *dq)
{
    const int len = q.rows;
    dq->resize(len, qDim * headCount);
    for (int head = 0; head < headCount; ++head) {
        const int qOff = head * qDim, ttOff = head * ttDim;
#pragma omp parallel for schedule(dynamic, 16)
        for (int from = 0; from < len; ++from) {
            for (int s = att.ptr[from]; s < att.ptr[from + 1]; ++s) {
                float sw = sumWeight.row(head)[from], mx = maxDP.row(head)[from];
                for (int to = att.start[s]; to <= att.finish[s]; ++to) {
                    float dp = CalcDP(*this, q, k, qOff, from, to);
                    float dDot = CalcDDot(*this, v, dValLookup, dScale, head, ttOff, from, to, dp, mx, sw);
                    float *dst = dq->row(from) + qOff;
                    const float *kr = k.row(to) + qOff;
                    for (int x = 0; x < qDim; ++x)
                        dst[x] += dDot * kr[x];
                }
            }
        }
    }
}

void Attention::GradK(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &revAtt,
                      Mat *dk, Mat *dv)
{
    const int len = q.rows;
    dk->resize(len, qDim * headCount);
    dv->resize(len, ttDim * headCount);
    for (int head = 0; head < headCount; ++head) {
        const int qOff = head * qDim, ttOff = head * ttDim;
#pragma omp parallel for schedule(dynamic, 16)
        for (int to = 0; to < len; ++to) {
            for (int s = revAtt.ptr[to]; s < revAtt.ptr[to + 1]; ++s) {
                for (int from = revAtt.start[s]; from <= revAtt.finish[s]; ++from) {
                    float sw = sumWeight.row(head)[from], mx = maxDP.row(head)[from];
                    float dp = CalcDP(*this, q, k, qOff, from, to);
                    float dDot = CalcDDot(*this, v, dValLookup, dScale, head, ttOff, from, to, dp, mx, sw);
                    float w = exp2(dp - mx) / sw;
                    float *dkr = dk->row(to) + qOff;
                    const float *qr = q.row(from) + qOff;
                    for (int x = 0; x < qDim; ++x)
                        dkr[x] += dDot * qr[x];
                    float *dvr = dv->row(to) + ttOff;
                    const float *dvl = dValLookup.row(from) + ttOff;
                    for (int x = 0; x < ttDim; ++x)
                        dvr[x] += w * dvl[x];
                }
            }
        }
    }
}

void ComputeDScale(int headCount, int ttDim, const Mat &valLookup, const Mat &dValLookup, Mat *dScale)
{
    const int len = valLookup.rows;
    dScale->resize(headCount, len);
    for (int t = 0; t < len; ++t)
        for (int k = 0; k < ttDim * headCount; ++k)
            dScale->row(k / ttDim)[t] += dValLookup.row(t)[k] * valLookup.row(t)[k];
}

} // namespace prim
} // namespace ts2o
