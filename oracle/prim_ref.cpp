// TEST INFRASTRUCTURE — the prim.h interface implemented by calling the
// reference's own compiled CPU functions (src/gpt/compute/cpu_util.cpp,
// src/gpt/compute/layer_att_reference.h, src/gpt/att/rope.cpp,
// src/gpt/att/att.cpp).  Built only where the reference source tree is
// present; the object files go to oracle/_ref/.  Matrices are copied into and
// out of the reference's TArray2D at every call.
//
// compile: g++ -std=c++17 -include util/pch.h -I<reference>/src ...
#include <gpt/compute/cpu_util.h>
#include <gpt/compute/layer_att_reference.h>
#include <gpt/att/rope.h>
#include <gpt/att/att.h>
#include <gpt/model_params/model_dim.h>
#include "prim.h"

namespace ts2o {
namespace prim {

const char *BackendName() { return "reference"; }

static TArray2D<float> ToRef(const Mat &m)
{
    TArray2D<float> r;
    r.SetSizes(m.cols, m.rows);
    for (int y = 0; y < m.rows; ++y)
        memcpy(r.GetRow(y), m.row(y), sizeof(float) * m.cols);
    return r;
}

static void FromRef(const TArray2D<float> &r, Mat *m)
{
    m->rows = (int)r.GetYSize();
    m->cols = (int)r.GetXSize();
    m->v.resize((size_t)m->rows * m->cols);
    for (int y = 0; y < m->rows; ++y)
        memcpy(m->row(y), r.GetRow(y), sizeof(float) * m->cols);
}

static TAttentionInfo ToRef(const AttInfo &a)
{
    TAttentionInfo r;
    r.SpanPtr.resize(0);
    for (int p : a.ptr)
        r.SpanPtr.push_back(p);
    for (size_t i = 0; i < a.start.size(); ++i)
        r.Spans.push_back(TAttentionSpan(a.start[i], a.finish[i]));
    return r;
}

static TModelDims Dims(int headCount, int qDim, int ttDim)
{
    TModelDims d;
    d.HeadCount = headCount;
    d.QDim = qDim;
    d.TTDim = ttDim;
    return d;
}

Mat MulForward(const Mat &x, const Mat &w)
{
    Mat y;
    FromRef(::MulForward(ToRef(x), ToRef(w)), &y);
    return y;
}

void MulBackwardWithAccum(Mat *dx, const Mat &w, const Mat &dy)
{
    TArray2D<float> d = ToRef(*dx);
    ::MulBackwardWithAccum(&d, ToRef(w), ToRef(dy));
    FromRef(d, dx);
}

void SumRankOne(const Mat &x, Mat *delta, const Mat &dy)
{
    TArray2D<float> d;
    ::SumRankOne(ToRef(x), &d, ToRef(dy));
    FromRef(d, delta);
}

Mat NormalizeState(const Mat &state, int headCount)
{
    Mat r;
    FromRef(::NormalizeState(ToRef(state), headCount), &r);
    return r;
}

void NormalizeStateBackward(const Mat &state, int headCount, const Mat &dnorm, Mat *grad)
{
    TArray2D<float> g;
    ::NormalizeStateBackward(ToRef(state), headCount, ToRef(dnorm), &g);
    FromRef(g, grad);
}

void LoLU(const Mat &gate, const Mat &vals, Mat *out)
{
    TArray2D<float> r;
    ::LoLU(ToRef(gate), ToRef(vals), &r);
    FromRef(r, out);
}

void BackpropLoLU(const Mat &gate, const Mat &vals, const Mat &grad, Mat *gradGate, Mat *gradVals)
{
    TArray2D<float> gg, gv;
    ::BackpropLoLU(ToRef(gate), ToRef(vals), ToRef(grad), &gg, &gv);
    FromRef(gg, gradGate);
    FromRef(gv, gradVals);
}

void FillRopeBuf(Mat *rope, int width, int len)
{
    TArray2D<float> r;
    ::FillRopeBuf(&r, width, (yint)len);
    FromRef(r, rope);
}

void ApplyRope(const Mat &rope, float dir, Mat *p)
{
    TArray2D<float> r = ToRef(*p);
    ::ApplyRope(ToRef(rope), dir, &r);
    FromRef(r, p);
}

AttInfo TransposeAttention(const AttInfo &att)
{
    TAttentionInfo r = ::TransposeAttention(ToRef(att));
    AttInfo res;
    for (yint i = 0; i < YSize(r.SpanPtr); ++i)
        res.ptr.push_back(r.SpanPtr[i]);
    for (yint i = 0; i < YSize(r.Spans); ++i) {
        res.start.push_back(r.Spans[i].Start);
        res.finish.push_back(r.Spans[i].Finish);
    }
    return res;
}

void Attention::Init(int headCount_, int qDim_, int ttDim_, float alibiSlope_)
{
    headCount = headCount_;
    qDim = qDim_;
    ttDim = ttDim_;
    alibiSlope = alibiSlope_;
    TAttentionComputer c(Dims(headCount, qDim, ttDim), alibiSlope, 1.0f);
    dotScale = c.AttDotScale;
}

void Attention::ComputeValLookup(const Mat &q, const Mat &k, const Mat &v, const AttInfo &att, Mat *valLookup)
{
    TModelDims dims = Dims(headCount, qDim, ttDim);
    TAttentionComputer c(dims, alibiSlope, 1.0f);
    TArray2D<float> res;
    c.ComputeValLookup(q.rows, dims, ToRef(q), ToRef(k), ToRef(v), ToRef(att), &res);
    FromRef(res, valLookup);
    FromRef(c.SumWeight, &sumWeight);
    FromRef(c.MaxDP, &maxDP);
}

void Attention::GradQ(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &att, Mat *dq)
{
    TModelDims dims = Dims(headCount, qDim, ttDim);
    TAttentionComputer c(dims, alibiSlope, 1.0f);
    c.SumWeight = ToRef(sumWeight);
    c.MaxDP = ToRef(maxDP);
    TArray2D<float> rq = ToRef(q), rk = ToRef(k), rv = ToRef(v), rdv = ToRef(dValLookup), rds = ToRef(dScale);
    TAttentionComputer::TGradData data(dims, rq, rk, rv, rdv, rds);
    TArray2D<float> res;
    c.GradQ(q.rows, dims, data, ToRef(att), &res);
    FromRef(res, dq);
}

void Attention::GradK(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &revAtt,
                      Mat *dk, Mat *dv)
{
    TModelDims dims = Dims(headCount, qDim, ttDim);
    TAttentionComputer c(dims, alibiSlope, 1.0f);
    c.SumWeight = ToRef(sumWeight);
    c.MaxDP = ToRef(maxDP);
    TArray2D<float> rq = ToRef(q), rk = ToRef(k), rv = ToRef(v), rdv = ToRef(dValLookup), rds = ToRef(dScale);
    TAttentionComputer::TGradData data(dims, rq, rk, rv, rdv, rds);
    TArray2D<float> rdk, rdvv;
    c.GradK(q.rows, dims, data, ToRef(revAtt), &rdk, &rdvv);
    FromRef(rdk, dk);
    FromRef(rdvv, dv);
}

void ComputeDScale(int headCount, int ttDim, const Mat &valLookup, const Mat &dValLookup, Mat *dScale)
{
    TModelDims dims = Dims(headCount, ttDim, ttDim);
    TArray2D<float> r;
    ::ComputeDScale(dims, ToRef(valLookup), ToRef(dValLookup), &r);
    FromRef(r, dScale);
}

} // namespace prim
} // namespace ts2o

// ---------------------------------------------------------------------------
// reference number-format conversions, exported from the reference build only
// so that the scalar restatements in ts2_oracle.cpp can be pinned against them.
#include <gpt/model_params/sse_utils.h>

extern "C" {
// ConvertToFp8e4m3, src/gpt/model_params/sse_utils.h:161-204 (n multiple of 8, src 32-byte aligned)
void ts2o_ref_convert_e4m3(uint8_t *dst, const float *src, int64_t n, float mult)
{
    ConvertToFp8e4m3((e4m3 *)dst, src, n, _mm256_set1_ps(mult));
}
// ConvertArray, src/gpt/model_params/sse_utils.h:73-78 (n multiple of 32)
void ts2o_ref_convert_i8(int8_t *dst, const float *src, int64_t n, float mult)
{
    ConvertArray((i8 *)dst, src, n, _mm256_set1_ps(mult));
}
// ConvertE4toFloat, src/util/fp8.h:4-22
float ts2o_ref_e4m3_to_float(uint8_t x) { return ConvertE4toFloat((i8)x); }
}
