// TEST INFRASTRUCTURE — CPU oracle of one TScale2 training step.
//
// The layer drivers below restate, on top of the prim.h primitives,
//   TFFLayer::ComputeForward/ComputeBackward   src/gpt/compute/layer_ffn.cu:190-248
//   TAttLayer::ComputeForward/ComputeBackward  src/gpt/compute/layer_att.cu:368-482
//   TMoELayer + CpuMoe/CpuBackpropMoe/...      src/gpt/compute/layer_moe.cu:287-537
//   TComputeContext::ComputeForward/Backprop   src/gpt/compute/cpu_transformer.cpp:80-198
//   TQuantizedMatrix::Convert/GetFastFloatData src/gpt/matrix/quant.h:42-79
// (those live in CUDA translation units of the reference and cannot be linked
// on a machine without the CUDA driver).  Weight gradients are captured where
// the reference calls HostApplyDelta(delta) (src/gpt/compute/cpu_util.h:86-95).
// Only tests, the smoke check and the benchmark's CPU baseline may use this.
#include "ts2_oracle.h"
#include "prim.h"
#include <cmath>
#include <cstring>
#include <chrono>
#include <algorithm>

using namespace ts2o;

namespace {

const float kModelDiscrScale = 1.f / 32; // MODEL_DISCR_SCALE, model_dim.h:9
const float kLog2 = 0.693147f;           // LOG2, model_dim.h:16
const float kMoeScale = 0.5f;            // MOE_SCALE, model_dim.h:19
const int kStateNormTile = 128;          // STATE_NORM_TILE, model_dim.h:20
inline float FinalLayerMult() { return 1.f / kLog2; } // CalcFinalLayerMult, model_dim.h:25

// ---------------------------------------------------------------------------
// number formats

float HalfToFloat(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            int sh = 0;
            while (!(m & 1024)) {
                m <<= 1;
                ++sh;
            }
            bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 1023) << 13);
        }
    } else if (e == 31) {
        bits = sign | 0x7f800000u | (m << 13);
    } else {
        bits = sign | ((e + 112) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// round-to-nearest-even fp32 -> fp16 (what _mm256_cvtps_ph(x, 0) does, quant.cpp:64-75)
uint16_t FloatToHalf(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000;
    int32_t e = (int32_t)((x >> 23) & 255) - 127 + 15;
    uint32_t m = x & 0x7fffff;
    if (((x >> 23) & 255) == 255)
        return (uint16_t)(sign | 0x7c00 | (m ? 0x200 : 0));
    if (e >= 31)
        return (uint16_t)(sign | 0x7c00);
    if (e <= 0) {
        if (e < -10)
            return (uint16_t)sign;
        m |= 0x800000;
        int shift = 14 - e;
        uint32_t hm = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1)))
            ++hm;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = m >> 13, rem = m & 0x1fff;
    uint16_t res = (uint16_t)(sign | ((uint32_t)e << 10) | hm);
    if (rem > 0x1000 || (rem == 0x1000 && (hm & 1)))
        ++res; // carry into the exponent is the correct rounding
    return res;
}

// ConvertToFp8e4m3, src/gpt/model_params/sse_utils.h:161-204: round half away
// from zero on the 4th mantissa bit, no subnormals on the way in, saturate to 448.
uint8_t FloatToE4M3Ref(float v)
{
    uint32_t bits;
    memcpy(&bits, &v, 4);
    uint32_t r0 = bits & 0xFF800000u, r1 = bits & 0xFF880000u;
    float f0, f1;
    memcpy(&f0, &r0, 4);
    memcpy(&f1, &r1, 4);
    v = v + (f1 - f0);
    memcpy(&bits, &v, 4);
    int32_t sign = bits >> 31;
    int32_t exponent = (int32_t)((bits & 0x7F800000u) >> 23) - (127 - 7);
    int32_t mantissa = (bits & 0x007FFFFFu) >> 20;
    int32_t fp8 = (sign << 7) | (exponent << 3) | mantissa;
    if (exponent > 15)
        fp8 = (sign << 7) | 0x7f;
    if (exponent < 0)
        fp8 = 0;
    fp8 &= 0xff; // the packus steps keep the low byte for in-range values
    uint8_t b = (uint8_t)fp8;
    if (b == 0xff)
        b = 0xfe;
    if (b == 0x7f)
        b = 0x7e;
    return b;
}

// ConvertE4toFloat, src/util/fp8.h:4-22
float E4M3ToFloatRef(uint8_t xb)
{
    int8_t x = (int8_t)xb;
    if (x == 0)
        return 0;
    float sign = (x & 0x80) ? -1.f : 1.f;
    int e = (x >> 3) & 15, m = x & 7;
    if (e == 0 && m > 0)
        return sign * exp2f(1 - 7) * (0 + exp2f(-3) * m);
    return sign * exp2f(e - 7) * (1 + exp2f(-3) * m);
}

// PackFloatToInt8, src/gpt/model_params/sse_utils.h:56-78: nearest-even, saturating
int8_t FloatToI8(float v)
{
    float r = nearbyintf(v);
    if (r > 127)
        r = 127;
    if (r < -128)
        r = -128;
    return (int8_t)r;
}

// TQuantizedMatrix::Convert + GetFastFloatData
void QuantizeMatrix(const float *w, int64_t xSize, int64_t ySize, int quant, bool noScale, void *qOut, float *deq, float *skoOut)
{
    double sum2 = 0;
    for (int64_t i = 0; i < xSize * ySize; ++i)
        sum2 += (double)w[i] * w[i];
    float sko = sqrt((float)sum2 / (xSize * ySize));
    if (skoOut)
        *skoOut = sko;
    if (quant == TS2O_QUANT_NONE) {
        // no quantization: the compute path sees w (or w / sko for the "no scale" matrices)
        for (int64_t i = 0; i < xSize * ySize; ++i)
            if (deq)
                deq[i] = noScale ? ((sko == 0) ? 0 : w[i] / sko) : w[i];
        return;
    }
    float discrScale = sko * kModelDiscrScale;
    float mult = (sko == 0) ? 0 : (1 / discrScale);
    float scale = kModelDiscrScale;
    if (!noScale)
        scale *= sko;
    for (int64_t i = 0; i < xSize * ySize; ++i) {
        float v = w[i] * mult, q;
        if (quant == TS2O_QUANT_I8) {
            int8_t b = FloatToI8(v);
            if (qOut)
                ((int8_t *)qOut)[i] = b;
            q = b;
        } else if (quant == TS2O_QUANT_E4M3) {
            uint8_t b = FloatToE4M3Ref(v);
            if (qOut)
                ((uint8_t *)qOut)[i] = b;
            q = E4M3ToFloatRef(b);
        } else {
            uint16_t h = FloatToHalf(v);
            if (qOut)
                ((uint16_t *)qOut)[i] = h;
            q = HalfToFloat(h);
        }
        if (deq)
            deq[i] = q * scale;
    }
}

// ---------------------------------------------------------------------------
// Engine-faithful activation rounding (ts2o_set_activation_quant).  The reference's CPU path keeps every activation
// and gradient in fp32; its GPU path, like the B200 engine, hands them to the fp8 contractions as e4m3 bytes
// (TNormStateFloat / TFastGradientFloat = e4m3, cfg_precision.h:28-35).  With this mode on, the drivers below round
// the same four operand tensors at the same points and scales as the engine: the normalized state and the gated
// activation at 16 (the engine's s_act), the state gradient entering a layer at the power of two that brings its
// largest magnitude just under 128 (ScaleGrad / ComputeGradMult, gpu_grad_scale.cuh:33-62), and the gradients of the
// first contraction's outputs in the engine's scale-free units.  The rounding is the OCP e4m3 conversion the hardware
// does (cvt.rn.satfinite: nearest even, subnormals down to 2^-9, magnitudes from 448 up saturate), not the weight
// encoder above.  What is left between the engine and this mode is fp16 rounding of intermediates and the fast
// exponentials; what is left between this mode and the fp32 mode is the format itself.
int g_actQuant = 0;

float RoundE4M3(float x)
{
    if (!(x == x))
        return x;
    float a = fabsf(x);
    if (a >= 448.f)
        return copysignf(448.f, x);
    int e;
    frexpf(a, &e);           // a = m * 2^e, m in [0.5, 1): the leading bit has weight 2^(e - 1)
    e = std::max(e - 1, -6); // below 2^-6 the spacing stays that of the smallest normal binade
    float q = ldexpf(1.f, e - 3);
    return copysignf(nearbyintf(a / q) * q, x); // default rounding mode: to nearest, ties to even
}

// mode 1: e4m3 at `scale`; mode 2 (the engine's int8 pipeline): int8, nearest even, saturating, at `scale_i8`
void QuantizeInPlace(Mat *m, float scale, float scale_i8 = 0)
{
    if (!g_actQuant)
        return;
    if (g_actQuant == 2) {
        if (scale_i8 == 0)
            return;
        for (float &v : m->v)
            v = (float)FloatToI8(v * scale_i8) / scale_i8;
        return;
    }
    const float inv = 1.f / scale;
    for (float &v : m->v)
        v = RoundE4M3(v * scale) * inv;
}

// mode 2: the gradient operand of a dX contraction, quantized per token row to int8 with scale max|row| / 127.  A row
// may consist of several blocks, each in its own units (factor[i]): the maximum is taken over the scaled row.  Nearest
// rounding here; the engine rounds stochastically (same variance class, different draws).
void RowQuantI8Joint(const std::vector<Mat *> &parts, const std::vector<float> &factor)
{
    const int T = parts[0]->rows;
    for (int t = 0; t < T; ++t) {
        float mx = 0;
        for (size_t i = 0; i < parts.size(); ++i)
            for (int x = 0; x < parts[i]->cols; ++x)
                mx = fmaxf(mx, fabsf(parts[i]->row(t)[x] * factor[i]));
        if (mx == 0)
            continue;
        const float scale = mx / 127;
        for (size_t i = 0; i < parts.size(); ++i)
            for (int x = 0; x < parts[i]->cols; ++x) {
                float &v = parts[i]->row(t)[x];
                v = (float)FloatToI8(v * factor[i] / scale) * scale / factor[i];
            }
    }
}

// the engine's grad_mult: largest power of two that keeps max |g| * mult <= 128
float GradMult(const Mat &g)
{
    float m = 0;
    for (float v : g.v)
        if (fabsf(v) > m && fabsf(v) < 3.0e38f)
            m = fabsf(v);
    if (!(m > 0))
        return 1;
    float e = floorf(log2f(128.f / m));
    e = std::min(std::max(e, -100.f), 100.f);
    return exp2f(e);
}

const float kActScale = 16.f;    // e4m3 pipeline
const float kActScaleI8 = 24.f;  // int8 pipeline (STATE_VEC_SCALE = 1 / 24, cfg_precision.h:72)

// ---------------------------------------------------------------------------
// model

struct Matrix {
    int64_t x = 0, y = 0;
    Mat data, dataNoScale; // what GetData / GetDataNoScale return
    float sko = 1;         // matrix scale of TQuantizedMatrix::Convert
    float *gradOut = nullptr;
};

void AddInto(Mat *dst, const Mat &src)
{
    for (size_t i = 0; i < src.v.size(); ++i)
        dst->v[i] += src.v[i] * 1;
}

void StoreDelta(Matrix &m, const Mat &delta)
{
    if (m.gradOut)
        memcpy(m.gradOut, delta.v.data(), sizeof(float) * delta.v.size());
}

// dstGradDelta: the gradient the weight-gradient product reads, where it differs from the one the dX product reads
// (int8 pipeline: dX from the row-quantized gradient, dW from the unquantized one)
void MatmulBackprop(Matrix &m, bool noScale, const Mat &src, const Mat &dstGrad, bool update, Mat *srcGrad, const Mat *dstGradDelta = nullptr)
{
    prim::MulBackwardWithAccum(srcGrad, noScale ? m.dataNoScale : m.data, dstGrad);
    if (update) {
        Mat delta;
        prim::SumRankOne(src, &delta, dstGradDelta ? *dstGradDelta : dstGrad);
        StoreDelta(m, delta);
    }
}

struct Common {
    Mat rope;
    std::vector<AttInfo> att, revAtt;
};

struct Dims {
    int dim, qDim, ttDim, headCount, ffnDim, expertDim, expertCount, selected;
};

// ---- FFN ------------------------------------------------------------------
void FfnRecompute(const Dims &d, Matrix *mm, const Mat &prevState, Mat &normState, Mat &wide, Mat &wideNorm, Mat &gate, Mat &rg)
{
    normState = prim::NormalizeState(prevState, d.dim / kStateNormTile);
    QuantizeInPlace(&normState, kActScale, kActScaleI8);
    wide = prim::MulForward(normState, mm[0].data);
    wideNorm = prim::NormalizeState(wide, d.ffnDim / 128);
    gate = prim::MulForward(normState, mm[1].dataNoScale);
    prim::LoLU(gate, wideNorm, &rg);
    QuantizeInPlace(&rg, kActScale, kActScaleI8);
}

void FfnForward(const Dims &d, Matrix *mm, const Mat &prevState, Mat *state)
{
    Mat normState, wide, wideNorm, gate, rg;
    FfnRecompute(d, mm, prevState, normState, wide, wideNorm, gate, rg);
    *state = prevState;
    AddInto(state, prim::MulForward(rg, mm[2].data));
}

void FfnBackward(const Dims &d, Matrix *mm, bool update, const Mat &prevState, Mat *grad)
{
    Mat normState, wide, wideNorm, gate, rg;
    FfnRecompute(d, mm, prevState, normState, wide, wideNorm, gate, rg);
    Mat dNormState(normState.rows, normState.cols);
    Mat drg(rg.rows, rg.cols);
    // the contractions see the state gradient as e4m3 at the step's power-of-two scale; the residual path keeps fp32
    Mat gFast = *grad;
    const float gradMult = g_actQuant ? GradMult(*grad) : 1.f;
    QuantizeInPlace(&gFast, gradMult);
    if (g_actQuant == 2)
        RowQuantI8Joint({&gFast}, {1.f});
    MatmulBackprop(mm[2], false, rg, gFast, update, &drg, g_actQuant == 2 ? grad : nullptr);
    Mat dgate, dwide;
    prim::BackpropLoLU(gate, wideNorm, drg, &dgate, &dwide);
    prim::NormalizeStateBackward(wide, d.ffnDim / 128, dwide, &dwide);
    Mat dwideFull = dwide, dgateFull = dgate;
    {
        // engine units: true gradient = stored value * fscale, fscale = sqrt(dim / ffnDim) * sko_contract / gradMult;
        // the expansion is used scale-free there (a normalisation follows it), so its gradient carries its matrix scale
        const float fscale = sqrtf((float)d.dim / (float)d.ffnDim) * mm[2].sko / gradMult;
        QuantizeInPlace(&dwide, mm[0].sko / fscale);
        QuantizeInPlace(&dgate, 1.f / fscale);
        if (g_actQuant == 2)
            RowQuantI8Joint({&dwide, &dgate}, {mm[0].sko / fscale, 1.f / fscale});
    }
    MatmulBackprop(mm[0], false, normState, dwide, update, &dNormState, g_actQuant == 2 ? &dwideFull : nullptr);
    MatmulBackprop(mm[1], true, normState, dgate, update, &dNormState, g_actQuant == 2 ? &dgateFull : nullptr);
    Mat dState;
    prim::NormalizeStateBackward(prevState, d.dim / kStateNormTile, dNormState, &dState);
    AddInto(grad, dState);
}

// ---- attention --------------------------------------------------------------
struct AttFwd {
    Mat normState, qSrc, kSrc, gate, vSrc, q, k, v, valLookup, rg;
    prim::Attention comp;
};

void AttRecompute(const Dims &d, Matrix *mm, const Common &c, float slope, int attType, const Mat &prevState, AttFwd &f)
{
    f.normState = prim::NormalizeState(prevState, d.dim / kStateNormTile);
    QuantizeInPlace(&f.normState, kActScale, kActScaleI8);
    f.comp.Init(d.headCount, d.qDim, d.ttDim, slope);
    f.qSrc = prim::MulForward(f.normState, mm[0].data);
    f.kSrc = prim::MulForward(f.normState, mm[1].data);
    f.gate = prim::MulForward(f.normState, mm[3].dataNoScale);
    f.vSrc = prim::MulForward(f.normState, mm[2].data);
    f.q = prim::NormalizeState(f.qSrc, d.headCount);
    f.k = f.kSrc;
    f.v = prim::NormalizeState(f.vSrc, d.headCount);
    prim::ApplyRope(c.rope, 1, &f.q);
    prim::ApplyRope(c.rope, 1, &f.k);
    f.comp.ComputeValLookup(f.q, f.k, f.v, c.att[attType], &f.valLookup);
    prim::LoLU(f.gate, f.valLookup, &f.rg);
    QuantizeInPlace(&f.rg, kActScale, kActScaleI8);
}

void AttForward(const Dims &d, Matrix *mm, const Common &c, float slope, int attType, const Mat &prevState, Mat *state)
{
    AttFwd f;
    AttRecompute(d, mm, c, slope, attType, prevState, f);
    *state = prevState;
    AddInto(state, prim::MulForward(f.rg, mm[4].data));
}

void AttBackward(const Dims &d, Matrix *mm, bool update, const Common &c, float slope, int attType, const Mat &prevState, Mat *grad)
{
    AttFwd f;
    AttRecompute(d, mm, c, slope, attType, prevState, f);
    Mat dNormState(f.normState.rows, f.normState.cols);
    Mat drg(f.rg.rows, f.rg.cols);
    Mat gFast = *grad;
    const float gradMult = g_actQuant ? GradMult(*grad) : 1.f;
    QuantizeInPlace(&gFast, gradMult);
    if (g_actQuant == 2)
        RowQuantI8Joint({&gFast}, {1.f});
    MatmulBackprop(mm[4], false, f.rg, gFast, update, &drg, g_actQuant == 2 ? grad : nullptr);
    Mat dgate, dValLookup;
    prim::BackpropLoLU(f.gate, f.valLookup, drg, &dgate, &dValLookup);
    Mat dScale;
    prim::ComputeDScale(d.headCount, d.ttDim, f.valLookup, dValLookup, &dScale);
    Mat dQ, dK, dV;
    f.comp.GradQ(f.q, f.k, f.v, dValLookup, dScale, c.att[attType], &dQ);
    f.comp.GradK(f.q, f.k, f.v, dValLookup, dScale, c.revAtt[attType], &dK, &dV);
    prim::ApplyRope(c.rope, -1, &dQ);
    prim::ApplyRope(c.rope, -1, &dK);
    prim::NormalizeStateBackward(f.qSrc, d.headCount, dQ, &dQ);
    prim::NormalizeStateBackward(f.vSrc, d.headCount, dV, &dV);
    {
        // engine units (see FfnBackward): Q and V are used scale-free there, K's matrix scale is folded into its
        // gradient so that the four-way dX contraction reads scale-free weights throughout
        const float fscale = sqrtf((float)d.dim / (float)(d.ttDim * d.headCount)) * mm[4].sko / gradMult;
        QuantizeInPlace(&dQ, mm[0].sko / fscale);
        QuantizeInPlace(&dK, mm[1].sko / fscale);
        QuantizeInPlace(&dV, mm[2].sko / fscale);
        QuantizeInPlace(&dgate, 1.f / fscale);
    }
    Mat dQFull = dQ, dKFull = dK, dVFull = dV, dgateFull = dgate;
    if (g_actQuant == 2) {
        const float fscale = sqrtf((float)d.dim / (float)(d.ttDim * d.headCount)) * mm[4].sko / gradMult;
        RowQuantI8Joint({&dQ, &dK, &dV, &dgate}, {mm[0].sko / fscale, mm[1].sko / fscale, mm[2].sko / fscale, 1.f / fscale});
    }
    const bool sep = g_actQuant == 2;
    MatmulBackprop(mm[0], false, f.normState, dQ, update, &dNormState, sep ? &dQFull : nullptr);
    MatmulBackprop(mm[1], false, f.normState, dK, update, &dNormState, sep ? &dKFull : nullptr);
    MatmulBackprop(mm[2], false, f.normState, dV, update, &dNormState, sep ? &dVFull : nullptr);
    MatmulBackprop(mm[3], true, f.normState, dgate, update, &dNormState, sep ? &dgateFull : nullptr);
    Mat dState;
    prim::NormalizeStateBackward(prevState, d.dim / kStateNormTile, dNormState, &dState);
    AddInto(grad, dState);
}

// ---- MoE --------------------------------------------------------------------
// CpuMoe, layer_moe.cu:287-328
void MoeSelect(const Mat &moeSrc, int expertCount, int selected, Mat *res)
{
    *res = moeSrc;
    float moeScale = sqrtf(expertCount);
    for (int t = 0; t < moeSrc.rows; ++t) {
        std::vector<float> src(expertCount);
        float maxVal = -1e10f;
        for (int x = 0; x < expertCount; ++x) {
            src[x] = moeSrc.row(t)[x];
            res->row(t)[x] = 0;
            maxVal = std::max(maxVal, src[x]);
        }
        float sum2 = 0;
        for (int z = 0; z < selected; ++z) {
            float top = -1e10;
            int topIdx = 0;
            for (int x = 0; x < expertCount; ++x) {
                if (src[x] > top) {
                    top = src[x];
                    topIdx = x;
                }
            }
            float w = exp((top - maxVal) * kMoeScale);
            res->row(t)[topIdx] = w;
            src[topIdx] = -1e10;
            sum2 += w * w;
        }
        float scale = moeScale * sqrt(1 / sum2);
        for (int x = 0; x < expertCount; ++x)
            res->row(t)[x] *= scale;
    }
}

// CpuBackpropMoe, layer_moe.cu:331-360
void MoeSelectBackward(const Mat &moe, int expertCount, Mat *dMoe)
{
    float moeScale = sqrtf(expertCount);
    for (int t = 0; t < moe.rows; ++t) {
        std::vector<float> src(expertCount), g(expertCount);
        for (int x = 0; x < expertCount; ++x) {
            src[x] = moe.row(t)[x] / moeScale;
            g[x] = dMoe->row(t)[x] * moeScale;
        }
        float avrg = 0;
        for (int x = 0; x < expertCount; ++x)
            avrg += src[x] * g[x];
        for (int x = 0; x < expertCount; ++x) {
            float w = src[x];
            dMoe->row(t)[x] = (w * g[x] - w * w * avrg) * kMoeScale;
        }
    }
}

// FwdContractMatrix, layer_moe.cu:407-421: src[[expert][e]][x] -> res[e][[expert][x]]
Mat FwdContract(const Mat &src, int xpCount)
{
    int xSize = src.cols, eSize = src.rows / xpCount;
    Mat res(eSize, xpCount * xSize);
    for (int xp = 0; xp < xpCount; ++xp)
        for (int e = 0; e < eSize; ++e)
            for (int x = 0; x < xSize; ++x)
                res.row(e)[xp * xSize + x] = src.row(xp * eSize + e)[x];
    return res;
}

// BwdContractMatrix, layer_moe.cu:424-438
Mat BwdContract(const Mat &src, int xpCount)
{
    int xSize = src.cols / xpCount, eSize = src.rows;
    Mat res(xpCount * eSize, xSize);
    for (int xp = 0; xp < xpCount; ++xp)
        for (int e = 0; e < eSize; ++e)
            for (int x = 0; x < xSize; ++x)
                res.row(xp * eSize + e)[x] = src.row(e)[xp * xSize + x];
    return res;
}

struct MoeFwd {
    Mat normState, wide, wideNorm, gate, moeSrc, rgSrc, moe, rg;
};

void MoeRecompute(const Dims &d, Matrix *mm, const Mat &prevState, MoeFwd &f)
{
    int moeDim = d.expertCount * d.expertDim;
    f.normState = prim::NormalizeState(prevState, d.dim / kStateNormTile);
    if (g_actQuant == 1)
        QuantizeInPlace(&f.normState, kActScale);
    f.wide = prim::MulForward(f.normState, mm[0].data);
    f.wideNorm = prim::NormalizeState(f.wide, moeDim / 128);
    f.gate = prim::MulForward(f.normState, mm[1].dataNoScale);
    f.moeSrc = prim::MulForward(f.normState, mm[3].dataNoScale);
    prim::LoLU(f.gate, f.wideNorm, &f.rgSrc);
    MoeSelect(f.moeSrc, d.expertCount, d.selected, &f.moe);
    f.rg = f.rgSrc;
    int expertSize = f.rg.cols / d.expertCount; // ScaleExperts, layer_moe.cu:363-378
    for (int t = 0; t < f.rg.rows; ++t)
        for (int e = 0; e < d.expertCount; ++e) {
            float s = f.moe.row(t)[e];
            for (int x = e * expertSize; x < (e + 1) * expertSize; ++x)
                f.rg.row(t)[x] *= s;
        }
    if (g_actQuant == 1) // the engine stores the gated activation with the routing weight folded in
        QuantizeInPlace(&f.rg, kActScale);
}

void MoeForward(const Dims &d, Matrix *mm, const Mat &prevState, Mat *state)
{
    MoeFwd f;
    MoeRecompute(d, mm, prevState, f);
    *state = prevState;
    AddInto(state, prim::MulForward(f.rg, FwdContract(mm[2].data, d.expertCount)));
}

void MoeBackward(const Dims &d, Matrix *mm, bool update, const Mat &prevState, Mat *grad)
{
    MoeFwd f;
    MoeRecompute(d, mm, prevState, f);
    int moeDim = d.expertCount * d.expertDim;
    Mat dNormState(f.normState.rows, f.normState.cols);
    Mat drg(f.rg.rows, f.rg.cols);
    Mat gFast = *grad;
    const float gradMult = g_actQuant == 1 ? GradMult(*grad) : 1.f;
    if (g_actQuant == 1)
        QuantizeInPlace(&gFast, gradMult);
    // engine units of the layer's intermediate gradients (see FfnBackward); the contract matrix is [dim][E * expertDim]
    const float fscale = sqrtf((float)d.dim / (float)moeDim) * mm[2].sko / gradMult;
    { // ContractMatmulBackprop, layer_moe.cu:441-452
        prim::MulBackwardWithAccum(&drg, FwdContract(mm[2].data, d.expertCount), gFast);
        if (update) {
            Mat delta;
            prim::SumRankOne(f.rg, &delta, gFast);
            StoreDelta(mm[2], BwdContract(delta, d.expertCount));
        }
    }
    Mat dMoe(f.moe.rows, f.moe.cols);
    { // BackpropScaleExperts, layer_moe.cu:380-404
        int expertSize = drg.cols / d.expertCount;
        for (int t = 0; t < drg.rows; ++t)
            for (int e = 0; e < d.expertCount; ++e) {
                float s = f.moe.row(t)[e], gm = 0;
                for (int x = e * expertSize; x < (e + 1) * expertSize; ++x) {
                    float g = drg.row(t)[x];
                    gm += f.rgSrc.row(t)[x] * g;
                    drg.row(t)[x] *= s;
                }
                dMoe.row(t)[e] = gm;
            }
    }
    MoeSelectBackward(f.moe, d.expertCount, &dMoe);
    if (g_actQuant == 1)
        QuantizeInPlace(&dMoe, 1.f / fscale);
    MatmulBackprop(mm[3], true, f.normState, dMoe, update, &dNormState);
    Mat dgate, dwide;
    prim::BackpropLoLU(f.gate, f.wideNorm, drg, &dgate, &dwide);
    prim::NormalizeStateBackward(f.wide, moeDim / 128, dwide, &dwide);
    if (g_actQuant == 1) {
        QuantizeInPlace(&dwide, mm[0].sko / fscale);
        QuantizeInPlace(&dgate, 1.f / fscale);
    }
    MatmulBackprop(mm[0], false, f.normState, dwide, update, &dNormState);
    MatmulBackprop(mm[1], true, f.normState, dgate, update, &dNormState);
    Mat dState;
    prim::NormalizeStateBackward(prevState, d.dim / kStateNormTile, dNormState, &dState);
    AddInto(grad, dState);
}

int LayerMatrixCount(int type)
{
    return type == TS2_LAYER_ATT ? 5 : type == TS2_LAYER_FFN ? 3 : type == TS2_LAYER_MOE ? 4 : -1;
}

} // namespace

extern "C" {

const char *ts2o_backend(void) { return prim::BackendName(); }

void ts2o_set_activation_quant(int mode) { g_actQuant = mode; }

// NormalizeVecsRowMaxKernel (src/gpt/compute/row_scale.cuh:12-43) with TCudaRngLCG (src/lib/cuda/cuda_util.cuh:538-559)
// for an int8 destination: the warp of the kernel becomes a loop over its 32 lanes.  The GPU code contracts
// buf * mult + u into one fused multiply-add (nvcc's default), then subtracts 0.5; fmaf states that here.
void ts2o_rowquant_i8(const float *x, int T, int D, int8_t *q, float *row_scale)
{
    for (int t = 0; t < T; ++t) {
        const float *buf = x + (size_t)t * D;
        float maxVal = 0;
        for (int d = 0; d < D; ++d)
            maxVal = fmaxf(maxVal, fabsf(buf[d]));
        float discrScale = 0;
        if (maxVal > 0) {
            discrScale = maxVal / 127; // GetMaxDiscrScale(maxVal, (i8 *)0), cuda_util.cuh:371-374
            float mult = 1 / discrScale;
            for (int h = 0; h < 32; ++h) {
                uint32_t a, b0;
                memcpy(&a, &buf[h], 4);
                memcpy(&b0, &buf[0], 4);
                uint32_t state = a * 0x398bf183u + b0 * 0x1affc3dfu + (uint32_t)t * 0x9023a049u;
                for (int d = h; d < D; d += 32) {
                    state = state * 0x448e3079u + 0xc484ef10u;
                    float u = state * (1.0f / float(1ll << 32));
                    q[(size_t)t * D + d] = FloatToI8(fmaf(buf[d], mult, u) - 0.5f); // cvt.rni.sat.s8.f32
                }
            }
        } else {
            for (int d = 0; d < D; ++d)
                q[(size_t)t * D + d] = 0;
        }
        row_scale[t] = discrScale;
    }
}

void ts2o_round_e4m3(const float *src, int64_t n, float *dst)
{
    for (int64_t i = 0; i < n; ++i)
        dst[i] = RoundE4M3(src[i]);
}

int ts2o_quantize_matrix(const float *w, int64_t x_size, int64_t y_size, int quant, int no_scale, void *q_out, float *deq_out,
                         float *sko_out)
{
    QuantizeMatrix(w, x_size, y_size, quant, no_scale != 0, q_out, deq_out, sko_out);
    return 0;
}

void ts2o_encode(const float *src, int64_t n, int quant, float mult, void *dst)
{
    for (int64_t i = 0; i < n; ++i) {
        float v = src[i] * mult;
        if (quant == TS2O_QUANT_I8)
            ((int8_t *)dst)[i] = FloatToI8(v);
        else if (quant == TS2O_QUANT_E4M3)
            ((uint8_t *)dst)[i] = FloatToE4M3Ref(v);
        else
            ((uint16_t *)dst)[i] = FloatToHalf(v);
    }
}

float ts2o_decode_e4m3(uint8_t x) { return E4M3ToFloatRef(x); }

int ts2o_backprop(const ts2_model_descr *descr, const ts2_matrix_view *mats, int n_mats, const float *bias,
                  const ts2_batch_nodes *nodes, int weight_quant, ts2o_outputs *out)
{
    auto t0 = std::chrono::steady_clock::now();
    Dims d;
    d.dim = descr->dim;
    d.qDim = descr->q_dim;
    d.ttDim = descr->tt_dim;
    d.headCount = descr->head_count;
    d.ffnDim = descr->ffn_tiles * 128;
    d.expertDim = descr->expert_dim;
    d.expertCount = descr->moe_expert_count;
    d.selected = descr->moe_selected;
    const int L = descr->layer_count, T = nodes->node_count, V = descr->output_token_count;

    // matrices: embedding is always half (TEmbedFloat, cfg_precision.h:62), the rest TFastModelFloat
    std::vector<Matrix> mm(n_mats);
    {
        int expect = 2;
        for (int l = 0; l < L; ++l) {
            int c = LayerMatrixCount(descr->layers[l].layer_type);
            if (c < 0)
                return TS2_ERR_UNSUPPORTED;
            expect += c;
        }
        if (expect != n_mats)
            return TS2_ERR_INVALID_ARG;
    }
    for (int i = 0; i < n_mats; ++i) {
        Matrix &m = mm[i];
        m.x = mats[i].x_size;
        m.y = mats[i].y_size;
        int q = (weight_quant == TS2O_QUANT_NONE) ? TS2O_QUANT_NONE : (i == 0 ? TS2O_QUANT_HALF : weight_quant);
        m.data.resize((int)m.y, (int)m.x);
        m.dataNoScale.resize((int)m.y, (int)m.x);
        QuantizeMatrix(mats[i].data, m.x, m.y, q, false, nullptr, m.data.v.data(), &m.sko);
        QuantizeMatrix(mats[i].data, m.x, m.y, q, true, nullptr, m.dataNoScale.v.data(), nullptr);
        m.gradOut = (out && out->grads) ? out->grads[i] : nullptr;
    }
    std::vector<int> layerMat(L);
    {
        int p = 2;
        for (int l = 0; l < L; ++l) {
            layerMat[l] = p;
            p += LayerMatrixCount(descr->layers[l].layer_type);
        }
    }

    // common data: TCommonDataCPU::Init / InitAttention, src/gpt/compute/layer.cpp:7-23
    Common common;
    prim::FillRopeBuf(&common.rope, d.qDim, T);
    for (int a = 0; a < nodes->attention_type_count; ++a) {
        AttInfo ai;
        const ts2_attention_info &src = nodes->att[a];
        ai.ptr.assign(src.span_ptr, src.span_ptr + T + 1);
        ai.start.assign(src.span_start, src.span_start + ai.ptr[T]);
        ai.finish.assign(src.span_finish, src.span_finish + ai.ptr[T]);
        common.att.push_back(ai);
        common.revAtt.push_back(prim::TransposeAttention(ai));
    }

    // ComputeEmbedding, cpu_transformer.cpp:66-90
    std::vector<Mat> states(L + 1);
    states[0].resize(T, d.dim);
    for (int t = 0; t < T; ++t) {
        for (uint32_t k = nodes->label_ptr[t]; k < nodes->label_ptr[t + 1]; ++k) {
            uint32_t label = nodes->label_arr[k];
            float w = (label & TS2_LABEL_NEGATIVE) ? -1 : 1;
            label &= TS2_LABEL_MASK;
            for (int x = 0; x < d.dim; ++x)
                states[0].row(t)[x] += mm[0].data.row(label)[x] * w;
        }
    }
    // layers forward
    for (int l = 0; l < L; ++l) {
        const ts2_layer_params &lp = descr->layers[l];
        Matrix *lm = &mm[layerMat[l]];
        if (lp.layer_type == TS2_LAYER_ATT)
            AttForward(d, lm, common, lp.alibi_slope, lp.attention_type_id, states[l], &states[l + 1]);
        else if (lp.layer_type == TS2_LAYER_FFN)
            FfnForward(d, lm, states[l], &states[l + 1]);
        else
            MoeForward(d, lm, states[l], &states[l + 1]);
    }
    Mat finalNorm = prim::NormalizeState(states[L], d.dim / kStateNormTile);
    Mat finalNormFast = finalNorm; // the engine's logits contraction reads e4m3, its final-layer dW contraction fp16
    QuantizeInPlace(&finalNormFast, kActScale, kActScaleI8);
    Mat pred = prim::MulForward(finalNormFast, mm[1].data);
    for (float &x : pred.v)
        x *= FinalLayerMult();
    // SoftMax, cpu_transformer.cpp:12-37
    for (int t = 0; t < T; ++t) {
        float *p = pred.row(t);
        float maxVal = 0;
        for (int k = 0; k < V; ++k)
            maxVal = fmaxf(maxVal, p[k]);
        double sumWeight = 0;
        for (int k = 0; k < V; ++k) {
            float w = exp2(p[k] + (bias ? bias[k] : 0.f) - maxVal);
            p[k] = w;
            sumWeight += w;
        }
        float scale = 1 / sumWeight;
        for (int k = 0; k < V; ++k)
            p[k] *= scale;
    }
    if (out) {
        double sum = 0;
        for (int i = 0; i < nodes->target_count; ++i) {
            float pr = pred.row(nodes->target_node[i])[nodes->target_id[i]];
            if (out->target_prob)
                out->target_prob[i] = pr;
            sum += log(pr);
        }
        out->score = nodes->target_count ? sum / nodes->target_count : 0;
        if (out->states)
            for (int l = 0; l <= L; ++l)
                memcpy(out->states + (size_t)l * T * d.dim, states[l].v.data(), sizeof(float) * T * d.dim);
    }

    // backward, cpu_transformer.cpp:128-198
    const bool updateLayers = !(descr->flags & TS2_MPF_DISABLE_TUNE_LAYERS);
    Mat grad(T, d.dim);
    {
        Mat gradArr(T, V);
        for (int i = 0; i < nodes->target_count; ++i) {
            int node = nodes->target_node[i];
            for (int q = 0; q < V; ++q)
                gradArr.row(node)[q] += -pred.row(node)[q];
            gradArr.row(node)[nodes->target_id[i]] += 1;
        }
        float gs = FinalLayerMult() * kLog2;
        for (float &x : gradArr.v)
            x *= gs;
        Mat normStateGrad(T, d.dim);
        prim::MulBackwardWithAccum(&normStateGrad, mm[1].data, gradArr);
        if (!(descr->flags & TS2_MPF_DISABLE_TUNE_FINAL_LAYER)) {
            Mat delta;
            prim::SumRankOne(finalNorm, &delta, gradArr);
            StoreDelta(mm[1], delta);
        }
        prim::NormalizeStateBackward(states[L], d.dim / kStateNormTile, normStateGrad, &grad);
    }
    if (out && out->state_grads)
        memcpy(out->state_grads + (size_t)L * T * d.dim, grad.v.data(), sizeof(float) * T * d.dim);
    for (int l = L - 1; l >= 0; --l) {
        const ts2_layer_params &lp = descr->layers[l];
        Matrix *lm = &mm[layerMat[l]];
        if (lp.layer_type == TS2_LAYER_ATT)
            AttBackward(d, lm, updateLayers, common, lp.alibi_slope, lp.attention_type_id, states[l], &grad);
        else if (lp.layer_type == TS2_LAYER_FFN)
            FfnBackward(d, lm, updateLayers, states[l], &grad);
        else
            MoeBackward(d, lm, updateLayers, states[l], &grad);
        if (out && out->state_grads)
            memcpy(out->state_grads + (size_t)l * T * d.dim, grad.v.data(), sizeof(float) * T * d.dim);
    }
    if (!(descr->flags & TS2_MPF_DISABLE_TUNE_EMBED)) {
        Mat deltaLabel(descr->label_count, d.dim);
        for (int t = 0; t < T; ++t) {
            for (uint32_t k = nodes->label_ptr[t]; k < nodes->label_ptr[t + 1]; ++k) {
                uint32_t label = nodes->label_arr[k];
                float w = (label & TS2_LABEL_NEGATIVE) ? -1 : 1;
                label &= TS2_LABEL_MASK;
                for (int x = 0; x < d.dim; ++x)
                    deltaLabel.row(label)[x] += grad.row(t)[x] * w;
            }
        }
        StoreDelta(mm[0], deltaLabel);
    }
    if (out)
        out->seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return TS2_OK;
}

// MatrixRowSum2Kernel + UpdateGlobalRowDisp + AddGradientKernel, agpu_cuda.cu:32-134; the same step on the host:
// THostModelMatrix::AddDelta, host_matrix.cpp:123-157, against which tests/test_optimizer_vs_reference.py checks this
int ts2o_apply_gradient(float *weights, float *avg_grad, const float *grad, int64_t x_size, int64_t y_size, float *row_disp,
                        int64_t row_disp_size, float *sum_weight, float sparsity, const ts2_training_step *step)
{
    if (row_disp_size <= 0 || y_size % row_disp_size != 0)
        return TS2_ERR_INVALID_ARG;
    std::vector<float> sum2(y_size), rowScale(y_size);
    for (int64_t y = 0; y < y_size; ++y) {
        float s = 0;
        for (int64_t x = 0; x < x_size; ++x)
            s += grad[y * x_size + x] * grad[y * x_size + x];
        sum2[y] = s;
    }
    float sw = *sum_weight * step->disp_decay + 1;
    float norm = 1 / sw;
    int64_t stepRows = y_size / row_disp_size;
    auto rowScaleOf = [](float disp) { return (disp > 0) ? 1 / sqrt(disp) : 0; };
    for (int64_t b = 0; b < row_disp_size; ++b) {
        float s = 0;
        for (int64_t k = 0; k < stepRows; ++k)
            s += sum2[b * stepRows + k];
        float disp = s / (x_size * stepRows);
        float rd = row_disp[b] * step->disp_decay + disp;
        row_disp[b] = rd;
        float rs = rowScaleOf(rd * norm);
        for (int64_t k = 0; k < stepRows; ++k)
            rowScale[b * stepRows + k] = rs;
    }
    *sum_weight = sw;
    float stepMult = step->rate * sqrt(sparsity);
    float shrink = 1 - stepMult * step->l2reg; // GetShrinkMult, train_step.h:29
    for (int64_t y = 0; y < y_size; ++y) {
        for (int64_t x = 0; x < x_size; ++x) {
            int64_t i = y * x_size + x;
            float delta = grad[i] * rowScale[y];
            float newAG = avg_grad[i] * step->beta1 + delta * (1 - step->beta1);
            float total = newAG * step->weight1 + delta * step->weight0;
            weights[i] = weights[i] * shrink + total * stepMult;
            avg_grad[i] = newAG;
        }
    }
    return TS2_OK;
}

// ---- primitives -------------------------------------------------------------
static Mat Wrap(const float *p, int rows, int cols)
{
    Mat m(rows, cols);
    if (p)
        memcpy(m.v.data(), p, sizeof(float) * (size_t)rows * cols);
    return m;
}
static void Unwrap(const Mat &m, float *p)
{
    if (p)
        memcpy(p, m.v.data(), sizeof(float) * m.v.size());
}

void ts2o_mul_forward(const float *x, const float *w, float *y, int T, int in_dim, int out_dim)
{
    Unwrap(prim::MulForward(Wrap(x, T, in_dim), Wrap(w, out_dim, in_dim)), y);
}
void ts2o_mul_backward_accum(float *dx, const float *w, const float *dy, int T, int in_dim, int out_dim)
{
    Mat d = Wrap(dx, T, in_dim);
    prim::MulBackwardWithAccum(&d, Wrap(w, out_dim, in_dim), Wrap(dy, T, out_dim));
    Unwrap(d, dx);
}
void ts2o_sum_rank_one(const float *x, const float *dy, float *delta, int T, int in_dim, int out_dim)
{
    Mat d;
    prim::SumRankOne(Wrap(x, T, in_dim), &d, Wrap(dy, T, out_dim));
    Unwrap(d, delta);
}
void ts2o_normalize_state(const float *state, float *out, int T, int dim, int head_count)
{
    Unwrap(prim::NormalizeState(Wrap(state, T, dim), head_count), out);
}
void ts2o_normalize_state_backward(const float *state, const float *dnorm, float *grad, int T, int dim, int head_count)
{
    Mat g;
    prim::NormalizeStateBackward(Wrap(state, T, dim), head_count, Wrap(dnorm, T, dim), &g);
    Unwrap(g, grad);
}
void ts2o_lolu(const float *gate, const float *vals, float *out, int64_t n)
{
    Mat r;
    prim::LoLU(Wrap(gate, 1, (int)n), Wrap(vals, 1, (int)n), &r);
    Unwrap(r, out);
}
void ts2o_backprop_lolu(const float *gate, const float *vals, const float *grad, float *dgate, float *dvals, int64_t n)
{
    Mat a, b;
    prim::BackpropLoLU(Wrap(gate, 1, (int)n), Wrap(vals, 1, (int)n), Wrap(grad, 1, (int)n), &a, &b);
    Unwrap(a, dgate);
    Unwrap(b, dvals);
}
void ts2o_rope(float *p, int T, int dim, int head_dim, float dir)
{
    Mat rope, m = Wrap(p, T, dim);
    prim::FillRopeBuf(&rope, head_dim, T);
    prim::ApplyRope(rope, dir, &m);
    Unwrap(m, p);
}
void ts2o_attention(const float *q, const float *k, const float *v, int T, int head_count, float alibi_slope,
                    const ts2_attention_info *att, float *val_lookup, float *sum_weight, float *max_dp,
                    const float *d_val_lookup, float *dq, float *dk, float *dv)
{
    const int hd = 128;
    AttInfo ai;
    ai.ptr.assign(att->span_ptr, att->span_ptr + T + 1);
    ai.start.assign(att->span_start, att->span_start + ai.ptr[T]);
    ai.finish.assign(att->span_finish, att->span_finish + ai.ptr[T]);
    prim::Attention comp;
    comp.Init(head_count, hd, hd, alibi_slope);
    Mat Q = Wrap(q, T, hd * head_count), K = Wrap(k, T, hd * head_count), V = Wrap(v, T, hd * head_count), val;
    comp.ComputeValLookup(Q, K, V, ai, &val);
    Unwrap(val, val_lookup);
    Unwrap(comp.sumWeight, sum_weight);
    Unwrap(comp.maxDP, max_dp);
    if (d_val_lookup) {
        Mat dVal = Wrap(d_val_lookup, T, hd * head_count), dScale, dQ, dK, dV;
        prim::ComputeDScale(head_count, hd, val, dVal, &dScale);
        comp.GradQ(Q, K, V, dVal, dScale, ai, &dQ);
        comp.GradK(Q, K, V, dVal, dScale, prim::TransposeAttention(ai), &dK, &dV);
        Unwrap(dQ, dq);
        Unwrap(dK, dk);
        Unwrap(dV, dv);
    }
}
void ts2o_moe_select(const float *logits, float *weights, int T, int expert_count, int selected)
{
    Mat r;
    MoeSelect(Wrap(logits, T, expert_count), expert_count, selected, &r);
    Unwrap(r, weights);
}
void ts2o_moe_select_backward(const float *weights, float *dmoe, int T, int expert_count)
{
    Mat d = Wrap(dmoe, T, expert_count);
    MoeSelectBackward(Wrap(weights, T, expert_count), expert_count, &d);
    Unwrap(d, dmoe);
}

} // extern "C"
