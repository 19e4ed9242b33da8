// TEST INFRASTRUCTURE — CPU oracle of the TScale2 training step.  Not part of
// the product: only tests/, __graft_entry__.smoke() and bench.py's CPU baseline
// may load what is built from this directory.
//
// prim.h: the primitive operations of the reference's CPU path, behind one
// interface with two implementations:
//   prim_port.cpp — a restatement in plain C++ (always built), and
//   prim_ref.cpp  — adapters that call the reference's own compiled functions
//                   (built only where the reference sources are present).
// The layer drivers in ts2_oracle.cpp are written once against this interface.
#pragma once
#include <vector>
#include <cstdint>
#include <cstddef>

namespace ts2o {

struct Mat {
    int rows = 0, cols = 0;
    std::vector<float> v;
    Mat() {}
    Mat(int r, int c) : rows(r), cols(c), v((size_t)r * c, 0.f) {}
    void resize(int r, int c) { rows = r; cols = c; v.assign((size_t)r * c, 0.f); }
    float *row(int r) { return v.data() + (size_t)r * cols; }
    const float *row(int r) const { return v.data() + (size_t)r * cols; }
};

// CSR of inclusive spans per node (TAttentionInfo, src/gpt/att/att.h:22-49)
struct AttInfo {
    std::vector<int> start, finish, ptr;
};

namespace prim {
const char *BackendName();
// src/gpt/compute/cpu_util.cpp:7-27
Mat MulForward(const Mat &x, const Mat &w);
// src/gpt/compute/cpu_util.cpp:30-47
void MulBackwardWithAccum(Mat *dx, const Mat &w, const Mat &dy);
// src/gpt/compute/cpu_util.cpp:50-67
void SumRankOne(const Mat &x, Mat *delta, const Mat &dy);
// src/gpt/compute/cpu_util.cpp:72-99
Mat NormalizeState(const Mat &state, int headCount);
// src/gpt/compute/cpu_util.cpp:102-134 (dnorm and grad may be the same object)
void NormalizeStateBackward(const Mat &state, int headCount, const Mat &dnorm, Mat *grad);
// src/gpt/compute/cpu_util.cpp:139-186
void LoLU(const Mat &gate, const Mat &vals, Mat *out);
void BackpropLoLU(const Mat &gate, const Mat &vals, const Mat &grad, Mat *gradGate, Mat *gradVals);
// src/gpt/att/rope.cpp:28-35, 77-83
void FillRopeBuf(Mat *rope, int width, int len);
void ApplyRope(const Mat &rope, float dir, Mat *p);
// src/gpt/att/att.cpp:25-55
AttInfo TransposeAttention(const AttInfo &att);

// TAttentionComputer, src/gpt/compute/layer_att_reference.h:23-212
struct Attention {
    Mat sumWeight, maxDP; // [head][t]
    float dotScale = 0, alibiSlope = 0;
    int headCount = 0, qDim = 0, ttDim = 0;
    void Init(int headCount_, int qDim_, int ttDim_, float alibiSlope_);
    void ComputeValLookup(const Mat &q, const Mat &k, const Mat &v, const AttInfo &att, Mat *valLookup);
    void GradQ(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &att, Mat *dq);
    void GradK(const Mat &q, const Mat &k, const Mat &v, const Mat &dValLookup, const Mat &dScale, const AttInfo &revAtt, Mat *dk,
               Mat *dv);
};
// src/gpt/compute/layer_att_reference.h:6-20, result [head][t]
void ComputeDScale(int headCount, int ttDim, const Mat &valLookup, const Mat &dValLookup, Mat *dScale);
} // namespace prim
} // namespace ts2o
