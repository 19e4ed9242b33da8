// Reference-side binding of libts2b200.so: an IModel / IModelInstance (src/gpt/compute/model.h:22-56) that forwards
// to the C ABI of include/ts2_b200.h.  A maintainer of the trainer adds this file to src/gpt/compute/ and one more
// branch to CreateTrainModel (src/gpt/train/main_gpt.cpp:34-47):
//     return CreateB200Transformer(params, deviceId, nodeCount);
// One process drives one GPU; for data parallel each process calls B200CommInit with the id rank 0 made.
//
// It is compiled here only as a syntax check against the reference's own headers
// (g++ -fsyntax-only -include util/pch.h -I<reference>/src -I<cuda>/include -I<this repo>/include).
#include <gpt/compute/model.h>
#include <ts2_b200.h>
#include <vector>

class TB200Model : public IModel, public IModelInstance
{
    TModelParams Params; // host copy: shapes, description, and the buffers GetParams hands back
    ts2_model *H = nullptr;
    TBatchNodes Nodes;
    TArray2D<float> SampleEmbed;
    std::vector<ts2_layer_params> Layers;

    // the trainer aborts on errors (Y_VERIFY); the library itself returns codes
    static void Check(int rc, ts2_model *h)
    {
        if (rc != TS2_OK) {
            DebugPrintf("ts2_b200: %s\n", ts2_last_error(h));
            abort();
        }
    }

    // matrix order of the C ABI: embedding, final layer, then every layer's matrices (EnumLayerMatrices order)
    template <class F>
    static void ForEachMatrix(TModelParams &p, F f)
    {
        f(p.MatrArr[MP_MODEL_EMBED]);
        f(p.MatrArr[MP_MODEL_FINAL]);
        for (TModelParams::TAttentionMatrices &layer : p.LayerArr) {
            for (TModelMatrix &mm : layer.MatrArr) {
                f(mm);
            }
        }
    }

    static ts2_matrix_view View(TArray2D<float> &a)
    {
        ts2_matrix_view v;
        v.data = a.GetRow(0); // TArray2D keeps its rows contiguous
        v.x_size = a.GetXSize();
        v.y_size = a.GetYSize();
        return v;
    }

public:
    TB200Model(const TModelParams &params, yint device, yint nodeCount, int precision) : Params(params)
    {
        const TModelDescr &d = Params.ModelDescr;
        for (const TModelDescr::TLayerParams &lp : d.LayerArr) {
            ts2_layer_params x;
            x.layer_type = (int32_t)lp.LayerType;
            x.alibi_slope = lp.AlibiSlope;
            x.attention_type_id = lp.AttentionTypeId;
            Layers.push_back(x);
        }
        ts2_model_descr md;
        memset(&md, 0, sizeof(md));
        md.dim = d.Dims.Dim;
        md.q_dim = d.Dims.QDim;
        md.tt_dim = d.Dims.TTDim;
        md.head_count = d.Dims.HeadCount;
        md.ffn_tiles = d.Dims.FfnTiles;
        md.expert_dim = d.Dims.ExpertDim;
        md.moe_expert_count = d.Dims.MoeExpertCount;
        md.moe_selected = d.Dims.MoeSelected;
        md.label_count = (int32_t)d.LabelCount;
        md.output_token_count = (int32_t)d.OutputTokenCount;
        md.attention_type_count = (int32_t)d.GetAttentionTypeCount();
        md.layer_count = (int32_t)Layers.size();
        md.layers = Layers.data();
        md.flags = d.Flags;
        md.precision = precision;
        std::vector<ts2_matrix_view> views;
        ForEachMatrix(Params, [&](TModelMatrix &mm) { views.push_back(View(mm.GetMatrix())); });
        Check(ts2_create(&md, views.data(), (int)views.size(), Params.Bias.data(), (int)device, (int)nodeCount, &H), nullptr);
        SetParams(Params); // momentum of a loaded checkpoint
    }
    ~TB200Model() { ts2_destroy(H); }
    ts2_model *GetHandle() { return H; }

    // ---- IModel ----
    const TModelDescr &GetModelDescr() override { return Params.ModelDescr; }
    // The parameters live on the device behind the C ABI; there is no per-matrix host object to hand out.
    // Callers that only train (TrainModel, BackpropBatch, CalcModelErr) never ask for these.
    TPtrArg<IModelOps> GetModelOps() override { return TPtrArg<IModelOps>(nullptr); }
    TPtrArg<IModelStorage> GetModelStorage() override { return TPtrArg<IModelStorage>(nullptr); }

    void GetParams(TModelParams *p) override
    {
        *p = Params;
        std::vector<ts2_matrix_view> w, g;
        ForEachMatrix(*p, [&](TModelMatrix &mm) {
            w.push_back(View(mm.GetMatrix()));
            g.push_back(View(mm.GetGrad1()));
        });
        Check(ts2_get_params(H, TS2_PARAM_WEIGHTS, w.data(), (int)w.size()), H);
        Check(ts2_get_params(H, TS2_PARAM_MOMENTUM, g.data(), (int)g.size()), H);
        int index = 0;
        ForEachMatrix(*p, [&](TModelMatrix &mm) {
            TVector<float> rowDisp = mm.GetRowDisp();
            float sumWeight = 0;
            Check(ts2_get_row_disp(H, index++, rowDisp.data(), (int64_t)YSize(rowDisp), &sumWeight), H);
            mm.SetRowDisp(sumWeight, rowDisp);
        });
    }

    void SetParams(const TModelParams &p) override
    {
        Params = p;
        std::vector<ts2_matrix_view> w, g;
        ForEachMatrix(Params, [&](TModelMatrix &mm) {
            w.push_back(View(mm.GetMatrix()));
            g.push_back(View(mm.GetGrad1()));
        });
        Check(ts2_set_params(H, TS2_PARAM_WEIGHTS, w.data(), (int)w.size()), H);
        Check(ts2_set_params(H, TS2_PARAM_MOMENTUM, g.data(), (int)g.size()), H);
    }

    TIntrusivePtr<IModelInstance> GetInstance(yint modelInstanceId) override
    {
        Y_VERIFY(modelInstanceId == 0 && "one instance per process: one process drives one GPU");
        return this;
    }

    void Backprop(const TTrainingStep &s, EAddToModel addToModel) override
    {
        ts2_training_step st = {s.Rate, s.L2Reg, s.Beta1, s.Weight0, s.Weight1, s.DispDecay};
        Check(ts2_backprop(H, &st, addToModel == GRADIENT_APPLY ? TS2_GRADIENT_APPLY : TS2_GRADIENT_ACCUMULATE), H);
    }
    void WaitAllCompute() override { Check(ts2_wait(H), H); }
    float GetAvrgTrainErr() override
    {
        float e = 0;
        Check(ts2_avg_train_err(H, &e), H);
        return e;
    }

    // ---- IModelInstance ----
    void WaitInstanceOpLaunch() override {} // ts2_set_batch has copied the host arrays when it returns
    TBatchNodes &GetNodes(yint microBatchId) override
    {
        Y_VERIFY(microBatchId == 0);
        return Nodes;
    }
    TArray2D<float> &GetSampleEmbedVectors(yint microBatchId) override
    {
        Y_VERIFY(microBatchId == 0);
        return SampleEmbed;
    }
    void Init(EInitType) override
    {
        // TAttentionSpan {Start, Finish} pairs -> the two arrays of ts2_attention_info
        std::vector<std::vector<int32_t>> starts(Nodes.AttArr.size()), finishes(Nodes.AttArr.size());
        std::vector<ts2_attention_info> att(Nodes.AttArr.size());
        for (size_t a = 0; a < att.size(); ++a) {
            const TAttentionInfo &ai = Nodes.AttArr[a];
            for (const TAttentionSpan &sp : ai.Spans) {
                starts[a].push_back(sp.Start);
                finishes[a].push_back(sp.Finish);
            }
            att[a].span_start = starts[a].data();
            att[a].span_finish = finishes[a].data();
            att[a].span_ptr = ai.SpanPtr.data();
        }
        std::vector<int32_t> targetNode, targetId;
        for (const TNodeTarget &t : Nodes.Target) {
            targetNode.push_back((int32_t)t.Node);
            targetId.push_back((int32_t)t.TargetId);
        }
        ts2_batch_nodes b;
        b.node_count = (int32_t)Nodes.GetNodeCount();
        b.label_arr = Nodes.Labels.LabelArr.data();
        b.label_ptr = Nodes.Labels.LabelPtr.data();
        b.target_count = (int32_t)targetNode.size();
        b.target_node = targetNode.data();
        b.target_id = targetId.data();
        b.attention_type_count = (int32_t)att.size();
        b.att = att.data();
        Check(ts2_set_batch(H, &b), H);
    }
    // inference outputs are outside the path this library replaces
    void ComputeFragmentPredictions(TVector<TVector<float>> *) override { Y_VERIFY(0 && "not provided by the B200 training backend"); }
    void ComputeFragmentPredictions(TVector<float> *) override { Y_VERIFY(0 && "not provided by the B200 training backend"); }
    float ComputeScore() override
    {
        float s = 0;
        Check(ts2_forward_score(H, &s), H);
        return s;
    }
};


TIntrusivePtr<IModel> CreateB200Transformer(const TModelParams &params, yint device, yint nodeCount)
{
    // the reference picks the arithmetic at compile time (cfg_precision.h:18-46); follow its weight type
    const int precision = sizeof(TFastModelFloat) == 2 ? TS2_PREC_F16 : TS2_PREC_FP8;
    return new TB200Model(params, device, nodeCount, precision);
}

// data parallel over the GPUs of one box: rank 0 obtains the id with ts2_comm_unique_id and passes the 128 bytes to
// the other trainer processes (the trainer's own master / worker TCP protocol will do)
void B200CommInit(IModel *model, yint rank, yint rankCount, const ui8 *id)
{
    TB200Model *m = dynamic_cast<TB200Model *>(model);
    Y_VERIFY(m && "not a B200 model");
    if (ts2_comm_init(m->GetHandle(), (int)rank, (int)rankCount, id) != TS2_OK) {
        DebugPrintf("ts2_b200: %s\n", ts2_last_error(m->GetHandle()));
        abort();
    }
}

// mixture-of-experts models: after B200CommInit on every rank, divides the experts over the ranks (the counterpart of
// TCudaMoELayer::GetExpertSpan over a device group, src/gpt/compute/layer_moe.cu:52-66); capacityFactor 0 = default
void B200SetExpertParallel(IModel *model, float capacityFactor)
{
    TB200Model *m = dynamic_cast<TB200Model *>(model);
    Y_VERIFY(m && "not a B200 model");
    if (ts2_set_expert_parallel(m->GetHandle(), capacityFactor) != TS2_OK) {
        DebugPrintf("ts2_b200: %s\n", ts2_last_error(m->GetHandle()));
        abort();
    }
}
