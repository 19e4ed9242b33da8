// TEST INFRASTRUCTURE — writes / re-reads a model file with the reference's OWN serializer
// (Serialize / IBinSaver, src/util/bin_saver.h; TModelParams SAVELOAD, src/gpt/model_params/model_params.h:7-18),
// compiled against the reference headers where they lie (oracle/Makefile, target ckpt).  Used to make the golden
// file tests/golden/tiny_model.bin and to check that a file written by tscale2_b200/checkpoint.py loads in the
// reference's code.
//   ckpt_ref write <file>   : a small deterministic model (values are simple functions of the indices)
//   ckpt_ref check <file>   : loads <file>, prints one line of facts (shapes, sums) for the caller to compare
#include <gpt/model_params/model_params.h>
#include <cstdio>

static void Fill(TModelMatrix *mm, yint xSize, yint ySize, yint rowDispSize, float sparsity, int salt)
{
    mm->SetSizes(xSize, ySize, rowDispSize, sparsity);
    TArray2D<float> &w = mm->GetMatrix(), &g = mm->GetGrad1();
    for (yint y = 0; y < ySize; ++y) {
        for (yint x = 0; x < xSize; ++x) {
            w[y][x] = (float)(((x * 7 + y * 13 + salt) % 31) - 15) / 64;
            g[y][x] = (float)(((x * 3 + y * 5 + salt) % 17) - 8) / 256;
        }
    }
    TVector<float> rd;
    for (yint i = 0; i < rowDispSize; ++i) {
        rd.push_back(0.25f + (float)((i + salt) % 5) / 8);
    }
    mm->SetRowDisp(1.5f + salt, rd);
}

int main(int argc, char **argv)
{
    if (argc != 3) {
        return 2;
    }
    TString mode = argv[1], fname = argv[2];
    if (mode == "write") {
        TModelParams p;
        TModelDescr &d = p.ModelDescr;
        d.Dims.Dim = 128;
        d.Dims.HeadCount = 1;
        d.Dims.FfnTiles = 1;
        d.Dims.Depth = 2;
        d.LabelCount = 33;
        d.InputTokenCount = 32;
        d.OutputTokenCount = 32;
        d.AttentionTypeArr.push_back(CasualAttn(16));
        d.AddLayer(MLT_ATT, 0, 0.25f);
        d.AddLayer(MLT_FFN);
        d.Flags = MPF_DISABLE_NOISE_LABELS;
        d.FragLen = 16;
        p.MatrArr.resize(MP_MODEL_COUNT);
        Fill(&p.MatrArr[MP_MODEL_EMBED], d.Dims.Dim, d.LabelCount, d.LabelCount, 1, 1);
        Fill(&p.MatrArr[MP_MODEL_FINAL], d.Dims.Dim, d.OutputTokenCount, d.OutputTokenCount, 1, 2);
        p.LayerArr.resize(d.GetDepth());
        int salt = 3;
        for (yint l = 0; l < d.GetDepth(); ++l) {
            d.EnumLayerMatrices(l, [&](yint xSize, yint ySize, yint, float sparsity) {
                TModelMatrix mm;
                Fill(&mm, xSize, ySize, 1, sparsity, salt++);
                p.LayerArr[l].MatrArr.push_back(mm);
            });
        }
        for (yint k = 0; k < d.OutputTokenCount; ++k) {
            p.Bias.push_back((float)(k % 7) / 16);
        }
        Serialize(IO_WRITE, fname, p);
        return 0;
    }
    if (mode == "check") {
        TModelParams p;
        Serialize(IO_READ, fname, p);
        double sum = 0, gsum = 0;
        yint count = 0;
        p.ForEachModelMatrix([&](TModelMatrix &mm) {
            for (yint y = 0; y < mm.GetYSize(); ++y) {
                for (yint x = 0; x < mm.GetXSize(); ++x) {
                    sum += mm.GetMatrix()[y][x];
                    gsum += mm.GetGrad1()[y][x];
                }
            }
            ++count;
        });
        printf("dim=%d heads=%d ffn=%d labels=%lld vocab=%lld layers=%lld matrices=%lld sum=%.6f gsum=%.6f bias=%lld flags=%llu\n",
            p.ModelDescr.Dims.Dim, p.ModelDescr.Dims.HeadCount, p.ModelDescr.Dims.FfnTiles, p.ModelDescr.LabelCount,
            p.ModelDescr.OutputTokenCount, (long long)YSize(p.ModelDescr.LayerArr), count, sum, gsum, (long long)YSize(p.Bias),
            (unsigned long long)p.ModelDescr.Flags);
        return 0;
    }
    return 2;
}
