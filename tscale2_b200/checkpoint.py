"""Model files in the reference's format: what its trainer writes with Serialize(IO_WRITE, fname, TModelParams)
(src/gpt/model_params/model_params.cpp:212-228) and its tools read back, so a model trained by this engine loads in the
reference's `infer` / `compute_exact_test` and the other way round.

The format is the reference's IBinSaver (src/util/bin_saver.h): plain-old-data values as their raw little-endian
bytes, a TVector as an int64 count followed by the elements (raw when the element is plain old data), a TArray2D as
int64 x size, int64 y size and the row-major data, a struct with SAVELOAD as its fields in order:

    TModelParams   = ModelDescr, LayerArr (per layer: MatrArr), MatrArr (embedding, final layer), Bias
                     (model_params.h:7-18)
    TModelDescr    = Dims, LabelCount, InputTokenCount, OutputTokenCount, AttentionTypeArr, LayerArr, Flags,
                     DocStartToken, FragLen                                     (model_dim.h:159-180)
    TModelDims     = Dim, QDim, TTDim, ExpertDim, HeadCount, FfnTiles, MoeExpertCount, MoeSelected, KVrep, Depth (int32)
    TModelMatrix   = Matr, Grad1 (momentum), SumWeight, RowDisp, Sparsity       (model_matrix.h:61-70)
"""
import io
import struct
from dataclasses import dataclass, field
from typing import List

import numpy as np

from . import host


@dataclass
class MatrixState:
    weights: np.ndarray          # [y][x] fp32
    momentum: np.ndarray         # Grad1, same shape
    sum_weight: float = 0.0
    row_disp: np.ndarray = field(default_factory=lambda: np.zeros(1, np.float32))
    sparsity: float = 1.0


@dataclass
class ModelFile:
    spec: host.ModelSpec
    matrices: List[MatrixState]  # C-ABI order: embedding, final layer, then every layer's matrices
    bias: np.ndarray
    input_token_count: int = 0
    attention_types: List[tuple] = field(default_factory=list)  # (width, type)
    doc_start_token: int = 0
    frag_len: int = 0
    kv_rep: int = 16
    depth: int = 60


class _Reader:
    def __init__(self, data):
        self.b = memoryview(data)
        self.p = 0

    def take(self, fmt):
        v = struct.unpack_from("<" + fmt, self.b, self.p)
        self.p += struct.calcsize("<" + fmt)
        return v if len(v) > 1 else v[0]

    def array(self, dtype, n):
        a = np.frombuffer(self.b, dtype, n, self.p).copy()
        self.p += a.nbytes
        return a

    def vec(self, dtype):
        return self.array(dtype, self.take("q"))

    def array2d(self):
        x, y = self.take("qq")
        return self.array(np.float32, x * y).reshape(y, x)

    def matrix(self):
        w, g = self.array2d(), self.array2d()
        sw = self.take("f")
        rd = self.vec(np.float32)
        return MatrixState(w, g, sw, rd, self.take("f"))


def load(path) -> ModelFile:
    with open(path, "rb") as f:
        r = _Reader(f.read())
    dim, q_dim, tt_dim, expert_dim, heads, ffn_tiles, experts, selected, kv_rep, depth = r.take("10i")
    label_count, input_tokens, output_tokens = r.take("qqq")
    n_att = r.take("q")
    att_types = [tuple(int(v) for v in r.array(np.int32, 2)) for _ in range(n_att)]
    n_layers = r.take("q")
    layers = []
    for _ in range(n_layers):
        lt, slope, att_id = r.take("ifi")
        layers.append(host.LayerSpec(lt, slope, att_id))
    flags, doc_start, frag_len = r.take("QQq")
    n_layer_arr = r.take("q")
    layer_mats = []
    for _ in range(n_layer_arr):
        layer_mats.append([r.matrix() for _ in range(r.take("q"))])
    top = [r.matrix() for _ in range(r.take("q"))]
    bias = r.vec(np.float32)
    if r.p != len(r.b):
        raise ValueError(f"{path}: {len(r.b) - r.p} bytes left over; not a TModelParams file of this format")
    # labels: models with noise labels or a document-start token have more embedding rows than vocabulary + 1
    spec = host.ModelSpec(dim=dim, head_count=heads, ffn_tiles=ffn_tiles, vocab=int(output_tokens), layers=layers,
                          attention_widths=[w for w, _ in att_types], expert_dim=expert_dim, moe_expert_count=experts,
                          moe_selected=selected, flags=int(flags), q_dim=q_dim, tt_dim=tt_dim, labels=int(label_count))
    mats = top + [m for lm in layer_mats for m in lm]
    return ModelFile(spec, mats, bias, int(input_tokens), att_types, int(doc_start), int(frag_len), kv_rep, depth)


def _w(out, fmt, *v):
    out.write(struct.pack("<" + fmt, *v))


def _w_array2d(out, a):
    a = np.ascontiguousarray(a, np.float32)
    _w(out, "qq", a.shape[1], a.shape[0])
    out.write(a.tobytes())


def _w_matrix(out, m: MatrixState):
    _w_array2d(out, m.weights)
    _w_array2d(out, m.momentum)
    _w(out, "f", m.sum_weight)
    rd = np.ascontiguousarray(m.row_disp, np.float32)
    _w(out, "q", rd.size)
    out.write(rd.tobytes())
    _w(out, "f", m.sparsity)


def save(path, mf: ModelFile):
    s = mf.spec
    out = io.BytesIO()
    _w(out, "10i", s.dim, s.q_dim, s.tt_dim, s.expert_dim, s.head_count, s.ffn_tiles, s.moe_expert_count, s.moe_selected,
       mf.kv_rep, mf.depth)
    _w(out, "qqq", mf.matrices[0].weights.shape[0], mf.input_token_count, s.vocab)
    att = mf.attention_types or [(w, 0) for w in s.attention_widths]
    _w(out, "q", len(att))
    for w, t in att:
        _w(out, "ii", w, t)
    _w(out, "q", len(s.layers))
    for l in s.layers:
        _w(out, "ifi", l.layer_type, l.alibi_slope, l.attention_type_id)
    _w(out, "QQq", s.flags, mf.doc_start_token, mf.frag_len)
    counts = {0: 5, 1: 5, 2: 3, 3: 4}  # ELayerType -> matrices (model_dim.h:219-258)
    _w(out, "q", len(s.layers))
    i = 2
    for l in s.layers:
        n = counts[l.layer_type]
        _w(out, "q", n)
        for m in mf.matrices[i:i + n]:
            _w_matrix(out, m)
        i += n
    _w(out, "q", 2)
    _w_matrix(out, mf.matrices[0])
    _w_matrix(out, mf.matrices[1])
    bias = np.ascontiguousarray(mf.bias, np.float32)
    _w(out, "q", bias.size)
    out.write(bias.tobytes())
    with open(path, "wb") as f:
        f.write(out.getvalue())


def from_model(model, bias=None, **kw) -> ModelFile:
    """Snapshot of an engine (tscale2_b200.model.Model): weights, momentum, dispersion of every matrix (GetParams)."""
    w, g = model.get_weights(), model.get_momentum()
    mats = []
    sparsity = model.spec.matrix_sparsity()
    for i, (a, b) in enumerate(zip(w, g)):
        rd, sw = model.get_row_disp(i)
        mats.append(MatrixState(a, b, sw, rd, sparsity[i]))
    vocab = model.spec.vocab
    return ModelFile(model.spec, mats, np.zeros(vocab, np.float32) if bias is None else np.asarray(bias, np.float32),
                     input_token_count=kw.pop("input_token_count", vocab), **kw)
