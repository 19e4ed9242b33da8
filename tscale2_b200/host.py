"""Host-side mirror of the reference types that feed the compute backend:
TModelDescr / TModelDims (src/gpt/model_params/model_dim.h:118-258), the batch
TBatchNodes built by InitLabelData (src/gpt/att/sliding_window.cpp:120-306) and
TTrainingStep (src/gpt/train_config/train_step.h).  numpy only; the arrays made
here are handed to the C ABI as plain pointers."""
import ctypes as C
from dataclasses import dataclass, field
from typing import List, Tuple

import numpy as np

from . import capi


@dataclass
class LayerSpec:
    layer_type: int
    alibi_slope: float = 0.0
    attention_type_id: int = 0


@dataclass
class ModelSpec:
    """TModelDescr.  dim % 128 == 0; q_dim = tt_dim = 128 (cfg_precision.h:79-80)."""
    dim: int
    head_count: int
    ffn_tiles: int
    vocab: int
    layers: List[LayerSpec] = field(default_factory=list)
    attention_widths: List[int] = field(default_factory=lambda: [1024])
    expert_dim: int = 128
    moe_expert_count: int = 0
    moe_selected: int = 2
    flags: int = 0
    precision: int = capi.PREC_FP8
    q_dim: int = 128
    tt_dim: int = 128
    labels: int = 0  # embedding rows; 0: vocab + 1

    @property
    def label_count(self) -> int:
        # GetLabelCount with MPF_DISABLE_NOISE_LABELS: InputTokenCount + 1 (sliding_window.cpp:47-68)
        return self.labels or self.vocab + 1

    def add_blocks(self, n_blocks: int, attention_type_id=0, alibi_slope=0.0, moe=False):
        for _ in range(n_blocks):
            self.layers.append(LayerSpec(capi.LAYER_ATT, alibi_slope, attention_type_id))
            self.layers.append(LayerSpec(capi.LAYER_MOE if moe else capi.LAYER_FFN))
        return self

    def matrix_shapes(self) -> List[Tuple[int, int]]:
        """(y_size=out, x_size=in) per matrix, in the order of the C ABI
        (EnumLayerMatrices, model_dim.h:219-258)."""
        q = self.q_dim * self.head_count
        tt = self.tt_dim * self.head_count
        f = 128 * self.ffn_tiles
        shapes = [(self.label_count, self.dim), (self.vocab, self.dim)]
        for l in self.layers:
            if l.layer_type == capi.LAYER_ATT:
                shapes += [(q, self.dim), (q, self.dim), (tt, self.dim), (tt, self.dim), (self.dim, tt)]
            elif l.layer_type == capi.LAYER_FFN:
                shapes += [(f, self.dim), (f, self.dim), (self.dim, f)]
            elif l.layer_type == capi.LAYER_MOE:
                xp, e = self.expert_dim, self.moe_expert_count
                shapes += [(xp * e, self.dim), (xp * e, self.dim), (self.dim * e, xp), (e, self.dim)]
            else:
                raise ValueError("unsupported layer type")
        return shapes

    def matrix_names(self) -> List[str]:
        names = ["embed", "final"]
        for i, l in enumerate(self.layers):
            if l.layer_type == capi.LAYER_ATT:
                names += [f"L{i}.att.{n}" for n in ("q", "k", "v", "gate", "combiner")]
            elif l.layer_type == capi.LAYER_FFN:
                names += [f"L{i}.ffn.{n}" for n in ("expand", "gate", "contract")]
            else:
                names += [f"L{i}.moe.{n}" for n in ("expand", "gate", "contract", "select")]
        return names

    def matrix_sparsity(self) -> List[float]:
        """Fraction of the tokens a matrix sees (TModelMatrix::Sparsity; EnumLayerMatrices, model_dim.h:230,252-254):
        selected / experts for the expert matrices of a mixture-of-experts layer, 1 elsewhere."""
        out = [1.0, 1.0]
        for l in self.layers:
            if l.layer_type == capi.LAYER_MOE:
                out += [self.moe_selected / self.moe_expert_count] * 3 + [1.0]
            else:
                out += [1.0] * (5 if l.layer_type == capi.LAYER_ATT else 3)
        return out

    def param_count(self) -> int:
        return sum(a * b for a, b in self.matrix_shapes())

    def to_c(self):
        """Returns (ModelDescr, keepalive)."""
        arr = (capi.LayerParams * len(self.layers))()
        for i, l in enumerate(self.layers):
            arr[i] = capi.LayerParams(l.layer_type, l.alibi_slope, l.attention_type_id)
        d = capi.ModelDescr(
            self.dim, self.q_dim, self.tt_dim, self.head_count, self.ffn_tiles, self.expert_dim,
            self.moe_expert_count, self.moe_selected, self.label_count, self.vocab,
            len(self.attention_widths), len(self.layers), arr, self.flags, self.precision, 0)
        return d, arr


def dp_layout(spec: ModelSpec):
    """(matrix_offset, bucket_offset, bucket_elems, bucket_first_matrix) of the engine's flat parameter buffers
    (ts2_dp_layout): what a data-parallel rank owns is bucket_elems / world elements of every bucket."""
    lib = capi.load_library()
    descr, keep = spec.to_c()
    n = len(spec.matrix_shapes())
    nb = 2 + sum(4 if l.layer_type == capi.LAYER_MOE else 1 for l in spec.layers)
    mo, bo, be = np.zeros(n, np.int64), np.zeros(nb, np.int64), np.zeros(nb, np.int64)
    bf = np.zeros(nb, np.int32)
    p64 = C.POINTER(C.c_int64)
    rc = lib.ts2_dp_layout(C.byref(descr), mo.ctypes.data_as(p64), n, bo.ctypes.data_as(p64), be.ctypes.data_as(p64),
                           bf.ctypes.data_as(C.POINTER(C.c_int32)), nb)
    if rc != nb:
        raise capi.Ts2Error(rc, lib.ts2_last_error(None).decode())
    return mo, bo, be, bf


def moe_exchange_plan(world: int, rank: int, counts: np.ndarray) -> dict:
    """The expert-parallel exchange of one mixture-of-experts layer as rank `rank` plans it from all ranks' per-expert
    row counts counts[world][experts] (ts2_moe_exchange_plan; host arithmetic of the CUDA library, no device needed).
    out / recv: arrays of (peer, first row in the sender's own layout or -1, first row in the owner's layout, rows)."""
    lib = capi.load_library()
    counts = np.ascontiguousarray(counts, np.int32)
    E = counts.shape[1]
    own_seg, x_seg, x_valid = np.zeros(E + 1, np.int32), np.zeros(E + 1, np.int32), np.zeros(E, np.int32)
    cap = E * (world + 1)
    moves = np.zeros((cap, 4), np.int32)
    n_out, n_in, max_x = C.c_int(), C.c_int(), C.c_int()
    rc = lib.ts2_moe_exchange_plan(world, rank, E, counts.ctypes.data, own_seg.ctypes.data, x_seg.ctypes.data, x_valid.ctypes.data,
                                   moves.ctypes.data, cap, C.byref(n_out), C.byref(n_in), C.byref(max_x))
    if rc != capi.TS2_OK:
        raise capi.Ts2Error(rc, lib.ts2_last_error(None).decode())
    return dict(own_seg=own_seg, x_seg=x_seg, x_valid=x_valid, out=moves[:n_out.value].copy(),
                recv=moves[n_out.value:n_out.value + n_in.value].copy(), max_x_rows=max_x.value)


def init_weights(spec: ModelSpec, seed: int, std: float = 0.02, select_std: float = None) -> List[np.ndarray]:
    """fp32 master weights ~ N(0, std) from numpy's default_rng(seed)."""
    rng = np.random.default_rng(seed)
    mats = []
    names = spec.matrix_names()
    for name, (y, x) in zip(names, spec.matrix_shapes()):
        s = select_std if (select_std is not None and name.endswith("moe.select")) else std
        mats.append((rng.standard_normal((y, x), dtype=np.float32) * np.float32(s)).astype(np.float32))
    return mats


def matrix_views(mats: List[np.ndarray]):
    arr = (capi.MatrixView * len(mats))()
    for i, m in enumerate(mats):
        assert m.dtype == np.float32 and m.flags["C_CONTIGUOUS"]
        arr[i] = capi.MatrixView(m.ctypes.data_as(C.POINTER(C.c_float)), m.shape[1], m.shape[0])
    return arr


class Batch:
    """TBatchNodes for fragments of tokens: one label per node (1 + token), at most one
    causal span per node [max(fragment start, t - width), t - 1] per attention type
    (AddAttSpans, sliding_window.cpp:113-118), target = the next token."""

    def __init__(self, fragments: np.ndarray, attention_widths: List[int]):
        fragments = np.asarray(fragments)
        n_frag, flen = fragments.shape
        length = flen - 1
        T = n_frag * length
        self.node_count = T
        self.label_arr = (fragments[:, :length].reshape(-1).astype(np.uint32) + np.uint32(1))
        self.label_ptr = np.arange(T + 1, dtype=np.uint32)
        self.target_node = np.arange(T, dtype=np.int32)
        self.target_id = fragments[:, 1:].reshape(-1).astype(np.int32)
        t = np.arange(T, dtype=np.int64)
        doc_start = (t // length) * length
        self.att = []
        for w in attention_widths:
            start = np.maximum(doc_start, t - w)
            finish = t - 1
            has = finish >= start
            ptr = np.concatenate([[0], np.cumsum(has)]).astype(np.int32)
            self.att.append((start[has].astype(np.int32), finish[has].astype(np.int32), ptr))
        self._build_c()

    @classmethod
    def from_arrays(cls, node_count, label_arr, label_ptr, target_node, target_id, att) -> "Batch":
        """A batch from its raw arrays as TBatchNodes holds them (src/gpt/att/nodes_batch.h): any number of labels per
        node (bit 31 = negative), att = [(span_start, span_finish, span_ptr)] per attention type."""
        b = object.__new__(cls)
        b.node_count = int(node_count)
        b.label_arr = np.ascontiguousarray(label_arr, np.uint32)
        b.label_ptr = np.ascontiguousarray(label_ptr, np.uint32)
        b.target_node = np.ascontiguousarray(target_node, np.int32)
        b.target_id = np.ascontiguousarray(target_id, np.int32)
        b.att = [tuple(np.ascontiguousarray(x, np.int32) for x in a) for a in att]
        b._build_c()
        return b

    def _build_c(self):
        ip = C.POINTER(C.c_int32)
        up = C.POINTER(C.c_uint32)
        self._att_c = (capi.AttentionInfo * len(self.att))()
        for i, (s, f, p) in enumerate(self.att):
            self._att_c[i] = capi.AttentionInfo(s.ctypes.data_as(ip), f.ctypes.data_as(ip), p.ctypes.data_as(ip))
        self.c = capi.BatchNodes(
            self.node_count, self.label_arr.ctypes.data_as(up), self.label_ptr.ctypes.data_as(up),
            len(self.target_node), self.target_node.ctypes.data_as(ip), self.target_id.ctypes.data_as(ip),
            len(self.att), self._att_c)

    @property
    def h2d_bytes(self) -> int:
        n = self.label_arr.nbytes + self.label_ptr.nbytes + self.target_node.nbytes + self.target_id.nbytes
        for s, f, p in self.att:
            n += s.nbytes + f.nbytes + p.nbytes
        return n


def synthetic_batch(spec: ModelSpec, n_fragments: int, seq_len: int, seed: int) -> Batch:
    """Uniform random tokens (the stand-in for the tokenized datasets the reference trains on)."""
    rng = np.random.default_rng(seed)
    frags = rng.integers(0, spec.vocab, size=(n_fragments, seq_len + 1), dtype=np.int64)
    return Batch(frags, spec.attention_widths)


def training_step(rate=0.01, l2reg=0.0, iteration=0) -> capi.TrainingStep:
    """TDescentConfig::GetStep without tail / slow start (src/gpt/train_config/train_config.h:27-52)."""
    decay = 1.0 - 0.5 / np.sqrt(1.0 + iteration)
    return capi.TrainingStep(rate, l2reg, decay, 0.2, 0.8, decay)
