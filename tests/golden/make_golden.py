"""Generates the golden fixtures in this directory from the REFERENCE-LINKED
oracle build (oracle/_ref/libts2_oracle_ref.so: the reference's own compiled
cpu_util.cpp / layer_att_reference.h / rope.cpp / att.cpp under the restated
layer drivers).  Run in a container that has the reference sources:

    make -C oracle ref && python tests/golden/make_golden.py

The fixtures hold per-tensor norms and a strided sample of every tensor (full
tensors would be tens of MB); tests/test_oracle_golden.py checks the restated
oracle (oracle/libts2_oracle.so) against them on any machine."""
import ctypes as C
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402
from tscale2_b200 import capi, host  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
STRIDE = 251


def configs():
    """name -> (spec, weight seed, batch(n_fragments, seq_len, seed), weight_quant)."""
    c1 = host.ModelSpec(dim=256, head_count=4, ffn_tiles=8, vocab=4096, attention_widths=[128]).add_blocks(2)
    c1_alibi = host.ModelSpec(dim=256, head_count=4, ffn_tiles=8, vocab=4096, attention_widths=[64]).add_blocks(
        2, alibi_slope=0.5)
    tiny_moe = host.ModelSpec(dim=128, head_count=1, ffn_tiles=2, vocab=256, attention_widths=[16, 48], expert_dim=128,
                              moe_expert_count=4, moe_selected=2)
    tiny_moe.add_blocks(1, attention_type_id=0).add_blocks(1, attention_type_id=1, alibi_slope=0.25, moe=True)
    return {
        "c1_e4m3": (c1, 1234, (4, 128, 4321), oracle.QUANT_E4M3),
        "c1_half": (c1, 1234, (4, 128, 4321), oracle.QUANT_HALF),
        "c1_alibi_i8": (c1_alibi, 1234, (4, 128, 4321), oracle.QUANT_I8),
        "tiny_moe_e4m3": (tiny_moe, 77, (3, 40, 78), oracle.QUANT_E4M3),
    }


def summarize(res):
    out = {"score": np.float64(res["score"]), "target_prob": res["target_prob"][::7].copy()}
    for i, g in enumerate(res["grads"]):
        out[f"grad_norm_{i}"] = np.float64(np.linalg.norm(g.astype(np.float64)))
        out[f"grad_sample_{i}"] = g.reshape(-1)[::STRIDE].copy()
    for name in ("states", "state_grads"):
        a = res[name]
        out[f"{name}_norm"] = np.linalg.norm(a.astype(np.float64).reshape(a.shape[0], -1), axis=1)
        out[f"{name}_sample"] = a.reshape(-1)[::STRIDE].copy()
    return out


def run(o, name):
    spec, wseed, (nf, sl, bseed), quant = configs()[name]
    sel = 1.0 if spec.moe_expert_count else None
    mats = host.init_weights(spec, wseed, select_std=sel)
    batch = host.synthetic_batch(spec, nf, sl, bseed)
    return o.backprop(spec, mats, batch, quant, want_states=True)


def primitive_vectors(o):
    """Number-format conversions of the reference (sse_utils.h) on seeded inputs."""
    rng = np.random.default_rng(99)
    n = 4096
    src = (rng.standard_normal(n) * rng.choice([0.01, 1.0, 30.0, 200.0, 1000.0], n)).astype(np.float32)
    src[:8] = [0.0, -0.0, 448.0, -448.0, 464.0, 1e-3, 0.0078125, -0.0078125]
    def aligned(count, dtype):  # the reference uses aligned 256-bit loads and stores
        raw = np.zeros(count * np.dtype(dtype).itemsize + 64, np.uint8)
        off = (-raw.ctypes.data) % 32
        return raw[off:off + count * np.dtype(dtype).itemsize].view(dtype)

    a = aligned(n, np.float32)
    a[:] = src
    e4 = aligned(n, np.uint8)
    i8 = aligned(n, np.int8)
    L = o.lib
    L.ts2o_ref_convert_e4m3.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
    L.ts2o_ref_convert_i8.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
    L.ts2o_ref_e4m3_to_float.restype = C.c_float
    L.ts2o_ref_e4m3_to_float.argtypes = [C.c_uint8]
    L.ts2o_ref_convert_e4m3(e4.ctypes.data, a.ctypes.data, n, 1.0)
    L.ts2o_ref_convert_i8(i8.ctypes.data, a.ctypes.data, n, 0.5)
    table = np.array([L.ts2o_ref_e4m3_to_float(b) for b in range(256)], np.float32)
    return dict(src=src, e4m3=e4.copy(), i8_half=i8.copy(), e4m3_table=table)


def main():
    o = oracle.Oracle("ref")
    assert o.backend() == "reference"
    for name in configs():
        if len(sys.argv) > 1 and name not in sys.argv[1:]:
            continue
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **summarize(run(o, name)))
        print("wrote", name)
    np.savez_compressed(os.path.join(HERE, "conversions.npz"), **primitive_vectors(o))
    print("wrote conversions")


if __name__ == "__main__":
    main()
