"""What can be checked of the CUDA library without a GPU: it loads, exports every symbol
that include/ts2_b200.h declares, and refuses to run without a device (no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from tscale2_b200 import capi, host

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(capi.LIB_PATH):
        from tscale2_b200 import build
        build.build()
    return capi.load_library()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ts2_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ts2_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ts2_b200.h but not exported"
    assert not lib._ts2_missing
    # and the ctypes table covers the header
    assert set(names) == set(lib._ts2_signatures), set(names) ^ set(lib._ts2_signatures)


def test_no_cpu_fallback(lib):
    if lib.ts2_device_count() > 0:
        pytest.skip("a CUDA device is present")
    spec = host.ModelSpec(dim=128, head_count=1, ffn_tiles=1, vocab=128).add_blocks(1)
    mats = host.init_weights(spec, 1)
    descr, keep = spec.to_c()
    h = C.c_void_p()
    rc = lib.ts2_create(C.byref(descr), host.matrix_views(mats), len(mats), None, 0, 128, C.byref(h))
    assert rc == capi.TS2_ERR_NO_DEVICE
    assert b"no CPU fallback" in lib.ts2_last_error(None)


def test_description_is_validated_without_a_device(lib):
    spec = host.ModelSpec(dim=256, head_count=2, ffn_tiles=4, vocab=512).add_blocks(2)
    descr, keep = spec.to_c()
    assert lib.ts2_matrix_count(C.byref(descr)) == 2 + 2 * 8
    x, y = C.c_int64(), C.c_int64()
    for i, (yy, xx) in enumerate(spec.matrix_shapes()):
        assert lib.ts2_matrix_shape(C.byref(descr), i, C.byref(x), C.byref(y)) == 0
        assert (x.value, y.value) == (xx, yy)
    bad = host.ModelSpec(dim=200, head_count=2, ffn_tiles=4, vocab=512).add_blocks(1)
    d2, k2 = bad.to_c()
    assert lib.ts2_matrix_count(C.byref(d2)) == capi.TS2_ERR_INVALID_ARG
    d3, k3 = spec.to_c()
    d3.q_dim = 64  # head dim 64 is not what the reference computes with (Q_DIM = 128)
    assert lib.ts2_matrix_count(C.byref(d3)) == capi.TS2_ERR_UNSUPPORTED
    for flag in (0x10, 0x10000, 0x20000):  # MPF_SAMPLE_EMBED_VECTORS, MPF_RNN, MPF_RNN_CROSS change the compute path
        d4, k4 = spec.to_c()
        d4.flags = flag
        assert lib.ts2_matrix_count(C.byref(d4)) == capi.TS2_ERR_UNSUPPORTED
    d5, k5 = spec.to_c()
    d5.flags = 0x800 | 0x4  # MPF_DISABLE_NOISE_LABELS, MPF_USE_DOC_START_TOKEN: data preparation only
    assert lib.ts2_matrix_count(C.byref(d5)) == 2 + 2 * 8


def test_host_batch_matches_reference_span_rule():
    """[max(fragment start, t - width), t - 1] per node, none for the first node of a fragment."""
    spec = host.ModelSpec(dim=128, head_count=1, ffn_tiles=1, vocab=64, attention_widths=[4, 1000])
    b = host.synthetic_batch(spec, 2, 10, 3)
    assert b.node_count == 20
    s, f, p = b.att[0]
    assert p[1] == 0 and p[2] == 1 and p[11] - p[10] == 0  # nodes 0 and 10 start fragments
    assert (s[0], f[0]) == (0, 0)  # node 1 sees node 0
    k = p[7]
    assert (s[k], f[k]) == (3, 6)  # node 7, width 4
    s, f, p = b.att[1]
    k = p[15]
    assert (s[k], f[k]) == (10, 14)
    assert np.array_equal(b.label_arr[:3], b.target_id[:0].astype(np.uint32).tolist() + list(b.label_arr[:3]))
    assert b.label_arr.max() <= spec.vocab and b.label_arr.min() >= 1


def test_reference_side_adapter_compiles_against_the_reference_headers():
    """tscale2_b200/adapter/b200_model.cpp is the IModel / IModelInstance a maintainer adds to the trainer.  Where the
    reference's sources are present it must pass a syntax check against their own model.h (all pure virtuals
    overridden with the right signatures)."""
    import shutil
    import subprocess
    ref = os.environ.get("TS2_REFERENCE", "/root/reference")
    if not os.path.exists(os.path.join(ref, "src", "gpt", "compute", "model.h")) or not shutil.which("g++"):
        pytest.skip("reference sources or g++ not present on this machine")
    cmd = ["g++", "-std=c++17", "-march=x86-64-v3", "-w", "-fsyntax-only", "-include", "util/pch.h", "-I" + os.path.join(ref, "src"),
           "-I/usr/local/cuda/include", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tscale2_b200", "adapter", "b200_model.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
