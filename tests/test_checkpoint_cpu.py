"""Model files in the reference's format (tscale2_b200/checkpoint.py).  tests/golden/tiny_model.bin.gz was written by
the reference's own serializer (oracle/ckpt_ref.cpp, `make -C oracle ckpt && oracle/_ref/ckpt_ref write <file>`):
reading it must give the model the tool built, writing it back must give the same bytes, and, where the
reference-linked tool is present, the reference's reader must load a file written here."""
import gzip
import os
import subprocess

import numpy as np
import pytest

from tscale2_b200 import capi, checkpoint

HERE = os.path.dirname(os.path.abspath(__file__))
TOOL = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "ckpt_ref")


@pytest.fixture()
def golden(tmp_path):
    raw = gzip.open(os.path.join(HERE, "golden", "tiny_model.bin.gz")).read()
    p = tmp_path / "tiny_model.bin"
    p.write_bytes(raw)
    return p, raw


def test_reads_what_the_reference_wrote(golden):
    path, _ = golden
    mf = checkpoint.load(path)
    s = mf.spec
    assert (s.dim, s.head_count, s.ffn_tiles, s.vocab, s.label_count) == (128, 1, 1, 32, 33)
    assert [l.layer_type for l in s.layers] == [capi.LAYER_ATT, capi.LAYER_FFN]
    assert s.layers[0].alibi_slope == 0.25 and mf.attention_types == [(16, 0)] and mf.frag_len == 16
    assert [m.weights.shape for m in mf.matrices] == s.matrix_shapes()
    # the tool fills w[y][x] = (((7 x + 13 y + salt) mod 31) - 15) / 64, momentum (((3 x + 5 y + salt) mod 17) - 8) / 256
    y, x = np.mgrid[0:33, 0:128]
    assert np.array_equal(mf.matrices[0].weights, (((x * 7 + y * 13 + 1) % 31) - 15).astype(np.float32) / 64)
    assert np.array_equal(mf.matrices[0].momentum, (((x * 3 + y * 5 + 1) % 17) - 8).astype(np.float32) / 256)
    assert mf.matrices[0].row_disp.size == 33 and mf.matrices[2].row_disp.size == 1
    assert mf.matrices[1].sum_weight == 3.5 and mf.matrices[4].sum_weight == 1.5 + 5
    assert np.array_equal(mf.bias, (np.arange(32) % 7).astype(np.float32) / 16)


def test_writes_the_same_bytes_back(golden, tmp_path):
    path, raw = golden
    out = tmp_path / "again.bin"
    checkpoint.save(out, checkpoint.load(path))
    assert out.read_bytes() == raw


def test_reference_reader_loads_a_file_written_here(golden, tmp_path):
    if not os.path.exists(TOOL):
        pytest.skip("reference-linked checkpoint tool not built on this machine")
    path, raw = golden
    mf = checkpoint.load(path)
    mf.matrices[3].weights[5, 7] = 2.0  # a changed model, so that the tool cannot be reading the golden file
    out = tmp_path / "changed.bin"
    checkpoint.save(out, mf)
    line = subprocess.run([TOOL, "check", str(out)], capture_output=True, text=True, check=True).stdout
    want = sum(float(m.weights.astype(np.float64).sum()) for m in mf.matrices)
    got = float(line.split("sum=")[1].split()[0])
    assert "dim=128 heads=1 ffn=1 labels=33 vocab=32 layers=2 matrices=10" in line and abs(got - want) < 1e-4, line
    # and the tool's own output is still the golden file
    again = tmp_path / "regen.bin"
    subprocess.run([TOOL, "write", str(again)], check=True)
    assert again.read_bytes() == raw
