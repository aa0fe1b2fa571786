"""CPU-only tests of the host logic that needs no device: the .q38 reader, its error behaviour, and the host
BQ spec decoder (reference tests/host/test_bq_layout.cpp pins the same decoder on the reference side)."""

import shutil
from pathlib import Path

import numpy as np
import pytest

import q38_testlib as tl
from q38b200 import engine as eng

GOLD = Path(__file__).resolve().parent / "golden"


def test_model_file_header_and_config():
    m = eng.Model(GOLD / "tiny_cfg1.q38")
    assert (m.vocab, m.hidden, m.layers) == (1024, 256, 4)
    assert "3 GDN" in m.summary() and "4q/1kv x256" in m.summary()
    m.close()


@pytest.mark.parametrize("name,n,k", [("0.gdn.qkvz", 1024, 256), ("0.mlp.gate_up", 1536, 256), ("lm_head", 1024, 256),
                                      ("3.attn.o", 256, 1024)])
def test_host_spec_decoder_matches_oracle(name, n, k):
    m = eng.Model(GOLD / "tiny_cfg1.q38")
    f = tl.bq.Q38File(GOLD / "tiny_cfg1.q38")
    assert np.array_equal(m.dequant(name, n, k), tl.oracle().dequant(f.packed(name)))
    m.close()


def test_truncated_and_foreign_files_are_rejected(tmp_path):
    src = GOLD / "tiny_cfg1.q38"
    cut = tmp_path / "cut.q38"
    data = src.read_bytes()
    cut.write_bytes(data[:len(data) // 2])
    with pytest.raises(eng.EngineError, match="outside the file"):
        eng.Model(cut)
    bad = tmp_path / "bad.q38"
    bad.write_bytes(b"NOTAQ38!" + data[8:])
    with pytest.raises(eng.EngineError, match="not a .q38 model file"):
        eng.Model(bad)
    with pytest.raises(eng.EngineError, match="cannot open"):
        eng.Model(tmp_path / "missing.q38")


def test_engine_library_exports_declared_symbols():
    import re
    header = (tl.ROOT / "include" / "q38_engine.h").read_text()
    declared = set(re.findall(r"\b(q38e_[a-z0-9_]+)\s*\(", header))
    lib = eng.lib()
    for name in declared:
        assert hasattr(lib, name), name
