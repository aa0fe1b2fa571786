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


def test_tuning_table_round_trip(tmp_path):
    """A table in the layout the GEMM sweep writes is installed into the dispatcher's lookup: the smallest matching
    m_max wins, unknown shapes fall back to the dispatcher's own choice (-1), an empty path clears the table."""
    import json
    table = {"device": "test", "entries": [
        {"bits": 5, "n": 5120, "k": 6144, "m_max": 64, "config": 3, "us": 21.8},
        {"bits": 5, "n": 5120, "k": 6144, "m_max": 8, "config": 0, "us": 16.7},
        {"bits": 4, "n": 34816, "k": 5120, "m_max": 512, "config": 6, "us": 148.0}]}
    path = tmp_path / "tuning.json"
    path.write_text(json.dumps(table))
    eng.load_tuning(path)
    assert eng.tuning_lookup(5, 5120, 6144, 1) == 0
    assert eng.tuning_lookup(5, 5120, 6144, 8) == 0
    assert eng.tuning_lookup(5, 5120, 6144, 9) == 3
    assert eng.tuning_lookup(5, 5120, 6144, 65) == -1
    assert eng.tuning_lookup(4, 34816, 5120, 300) == 6
    assert eng.tuning_lookup(8, 248320, 5120, 1) == -1
    eng.load_tuning("")
    assert eng.tuning_lookup(5, 5120, 6144, 1) == -1
    (tmp_path / "bad.json").write_text("{not json")
    with pytest.raises(eng.EngineError, match="malformed tuning table"):
        eng.load_tuning(tmp_path / "bad.json")


def test_step_status_turns_a_device_error_word_into_a_failed_step():
    """The runner reads the library's device error word after every step's synchronisation. A clean word lets the
    step through; any other value fails it with a message that names the step and the word (no GPU involved: this is
    the host-side decision alone)."""
    lib = eng.lib()
    assert lib.q38e_step_status(0, b"decode step") == 0
    assert lib.q38e_step_status(0x303, b"decode step") == -1
    msg = lib.q38e_last_error().decode()
    assert "decode step" in msg and "0x303" in msg and "discarded" in msg
    assert lib.q38e_step_status(0x212, b"prefill step") == -1
    assert "prefill step" in lib.q38e_last_error().decode()


@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_tensor_packer_gives_the_numpy_packers_bytes(bits):
    """pack() on a GPU tensor runs as tensor arithmetic; the same routine on CPU tensors must produce the planes of
    the numpy packer (which the golden fixtures pin to the reference's bytes)."""
    import torch
    g = torch.Generator().manual_seed(bits)
    codes, scales = tl.bq.quantize_absmax(torch.randn((256, 320), generator=g) * 0.02, bits)
    a, b = tl.bq.pack(codes, scales, bits), tl.bq._pack_on_device(codes, scales, bits)
    assert (a.lo, a.hi, a.scales) == (b.lo, b.hi, b.scales)
