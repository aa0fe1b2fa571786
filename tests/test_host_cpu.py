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


def test_converter_front_end_reproduces_the_direct_writer(tmp_path):
    """A tiny random checkpoint saved the Hugging Face way (config.json + safetensors with the `model.` prefix) and
    converted by the front end gives, byte for byte, the file the writer produces from the same tensors in memory
    (whose quantiser, packer and tensor semantics the golden fixtures pin to the reference converter)."""
    import json
    import torch
    from safetensors.torch import save_file
    from q38b200 import convert, synth
    cfg = synth.model_config(hidden=256, vocab=256, layers=4, intermediate=256, nq=2, nkv=1, lk=1, lv=1)
    ckpt = synth.random_checkpoint(cfg, seed=3)
    hf = tmp_path / "hf"
    hf.mkdir()
    names = {("lm_head.weight" if k == "lm_head.weight" else "model." + k): v.contiguous() for k, v in ckpt.items()}
    save_file(names, str(hf / "model.safetensors"))
    (hf / "config.json").write_text(json.dumps({
        "hidden_size": 256, "num_hidden_layers": 4, "vocab_size": 256, "intermediate_size": 256, "num_attention_heads": 2,
        "num_key_value_heads": 1, "head_dim": 256, "partial_rotary_factor": 0.25, "rope_theta": 1e7,
        "linear_num_key_heads": 1, "linear_num_value_heads": 1, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
        "linear_conv_kernel_dim": 4, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096, "eos_token_id": [1000, 1001],
        "full_attention_interval": 4}))
    got = convert.convert(hf, tmp_path / "a.q38", recipe="default", device="cpu")
    assert got["layer_types"] == cfg["layer_types"] and got["rotary_dim"] == 64
    synth.write_q38(tmp_path / "b.q38", got, ckpt, recipe="default", device="cpu")
    assert (tmp_path / "a.q38").read_bytes() == (tmp_path / "b.q38").read_bytes()
    m = eng.Model(tmp_path / "a.q38")
    assert (m.vocab, m.hidden, m.layers) == (256, 256, 4)
    m.close()
    two = convert.convert(hf, tmp_path / "c.q38", layers=2, device="cpu")
    assert two["num_layers"] == 2
