"""CPU-only: pins the oracle restatement and the BQ / .q38 format code against the reference.

Two anchors: (1) the golden fixtures in tests/golden/, produced by the reference's own Python tools and
its own C++ CPU model (tests/golden/make_golden.py); (2) where oracle/_ref has been built from a
reference checkout, the reference's functions themselves on fresh random inputs.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

import q38_testlib as tl
from oracle_model import OracleModel, greedy
from q38_testlib import bq, synth

GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def bqg():
    return np.load(GOLD / "bq_golden.npz")


@pytest.fixture(scope="module")
def opsg():
    return np.load(GOLD / "ops_golden.npz")


def _packed(g, bits):
    return bq.Packed(bits, 128, 192, g[f"lo{bits}"].tobytes(), g[f"hi{bits}"].tobytes(), g[f"sc{bits}"].tobytes())


@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_quantiser_and_packer_match_reference_bytes(bqg, bits):
    w = torch.from_numpy(bqg[f"w{bits}"])
    codes, scales = bq.quantize_matrix(w, bits, grid=24)
    assert np.array_equal(codes.numpy(), bqg[f"codes{bits}"])
    assert np.array_equal(scales.numpy(), bqg[f"scales{bits}"])
    p = bq.pack(codes, scales, bits)
    assert p.lo == bqg[f"lo{bits}"].tobytes()
    assert p.hi == bqg[f"hi{bits}"].tobytes()
    assert p.scales == bqg[f"sc{bits}"].tobytes()
    c2, s2 = bq.unpack(p)
    assert torch.equal(c2, codes) and torch.equal(s2, scales)
    assert len(p.lo), len(p.hi) == bq.plane_bytes(128, 192, bits)[:2]


@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_oracle_decoder_is_bit_exact_with_reference_decoder(bqg, bits):
    p = _packed(bqg, bits)
    deq = tl.oracle().dequant(p)
    assert np.array_equal(deq, bqg[f"deq{bits}"])
    codes, sbits = tl.oracle().codes(p)
    assert np.array_equal(codes, bqg[f"codes{bits}"].astype(np.int32))
    want_bits = torch.from_numpy(bqg[f"scales{bits}"]).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(sbits, want_bits)
    # the python dequantiser agrees too
    assert np.array_equal(bq.dequantize(*bq.unpack(p)).numpy(), deq)


def test_oracle_gemm_epilogues_match_reference(opsg):
    o = tl.oracle()
    a, w, rs = opsg["gemm_a"], opsg["gemm_w"], opsg["gemm_rs"]
    m, n = a.shape[0], w.shape[0]
    for ep, name in ((0, "bf16"), (1, "swiglu"), (3, "f32")):
        out = np.zeros_like(opsg[f"gemm_{name}"])
        o.qgemm(a, w, rs, ep, out=out, ldo=out.shape[1])
        assert np.array_equal(out, opsg[f"gemm_{name}"]), name
    res = opsg["gemm_res_in"].copy()
    xbf, part = np.zeros((m, n), np.float32), np.zeros((m, n // 128), np.float32)
    o.qgemm(a, w, None, 2, residual=res, xbf=xbf, partials=part)
    assert np.array_equal(res, opsg["gemm_res"]) and np.array_equal(xbf, opsg["gemm_xbf"])
    assert np.array_equal(part, opsg["gemm_part"])


def test_oracle_int8_kv_roundtrip_matches_reference(opsg):
    assert np.array_equal(tl.oracle().int8_group_roundtrip(opsg["i8_in"]), opsg["i8_out"])


def test_oracle_attention_matches_reference(opsg):
    nq, nkv = 4, 2
    kv = tl.OracleKv(tl.oracle(), nkv, 80)
    rows = opsg["attn_rows"]
    for pos in range(rows.shape[0]):
        q = kv.append(nq, 1e-6, 1e7, rows[pos], pos, opsg["attn_qn"], opsg["attn_kn"], 2)
        assert np.array_equal(q, opsg["attn_q"][pos]), pos
        out = kv.attend(nq, q, rows[pos, nq * 256:2 * nq * 256], pos)
        assert np.array_equal(out, opsg["attn_out"][pos]), pos
    assert np.array_equal(kv.k, opsg["attn_k"]) and np.array_equal(kv.v, opsg["attn_v"])


def test_oracle_gdn_matches_reference(opsg):
    lk, lv = 2, 4
    cd = 2 * lk * 128 + lv * 128
    s, cs = np.zeros(lv * 128 * 128, np.float32), np.zeros(3 * cd, np.float32)
    for i in range(opsg["gdn_proj"].shape[0]):
        out = tl.oracle().gdn_token(lk, lv, 1e-6, opsg["gdn_proj"][i], opsg["gdn_ab"][i], opsg["gdn_conv_w"],
                                    opsg["gdn_A"], opsg["gdn_dt"], opsg["gdn_nw"], s, cs)
        assert np.array_equal(out, opsg["gdn_out"][i]), i
    assert np.array_equal(s, opsg["gdn_state"]) and np.array_equal(cs, opsg["gdn_conv_state"])


@pytest.mark.parametrize("tag", ["", "_unit"])
def test_oracle_model_reproduces_reference_logits_and_tokens(tag):
    """The whole-model oracle against `qwen38-ref` (engine mode, int8 KV) on the config-1 model."""
    gold = np.load(GOLD / "tiny_cfg1_golden.npz")
    model = OracleModel(GOLD / f"tiny_cfg1{tag}.q38", max_positions=256)
    for i in (0, 2):  # prompts of 17 and 65 tokens (page boundary) keep the CPU suite short
        prompt, gen = gold[f"prompt{i}"], gold[f"gen{tag}{i}"]
        seq = model.new_sequence()
        full = np.concatenate([prompt, gen])
        logits = model.forward(seq, full, all_logits=True)
        assert np.array_equal(logits, gold[f"logits{tag}{i}"])
        for j, t in enumerate(gen):
            assert greedy(logits[len(prompt) - 1 + j]) == int(t)


def test_own_converter_writes_the_reference_converters_bytes():
    """synth.write_q38 on the same checkpoint = the file the reference converter wrote (payloads + records)."""
    cfg = synth.model_config()
    ref_file = bq.Q38File(GOLD / "tiny_cfg1.q38")
    import tempfile
    with tempfile.TemporaryDirectory() as td:
        path = Path(td) / "mine.q38"
        synth.write_q38(path, cfg, synth.random_checkpoint(cfg, seed=1234, init="n002"))
        mine = bq.Q38File(path)
        assert mine.config == ref_file.config
        assert list(mine.tensors) == list(ref_file.tensors)
        for name, rec in ref_file.tensors.items():
            assert mine.tensors[name] == rec, name
            if "planes" in rec:
                for plane, (off, size) in rec["planes"].items():
                    assert mine.raw(off, size) == ref_file.raw(off, size), (name, plane)
            else:
                assert mine.raw(rec["offset"], rec["bytes"]) == ref_file.raw(rec["offset"], rec["bytes"]), name


def test_restatement_equals_reference_build_on_random_inputs():
    """Fresh random inputs through oracle/_ref (the reference's own objects), where it has been built."""
    ref = tl.reference_ops()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine (needs the reference checkout)")
    o = tl.oracle()
    r = np.random.default_rng(3)
    for bits in (4, 5, 6, 8):
        p = tl.make_bq(128, 128, bits, seed=bits, fast=True)
        assert np.array_equal(o.dequant(p), ref.dequant(p))
    a = tl.bf16_round(r.standard_normal((2, 128)))
    w = tl.bf16_round(r.standard_normal((256, 128)) * 0.1)
    for ep in (0, 1, 3):
        x, y = np.zeros((2, 256), np.float32), np.zeros((2, 256), np.float32)
        o.qgemm(a, w, np.ones(2, np.float32), ep, out=x, ldo=256)
        ref.qgemm(a, w, np.ones(2, np.float32), ep, out=y, ldo=256)
        assert np.array_equal(x, y)
    part = r.random(40).astype(np.float32) * 100
    assert o.norm_row_scale(part, 5120, 1e-6) == ref.norm_row_scale(part, 5120, 1e-6)
    row = r.standard_normal(256).astype(np.float32)
    assert np.array_equal(o.norm_partials(row), ref.norm_partials(row))
    # long-context RoPE positions
    nq, nkv = 2, 1
    ld = 2 * nq * 256 + 2 * nkv * 256
    for pos in (0, 1, 4095, 262143):
        rows = tl.bf16_round(r.standard_normal(ld))
        ka, kb = tl.OracleKv(o, nkv, 1), tl.OracleKv(ref, nkv, 1)
        ones = np.ones(256, np.float32)
        # capacity 1: write at index 0 while rotating with `pos` is not expressible; compare q only
        qa = np.empty(nq * 256, np.float32)
        ka2, kb2 = tl.OracleKv(o, nkv, pos + 1), tl.OracleKv(ref, nkv, pos + 1)
        qa = ka2.append(nq, 1e-6, 1e7, rows, pos, ones, ones, 2)
        qb = kb2.append(nq, 1e-6, 1e7, rows, pos, ones, ones, 2)
        assert np.array_equal(qa, qb) and np.array_equal(ka2.k[:, pos], kb2.k[:, pos])
        del ka, kb


def test_c_abi_library_exports_every_declared_symbol():
    import re
    header = (tl.ROOT / "include" / "q38_kernels.h").read_text()
    declared = set(re.findall(r"\b(q38_[a-z0-9_]+)\s*\(", header))
    declared -= {"q38_gemm_tuning_lookup"}
    assert declared == set(tl.pkg.KERNEL_API), declared ^ set(tl.pkg.KERNEL_API)
    lib = tl.pkg.kernels()  # loads without a GPU; no compute call is made
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.q38_qgemm_num_configs() >= 4
    # the dispatcher's rule: streaming kernel up to 16 tokens, then the tcgen05 kernel with the weights in TMEM at the
    # smallest token operand that fits, two 256-token blocks per launch above 256
    picks = {m: lib.q38_qgemm_config_name(lib.q38_qgemm_auto_config(4, 34816, 5120, m)).decode()
             for m in (1, 8, 9, 16, 17, 64, 65, 128, 256, 257, 512)}
    assert picks == {1: "stream_m8", 8: "stream_m8", 9: "stream_m16", 16: "stream_m16", 17: "tmem_t32", 64: "tmem_t64",
                     65: "tmem_t128", 128: "tmem_t128", 256: "tmem_t256", 257: "tmem_t256x2", 512: "tmem_t256x2"}, picks
    assert lib.q38_kv_page_bytes(0, 4) == 135168
    # about sixteen (sequence, kv head, split) work items per SM, within [1, max_splits]
    assert lib.q38_attention_decode_splits(64, 4, 148, 64) == 10
    assert lib.q38_attention_decode_splits(1, 4, 148, 64) == 64
    assert lib.q38_attention_decode_splits(4096, 4, 148, 64) == 1
    assert lib.q38_attention_decode_splits(64, 4, 148, 4) == 4


def test_sampler_restatement_obeys_its_definition():
    """The CPU sampler (the checker of the GPU sampler's token ids) on the 27B vocabulary: top-k = 1 is the argmax,
    top-k keeps the k largest, min-p keeps only tokens whose probability ratio to the maximum reaches min_p, a draw is
    a pure function of (seed, step), and top-3 frequencies follow the softmax."""
    V = 248320
    rng = np.random.default_rng(1)
    o = tl.oracle()
    row = (2.0 * rng.standard_normal(V)).astype(np.float32)
    seeds = rng.integers(1, 2 ** 63, size=256, dtype=np.uint64)
    steps = rng.integers(0, 5000, size=256).astype(np.int32)
    tok, _ = o.sample_draws(row, 1.0, 1, 1.0, 0.0, seeds, steps)
    assert set(tok.tolist()) == {int(row.argmax())}
    tok, lp = o.sample_draws(row, 1.0, 50, 1.0, 0.0, seeds, steps)
    assert set(tok.tolist()) <= set(np.argsort(row)[-50:].tolist()) and len(set(tok.tolist())) > 20
    again, lp2 = o.sample_draws(row, 1.0, 50, 1.0, 0.0, seeds, steps)
    assert np.array_equal(tok, again) and np.array_equal(lp, lp2)
    tok, _ = o.sample_draws(row, 1.3, 0, 1.0, 0.05, seeds, steps)
    assert np.exp((row[tok] - row.max()) / 1.3).min() >= 0.05 * (1 - 1e-6)
    many = rng.integers(1, 2 ** 63, size=20000, dtype=np.uint64)
    tok, _ = o.sample_draws(row, 1.0, 3, 1.0, 0.0, many, np.zeros(20000, np.int32))
    top = np.argsort(row)[-3:]
    pr = np.exp(row[top] - row[top].max())
    pr /= pr.sum()
    for i, p in zip(top, pr):
        assert abs((tok == i).mean() - p) < 5 * np.sqrt(p * (1 - p) / 20000)
    pen = o.sample_penalties(row, [5, 5, 7], 0.5, 2.0, 16)
    for t in (5, 7):
        assert pen[t] == np.float32(np.float32(row[t] / 2 if row[t] > 0 else row[t] * 2) - np.float32(0.5))
    assert np.array_equal(np.delete(pen, [5, 7]), np.delete(row, [5, 7]))
