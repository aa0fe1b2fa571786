"""Generates the golden fixtures of tests/golden/ from the REFERENCE's own code.

Run once on a machine that has the reference checkout (--reference PATH) and oracle/_ref built
(`make -C oracle ref`). The GPU box has neither; it only reads the committed fixtures.

    python tests/golden/make_golden.py --reference PATH

Fixtures written:
  bq_golden.npz        per bit width: a weight matrix, the reference quantiser's codes / scales
                       (tools/bqpack.py quantize_matrix), the reference packer's plane bytes (pack_bq) and
                       the dequantised values of the reference's C++ spec decoder (BQView, via oracle/_ref)
  tiny_cfg1.q38        config-1 model (hidden 256, vocab 1024, 4 layers [GDN, GDN, GDN, attention],
                       4q/1kv heads, MLP 768, GDN 2k/2v heads; weights ~N(0, 0.02), seed 1234) written by
                       the reference converter (tools/convert.py) from a synthetic in-memory checkpoint
  tiny_cfg1_unit.q38   the same geometry with the O(1)-activation initialisation (seed 1234)
  tiny_cfg1_golden.npz prompts (lengths 17/64/65/130, ids uniform in [0, 1000), numpy default_rng(7)),
                       32 greedy continuation tokens per prompt and the logits of `qwen38-ref` (engine
                       mode, int8 KV) at every position of prompt + continuation, for both models
  ops_golden.npz       single-op inputs/outputs of the reference's ref:: functions (qgemm epilogues,
                       int8 KV round trip, q/k-norm + RoPE + append, attention, GDN token)
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import q38_testlib as tl  # noqa: E402
from oracle_model import OracleModel, greedy  # noqa: E402
from q38b200 import synth  # noqa: E402


def reference_convert(ref_tools: Path, cfg: dict, ckpt: dict, out: Path, recipe: str = "default") -> None:
    """Drives the reference Converter as a library with an in-memory checkpoint."""
    sys.path.insert(0, str(ref_tools))
    import convert as refconv  # reference tools/convert.py

    class MemSource:
        def get(self, name):
            return ckpt[name]

    conv = refconv.Converter.__new__(refconv.Converter)
    conv.args = types.SimpleNamespace(recipe=recipe, grid=24, block_rows=8192, layers=None, bits=None, device="cpu",
                                      out=str(out), no_tokenizer=True, source_id="synthetic", verbose=False,
                                      model="synthetic")
    conv.model_dir = Path(tempfile.mkdtemp())
    conv.src = MemSource()
    conv.cfg = dict(cfg)
    conv.recipe = dict(refconv.RECIPES[recipe])
    conv.overrides = {}
    conv.device = "cpu"
    conv.report = {}
    conv.run()
    for extra in (out.with_suffix(out.suffix + ".report.json"),):
        if extra.exists():
            extra.unlink()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("Q38_REFERENCE", ""), required=not os.environ.get("Q38_REFERENCE"),
                    help="checkout of the reference project (or set Q38_REFERENCE)")
    args = ap.parse_args()
    ref_root = Path(args.reference)
    ref_ops = tl.reference_ops()
    ref_bin = tl.reference_binary()
    assert ref_ops is not None and ref_bin is not None, "build oracle/_ref first: make -C oracle ref"
    sys.path.insert(0, str(ref_root / "tools"))
    import bqpack as refbq  # reference tools/bqpack.py

    # ---- BQ quantiser / packer / decoder -----------------------------------------------------------
    out = {}
    for bits in (4, 5, 6, 8):
        g = torch.Generator().manual_seed(100 + bits)
        w = torch.randn((128, 192), generator=g) * 0.02
        w[5, 64:128] = 0.0  # an all-zero group
        codes, scales = refbq.quantize_matrix(w, bits, grid=24)
        p = refbq.pack_bq(codes, scales, bits)
        deq = ref_ops.dequant(tl.bq.Packed(bits, p.n, p.k, p.lo, p.hi, p.scales))
        out[f"w{bits}"] = w.numpy()
        out[f"codes{bits}"] = codes.numpy()
        out[f"scales{bits}"] = scales.numpy()
        out[f"lo{bits}"] = np.frombuffer(p.lo, dtype=np.uint8)
        out[f"hi{bits}"] = np.frombuffer(p.hi, dtype=np.uint8)
        out[f"sc{bits}"] = np.frombuffer(p.scales, dtype=np.uint8)
        out[f"deq{bits}"] = deq
    np.savez_compressed(HERE / "bq_golden.npz", **out)

    # ---- tiny models through the reference converter + qwen38-ref -------------------------------------
    cfg = synth.model_config()
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, 1000, size=n).astype(np.int32) for n in (17, 64, 65, 130)]
    gold = {f"prompt{i}": p for i, p in enumerate(prompts)}
    for tag, init in (("", "n002"), ("_unit", "unit")):
        path = HERE / f"tiny_cfg1{tag}.q38"
        reference_convert(ref_root / "tools", cfg, synth.random_checkpoint(cfg, seed=1234, init=init), path)
        model = OracleModel(path, ops=ref_ops, max_positions=256)
        for i, prompt in enumerate(prompts):
            seq = model.new_sequence()
            logits = model.forward(seq, prompt)[-1]
            gen = []
            for _ in range(32):
                gen.append(greedy(logits))
                logits = model.forward(seq, [gen[-1]])[-1]
            full = np.concatenate([prompt, np.array(gen, dtype=np.int32)])
            with tempfile.TemporaryDirectory() as td:
                tok, lg = Path(td) / "t.i32", Path(td) / "l.f32"
                full.astype("<i4").tofile(tok)
                subprocess.run([str(ref_bin), "--model", str(path), "--tokens", str(tok), "--out", str(lg),
                                "--all-logits", "--kv", "int8"], check=True, capture_output=True)
                ref_logits = np.fromfile(lg, dtype="<f4").reshape(len(full), cfg["vocab_size"])
            # the binary's logits must reproduce the greedy continuation found through the shim
            for j, tokn in enumerate(gen):
                assert int(np.argmax(ref_logits[len(prompt) - 1 + j])) == tokn, (tag, i, j)
            gold[f"gen{tag}{i}"] = np.array(gen, dtype=np.int32)
            gold[f"logits{tag}{i}"] = ref_logits.astype(np.float32)
    np.savez_compressed(HERE / "tiny_cfg1_golden.npz", **gold)

    # ---- single ops ---------------------------------------------------------------------------------
    r = np.random.default_rng(11)
    ops = {}
    m, n, k = 3, 256, 192
    a = tl.bf16_round(r.standard_normal((m, k)))
    w = tl.bf16_round(r.standard_normal((n, k)) * 0.05)
    rs = (0.5 + r.random(m)).astype(np.float32)
    ops["gemm_a"], ops["gemm_w"], ops["gemm_rs"] = a, w, rs
    for ep, name in ((0, "bf16"), (1, "swiglu"), (3, "f32")):
        o = np.zeros((m, n if ep != 1 else n // 2), dtype=np.float32)
        ref_ops.qgemm(a, w, rs, ep, out=o, ldo=o.shape[1])
        ops[f"gemm_{name}"] = o
    res = (r.standard_normal((m, n)) * 3).astype(np.float32)
    ops["gemm_res_in"] = res.copy()
    xbf, part = np.zeros((m, n), np.float32), np.zeros((m, n // 128), np.float32)
    ref_ops.qgemm(a, w, None, 2, residual=res, xbf=xbf, partials=part)
    ops["gemm_res"], ops["gemm_xbf"], ops["gemm_part"] = res, xbf, part
    x = r.standard_normal(512).astype(np.float32) * 2
    x[64:128] = 0
    ops["i8_in"], ops["i8_out"] = x, ref_ops.int8_group_roundtrip(x)
    nq, nkv = 4, 2
    ld = 2 * nq * 256 + 2 * nkv * 256
    qn, kn = (1 + 0.2 * r.standard_normal(256)).astype(np.float32), (1 + 0.2 * r.standard_normal(256)).astype(np.float32)
    kv = tl.OracleKv(ref_ops, nkv, 80)
    rows = tl.bf16_round(r.standard_normal((70, ld)))
    qs, outs = [], []
    for pos in range(70):
        q = kv.append(nq, 1e-6, 1e7, rows[pos], pos, qn, kn, 2)
        qs.append(q)
        outs.append(kv.attend(nq, q, rows[pos, nq * 256:2 * nq * 256], pos))
    ops.update(attn_rows=rows, attn_qn=qn, attn_kn=kn, attn_q=np.stack(qs), attn_out=np.stack(outs),
               attn_k=kv.k.copy(), attn_v=kv.v.copy())
    lk, lv = 2, 4
    cd = 2 * lk * 128 + lv * 128
    proj = tl.bf16_round(r.standard_normal((6, cd + lv * 128)))
    ab = r.standard_normal((6, 2 * lv)).astype(np.float32)
    conv_w = (0.4 * r.standard_normal((cd, 4))).astype(np.float32)
    A = (-r.uniform(0.5, 8, lv)).astype(np.float32)
    dt = (0.5 * r.standard_normal(lv)).astype(np.float32)
    nw = (1 + 0.2 * r.standard_normal(128)).astype(np.float32)
    s, cs = np.zeros(lv * 128 * 128, np.float32), np.zeros(3 * cd, np.float32)
    gout = [ref_ops.gdn_token(lk, lv, 1e-6, proj[i], ab[i], conv_w, A, dt, nw, s, cs) for i in range(6)]
    ops.update(gdn_proj=proj, gdn_ab=ab, gdn_conv_w=conv_w, gdn_A=A, gdn_dt=dt, gdn_nw=nw, gdn_out=np.stack(gout),
               gdn_state=s, gdn_conv_state=cs)
    np.savez_compressed(HERE / "ops_golden.npz", **ops)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
