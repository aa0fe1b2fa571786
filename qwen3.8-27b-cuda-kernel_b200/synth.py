"""Seeded random Qwen3.8-architecture models written as `.q38` files.

`random_checkpoint` draws tensors under their Hugging Face names (the names the reference converter
asks its `Source` for, reference tools/convert.py:252-339); `write_q38` turns such a checkpoint into
a model file the way the reference converter does: q/gate de-interleave of `q_proj`, `(1 + w)` norm
folding into the following projection, gate/up row interleave, `[b | a]` gate rows, `A = -exp(A_log)`.
"""

from __future__ import annotations

import math
from pathlib import Path

import torch

from . import bqformat as bq


def model_config(hidden=256, vocab=1024, layers=4, intermediate=768, nq=4, nkv=1, lk=2, lv=2, layer_types=None,
                 max_pos=4096, eos=(1000, 1001)) -> dict:
    """Header `config` block (reference docs/FORMAT.md 1.1). Head geometry is fixed by the kernels."""
    if layer_types is None:
        layer_types = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(layers)]
    return {
        "architecture": "qwen3_5_dense", "hidden_size": hidden, "num_layers": layers, "layer_types": list(layer_types),
        "vocab_size": vocab, "intermediate_size": intermediate, "num_attention_heads": nq,
        "num_key_value_heads": nkv, "head_dim": 256, "rotary_dim": 64, "rope_theta": 10_000_000.0,
        "linear_num_key_heads": lk, "linear_num_value_heads": lv, "linear_key_head_dim": 128,
        "linear_value_head_dim": 128, "linear_conv_kernel_dim": 4, "rms_norm_eps": 1e-6,
        "max_position_embeddings": max_pos, "tie_word_embeddings": False, "norm_folded": True,
        "eos_token_ids": list(eos),
    }


CONFIG_27B = dict(hidden=5120, vocab=248320, layers=64, intermediate=17408, nq=24, nkv=4, lk=16, lv=48,
                  max_pos=262144, eos=(248046, 248044))


def random_checkpoint(cfg: dict, seed: int = 1234, init: str = "n002") -> dict[str, torch.Tensor]:
    """init "n002": every matrix ~N(0, 0.02); init "unit": fan-in scaled matrices that keep activations O(1)
    (the magnitudes of reference tools/make_tiny_model.py:46-71)."""
    g = torch.Generator().manual_seed(seed)
    H, V, I = cfg["hidden_size"], cfg["vocab_size"], cfg["intermediate_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lk, lv, dk, dv = (cfg["linear_num_key_heads"], cfg["linear_num_value_heads"], cfg["linear_key_head_dim"],
                      cfg["linear_value_head_dim"])
    conv_dim = 2 * lk * dk + lv * dv

    def randn(*shape, std=1.0, mean=0.0):
        return torch.randn(shape, generator=g) * std + mean

    def mat(n, k):
        return randn(n, k, std=0.02 if init == "n002" else 1.0 / math.sqrt(k))

    t: dict[str, torch.Tensor] = {}
    t["embed_tokens.weight"] = randn(V, H, std=0.02 if init == "n002" else 1.0)
    for i, kind in enumerate(cfg["layer_types"]):
        p = f"layers.{i}."
        t[p + "input_layernorm.weight"] = randn(H, std=0.2)
        t[p + "post_attention_layernorm.weight"] = randn(H, std=0.2)
        if kind == "full_attention":
            t[p + "self_attn.q_proj.weight"] = mat(nq * 2 * hd, H)
            t[p + "self_attn.k_proj.weight"] = mat(nkv * hd, H)
            t[p + "self_attn.v_proj.weight"] = mat(nkv * hd, H)
            t[p + "self_attn.o_proj.weight"] = mat(H, nq * hd)
            t[p + "self_attn.q_norm.weight"] = randn(hd, std=0.2)
            t[p + "self_attn.k_norm.weight"] = randn(hd, std=0.2)
        else:
            t[p + "linear_attn.in_proj_qkv.weight"] = mat(conv_dim, H)
            t[p + "linear_attn.in_proj_z.weight"] = mat(lv * dv, H)
            t[p + "linear_attn.in_proj_b.weight"] = mat(lv, H)
            t[p + "linear_attn.in_proj_a.weight"] = mat(lv, H)
            t[p + "linear_attn.out_proj.weight"] = mat(H, lv * dv)
            t[p + "linear_attn.conv1d.weight"] = randn(conv_dim, 1, 4, std=0.4)
            t[p + "linear_attn.A_log"] = torch.log(torch.empty(lv).uniform_(0.5, 8.0, generator=g))
            t[p + "linear_attn.dt_bias"] = randn(lv, std=0.5)
            t[p + "linear_attn.norm.weight"] = randn(dv, std=0.2, mean=1.0)
        t[p + "mlp.gate_proj.weight"] = mat(I, H)
        t[p + "mlp.up_proj.weight"] = mat(I, H)
        t[p + "mlp.down_proj.weight"] = mat(H, I)
    t["norm.weight"] = randn(H, std=0.2)
    t["lm_head.weight"] = randn(V, H, std=0.02 if init == "n002" else 3.0 / math.sqrt(H))
    return t


def write_q38(path: str | Path, cfg: dict, ckpt: dict[str, torch.Tensor], recipe: str = "default", grid: int = 24,
              overrides: dict[str, int] | None = None, device: str = "cpu") -> None:
    """Checkpoint -> .q38 (tensor names and semantics: reference docs/FORMAT.md 1.3)."""
    bits_of = dict(bq.RECIPES[recipe])
    bits_of.update(overrides or {})
    H = cfg["hidden_size"]
    nq, hd = cfg["num_attention_heads"], cfg["head_dim"]
    I = cfg["intermediate_size"]
    w = bq.Q38Writer(cfg, recipe)
    f32 = lambda name: ckpt[name].to(torch.float32)
    gamma = lambda name: 1.0 + f32(name)

    w.add_direct("embed", ckpt["embed_tokens.weight"], "bf16")
    for i, kind in enumerate(cfg["layer_types"]):
        p = f"layers.{i}."
        g_in = gamma(p + "input_layernorm.weight")
        if kind == "full_attention":
            qp = f32(p + "self_attn.q_proj.weight").view(nq, 2 * hd, H)
            q, gate = qp[:, :hd, :].reshape(nq * hd, H), qp[:, hd:, :].reshape(nq * hd, H)
            qkvg = torch.cat([q, gate, f32(p + "self_attn.k_proj.weight"), f32(p + "self_attn.v_proj.weight")], dim=0)
            w.add_bq(f"{i}.attn.qkvg", qkvg * g_in[None, :], bits_of["attn.qkvg"], grid, device=device)
            w.add_bq(f"{i}.attn.o", f32(p + "self_attn.o_proj.weight"), bits_of["attn.o"], grid, device=device)
            w.add_direct(f"{i}.attn.q_norm", gamma(p + "self_attn.q_norm.weight"), "f32")
            w.add_direct(f"{i}.attn.k_norm", gamma(p + "self_attn.k_norm.weight"), "f32")
        else:
            qkvz = torch.cat([f32(p + "linear_attn.in_proj_qkv.weight"), f32(p + "linear_attn.in_proj_z.weight")], dim=0)
            w.add_bq(f"{i}.gdn.qkvz", qkvz * g_in[None, :], bits_of["gdn.qkvz"], grid, device=device)
            ab = torch.cat([f32(p + "linear_attn.in_proj_b.weight"), f32(p + "linear_attn.in_proj_a.weight")], dim=0)
            w.add_direct(f"{i}.gdn.ab", ab * g_in[None, :], "bf16")
            conv = f32(p + "linear_attn.conv1d.weight")
            w.add_direct(f"{i}.gdn.conv", conv.reshape(conv.shape[0], -1), "f32")
            w.add_direct(f"{i}.gdn.A", -torch.exp(f32(p + "linear_attn.A_log")), "f32")
            w.add_direct(f"{i}.gdn.dt_bias", f32(p + "linear_attn.dt_bias"), "f32")
            w.add_direct(f"{i}.gdn.norm", f32(p + "linear_attn.norm.weight"), "f32")
            w.add_bq(f"{i}.gdn.out", f32(p + "linear_attn.out_proj.weight"), bits_of["gdn.out"], grid, device=device)
        g_post = gamma(p + "post_attention_layernorm.weight")
        gu = torch.stack([f32(p + "mlp.gate_proj.weight"), f32(p + "mlp.up_proj.weight")], dim=1).reshape(2 * I, H)
        w.add_bq(f"{i}.mlp.gate_up", gu * g_post[None, :], bits_of["mlp.gate_up"], grid, device=device)
        w.add_bq(f"{i}.mlp.down", f32(p + "mlp.down_proj.weight"), bits_of["mlp.down"], grid, device=device)
    w.add_bq("lm_head", f32("lm_head.weight") * gamma("norm.weight")[None, :], bits_of["lm_head"], grid, device=device)
    w.write(path)


def write_random_planes_q38(path: str | Path, cfg: dict, recipe: str = "default", seed: int = 11,
                            weight_std: float = 0.02) -> None:
    """A benchmark-sized model without running the quantiser: every BQ tensor gets uniformly random codes
    and scales chosen so that the dequantised weights have standard deviation `weight_std`. One layer's
    random bytes are drawn per (role, bits) and reused by every layer of that kind: the engine still streams
    every layer's own copy from HBM, only the byte values repeat. Throughput runs only — parity runs use
    write_q38 with the real quantiser."""
    import json
    import struct

    import numpy as np

    rng = np.random.default_rng(seed)
    bits_of = bq.RECIPES[recipe]
    H, V, I = cfg["hidden_size"], cfg["vocab_size"], cfg["intermediate_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lk, lv = cfg["linear_num_key_heads"], cfg["linear_num_value_heads"]
    conv_dim = 2 * lk * 128 + lv * 128
    up = lambda x, a: (x + a - 1) // a * a
    records, blobs, cursor = {}, [], 0

    def place(blob: bytes) -> int:
        nonlocal cursor
        cursor = up(cursor, 256)
        at = cursor
        blobs.append((at, blob))
        cursor += len(blob)
        return at

    cache: dict = {}

    def bq_planes(role: str, rows: int, k: int):
        bits = bits_of[role]
        n = up(rows, 128)
        key = (role, n, k, bits)
        if key not in cache:
            lo_b, hi_b, sc_b = bq.plane_bytes(n, k, bits)
            lo = rng.integers(0, 256, size=lo_b, dtype=np.uint8).tobytes()
            hi = rng.integers(0, 256, size=hi_b, dtype=np.uint8).tobytes() if hi_b else b""
            s = weight_std * (12 ** 0.5) / (1 << bits)
            sc = (torch.full((sc_b // 2,), s) * (0.75 + 0.5 * torch.rand(sc_b // 2))).to(torch.bfloat16)
            cache[key] = (lo, hi, sc.view(torch.int16).numpy().tobytes())
        return bits, n, cache[key]

    def add_bq(name: str, role: str, rows: int, k: int):
        bits, n, (lo, hi, sc) = bq_planes(role, rows, k)
        planes = {"lo": [place(lo), len(lo)]}
        if hi:
            planes["hi"] = [place(hi), len(hi)]
        planes["scales"] = [place(sc), len(sc)]
        rec = {"dtype": f"bq{bits}", "shape": [n, k], "group_size": 64, "planes": planes}
        if n != rows:
            rec["rows"] = rows
        records[name] = rec

    def add_direct(name: str, t: torch.Tensor, dtype: str):
        blob = (t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes() if dtype == "bf16"
                else t.to(torch.float32).contiguous().numpy().tobytes())
        records[name] = {"dtype": dtype, "shape": list(t.shape), "offset": place(blob), "bytes": len(blob)}

    g = torch.Generator().manual_seed(seed)
    base = torch.randn((min(V, 4096), H), generator=g) * weight_std
    add_direct("embed", base.repeat((V + base.shape[0] - 1) // base.shape[0], 1)[:V], "bf16")
    small = {
        "q_norm": 1.0 + 0.2 * torch.randn(hd, generator=g), "k_norm": 1.0 + 0.2 * torch.randn(hd, generator=g),
        "ab": torch.randn((2 * lv, H), generator=g) * weight_std, "conv": 0.4 * torch.randn((conv_dim, 4), generator=g),
        "A": -torch.empty(lv).uniform_(0.5, 8.0, generator=g), "dt": 0.5 * torch.randn(lv, generator=g),
        "norm": 1.0 + 0.2 * torch.randn(128, generator=g),
    }
    for i, kind in enumerate(cfg["layer_types"]):
        if kind == "full_attention":
            add_bq(f"{i}.attn.qkvg", "attn.qkvg", 2 * nq * hd + 2 * nkv * hd, H)
            add_bq(f"{i}.attn.o", "attn.o", H, nq * hd)
            add_direct(f"{i}.attn.q_norm", small["q_norm"], "f32")
            add_direct(f"{i}.attn.k_norm", small["k_norm"], "f32")
        else:
            add_bq(f"{i}.gdn.qkvz", "gdn.qkvz", conv_dim + lv * 128, H)
            add_direct(f"{i}.gdn.ab", small["ab"], "bf16")
            add_direct(f"{i}.gdn.conv", small["conv"], "f32")
            add_direct(f"{i}.gdn.A", small["A"], "f32")
            add_direct(f"{i}.gdn.dt_bias", small["dt"], "f32")
            add_direct(f"{i}.gdn.norm", small["norm"], "f32")
            add_bq(f"{i}.gdn.out", "gdn.out", H, lv * 128)
        add_bq(f"{i}.mlp.gate_up", "mlp.gate_up", 2 * I, H)
        add_bq(f"{i}.mlp.down", "mlp.down", H, I)
    add_bq("lm_head", "lm_head", V, H)

    header = {"format": "qwen38-model", "format_version": 1, "config": cfg, "recipe": {"name": recipe},
              "tensors": records, "resources": {},
              "provenance": {"source": "synthetic random planes", "converter": "qwen38-b200 synth"}}
    hb = json.dumps(header).encode("utf-8")
    start = up(16 + len(hb), 4096)
    tmp = Path(str(path) + ".partial")
    with open(tmp, "wb") as f:
        f.write(bq.MAGIC + struct.pack("<Q", len(hb)) + hb)
        f.write(b"\0" * (start - f.tell()))
        for at, blob in blobs:
            f.seek(start + at)
            f.write(blob)
        f.seek(start + cursor)
        f.truncate()
    tmp.replace(path)
