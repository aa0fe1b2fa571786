"""Tensor-parallel shard arithmetic on the CPU: row and k shards of a BQ tensor decode to the same weights as the
corresponding slices of the whole tensor, and the rank plans tile every head / column range exactly once."""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

entry.load_package()
from q38b200 import bqformat as bq, synth, tp  # noqa: E402


def _packed(n, k, bits, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((n, k), generator=g) * 0.02
    c, s = bq.quantize_absmax(w, bits)
    return bq.pack(c, s, bits), bq.dequantize(c, s)


def test_row_and_k_shards_decode_to_slices_of_the_whole():
    for bits in (4, 5, 6, 8):
        p, w = _packed(512, 384, bits, seed=bits)
        ranges = [(64, 192), (256, 320), (448, 512)]
        ps = tp.shard_rows(p, ranges)
        rows = [r for a, b in ranges for r in range(a, b)]
        assert ps.n == len(rows) and ps.k == 384
        assert torch.equal(bq.dequantize(*bq.unpack(ps)), w[rows])
        pk = tp.shard_k(p, 128, 320)
        assert pk.n == 512 and pk.k == 192
        assert torch.equal(bq.dequantize(*bq.unpack(pk)), w[:, 128:320])
        padded = tp._pad128(tp.shard_rows(p, [(0, 64)]))
        wp = bq.dequantize(*bq.unpack(padded))
        assert padded.n == 128 and torch.equal(wp[:64], w[:64]) and float(wp[64:].abs().sum()) == 0.0


def test_rank_plans_partition_the_model():
    for cfg, world in ((synth.model_config(**synth.CONFIG_27B), 8), (synth.model_config(), 2), (synth.model_config(), 1)):
        plans = [tp.rank_plan(cfg, r, world) for r in range(world)]
        cat = lambda key: [x for p in plans for x in getattr(p, key)]
        assert cat("q_heads") == list(range(cfg["num_attention_heads"]))
        assert cat("k_heads") == list(range(cfg["linear_num_key_heads"]))
        assert cat("v_heads") == list(range(cfg["linear_num_value_heads"]))
        assert cat("mlp_cols") == list(range(cfg["intermediate_size"]))
        tiles = (cfg["vocab_size"] + 127) // 128
        assert cat("vocab_rows") == list(range(128 * tiles))
        group = cfg["num_attention_heads"] // cfg["num_key_value_heads"]
        ratio = cfg["linear_num_value_heads"] // cfg["linear_num_key_heads"]
        for p in plans:
            assert all(h // group in p.kv_heads for h in p.q_heads), "query heads stay with their kv head"
            assert all(v // ratio in p.k_heads for v in p.v_heads), "value heads stay with their key head"
            for ranges in (tp.qkvg_row_ranges(cfg, p), tp.qkvz_row_ranges(cfg, p)):
                assert sum(b - a for a, b in ranges) % 128 == 0 and all(a % 64 == 0 and b % 64 == 0 for a, b in ranges)
