"""Whole-model CPU oracle: the reference's token-at-a-time forward pass (reference
src/ref/ref_model.cpp:21-127) restated over the oracle operations of oracle/q38_oracle.cpp.

TEST INFRASTRUCTURE: used by the parity tests, the smoke check and the benchmark's CPU-baseline leg.
"""

from __future__ import annotations

import numpy as np
import torch

from q38_testlib import OracleKv, bq, oracle


class OracleModel:
    def __init__(self, path, kv_dtype: int = 2, exact: bool = False, max_positions: int = 4096, ops=None):
        self.ops = ops or oracle()
        self.f = bq.Q38File(path)
        c = self.cfg = self.f.config
        self.exact, self.kv_dtype, self.max_positions = exact, kv_dtype, max_positions
        self.H, self.V, self.I = c["hidden_size"], c["vocab_size"], c["intermediate_size"]
        self.nq, self.nkv = c["num_attention_heads"], c["num_key_value_heads"]
        self.lk, self.lv = c["linear_num_key_heads"], c["linear_num_value_heads"]
        self.eps, self.theta = float(c["rms_norm_eps"]), float(c["rope_theta"])
        self.conv_dim = 2 * self.lk * 128 + self.lv * 128
        dq = lambda name: self.ops.dequant(self.f.packed(name))
        f32 = lambda name: self.f.direct(name).to(torch.float32).numpy().copy()
        self.embed = self.f.direct("embed").to(torch.float32).numpy()
        self.lm_head = dq("lm_head")
        self.layers = []
        for i, kind in enumerate(c["layer_types"]):
            L = {"attn": kind == "full_attention"}
            p = f"{i}."
            if L["attn"]:
                L["w_in"], L["w_out"] = dq(p + "attn.qkvg"), dq(p + "attn.o")
                L["q_norm"], L["k_norm"] = f32(p + "attn.q_norm"), f32(p + "attn.k_norm")
            else:
                L["w_in"], L["w_out"] = dq(p + "gdn.qkvz"), dq(p + "gdn.out")
                L["w_ab"] = f32(p + "gdn.ab")
                L["conv"], L["A"], L["dt"], L["norm"] = (f32(p + "gdn.conv"), f32(p + "gdn.A"), f32(p + "gdn.dt_bias"),
                                                         f32(p + "gdn.norm"))
            L["w_gate_up"], L["w_down"] = dq(p + "mlp.gate_up"), dq(p + "mlp.down")
            self.layers.append(L)

    def new_sequence(self):
        seq = {"pos": 0, "kv": [], "gdn": []}
        for L in self.layers:
            if L["attn"]:
                seq["kv"].append(OracleKv(self.ops, self.nkv, self.max_positions))
            else:
                seq["gdn"].append((np.zeros(self.lv * 128 * 128, dtype=np.float32),
                                   np.zeros(3 * self.conv_dim, dtype=np.float32)))
        return seq

    def forward(self, seq, tokens, all_logits: bool = False) -> np.ndarray:
        """Appends `tokens`; returns logits [n_out][vocab] (every position, or the last one)."""
        o, H, ex = self.ops, self.H, self.exact
        outs = []
        for t, token in enumerate(tokens):
            residual = self.embed[int(token)].astype(np.float32).copy()[None, :]
            xbf = residual.copy()
            partials = o.norm_partials(residual[0])[None, :].copy()
            ai = gi = 0
            for L in self.layers:
                rs = np.array([o.norm_row_scale(partials[0], H, self.eps)], dtype=np.float32)
                n_in = L["w_in"].shape[0]
                proj = np.zeros((1, n_in), dtype=np.float32)
                o.qgemm(xbf, L["w_in"], rs, 0, out=proj, ldo=n_in, exact=ex)
                if L["attn"]:
                    kv = seq["kv"][ai]
                    ai += 1
                    q = kv.append(self.nq, self.eps, self.theta, proj[0], seq["pos"], L["q_norm"], L["k_norm"],
                                  self.kv_dtype, ex)
                    mixer = kv.attend(self.nq, q, proj[0, self.nq * 256:2 * self.nq * 256], seq["pos"], ex)
                else:
                    rows = L["w_ab"].shape[0]
                    ab = np.zeros((1, rows), dtype=np.float32)
                    o.qgemm(xbf, L["w_ab"], rs, 3, out=ab, ldo=rows, exact=ex)
                    s, conv = seq["gdn"][gi]
                    gi += 1
                    mixer = o.gdn_token(self.lk, self.lv, self.eps, proj[0], ab[0], L["conv"], L["A"], L["dt"],
                                        L["norm"], s, conv, ex)
                o.qgemm(mixer[None, :], L["w_out"], None, 2, residual=residual, xbf=xbf, partials=partials, exact=ex)
                rs = np.array([o.norm_row_scale(partials[0], H, self.eps)], dtype=np.float32)
                act = np.zeros((1, self.I), dtype=np.float32)
                o.qgemm(xbf, L["w_gate_up"], rs, 1, out=act, ldo=self.I, exact=ex)
                o.qgemm(act, L["w_down"], None, 2, residual=residual, xbf=xbf, partials=partials, exact=ex)
            seq["pos"] += 1
            if all_logits or t + 1 == len(tokens):
                rs = np.array([o.norm_row_scale(partials[0], H, self.eps)], dtype=np.float32)
                logits = np.zeros((1, self.V), dtype=np.float32)
                o.qgemm(xbf, self.lm_head, rs, 3, out=logits, ldo=self.V, exact=ex)
                outs.append(logits[0])
        return np.stack(outs)


def greedy(logits_row: np.ndarray) -> int:
    return int(np.argmax(logits_row))  # numpy returns the first maximum = lowest id, like the reference
