"""Tensor-parallel execution of one long request (the 262,144-token configuration): the model's projections are
sharded over the ranks of a torch.distributed group, every rank runs this library's kernels on its shard, and the
two row-parallel projections of a layer are followed by one all-reduce (NCCL over NVLink on GPUs).

Partitioning (reference docs/FORMAT.md 2.2: BQ planes are n-block-major, so a range of 64-row blocks is a byte range
of every plane, and the k16 slabs / k64 scale groups of one block are contiguous in k):
  column-parallel (rows of W)   attn.qkvg, gdn.qkvz, gdn.ab, gdn.conv, mlp.gate_up, lm_head - whole heads per rank;
                                q/gate heads follow their kv head, gate/up row pairs stay together
  row-parallel (k of W)         attn.o, gdn.out, mlp.down - the k range of the rank's heads / MLP columns; the
                                products are stored as fp32 (Q38_EPI_STORE_F32), summed over the ranks, and enter
                                the residual through q38_residual_update
  replicated                    embedding, norms' vectors, the residual stream itself
KV cache and GDN state hold only the rank's heads. With fewer kv heads than ranks a kv head is held by
world / kv_heads ranks, each serving its own query heads of that kv head.

Python here is plumbing (shard slicing with numpy, buffers as torch tensors, torch.distributed for the all-reduce);
every operator is a kernel of libq38_kernels.so called through the C ABI.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import bqformat as bq

PAGE, HD, GD = 64, 256, 128


# ----------------------------------------------------------------------------------------------------
# shard arithmetic (pure numpy: also exercised by the CPU tests)
# ----------------------------------------------------------------------------------------------------
def _hi_slab_bytes(bits: int) -> int:
    return {4: 0, 5: 128, 6: 256, 8: 512}[bits]


def shard_rows(p: bq.Packed, ranges) -> bq.Packed:
    """The rows [a, b) of every range (multiples of 64), concatenated, as a BQ tensor of its own."""
    blocks = []
    for a, b in ranges:
        assert a % 64 == 0 and b % 64 == 0 and 0 <= a <= b <= p.n, (a, b, p.n)
        blocks += list(range(a // 64, b // 64))
    nb = p.n // 64

    def take(raw: bytes) -> bytes:
        if not raw:
            return b""
        return np.frombuffer(raw, dtype=np.uint8).reshape(nb, -1)[blocks].tobytes()
    return bq.Packed(p.bits, 64 * len(blocks), p.k, take(p.lo), take(p.hi), take(p.scales))


def shard_k(p: bq.Packed, k0: int, k1: int) -> bq.Packed:
    """Columns [k0, k1) (multiples of 64) of every row."""
    assert k0 % 64 == 0 and k1 % 64 == 0 and 0 <= k0 < k1 <= p.k
    nb = p.n // 64
    lo = np.frombuffer(p.lo, dtype=np.uint8).reshape(nb, p.k // 16, 512)[:, k0 // 16:k1 // 16].tobytes()
    hb = _hi_slab_bytes(p.bits)
    hi = (np.frombuffer(p.hi, dtype=np.uint8).reshape(nb, p.k // 16, hb)[:, k0 // 16:k1 // 16].tobytes() if hb else b"")
    sc = np.frombuffer(p.scales, dtype=np.uint8).reshape(nb, p.k // 64, 128)[:, k0 // 64:k1 // 64].tobytes()
    return bq.Packed(p.bits, p.n, k1 - k0, lo, hi, sc)


@dataclass
class RankPlan:
    rank: int
    world: int
    q_heads: range        # attention query heads of this rank
    kv_head: int          # its (single) kv head when world >= kv heads, else first of kv_heads
    kv_heads: range
    k_heads: range        # GDN key heads
    v_heads: range        # GDN value heads
    mlp_cols: range       # columns of the MLP intermediate
    vocab_rows: range     # rows of the LM head (multiples of 128)


def rank_plan(cfg: dict, rank: int, world: int) -> RankPlan:
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    lk, lv, inter, vocab = (cfg["linear_num_key_heads"], cfg["linear_num_value_heads"], cfg["intermediate_size"],
                            cfg["vocab_size"])
    assert nq % world == 0 and lk % world == 0 and lv % world == 0 and (inter // 64) % world == 0, "heads must divide"
    assert nkv % world == 0 or world % nkv == 0
    qh = range(rank * nq // world, (rank + 1) * nq // world)
    if nkv >= world:
        kvh = range(rank * nkv // world, (rank + 1) * nkv // world)
    else:
        kvh = range(qh.start // (nq // nkv), qh.start // (nq // nkv) + 1)
        assert (qh.stop - 1) // (nq // nkv) == kvh.start, "a rank's query heads must share one kv head"
    tiles = (vocab + 127) // 128
    t0, t1 = rank * tiles // world, (rank + 1) * tiles // world
    return RankPlan(rank, world, qh, kvh.start, kvh, range(rank * lk // world, (rank + 1) * lk // world),
                    range(rank * lv // world, (rank + 1) * lv // world),
                    range(rank * inter // world, (rank + 1) * inter // world), range(128 * t0, 128 * t1))


def qkvg_row_ranges(cfg: dict, plan: RankPlan):
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    q0, g0, k0, v0 = 0, nq * HD, 2 * nq * HD, 2 * nq * HD + nkv * HD
    return [(q0 + plan.q_heads.start * HD, q0 + plan.q_heads.stop * HD),
            (g0 + plan.q_heads.start * HD, g0 + plan.q_heads.stop * HD),
            (k0 + plan.kv_heads.start * HD, k0 + plan.kv_heads.stop * HD),
            (v0 + plan.kv_heads.start * HD, v0 + plan.kv_heads.stop * HD)]


def qkvz_row_ranges(cfg: dict, plan: RankPlan):
    lk, lv = cfg["linear_num_key_heads"], cfg["linear_num_value_heads"]
    q0, k0, v0, z0 = 0, lk * GD, 2 * lk * GD, 2 * lk * GD + lv * GD
    return [(q0 + plan.k_heads.start * GD, q0 + plan.k_heads.stop * GD),
            (k0 + plan.k_heads.start * GD, k0 + plan.k_heads.stop * GD),
            (v0 + plan.v_heads.start * GD, v0 + plan.v_heads.stop * GD),
            (z0 + plan.v_heads.start * GD, z0 + plan.v_heads.stop * GD)]


def _pad128(p: bq.Packed) -> bq.Packed:
    """Zero-row padding up to a multiple of 128 rows (a GEMM tile is two 64-row blocks)."""
    if p.n % 128 == 0:
        return p
    z = lambda raw: raw + bytes(len(raw) // (p.n // 64)) if raw else b""
    return bq.Packed(p.bits, p.n + 64, p.k, z(p.lo), z(p.hi), z(p.scales))


# ----------------------------------------------------------------------------------------------------
# runner
# ----------------------------------------------------------------------------------------------------
class _DevBQ:
    def __init__(self, pkg, p: bq.Packed, rows=None):
        p = _pad128(p)
        up = lambda raw: torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda() if raw else None
        self.lo, self.hi, self.sc = up(p.lo), up(p.hi), up(p.scales)
        self.n, self.k, self.rows = p.n, p.k, rows if rows is not None else p.n
        self.desc = pkg.BQWeight(pkg.ptr(self.lo), pkg.ptr(self.hi), pkg.ptr(self.sc), p.bits, p.n, p.k, self.rows)


class PeerBuffers:
    """Receive buffers, flags and call counters of the all-reduce that runs inside the row-parallel GEMM
    (Q38_EPI_ALLREDUCE_RESIDUAL): allocated by the library so that other processes can map them, the handles exchanged
    over `dist`, every peer's memory opened here. `dist=None`: a single rank, which pushes to and pulls from itself."""

    def __init__(self, pkg, hidden: int, rank: int, world: int, dist=None, poll_limit: int = 0):
        assert 1 <= world <= pkg.MAX_PEERS and hidden % 128 == 0
        self.pkg, self.K, self.world, self.rank = pkg, pkg.kernels(), world, rank
        tiles = hidden // 128
        sizes = (2 * world * pkg.ALLREDUCE_ROWS * hidden * 4, tiles * world * 4)
        self.own = []
        for nbytes in sizes + (tiles * 4,):
            ptr = C.c_void_p()
            pkg.check(self.K.q38_peer_alloc(nbytes, C.byref(ptr)))
            self.own.append(ptr.value)
        handles = []
        for ptr in self.own[:2]:
            h = C.create_string_buffer(64)
            pkg.check(self.K.q38_peer_export(ptr, h))
            handles.append(h.raw)
        everyone = [None] * world
        if dist is not None and world > 1:
            dist.all_gather_object(everyone, handles)
        else:
            everyone[rank] = handles
        self.opened = []
        self.absent = []  # world > 1 without a group (tests of the bounded wait): local stand-ins nobody ever writes
        self.desc = pkg.PeerAllreduce()
        self.desc.world, self.desc.rank, self.desc.seq, self.desc.poll_limit = world, rank, self.own[2], poll_limit
        for r in range(world):
            if r == rank:
                self.desc.recv[r], self.desc.flags[r] = self.own[0], self.own[1]
                continue
            for which in range(2):
                ptr = C.c_void_p()
                if everyone[r] is None:
                    pkg.check(self.K.q38_peer_alloc(sizes[which], C.byref(ptr)))
                    self.absent.append(ptr.value)
                else:
                    pkg.check(self.K.q38_peer_open(everyone[r][which], C.byref(ptr)))
                    self.opened.append(ptr.value)
                if which == 0:
                    self.desc.recv[r] = ptr.value
                else:
                    self.desc.flags[r] = ptr.value
        if dist is not None and world > 1:
            dist.barrier()  # nobody pushes before everybody has its buffers mapped

    def close(self, dist=None):
        """Unmaps the peers' memory, then (after a barrier: nobody may still be writing here) frees this rank's."""
        for ptr in self.opened:
            self.K.q38_peer_close(ptr)
        self.opened = []
        if dist is not None and self.world > 1:
            dist.barrier()
        for ptr in self.own + self.absent:
            self.K.q38_peer_free(ptr)
        self.own, self.absent = [], []


class TPRunner:
    """One request, sharded over `dist`'s ranks (dist=None: a single rank, the same code path without all-reduce).
    `fused_allreduce`: steps of up to 16 tokens sum the row-parallel projections inside the GEMM kernel, over peer
    memory (PeerBuffers), instead of NCCL all-reduce + q38_residual_update."""

    def __init__(self, pkg, model_path, rank: int = 0, world: int = 1, dist=None, max_tokens: int = 512,
                 max_context: int = 4096, fused_allreduce: bool = False, poll_limit: int = 0):
        self.pkg, self.K, self.dist = pkg, pkg.kernels(), dist if world > 1 else None
        self.rank, self.world = rank, world
        self.peers = None
        self._fused, self._poll_limit = fused_allreduce, poll_limit
        self.use_fused = True  # False: keep the peer buffers but take the NCCL path (for comparisons)
        f = bq.Q38File(model_path)
        cfg = self.cfg = f.config
        plan = self.plan = rank_plan(cfg, rank, world)
        H, self.H = cfg["hidden_size"], cfg["hidden_size"]
        self.eps = float(cfg["rms_norm_eps"])
        dev = lambda t: t.contiguous().cuda()
        self.nq, self.nkv = len(plan.q_heads), len(plan.kv_heads)
        self.lk, self.lv = len(plan.k_heads), len(plan.v_heads)
        self.conv_dim = (2 * self.lk + self.lv) * GD
        self.inter = len(plan.mlp_cols)
        self.embed = dev(f.direct("embed"))
        self.layers = []
        for i, kind in enumerate(cfg["layer_types"]):
            L = {"attention": kind == "full_attention"}
            if L["attention"]:
                L["in"] = _DevBQ(pkg, shard_rows(f.packed(f"{i}.attn.qkvg"), qkvg_row_ranges(cfg, plan)))
                L["out"] = _DevBQ(pkg, shard_k(f.packed(f"{i}.attn.o"), plan.q_heads.start * HD, plan.q_heads.stop * HD),
                                  rows=H)
                L["q_norm"], L["k_norm"] = dev(f.direct(f"{i}.attn.q_norm")), dev(f.direct(f"{i}.attn.k_norm"))
            else:
                L["in"] = _DevBQ(pkg, shard_rows(f.packed(f"{i}.gdn.qkvz"), qkvz_row_ranges(cfg, plan)))
                L["out"] = _DevBQ(pkg, shard_k(f.packed(f"{i}.gdn.out"), plan.v_heads.start * GD, plan.v_heads.stop * GD),
                                  rows=H)
                lv_all = cfg["linear_num_value_heads"]
                ab = f.direct(f"{i}.gdn.ab")
                vs = slice(plan.v_heads.start, plan.v_heads.stop)
                L["ab"] = dev(torch.cat([ab[vs], ab[lv_all + plan.v_heads.start:lv_all + plan.v_heads.stop]]))
                conv = f.direct(f"{i}.gdn.conv")
                rows = [r for a, b in qkvz_row_ranges(cfg, plan)[:3] for r in range(a, b)]
                L["conv"] = dev(conv[rows])
                L["A"], L["dt"] = dev(f.direct(f"{i}.gdn.A")[vs]), dev(f.direct(f"{i}.gdn.dt_bias")[vs])
                L["norm"] = dev(f.direct(f"{i}.gdn.norm"))
            gu = f.packed(f"{i}.mlp.gate_up")
            L["gate_up"] = _DevBQ(pkg, shard_rows(gu, [(2 * plan.mlp_cols.start, 2 * plan.mlp_cols.stop)]))
            L["down"] = _DevBQ(pkg, shard_k(f.packed(f"{i}.mlp.down"), plan.mlp_cols.start, plan.mlp_cols.stop), rows=H)
            self.layers.append(L)
        head = f.packed("lm_head")
        self.vocab = cfg["vocab_size"]
        v1 = min(plan.vocab_rows.stop, head.n)
        self.head = _DevBQ(pkg, shard_rows(head, [(plan.vocab_rows.start, v1)]),
                           rows=max(0, min(self.vocab, v1) - plan.vocab_rows.start))
        self.head_rows_max = 128 * (((self.vocab + 127) // 128 + world - 1) // world)

        # ---- state: this rank's kv heads / GDN heads, one sequence (slot 0) ----
        n_attn = sum(1 for L in self.layers if L["attention"])
        n_gdn = len(self.layers) - n_attn
        self.pages = (max_context + PAGE - 1) // PAGE
        self.page_bytes = int(self.K.q38_kv_page_bytes(pkg.KV_INT8, self.nkv))
        self.kv_pool = torch.zeros(max(1, n_attn) * self.pages * self.page_bytes, dtype=torch.uint8, device="cuda")
        self.table = torch.arange(self.pages, dtype=torch.int32, device="cuda").reshape(1, -1).contiguous()
        self.kv = pkg.KvCacheDesc(pkg.ptr(self.kv_pool), pkg.KV_INT8, self.nkv, self.pages, self.page_bytes,
                                  self.pages * self.page_bytes, pkg.ptr(self.table), self.pages)
        self.rec = torch.zeros((1, max(1, n_gdn), self.lv, GD, GD), dtype=torch.float32, device="cuda")
        self.conv_state = torch.zeros((1, max(1, n_gdn), 3, self.conv_dim), dtype=torch.bfloat16, device="cuda")
        self.gdn_state = pkg.GdnStateDesc(pkg.ptr(self.rec), pkg.ptr(self.conv_state), max(1, n_gdn))
        self.gdn_dims = None

        # ---- activations ----
        T = self.T = max_tokens
        f32 = lambda *s: torch.empty(s, dtype=torch.float32, device="cuda")
        b16 = lambda *s: torch.empty(s, dtype=torch.bfloat16, device="cuda")
        self.proj_ld = max(2 * self.nq * HD + 2 * self.nkv * HD, self.conv_dim + self.lv * GD)
        self.residual, self.xbf, self.partials = f32(T, H), b16(T, H), f32(T, H // 128)
        self.proj, self.delta = b16(T, self.proj_ld), f32(T, H)
        self.ab, self.qkv = f32(T, 2 * self.lv), f32(T, self.conv_dim)
        self.mixer, self.act = b16(T, max(self.nq * HD, self.lv * GD)), b16(T, self.inter)
        self.q16 = torch.empty((T, self.nq, HD), dtype=torch.float16, device="cuda")
        # decode: one row, up to 256 splits (one sequence must fill the GPU); prefill: one row per token of a chunk with up
        # to 16 splits, so that the few query tiles of a rank (one kv head) cut their keys over several CTAs
        self.prefill_splits = 16
        self.split = f32(max(1, self.nq) * max(256, T * self.prefill_splits) * (HD + 2))
        self.logits_local = f32(self.head_rows_max)
        self.gdn_scratch = f32(int(self.K.q38_gdn_chunk_scratch_floats(T, 1, max(1, self.lv))))
        sms = self.K.q38_num_sms()
        self.ws_partials = f32(2 * sms * 128 * 512)
        self.ws_counters = torch.zeros(65536, dtype=torch.int32, device="cuda")
        self.ws = pkg.GemmWorkspace(pkg.ptr(self.ws_partials), self.ws_partials.numel(), pkg.ptr(self.ws_counters), 65536)
        self.gdn_dims = pkg.GdnDims(self.lk, self.lv, self.conv_dim, self.proj_ld)
        self.reduce_calls = self.fused_calls = 0
        if self._fused:
            self.peers = PeerBuffers(pkg, H, rank, world, self.dist, self._poll_limit)
        # step inputs live in fixed device buffers, so that a captured decode step can be replayed
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")
        self.m_seq_start, self.m_seq_slot, self.m_seq_pos0 = i32(2), i32(1), i32(1)
        self.m_tok_pos, self.m_tok_seq, self.m_tokens = i32(T), i32(T), i32(T)
        self._graph = None

    # ------------------------------------------------------------------------------------------------
    def _gemm(self, a, m, w, ep):
        self.pkg.check(self.K.q38_qgemm(self.pkg.ptr(a), m, C.byref(w.desc), C.byref(ep), C.byref(self.ws),
                                        self._stream, -1))

    def _into_residual(self, a, m, w):
        """Row-parallel projection: fp32 partial product, sum over the ranks, then the Residual epilogue as an op."""
        pkg = self.pkg
        if self.peers is not None and self.use_fused and m <= pkg.ALLREDUCE_ROWS:
            # one kernel: the partial product, its sum over the ranks through peer memory, the residual update
            ep = pkg.GemmEpilogue(pkg.EPI_ALLREDUCE_RESIDUAL, None, 0, 0, pkg.ptr(self.residual), pkg.ptr(self.xbf),
                                  pkg.ptr(self.partials), None, 0, self.eps, C.pointer(self.peers.desc))
            self._gemm(a, m, w, ep)
            self.fused_calls += 1
            return
        ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(self.delta), self.H, self.H, None, None, None, None, 0, self.eps)
        self._gemm(a, m, w, ep)
        if self.dist is not None:
            self.dist.all_reduce(self.delta[:m])
            self.reduce_calls += 1
        pkg.check(self.K.q38_residual_update(pkg.ptr(self.delta), m, self.H, pkg.ptr(self.residual), pkg.ptr(self.xbf),
                                             pkg.ptr(self.partials), self._stream))

    def _set_inputs(self, tokens, pos0: int) -> int:
        m = int(len(tokens))
        assert 0 < m <= self.T and pos0 + m <= self.pages * PAGE
        host = lambda v: torch.tensor(v, dtype=torch.int32)
        self.m_seq_start.copy_(host([0, m]))
        self.m_seq_pos0.copy_(host([pos0]))
        self.m_tok_pos[:m].copy_(host(list(range(pos0, pos0 + m))))
        self.m_tokens[:m].copy_(host([int(t) for t in tokens]))
        return m

    def forward(self, tokens, pos0: int):
        """Runs `tokens` (1-D int array) of the request at positions pos0.. through all layers (the residual of the
        last token is what logits() reads)."""
        m = self._set_inputs(tokens, pos0)
        self._run(m)

    def decode_replay(self, token: int, pos: int):
        """One decode step as a CUDA graph: captured on first use (kernels and all-reduces alike), replayed after."""
        self._set_inputs([token], pos)
        if self._graph is None:
            self._run(1)  # warm-up outside capture (one-time attribute set-up inside the launchers)
            torch.cuda.synchronize()
            self._set_inputs([token], pos)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._run(1)
            self._graph = g
            # the capture did not execute: the state still holds the warm-up step's effect, which equals this step's
            return
        self._graph.replay()

    def _run(self, m: int):
        pkg, K = self.pkg, self.K
        self._stream = torch.cuda.current_stream().cuda_stream
        s = self._stream
        batch = pkg.BatchDesc(1, m, m, pkg.ptr(self.m_seq_start), pkg.ptr(self.m_seq_slot), pkg.ptr(self.m_seq_pos0),
                              pkg.ptr(self.m_tok_pos), pkg.ptr(self.m_tok_seq))
        tok = self.m_tokens
        H, eps = self.H, self.eps
        pkg.check(K.q38_embed(pkg.ptr(self.embed), pkg.ptr(tok), m, H, pkg.ptr(self.residual), pkg.ptr(self.xbf),
                              pkg.ptr(self.partials), s))
        decode = m == 1
        attn_i = gdn_i = 0
        for L in self.layers:
            ep = pkg.GemmEpilogue(pkg.EPI_STORE_BF16, pkg.ptr(self.proj), self.proj_ld, L["in"].rows, None, None, None,
                                  pkg.ptr(self.partials), H, eps)
            self._gemm(self.xbf, m, L["in"], ep)
            if L["attention"]:
                qp = pkg.QkNormRopeParams(pkg.ptr(self.proj), self.proj_ld, pkg.ptr(L["q_norm"]), pkg.ptr(L["k_norm"]), eps,
                                          float(self.cfg["rope_theta"]), self.nq, self.nkv, pkg.ptr(self.q16), attn_i)
                pkg.check(K.q38_qk_norm_rope_append(C.byref(qp), C.byref(batch), C.byref(self.kv), s))
                ap = pkg.AttentionParams(pkg.ptr(self.q16), pkg.ptr(self.proj) + self.nq * HD * 2, self.proj_ld,
                                         pkg.ptr(self.mixer), self.nq, self.nkv, attn_i, pkg.ptr(self.split),
                                         256 if decode else self.prefill_splits, 1 if decode else self.T)
                fn = K.q38_attention_decode if decode else K.q38_attention_prefill
                pkg.check(fn(C.byref(ap), C.byref(batch), C.byref(self.kv), s))
                attn_i += 1
            else:
                pkg.check(K.q38_gdn_ab(pkg.ptr(self.xbf), m, H, pkg.ptr(L["ab"]), 2 * self.lv, pkg.ptr(self.partials), eps,
                                       pkg.ptr(self.ab), s))
                cp = pkg.GdnConvParams(pkg.ptr(self.proj), pkg.ptr(L["conv"]), pkg.ptr(self.qkv), gdn_i)
                pkg.check(K.q38_gdn_conv(C.byref(cp), C.byref(self.gdn_dims), C.byref(batch), C.byref(self.gdn_state), s))
                rp = pkg.GdnRecurrenceParams(pkg.ptr(self.qkv), pkg.ptr(self.ab), pkg.ptr(L["A"]), pkg.ptr(L["dt"]),
                                             pkg.ptr(self.proj) + self.conv_dim * 2, self.proj_ld, pkg.ptr(L["norm"]), eps,
                                             pkg.ptr(self.mixer), gdn_i)
                if m >= 16:
                    pkg.check(K.q38_gdn_recurrence_chunked(C.byref(rp), C.byref(self.gdn_dims), C.byref(batch),
                                                           C.byref(self.gdn_state), pkg.ptr(self.gdn_scratch),
                                                           self.gdn_scratch.numel(), s))
                else:
                    pkg.check(K.q38_gdn_recurrence(C.byref(rp), C.byref(self.gdn_dims), C.byref(batch),
                                                   C.byref(self.gdn_state), s))
                gdn_i += 1
            self._into_residual(self.mixer, m, L["out"])
            ep = pkg.GemmEpilogue(pkg.EPI_SWIGLU, pkg.ptr(self.act), self.inter, 0, None, None, None, pkg.ptr(self.partials),
                                  H, eps)
            self._gemm(self.xbf, m, L["gate_up"], ep)
            self._into_residual(self.act, m, L["down"])
        self._last = m - 1

    def logits(self) -> np.ndarray:
        """Full-vocabulary fp32 logits of the last token forward() ran (every rank returns the same array)."""
        pkg = self.pkg
        self._stream = torch.cuda.current_stream().cuda_stream  # not the stream a captured step was recorded on
        row = self._last
        x = self.xbf[row:row + 1]
        part = self.partials[row:row + 1]
        n_local = self.head.rows
        ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(self.logits_local), self.head_rows_max, n_local, None, None, None,
                              pkg.ptr(part), self.H, self.eps)
        if n_local > 0:
            self._gemm(x, 1, self.head, ep)
        if self.dist is None:
            torch.cuda.synchronize()
            return self.logits_local[:self.vocab].cpu().numpy()
        gathered = [torch.empty_like(self.logits_local) for _ in range(self.world)]
        self.dist.all_gather(gathered, self.logits_local)
        out = []
        for r, g in enumerate(gathered):
            p = rank_plan(self.cfg, r, self.world)
            out.append(g[:max(0, min(self.vocab, p.vocab_rows.stop) - p.vocab_rows.start)])
        torch.cuda.synchronize()
        return torch.cat(out).cpu().numpy()

    def close(self):
        """Drops the captured step. Call before the process group is destroyed: a live graph that holds captured
        collectives keeps the communicator busy and the group's shutdown waits for it."""
        torch.cuda.synchronize()
        self._graph = None
        if self.peers is not None:
            self.peers.close(self.dist)
            self.peers = None

    def device_error(self) -> int:
        return int(self.K.q38_device_error(1))
