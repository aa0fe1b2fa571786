"""GPU parity tests: every kernel, called through the C ABI, against the CPU oracle on the same seeded
inputs. Shapes, seeds and tolerances restate the reference's own kernel tests
(reference tests/gpu/test_kernels.cu); cases the reference does not cover (ragged B > 1, GQA with 4 KV
heads, several layers in the pools, shuffled page tables, 27B-sized matrices) are added."""

import ctypes as C

import numpy as np
import pytest
import torch

import q38_testlib as tl
from q38_testlib import bq, pkg

pytestmark = pytest.mark.gpu


def K():
    return pkg.kernels()


def sync_ok():
    torch.cuda.synchronize()
    assert K().q38_device_error(1) == 0


# ---------------------------------------------------------------------------------------------------
# BQ decode: bit-exact dequantised weights
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_dequantised_weights_are_bit_exact(bits):
    gold = np.load(tl.ROOT / "tests" / "golden" / "bq_golden.npz")
    cases = [bq.Packed(bits, 128, 192, gold[f"lo{bits}"].tobytes(), gold[f"hi{bits}"].tobytes(),
                       gold[f"sc{bits}"].tobytes()),
             tl.make_bq(256, 320, bits, seed=40 + bits)]
    for p in cases:
        w = tl.DeviceBQ(p)
        out = torch.empty((p.n, p.k), dtype=torch.bfloat16, device="cuda")
        pkg.check(K().q38_bq_dequant(C.byref(w.desc), pkg.ptr(out), None))
        sync_ok()
        want = tl.oracle().dequant(p)
        assert np.array_equal(out.float().cpu().numpy(), want)


# ---------------------------------------------------------------------------------------------------
# qgemm
# ---------------------------------------------------------------------------------------------------
def run_gemm_f32(a_dev, m, w, ws, config, sync=True):
    out = torch.empty((m, w.packed.n), dtype=torch.float32, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(out), w.packed.n, 0, None, None, None, None, 0, 1e-6)
    pkg.check(K().q38_qgemm(pkg.ptr(a_dev), m, C.byref(w.desc), C.byref(ep), C.byref(ws) if ws else None, None, config))
    if sync:
        torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_qgemm_matches_oracle_all_configs(bits):
    rng = np.random.default_rng(42)
    ws = tl.Workspace()
    for (n, k) in ((256, 256), (1536, 192), (384, 1024)):
        p = tl.make_bq(n, k, bits, seed=bits * 100 + n, std=0.05, fast=(n > 256))
        w = tl.DeviceBQ(p)
        wd = tl.oracle().dequant(p)
        for m in (1, 3, 16, 17, 40, 64, 130, 300, 512):
            a = tl.bf16_round(rng.standard_normal((m, k)))
            a_dev = tl.to_dev_bf16(a)
            want = np.zeros((m, n), np.float32)
            tl.oracle().qgemm(a, wd, None, 3, out=want, ldo=n)
            mag = np.abs(a).astype(np.float64) @ np.abs(wd).astype(np.float64).T
            for cfg in range(K().q38_qgemm_num_configs()):
                if bits == 8 and K().q38_qgemm_config_name(cfg) == b"umma_t512":
                    with pytest.raises(pkg.KernelError):  # not built: shared memory cannot hold two raw stages
                        run_gemm_f32(a_dev, m, w, ws.desc, cfg)
                    continue
                for use_ws in (True, False):
                    got = run_gemm_f32(a_dev, m, w, ws.desc if use_ws else None, cfg)
                    err = np.abs(got.cpu().numpy().astype(np.float64) - want)
                    bad = err > 1e-6 + 2e-3 * mag
                    assert not bad.any(), (bits, n, k, m, cfg, use_ws, float(err.max()))
                    again = run_gemm_f32(a_dev, m, w, ws.desc if use_ws else None, cfg)
                    assert torch.equal(got, again), "second run is not bit-identical"
    sync_ok()
    assert int(ws.counters.abs().sum()) == 0, "tile counters must reset themselves"


def _epilogue_case(m, H, I, n_in, n_store, seed, bits=(5, 4, 6)):
    """Inputs and oracle results of the three fused epilogues for one token count."""
    rng = np.random.default_rng(seed)
    o = tl.oracle()
    residual = tl.bf16_round(rng.standard_normal((m, H)) * 3)
    xbf = tl.bf16_round(residual)
    partials = np.stack([o.norm_partials(residual[i]) for i in range(m)])
    rs = np.array([o.norm_row_scale(partials[i], H, 1e-6) for i in range(m)], np.float32)
    c = {"m": m, "H": H, "I": I, "n_in": n_in, "n_store": n_store, "residual": residual, "partials": partials,
         "xbf_dev": tl.to_dev_bf16(xbf), "part_dev": torch.from_numpy(partials).cuda()}
    # StoreBF16 + folded-norm row scale, with padded rows trimmed by n_store
    p = tl.make_bq(n_in, H, bits[0], seed=seed + 1, std=0.05, fast=True)
    c["w_store"], wd = tl.DeviceBQ(p, rows=n_store), o.dequant(p)
    c["want_store"] = np.zeros((m, n_in), np.float32)
    o.qgemm(xbf, wd, rs, 0, out=c["want_store"], ldo=n_in)
    # SwiGLU on interleaved gate/up columns
    p = tl.make_bq(2 * I, H, bits[1], seed=seed + 2, std=0.05, fast=True)
    c["w_swiglu"], wd = tl.DeviceBQ(p), o.dequant(p)
    c["want_swiglu"] = np.zeros((m, I), np.float32)
    o.qgemm(xbf, wd, rs, 1, out=c["want_swiglu"], ldo=I)
    # Residual: residual += C, xbf == bf16(residual) exactly, next-norm partials
    p = tl.make_bq(H, I, bits[2], seed=seed + 3, std=0.05, fast=True)
    c["w_res"], wd = tl.DeviceBQ(p), o.dequant(p)
    act = tl.bf16_round(rng.standard_normal((m, I)) * 0.5)
    c["act_dev"] = tl.to_dev_bf16(act)
    c["res_want"], c["xbf_want"], c["part_want"] = residual.copy(), np.zeros_like(residual), np.zeros_like(partials)
    o.qgemm(act, wd, None, 2, residual=c["res_want"], xbf=c["xbf_want"], partials=c["part_want"])
    return c


def _check_epilogues(c, ws, config):
    m, H, I, n_in, n_store = c["m"], c["H"], c["I"], c["n_in"], c["n_store"]
    tag = (m, K().q38_qgemm_config_name(config) if config >= 0 else "auto")
    out = torch.full((m, n_in), 7.0, dtype=torch.bfloat16, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_STORE_BF16, pkg.ptr(out), n_in, n_store, None, None, None, pkg.ptr(c["part_dev"]), H, 1e-6)
    pkg.check(K().q38_qgemm(pkg.ptr(c["xbf_dev"]), m, C.byref(c["w_store"].desc), C.byref(ep), C.byref(ws.desc), None, config))
    got, want = out.float().cpu().numpy(), c["want_store"]
    assert np.all(np.abs(got[:, :n_store] - want[:, :n_store]) <= 1e-3 + 2e-2 * np.abs(want[:, :n_store])), tag
    assert np.all(got[:, n_store:] == 7.0), ("columns beyond n_store must not be written", tag)

    out = torch.empty((m, I), dtype=torch.bfloat16, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_SWIGLU, pkg.ptr(out), I, 0, None, None, None, pkg.ptr(c["part_dev"]), H, 1e-6)
    pkg.check(K().q38_qgemm(pkg.ptr(c["xbf_dev"]), m, C.byref(c["w_swiglu"].desc), C.byref(ep), C.byref(ws.desc), None, config))
    got, want = out.float().cpu().numpy(), c["want_swiglu"]
    assert np.all(np.abs(got - want) <= 2e-2 * (np.abs(want) + 1e-3 * np.abs(want).max())), tag

    res_dev = torch.from_numpy(c["residual"].copy()).cuda()
    xbf_out = torch.empty((m, H), dtype=torch.bfloat16, device="cuda")
    part_out = torch.empty((m, H // 128), dtype=torch.float32, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_RESIDUAL, None, 0, 0, pkg.ptr(res_dev), pkg.ptr(xbf_out), pkg.ptr(part_out), None, 0, 1e-6)
    pkg.check(K().q38_qgemm(pkg.ptr(c["act_dev"]), m, C.byref(c["w_res"].desc), C.byref(ep), C.byref(ws.desc), None, config))
    sync_ok()
    res_got = res_dev.cpu().numpy()
    assert np.all(np.abs(res_got - c["res_want"]) <= 1e-3 + 1e-3 * np.abs(c["res_want"])), tag
    assert np.array_equal(xbf_out.float().cpu().numpy(), tl.bf16_round(res_got)), tag
    assert np.all(np.abs(part_out.cpu().numpy() - c["part_want"]) <= 1e-3 + 1e-4 * np.abs(c["part_want"])), tag


@pytest.mark.parametrize("m", [1, 5, 16, 17, 33, 64, 77, 130, 257, 300])
def test_qgemm_epilogues(m):
    """StoreBF16 (+ n_store trimming), SwiGLU and Residual through the dispatcher's own choice and through every
    tile configuration of both kernels (a configuration smaller than m is applied to row blocks)."""
    c = _epilogue_case(m, H=512, I=1024, n_in=1152, n_store=1100, seed=7)
    ws = tl.Workspace()
    for config in range(-1, K().q38_qgemm_num_configs()):
        _check_epilogues(c, ws, config)
    assert int(ws.counters.abs().sum()) == 0


@pytest.mark.parametrize("m", [33, 64])
def test_qgemm_epilogues_27b_width(m):
    """The epilogues at the 27B hidden size (40 weight tiles for the Residual projections, the cut of every tile over
    three CTAs) and a 4-bit gate/up block of 68 tiles, decode-batch token counts."""
    c = _epilogue_case(m, H=5120, I=4352, n_in=2048, n_store=2000, seed=11)
    ws = tl.Workspace()
    names = {K().q38_qgemm_config_name(i).decode(): i for i in range(K().q38_qgemm_num_configs())}
    for config in (-1, names["tmem_t64"], names["tmem_t128"], names["umma_t64"], names["stream_m16"]):
        _check_epilogues(c, ws, config)
    assert int(ws.counters.abs().sum()) == 0


@pytest.mark.parametrize("n,k,bits", [(34816, 5120, 4), (5120, 17408, 6)])
def test_qgemm_27b_shapes(n, k, bits):
    """Full-size projection matrices; the oracle is evaluated on a seeded subset of output columns."""
    g = torch.Generator(device="cuda").manual_seed(n)
    wt = torch.randn((n, k), generator=g, device="cuda") * 0.02
    codes, scales = bq.quantize_absmax(wt, bits)
    p = bq.pack(codes.cpu(), scales.cpu(), bits)
    w = tl.DeviceBQ(p)
    ws = tl.Workspace()
    rng = np.random.default_rng(5)
    cols = np.sort(rng.choice(n, size=192, replace=False))
    wd = bq.dequantize(codes[cols].cpu(), scales[cols].cpu()).numpy()
    # whole-matrix dequant check against the python definition (bit-exact)
    deq = torch.empty((n, k), dtype=torch.bfloat16, device="cuda")
    pkg.check(K().q38_bq_dequant(C.byref(w.desc), pkg.ptr(deq), None))
    assert torch.equal(deq[cols].float().cpu(), torch.from_numpy(wd))
    for m in (1, 8, 64, 300):  # streaming kernel, tcgen05 kernel with the weights in TMEM, two 256-token blocks per launch
        a = tl.bf16_round(rng.standard_normal((m, k)))
        want = np.zeros((m, len(cols)), np.float32)
        tl.oracle().qgemm(a, wd, None, 3, out=want, ldo=len(cols))
        mag = np.abs(a).astype(np.float64) @ np.abs(wd).astype(np.float64).T
        a_dev = tl.to_dev_bf16(a)
        got = run_gemm_f32(a_dev, m, w, ws.desc, -1)
        err = np.abs(got[:, cols].cpu().numpy().astype(np.float64) - want)
        assert not (err > 1e-6 + 2e-3 * mag).any(), (m, float(err.max()))
        assert torch.equal(got, run_gemm_f32(a_dev, m, w, ws.desc, -1))
    sync_ok()


@pytest.mark.parametrize("bits", [5, 8])
def test_qgemm_even_cut_over_all_sms(bits):
    """More than four tiles per SM (the LM head's regime): the tcgen05 kernel cuts the list of (tile, k-group) evenly
    over the SMs, so segments begin and end anywhere inside a tile - partial stages, units of one k-group, segments
    of a single unit - and the tiles' pieces meet in the workspace. 11 k-groups per tile make every remainder occur.
    Each configuration against the oracle on a seeded subset of columns, both operand paths bit-identical, and twenty
    launches back to back (each overlapping the tail of the one before) equal to a launch on its own."""
    n, k = 76800, 704
    g = torch.Generator(device="cuda").manual_seed(bits)
    wt = torch.randn((n, k), generator=g, device="cuda") * 0.02
    codes, scales = bq.quantize_absmax(wt, bits)
    p = bq.pack(codes, scales, bits)
    w = tl.DeviceBQ(p)
    ws = tl.Workspace()
    names = {K().q38_qgemm_config_name(c).decode(): c for c in range(K().q38_qgemm_num_configs())}
    rng = np.random.default_rng(bits)
    cols = np.sort(rng.choice(n, size=160, replace=False))
    wd = bq.dequantize(codes[cols].cpu(), scales[cols].cpu()).numpy()
    for m, tok in ((24, 32), (64, 64), (100, 128)):
        a = tl.bf16_round(rng.standard_normal((m, k)))
        want = np.zeros((m, len(cols)), np.float32)
        tl.oracle().qgemm(a, wd, None, 3, out=want, ldo=len(cols))
        mag = np.abs(a).astype(np.float64) @ np.abs(wd).astype(np.float64).T
        a_dev = tl.to_dev_bf16(a)
        outs = {}
        for name in (f"tmem_t{tok}", f"umma_t{tok}"):
            got = run_gemm_f32(a_dev, m, w, ws.desc, names[name])
            err = np.abs(got[:, cols].cpu().numpy().astype(np.float64) - want)
            assert not (err > 1e-6 + 2e-3 * mag).any(), (bits, m, name, float(err.max()))
            outs[name] = got
        assert torch.equal(outs[f"tmem_t{tok}"], outs[f"umma_t{tok}"]), (bits, m)
        for name in (f"tmem_t{tok}", f"umma_t{tok}"):
            for _ in range(20):
                last = run_gemm_f32(a_dev, m, w, ws.desc, names[name], sync=False)
            assert torch.equal(last, outs[name]), (bits, m, name, "back-to-back launches")
    sync_ok()
    assert int(ws.counters.abs().sum()) == 0, "tile counters must reset themselves"


@pytest.mark.parametrize("bits", [4, 5, 8])
def test_qgemm_operand_paths_give_the_same_bits(bits):
    """The tcgen05 kernel hands the decoded weights to the MMA either through shared memory (umma_*) or through
    tensor memory (tmem_*); the MMAs, their order over k and the epilogue are the same, so the outputs must be
    bit-identical, cut over k (with a workspace) or not."""
    names = {K().q38_qgemm_config_name(c).decode(): c for c in range(K().q38_qgemm_num_configs())}
    rng = np.random.default_rng(bits)
    ws = tl.Workspace()
    p = tl.make_bq(2048, 1536, bits, seed=40 + bits, std=0.05, fast=True)
    w = tl.DeviceBQ(p)
    for m, pairs in ((20, [("umma_t32", "tmem_t32")]), (64, [("umma_t64", "tmem_t64")]), (100, [("umma_t128", "tmem_t128")]),
                     (300, [("umma_t256", "tmem_t256"), ("umma_t256x2", "tmem_t256x2")])):
        a_dev = tl.to_dev_bf16(tl.bf16_round(rng.standard_normal((m, 1536))))
        for smem_cfg, tmem_cfg in pairs:
            for use_ws in (True, False):
                x = run_gemm_f32(a_dev, m, w, ws.desc if use_ws else None, names[smem_cfg])
                y = run_gemm_f32(a_dev, m, w, ws.desc if use_ws else None, names[tmem_cfg])
                assert torch.equal(x, y), (bits, m, smem_cfg, tmem_cfg, use_ws)
    sync_ok()


@pytest.mark.parametrize("bits", [4, 5, 6, 8])
def test_quantiser_on_gpu_equals_cpu(bits):
    """The MSE-search quantiser (reference tools/bqpack.py:40-102) is plain tensor arithmetic: run on the GPU it must
    give the codes and scales of the CPU run (which the golden fixtures pin to the reference's bytes)."""
    g = torch.Generator().manual_seed(100 + bits)
    w = torch.randn((384, 1024), generator=g) * 0.02
    w[5, 64:128] = 0.0          # a dead group
    w[7, 0] = 3.0               # an outlier
    c_cpu, s_cpu = bq.quantize_matrix(w, bits)
    c_gpu, s_gpu = bq.quantize_matrix(w.cuda(), bits)
    assert torch.equal(s_gpu.cpu(), s_cpu)
    assert torch.equal(c_gpu.cpu(), c_cpu)


# ---------------------------------------------------------------------------------------------------
# embed, ragged packing
# ---------------------------------------------------------------------------------------------------
def test_embed_matches_oracle():
    H, V = 512, 1024
    g = torch.Generator().manual_seed(1)
    table = (torch.randn((V, H), generator=g)).to(torch.bfloat16)
    tokens = torch.tensor([0, 5, 1023, 17, 17, 400], dtype=torch.int32)
    m = len(tokens)
    # device table and mapped pinned host table (zero-copy)
    host_table = table.clone().pin_memory()
    for tab in (table.cuda(), host_table):
        res = torch.empty((m, H), dtype=torch.float32, device="cuda")
        xbf = torch.empty((m, H), dtype=torch.bfloat16, device="cuda")
        part = torch.empty((m, H // 128), dtype=torch.float32, device="cuda")
        tok_d = tokens.cuda()
        pkg.check(K().q38_embed(pkg.ptr(tab), pkg.ptr(tok_d), m, H, pkg.ptr(res), pkg.ptr(xbf), pkg.ptr(part), None))
        sync_ok()
        rows = table[tokens.long()].float().numpy()
        assert np.array_equal(res.cpu().numpy(), rows)
        assert np.array_equal(xbf.float().cpu().numpy(), rows)
        want = np.stack([tl.oracle().norm_partials(rows[i]) for i in range(m)])
        assert np.all(np.abs(part.cpu().numpy() - want) <= 1e-4 + 1e-5 * np.abs(want))


def test_pack_ragged_matches_host_loops():
    rng = np.random.default_rng(3)
    for nseq in (1, 4, 64, 1500):
        counts = rng.integers(0, 9, size=nseq).astype(np.int32)
        counts[0] = max(counts[0], 1)
        pos0 = rng.integers(0, 5000, size=nseq).astype(np.int32)
        total = int(counts.sum())
        d = lambda a: torch.from_numpy(a).cuda()
        seq_start = torch.empty(nseq + 1, dtype=torch.int32, device="cuda")
        tok_pos = torch.empty(max(total, 1), dtype=torch.int32, device="cuda")
        tok_seq = torch.empty(max(total, 1), dtype=torch.int32, device="cuda")
        counts_d, pos0_d = d(counts), d(pos0)
        pkg.check(K().q38_pack_ragged(pkg.ptr(counts_d), pkg.ptr(pos0_d), nseq, total, pkg.ptr(seq_start),
                                      pkg.ptr(tok_pos), pkg.ptr(tok_seq), None))
        sync_ok()
        want_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        assert np.array_equal(seq_start.cpu().numpy(), want_start)
        want_pos = np.concatenate([pos0[b] + np.arange(counts[b]) for b in range(nseq)]).astype(np.int32)
        want_seq = np.concatenate([np.full(counts[b], b) for b in range(nseq)]).astype(np.int32)
        assert np.array_equal(tok_pos.cpu().numpy()[:total], want_pos)
        assert np.array_equal(tok_seq.cpu().numpy()[:total], want_seq)


# ---------------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------------
def run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode, split_rows=4):
    n = batch.num_tokens
    ld = proj.shape[1]
    proj_dev = tl.to_dev_bf16(proj)
    q16 = torch.empty((n, nq, 256), dtype=torch.float16, device="cuda")
    out = torch.empty((n, nq * 256), dtype=torch.bfloat16, device="cuda")
    qp = pkg.QkNormRopeParams(pkg.ptr(proj_dev), ld, pkg.ptr(qn_dev), pkg.ptr(kn_dev), 1e-6, 1e7, nq, nkv, pkg.ptr(q16), layer)
    pkg.check(K().q38_qk_norm_rope_append(C.byref(qp), C.byref(batch.desc), C.byref(pool.desc), None))
    scratch_rows = max(split_rows, batch.desc.num_seqs)
    max_splits = 64 if scratch_rows <= 64 else 16
    split = torch.empty(scratch_rows * nq * max_splits * 258, dtype=torch.float32, device="cuda")
    ap = pkg.AttentionParams(pkg.ptr(q16), pkg.ptr(proj_dev) + nq * 256 * 2, ld, pkg.ptr(out), nq, nkv, layer,
                             pkg.ptr(split), max_splits, scratch_rows)
    fn = K().q38_attention_decode if decode else K().q38_attention_prefill
    pkg.check(fn(C.byref(ap), C.byref(batch.desc), C.byref(pool.desc), None))
    sync_ok()
    return q16.float().cpu().numpy().reshape(n, nq * 256), out.float().cpu().numpy()


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("prefix", [0, 1, 63, 64, 300, 2100])
def test_attention_matches_oracle(dtype, prefix):
    """One sequence: chunked prefill up to `prefix`, then two decode tokens (6 q heads / 1 kv head)."""
    nq, nkv = 6, 1
    ld = 2 * nq * 256 + 2 * nkv * 256
    rng = np.random.default_rng(11 + prefix)
    r3 = np.random.default_rng(3)
    qn, kn = (1 + 0.2 * r3.standard_normal(256)).astype(np.float32), (1 + 0.2 * r3.standard_normal(256)).astype(np.float32)
    qn_dev, kn_dev = torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda()
    pool = tl.KvPool(nkv, layers=2, num_pages=64, slots=4, max_pages_per_seq=64, dtype=dtype)
    perm = np.random.default_rng(5).permutation(64).astype(np.int32)
    pool.table[2] = torch.from_numpy(perm).cuda()
    chunks, pos = [], 0
    sizes = (37, 64, 90, 211)
    while pos < prefix:
        n = min(sizes[len(chunks) % 4], prefix - pos)
        chunks.append((pos, n))
        pos += n
    chunks += [(prefix, 1), (prefix + 1, 1)]
    o = tl.oracle()
    okv = tl.OracleKv(o, nkv, prefix + 2)
    got_all, want_all = [], []
    layer = 1
    for pos0, n in chunks:
        proj = tl.bf16_round(rng.standard_normal((n, ld)))
        batch = tl.Batch([(2, pos0, n)])
        q_got, out_got = run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode=(n == 1))
        kd, vd = pool.read_sequence(layer, 2, pos0 + n)
        for i in range(n):
            q_ref = okv.append(nq, 1e-6, 1e7, proj[i], pos0 + i, qn, kn, 2 if dtype == 0 else 1)
            assert np.all(np.abs(q_got[i] - q_ref) <= 2e-3 + 2e-3 * np.abs(q_ref)), (pos0 + i)
            # K written by the kernel vs the oracle's quantisation: at most one int8 step apart
            for h in range(nkv):
                diff = np.abs(kd[h, pos0 + i] - okv.k[h, pos0 + i]).max()
                assert diff <= np.abs(okv.k[h, pos0 + i]).max() / 100.0 + 1e-3
        # attention over the cache contents the kernel actually wrote
        seen = tl.OracleKv(o, nkv, pos0 + n)
        seen.k[:], seen.v[:] = kd, vd
        for i in range(n):
            want_all.append(seen.attend(nq, q_got[i], proj[i, nq * 256:2 * nq * 256], pos0 + i))
            got_all.append(out_got[i])
    got, want = np.stack(got_all), np.stack(want_all)
    assert np.all(np.abs(got - want) <= 2e-2 * (np.abs(want) + 0.02 * np.abs(want).max()))


def test_attention_ragged_batch_gqa4_long_context():
    """B = 5 sequences decoded together, 8 q / 4 kv heads (group 2) and 24 / 4 (group 6), contexts up to 9000,
    shuffled page table, attention layer 2 of 3."""
    rng = np.random.default_rng(21)
    o = tl.oracle()
    for nq, nkv in ((8, 4), (24, 4)):
        ld = 2 * nq * 256 + 2 * nkv * 256
        qn = (1 + 0.2 * rng.standard_normal(256)).astype(np.float32)
        kn = (1 + 0.2 * rng.standard_normal(256)).astype(np.float32)
        qn_dev, kn_dev = torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda()
        ctx = [1, 64, 130, 4100, 9000]
        pages_needed = sum((c + 64) // 64 + 1 for c in ctx)
        pool = tl.KvPool(nkv, layers=3, num_pages=pages_needed + 3, slots=8, max_pages_per_seq=160, dtype=0)
        perm = np.random.default_rng(5).permutation(pages_needed + 3).astype(np.int32)
        used = 0
        slots = [6, 0, 3, 1, 5]
        for s, c in zip(slots, ctx):
            need = (c + 64) // 64 + 1
            pool.table[s, :need] = torch.from_numpy(perm[used:used + need]).cuda()
            used += need
        layer = 2
        # fill the caches by prefill chunks of 512 through the append kernel (K/V only matter here)
        for s, c in zip(slots, ctx):
            for p0 in range(0, c - 1, 512):
                n = min(512, c - 1 - p0)
                proj = tl.bf16_round(rng.standard_normal((n, ld)))
                batch = tl.Batch([(s, p0, n)])
                q16 = torch.empty((n, nq, 256), dtype=torch.float16, device="cuda")
                proj_d = tl.to_dev_bf16(proj)
                qp = pkg.QkNormRopeParams(pkg.ptr(proj_d), ld, pkg.ptr(qn_dev), pkg.ptr(kn_dev), 1e-6, 1e7,
                                          nq, nkv, pkg.ptr(q16), layer)
                pkg.check(K().q38_qk_norm_rope_append(C.byref(qp), C.byref(batch.desc), C.byref(pool.desc), None))
        # one decode step for all five
        proj = tl.bf16_round(rng.standard_normal((len(ctx), ld)))
        batch = tl.Batch([(s, c - 1, 1) for s, c in zip(slots, ctx)])
        q_got, out_got = run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode=True, split_rows=8)
        for b, (s, c) in enumerate(zip(slots, ctx)):
            kd, vd = pool.read_sequence(layer, s, c)
            seen = tl.OracleKv(o, nkv, c)
            seen.k[:], seen.v[:] = kd, vd
            want = seen.attend(nq, q_got[b], proj[b, nq * 256:2 * nq * 256], c - 1)
            assert np.all(np.abs(out_got[b] - want) <= 2e-2 * (np.abs(want) + 0.02 * np.abs(want).max())), (nq, b)
        # the same tokens as a ragged "prefill" batch of single-token chunks must agree as well
        _, out_pf = run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode=False, split_rows=8)
        assert np.all(np.abs(out_pf - out_got) <= 2e-2 * (np.abs(out_got) + 0.02 * np.abs(out_got).max()))


def fill_kv_random(pool, layer, nq, nkv, slot, upto, qn_dev, kn_dev, gen):
    """Appends `upto` tokens of N(0, 1) projections (drawn on the device) to a sequence's cache, 512 at a time."""
    ld = 2 * nq * 256 + 2 * nkv * 256
    for p0 in range(0, upto, 512):
        n = min(512, upto - p0)
        proj_d = torch.randn((n, ld), generator=gen, device="cuda").to(torch.bfloat16)
        batch = tl.Batch([(slot, p0, n)])
        q16 = torch.empty((n, nq, 256), dtype=torch.float16, device="cuda")
        qp = pkg.QkNormRopeParams(pkg.ptr(proj_d), ld, pkg.ptr(qn_dev), pkg.ptr(kn_dev), 1e-6, 1e7, nq, nkv, pkg.ptr(q16), layer)
        pkg.check(K().q38_qk_norm_rope_append(C.byref(qp), C.byref(batch.desc), C.byref(pool.desc), None))


def test_attention_decode_16_sequences_up_to_32768():
    """The decode step of a 16-sequence ragged batch, 24 q / 4 kv heads, contexts log-uniform in 128..32768 (seed 3)
    with the longest forced to 32768, page ids from a seeded shuffle."""
    nq, nkv, layer = 24, 4, 0
    ld = 2 * nq * 256 + 2 * nkv * 256
    r3 = np.random.default_rng(3)
    ctx = [int(round(np.exp(u))) for u in r3.uniform(np.log(128), np.log(32768), size=16)]
    ctx[5] = 32768
    qn = (1 + 0.2 * r3.standard_normal(256)).astype(np.float32)
    kn = (1 + 0.2 * r3.standard_normal(256)).astype(np.float32)
    qn_dev, kn_dev = torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda()
    need = [(c + 63) // 64 for c in ctx]
    pool = tl.KvPool(nkv, layers=1, num_pages=sum(need) + 5, slots=16, max_pages_per_seq=max(need), dtype=0)
    perm = np.random.default_rng(5).permutation(sum(need) + 5).astype(np.int32)
    used = 0
    for s, pages in enumerate(need):
        pool.table[s, :pages] = torch.from_numpy(perm[used:used + pages]).cuda()
        used += pages
    gen = torch.Generator(device="cuda").manual_seed(33)
    for s, c in enumerate(ctx):
        fill_kv_random(pool, layer, nq, nkv, s, c - 1, qn_dev, kn_dev, gen)
    proj = tl.bf16_round(np.random.default_rng(34).standard_normal((16, ld)))
    batch = tl.Batch([(s, c - 1, 1) for s, c in enumerate(ctx)])
    q_got, out_got = run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode=True, split_rows=64)
    o = tl.oracle()
    for s, c in enumerate(ctx):
        kd, vd = pool.read_sequence(layer, s, c)
        seen = tl.OracleKv(o, nkv, c)
        seen.k[:], seen.v[:] = kd, vd
        want = seen.attend(nq, q_got[s], proj[s, nq * 256:2 * nq * 256], c - 1)
        assert np.all(np.abs(out_got[s] - want) <= 2e-2 * (np.abs(want) + 0.02 * np.abs(want).max())), (s, c)


@pytest.mark.parametrize("dtype", [0, 1], ids=["int8", "bf16"])
@pytest.mark.parametrize("nq,nkv,split_rows", [(24, 4, 4), (3, 1, 800)])
def test_attention_prefill_ragged_chunks_at_long_prefixes(nq, nkv, split_rows, dtype):
    """One ragged prefill step of three sequences: a 512-token chunk behind an 8,200-token prefix, a 200-token chunk
    behind 300 tokens and a 65-token chunk at position 0 (query tiles that start inside a page, end inside a page and
    span pages). 24 q / 4 kv heads is the 27B layer (ten tokens x six heads per tile); 3 q / 1 kv head is one rank of
    the 8-way tensor-parallel layout, where the few tiles cut their keys over several CTAs and the merge kernel
    finishes (the scratch is sized per token for it). Both cache types: int8 pages come through the raw ring, bf16 pages
    by plain loads into the same fp16 tiles. The oracle attends over the cache as the kernel wrote it, on a
    sample of the prompt tokens (every position of the short chunks, every 29th and the ends of the long one)."""
    ld = 2 * nq * 256 + 2 * nkv * 256
    r3 = np.random.default_rng(3)
    qn = (1 + 0.2 * r3.standard_normal(256)).astype(np.float32)
    kn = (1 + 0.2 * r3.standard_normal(256)).astype(np.float32)
    qn_dev, kn_dev = torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda()
    prefix, chunk, slots, layer = [8200, 300, 0], [512, 200, 65], [2, 0, 1], 1
    need = [(a + c + 63) // 64 for a, c in zip(prefix, chunk)]
    pool = tl.KvPool(nkv, layers=2, num_pages=sum(need) + 3, slots=3, max_pages_per_seq=max(need), dtype=dtype)
    perm = np.random.default_rng(5).permutation(sum(need) + 3).astype(np.int32)
    used = 0
    for s, pages in zip(slots, need):
        pool.table[s, :pages] = torch.from_numpy(perm[used:used + pages]).cuda()
        used += pages
    gen = torch.Generator(device="cuda").manual_seed(44)
    for s, a in zip(slots, prefix):
        fill_kv_random(pool, layer, nq, nkv, s, a, qn_dev, kn_dev, gen)
    n = sum(chunk)
    proj = tl.bf16_round(np.random.default_rng(45).standard_normal((n, ld)))
    batch = tl.Batch([(s, a, c) for s, a, c in zip(slots, prefix, chunk)])
    q_got, out_got = run_attention_chunk(pool, layer, nq, nkv, proj, batch, qn_dev, kn_dev, decode=False,
                                         split_rows=split_rows)
    o = tl.oracle()
    row0 = 0
    got_rows, want_rows, where = [], [], []
    for s, a, c in zip(slots, prefix, chunk):
        kd, vd = pool.read_sequence(layer, s, a + c)
        picks = sorted(set(range(c)) if c <= 200 else set(range(0, c, 29)) | {1, 63, 64, c - 2, c - 1})
        for i in picks:
            pos = a + i
            seen = tl.OracleKv(o, nkv, pos + 1)
            seen.k[:], seen.v[:] = kd[:, :pos + 1], vd[:, :pos + 1]
            want_rows.append(seen.attend(nq, q_got[row0 + i], proj[row0 + i, nq * 256:2 * nq * 256], pos))
            got_rows.append(out_got[row0 + i])
            where.append((s, i, pos))
        row0 += c
    # the reference's bound (tests/gpu/test_kernels.cu:486-492): |got - want| <= 2e-2 (|want| + 0.02 max|want|) with the
    # maximum taken over the whole run
    got, want = np.stack(got_rows), np.stack(want_rows)
    bad = np.abs(got - want) > 2e-2 * (np.abs(want) + 0.02 * np.abs(want).max())
    assert not bad.any(), [where[r] for r in np.nonzero(bad.any(axis=1))[0][:5]]


# ---------------------------------------------------------------------------------------------------
# Gated DeltaNet
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("nk,nv,H", [(2, 6, 512), (2, 2, 512), (16, 32, 5120), (16, 48, 5120)])
def test_gdn_matches_oracle(nk, nv, H, chunked):
    """Chunk lengths {37, 64, 1, 1, 100, 1, 17, 300} on slot 1 of 3, GDN layer 1 of 2; a second sequence runs in
    the same ragged batch on slot 2 with its own lengths. Head counts: small ones, 16 key / 32 value heads (value
    heads share a key head in pairs) and the 27B model's 16 / 48 at its hidden size 5120."""
    rng = np.random.default_rng(5)
    o = tl.oracle()
    conv_dim = 2 * nk * 128 + nv * 128
    ld = conv_dim + nv * 128
    layers, layer, slots = 2, 1, 3
    w_ab = tl.bf16_round(rng.standard_normal((2 * nv, H)) / np.sqrt(H))
    conv_w = (0.4 * rng.standard_normal((conv_dim, 4))).astype(np.float32)
    A = (-rng.uniform(0.5, 8, nv)).astype(np.float32)
    dt = (0.5 * rng.standard_normal(nv)).astype(np.float32)
    nw = (1 + 0.2 * rng.standard_normal(128)).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    w_ab_d, conv_w_d, A_d, dt_d, nw_d = tl.to_dev_bf16(w_ab), dev(conv_w), dev(A), dev(dt), dev(nw)
    rec = torch.zeros((slots, layers, nv, 128, 128), dtype=torch.float32, device="cuda")
    conv = torch.zeros((slots, layers, 3, conv_dim), dtype=torch.bfloat16, device="cuda")
    st = pkg.GdnStateDesc(pkg.ptr(rec), pkg.ptr(conv), layers)
    dims = pkg.GdnDims(nk, nv, conv_dim, ld)
    ref_state = {1: (np.zeros(nv * 128 * 128, np.float32), np.zeros(3 * conv_dim, np.float32)),
                 2: (np.zeros(nv * 128 * 128, np.float32), np.zeros(3 * conv_dim, np.float32))}
    pos = {1: 0, 2: 0}
    for n1, n2 in zip((37, 64, 1, 1, 100, 1, 17, 300), (1, 2, 3, 70, 1, 1, 1, 129)):
        seqs = [(1, pos[1], n1), (2, pos[2], n2)]
        batch = tl.Batch(seqs)
        n = n1 + n2
        proj = tl.bf16_round(rng.standard_normal((n, ld)))
        x = tl.bf16_round(rng.standard_normal((n, H)))
        partials = np.stack([o.norm_partials(x[i]) for i in range(n)])
        ab = torch.empty((n, 2 * nv), dtype=torch.float32, device="cuda")
        qkv = torch.empty((n, conv_dim), dtype=torch.float32, device="cuda")
        out = torch.empty((n, nv * 128), dtype=torch.bfloat16, device="cuda")
        proj_d = tl.to_dev_bf16(proj)
        x_d, part_d = tl.to_dev_bf16(x), dev(partials)
        pkg.check(K().q38_gdn_ab(pkg.ptr(x_d), n, H, pkg.ptr(w_ab_d), 2 * nv, pkg.ptr(part_d), 1e-6, pkg.ptr(ab), None))
        cp = pkg.GdnConvParams(pkg.ptr(proj_d), pkg.ptr(conv_w_d), pkg.ptr(qkv), layer)
        pkg.check(K().q38_gdn_conv(C.byref(cp), C.byref(dims), C.byref(batch.desc), C.byref(st), None))
        rp = pkg.GdnRecurrenceParams(pkg.ptr(qkv), pkg.ptr(ab), pkg.ptr(A_d), pkg.ptr(dt_d), pkg.ptr(proj_d) + conv_dim * 2,
                                     ld, pkg.ptr(nw_d), 1e-6, pkg.ptr(out), layer)
        if chunked:  # the 64-token chunked form, also for the short runs (they are padded to a chunk)
            need = K().q38_gdn_chunk_scratch_floats(n, len(seqs), nv)
            scratch = torch.empty(need, dtype=torch.float32, device="cuda")
            pkg.check(K().q38_gdn_recurrence_chunked(C.byref(rp), C.byref(dims), C.byref(batch.desc), C.byref(st),
                                                     pkg.ptr(scratch), need, None))
        else:
            pkg.check(K().q38_gdn_recurrence(C.byref(rp), C.byref(dims), C.byref(batch.desc), C.byref(st), None))
        sync_ok()
        ab_got = ab.cpu().numpy()
        rs = np.array([o.norm_row_scale(partials[i], H, 1e-6) for i in range(n)], np.float32)
        ab_ref = np.zeros((n, 2 * nv), np.float32)
        o.qgemm(x, w_ab, rs, 3, out=ab_ref, ldo=2 * nv)
        assert np.all(np.abs(ab_got - ab_ref) <= 1e-3 + 1e-3 * np.abs(ab_ref))
        got = out.float().cpu().numpy()
        row = 0
        for slot, _, cnt in seqs:
            s, cs = ref_state[slot]
            for i in range(cnt):
                want = o.gdn_token(nk, nv, 1e-6, proj[row], ab_got[row], conv_w, A, dt, nw, s, cs)
                assert np.all(np.abs(got[row] - want) <= 2e-2 * (np.abs(want) + 0.05)), (slot, pos[slot] + i)
                row += 1
            pos[slot] += cnt
    for slot in (1, 2):
        s_got = rec[slot, layer].cpu().numpy().reshape(-1)
        assert np.all(np.abs(s_got - ref_state[slot][0]) <= 1e-3 + 1e-2 * np.abs(ref_state[slot][0]))
        c_got = conv[slot, layer].float().cpu().numpy().reshape(-1)
        assert np.array_equal(c_got, ref_state[slot][1])
    assert float(rec[0].abs().sum()) == 0 and float(rec[:, 0].abs().sum()) == 0, "other slots / layers untouched"


@pytest.mark.parametrize("tensor_cores", [0, 1])
@pytest.mark.parametrize("seqs", [2, 30])
def test_gdn_chunked_matches_sequential_kernel(seqs, tensor_cores):
    """The chunked form against the token-sequential kernel on the same inputs: few (head, sequence) pairs take the
    two-CTAs-per-head scan with the separate norm kernel, many take the one-CTA scan. Both forms of the scan's products
    (fp32 on the CUDA cores; split-TF32, three MMAs per product, on the tensor cores) must agree with the sequential
    kernel to fp32-like rounding."""
    K().q38_gdn_set_chunk_scan_tensor_cores(tensor_cores)
    rng = np.random.default_rng(31)
    nk, nv, layers, layer = 2, 6, 1, 0
    conv_dim = 2 * nk * 128 + nv * 128
    ld = conv_dim + nv * 128
    lens = [int(x) for x in rng.integers(1, 150, size=seqs)]
    n = sum(lens)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    A_d = dev((-rng.uniform(0.5, 8, nv)).astype(np.float32))
    dt_d = dev((0.5 * rng.standard_normal(nv)).astype(np.float32))
    nw_d = dev((1 + 0.2 * rng.standard_normal(128)).astype(np.float32))
    qkv_np = rng.standard_normal((n, conv_dim)).astype(np.float32)
    for h in range(2 * nk):  # q and k heads normalised as the conv kernel leaves them
        blk = qkv_np[:, h * 128:(h + 1) * 128]
        blk /= np.sqrt((blk * blk).sum(axis=1, keepdims=True) + 1e-6)
    qkv = dev(qkv_np)
    ab = dev(rng.standard_normal((n, 2 * nv)).astype(np.float32))
    proj_d = tl.to_dev_bf16(tl.bf16_round(rng.standard_normal((n, ld))))
    rec0 = dev((0.1 * rng.standard_normal((seqs, layers, nv, 128, 128))).astype(np.float32))
    batch = tl.Batch([(b, 0, lens[b]) for b in range(seqs)])
    dims = pkg.GdnDims(nk, nv, conv_dim, ld)
    res = []
    for chunked in (False, True):
        rec = rec0.clone()
        conv = torch.zeros((seqs, layers, 3, conv_dim), dtype=torch.bfloat16, device="cuda")
        st = pkg.GdnStateDesc(pkg.ptr(rec), pkg.ptr(conv), layers)
        out = torch.zeros((n, nv * 128), dtype=torch.bfloat16, device="cuda")
        rp = pkg.GdnRecurrenceParams(pkg.ptr(qkv), pkg.ptr(ab), pkg.ptr(A_d), pkg.ptr(dt_d), pkg.ptr(proj_d) + conv_dim * 2,
                                     ld, pkg.ptr(nw_d), 1e-6, pkg.ptr(out), layer)
        if chunked:
            need = K().q38_gdn_chunk_scratch_floats(n, seqs, nv)
            scratch = torch.empty(need, dtype=torch.float32, device="cuda")
            pkg.check(K().q38_gdn_recurrence_chunked(C.byref(rp), C.byref(dims), C.byref(batch.desc), C.byref(st),
                                                     pkg.ptr(scratch), need, None))
        else:
            pkg.check(K().q38_gdn_recurrence(C.byref(rp), C.byref(dims), C.byref(batch.desc), C.byref(st), None))
        sync_ok()
        res.append((out.float().cpu().numpy(), rec.cpu().numpy()))
    K().q38_gdn_set_chunk_scan_tensor_cores(1)
    (o_seq, s_seq), (o_chk, s_chk) = res
    assert np.all(np.abs(o_chk - o_seq) <= 2e-2 * (np.abs(o_seq) + 0.05))
    err = np.abs(s_chk - s_seq)
    assert np.all(err <= 1e-4 + 1e-3 * np.abs(s_seq)), float((err / (1e-4 + 1e-3 * np.abs(s_seq))).max())


def test_gdn_decode_kernel_equals_general_kernel():
    """Batches in which every sequence advances by one token take the persistent state-streaming kernel; it must
    reproduce the general kernel bit for bit (outputs and states), also with an empty sequence in the batch and
    with more (sequence, head) items than SMs."""
    rng = np.random.default_rng(21)
    nk, nv, layers, layer, slots = 2, 4, 2, 1, 70
    conv_dim = 2 * nk * 128 + nv * 128
    ld = conv_dim + nv * 128
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    A_d = dev((-rng.uniform(0.5, 8, nv)).astype(np.float32))
    dt_d = dev((0.5 * rng.standard_normal(nv)).astype(np.float32))
    nw_d = dev((1 + 0.2 * rng.standard_normal(128)).astype(np.float32))
    rec0 = torch.from_numpy(rng.standard_normal((slots, layers, nv, 128, 128)).astype(np.float32) * 0.1).cuda()
    seqs = [(slot, 5, 0 if slot == 17 else 1) for slot in range(2, 66)]
    n = sum(c for _, _, c in seqs)
    dims = pkg.GdnDims(nk, nv, conv_dim, ld)
    results = []
    for force_general in (False, True):
        rec = rec0.clone()
        conv = torch.zeros((slots, layers, 3, conv_dim), dtype=torch.bfloat16, device="cuda")
        st = pkg.GdnStateDesc(pkg.ptr(rec), pkg.ptr(conv), layers)
        outs = []
        step_rng = np.random.default_rng(22)
        for step in range(3):
            batch = tl.Batch(seqs)
            if force_general:
                batch.desc.max_tokens_per_seq = 2
            qkv = dev(step_rng.standard_normal((n, conv_dim)).astype(np.float32) * 0.3)
            ab = dev(step_rng.standard_normal((n, 2 * nv)).astype(np.float32))
            proj_d = tl.to_dev_bf16(tl.bf16_round(step_rng.standard_normal((n, ld))))
            out = torch.zeros((n, nv * 128), dtype=torch.bfloat16, device="cuda")
            rp = pkg.GdnRecurrenceParams(pkg.ptr(qkv), pkg.ptr(ab), pkg.ptr(A_d), pkg.ptr(dt_d),
                                         pkg.ptr(proj_d) + conv_dim * 2, ld, pkg.ptr(nw_d), 1e-6, pkg.ptr(out), layer)
            pkg.check(K().q38_gdn_recurrence(C.byref(rp), C.byref(dims), C.byref(batch.desc), C.byref(st), None))
            sync_ok()
            outs.append(out.view(torch.int16).cpu().numpy())
        results.append((outs, rec.cpu().numpy()))
    for a, b in zip(results[0][0], results[1][0]):
        assert np.array_equal(a, b)
    assert np.array_equal(results[0][1], results[1][1])
    assert np.array_equal(results[0][1][17], rec0[17].cpu().numpy()), "the empty sequence's state is untouched"
    assert not np.array_equal(results[0][1][2, layer], rec0[2, layer].cpu().numpy())


# ---------------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------------
def run_sampler(logits, params, step, history=None, hist_len=None, cap=16):
    B, V = logits.shape
    lg = torch.from_numpy(logits.copy()).cuda()
    prm = (pkg.SamplingParamsDev * B)(*params)
    prm_dev = torch.frombuffer(bytearray(bytes(prm)), dtype=torch.uint8).cuda()
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    steps = torch.full((B,), step, dtype=torch.int32, device="cuda")
    hl = torch.zeros(B, dtype=torch.int32, device="cuda") if hist_len is None else torch.tensor(hist_len, dtype=torch.int32, device="cuda")
    hist = torch.zeros((B, cap), dtype=torch.int32, device="cuda") if history is None else torch.tensor(history, dtype=torch.int32, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    lp = torch.empty(B, dtype=torch.float32, device="cuda")
    a = pkg.SamplingArgs(pkg.ptr(lg), V, V, pkg.ptr(prm_dev), pkg.ptr(slot), pkg.ptr(hist), pkg.ptr(hl), cap,
                         pkg.ptr(steps), pkg.ptr(out), pkg.ptr(lp))
    pkg.check(K().q38_sample(C.byref(a), B, None))
    torch.cuda.synchronize()
    return out.cpu().numpy(), lp.cpu().numpy(), lg.cpu().numpy(), hl.cpu().numpy(), hist.cpu().numpy()


def P(t=0.0, k=0, p=1.0, minp=0.0, pres=0.0, rep=1.0, seed=1):
    return pkg.SamplingParamsDev(t, k, p, minp, pres, rep, seed)


def test_sampling_filters_and_determinism():
    V, B = 248320, 4
    rng = np.random.default_rng(9)
    logits = (2.0 * rng.standard_normal((B, V))).astype(np.float32)
    logits[3] = -1e4
    toks, lps = [10, 20, 30, 40, 50], [0.0, -0.5, -1.0, -2.0, -8.0]
    for t, l in zip(toks, lps):
        logits[3, t] = l
    logits[1, 77] = logits[1].max() + 1.0
    logits[1, 50000] = logits[1, 77]  # a tie: the lowest id wins
    argmax = logits.argmax(axis=1)
    assert argmax[1] == 77
    got, lp, _, hl, hist = run_sampler(logits, [P()] * B, 0)
    assert np.array_equal(got, argmax) and np.all(lp == 0.0)
    assert np.all(hl == 1) and np.array_equal(hist[:, 0], argmax), "the sampled token is appended to the history"
    got, *_ = run_sampler(logits, [P(t=1.0, k=1)] * B, 0)
    assert np.array_equal(got, argmax)
    # top-p 0.9 on row 3: nucleus {10, 20, 30}
    counts, trials = {}, 1500
    for s in range(trials):
        t = int(run_sampler(logits, [P(t=1.0, p=0.9, seed=1234)] * B, s)[0][3])
        counts[t] = counts.get(t, 0) + 1
    assert set(counts) <= {10, 20, 30}
    z = sum(np.exp(l) for l in lps[:3])
    for t, l in zip(toks[:3], lps[:3]):
        expect = np.exp(l) / z * trials
        assert abs(counts.get(t, 0) - expect) < 5 * np.sqrt(expect)
    for s in range(200):  # min_p 0.3 keeps logits >= log 0.3
        assert int(run_sampler(logits, [P(t=1.0, minp=0.3, seed=99)] * B, s)[0][3]) in (10, 20, 30)
    a = run_sampler(logits, [P(t=0.8, k=50, p=0.95, seed=777)] * B, 5)[0]
    b = run_sampler(logits, [P(t=0.8, k=50, p=0.95, seed=777)] * B, 5)[0]
    assert np.array_equal(a, b)
    # penalties: each distinct history token is penalised once
    history = np.zeros((B, 16), np.int32)
    history[0, :3] = [argmax[0], argmax[0], 5]
    _, _, lg_after, _, _ = run_sampler(logits, [P(pres=0.5, rep=2.0)] * B, 0, history=history.tolist(), hist_len=[3, 0, 0, 0])
    l0 = logits[0, argmax[0]]
    assert np.isclose(lg_after[0, argmax[0]], (l0 / 2.0 if l0 > 0 else l0 * 2.0) - 0.5)
    l5 = logits[0, 5]
    assert np.isclose(lg_after[0, 5], (l5 / 2.0 if l5 > 0 else l5 * 2.0) - 0.5)


def test_sampler_draws_equal_the_cpu_restatement():
    """The stochastic sampler against its CPU restatement (oracle/q38_oracle.cpp): sampled token ids must be
    identical, draw for draw, on the 27B vocabulary (248,320 logits) for top-k, top-p, min-p, their combinations and
    penalties: 10,240 draws = 10 parameter sets x 4 logit rows x 256 (seed, step) pairs. Both sides compute the
    fixed-point masses and thresholds with the same IEEE operations, so there is no tolerance on the ids; the reported
    log-probability goes through a library log and is compared to 1e-5."""
    V, D = 248320, 256
    rng = np.random.default_rng(90)
    o = tl.oracle()
    rows = [(2.0 * rng.standard_normal(V)).astype(np.float32),            # flat: thousands of candidates
            (6.0 * rng.standard_normal(V)).astype(np.float32),            # peaked
            np.round(3.0 * rng.standard_normal(V)).astype(np.float32),    # heavy ties (integer logits)
            (0.02 * rng.standard_normal(V)).astype(np.float32) * 70.0]    # the range of a random-weight model
    psets = [dict(t=1.0, k=50), dict(t=0.7, k=0, p=0.9), dict(t=1.3, minp=0.05), dict(t=0.8, k=20, p=0.95),
             dict(t=1.0, k=1000, p=0.5, minp=0.001), dict(t=0.6), dict(t=2.5, p=0.99), dict(t=1.0, k=40, pres=0.7, rep=1.3),
             dict(t=0.9, p=0.8, pres=-0.5, rep=0.8), dict(t=1.0, k=5, minp=0.2, rep=2.0)]
    cap = 64
    mism = 0
    for pi, ps in enumerate(psets):
        for ri, row in enumerate(rows):
            seeds = rng.integers(1, 2 ** 63, size=D, dtype=np.uint64)
            steps = rng.integers(0, 5000, size=D).astype(np.int32)
            order = np.argsort(row)
            hist = np.concatenate([order[-20:], order[-5:], rng.integers(0, V, size=cap - 25)]).astype(np.int32)
            assert hist.shape == (cap,)  # the kernel addresses history rows of exactly `cap` entries
            use_hist = ("pres" in ps) or ("rep" in ps)
            prm = [P(t=ps["t"], k=ps.get("k", 0), p=ps.get("p", 1.0), minp=ps.get("minp", 0.0), pres=ps.get("pres", 0.0),
                     rep=ps.get("rep", 1.0), seed=int(sd)) for sd in seeds]
            lg = torch.from_numpy(row).cuda().repeat(D, 1).contiguous()
            prm_dev = torch.frombuffer(bytearray(bytes((pkg.SamplingParamsDev * D)(*prm))), dtype=torch.uint8).cuda()
            slot = torch.arange(D, dtype=torch.int32, device="cuda")
            steps_d = torch.from_numpy(steps).cuda()
            hl = torch.full((D,), len(hist) if use_hist else 0, dtype=torch.int32, device="cuda")
            hist_d = torch.from_numpy(np.tile(hist, (D, 1))).cuda().contiguous()
            out = torch.full((D,), -1, dtype=torch.int32, device="cuda")
            lp = torch.empty(D, dtype=torch.float32, device="cuda")
            a = pkg.SamplingArgs(pkg.ptr(lg), V, V, pkg.ptr(prm_dev), pkg.ptr(slot), pkg.ptr(hist_d), pkg.ptr(hl), cap,
                                 pkg.ptr(steps_d), pkg.ptr(out), pkg.ptr(lp))
            pkg.check(K().q38_sample(C.byref(a), D, None))
            sync_ok()
            pen = o.sample_penalties(row, hist if use_hist else [], ps.get("pres", 0.0), ps.get("rep", 1.0), cap)
            assert np.array_equal(lg[0].cpu().numpy(), pen), "penalised logits differ"
            want, want_lp = o.sample_draws(pen, ps["t"], ps.get("k", 0), ps.get("p", 1.0), ps.get("minp", 0.0), seeds, steps)
            got = out.cpu().numpy()
            mism += int((got != want).sum())
            assert np.array_equal(got, want), (pi, ri, int((got != want).sum()), got[:8], want[:8])
            assert np.allclose(lp.cpu().numpy(), want_lp, atol=1e-5, rtol=1e-5), (pi, ri)
            assert len(np.unique(got)) > 1 or ps.get("k", 0) == 1
    assert mism == 0


def test_target_logprobs_matches_oracle():
    rng = np.random.default_rng(2)
    V, rows = 4096, 5
    logits = (3 * rng.standard_normal((rows, V))).astype(np.float32)
    targets = rng.integers(0, V, size=rows).astype(np.int32)
    out = torch.empty(rows, dtype=torch.float32, device="cuda")
    lg_d, tg_d = torch.from_numpy(logits).cuda(), torch.from_numpy(targets).cuda()
    pkg.check(K().q38_target_logprobs(pkg.ptr(lg_d), V, V, pkg.ptr(tg_d), rows, pkg.ptr(out), None))
    torch.cuda.synchronize()
    lib = tl.oracle().fn("target_logprob", C.c_float)
    want = [lib(logits[i].ctypes.data_as(C.c_void_p), C.c_int(V), C.c_int(int(targets[i]))) for i in range(rows)]
    assert np.allclose(out.cpu().numpy(), np.array(want, np.float32), atol=1e-5)


def test_launchers_reject_bad_arguments_without_launching():
    p = tl.make_bq(128, 64, 4, seed=1, fast=True)
    w = tl.DeviceBQ(p)
    a = torch.zeros((1, 64), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((1, 128), dtype=torch.float32, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_STORE_F32, pkg.ptr(out), 128, 0, None, None, None, None, 0, 1e-6)
    assert K().q38_qgemm(pkg.ptr(a), 0, C.byref(w.desc), C.byref(ep), None, None, -1) == -1
    assert b"m must be positive" in K().q38_last_error()
    bad = pkg.BQWeight(w.desc.lo, None, w.desc.scales, 7, 128, 64, 128)
    assert K().q38_qgemm(pkg.ptr(a), 1, C.byref(bad), C.byref(ep), None, None, -1) == -1
    assert K().q38_embed(None, None, 0, 128, None, None, None, None) == 0  # m == 0 is a no-op
    # the all-reduce epilogue: its peer description is required, it serves up to 16 tokens, and only the streaming kernel
    res = torch.zeros((32, 128), dtype=torch.float32, device="cuda")
    xbf = torch.zeros((32, 128), dtype=torch.bfloat16, device="cuda")
    part = torch.zeros((32, 1), dtype=torch.float32, device="cuda")
    ep = pkg.GemmEpilogue(pkg.EPI_ALLREDUCE_RESIDUAL, None, 0, 0, pkg.ptr(res), pkg.ptr(xbf), pkg.ptr(part), None, 0, 1e-6)
    assert K().q38_qgemm(pkg.ptr(a), 1, C.byref(w.desc), C.byref(ep), None, None, -1) == -1
    assert b"peer description" in K().q38_last_error()
    ar = pkg.PeerAllreduce()
    ar.world, ar.rank = 1, 0
    buf = torch.zeros(2 * 16 * 128, dtype=torch.float32, device="cuda")
    words = torch.zeros(8, dtype=torch.int32, device="cuda")
    ar.recv[0], ar.flags[0], ar.seq = pkg.ptr(buf), pkg.ptr(words), pkg.ptr(words) + 16
    ep = pkg.GemmEpilogue(pkg.EPI_ALLREDUCE_RESIDUAL, None, 0, 0, pkg.ptr(res), pkg.ptr(xbf), pkg.ptr(part), None, 0, 1e-6,
                          C.pointer(ar))
    a32 = torch.zeros((32, 64), dtype=torch.bfloat16, device="cuda")
    assert K().q38_qgemm(pkg.ptr(a32), 17, C.byref(w.desc), C.byref(ep), None, None, -1) == -1
    assert b"up to 16 tokens" in K().q38_last_error()
    names = {K().q38_qgemm_config_name(c).decode(): c for c in range(K().q38_qgemm_num_configs())}
    assert K().q38_qgemm(pkg.ptr(a32), 8, C.byref(w.desc), C.byref(ep), None, None, names["tmem_t32"]) == -1
    assert b"streaming kernel only" in K().q38_last_error()
    ar.world = 9
    assert K().q38_qgemm(pkg.ptr(a), 1, C.byref(w.desc), C.byref(ep), None, None, -1) == -1
