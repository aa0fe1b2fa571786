"""Models of two hand-shake protocols of the kernels, run under random schedules on the CPU.

These do not execute the kernels: they restate, role by role, which barrier each role of a kernel waits for and which
it arrives on (with the parity arithmetic of the source), and let a scheduler interleave the roles at random. They
exist because that is how a race in the tcgen05 GEMM was found that the GPU only showed as a bounded wait giving up:
a decode warp without work in a partial last stage released the raw stage without waiting for it, and with a
two-stage ring its arrival could complete the previous use of the stage. The negative controls below keep the models
honest: the old behaviour must still fail in them.

  * qgemm_umma_kernel (weights-in-TMEM variant, two k-groups per unit): raw ring, operand ring, one or two issuing
    warps, accumulator hand-over; source csrc/qgemm_umma.cu.
  * Q38_EPI_ALLREDUCE_RESIDUAL (csrc/qgemm_stream.cu): push to every rank's buffer, per-source flags, pull; two
    receive buffers used in turn.
"""

import random

import pytest


# ----------------------------------------------------------------------------------------------------
# mbarrier with parity waits
# ----------------------------------------------------------------------------------------------------
class Bar:
    def __init__(self, count, log):
        self.count, self.pending, self.phase, self.log = count, count, 0, log

    def arrive(self):
        self.log[0] += 1
        self.pending -= 1
        if self.pending == 0:
            self.pending = self.count
            self.phase += 1

    def ready(self, parity):  # try_wait.parity: the phase of that parity has completed
        return (self.phase & 1) != parity


def u_begin(cta, grid, tiles, kg, split):
    return cta * tiles * kg // grid if split else (cta * tiles // grid) * kg


def gemm_roles_finish(cta, tiles, kg, grid, split, units, issuers, stages, wait_before_release, seed):
    """True when every role of one CTA runs to completion under a random schedule; False when no role can move."""
    log = [0]
    u0, u1 = u_begin(cta, grid, tiles, kg, split), u_begin(cta + 1, grid, tiles, kg, split)
    op_full = [Bar(4 + 1, log) for _ in range(units)]   # four decode warps + the activation copy's arrival
    op_empty = [Bar(1, log) for _ in range(units)]
    acc_full, acc_empty = Bar(issuers, log), Bar(16, log)
    raw_full = [Bar(1, log) for _ in range(stages)]
    raw_empty = [Bar(8, log) for _ in range(stages)]

    def segments():
        u = u0
        while u < u1:
            a = u % kg
            b = min(kg, a + (u1 - u))
            yield a, b
            u += b - a

    def raw_producer():
        it = 0
        for a, b in segments():
            for _ in range(a, b, 4):
                s = it % stages
                while not raw_empty[s].ready(((it // stages) & 1) ^ 1):
                    yield
                raw_full[s].arrive()
                it += 1

    def activation_producer():
        uc = 0
        for a, b in segments():
            for _ in range(a, b, 2):
                slot = uc % units
                while not op_empty[slot].ready(((uc // units) & 1) ^ 1):
                    yield
                op_full[slot].arrive()
                uc += 1

    def issuer(iss):
        seg = uc0 = 0
        for a, b in segments():
            n = (b - a + 1) // 2
            while not acc_empty.ready((seg & 1) ^ 1):
                yield
            i = ((iss - uc0) & 1) if issuers == 2 else 0
            slot, par = (uc0 + i) % units, ((uc0 + i) // units) & 1
            while i < n:
                while not op_full[slot].ready(par):
                    yield
                op_empty[slot].arrive()  # the commit of the unit's MMAs
                slot += issuers
                if slot >= units:
                    slot -= units
                    par ^= 1
                i += issuers
            acc_full.arrive()
            uc0 += n
            seg += 1

    def decode_warp(dw):
        seg = stage_no = s = s_par = u_slot = u_par = 0
        group, ui = dw >> 3, (dw >> 2) & 1
        for a, b in segments():
            nst = (b - a + 3) // 4
            j0 = (group - stage_no) & 1
            ws, ws_par = s + j0, s_par
            if ws >= stages:
                ws, ws_par = ws - stages, ws_par ^ 1
            slot, par = u_slot + 2 * j0 + ui, u_par
            if slot >= units:
                slot, par = slot - units, par ^ 1
            for j in range(j0, nst, 2):
                ng = min(4, b - a - 4 * j)
                has_unit = ui * 2 < ng
                if wait_before_release or has_unit:
                    while not raw_full[ws].ready(ws_par):
                        yield
                if has_unit:
                    while not op_empty[slot].ready(par ^ 1):
                        yield
                    op_full[slot].arrive()
                raw_empty[ws].arrive()
                ws += 2
                if ws >= stages:
                    ws, ws_par = ws - stages, ws_par ^ 1
                slot += 4
                if slot >= units:
                    slot, par = slot - units, par ^ 1
            nun = (b - a + 1) // 2
            sn, un = s + nst, u_slot + nun
            s_par ^= (sn // stages) & 1
            s = sn % stages
            u_par ^= (un // units) & 1
            u_slot = un % units
            stage_no += nst
            while not acc_full.ready(seg & 1):
                yield
            acc_empty.arrive()
            seg += 1

    roles = [raw_producer(), activation_producer()] + [issuer(i) for i in range(issuers)] + [decode_warp(d) for d in range(16)]
    live = set(range(len(roles)))
    rng = random.Random(seed)
    while live:
        before = log[0]
        order = list(live)
        rng.shuffle(order)
        for r in order:
            try:
                next(roles[r])  # runs the role until its next unsatisfied wait
            except StopIteration:
                live.discard(r)
        if live and log[0] == before:
            return False  # a whole round without one arrival: nobody can move any more
    return True


GEMM_CASES = [  # tiles, k-groups per tile, even cut, operand units, issuers, raw stages
    (600, 80, 1, 6, 2, 2),    # 8-bit weights: two raw stages; even cut over all SMs
    (1940, 80, 1, 6, 2, 2),   # LM head
    (600, 77, 1, 6, 2, 6),    # a k extent that leaves partial stages of every size
    (600, 77, 1, 4, 2, 4),
    (272, 80, 0, 6, 2, 6),    # whole tiles (gate/up)
    (40, 272, 1, 6, 2, 6),    # split inside tiles (down projection)
    (600, 80, 1, 6, 1, 2),    # one issuer
]


@pytest.mark.parametrize("tiles,kg,split,units,issuers,stages", GEMM_CASES)
def test_gemm_ring_protocol_completes_under_random_schedules(tiles, kg, split, units, issuers, stages):
    for cta in (0, 1, 3, 5, 45, 63, 147):
        for seed in range(3):
            assert gemm_roles_finish(cta, tiles, kg, 148, split, units, issuers, stages, True, seed), (cta, seed)


def test_gemm_ring_model_catches_the_release_without_wait():
    """Negative control: a warp that releases a raw stage it did not wait for lets the producer run a turn ahead; with
    two raw stages some schedule of some CTA ends with waits that can never be satisfied."""
    stuck = sum(not gemm_roles_finish(cta, 600, 80, 148, 1, 6, issuers, 2, False, seed)
                for cta in range(0, 12) for seed in range(3) for issuers in (1, 2))
    assert stuck > 0


# ----------------------------------------------------------------------------------------------------
# all-reduce inside the row-parallel GEMM: push, flags, pull, two buffers in turn
# ----------------------------------------------------------------------------------------------------
def allreduce_reads_are_consistent(world, calls, buffers, seed):
    """Every rank pushes (source, call) tags into slot [call % buffers][source] of every rank, raises its flag there to
    the call number, waits for all flags in its own memory, then reads the slots one at a time. True when every read
    returns the tag of the current call."""
    recv = [[[None] * world for _ in range(buffers)] for _ in range(world)]  # [rank][buffer][source]
    flags = [[0] * world for _ in range(world)]                              # [rank][source]
    ok = [True]

    def rank(r):
        for call in range(1, calls + 1):
            buf = call % buffers
            for p in range(world):
                recv[p][buf][r] = call
                yield
            for p in range(world):
                flags[p][r] = call
                yield
            while any(flags[r][src] < call for src in range(world)):
                yield
            for src in range(world):
                if recv[r][buf][src] != call:
                    ok[0] = False
                yield

    progs = [rank(r) for r in range(world)]
    live = set(range(world))
    rng = random.Random(seed)
    while live:
        r = rng.choice(sorted(live))
        for _ in range(rng.randint(1, 12)):  # a rank runs in bursts, so that it can get ahead of the others
            try:
                next(progs[r])
            except StopIteration:
                live.discard(r)
                break
    return ok[0]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_two_buffers_are_enough(world):
    for seed in range(40):
        assert allreduce_reads_are_consistent(world, calls=12, buffers=2, seed=seed), seed


def test_allreduce_model_catches_a_single_buffer():
    """Negative control: with one buffer a rank that is a call ahead overwrites a slot another rank has not read yet."""
    assert any(not allreduce_reads_are_consistent(4, calls=12, buffers=1, seed=seed) for seed in range(40))
