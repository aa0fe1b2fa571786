"""ctypes binding of the host engine's C ABI (include/q38_engine.h): ModelFile, ModelRunner, Engine.

Thin on purpose: every method is one native call; scheduling, memory planning, CUDA graphs and all compute
live in libq38_engine.so / libq38_kernels.so.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _load, kernels


class Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("repetition_penalty", C.c_float), ("seed", C.c_uint64)]


def greedy() -> Sampling:
    return Sampling(0.0, 0, 1.0, 0.0, 0.0, 1.0, 0)


class RunnerOptions(C.Structure):
    _fields_ = [("max_batch", C.c_int), ("prefill_chunk", C.c_int), ("kv_dtype", C.c_int), ("kv_tokens", C.c_int64),
                ("max_context", C.c_int), ("reserve_mib", C.c_size_t), ("embedding_on_host", C.c_int),
                ("cuda_graphs", C.c_int), ("history_cap", C.c_int), ("verbose", C.c_int)]


class DecodeRow(C.Structure):
    _fields_ = [("slot", C.c_int), ("position", C.c_int), ("token", C.c_int32), ("sampling", Sampling),
                ("step", C.c_int)]


class PrefillRow(C.Structure):
    _fields_ = [("slot", C.c_int), ("pos0", C.c_int), ("tokens", C.POINTER(C.c_int32)), ("num_tokens", C.c_int),
                ("sample", C.c_int), ("sampling", Sampling), ("step", C.c_int)]


class EngineOptions(C.Structure):
    _fields_ = [("runner", RunnerOptions), ("seed", C.c_uint64), ("ragged_prefill", C.c_int), ("mixed_steps", C.c_int)]


class Stats(C.Structure):
    _fields_ = [("prefill_tokens", C.c_int64), ("prefill_s", C.c_double), ("decode_tokens", C.c_int64),
                ("decode_s", C.c_double), ("decode_steps", C.c_int64), ("requests_done", C.c_int64)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        kernels()  # dependency, loaded RTLD_GLOBAL
        L = _load("libq38_engine.so")
        L.q38e_last_error.restype = C.c_char_p
        L.q38e_model_summary.restype = C.c_char_p
        _lib = L
    return _lib


class EngineError(RuntimeError):
    pass


def _ok(rc: int) -> None:
    if rc != 0:
        raise EngineError(lib().q38e_last_error().decode())


def default_runner_options(**kw) -> RunnerOptions:
    o = RunnerOptions()
    lib().q38e_default_runner_options(C.byref(o))
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def load_tuning(path) -> None:
    """Installs a GEMM tile-configuration table (JSON written by gemm_bench.py --sweep --save); "" clears it."""
    _ok(lib().q38e_tuning_load(str(path).encode()))


def tuning_lookup(bits: int, n: int, k: int, m: int) -> int:
    """Configuration id the installed table gives for a call, -1 = the dispatcher's own choice."""
    return int(lib().q38e_tuning_lookup(bits, n, k, m))


class Model:
    def __init__(self, path):
        self.h = C.c_void_p()
        _ok(lib().q38e_model_open(str(path).encode(), C.byref(self.h)))
        self.vocab = lib().q38e_model_vocab(self.h)
        self.hidden = lib().q38e_model_hidden(self.h)
        self.layers = lib().q38e_model_layers(self.h)

    def summary(self) -> str:
        return lib().q38e_model_summary(self.h).decode()

    def dequant(self, name: str, n: int, k: int) -> np.ndarray:
        out = np.empty((n, k), dtype=np.float32)
        _ok(lib().q38e_model_dequant(self.h, name.encode(), out.ctypes.data_as(C.c_void_p), C.c_size_t(out.size)))
        return out

    def close(self):
        if self.h:
            lib().q38e_model_close(self.h)
            self.h = C.c_void_p()


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


class Runner:
    def __init__(self, model: Model, options: RunnerOptions | None = None, _borrowed=None):
        self.model = model
        self.owned = _borrowed is None
        if _borrowed is not None:
            self.h = _borrowed
        else:
            self.h = C.c_void_p()
            _ok(lib().q38e_runner_create(model.h, C.byref(options or default_runner_options()), C.byref(self.h)))

    def close(self):
        if self.owned and self.h:
            lib().q38e_runner_destroy(self.h)
            self.h = C.c_void_p()

    def reset_slot(self, slot: int):
        _ok(lib().q38e_runner_reset_slot(self.h, slot))

    def kv_ensure(self, slot: int, tokens: int) -> bool:
        ok = C.c_int()
        _ok(lib().q38e_runner_kv_ensure(self.h, slot, tokens, C.byref(ok)))
        return bool(ok.value)

    def kv_release(self, slot: int):
        _ok(lib().q38e_runner_kv_release(self.h, slot))

    def kv_pages(self, slot: int) -> list[int]:
        buf = (C.c_int * 8192)()
        n = C.c_int()
        _ok(lib().q38e_runner_kv_pages(self.h, slot, buf, 8192, C.byref(n)))
        return list(buf[:n.value])

    def kv_free_pages(self) -> int:
        n = C.c_int()
        _ok(lib().q38e_runner_kv_free_pages(self.h, C.byref(n)))
        return n.value

    def prefill(self, rows) -> tuple[np.ndarray, np.ndarray]:
        """rows: iterable of (slot, pos0, tokens, sampling_or_None, step)."""
        rows = list(rows)
        arr = (PrefillRow * len(rows))()
        keep = []
        for i, (slot, pos0, tokens, sampling, step) in enumerate(rows):
            t = _i32(tokens)
            keep.append(t)
            arr[i] = PrefillRow(slot, pos0, t.ctypes.data_as(C.POINTER(C.c_int32)), len(t), int(sampling is not None),
                                sampling if sampling is not None else greedy(), step)
        toks = np.zeros(len(rows), dtype=np.int32)
        lps = np.zeros(len(rows), dtype=np.float32)
        n = C.c_int()
        _ok(lib().q38e_runner_prefill(self.h, arr, len(rows), toks.ctypes.data_as(C.c_void_p),
                                      lps.ctypes.data_as(C.c_void_p), C.byref(n)))
        return toks[:n.value], lps[:n.value]

    def decode(self, rows) -> tuple[np.ndarray, np.ndarray]:
        """rows: iterable of (slot, position, token, sampling, step)."""
        rows = list(rows)
        arr = (DecodeRow * len(rows))(*[DecodeRow(s, p, int(t), sm, st) for s, p, t, sm, st in rows])
        toks = np.zeros(len(rows), dtype=np.int32)
        lps = np.zeros(len(rows), dtype=np.float32)
        _ok(lib().q38e_runner_decode(self.h, arr, len(rows), toks.ctypes.data_as(C.c_void_p),
                                     lps.ctypes.data_as(C.c_void_p)))
        return toks, lps

    def prefill_logits(self, slot: int, pos0: int, tokens) -> np.ndarray:
        t = _i32(tokens)
        out = np.empty((len(t), self.model.vocab), dtype=np.float32)
        _ok(lib().q38e_runner_prefill_logits(self.h, slot, pos0, t.ctypes.data_as(C.c_void_p), len(t),
                                             out.ctypes.data_as(C.c_void_p)))
        return out

    def score(self, slot: int, pos0: int, tokens, targets) -> np.ndarray:
        t, g = _i32(tokens), _i32(targets)
        out = np.empty(len(t), dtype=np.float32)
        _ok(lib().q38e_runner_score(self.h, slot, pos0, t.ctypes.data_as(C.c_void_p), g.ctypes.data_as(C.c_void_p), len(t),
                                    out.ctypes.data_as(C.c_void_p)))
        return out

    def set_profiling(self, on: bool):
        _ok(lib().q38e_runner_set_profiling(self.h, int(on)))

    def set_graphs(self, on: bool):
        _ok(lib().q38e_runner_set_graphs(self.h, int(on)))

    def profile(self, clear: bool = True) -> dict[str, tuple[float, int]]:
        buf = C.create_string_buffer(16384)
        _ok(lib().q38e_runner_profile(self.h, buf, 16384, int(clear)))
        out = {}
        for line in buf.value.decode().splitlines():
            name, ms, calls = line.split()
            out[name] = (float(ms), int(calls))
        return out

    def last_step_ms(self) -> float:
        ms = C.c_float()
        _ok(lib().q38e_runner_last_step_ms(self.h, C.byref(ms)))
        return ms.value

    def replay_decode_core(self, rows: int, iters: int) -> float:
        ms = C.c_float()
        _ok(lib().q38e_runner_replay_decode_core(self.h, rows, iters, C.byref(ms)))
        return ms.value

    def last_logits(self, rows: int) -> np.ndarray:
        out = np.empty((rows, self.model.vocab), dtype=np.float32)
        _ok(lib().q38e_runner_last_logits(self.h, rows, out.ctypes.data_as(C.c_void_p)))
        return out

    def memory(self) -> dict:
        w, ws, st, kv = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        kt = C.c_int64()
        _ok(lib().q38e_runner_memory(self.h, C.byref(w), C.byref(ws), C.byref(st), C.byref(kv), C.byref(kt)))
        return {"weights": w.value, "workspace": ws.value, "state": st.value, "kv": kv.value, "kv_tokens": kt.value}


@dataclass
class Finished:
    id: int
    tokens: np.ndarray
    logprobs: np.ndarray
    finish: str
    error: str
    times: tuple = field(default_factory=tuple)


class Engine:
    REASONS = ("none", "stop", "length", "error")

    def __init__(self, model: Model, runner_options: RunnerOptions | None = None, seed: int = 0x5eed,
                 ragged_prefill: bool = False, mixed_steps: bool = False):
        self.model = model
        o = EngineOptions(runner_options or default_runner_options(), seed, int(ragged_prefill), int(mixed_steps))
        self.h = C.c_void_p()
        _ok(lib().q38e_engine_create(model.h, C.byref(o), C.byref(self.h)))
        rh = C.c_void_p()
        _ok(lib().q38e_engine_runner(self.h, C.byref(rh)))
        self.runner = Runner(model, _borrowed=rh)

    def close(self):
        if self.h:
            lib().q38e_engine_destroy(self.h)
            self.h = C.c_void_p()

    def submit(self, prompt, sampling: Sampling | None = None, max_new_tokens: int = 4096, stop_tokens=None,
               ignore_eos: bool = False) -> int:
        p = _i32(prompt)
        st = _i32(stop_tokens) if stop_tokens is not None and len(stop_tokens) else None
        rid = C.c_int()
        s = sampling if sampling is not None else Sampling(1.0, 20, 0.95, 0.0, 0.0, 1.0, 0)
        _ok(lib().q38e_engine_submit(self.h, p.ctypes.data_as(C.c_void_p), len(p), C.byref(s), max_new_tokens,
                                     st.ctypes.data_as(C.c_void_p) if st is not None else None,
                                     0 if st is None else len(st), int(ignore_eos), C.byref(rid)))
        return rid.value

    def step(self) -> bool:
        more = C.c_int()
        _ok(lib().q38e_engine_step(self.h, C.byref(more)))
        return bool(more.value)

    def run(self):
        _ok(lib().q38e_engine_run(self.h))

    def idle(self) -> bool:
        v = C.c_int()
        _ok(lib().q38e_engine_idle(self.h, C.byref(v)))
        return bool(v.value)

    def take_finished(self) -> list[Finished]:
        out = []
        while True:
            rid, n, why = C.c_int(), C.c_int(), C.c_int()
            _ok(lib().q38e_engine_finished_next(self.h, C.byref(rid), C.byref(n), C.byref(why)))
            if rid.value < 0:
                return out
            toks = np.zeros(n.value, dtype=np.int32)
            lps = np.zeros(n.value, dtype=np.float32)
            err = C.create_string_buffer(256)
            times = (C.c_double * 3)()
            _ok(lib().q38e_engine_finished_take(self.h, toks.ctypes.data_as(C.c_void_p), lps.ctypes.data_as(C.c_void_p),
                                                err, 256, times))
            out.append(Finished(rid.value, toks, lps, self.REASONS[why.value], err.value.decode(), tuple(times)))

    def stats(self, reset: bool = False) -> Stats:
        s = Stats()
        _ok(lib().q38e_engine_stats(self.h, C.byref(s), int(reset)))
        return s
