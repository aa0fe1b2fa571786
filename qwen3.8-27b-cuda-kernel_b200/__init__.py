"""qwen38-b200: B200 (sm_100a) kernels and host engine for the ragged continuous-batching step of the
Qwen3.8 hybrid model, behind the reference engine's own interfaces.

Python here is glue only: it loads the native libraries (ctypes over the C ABI of
include/q38_kernels.h and include/q38_engine.h) and offers thin helpers for tests and benchmarks.
There is no Python or CPU implementation of any kernel: if the CUDA library is missing, loading fails.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_DIR = HERE / "lib"


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str) -> C.CDLL:
    path = LIB_DIR / name
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} is missing: build it with `python {HERE / 'build.py'}` (there is no fallback path)")
    return C.CDLL(str(path), mode=C.RTLD_GLOBAL)


# ---- struct mirrors of include/q38_kernels.h ------------------------------------------------------
class BatchDesc(C.Structure):
    _fields_ = [("num_seqs", C.c_int), ("num_tokens", C.c_int), ("max_tokens_per_seq", C.c_int),
                ("seq_start", C.c_void_p), ("seq_slot", C.c_void_p), ("seq_pos0", C.c_void_p),
                ("tok_pos", C.c_void_p), ("tok_seq", C.c_void_p)]


class KvCacheDesc(C.Structure):
    _fields_ = [("pool", C.c_void_p), ("dtype", C.c_int), ("kv_heads", C.c_int), ("num_pages", C.c_int),
                ("page_bytes", C.c_size_t), ("layer_stride", C.c_size_t), ("block_table", C.c_void_p),
                ("max_pages_per_seq", C.c_int)]


class BQWeight(C.Structure):
    _fields_ = [("lo", C.c_void_p), ("hi", C.c_void_p), ("scales", C.c_void_p), ("bits", C.c_int), ("n", C.c_int),
                ("k", C.c_int), ("rows", C.c_int)]


MAX_PEERS, ALLREDUCE_ROWS = 8, 16


class PeerAllreduce(C.Structure):
    """q38_peer_allreduce: the ranks' receive buffers and flags as mapped into this process."""
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("recv", C.c_void_p * MAX_PEERS),
                ("flags", C.c_void_p * MAX_PEERS), ("seq", C.c_void_p), ("poll_limit", C.c_uint)]


class GemmEpilogue(C.Structure):
    _fields_ = [("kind", C.c_int), ("out", C.c_void_p), ("ldo", C.c_int), ("n_store", C.c_int),
                ("residual", C.c_void_p), ("xbf", C.c_void_p), ("partials_out", C.c_void_p),
                ("partials_in", C.c_void_p), ("hidden", C.c_int), ("eps", C.c_float),
                ("allreduce", C.POINTER(PeerAllreduce))]


class GemmWorkspace(C.Structure):
    _fields_ = [("partials", C.c_void_p), ("partial_floats", C.c_size_t), ("counters", C.c_void_p),
                ("num_counters", C.c_int)]


class QkNormRopeParams(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("ld_proj", C.c_int), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("eps", C.c_float), ("rope_theta", C.c_float), ("num_q_heads", C.c_int), ("num_kv_heads", C.c_int),
                ("q_out", C.c_void_p), ("attn_layer", C.c_int)]


class AttentionParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("gate", C.c_void_p), ("ld_gate", C.c_int), ("out", C.c_void_p),
                ("num_q_heads", C.c_int), ("num_kv_heads", C.c_int), ("attn_layer", C.c_int),
                ("split_scratch", C.c_void_p), ("max_splits", C.c_int), ("scratch_rows", C.c_int)]


class GdnDims(C.Structure):
    _fields_ = [("num_k_heads", C.c_int), ("num_v_heads", C.c_int), ("conv_dim", C.c_int), ("ld_proj", C.c_int)]


class GdnStateDesc(C.Structure):
    _fields_ = [("recurrent", C.c_void_p), ("conv", C.c_void_p), ("num_gdn_layers", C.c_int)]


class GdnConvParams(C.Structure):
    _fields_ = [("proj", C.c_void_p), ("conv_w", C.c_void_p), ("qkv", C.c_void_p), ("gdn_layer", C.c_int)]


class GdnRecurrenceParams(C.Structure):
    _fields_ = [("qkv", C.c_void_p), ("ab", C.c_void_p), ("A", C.c_void_p), ("dt_bias", C.c_void_p),
                ("z", C.c_void_p), ("ld_z", C.c_int), ("norm_w", C.c_void_p), ("eps", C.c_float),
                ("out", C.c_void_p), ("gdn_layer", C.c_int)]


class SamplingParamsDev(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("repetition_penalty", C.c_float), ("seed", C.c_uint64)]


class SamplingArgs(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld", C.c_int), ("vocab", C.c_int), ("params", C.c_void_p),
                ("row_slot", C.c_void_p), ("history", C.c_void_p), ("history_len", C.c_void_p),
                ("history_cap", C.c_int), ("step", C.c_void_p), ("tokens_out", C.c_void_p),
                ("logprob_out", C.c_void_p)]


EPI_STORE_BF16, EPI_SWIGLU, EPI_RESIDUAL, EPI_STORE_F32, EPI_ALLREDUCE_RESIDUAL = 0, 1, 2, 3, 4
KV_INT8, KV_BF16 = 0, 1

# every entry point include/q38_kernels.h declares, with its ctypes signature
KERNEL_API = {
    "q38_kv_page_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "q38_qgemm_num_configs": (C.c_int, []),
    "q38_qgemm_config_name": (C.c_char_p, [C.c_int]),
    "q38_qgemm_config_tile_m": (C.c_int, [C.c_int]),
    "q38_qgemm_auto_config": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "q38_qgemm": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(BQWeight), C.POINTER(GemmEpilogue),
                            C.POINTER(GemmWorkspace), C.c_void_p, C.c_int]),
    "q38_qgemm_static": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(BQWeight), C.POINTER(GemmEpilogue), C.c_void_p]),
    "q38_set_qgemm_tuning": (None, [C.c_void_p]),
    "q38_bq_dequant": (C.c_int, [C.POINTER(BQWeight), C.c_void_p, C.c_void_p]),
    "q38_embed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "q38_residual_update": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "q38_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "q38_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "q38_peer_free": (C.c_int, [C.c_void_p]),
    "q38_peer_export": (C.c_int, [C.c_void_p, C.c_char_p]),
    "q38_peer_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "q38_peer_close": (C.c_int, [C.c_void_p]),
    "q38_qk_norm_rope_append": (C.c_int, [C.POINTER(QkNormRopeParams), C.POINTER(BatchDesc), C.POINTER(KvCacheDesc),
                                          C.c_void_p]),
    "q38_attention_decode_splits": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "q38_attention_decode": (C.c_int, [C.POINTER(AttentionParams), C.POINTER(BatchDesc), C.POINTER(KvCacheDesc),
                                       C.c_void_p]),
    "q38_attention_prefill": (C.c_int, [C.POINTER(AttentionParams), C.POINTER(BatchDesc), C.POINTER(KvCacheDesc),
                                        C.c_void_p]),
    "q38_gdn_ab": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_void_p,
                             C.c_void_p]),
    "q38_gdn_conv": (C.c_int, [C.POINTER(GdnConvParams), C.POINTER(GdnDims), C.POINTER(BatchDesc),
                               C.POINTER(GdnStateDesc), C.c_void_p]),
    "q38_gdn_recurrence": (C.c_int, [C.POINTER(GdnRecurrenceParams), C.POINTER(GdnDims), C.POINTER(BatchDesc),
                                     C.POINTER(GdnStateDesc), C.c_void_p]),
    "q38_gdn_set_chunk_scan_tensor_cores": (None, [C.c_int]),
    "q38_gdn_chunk_scratch_floats": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "q38_gdn_recurrence_chunked": (C.c_int, [C.POINTER(GdnRecurrenceParams), C.POINTER(GdnDims), C.POINTER(BatchDesc),
                                             C.POINTER(GdnStateDesc), C.c_void_p, C.c_size_t, C.c_void_p]),
    "q38_sample": (C.c_int, [C.POINTER(SamplingArgs), C.c_int, C.c_void_p]),
    "q38_target_logprobs": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "q38_pack_ragged": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_void_p]),
    "q38_last_error": (C.c_char_p, []),
    "q38_set_dependent_launch": (None, [C.c_int]),
    "q38_device_error": (C.c_uint, [C.c_int]),
    "q38_device_error_collect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "q38_device_error_inject": (C.c_int, [C.c_uint]),
    "q38_num_sms": (C.c_int, []),
}

_kernels = None


def kernels() -> C.CDLL:
    """The CUDA kernel library (loaded once). Raises NativeLibraryMissing if it has not been built."""
    global _kernels
    if _kernels is None:
        lib = _load("libq38_kernels.so")
        for name, (res, args) in KERNEL_API.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _kernels = lib
    return _kernels


class KernelError(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        raise KernelError(kernels().q38_last_error().decode())


def ptr(t) -> int:
    """Device (or host) address of a torch tensor, None -> NULL."""
    return None if t is None else t.data_ptr()
