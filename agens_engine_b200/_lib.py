"""ctypes bindings of the native libraries (C ABI ``b2_*``), the counterpart of the reference's Rust FFI crate
(``crates/agens-cuda/src/lib.rs``).  Structures mirror the ``*.cuh`` headers under ``csrc/`` field by field."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIBDIR = Path(__file__).resolve().parent / "lib"
_cuda = None
_host = None

B2_OK, B2_ERR_ARG, B2_ERR_LAUNCH, B2_ERR_TIMEOUT, B2_ERR_BOUNDS = range(5)
STATUS_NAMES = {0: "ok", 1: "bad argument", 2: "launch failed", 3: "device wait timed out", 4: "index out of bounds"}


class B2Error(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what}: {STATUS_NAMES.get(code, code)}")
        self.code = code


def check(code: int, what: str):
    if code != 0:
        raise B2Error(what, code)


def _ensure_built():
    if os.environ.get("B200E_NO_BUILD") == "1":
        return
    if not (_LIBDIR / "libagens_b200.so").exists():
        from . import _build
        _build.build()


def cuda_lib() -> C.CDLL:
    """The CUDA library.  Raises if it is missing: callers on a GPU box must never fall back silently."""
    global _cuda
    if _cuda is None:
        _ensure_built()
        path = _LIBDIR / "libagens_b200.so"
        if not path.exists():
            raise RuntimeError(f"native library {path} is missing; run `python -m agens_engine_b200._build`")
        _cuda = C.CDLL(str(path))
        _declare(_cuda)
    return _cuda


def host_lib() -> C.CDLL:
    """Host-only library (no CUDA dependency) for CPU tests of the runtime, scheduler and server code."""
    global _host
    if _host is None:
        override = os.environ.get("B200E_HOST_LIB", "")       # a sanitizer build of the host sources (tools/sanitize.py)
        if override:
            _host = C.CDLL(override)
            return _host
        _ensure_built()
        path = _LIBDIR / "libagens_b200_host.so"
        if not path.exists():
            from . import _build
            _build.build()
        _host = C.CDLL(str(path))
    return _host


# ---------------------------------------------------------------------------------------------------------------
# structure mirrors
# ---------------------------------------------------------------------------------------------------------------
K_MAX_TP = 8
K_MAX_KS = 64


class TpPush(C.Structure):
    _fields_ = [
        ("inbox", C.c_void_p * K_MAX_TP),
        ("rank", C.c_int), ("size", C.c_int),
        ("slot_off", C.c_long), ("clear_off", C.c_long), ("slot_stride", C.c_long),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_ulonglong),
        ("skip_push", C.c_int),
    ]


class CommArgs(C.Structure):
    _fields_ = [
        ("inbox", C.c_void_p * K_MAX_TP),
        ("rank", C.c_int), ("size", C.c_int),
        ("slot_off", C.c_long), ("clear_off", C.c_long), ("clear_n", C.c_long), ("slot_stride", C.c_long),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_ulonglong),
        ("skip_push", C.c_int),
    ]


class WqGemvArgs(C.Structure):
    _fields_ = [
        ("wq", C.c_void_p),
        ("n", C.c_int), ("k", C.c_int), ("m", C.c_int),
        ("bits", C.c_int), ("group", C.c_int),
        ("ks", C.c_int), ("rb", C.c_int),
        ("vworkers", C.c_int), ("fmax", C.c_int),
        ("pro", C.c_int),
        ("x", C.c_void_p), ("ldx", C.c_long),
        ("ss_in", C.c_void_p), ("ss_parts", C.c_int), ("ss_ld", C.c_int),
        ("norm_w", C.c_void_p), ("eps", C.c_float),
        ("epi", C.c_int),
        ("y", C.c_void_p), ("ldy", C.c_long),
        ("resid", C.c_void_p), ("ldr", C.c_long),
        ("ss_out", C.c_void_p),
        ("yf", C.c_void_p),
        ("amax_val", C.c_void_p), ("amax_idx", C.c_void_p), ("n_valid", C.c_int),
        ("scratch", C.c_void_p), ("counters", C.c_void_p),
        ("status", C.c_void_p),
        ("debug", C.c_int),
        ("tp", TpPush),
        ("trace", C.c_void_p),
    ]


class AttnDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("ldq", C.c_long),
        ("kv_pool", C.c_void_p), ("n_pages", C.c_int),
        ("block_table", C.c_void_p), ("bt_ld", C.c_int),
        ("grp_tok0", C.c_void_p), ("grp_cnt", C.c_void_p), ("n_groups", C.c_int),
        ("tok_pos", C.c_void_p), ("tok_seq", C.c_void_p),
        ("tree_mask", C.c_void_p),
        ("hq", C.c_int), ("hkv", C.c_int),
        ("split_keys", C.c_int), ("max_splits", C.c_int),
        ("scale_log2", C.c_float),
        ("part_o", C.c_void_p), ("part_ml", C.c_void_p),
        ("out", C.c_void_p), ("ldo", C.c_long),
        ("n_tok", C.c_int),
        ("status", C.c_void_p),
        ("split_lo", C.c_int), ("split_hi", C.c_int), ("phase", C.c_int),
        ("shared_kv", C.c_int),
    ]


class WqMmArgs(C.Structure):
    _fields_ = [
        ("wq", C.c_void_p), ("n", C.c_int), ("k", C.c_int), ("m", C.c_int),
        ("bits", C.c_int), ("group", C.c_int),
        ("ks", C.c_int), ("n_pad", C.c_int), ("stages", C.c_int),
        ("epi", C.c_int),
        ("y", C.c_void_p), ("ldy", C.c_long),
        ("resid", C.c_void_p), ("ldr", C.c_long),
        ("ss_out", C.c_void_p), ("ss_ld", C.c_int),
        ("yf", C.c_void_p),
        ("amax_val", C.c_void_p), ("amax_idx", C.c_void_p), ("n_valid", C.c_int),
        ("scratch", C.c_void_p), ("counters", C.c_void_p),
        ("status", C.c_void_p),
        ("dbg", C.c_int),
    ]


class SampleArgs(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p), ("ld", C.c_long), ("vocab", C.c_int),
        ("temperature", C.c_void_p), ("top_k", C.c_void_p), ("top_p", C.c_void_p), ("min_p", C.c_void_p),
        ("seed", C.c_void_p), ("position", C.c_void_p),
        ("out", C.c_void_p),
    ]


PRO_PLAIN, PRO_NORM = 0, 1
EPI_STORE, EPI_RESID, EPI_SWIGLU, EPI_F32, EPI_ARGMAX, EPI_TP_RESID = range(6)


def _declare(lib: C.CDLL):
    vp, i, l, f = C.c_void_p, C.c_int, C.c_long, C.c_float
    sig = {
        "b2_wq_gemv": ([C.POINTER(WqGemvArgs), vp], i),
        "b2_wq_gemv_scratch_floats": ([i, i, i, i, i], l),
        "b2_wq_gemv_vworkers": ([i, i, i, i], i),
        "b2_wq_gemv_fmax": ([i, i, i, i], i),
        "b2_wq_bytes": ([i, i, i, i], l),
        "b2_wq_dequant": ([vp, i, i, i, i, vp, l, vp], i),
        "b2_wq_repack": ([vp, vp, i, vp, i, i, i, i, vp, vp], i),
        "b2_wq_random": ([vp, i, i, i, i, f, C.c_ulonglong, vp], i),
        "b2_embed": ([vp, i, vp, i, i, vp, vp, vp, l, vp, vp, vp], i),
        "b2_rmsnorm": ([vp, l, vp, l, vp, l, vp, f, i, i, vp, l, vp], i),
        "b2_sumsq": ([vp, l, i, i, vp, vp], i),
        "b2_rope_kvstore": ([vp, l, i, i, i, i, vp, vp, vp, vp, vp, i, vp, i, i, vp, l, vp, vp], i),
        "b2_rope_kvstore_m": ([vp, l, i, i, i, i, vp, vp, vp, vp, vp, vp, i, vp, i, i, vp, l, vp, vp], i),
        "b2_swiglu_interleaved": ([vp, l, i, i, vp, l, vp], i),
        "b2_argmax_final": ([vp, vp, i, i, i, vp, vp, vp], i),
        "b2_argmax_rows": ([vp, l, i, i, vp, vp], i),
        "b2_decode_step_prep": ([i, vp, vp, vp, vp, vp, vp, vp], i),
        "b2_fill_u32": ([vp, C.c_uint32, l, vp], i),
        "b2_attn_decode": ([C.POINTER(AttnDecodeArgs), i, vp], i),
        "b2_attn_decode_smem_bytes": ([i], i),
        "b2_ipc_alloc": ([C.c_size_t, C.POINTER(vp), C.c_char_p], i),
        "b2_ipc_open": ([C.c_char_p, C.POINTER(vp)], i),
        "b2_ipc_close": ([vp], i),
        "b2_ipc_free": ([vp], i),
        "b2_can_access_peer": ([i, i], i),
        "b2_comm_all_reduce": ([C.POINTER(CommArgs), vp, vp, l, vp, vp, vp], i),
        "b2_comm_all_gather": ([C.POINTER(CommArgs), vp, l, vp, vp], i),
        "b2_comm_reduce_scatter": ([C.POINTER(CommArgs), vp, l, vp, vp], i),
        "b2_comm_collect_gather": ([C.POINTER(CommArgs), l, i, i, i, vp, vp], i),
        "b2_comm_barrier": ([C.POINTER(CommArgs), vp], i),
        "b2_comm_argmax_combine": ([C.POINTER(CommArgs), vp, vp, i, vp, vp, vp], i),
        "b2_wq_mm": ([C.POINTER(WqMmArgs), vp, l, vp, i, i, vp, f, vp, vp], i),
        "b2_wq_mm_ks": ([i, i], i), "b2_wq_mm_npad": ([i], i), "b2_wq_mm_scratch_floats": ([i, i, i], l),
        "b2_sample_rows": ([C.POINTER(SampleArgs), i, vp], i),
        "b2_spec_accept": ([vp, vp, vp, vp, i, vp, vp, i, vp], i),
        "b2_gemm_bf16": ([vp, l, vp, l, i, i, i, vp, vp, l, vp, l, vp, vp], i),
        "b2_bf16_gemv": ([vp, l, vp, l, i, i, i, vp, vp, l, vp, l, vp], i),
        "b2_gemm_bf16_push": ([vp, l, vp, l, i, i, i, vp, i, i, l, l, i, vp, vp], i),
    }
    for name, (args, res) in sig.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = res


def declare_optional(lib: C.CDLL, name: str, args, res):
    if hasattr(lib, name):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
        return fn
    return None


def ptr(t) -> int:
    """Device (or host) address of a torch tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()


def current_stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream
