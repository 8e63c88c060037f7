"""ctypes binding of libtwilight_b200.so (the C ABI declared in include/twilight_b200.h).

There is no fallback: if the shared library is missing, importing an operator raises with the
build command.  Tensors cross the boundary as raw device pointers and sizes only.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtwilight_b200.so"

i32, i64, f32, u32 = C.c_int32, C.c_int64, C.c_float, C.c_uint32
ptr, sz = C.c_void_p, C.c_size_t

# name -> (restype, argtypes); must list every symbol of include/twilight_b200.h
SIGNATURES = {
    "twl_version": (C.c_int, []),
    "twl_status_string": (C.c_char_p, [C.c_int]),
    "twl_last_cuda_error": (C.c_char_p, []),
    "twl_top_p_return_mask_f32": (C.c_int, [ptr, ptr, ptr, f32, u32, u32, ptr, ptr]),
    "twl_top_p_return_mask_f16": (C.c_int, [ptr, C.c_int, ptr, ptr, f32, u32, u32, ptr, ptr]),
    "twl_quest_page_scores": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, i32, i32, i32, i32, ptr, i32,
                                        ptr, ptr]),
    "twl_quest_topk_pages": (C.c_int, [ptr, i32, ptr, i32, i32, i32, ptr, ptr, i32, ptr]),
    "twl_quest_select": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, i32, i32, i32, i32, i32, ptr, i32, ptr, ptr,
                                   i32, ptr, ptr, ptr]),
    "twl_estimate_int4": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32, i32,
                                    i32, f32, ptr, i32, i32, ptr, ptr]),
    "twl_topp_prune": (C.c_int, [ptr, i32, ptr, ptr, ptr, ptr, i32, i32, i32, ptr, f32, ptr, i32,
                                 ptr, ptr, ptr, ptr]),
    "twl_threshold_prune": (C.c_int, [ptr, i32, ptr, ptr, ptr, ptr, i32, i32, i32, f32, ptr, i32, ptr, ptr,
                                      ptr, ptr]),
    "twl_sparse_attn_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "twl_sparse_decode_attn": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, i32, ptr, i32, i32,
                                         i32, i32, f32, ptr, ptr, sz, i32, ptr, ptr]),
    "twl_prune_with_weights": (C.c_int, [i32, ptr, i32, ptr, ptr, ptr, ptr, i32, i32, i32, ptr, f32, ptr, i32,
                                         ptr, ptr, ptr, ptr, ptr]),
    "twl_sparse_decode_attn_weighted": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, i32, ptr, ptr, i32,
                                                  i32, i32, i32, f32, ptr, ptr, sz, i32, ptr, ptr]),
    "twl_sparse_decode_attn_static": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, i32, ptr, i32, i32,
                                                i32, i32, f32, ptr, i32, ptr, ptr]),
    "twl_quantize_k_pages": (C.c_int, [ptr, C.c_int, ptr, i64, ptr]),
    "twl_build_page_meta": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, i32, i32, i32, i32, ptr]),
    "twl_append_kv": (C.c_int, [ptr, ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32,
                                ptr, ptr]),
    "twl_indices_to_mask": (C.c_int, [ptr, i32, ptr, i32, ptr, i32, ptr]),
    "twl_step_workspace_layout": (C.c_int, [i32, i32, i32, i32, i32, i32, ptr]),
    "twl_step_workspace_bytes": (sz, [i32, i32, i32, i32, i32, i32]),
    "twl_select_prune_attend_step": (C.c_int, [ptr, C.c_int, ptr, ptr, ptr, ptr, ptr, ptr, ptr, i32, i32, i32,
                                               i32, i32, i32, i32, f32, ptr, f32, i32, i32, i32, ptr, ptr, sz,
                                               ptr, ptr]),
    "twl_round_scores": (C.c_int, [ptr, i64, C.c_int, f32, ptr]),
}


class StepLayout(C.Structure):
    """``twl_step_layout`` of include/twilight_b200.h: byte offsets of the parts of the step workspace."""
    _fields_ = [(n, C.c_uint64) for n in ("attn", "attn_bytes", "page_scores", "cand_pages", "cand_npages",
                                          "scores", "indices", "budget", "threshold", "weights", "total")] + \
               [(n, C.c_int32) for n in ("max_k", "stride", "kernels", "reserved")]

_lib = None


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Returns the loaded library with typed entry points; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m twilight_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback for these operators)")
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class TwilightError(RuntimeError):
    """A C-ABI call returned a negative status (the reference raises RuntimeError through
    TORCH_CHECK in csrc/src/sampling.cu:25-40)."""


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.twl_status_string(status).decode()
        if status == -4:
            msg += ": " + lib.twl_last_cuda_error().decode()
        raise TwilightError(f"{what}: {msg} (status {status})")
