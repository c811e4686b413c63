"""ctypes door onto libb200_kernels.so (the C ABI of include/b200_kernels.h).

There is no fallback: if the library is missing or a symbol is absent, import
fails.  Nothing here touches a GPU until a kernel entry point is called.
"""
import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_DIR = PKG / "_lib"

F32, F16, BF16 = 0, 1, 2
REDUCE_SUM, REDUCE_MAX = 0, 1

ERRORS = {0: "ok", -1: "invalid argument", -2: "unsupported", -3: "workspace too small",
          -4: "CUDA error", -5: "alignment"}


class FlashAttnParams(C.Structure):
    _fields_ = (
        [(n, C.c_int64) for n in (
            "q_batch_stride", "k_batch_stride", "v_batch_stride", "o_batch_stride",
            "q_row_stride", "k_row_stride", "v_row_stride", "o_row_stride",
            "q_head_stride", "k_head_stride", "v_head_stride", "o_head_stride",
            "b", "h", "h_k", "d", "d_rounded")]
        + [("softmax_scale", C.c_float)]
        + [(n, C.c_int64) for n in ("seqlen_q", "seqlen_k", "seqlen_q_rounded", "seqlen_k_rounded")]
        + [("p_dropout", C.c_float), ("window_size_left", C.c_int64), ("window_size_right", C.c_int64)]
    )


class FlashKvCacheParams(C.Structure):
    _fields_ = (
        [(n, C.c_int64) for n in (
            "q_batch_stride", "k_batch_stride", "v_batch_stride", "knew_batch_stride", "vnew_batch_stride",
            "o_batch_stride",
            "q_row_stride", "k_row_stride", "v_row_stride", "knew_row_stride", "vnew_row_stride", "o_row_stride",
            "q_head_stride", "k_head_stride", "v_head_stride", "knew_head_stride", "vnew_head_stride",
            "o_head_stride",
            "b", "h", "h_k", "d", "d_rounded", "seqlen_knew")]
        + [("softmax_scale", C.c_float)]
        + [(n, C.c_int64) for n in ("seqlen_q", "seqlen_k", "seqlen_q_rounded", "seqlen_k_rounded",
                                    "window_size_left", "window_size_right")]
    )


_vp, _i64, _int, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t

# symbol -> (restype, argtypes); every symbol include/b200_kernels.h declares
SIGNATURES = {
    "b200_version": (C.c_char_p, []),
    "b200_last_cuda_error": (_int, []),
    "b200_error_string": (C.c_char_p, [_int]),
    "b200_reduce_workspace_bytes": (_sz, [_int, _int, _i64, _i64, _i64]),
    "b200_reduce": (_int, [_int, _int, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "b200_reduce_sum_to_f32": (_int, [_int, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    "b200_cast_from_f32": (_int, [_int, _vp, _vp, _i64, _vp]),
    "b200_fill": (_int, [_int, _vp, _i64, C.c_uint64, _vp]),
    "b200_sharded_sum_inbox_bytes": (_sz, [_int, _i64]),
    "b200_reduce_reserve_blocks": (None, [_int]),
    "b200_sharded_sum_finish": (_int, [_int, _vp, C.POINTER(_vp), C.POINTER(_vp), _int, _int, _i64, _vp, _vp, _vp, _vp]),
    "b200_reduce_no_alloc_max_bytes": (_sz, []),
    "b200_reduce_no_alloc": (_int, [_int, _int, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_index_select": (_int, [_int, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "b200_index_put_workspace_bytes": (_sz, [_int, _i64, _i64, _i64]),
    "b200_index_put_prepare": (_int, [_vp]),
    "b200_index_put_release": (_int, [_vp]),
    "b200_index_put_add": (_int, [_int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp, _vp]),
    "b200_transpose_batched": (_int, [_int, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_permute": (_int, [_int, _vp, _vp, _int, C.POINTER(_i64), C.POINTER(_i64), _vp]),
    "b200_flash_attn_fwd": (_int, [_int, _vp, _vp, _vp, _vp, _vp, C.POINTER(FlashAttnParams), _vp]),
    "b200_flash_attn_bwd": (_int, [_int] + [_vp] * 11 + [C.POINTER(FlashAttnParams), _vp]),
    "b200_flash_attn_take_status": (_int, [C.POINTER(_int)]),
    "b200_flash_attn_kvcache_workspace_bytes": (_i64, [C.POINTER(FlashKvCacheParams)]),
    "b200_flash_attn_kvcache": (_int, [_int] + [_vp] * 8 + [C.POINTER(FlashKvCacheParams), _vp, _sz, _vp]),
}
# tuning doors that pick a code path explicitly (0 = automatic); not in the header
EXTRA = {
    "b200_index_select_path": (_int, [_int, _int, _int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "b200_transpose_batched_path": (_int, [_int, _int, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_flash_attn_kvcache_tune": (None, [_int]),
    "b200_reduce_cols_plan_override": (None, [_int]),
    "b200_index_put_tune": (None, [_int]),
    "b200_sharded_sum_finish_nvls": (_int, [_int, _vp, _vp, _vp, C.POINTER(_vp), _int, _int, _i64, _vp, _vp, _vp, _vp]),
    "b200_transpose_tune": (None, [_int, _int, _int]),
    "b200_reduce_tune": (None, [_int, _int, _int, _int]),
    "b200_flash_attn_debug": (None, [_int, C.c_uint]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = LIB_DIR / "libb200_kernels.so"
        if not path.exists():
            raise ImportError(
                f"{path} is missing: build it with `python -m byteir_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)")
        h = C.CDLL(str(path))
        for name, (res, args) in {**SIGNATURES, **EXTRA}.items():
            fn = getattr(h, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


class B200Error(RuntimeError):
    pass


def check(rc, what):
    if rc != 0:
        detail = ""
        if rc == -4:
            detail = f" (cudaError {lib().b200_last_cuda_error()})"
        raise B200Error(f"{what}: {ERRORS.get(rc, rc)}{detail}")
