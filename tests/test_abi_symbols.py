"""CPU checks of the drop-in boundary: every function the C headers declare is exported by the
built libraries (no compute calls: there is no GPU here), workspace sizing works without a
device, and libflash_attn.so exports what the reference's custom-call bridge looks up."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "byteir_b200" / "_lib"


def _declared(header):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef struct \{.*?\} \w+;", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+|brt_\w+)\s*\(", text)))


def test_kernel_abi_exports_every_declared_symbol():
    names = _declared("b200_kernels.h")
    assert len(names) >= 15
    lib = C.CDLL(str(LIB / "libb200_kernels.so"))
    for n in names:
        assert hasattr(lib, n), n
    from byteir_b200 import _native
    assert set(names) <= set(_native.SIGNATURES), set(names) - set(_native.SIGNATURES)
    _native.lib()


def test_brt_c_api_exports_every_declared_symbol():
    names = [n for n in _declared("brt_c_api.h") if n not in ("brt_session", "brt_request")]
    lib = C.CDLL(str(LIB / "libbrt_b200.so"))
    for n in names:
        assert hasattr(lib, n), n


def test_flash_attn_library_exports_the_custom_call_symbols():
    lib = C.CDLL(str(LIB / "libflash_attn.so"))
    for n in ("run_flash_attn_fwd", "run_flash_attn_bwd", "run_flash_attn_kvcache",
              "run_flash_attn_fwd_bf16", "run_flash_attn_bwd_bf16", "b200_custom_last_error"):
        assert hasattr(lib, n), n
    version = C.c_char_p.in_dll(lib, "VERSION")  # a `const char *` variable, as in flash_api.cu:7-9
    assert version.value == b"2.5.3"


def test_workspace_sizes_are_pure_functions_of_the_shape():
    from byteir_b200 import _native as N
    lib = N.lib()
    assert lib.b200_reduce_workspace_bytes(0, N.F32, 1024, 4096, 1) == 0          # config 1: one pass
    ws = lib.b200_reduce_workspace_bytes(0, N.F16, 1, 64 * 512, 1024)              # config 2a: split-K partials
    assert ws > 0 and ws % (1024 * 4) == 0
    assert lib.b200_reduce_workspace_bytes(1, N.F16, 64 * 512, 1024, 1) == 0       # config 2b
    assert lib.b200_index_put_workspace_bytes(N.F16, 1_000_000, 262_144, 128) > 4 * 262_144 * 4
    assert lib.b200_index_put_workspace_bytes(N.F16, 10, 0, 4) == 0
    assert lib.b200_reduce_no_alloc_max_bytes() == 1 << 20
    assert lib.b200_error_string(-3) == b"workspace missing or too small"


def test_ops_refuse_cpu_tensors():
    import torch
    from byteir_b200 import ops
    with pytest.raises(ValueError, match="no CPU path"):
        ops.reduce_sum(torch.zeros(4, 4), [1])


def test_kvcache_plan_is_a_pure_function_of_the_shapes():
    """workspace size and argument checks of the decode entry need no device"""
    import ctypes as C
    from byteir_b200 import _native as N

    def params(b=16, sq=1, h=32, hk=8, d=128, cap=8192):
        p = N.FlashKvCacheParams()
        p.b, p.seqlen_q, p.h, p.h_k, p.d, p.seqlen_k, p.seqlen_knew = b, sq, h, hk, d, cap, 1
        p.q_row_stride = p.o_row_stride = h * d
        p.q_batch_stride = p.o_batch_stride = sq * h * d
        p.k_row_stride = p.v_row_stride = p.knew_row_stride = p.vnew_row_stride = hk * d
        p.k_batch_stride = p.v_batch_stride = cap * hk * d
        p.knew_batch_stride = p.vnew_batch_stride = hk * d
        for n in ("q", "k", "v", "knew", "vnew", "o"):
            setattr(p, n + "_head_stride", d)
        p.softmax_scale = 0.1
        p.window_size_left = p.window_size_right = -1
        return p

    need = N.lib().b200_flash_attn_kvcache_workspace_bytes
    big = need(C.byref(params()))
    assert big > 0 and big % 4 == 0
    assert need(C.byref(params(b=1, h=1, hk=1, d=32, cap=64))) == 0      # one range: no partial results
    assert need(C.byref(params(d=12))) == -1 and need(C.byref(params(d=264))) == -1
    assert need(C.byref(params(h=30))) == -1 and need(C.byref(params(cap=0))) == -1
    # rows * ranges * (d + 2) floats, with at most 128 ranges
    rows = 16 * 32
    assert big % (rows * (128 + 2) * 4) == 0 and big // (rows * (128 + 2) * 4) <= 128
    # the checks come before any launch: a null tensor is refused without a device
    rc = N.lib().b200_flash_attn_kvcache(1, None, None, None, None, None, None, None,
                                         None, C.byref(params()), None, 0, None)
    assert rc != 0
