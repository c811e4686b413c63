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
