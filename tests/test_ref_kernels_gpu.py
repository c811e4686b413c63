"""The reference's own CUDA kernels (compiled for sm_100a into oracle/_ref/libref_kernels.so by
`make -C oracle _ref`) as a second opinion on the GPU: they must agree with the CPU oracle and with
this build's kernels on the same seeded inputs.  Skipped when the library was not prebuilt."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle_lib as O

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_kernels.so"


@pytest.fixture(scope="module")
def ref():
    if not REF.exists():
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference checkout at build time)")
    lib = C.CDLL(str(REF))
    lib.ref_reduce_workspace_bytes.restype = C.c_size_t
    lib.ref_reduce_workspace_bytes.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t]
    lib.ref_reduce.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                               C.c_void_p, C.c_void_p]
    lib.ref_index_select.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [C.c_void_p]
    lib.ref_index_put_f32.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p]
    lib.ref_transpose2d.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    return lib


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("op,dt,A,B,Cc", [(0, "f32", 1024, 4096, 1), (1, "f32", 64, 1000, 1), (0, "f32", 2, 128, 256),
                                          (0, "f16", 1, 2048, 1024), (1, "f16", 4096, 1024, 1), (1, "f16", 3, 500, 64)])
def test_reference_reduce_agrees(ref, op, dt, A, B, Cc):
    from byteir_b200 import ops
    rng = np.random.default_rng(A + B)
    x = rng.standard_normal((A, B, Cc), dtype=np.float32)
    x = x if dt == "f32" else x.astype(np.float16)
    xd = torch.from_numpy(x).cuda()
    out = torch.empty(A * Cc, dtype=xd.dtype, device="cuda")
    ws = torch.empty(max(ref.ref_reduce_workspace_bytes(0, A, B, Cc), 16), dtype=torch.uint8, device="cuda")
    assert ref.ref_reduce(op, 0 if dt == "f32" else 1, xd.data_ptr(), out.data_ptr(), A, B, Cc, ws.data_ptr(), _s()) == 0
    torch.cuda.synchronize()
    want = O.reduce("sum" if op == 0 else "max", x, A, B, Cc)
    ours = (ops.reduce_sum if op == 0 else ops.reduce_max)(xd, [1]).reshape(-1)
    if op == 1:
        assert np.array_equal(out.cpu().numpy().view(np.uint16 if dt == "f16" else np.uint32),
                              want.view(np.uint16 if dt == "f16" else np.uint32))
        assert torch.equal(out, ours)
    else:
        tol = dict(rtol=2e-2, atol=1e-2) if dt == "f16" else dict(rtol=1e-4, atol=1e-3)
        np.testing.assert_allclose(out.cpu().numpy().astype(np.float64), want.astype(np.float64), **tol)
        np.testing.assert_allclose(ours.cpu().numpy().astype(np.float64), out.cpu().numpy().astype(np.float64), **tol)


def test_reference_index_select_and_transpose_agree_bit_for_bit(ref):
    from byteir_b200 import ops
    rng = np.random.default_rng(5)
    table = rng.standard_normal((30522, 128)).astype(np.float16)
    idx = rng.integers(0, 30522, 4096).astype(np.int64)
    td, idd = torch.from_numpy(table).cuda(), torch.from_numpy(idx).cuda()
    out = torch.empty(4096, 128, dtype=torch.float16, device="cuda")
    assert ref.ref_index_select(2, td.data_ptr(), idd.data_ptr(), out.data_ptr(), 1, 30522, 4096, 128, _s()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ops.index_select(td, idd, 0))
    assert np.array_equal(out.cpu().numpy(), O.index_select(table, idx, 0)[0])

    x = rng.uniform(-1, 1, (1000, 512)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    t = torch.empty(512, 1000, dtype=torch.float32, device="cuda")
    assert ref.ref_transpose2d(0, xd.data_ptr(), t.data_ptr(), 1000, 512, _s()) == 0
    torch.cuda.synchronize()
    assert torch.equal(t, ops.transpose(xd, (1, 0)))
    assert np.array_equal(t.cpu().numpy(), O.transpose(x, (1, 0)))


def test_reference_index_put_atomics_agree_within_f32_tolerance(ref):
    from byteir_b200 import ops
    rng = np.random.default_rng(6)
    x = rng.standard_normal((256, 128)).astype(np.float32)
    idx = rng.integers(0, 256, 4096).astype(np.int64)
    upd = rng.standard_normal((4096, 128)).astype(np.float32)
    xd, idd, ud = (torch.from_numpy(a).cuda() for a in (x, idx, upd))
    out = torch.empty_like(xd)
    assert ref.ref_index_put_f32(xd.data_ptr(), idd.data_ptr(), ud.data_ptr(), out.data_ptr(), 4096, 128, 256 * 128, _s()) == 0
    torch.cuda.synchronize()
    want, _ = O.index_put_add(x, idx, upd)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-4, atol=1e-4)  # atomics: order varies
    np.testing.assert_allclose(ops.index_put_add(xd, idd, ud).cpu().numpy(), want, rtol=1e-5, atol=1e-5)
