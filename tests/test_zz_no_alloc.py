"""The reduction entry point for callers that cannot provide scratch memory
(b200_reduce_no_alloc): its partial sums live in a fixed 1 MiB block inside the
library instead of a caller workspace.  It must give exactly what b200_reduce
gives, call after call, because the block is shared and keeps old contents.

This file sorts last on purpose: a run that stops at the first failure has then
already been through every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("op", [0, 1])
@pytest.mark.parametrize("dt,code", [(torch.float16, 1), (torch.float32, 0)])
def test_no_alloc_reduce_matches_the_workspace_entry_point_twice(op, dt, code):
    from byteir_b200 import _native as N
    lib = N.lib()
    A, B, Cc = 2, 4096, 1024  # column reduction that is split over blocks: it needs scratch
    need = lib.b200_reduce_workspace_bytes(op, code, A, B, Cc)
    assert 0 < need <= lib.b200_reduce_no_alloc_max_bytes()
    gen = torch.Generator(device="cuda").manual_seed(7)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    for call in range(2):  # second call: the block still holds the first call's partials
        x = torch.randn(A, B, Cc, device="cuda", dtype=torch.float32, generator=gen).to(dt)
        want = torch.empty(A, Cc, dtype=dt, device="cuda")
        got = torch.full((A, Cc), float("nan"), dtype=dt, device="cuda")
        N.check(lib.b200_reduce(op, code, x.data_ptr(), want.data_ptr(), A, B, Cc, ws.data_ptr(), need, _stream()),
                "b200_reduce")
        N.check(lib.b200_reduce_no_alloc(op, code, x.data_ptr(), got.data_ptr(), A, B, Cc, _stream()),
                "b200_reduce_no_alloc")
        torch.cuda.synchronize()
        # same kernels, same launch plan, same summation order: bit-identical
        assert torch.equal(got.view(torch.int16 if dt == torch.float16 else torch.int32),
                           want.view(torch.int16 if dt == torch.float16 else torch.int32)), f"call {call}"
        ref = x.float().sum(1) if op == 0 else x.float().amax(1)
        torch.testing.assert_close(got.float(), ref, rtol=2e-2 if dt == torch.float16 else 1e-5,
                                   atol=1e-2 if dt == torch.float16 else 1e-4)


def test_no_alloc_reduce_without_scratch_need_and_oversize_refusal():
    from byteir_b200 import _native as N
    lib = N.lib()
    # a row reduction needs no scratch at all
    x = torch.randn(512, 1024, device="cuda")
    got = torch.empty(512, device="cuda")
    assert lib.b200_reduce_workspace_bytes(0, 0, 512, 1024, 1) == 0
    N.check(lib.b200_reduce_no_alloc(0, 0, x.data_ptr(), got.data_ptr(), 512, 1024, 1, _stream()), "no_alloc")
    torch.testing.assert_close(got, x.sum(1), rtol=1e-5, atol=1e-4)
    # a shape whose partials do not fit the fixed block is refused, nothing runs
    A, B, Cc = 580, 64, 256
    assert lib.b200_reduce_workspace_bytes(0, 1, A, B, Cc) > lib.b200_reduce_no_alloc_max_bytes()
    y = torch.zeros(A, B, Cc, device="cuda", dtype=torch.float16)
    out = torch.full((A, Cc), 5.0, device="cuda", dtype=torch.float16)
    rc = lib.b200_reduce_no_alloc(0, 1, y.data_ptr(), out.data_ptr(), A, B, Cc, _stream())
    assert rc == -3  # B200_ERR_WORKSPACE
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())
