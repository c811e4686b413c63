"""Flash-attention forward/backward on the GPU against the CPU oracle.
Tolerance for 16-bit outputs: rel 2e-2, abs 1e-2; LSE (f32): 1e-3."""
import numpy as np
import pytest
import torch

import oracle_lib as O

pytestmark = pytest.mark.gpu


def _mk(rng, shape, dt):
    x = rng.standard_normal(shape, dtype=np.float32)
    return x.astype(np.float16) if dt == "f16" else O.f32_to_bf16(x)


def _dev(a):
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(a).cuda()


def _host(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


FWD_CASES = [
    # b, sq, sk, h, hk, causal
    (1, 128, 128, 1, 1, False),
    (1, 128, 128, 1, 1, True),
    (2, 512, 512, 4, 4, True),
    (1, 384, 640, 2, 2, False),
    (1, 300, 300, 3, 1, True),     # ragged, grouped heads
    (1, 200, 456, 2, 2, True),     # bottom-right aligned causal, Sk > Sq
    (1, 1024, 1024, 2, 2, True),
    (4, 1024, 1152, 40, 8, True),  # 640 work items on 148 persistent blocks: several query tiles per block
    (3, 640, 640, 56, 56, False),  # odd number of query tiles: the middle one has no partner
]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("b,sq,sk,h,hk,causal", FWD_CASES)
def test_flash_attn_fwd(b, sq, sk, h, hk, causal, dt):
    from byteir_b200 import ops
    rng = np.random.default_rng(sq * 7 + sk + h)
    q, k, v = _mk(rng, (b, sq, h, 128), dt), _mk(rng, (b, sk, hk, 128), dt), _mk(rng, (b, sk, hk, 128), dt)
    scale = 1.0 / np.sqrt(128.0)
    want_o, want_lse = O.flash_attn_fwd(q, k, v, scale, causal)
    for _ in range(2):
        o, lse = ops.flash_attn_fwd(_dev(q), _dev(k), _dev(v), scale, causal)
    torch.cuda.synchronize()
    go, gl = O.to_f32(_host(o)), lse.cpu().numpy()
    np.testing.assert_allclose(gl, want_lse, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(go, O.to_f32(want_o), rtol=2e-2, atol=1e-2)


BWD_CASES = [
    (1, 128, 128, 1, 1, False),
    (1, 128, 128, 1, 1, True),
    (1, 256, 256, 2, 2, True),
    (2, 512, 512, 4, 2, True),     # grouped heads: dK/dV sum over the group
    (1, 384, 640, 2, 2, False),
    (1, 300, 300, 2, 1, True),     # ragged
    (1, 200, 456, 2, 2, True),
]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("b,sq,sk,h,hk,causal", BWD_CASES)
def test_flash_attn_bwd(b, sq, sk, h, hk, causal, dt):
    from byteir_b200 import ops
    rng = np.random.default_rng(sq * 11 + sk + h)
    q, k, v = _mk(rng, (b, sq, h, 128), dt), _mk(rng, (b, sk, hk, 128), dt), _mk(rng, (b, sk, hk, 128), dt)
    do = _mk(rng, (b, sq, h, 128), dt)
    scale = 1.0 / np.sqrt(128.0)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, causal)
    for _ in range(2):
        dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal)
    torch.cuda.synchronize()
    # the oracle differentiates the same forward: feed it the device's O and LSE
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o), lse.cpu().numpy(), scale, causal)
    for name, got, want in (("dq", dq, wq), ("dk", dk, wk), ("dv", dv, wv)):
        np.testing.assert_allclose(O.to_f32(_host(got)), O.to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)
    again = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal)
    for a, b_ in zip(again, (dq, dk, dv)):
        assert torch.equal(a.view(torch.int16), b_.view(torch.int16)), "backward is not deterministic"


def _fwd_bwd_check(q, k, v, do, causal, window, check_bwd=True, grad_atol_of_max=0.0):
    """grad_atol_of_max: extra absolute tolerance for the gradients as a fraction of the largest
    gradient magnitude, for inputs whose gradients are sums of large cancelling 16-bit products
    (one 16-bit ulp of a partial product is then far above the fixed 1e-2)."""
    from byteir_b200 import ops
    scale = 1.0 / np.sqrt(128.0)
    want_o, want_lse = O.flash_attn_fwd(q, k, v, scale, causal, window=window)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, causal, window)
    torch.cuda.synchronize()
    gl = lse.cpu().numpy()
    assert np.array_equal(np.isinf(gl), np.isinf(want_lse)), "rows without a visible key must have LSE = +inf"
    fin = np.isfinite(want_lse)
    np.testing.assert_allclose(gl[fin], want_lse[fin], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
    if not check_bwd:
        return
    dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal, window)
    torch.cuda.synchronize()
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o), gl, scale, causal, window=window)
    for name, got, want in (("dq", dq, wq), ("dk", dk, wk), ("dv", dv, wv)):
        w = O.to_f32(want)
        atol = max(1e-2, grad_atol_of_max * float(np.abs(w).max()))
        np.testing.assert_allclose(O.to_f32(_host(got)), w, rtol=2e-2, atol=atol, err_msg=name)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attn_scores_that_keep_growing(causal, dt):
    """Keys get larger along the sequence, so the running maximum of a row moves by more than 2^8
    again and again: the accumulator is rescaled at many key tiles, by both softmax groups."""
    rng = np.random.default_rng(77)
    b, sq, sk, h = 1, 256, 1152, 2
    q = rng.standard_normal((b, sq, h, 128), dtype=np.float32)
    k = rng.standard_normal((b, sk, h, 128), dtype=np.float32) * (1.0 + np.arange(sk, dtype=np.float32) / 48.0)[None, :, None, None]
    v = rng.standard_normal((b, sk, h, 128), dtype=np.float32)
    do = rng.standard_normal((b, sq, h, 128), dtype=np.float32)
    cast = (lambda x: x.astype(np.float16)) if dt == "f16" else O.f32_to_bf16
    _fwd_bwd_check(cast(q), cast(k), cast(v), cast(do), causal, (-1, -1), grad_atol_of_max=4e-3)


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("causal,window,sq,sk", [
    (False, (100, 50), 384, 384),   # local band, both sides bounded
    (True, (64, -1), 512, 512),     # sliding window: causal with a left bound
    (False, (-1, 30), 200, 456),    # right bound only, Sk > Sq (bottom-right aligned)
    (True, (-1, -1), 300, 200),     # Sk < Sq: the first 100 query rows see no key at all
    (False, (40, 0), 333, 210),     # left bound, ragged, rows without keys at both ends
])
def test_flash_attn_windows_and_rows_without_keys(causal, window, sq, sk, dt):
    rng = np.random.default_rng(sq + 3 * sk)
    b, h, hk = 1, 2, 1
    q, k, v = _mk(rng, (b, sq, h, 128), dt), _mk(rng, (b, sk, hk, 128), dt), _mk(rng, (b, sk, hk, 128), dt)
    do = _mk(rng, (b, sq, h, 128), dt)
    _fwd_bwd_check(q, k, v, do, causal, window)
