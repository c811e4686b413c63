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
