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


# The configuration the benchmark times: S = 4096, D = 128, causal, bf16 (32 x 32 tiles per (batch, head), every
# ring of the forward and of both backward passes wraps many times), on slices the oracle finishes in seconds.
FULL_SEQ_CASES = [
    # b, sq, sk, h, hk, causal
    (1, 4096, 4096, 2, 2, True),
    (1, 4096, 4096, 4, 1, True),     # grouped heads: four query heads on one key/value head
    (1, 4096, 4224, 2, 2, False),    # no mask, Sk > Sq: 33 key tiles for every query tile
]


@pytest.mark.parametrize("b,sq,sk,h,hk,causal", FULL_SEQ_CASES)
def test_flash_attn_fwd_bwd_at_benchmark_sequence_length(b, sq, sk, h, hk, causal):
    from byteir_b200 import ops
    dt = "bf16"
    rng = np.random.default_rng(sq + sk + h * 13)
    q, k, v = _mk(rng, (b, sq, h, 128), dt), _mk(rng, (b, sk, hk, 128), dt), _mk(rng, (b, sk, hk, 128), dt)
    do = _mk(rng, (b, sq, h, 128), dt)
    scale = 1.0 / np.sqrt(128.0)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    want_o, want_lse = O.flash_attn_fwd(q, k, v, scale, causal)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, causal)
    dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal)
    torch.cuda.synchronize()
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o), lse.cpu().numpy(), scale, causal)
    for name, got, want in (("dq", dq, wq), ("dk", dk, wk), ("dv", dv, wv)):
        np.testing.assert_allclose(O.to_f32(_host(got)), O.to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)
    o2, lse2 = ops.flash_attn_fwd(qd, kd, vd, scale, causal)
    again = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal)
    assert torch.equal(o2.view(torch.int16), o.view(torch.int16)) and torch.equal(lse2, lse)
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


# ---- decode step over a key/value cache -------------------------------------------------------------
KV_GOLDEN = __import__("pathlib").Path(__file__).parent / "golden" / "flash_attn_kvcache_b2_s128_h3_d32_f16.npz"


def test_flash_attn_kvcache_reference_golden():
    """the vectors of the reference's own kv-cache test (flash_attn_fwd_test.cc:183-330): output and
    both updated caches"""
    from byteir_b200 import ops
    g = np.load(KV_GOLDEN)
    kc, vc = _dev(g["kcache"].copy()), _dev(g["vcache"].copy())
    lens = torch.from_numpy(g["cache_seqlens"]).cuda()
    o, lse = ops.flash_attn_kvcache(_dev(g["q"]), kc, vc, _dev(g["k"]), _dev(g["v"]), lens, 0.5, causal=True)
    torch.cuda.synchronize()
    assert np.array_equal(_host(kc), g["kcache_out"]) and np.array_equal(_host(vc), g["vcache_out"])
    got, want = _host(o), g["out"]
    key = lambda x: np.where(x.view(np.uint16) & 0x8000, -(x.view(np.uint16).astype(np.int32) & 0x7fff),
                             x.view(np.uint16).astype(np.int32))
    assert np.abs(key(got) - key(want)).max() <= 1
    assert torch.isfinite(lse).all()


KV_CASES = [
    # b, sq, h, hk, d, capacity, new rows, causal, window, lengths ("full" = no length tensor)
    (2, 1, 8, 8, 128, 4096, 1, True, (-1, -1), [4000, 77]),            # one query row per head, many splits
    (4, 1, 32, 4, 128, 2048, 1, True, (-1, -1), [2047, 0, 1000, 513]),   # eight heads share a cache head
    (1, 1, 4, 4, 64, 8192, 1, False, (-1, -1), [8191]),                # the most splits
    (3, 5, 6, 2, 96, 300, 4, True, (-1, -1), [296, 10, 0]),            # several query rows, 12 of 16 lanes active
    (2, 3, 4, 4, 256, 700, 0, True, (-1, -1), [700, 1]),               # nothing appended, widest head
    (2, 2, 4, 2, 32, 500, 2, True, (100, 0), [498, 250]),              # sliding window
    (2, 2, 4, 2, 32, 500, 2, False, (64, 3), [499, 30]),               # window on both sides; one new row dropped
    (2, 1, 2, 2, 128, 256, 0, True, (-1, -1), "full"),                 # no length tensor: the whole cache
    (2, 4, 2, 1, 128, 64, 0, True, (-1, -1), [0, 2]),                  # rows that see no key at all
    (1, 1, 128, 8, 128, 16384, 1, True, (-1, -1), [16000]),            # 16 heads per cache head: a full row tile
    (2, 3, 16, 2, 64, 1000, 3, True, (-1, -1), [997, 5]),              # 24 rows per cache head: two row chunks
    (2, 2, 8, 2, 128, 700, 2, True, (100, 0), [698, 300]),             # sliding window on the tensor-core path
    (2, 2, 8, 2, 64, 700, 2, False, (30, 5), [690, 0]),                # window on both sides, head dim 64
    (3, 7, 4, 4, 128, 50, 7, True, (-1, -1), [43, 0, 20]),             # more new rows than a block step of the append
    (8, 1, 8, 2, 128, 4096, 1, True, (-1, -1), [4000, 3, 0, 10, 1, 0, 7, 2]),  # one entry holds nearly all the keys
    (150, 1, 4, 2, 64, 300, 1, True, (-1, -1), "ragged"),              # more batch entries than threads in a block
]


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("b,sq,h,hk,d,cap,s_new,causal,window,lens", KV_CASES)
def test_flash_attn_kvcache(b, sq, h, hk, d, cap, s_new, causal, window, lens, dt):
    from byteir_b200 import ops
    rng = np.random.default_rng(cap + d + h)
    q = _mk(rng, (b, sq, h, d), dt)
    kc, vc = _mk(rng, (b, cap, hk, d), dt), _mk(rng, (b, cap, hk, d), dt)
    kn = _mk(rng, (b, s_new, hk, d), dt) if s_new else None
    vn = _mk(rng, (b, s_new, hk, d), dt) if s_new else None
    if lens == "ragged":  # from empty to full, a quarter of them empty
        lens = [0 if i % 4 == 1 else int(v) for i, v in enumerate(rng.integers(0, cap - s_new + 1, b))]
    lens_h = None if lens == "full" else np.array(lens, np.int32)
    scale = 1.0 / np.sqrt(d)
    want_k, want_v = kc.copy(), vc.copy()
    want_o, want_lse = O.flash_attn_kvcache(q, want_k, want_v, kn, vn, lens_h, scale, causal, window)
    kd, vd = _dev(kc), _dev(vc)
    o, lse = ops.flash_attn_kvcache(_dev(q), kd, vd, None if kn is None else _dev(kn),
                                    None if vn is None else _dev(vn),
                                    None if lens_h is None else torch.from_numpy(lens_h).cuda(),
                                    scale, causal, window)
    torch.cuda.synchronize()
    assert np.array_equal(_host(kd), want_k) and np.array_equal(_host(vd), want_v)
    gl = lse.cpu().numpy()
    assert np.array_equal(np.isinf(gl), np.isinf(want_lse))
    fin = np.isfinite(want_lse)
    np.testing.assert_allclose(gl[fin], want_lse[fin], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)


def test_flash_attn_kvcache_caller_workspace_and_strided_cache():
    """a caller-provided workspace, and caches that are views into a larger allocation"""
    from byteir_b200 import ops, _native as N
    import ctypes as C
    rng = np.random.default_rng(5)
    b, h, d, cap = 2, 4, 128, 3000
    q = _mk(rng, (b, 1, h, d), "f16")
    big_k, big_v = _mk(rng, (b, cap, h, 2 * d), "f16"), _mk(rng, (b, cap, h, 2 * d), "f16")
    kn, vn = _mk(rng, (b, 1, h, d), "f16"), _mk(rng, (b, 1, h, d), "f16")
    lens = np.array([2999, 1500], np.int32)
    want_k, want_v = np.ascontiguousarray(big_k[..., d:]), np.ascontiguousarray(big_v[..., :d])
    want_o, want_lse = O.flash_attn_kvcache(q, want_k, want_v, kn, vn, lens, 0.09, True)
    bk, bv = _dev(big_k), _dev(big_v)
    kd, vd = bk[..., d:], bv[..., :d]
    qd = _dev(q)
    out = torch.empty_like(qd)
    p = ops.kvcache_params(qd, kd, vd, _dev(kn), _dev(vn), out, 0.09, True)
    need = N.lib().b200_flash_attn_kvcache_workspace_bytes(C.byref(p))
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    o, lse = ops.flash_attn_kvcache(qd, kd, vd, _dev(kn), _dev(vn), torch.from_numpy(lens).cuda(), 0.09, True,
                                    out=out, workspace=ws)
    torch.cuda.synchronize()
    assert np.array_equal(_host(kd.contiguous()), want_k) and np.array_equal(_host(vd.contiguous()), want_v)
    # the halves of the large allocation next to the caches are untouched
    assert np.array_equal(_host(bk[..., :d].contiguous()), big_k[..., :d])
    assert np.array_equal(_host(bv[..., d:].contiguous()), big_v[..., d:])
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
    with pytest.raises(Exception):
        ops.flash_attn_kvcache(qd, kd, vd, None, None, None, 0.09, True, workspace=ws[:64])


# ---- bounded waits and the status word -------------------------------------------------------------
@pytest.mark.parametrize("which", ["fwd", "bwd"])
def test_flash_attn_wait_that_runs_out_sets_the_status_word(which):
    """The elementwise warps leave out one arrival (a flag that nothing sets) and the waits get a short
    limit: the kernel must end by itself, report 2 (forward) or 3 (backward) through the sticky status
    word, and the next call on the same context must work and leave the word at zero."""
    import ctypes as C
    from byteir_b200 import ops, _native as N
    lib = N.lib()
    rng = np.random.default_rng(5)
    q, k, v, do = (_mk(rng, (1, 256, 2, 128), "bf16") for _ in range(4))
    scale = 1.0 / np.sqrt(128.0)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, True)
    torch.cuda.synchronize()
    st = C.c_int(-1)
    assert lib.b200_flash_attn_take_status(C.byref(st)) == 0 and st.value == 0
    try:
        lib.b200_flash_attn_debug(1, 50)  # 50 polls of at most 20 us per wait
        if which == "fwd":
            ops.flash_attn_fwd(qd, kd, vd, scale, True)
        else:
            ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, True)
        torch.cuda.synchronize()
    finally:
        lib.b200_flash_attn_debug(0, 0)
    assert lib.b200_flash_attn_take_status(C.byref(st)) == 0
    assert st.value == (2 if which == "fwd" else 3)
    # the context is intact and the word was cleared by the read
    o2, lse2 = ops.flash_attn_fwd(qd, kd, vd, scale, True)
    dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o2, lse2, scale, True)
    torch.cuda.synchronize()
    assert torch.equal(o2.view(torch.int16), o.view(torch.int16))
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o2), lse2.cpu().numpy(), scale, True)
    np.testing.assert_allclose(O.to_f32(_host(dq)), O.to_f32(wq), rtol=2e-2, atol=1e-2)
    assert lib.b200_flash_attn_take_status(C.byref(st)) == 0 and st.value == 0


def test_kernels_with_large_shared_memory_on_a_second_device():
    """The dynamic shared-memory limit of a kernel is a per-device attribute: every entry point that needs
    more than 48 KiB must work with any device current, not only the first one a process used."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from byteir_b200 import ops
    rng = np.random.default_rng(6)
    q, k, v, do = (_mk(rng, (1, 256, 2, 128), "bf16") for _ in range(4))
    scale = 1.0 / np.sqrt(128.0)
    want_o, _ = O.flash_attn_fwd(q, k, v, scale, True)
    table = rng.standard_normal((4096, 512), dtype=np.float32)
    idx = rng.integers(0, 4096, 3000).astype(np.int64)
    for dev in (0, 1):
        with torch.cuda.device(dev):
            to = lambda a: _dev(a).to(f"cuda:{dev}")
            o, lse = ops.flash_attn_fwd(to(q), to(k), to(v), scale, True)
            dq, dk, dv = ops.flash_attn_bwd(to(do), to(q), to(k), to(v), o, lse, scale, True)
            g = ops.index_select(torch.from_numpy(table).to(f"cuda:{dev}"), torch.from_numpy(idx).to(f"cuda:{dev}"), 0)
            torch.cuda.synchronize()
            np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
            assert np.array_equal(g.cpu().numpy(), table[idx])


# ---- head dims below 128, and the reference's own vectors on the training kernels ---------------------------
GOLDEN = __import__("pathlib").Path(__file__).parent / "golden" / "flash_attn_b1_s128_h3_d32_f16.npz"


def _ulp_f16(a, b):
    key = lambda x: np.where(x.view(np.uint16) & 0x8000, -(x.view(np.uint16).astype(np.int32) & 0x7fff),
                             x.view(np.uint16).astype(np.int32))
    return np.abs(key(a) - key(b))


def test_flash_attn_training_kernels_on_the_reference_golden_vectors():
    """b1 s128 h3 d32 fp16 causal scale 0.5 (flash_attn_fwd_test.cc / flash_attn_bwd_test.cc): the forward within one
    fp16 step of the reference's output, the gradients within the 16-bit tolerance and a median distance of at most
    one fp16 step"""
    from byteir_b200 import ops
    g = np.load(GOLDEN)
    q, k, v, do = (_dev(g[n]) for n in ("q", "k", "v", "dout"))
    o, lse = ops.flash_attn_fwd(q, k, v, 0.5, True)
    torch.cuda.synchronize()
    ulp = _ulp_f16(_host(o), g["out"])
    assert ulp.max() <= 1 and (ulp == 0).mean() > 0.95, (ulp.max(), (ulp == 0).mean())
    dq, dk, dv = ops.flash_attn_bwd(do, q, k, v, _dev(g["out"]), lse, 0.5, True)
    torch.cuda.synchronize()
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        np.testing.assert_allclose(_host(got).astype(np.float32), g[name].astype(np.float32), rtol=2e-2, atol=1e-2,
                                   err_msg=name)
        assert np.median(_ulp_f16(_host(got), g[name])) <= 1, name


@pytest.mark.parametrize("dt", ["bf16", "f16"])
@pytest.mark.parametrize("d", [32, 64, 96, 8, 120])
@pytest.mark.parametrize("b,sq,sk,h,hk,causal", [(2, 300, 300, 4, 2, True), (1, 384, 640, 2, 2, False)])
def test_flash_attn_head_dims_below_128(b, sq, sk, h, hk, causal, d, dt):
    from byteir_b200 import ops
    rng = np.random.default_rng(d + sq)
    q, k, v = _mk(rng, (b, sq, h, d), dt), _mk(rng, (b, sk, hk, d), dt), _mk(rng, (b, sk, hk, d), dt)
    do = _mk(rng, (b, sq, h, d), dt)
    scale = 1.0 / np.sqrt(d)
    want_o, want_lse = O.flash_attn_fwd(q, k, v, scale, causal)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, causal)
    dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal)
    torch.cuda.synchronize()
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o), lse.cpu().numpy(), scale, causal)
    for name, got, want in (("dq", dq, wq), ("dk", dk, wk), ("dv", dv, wv)):
        np.testing.assert_allclose(O.to_f32(_host(got)), O.to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)
