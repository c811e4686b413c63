"""CPU tests of the oracle itself: the golden-vector pin and the known-answer
grid of the reference's own kernel tests."""
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as O

GOLDEN = Path(__file__).parent / "golden" / "flash_attn_b1_s128_h3_d32_f16.npz"


def _ulp_diff_f16(a, b):
    """distance in fp16 representable steps (monotone integer image of fp16)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7fff), u)
    return np.abs(key(a) - key(b))


# ---- golden pin: reference flash-attn vectors (b1 s128 h3 d32 fp16 causal, scale 0.5)
def test_flash_attn_fwd_matches_reference_golden():
    g = np.load(GOLDEN)
    out, _ = O.flash_attn_fwd(g["q"], g["k"], g["v"], 0.5, causal=True, round_p=True)
    ulp = _ulp_diff_f16(out, g["out"])
    # the reference test demands fp16-exact equality from the reference kernel;
    # the oracle sums in another order, so allow one fp16 step on a few elements
    assert ulp.max() <= 1, ulp.max()
    assert (ulp == 0).mean() > 0.97, (ulp == 0).mean()


def test_flash_attn_bwd_matches_reference_golden():
    g = np.load(GOLDEN)
    out, lse = O.flash_attn_fwd(g["q"], g["k"], g["v"], 0.5, causal=True)
    dq, dk, dv = O.flash_attn_bwd(g["dout"], g["q"], g["k"], g["v"], g["out"], lse, 0.5, causal=True)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        want = g[name]
        # the kernel that made the goldens rounds P and dS to fp16 before its
        # matmuls; stay within the build's stated tolerance for 16-bit outputs
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32),
                                   rtol=2e-2, atol=1e-2, err_msg=name)
        ulp = _ulp_diff_f16(got, want)
        assert np.median(ulp) <= 1, (name, np.median(ulp))


# ---- golden pin of the decode step: b2, cache of 128 rows with 64 in use, one new row
KV_GOLDEN = Path(__file__).parent / "golden" / "flash_attn_kvcache_b2_s128_h3_d32_f16.npz"


def test_flash_attn_kvcache_matches_reference_golden():
    g = np.load(KV_GOLDEN)
    kcache, vcache = g["kcache"].copy(), g["vcache"].copy()
    out, lse = O.flash_attn_kvcache(g["q"], kcache, vcache, g["k"], g["v"], g["cache_seqlens"], 0.5, causal=True)
    # the updated caches are copies of 16-bit values: exact
    assert np.array_equal(kcache, g["kcache_out"]) and np.array_equal(vcache, g["vcache_out"])
    ulp = _ulp_diff_f16(out, g["out"])
    assert ulp.max() <= 1, ulp.max()
    assert (ulp == 0).mean() > 0.9, (ulp == 0).mean()
    assert np.isfinite(lse).all()


def test_flash_attn_kvcache_equals_forward_on_the_rows_in_use():
    """ragged lengths, grouped heads, several query rows, a window; new rows that do not fit are dropped"""
    rng = np.random.default_rng(3)
    b, sq, h, hk, d, cap, s_new = 3, 2, 4, 2, 16, 40, 3
    q = rng.standard_normal((b, sq, h, d)).astype(np.float16)
    kc = rng.standard_normal((b, cap, hk, d)).astype(np.float16)
    vc = rng.standard_normal((b, cap, hk, d)).astype(np.float16)
    kn = rng.standard_normal((b, s_new, hk, d)).astype(np.float16)
    vn = rng.standard_normal((b, s_new, hk, d)).astype(np.float16)
    lens = np.array([0, 17, 38], np.int32)  # the last one has room for two of the three new rows
    for causal, window in ((True, (-1, -1)), (False, (-1, -1)), (False, (5, 1))):
        k2, v2 = kc.copy(), vc.copy()
        out, lse = O.flash_attn_kvcache(q, k2, v2, kn, vn, lens, 0.3, causal=causal, window=window)
        for i in range(b):
            n = min(int(lens[i]) + s_new, cap)
            kk = np.concatenate([kc[i, :lens[i]], kn[i, :n - lens[i]]])[None]
            vv = np.concatenate([vc[i, :lens[i]], vn[i, :n - lens[i]]])[None]
            assert np.array_equal(k2[i, :n], kk[0]) and np.array_equal(k2[i, n:], kc[i, n:])
            assert np.array_equal(v2[i, :n], vv[0]) and np.array_equal(v2[i, n:], vc[i, n:])
            want, want_lse = O.flash_attn_fwd(q[i:i + 1], kk, vv, 0.3, causal=causal, window=window)
            assert np.array_equal(out[i:i + 1], want)
            np.testing.assert_array_equal(lse[i:i + 1], want_lse)


def test_flash_attn_fwd_vs_numpy_noncausal_gqa():
    rng = np.random.default_rng(7)
    q = rng.standard_normal((2, 40, 4, 16)).astype(np.float16)
    k = rng.standard_normal((2, 56, 2, 16)).astype(np.float16)
    v = rng.standard_normal((2, 56, 2, 16)).astype(np.float16)
    out, lse = O.flash_attn_fwd(q, k, v, 0.25, causal=False)
    kk = np.repeat(k, 2, axis=2).astype(np.float64)
    vv = np.repeat(v, 2, axis=2).astype(np.float64)
    s = np.einsum("bihd,bjhd->bhij", q.astype(np.float64), kk) * 0.25
    m = s.max(-1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(-1, keepdims=True)
    ref = np.einsum("bhij,bjhd->bihd", p / l, vv)
    np.testing.assert_allclose(out.astype(np.float64), ref, rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(lse, (m + np.log(l))[..., 0], rtol=1e-5, atol=1e-5)


def test_flash_attn_bwd_vs_finite_difference():
    rng = np.random.default_rng(11)
    b, s, h, d = 1, 12, 2, 8
    q, k, v, do = (rng.standard_normal((b, s, h, d)).astype(np.float32) for _ in range(4))

    def fwd(q, k, v):
        return O.flash_attn_fwd(q, k, v, 0.3, causal=True)

    out, lse = fwd(q, k, v)
    dq, dk, dv = O.flash_attn_bwd(do, q, k, v, out, lse, 0.3, causal=True)
    eps = 1e-2
    for name, x, g in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        for idx in [(0, 3, 1, 2), (0, 11, 0, 7), (0, 0, 1, 0)]:
            xp, xm = x.copy(), x.copy()
            xp[idx] += eps
            xm[idx] -= eps
            args_p = dict(q=q, k=k, v=v); args_p[name] = xp
            args_m = dict(q=q, k=k, v=v); args_m[name] = xm
            fd = ((fwd(**args_p)[0] - fwd(**args_m)[0]) * do).sum() / (2 * eps)
            assert abs(fd - g[idx]) < 2e-3 + 2e-2 * abs(fd), (name, idx, fd, g[idx])


# ---- reductions: grid of kernel/reduction_test.cc:171-180
RED_CASES = [((1, 16, 32), d) for d in ([0], [1], [2], [0, 1], [0, 2])] + [
    ((1, 128, 128), [0, 1]), ((2, 128, 256), [0, 1]), ((2, 16, 8, 64), [1, 2])]


@pytest.mark.parametrize("shape,dims", RED_CASES)
@pytest.mark.parametrize("op", ["sum", "max"])
def test_reduce_grid(shape, dims, op):
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    A, B, Cc = O.reduce_abc(shape, dims)
    got = O.reduce(op, x, A, B, Cc)
    want = (x.astype(np.float64).sum if op == "sum" else x.max)(axis=tuple(dims)).reshape(-1)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4 if op == "sum" else 0)


def test_reduce_max_rules():
    nan = np.float32("nan")
    x = np.array([[1, nan, 3, 2], [-0.0, 0.0, -1, -0.0], [0.0, -0.0, -5, -7], [-3, -3, -3, -3]], np.float32)
    got = O.reduce("max", x, 4, 4, 1)
    assert np.isnan(got[0])
    assert got[1] == 0 and np.signbit(got[1])      # last of the equal zeros is -0
    assert got[2] == 0 and np.signbit(got[2])
    assert got[3] == -3
    h = x.astype(np.float16)
    goth = O.reduce("max", h, 4, 4, 1)
    assert np.isnan(goth[0]) and np.signbit(goth[1]) and goth[3] == -3
    # NaN over 1024 elements, reduction_test.cc:182-215
    y = np.random.default_rng(0).uniform(-1, 1, 1024).astype(np.float32)
    y[517] = nan
    assert np.isnan(O.reduce("max", y, 1, 1024, 1)[0])
    assert np.isnan(O.reduce("sum", y, 1, 1024, 1)[0])


def test_reduce_sum_f16_single_rounding():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 33, 7)).astype(np.float16)
    got = O.reduce("sum", x, 1, 64 * 33, 7)
    want = x.astype(np.float64).reshape(-1, 7).sum(0).astype(np.float16)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


# ---- index ops: shapes of kernel/index_test.cc:300-331
@pytest.mark.parametrize("shape,dim,n", [((2, 3, 4, 5), 0, 7), ((2, 3, 4, 5), 1, 3), ((2, 3, 4, 5), 2, 9),
                                         ((2, 3, 4, 5), 3, 4), ((256, 64, 128), 1, 100), ((30522, 128), 0, 128)])
@pytest.mark.parametrize("idt", [np.int64, np.uint32])
def test_index_select(shape, dim, n, idt):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(shape).astype(np.float32)
    idx = rng.integers(0, shape[dim], n).astype(idt)
    got, rc = O.index_select(x, idx, dim)
    assert rc == 0
    assert np.array_equal(got, np.take(x, idx.astype(np.int64), axis=dim))


def test_index_select_out_of_range_is_refused():
    x = np.zeros((4, 2), np.float32)
    _, rc = O.index_select(x, np.array([0, 4], np.int64), 0)
    assert rc == -1


@pytest.mark.parametrize("shape,n", [((3, 2), 5), ((256, 128), 128 * 32), ((30522, 128), 128)])
def test_index_put_add(shape, n):
    rng = np.random.default_rng(2)
    x = rng.standard_normal(shape).astype(np.float32)
    idx = rng.integers(0, shape[0], n)
    upd = rng.standard_normal((n,) + shape[1:]).astype(np.float32)
    got, rc = O.index_put_add(x, idx, upd)
    assert rc == 0
    want = x.astype(np.float64)
    np.add.at(want, idx, upd.astype(np.float64))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    seq, _ = O.index_put_add_seq_f32(x, idx, upd)
    np.testing.assert_allclose(seq, want, rtol=1e-5, atol=1e-5)


def test_index_put_add_f16_heavy_duplicates():
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((50, 8)) * 0.02).astype(np.float16)
    idx = np.minimum((rng.zipf(1.1, 4000) - 1), 49)
    upd = rng.standard_normal((4000, 8)).astype(np.float16)
    got, _ = O.index_put_add(x, idx, upd)
    want = x.astype(np.float64)
    np.add.at(want, idx, upd.astype(np.float64))
    assert np.array_equal(got.view(np.uint16), want.astype(np.float16).view(np.uint16))


# ---- transpose: shapes of kernel/transpose_test.cc:152-168
@pytest.mark.parametrize("shape,perm", [((32, 64), (1, 0)), ((1000, 512), (1, 0)),
                                        ((10, 20, 30, 40), (0, 2, 3, 1)), ((10, 20, 30, 40), (0, 3, 1, 2)),
                                        ((3, 5, 7), (2, 0, 1))])
@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_transpose(shape, perm, dt):
    x = np.random.default_rng(6).uniform(-1, 1, shape).astype(dt)
    assert np.array_equal(O.transpose(x, perm), np.transpose(x, perm))


TRANSPOSE_GOLDENS = ["transpose_f32_1x32x64x64_perm0231.npz", "transpose_f32_1x3x224x224_perm0231.npz"]


def transpose_golden(name):
    """input and output of the reference's own CPU code for f32 [1, C, H, W] -> (0, 2, 3, 1): its compiler's
    LLVM IR (runtime/test/test_files/LLJIT/transpose_{32_64_64,3_224_224}.ll) run by
    tests/golden/make_transpose_llvm_golden.py"""
    g = np.load(Path(__file__).parent / "golden" / name)
    shape, perm = tuple(int(v) for v in g["shape"]), tuple(int(v) for v in g["perm"])
    x = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)
    out = np.cumsum(g["delta"].astype(np.int64)).astype(np.float32).reshape([shape[p] for p in perm])
    return x, perm, out


@pytest.mark.parametrize("name", TRANSPOSE_GOLDENS)
def test_transpose_matches_the_references_compiled_cpu_code(name):
    x, perm, want = transpose_golden(name)
    assert np.array_equal(O.transpose(x, perm).view(np.uint32), want.view(np.uint32))


def test_bf16_conversion_round_trip():
    x = np.random.default_rng(8).standard_normal(10000).astype(np.float32)
    b = O.f32_to_bf16(x)
    back = O.bf16_to_f32(b)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2 ** -8)
    assert np.array_equal(O.f32_to_bf16(back), b)
