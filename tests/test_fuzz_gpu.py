"""Seeded random shapes through the four memory-bound families on the GPU, against the CPU oracle: the
dispatchers pick among several kernels by row size, alignment and grid (bulk-copy ring, tensor-map
gather, vector loads; one-wave, cluster and two-pass reductions; TMA and padded-tile transposes), and
the fixed cases of test_kernels_gpu.py sit at chosen points of that space.  These draw the points."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from test_kernels_gpu import _bits, _make, _to_dev, _to_host, _assert_max_equal

pytestmark = pytest.mark.gpu

DTYPES = ["f32", "f16", "bf16"]


@pytest.fixture(scope="module")
def ops():
    from byteir_b200 import ops as _ops
    return _ops


def _dim(rng, big):
    """a dimension: mostly small and odd, now and then a power of two or a large one"""
    k = rng.integers(0, 10)
    if k < 5:
        return int(rng.integers(1, 40))
    if k < 7:
        return int(2 ** rng.integers(0, 9))
    if k < 9:
        return int(rng.integers(40, 700))
    return int(rng.integers(700, big))


def _shape(rng, rank, limit):
    while True:
        shape = tuple(_dim(rng, 20000) for _ in range(rank))
        if 0 < int(np.prod(shape)) <= limit:
            return shape


@pytest.mark.parametrize("seed", range(60))
def test_reduce_random_shapes(ops, seed):
    rng = np.random.default_rng(7000 + seed)
    rank = int(rng.integers(1, 5))
    shape = _shape(rng, rank, 6_000_000)
    first = int(rng.integers(0, rank))
    last = int(rng.integers(first, rank))
    dims = list(range(first, last + 1))  # consecutive, as the reference's compiler emits them
    dt = DTYPES[seed % 3]
    op = "sum" if (seed // 3) % 2 == 0 else "max"
    x = _make(rng, shape, dt, "normal" if seed % 2 else "uniform")
    A = int(np.prod(shape[:first], dtype=np.int64))
    B = int(np.prod(shape[first:last + 1], dtype=np.int64))
    Cc = int(np.prod(shape[last + 1:], dtype=np.int64))
    xd = _to_dev(x)
    got = _to_host(ops.reduce_sum(xd, dims) if op == "sum" else ops.reduce_max(xd, dims)).reshape(-1)
    want = O.reduce(op, x, A, B, Cc)
    if op == "max":
        _assert_max_equal(got, want)
    else:
        ref = O.reduce_sum_f64(x, A, B, Cc)
        mag = np.abs(O.to_f32(x).astype(np.float64)).reshape(A, B, Cc).sum(axis=1).reshape(-1)
        g = O.to_f32(got).astype(np.float64)
        if dt == "f32":
            assert np.all(np.abs(g - ref) <= 1e-5 * mag + 1e-6)
        else:  # one rounding of the f32 sum to the 16-bit type
            ulp = 2.0 ** (-10 if dt == "f16" else -7)
            assert np.all(np.abs(g - ref) <= ulp * np.abs(ref) + 1e-5 * mag + 1e-6)


@pytest.mark.parametrize("seed", range(40))
def test_reduce_random_dims_that_are_not_consecutive(seed):
    """through a Session: the provider reduces groups of consecutive dimensions one after the other (the typed
    entry points take one A x B x C collapse, as the reference's launcher does)"""
    from test_brt_gpu import _run
    from test_brt_host import reduce_mlir
    rng = np.random.default_rng(7500 + seed)
    rank = int(rng.integers(3, 5))
    shape = _shape(rng, rank, 3_000_000)
    dims = tuple(sorted(rng.choice(rank, size=int(rng.integers(2, rank)), replace=False).tolist()))
    t, npdt = [("f32", np.float32), ("f16", np.float16)][seed % 2]
    x = rng.uniform(-1, 1, shape).astype(npdt)
    out_shape = tuple(s for i, s in enumerate(shape) if i not in dims)
    dims_s = "dense<[" + ", ".join(map(str, dims)) + f"]> : tensor<{len(dims)}xi64>"
    x64 = x.astype(np.float64)
    got_max = _run(reduce_mlir(f"ReduceMaxOp_{t}_{t}", t, shape, out_shape, dims_s), {"Input0": x})["Output0"]
    assert np.array_equal(got_max.reshape(-1), x.max(axis=dims).reshape(-1))  # no NaN, no zeros of two signs here
    got = _run(reduce_mlir(f"ReduceSumOp_{t}_{t}", t, shape, out_shape, dims_s), {"Input0": x})["Output0"]
    got = got.astype(np.float64).reshape(-1)
    ref = x64.sum(axis=dims).reshape(-1)
    mag = np.abs(x64).sum(axis=dims).reshape(-1)
    ulp = {"f32": 0.0, "f16": 2.0 ** -10}[t]
    assert np.all(np.abs(got - ref) <= ulp * np.abs(ref) + 1e-5 * mag + 1e-6)


@pytest.mark.parametrize("seed", range(60))
def test_index_select_random_shapes(ops, seed):
    rng = np.random.default_rng(8000 + seed)
    rank = int(rng.integers(1, 4))
    shape = _shape(rng, rank, 4_000_000)
    dim = int(rng.integers(0, rank))
    n = int(rng.integers(1, 5000))
    dt = DTYPES[seed % 3]
    x = _make(rng, shape, dt)
    idx = rng.integers(0, shape[dim], n)
    idx = idx.astype(np.int64) if seed % 2 else idx.astype(np.uint32)
    want, rc = O.index_select(x, idx.astype(np.int64), dim)
    assert rc == 0
    got = _to_host(ops.index_select(_to_dev(x), _to_dev(idx), dim))
    assert got.shape == want.shape
    assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("seed", range(40))
def test_index_put_add_random_shapes(ops, seed):
    rng = np.random.default_rng(9000 + seed)
    rows = int(rng.integers(1, 60000))
    feat = [1, 3, 8, 16, 24, 64, 100, 128, 136, 256, 512][int(rng.integers(0, 11))]
    n = int(rng.integers(1, 80000))
    dt = DTYPES[seed % 3]
    x = _make(rng, (rows, feat), dt, "normal")
    upd = _make(rng, (n, feat), dt, "normal")
    hot = rng.random() < 0.5
    idx = (rng.zipf(1.3, n) % rows if hot else rng.integers(0, rows, n)).astype(np.int64)
    want, rc = O.index_put_add(x, idx, upd)
    assert rc == 0
    xd, idd, ud = _to_dev(x), _to_dev(idx), _to_dev(upd)
    got = _to_host(ops.index_put_add(xd, idd, ud))
    again = _to_host(ops.index_put_add(xd, idd, ud))
    assert np.array_equal(_bits(got), _bits(again)), "not deterministic"
    g, w = O.to_f32(got).astype(np.float64), O.to_f32(want).astype(np.float64)
    # |sum of the row's updates| bounds the f32 rounding of a long run: tolerance relative to the row's magnitude
    mag = np.abs(O.to_f32(x).astype(np.float64))
    np.add.at(mag, idx, np.abs(O.to_f32(upd).astype(np.float64)))
    ulp = {"f32": 2.0 ** -22, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dt]
    assert np.all(np.abs(g - w) <= ulp * np.abs(w) + 2e-6 * mag + 1e-6)
    untouched = np.setdiff1d(np.arange(rows), idx)
    assert np.array_equal(_bits(got)[untouched], _bits(x)[untouched])
    inplace = xd.clone()
    ops.index_put_add(inplace, idd, ud, out=inplace)
    assert np.array_equal(_bits(_to_host(inplace)), _bits(got)), "in place differs"


@pytest.mark.parametrize("seed", range(80))
def test_transpose_random_shapes_and_permutations(ops, seed):
    rng = np.random.default_rng(10000 + seed)
    rank = int(rng.integers(2, 6))
    shape = _shape(rng, rank, 5_000_000)
    perm = tuple(int(p) for p in rng.permutation(rank))
    dt = DTYPES[seed % 3]
    x = _make(rng, shape, dt)
    want = O.transpose(x, perm)
    got = _to_host(ops.transpose(_to_dev(x), perm))
    assert got.shape == want.shape
    assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("seed", range(36))
def test_flash_attn_random_shapes_masks_and_head_dims(ops, seed):
    """forward and backward of the tcgen05 kernels on drawn shapes: ragged sequence lengths, Sq != Sk, grouped
    heads, head dims below 128, causal / sliding-window / no mask; tolerances of test_flash_attn_gpu.py"""
    from test_flash_attn_gpu import _dev, _host, _mk
    rng = np.random.default_rng(11000 + seed)
    b = int(rng.integers(1, 3))
    sq = int(rng.integers(1, 700))
    sk = sq if rng.random() < 0.4 else int(rng.integers(max(1, sq - 50), sq + 400))
    hk = int(rng.integers(1, 4))
    h = hk * int(rng.integers(1, 4))
    d = [128, 128, 64, 96, 32, 120, 8][int(rng.integers(0, 7))]
    dt = "bf16" if seed % 2 else "f16"
    mode = int(rng.integers(0, 4))
    causal, window = (mode == 1), (-1, -1)
    if mode == 2:
        window = (int(rng.integers(0, 300)), int(rng.integers(0, 200)))
    elif mode == 3:
        window = (int(rng.integers(0, 300)), 0)
    q, k, v = _mk(rng, (b, sq, h, d), dt), _mk(rng, (b, sk, hk, d), dt), _mk(rng, (b, sk, hk, d), dt)
    do = _mk(rng, (b, sq, h, d), dt)
    scale = float(1.0 / np.sqrt(d))
    want_o, want_lse = O.flash_attn_fwd(q, k, v, scale, causal, window=window)
    qd, kd, vd, dod = _dev(q), _dev(k), _dev(v), _dev(do)
    o, lse = ops.flash_attn_fwd(qd, kd, vd, scale, causal, window=window)
    dq, dk, dv = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal, window=window)
    torch.cuda.synchronize()
    gl = lse.cpu().numpy()
    seen = np.isfinite(want_lse)  # a row that sees no key: LSE = +inf in both, output zero
    assert np.array_equal(np.isfinite(gl), seen)
    np.testing.assert_allclose(gl[seen], want_lse[seen], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, _host(o), gl, scale, causal, window=window)
    for name, got, want in (("dq", dq, wq), ("dk", dk, wk), ("dv", dv, wv)):
        np.testing.assert_allclose(O.to_f32(_host(got)), O.to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)
    again = ops.flash_attn_bwd(dod, qd, kd, vd, o, lse, scale, causal, window=window)
    for a, b_ in zip(again, (dq, dk, dv)):
        assert torch.equal(a.view(torch.int16), b_.view(torch.int16)), "backward is not deterministic"


@pytest.mark.parametrize("seed", range(30))
def test_flash_attn_kvcache_random_shapes(ops, seed):
    """the decode step on drawn shapes: batch, rows in use per entry (empty to full), appended rows, query rows,
    heads per cache head, head dims on both kernels (tensor-core tiles for 64 / 128, the scalar kernel
    otherwise), causal / window / no mask"""
    from test_flash_attn_gpu import _dev, _host, _mk
    rng = np.random.default_rng(12000 + seed)
    b = int(rng.integers(1, 9))
    sq = int(rng.integers(1, 5))
    hk = int(rng.integers(1, 5))
    h = hk * [1, 1, 2, 4, 8][int(rng.integers(0, 5))]
    d = [128, 128, 64, 64, 32, 96, 256, 8][int(rng.integers(0, 8))]
    cap = int(rng.integers(8, 3000))
    s_new = int(rng.integers(0, min(cap, 5) + 1))
    dt = "bf16" if seed % 2 else "f16"
    mode = int(rng.integers(0, 3))
    causal, window = (mode == 0), (-1, -1)
    if mode == 2:
        window = (int(rng.integers(0, 400)), int(rng.integers(0, 4)))
    lens_h = None
    if rng.random() < 0.85 or s_new:
        lens_h = rng.integers(0, cap - s_new + 1, b).astype(np.int32)
        lens_h[rng.random(b) < 0.15] = 0
        lens_h[rng.random(b) < 0.15] = cap - s_new
    q = _mk(rng, (b, sq, h, d), dt)
    kc, vc = _mk(rng, (b, cap, hk, d), dt), _mk(rng, (b, cap, hk, d), dt)
    kn = _mk(rng, (b, s_new, hk, d), dt) if s_new else None
    vn = _mk(rng, (b, s_new, hk, d), dt) if s_new else None
    scale = float(1.0 / np.sqrt(d))
    want_k, want_v = kc.copy(), vc.copy()
    want_o, want_lse = O.flash_attn_kvcache(q, want_k, want_v, kn, vn, lens_h, scale, causal, window)
    kd, vd = _dev(kc), _dev(vc)
    o, lse = ops.flash_attn_kvcache(_dev(q), kd, vd, None if kn is None else _dev(kn), None if vn is None else _dev(vn),
                                    None if lens_h is None else torch.from_numpy(lens_h).cuda(), scale, causal, window)
    torch.cuda.synchronize()
    assert np.array_equal(_host(kd), want_k) and np.array_equal(_host(vd), want_v)
    gl = lse.cpu().numpy()
    assert np.array_equal(np.isinf(gl), np.isinf(want_lse))
    fin = np.isfinite(want_lse)
    np.testing.assert_allclose(gl[fin], want_lse[fin], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(_host(o)), O.to_f32(want_o), rtol=2e-2, atol=1e-2)
