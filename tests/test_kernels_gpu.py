"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the
CPU oracle on the same seeded inputs.  Bit-exact for max / gather / transpose;
stated tolerances for sums."""
import numpy as np
import pytest
import torch

import oracle_lib as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from byteir_b200 import ops as _ops
    return _ops


def _to_dev(a):
    if a.dtype == np.uint16:  # bf16 bits
        return torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def _to_host(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def _make(rng, shape, dt, dist="uniform"):
    x = rng.uniform(-1, 1, shape) if dist == "uniform" else rng.standard_normal(shape)
    x = x.astype(np.float32)
    if dt == "f32":
        return x
    if dt == "f16":
        return x.astype(np.float16)
    return O.f32_to_bf16(x)


def _bits(a):
    return a.view({2: np.uint16, 4: np.uint32}[a.itemsize])


def _assert_max_equal(got, want):
    gf, wf = O.to_f32(got), O.to_f32(want)
    nan = np.isnan(wf)
    assert np.array_equal(np.isnan(gf), nan)
    assert np.array_equal(_bits(got)[~nan], _bits(want)[~nan])


# ---------------------------------------------------------------- reductions
RED_CASES = [((1, 16, 32), d) for d in ([0], [1], [2], [0, 1], [0, 2])] + [
    ((1, 128, 128), [0, 1]), ((2, 128, 256), [0, 1]), ((2, 16, 8, 64), [1, 2]),  # reduction_test.cc:171-180
    ((7, 33, 5), [1]), ((3, 1000), [1]), ((5, 4099), [1]), ((40, 70000), [1]),    # ragged / unaligned
    ((2, 300000), [1]), ((1, 3000000), [1]),                                       # cluster and two-pass rows
    ((4096, 3), [0]), ((1000, 17), [0]), ((6, 50, 36), [1]), ((9, 2048), [0]),     # narrow / odd columns
    ((1024, 4096), [1]),                                                           # config 1
]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("op", ["sum", "max"])
@pytest.mark.parametrize("shape,dims", RED_CASES)
def test_reduce(ops, shape, dims, op, dt):
    rng = np.random.default_rng(hash((shape, tuple(dims))) % 2**32)
    x = _make(rng, shape, dt)
    A, B, C = O.reduce_abc(shape, dims)
    want = O.reduce(op, x, A, B, C)
    fn = ops.reduce_sum if op == "sum" else ops.reduce_max
    for _ in range(2):  # the reference tests run every op twice on one context
        got = _to_host(fn(_to_dev(x), dims)).reshape(-1)
    if A == 0 and B == 0:  # only size-1 dims named: nothing to reduce, a copy
        assert np.array_equal(_bits(got), _bits(want))
    elif op == "max":
        _assert_max_equal(got, want)
    else:
        g, w = O.to_f32(got).astype(np.float64), O.to_f32(want).astype(np.float64)
        if dt == "f32":
            # rel 1e-5 of the row's magnitude scale (sum of |x|), the usual bound for f32 trees
            scale = O.reduce_sum_f64(np.abs(O.to_f32(x)), A, B, C)
            assert np.all(np.abs(g - w) <= 1e-5 * np.maximum(np.abs(w), 1e-2 * scale) + 1e-6)
        else:
            np.testing.assert_allclose(g, w, rtol=2e-2, atol=1e-2)


def test_reduce_max_zero_sign_and_nan(ops):
    rng = np.random.default_rng(5)
    for dt in ("f32", "f16", "bf16"):
        # rows whose maximum is a zero: the sign of the last zero must survive
        x = -np.abs(rng.standard_normal((64, 1024)).astype(np.float32)) - 0.5
        for r in range(64):
            pos = rng.integers(0, 1024, 6)
            x[r, pos] = np.where(rng.random(6) < 0.5, 0.0, -0.0)
        x[3, :] = 0.0
        x[4, :] = -0.0
        x[5, 100] = np.nan
        x[6, 0] = np.nan
        xs = x if dt == "f32" else (x.astype(np.float16) if dt == "f16" else O.f32_to_bf16(x))
        for shape, dims in (((64, 1024), [1]), ((64, 1024), [0]), ((8, 8, 1024), [1]), ((1, 65536), [1])):
            xv = xs.reshape(shape)
            A, B, C = O.reduce_abc(shape, dims)
            want = O.reduce("max", xv, A, B, C)
            got = _to_host(ops.reduce_max(_to_dev(xv), dims)).reshape(-1)
            _assert_max_equal(got, want)


def test_reduce_sum_nan_propagates(ops):
    x = np.random.default_rng(0).uniform(-1, 1, 1024).astype(np.float32)
    x[517] = np.nan  # reduction_test.cc:182-215
    assert np.isnan(_to_host(ops.reduce_sum(_to_dev(x.reshape(1, 1024)), [1]))[0])
    assert np.isnan(_to_host(ops.reduce_max(_to_dev(x.reshape(1, 1024)), [1]))[0])


def test_reduce_nothing_to_reduce_is_a_copy(ops):
    x = _make(np.random.default_rng(1), (1, 37, 5), "f16")
    got = _to_host(ops.reduce_sum(_to_dev(x), [0]))
    assert np.array_equal(_bits(got).reshape(-1), _bits(x).reshape(-1))


def test_reduce_config2_f16_multi_axis(ops):
    """[64, 512, 1024] f16 N(0,1): sum over {0,1} (f32 accumulate) and max over {2} (bit-exact)."""
    rng = np.random.default_rng(1234 + 1)
    x = rng.standard_normal((64, 512, 1024), dtype=np.float32).astype(np.float16)
    xd = _to_dev(x)
    got = _to_host(ops.reduce_sum(xd, [0, 1])).astype(np.float64)
    want = O.reduce("sum", x, 1, 64 * 512, 1024).astype(np.float64)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=1e-2)
    # the f32 partial the multi-device path exchanges agrees with f64 to f32 accuracy
    part = _to_host(ops.reduce_sum_to_f32(xd, [0, 1])).astype(np.float64)
    ref64 = O.reduce_sum_f64(x, 1, 64 * 512, 1024)
    assert np.abs(part - ref64).max() <= 1e-5 * np.abs(x.astype(np.float64)).sum(axis=(0, 1)).max()
    gm = _to_host(ops.reduce_max(xd, [2])).reshape(-1)
    wm = O.reduce("max", x, 64 * 512, 1024, 1)
    assert np.array_equal(_bits(gm), _bits(wm))


@pytest.mark.parametrize("reserve", [1, 5])
def test_reduce_with_block_slots_left_free(ops, reserve):
    """b200_reduce_reserve_blocks: the one-wave grids leave room for a kernel that runs beside them; the column
    sum (its split of the reduced axis follows the grid) stays within tolerance, the row max bit-exact"""
    from byteir_b200 import _native as N
    rng = np.random.default_rng(31)
    x = rng.standard_normal((64, 512, 1024), dtype=np.float32).astype(np.float16)
    x32 = rng.uniform(-1, 1, (1024, 4096)).astype(np.float32)
    xd, x32d = _to_dev(x), _to_dev(x32)
    full = _to_host(ops.reduce_max(xd, [2]))
    try:
        N.lib().b200_reduce_reserve_blocks(reserve)
        got = _to_host(ops.reduce_sum(xd, [0, 1])).astype(np.float64)
        part = _to_host(ops.reduce_sum_to_f32(xd, [0, 1])).astype(np.float64)
        gm = _to_host(ops.reduce_max(xd, [2]))
        rows = _to_host(ops.reduce_sum(x32d, [1])).astype(np.float64)
    finally:
        N.lib().b200_reduce_reserve_blocks(0)
    want = O.reduce("sum", x, 1, 64 * 512, 1024).astype(np.float64)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=1e-2)
    ref64 = O.reduce_sum_f64(x, 1, 64 * 512, 1024)
    assert np.abs(part - ref64).max() <= 1e-5 * np.abs(x.astype(np.float64)).sum(axis=(0, 1)).max()
    assert np.array_equal(_bits(gm), _bits(full))
    np.testing.assert_allclose(rows, x32.astype(np.float64).sum(axis=1), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("op", ["sum", "max"])
@pytest.mark.parametrize("shape", [(64 * 512, 1024), (20000, 96), (3, 9000, 40), (100000, 7)])
def test_reduce_columns_every_slab_width(ops, shape, op, dt):
    """The column plan may give a slab 4 to 32 threads per row: every width agrees with the oracle
    (max bit for bit, sums within the stated tolerance) and is deterministic."""
    from byteir_b200 import _native as N
    rng = np.random.default_rng(31)
    x = _make(rng, shape, dt, "normal")
    dims = [len(shape) - 2]
    fn = ops.reduce_sum if op == "sum" else ops.reduce_max
    xd = _to_dev(x)
    A, B, C = O.reduce_abc(shape, dims)
    want = O.reduce(op, x, A, B, C)
    try:
        for lpr in (0, 32, 16, 8, 4):
            N.lib().b200_reduce_cols_plan_override(lpr)
            got = _to_host(fn(xd, dims)).reshape(-1)
            again = _to_host(fn(xd, dims)).reshape(-1)
            nan = np.isnan(O.to_f32(got))
            assert np.array_equal(_bits(got)[~nan], _bits(again)[~nan])
            if op == "max":
                _assert_max_equal(got, want)
            else:
                np.testing.assert_allclose(O.to_f32(got).astype(np.float64), O.to_f32(want).astype(np.float64),
                                           rtol=2e-2 if dt != "f32" else 1e-5, atol=1e-2 if dt != "f32" else 2e-4)
    finally:
        N.lib().b200_reduce_cols_plan_override(0)


def test_reduce_sum_sharded_partials_then_single_rounding(ops):
    """dim-0 sharding: f32 partials of the shards, summed, rounded once == unsharded result."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((8, 64, 256), dtype=np.float32).astype(np.float16)
    xd = _to_dev(x)
    whole = _to_host(ops.reduce_sum(xd, [0, 1]))
    parts = [ops.reduce_sum_to_f32(xd[i * 2:(i + 1) * 2].contiguous(), [0, 1]) for i in range(4)]
    total = parts[0] + parts[1] + parts[2] + parts[3]
    sharded = _to_host(ops.cast_from_f32(total, torch.float16))
    want = O.reduce("sum", x, 1, 8 * 64, 256)
    np.testing.assert_allclose(sharded.astype(np.float64), want.astype(np.float64), rtol=2e-3, atol=1e-3)
    np.testing.assert_allclose(sharded.astype(np.float64), whole.astype(np.float64), rtol=2e-3, atol=1e-3)


# ---------------------------------------------------------------- gather
SEL_CASES = [((2, 3, 4, 5), 0, 7), ((2, 3, 4, 5), 1, 3), ((2, 3, 4, 5), 2, 9), ((2, 3, 4, 5), 3, 4),
             ((256, 64, 128), 1, 100), ((30522, 128), 0, 128),  # index_test.cc:311-331
             ((1000, 128), 0, 5000), ((1000, 8), 0, 333), ((50, 12288), 0, 77), ((4, 100, 40), 1, 1000),
             ((513, 1), 0, 2000)]


@pytest.mark.parametrize("path", [0, 1, 2])
@pytest.mark.parametrize("dt,idt", [("f32", np.uint32), ("f32", np.int64), ("f16", np.int64)])
@pytest.mark.parametrize("shape,dim,n", SEL_CASES)
def test_index_select(ops, shape, dim, n, dt, idt, path):
    rng = np.random.default_rng(n)
    x = _make(rng, shape, dt, "normal")
    idx = rng.integers(0, shape[dim], n).astype(idt)
    want, rc = O.index_select(x, idx, dim)
    assert rc == 0
    inner = int(np.prod(shape[dim + 1:])) * x.itemsize
    if path == 1 and inner % 16 != 0:
        pytest.skip("bulk-copy path needs rows that are multiples of 16 bytes")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        got = _to_host(ops.index_select(_to_dev(x), _to_dev(idx), dim, status=status, path=path))
    assert int(status.item()) == 0
    assert np.array_equal(_bits(got), _bits(want))


VARIANT_CASES = [((1000, 128), 0, 5000), ((30522, 128), 0, 128), ((256, 64, 128), 1, 100),
                 ((4, 100, 40), 1, 1001), ((777, 32), 0, 3), ((50, 256), 0, 77)]


def _check_gather_variant(ops, shape, dim, n, dt, idt, path):
    """the persistent vector kernel (paths 3-6) and the tensor-map gather (paths 7, 8), bit for bit,
    including an index out of range (zero row, status 1)"""
    from byteir_b200 import _native as N
    rng = np.random.default_rng(n + path)
    x = _make(rng, shape, dt, "normal")
    idx = rng.integers(0, shape[dim], n).astype(idt)
    inner = int(np.prod(shape[dim + 1:])) * x.itemsize
    ok = inner % 16 == 0 and (path < 7 or (64 <= inner <= 1024 and inner % 32 == 0))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if not ok:
        with pytest.raises(N.B200Error):
            ops.index_select(_to_dev(x), _to_dev(idx), dim, status=status, path=path)
        return
    want, _ = O.index_select(x, idx, dim)
    got = _to_host(ops.index_select(_to_dev(x), _to_dev(idx), dim, status=status, path=path))
    assert int(status.item()) == 0
    assert np.array_equal(_bits(got), _bits(want))
    if idt == np.int64:
        bad = idx.copy()
        bad[n // 2] = shape[dim] + 5
        bad[0] = -1
        got = _to_host(ops.index_select(_to_dev(x), _to_dev(bad), dim, status=status, path=path))
        assert int(status.item()) == 1
        g = np.moveaxis(got, dim, 0)
        w = np.moveaxis(want, dim, 0).copy()
        w[n // 2] = 0
        w[0] = 0
        assert np.array_equal(_bits(np.ascontiguousarray(g)), _bits(np.ascontiguousarray(w)))



@pytest.mark.parametrize("path", [3, 4, 5, 6])
@pytest.mark.parametrize("dt,idt", [("f32", np.uint32), ("f16", np.int64)])
@pytest.mark.parametrize("shape,dim,n", VARIANT_CASES)
def test_index_select_persistent_vector_variants(ops, shape, dim, n, dt, idt, path):
    _check_gather_variant(ops, shape, dim, n, dt, idt, path)


@pytest.mark.parametrize("path", [7, 8, 9, 10])
@pytest.mark.parametrize("dt,idt", [("f32", np.uint32), ("f16", np.int64)])
@pytest.mark.parametrize("shape,dim,n", VARIANT_CASES)
def test_index_select_tensor_map_gather(ops, shape, dim, n, dt, idt, path):
    _check_gather_variant(ops, shape, dim, n, dt, idt, path)


def test_index_select_tensor_map_gather_full_size_table(ops):
    rng = np.random.default_rng(1234 + 2)
    table = (rng.standard_normal((1_000_000, 128), dtype=np.float32) * 0.02).astype(np.float16)
    idx = rng.integers(0, 1_000_000, 262_144).astype(np.int64)
    want, _ = O.index_select(table, idx, 0)
    td, idd = _to_dev(table), _to_dev(idx)
    for path in (7, 8, 9, 10):
        got = _to_host(ops.index_select(td, idd, 0, path=path))
        assert np.array_equal(_bits(got), _bits(want))


def test_index_select_config3_shape(ops):
    rng = np.random.default_rng(1234 + 2)
    table = (rng.standard_normal((200000, 128), dtype=np.float32) * 0.02).astype(np.float16)
    idx = rng.integers(0, 200000, 262144).astype(np.int64)
    want, _ = O.index_select(table, idx, 0)
    for path in (1, 2):
        got = _to_host(ops.index_select(_to_dev(table), _to_dev(idx), 0, path=path))
        assert np.array_equal(_bits(got), _bits(want))


def test_index_select_full_size_table(ops):
    """the benchmark's own gather: f16 table [1,000,000 x 128] N(0, 0.02), 262,144 uniform int64 indices"""
    rng = np.random.default_rng(1234 + 2)
    table = (rng.standard_normal((1_000_000, 128), dtype=np.float32) * 0.02).astype(np.float16)
    idx = rng.integers(0, 1_000_000, 262_144).astype(np.int64)
    want, _ = O.index_select(table, idx, 0)
    td, idd = _to_dev(table), _to_dev(idx)
    for path in (0, 1, 2, 3, 5):
        got = _to_host(ops.index_select(td, idd, 0, path=path))
        assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("path", [1, 2])
def test_index_select_out_of_range_is_flagged_not_read(ops, path):
    x = _make(np.random.default_rng(3), (100, 64), "f32")
    idx = np.array([5, 100, 7, -1, 99], np.int64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = _to_host(ops.index_select(_to_dev(x), _to_dev(idx), 0, status=status, path=path))
    assert int(status.item()) == 1
    assert np.array_equal(got[[0, 2, 4]], x[[5, 7, 99]])
    assert np.all(got[[1, 3]] == 0)


# ---------------------------------------------------------------- scatter-add
def _zipf_indices(rng, n, rows, s=1.1):
    """Zipf(s) over [0, rows) by inverse CDF on ranks, hot rows scattered by a fixed permutation."""
    w = 1.0 / np.arange(1, rows + 1, dtype=np.float64) ** s
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n))
    return rng.permutation(rows)[np.minimum(ranks, rows - 1)].astype(np.int64)


PUT_CASES = [((3, 2), 5), ((256, 128), 128 * 32), ((30522, 128), 128),  # index_test.cc:300-309
             ((1000, 128), 70000), ((77, 24), 3000), ((5000, 1), 20000), ((64, 1024), 999)]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape,n", PUT_CASES)
def test_index_put_add(ops, shape, n, dt):
    rng = np.random.default_rng(n + 1)
    x = _make(rng, shape, dt, "normal")
    upd = _make(rng, (n,) + shape[1:], dt, "normal")
    idx = rng.integers(0, shape[0], n).astype(np.int64)
    want, rc = O.index_put_add(x, idx, upd)
    assert rc == 0
    xd, ud, idd = _to_dev(x), _to_dev(upd), _to_dev(idx)
    got1 = _to_host(ops.index_put_add(xd, idd, ud))
    got2 = _to_host(ops.index_put_add(xd, idd, ud))
    assert np.array_equal(_bits(got1), _bits(got2)), "not deterministic"
    g, w = O.to_f32(got1).astype(np.float64), O.to_f32(want).astype(np.float64)
    if dt == "f32":
        np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-5)  # eps of index_test.cc:143
    else:
        ulp = 2.0 ** (-10 if dt == "f16" else -7)
        assert np.all(np.abs(g - w) <= ulp * np.abs(w) + 1e-6)
    # rows nobody indexes are copied untouched
    untouched = np.setdiff1d(np.arange(shape[0]), idx)
    assert np.array_equal(_bits(got1)[untouched], _bits(x)[untouched])


def test_index_put_add_zipf_duplicates_f16(ops):
    """config 3b at a size the oracle finishes quickly: heavy duplicates, deterministic, rel 1e-3."""
    rng = np.random.default_rng(1234 + 3)
    rows, n, feat = 100000, 262144, 128
    table = (rng.standard_normal((rows, feat), dtype=np.float32) * 0.02).astype(np.float16)
    upd = rng.standard_normal((n, feat), dtype=np.float32).astype(np.float16)
    idx = _zipf_indices(rng, n, rows)
    assert np.bincount(idx).max() > 5000  # the hot row really is hot
    want, _ = O.index_put_add(table, idx, upd)
    td, ud, idd = _to_dev(table), _to_dev(upd), _to_dev(idx)
    got = _to_host(ops.index_put_add(td, idd, ud))
    again = _to_host(ops.index_put_add(td, idd, ud))
    assert np.array_equal(_bits(got), _bits(again))
    g, w = got.astype(np.float64), want.astype(np.float64)
    assert np.all(np.abs(g - w) <= 1e-3 * np.abs(w) + 1e-4)
    # in place gives the same bits
    inplace = td.clone()
    ops.index_put_add(inplace, idd, ud, out=inplace)
    assert np.array_equal(_bits(_to_host(inplace)), _bits(got))


def test_index_put_add_full_size_table_zipf(ops):
    """the benchmark's own scatter-add: f16 table [1,000,000 x 128], 262,144 updates N(0,1), Zipf(1.1) indices;
    deterministic, within rel 1e-3 of the oracle, untouched rows copied bit for bit"""
    rng = np.random.default_rng(1234 + 3)
    rows, n, feat = 1_000_000, 262_144, 128
    table = (rng.standard_normal((rows, feat), dtype=np.float32) * 0.02).astype(np.float16)
    upd = rng.standard_normal((n, feat), dtype=np.float32).astype(np.float16)
    idx = _zipf_indices(rng, n, rows)
    want, _ = O.index_put_add(table, idx, upd)
    td, ud, idd = _to_dev(table), _to_dev(upd), _to_dev(idx)
    got = _to_host(ops.index_put_add(td, idd, ud))
    again = _to_host(ops.index_put_add(td, idd, ud))
    assert np.array_equal(_bits(got), _bits(again)), "not deterministic"
    touched = np.zeros(rows, bool)
    touched[idx] = True
    assert np.array_equal(_bits(got)[~touched], _bits(table)[~touched])
    g, w = got[touched].astype(np.float64), want[touched].astype(np.float64)
    assert np.all(np.abs(g - w) <= 1e-3 * np.abs(w) + 1e-4)


def test_index_put_add_three_radix_passes_and_staged_tiles(ops):
    """a table of more than 2^20 rows (three digits of the radix sort) with 1 KiB rows (four shared-memory
    tiles per row in the accumulate pass), f32: against the sequential f32 oracle"""
    rng = np.random.default_rng(21)
    rows, n, feat = 3_000_000, 50_000, 16
    x = rng.standard_normal((rows, feat), dtype=np.float32)
    upd = rng.standard_normal((n, feat), dtype=np.float32)
    idx = np.concatenate([rng.integers(0, rows, n - 5000), np.full(5000, rows - 1)]).astype(np.int64)
    rng.shuffle(idx)
    want, _ = O.index_put_add(x, idx, upd)
    got = _to_host(ops.index_put_add(_to_dev(x), _to_dev(idx), _to_dev(upd)))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    rows, n, feat = 3000, 40_000, 256
    x = rng.standard_normal((rows, feat), dtype=np.float32)
    upd = rng.standard_normal((n, feat), dtype=np.float32)
    idx = rng.integers(0, rows, n).astype(np.int64)
    want, _ = O.index_put_add(x, idx, upd)
    got = _to_host(ops.index_put_add(_to_dev(x), _to_dev(idx), _to_dev(upd)))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("chunk_path", [1, 2])
def test_index_put_add_both_accumulate_kernels_agree_bit_for_bit(ops, chunk_path):
    """rows through registers and rows staged in shared memory add in the same order"""
    from byteir_b200 import _native as N
    rng = np.random.default_rng(22)
    rows, n, feat = 20_000, 100_000, 128
    x = (rng.standard_normal((rows, feat), dtype=np.float32) * 0.02).astype(np.float16)
    upd = rng.standard_normal((n, feat), dtype=np.float32).astype(np.float16)
    idx = _zipf_indices(rng, n, rows)
    ref = _to_host(ops.index_put_add(_to_dev(x), _to_dev(idx), _to_dev(upd)))
    try:
        N.lib().b200_index_put_tune(chunk_path)
        got = _to_host(ops.index_put_add(_to_dev(x), _to_dev(idx), _to_dev(upd)))
    finally:
        N.lib().b200_index_put_tune(0)
    assert np.array_equal(_bits(got), _bits(ref))


def test_index_put_helper_stream_prepare_and_release(ops):
    import ctypes as C
    from byteir_b200 import _native as N
    s = torch.cuda.Stream()
    h = C.c_void_p(s.cuda_stream)
    assert N.lib().b200_index_put_prepare(h) == 0
    assert N.lib().b200_index_put_prepare(h) == 0  # idempotent
    rng = np.random.default_rng(23)
    x = rng.standard_normal((40_000, 64), dtype=np.float32)  # 10 MB: large enough to fork the sort
    upd = rng.standard_normal((5000, 64), dtype=np.float32)
    idx = rng.integers(0, 40_000, 5000).astype(np.int64)
    want, _ = O.index_put_add(x, idx, upd)
    xd, idd, ud = _to_dev(x), _to_dev(idx), _to_dev(upd)
    with torch.cuda.stream(s):
        got = ops.index_put_add(xd, idd, ud)
    s.synchronize()
    np.testing.assert_allclose(_to_host(got), want, rtol=1e-5, atol=1e-5)
    assert N.lib().b200_index_put_release(h) == 0
    assert N.lib().b200_index_put_release(h) == 0  # nothing left to release


def test_index_put_add_out_of_range_skipped_and_flagged(ops):
    x = np.zeros((10, 4), np.float32)
    upd = np.ones((4, 4), np.float32)
    idx = np.array([1, 10, -3, 1], np.int64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = _to_host(ops.index_put_add(_to_dev(x), _to_dev(idx), _to_dev(upd), status=status))
    assert int(status.item()) == 1
    want = x.copy()
    want[1] = 2
    assert np.array_equal(got, want)


# ---------------------------------------------------------------- transpose
TR_CASES = [((32, 64), (1, 0)), ((1000, 512), (1, 0)), ((10, 20, 30, 40), (0, 2, 3, 1)),
            ((10, 20, 30, 40), (0, 3, 1, 2)),  # transpose_test.cc:152-168
            ((3, 5, 7), (2, 0, 1)), ((4, 8, 16, 32), (3, 1, 0, 2)), ((513, 1031), (1, 0)),
            ((2, 128, 64, 64), (0, 2, 3, 1)), ((1024, 1024), (1, 0)), ((5, 72, 200), (0, 2, 1)),
            ((1, 64, 1, 128), (0, 3, 2, 1))]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape,perm", TR_CASES)
def test_transpose(ops, shape, perm, dt):
    x = _make(np.random.default_rng(len(shape)), shape, dt)
    want = O.transpose(x, perm)
    for _ in range(2):
        got = _to_host(ops.transpose(_to_dev(x), perm))
    assert got.shape == want.shape
    assert np.array_equal(_bits(got), _bits(want))


@pytest.mark.parametrize("name", ["transpose_f32_1x32x64x64_perm0231.npz", "transpose_f32_1x3x224x224_perm0231.npz"])
def test_transpose_matches_the_references_compiled_cpu_code(ops, name):
    """the vectors made by the reference's own CPU code (its compiler's LLVM IR for f32 [1, C, H, W] -> (0, 2, 3, 1))"""
    from test_oracle import transpose_golden
    x, perm, want = transpose_golden(name)
    got = _to_host(ops.transpose(_to_dev(x), perm))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    x16 = (x % 2048).astype(np.float16)  # the same permutation through the 2-byte kernel, values exact in f16
    assert np.array_equal(_bits(_to_host(ops.transpose(_to_dev(x16), perm))), _bits((want % 2048).astype(np.float16)))


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("b,r,c", [(1, 64, 64), (3, 200, 136), (2, 72, 1000), (1, 8, 8), (4, 4096, 128)])
def test_transpose_batched_both_paths(ops, b, r, c, dt, path):
    x = _make(np.random.default_rng(r), (b, r, c), dt)
    want = np.ascontiguousarray(np.transpose(x, (0, 2, 1)))
    got = _to_host(ops.transpose_batched(_to_dev(x), path=path))
    assert np.array_equal(_bits(got), _bits(want))


def test_transpose_config4_shapes(ops):
    rng = np.random.default_rng(1234 + 4)
    x = rng.uniform(-1, 1, (32, 128, 64, 64)).astype(np.float16)
    got = _to_host(ops.transpose(_to_dev(x), (0, 2, 3, 1)))
    assert np.array_equal(_bits(got), _bits(np.ascontiguousarray(np.transpose(x, (0, 2, 3, 1)))))
    y = O.f32_to_bf16(rng.uniform(-1, 1, (8192, 8192)).astype(np.float32))
    got = _to_host(ops.transpose(_to_dev(y), (1, 0)))
    assert np.array_equal(got, np.ascontiguousarray(y.T))


def test_sharded_sum_finish_single_rank_protocol(ops):
    """world = 1: the rank pushes to its own inbox, waits for its own flag, folds, rounds; repeated
    calls alternate inbox slots and advance the epoch."""
    from byteir_b200 import _native as N
    n = 1024
    inbox = torch.zeros(N.lib().b200_sharded_sum_inbox_bytes(1, n) // 4, dtype=torch.float32, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ss = ops.ShardedSum(0, 1, n, [inbox.data_ptr()], [flags.data_ptr()], counter, status)
    out = torch.empty(n, dtype=torch.float16, device="cuda")
    for step in range(5):
        part = torch.randn(n, device="cuda") * 100
        ss(part, out)
        torch.cuda.synchronize()
        assert torch.equal(out, part.to(torch.float16))
        assert int(counter.item()) == step + 1 and int(flags[0].item()) == step + 1
    assert int(status.item()) == 0


def test_sharded_sum_finish_times_out_instead_of_hanging(ops):
    """a peer that never publishes: the bounded wait expires, the status word says so, the context
    stays usable (world = 2 with the second rank's memory emulated locally and left silent)"""
    from byteir_b200 import _native as N
    n = 256
    nb = N.lib().b200_sharded_sum_inbox_bytes(2, n) // 4
    inbox0, inbox1 = (torch.zeros(nb, dtype=torch.float32, device="cuda") for _ in range(2))
    flags0, flags1 = (torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2))
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ss = ops.ShardedSum(0, 2, n, [inbox0.data_ptr(), inbox1.data_ptr()], [flags0.data_ptr(), flags1.data_ptr()],
                        counter, status)
    out = torch.full((n,), -7.0, dtype=torch.float32, device="cuda")
    ss(torch.ones(n, device="cuda"), out)
    torch.cuda.synchronize()  # returns after the 2 s limit
    assert int(status.item()) == 3
    assert int(flags1[0].item()) == 1  # rank 0 did publish to its peer
    assert torch.all(out == -7.0) and int(counter.item()) == 0  # no stale sum written, the epoch did not advance
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


@pytest.mark.parametrize("dtype", [torch.uint8, torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("n,head", [(1, 0), (5, 1), (4099, 3), (1 << 20, 0), ((1 << 20) + 7, 5)])
def test_fill_any_alignment(dtype, n, head):
    """b200_fill writes exactly [0, n): unaligned starts and ragged ends, all element sizes"""
    from byteir_b200 import _native as N
    buf = torch.zeros(n + head + 16, dtype=dtype, device="cuda")
    value = torch.tensor([3], dtype=dtype)
    bits = int.from_bytes(value.numpy().tobytes(), "little")
    rc = N.lib().b200_fill(buf.element_size(), buf.data_ptr() + head * buf.element_size(), n, bits,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.all(buf[head:head + n] == 3)
    assert torch.all(buf[:head] == 0) and torch.all(buf[head + n:] == 0)
