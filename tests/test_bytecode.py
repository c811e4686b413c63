"""The ByRE bytecode reader (byre_serial 1.0.0 in an MLIR 17 bytecode container): the reference's own
fixture, and modules written by tests/byre_bytecode_writer.py against their text twins."""
from pathlib import Path

import numpy as np
import pytest

from byteir_b200 import brt
from byre_bytecode_writer import write_module, varint
from test_brt_host import plugin  # noqa: F401  (registers the host kernels)

FIXTURE = Path(__file__).parent / "golden" / "byre_serial_v1_lljit_case0.mlirbc"
# compiler/test/E2E/Host/Case0_Bytecode/Output.mlirbc: the same module as the compiler's own end-to-end test
# writes it, with the producer string the dialect's writer puts in ("BYRE_1_0_0" instead of the MLIR version)
FIXTURE_E2E = Path(__file__).parent / "golden" / "byre_serial_v1_host_case0_bytecode.mlirbc"


def _load(data, tmp_path, device="cpu", name="m.mlirbc"):
    path = tmp_path / name
    path.write_bytes(data)
    s = brt.Session(device)
    s.load(str(path))
    return s


@pytest.mark.parametrize("fixture", [FIXTURE, FIXTURE_E2E], ids=["runtime_lljit_case0", "compiler_e2e_case0_bytecode"])
def test_reference_fixture_loads(tmp_path, fixture):
    """runtime/test/test_files/LLJIT/Case0_v1_0_0/entry.mlirbc and compiler/test/E2E/Host/Case0_Bytecode/
    Output.mlirbc: six host memrefs, one compute op whose attributes came through the extra_args
    dictionary (checked by the stub kernel's constructor)"""
    s = _load(fixture.read_bytes(), tmp_path)
    got = [(a.name, a.argtype, a.dtype, tuple(a.shape), a.space) for a in s.args()]
    assert got == [("Input0", 1, "i64", (1,), "cpu"), ("Input1", 1, "i64", (1,), "cpu"), ("Input2", 1, "i64", (1,), "cpu"),
                   ("Input3", 1, "i32", (1, 128), "cpu"), ("Output0", 2, "i32", (1, 128), "cpu"),
                   ("Output1", 2, "i32", (1, 128), "cpu")]
    req = s.new_request()
    req.finish_io_binding()
    req.run()
    req.sync()


def test_writer_reproduces_the_fixtures_module(tmp_path):
    """the same module written by the test writer loads to the same metadata"""
    desc = {"name": "main",
            "args": [("Input0", 1, "i64", (1,), "cpu"), ("Input1", 1, "i64", (1,), "cpu"), ("Input2", 1, "i64", (1,), "cpu"),
                     ("Input3", 1, "i32", (1, 128), "cpu"), ("Output0", 2, "i32", (1, 128), "cpu"),
                     ("Output1", 2, "i32", (1, 128), "cpu")],
            "ops": [("compute", "LLVMJITOp", [0, 1, 2, 3, 4, 5],
                     {"device": "cpu", "kernel_name": "Unknown0", "llvm_file_name": "host_kernels.bc"},
                     [1, 1, 1, 1, 2, 2])]}
    a = _load(write_module(desc), tmp_path, name="a.mlirbc")
    b = _load(FIXTURE.read_bytes(), tmp_path, name="b.mlirbc")
    assert [vars(x) for x in a.args()] == [vars(x) for x in b.args()]


def test_bytecode_from_memory():
    s = brt.Session("cpu")
    s.load_from_memory(FIXTURE.read_bytes())
    assert [a.name for a in s.args()][:2] == ["Input0", "Input1"]
    s.load_from_memory(TEXT.encode())  # text as bytes takes the same door
    assert s.arg_num() == 4
    with pytest.raises(brt.BrtError):
        s.load_from_memory(FIXTURE.read_bytes()[:100])


def test_varints_of_every_length():
    assert varint(0) == b"\x01" and varint(127) == b"\xff" and varint(128) == b"\x02\x02"
    assert varint(6400) == bytes([0x02, 0x64])  # (6400 << 2 | 2) little endian
    assert len(varint((1 << 56) - 1)) == 8 and len(varint(1 << 56)) == 9 and varint(1 << 63)[0] == 0


TEXT = """
module attributes {byre.container_module} {
  func.func @main(%arg0 : memref<100x32xf32, "cpu"> {byre.argname = "A", byre.argtype = 1: i32},
                  %arg1 : memref<100x32xf32, "cpu"> {byre.argname = "B", byre.argtype = 1: i32},
                  %arg2 : memref<100x32xf32, "cpu"> {byre.argname = "C", byre.argtype = 2: i32},
                  %arg3 : memref<50x32xf32, "cpu"> {byre.argname = "Tail", byre.argtype = 2: i32}) attributes {byre.entry_point} {
    %0 = memref.alloc() : memref<12800xi8, "cpu">
    %1 = "byre.alias"(%0) {offset = 0 : i64} : (memref<12800xi8, "cpu">) -> memref<100x32xf32, "cpu">
    %2 = "byre.alias"(%0) {offset = 6400 : i64} : (memref<12800xi8, "cpu">) -> memref<50x32xf32, "cpu">
    byre.compute @AddOp_f32f32_f32(%arg0, %arg1, %1) {device = "cpu", memory_effects = [1 : i32, 1 : i32, 2 : i32]} : memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">
    byre.compute @ScaleOp_f32_f32(%1, %arg2) {factor = -2.500000e+00 : f32, shift = -3 : i64} : memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">
    byre.compute @ScaleOp_f32_f32(%2, %arg3) {factor = 5.000000e-01 : f32} : memref<50x32xf32, "cpu">, memref<50x32xf32, "cpu">
    return
  }
}
"""
DESC = {"name": "main",
        "args": [("A", 1, "f32", (100, 32), "cpu"), ("B", 1, "f32", (100, 32), "cpu"), ("C", 2, "f32", (100, 32), "cpu"),
                 ("Tail", 2, "f32", (50, 32), "cpu")],
        "ops": [("alloc", "i8", (12800,), "cpu"),
                ("alias", 4, 0, "f32", (100, 32), "cpu"),
                ("alias", 4, 6400, "f32", (50, 32), "cpu"),
                ("compute", "AddOp_f32f32_f32", [0, 1, 5], {"device": "cpu"}, [1, 1, 2]),
                ("compute", "ScaleOp_f32_f32", [5, 2], {"factor": -2.5, "shift": -3}, None),
                ("compute", "ScaleOp_f32_f32", [6, 3], {"factor": 0.5}, None)]}


def _run(s, a, b):
    req = s.new_request()
    c, tail = np.zeros((100, 32), np.float32), np.zeros((50, 32), np.float32)
    for name, arr in (("A", a), ("B", b), ("C", c), ("Tail", tail)):
        req.bind_arg(s.arg_offset(name), arr.ctypes.data)
    req.finish_io_binding()
    req.run()
    req.sync()
    return c, tail


def test_bytecode_and_text_twins_run_alike(tmp_path):
    """alloc, alias offsets, float and negative integer attributes, results numbered after the arguments"""
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((100, 32)).astype(np.float32), rng.standard_normal((100, 32)).astype(np.float32)
    st = brt.Session("cpu")
    st.load_from_memory(TEXT)
    want_c, want_tail = _run(st, a, b)
    for isolated in (False, True):  # the function body inline, or in a nested IR section
        sb = _load(write_module(DESC, isolated_func=isolated), tmp_path)
        got_c, got_tail = _run(sb, a, b)
        np.testing.assert_array_equal(got_c, want_c)
        np.testing.assert_array_equal(got_tail, want_tail)
    np.testing.assert_array_equal(got_c, (a + b) * np.float32(-2.5) - 3)
    np.testing.assert_array_equal(got_tail, ((a + b) * np.float32(0.5))[50:])


@pytest.mark.parametrize("dims", [("dense", "i64", (2,), [0, 1]), ("dense", "i64", (1,), [1]), ("array", "i64", [0, 1])])
def test_cuda_ops_take_dense_attributes_from_bytecode(tmp_path, dims):
    """a reduction's `dimensions` as DenseIntOrFPElements (two values; one value = splat) and as a dense
    array; the kernel's constructor checks them against the shapes"""
    out_shape = (1024,) if len(dims[-1]) == 2 else (64, 1024)
    desc = {"name": "main",
            "args": [("X", 1, "f16", (64, 512, 1024), "cuda"), ("Y", 2, "f16", out_shape, "cuda")],
            "ops": [("compute", "ReduceSumOp_f16_f16", [0, 1], {"dimensions": dims, "device": "cuda"}, [1, 2])]}
    s = _load(write_module(desc), tmp_path, device="cuda")
    assert [a.name for a in s.args()] == ["X", "Y"] and s.arg_info(0).dtype == "f16"
    bad = dict(desc, args=[desc["args"][0], ("Y", 2, "f16", (7,), "cuda")])
    with pytest.raises(brt.BrtError):
        _load(write_module(bad), tmp_path, device="cuda", name="bad.mlirbc")


def test_fill_values_from_bytecode(tmp_path):
    """FillOp's `value`: an f16 splat, three f16 values, an i1 splat, an i64 splat"""
    desc = {"name": "main",
            "args": [("H", 2, "f16", (1001,), "cuda"), ("T", 2, "f16", (3,), "cuda"), ("F", 2, "i1", (3,), "cuda"),
                     ("S", 2, "i64", (37,), "cuda")],
            "ops": [("compute", "FillOp", [0], {"value": ("dense", "f16", (1001,), [0.5])}, None),
                    ("compute", "FillOp", [1], {"value": ("dense", "f16", (3,), [1.0, 2.0, 3.0])}, None),
                    ("compute", "FillOp", [2], {"value": ("dense", "i1", (3,), [True])}, None),
                    ("compute", "FillOp", [3], {"value": ("dense", "i64", (37,), [-7])}, None)]}
    s = _load(write_module(desc), tmp_path, device="cuda")
    assert s.arg_info(2).nbytes == 3
    wrong = dict(desc, ops=[("compute", "FillOp", [1], {"value": ("dense", "f16", (2,), [1.0, 2.0])}, None)])
    with pytest.raises(brt.BrtError, match="FillOp"):
        _load(write_module(wrong), tmp_path, device="cuda", name="wrong.mlirbc")


def test_damaged_bytecode_is_an_error_not_a_crash(tmp_path):
    good = FIXTURE.read_bytes()
    for cut in (5, 20, 60, 150, 200, 300, len(good) - 1):
        with pytest.raises(brt.BrtError):
            _load(good[:cut], tmp_path, name=f"cut{cut}.mlirbc")
    rng = np.random.default_rng(1)
    for trial in range(200):  # flipped bytes: any outcome but a crash
        data = bytearray(good)
        for pos in rng.integers(4, len(good), 3):
            data[pos] = int(rng.integers(0, 256))
        try:
            _load(bytes(data), tmp_path, name="fuzz.mlirbc")
        except brt.BrtError:
            pass
    with pytest.raises(brt.BrtError, match="version"):
        _load(b"ML\xefR" + varint(6) + good[5:], tmp_path, name="v6.mlirbc")


def test_group_copy_is_its_copies_in_order(tmp_path):
    """group_copy_v1 (ByreSerial.td:407-413): sources first, then as many targets; decoded as one byre.copy per
    pair with the group's callee.  Loaded into a CUDA session (no device needed to load), the plan holds the two
    cuda2cuda kernels; an odd operand count is an error."""
    desc = {"name": "main",
            "args": [("A", 1, "f32", (64,), "cuda"), ("B", 1, "f16", (8, 4), "cuda"), ("OutA", 2, "f32", (64,), "cuda"),
                     ("OutB", 2, "f16", (8, 4), "cuda")],
            "ops": [("group_copy", [0, 1], [2, 3], "cuda2cuda")]}
    s = brt.Session("cuda")
    s.load_from_memory(write_module(desc))
    assert [a.name for a in s.args()] == ["A", "B", "OutA", "OutB"]
    bad = dict(desc, ops=[("group_copy", [0, 1], [2], "cuda2cuda")])
    with pytest.raises(brt.BrtError, match="as many targets as sources"):
        brt.Session("cuda").load_from_memory(write_module(bad))
