"""CPU tests of the brt host runtime: the ByRE text loader, the execution plan,
frames, argument binding, events, kernel plug-ins and error reporting.  They
mirror runtime/test/{session,context,framework,ir} of the reference on a host
device, so they run without a GPU."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

from byteir_b200 import brt

ROOT = Path(__file__).resolve().parent.parent
PLUGIN = ROOT / "tests" / "cpp" / "_build" / "libhost_kernels.so"


@pytest.fixture(scope="session", autouse=True)
def plugin():
    src = ROOT / "tests" / "cpp" / "host_kernels.cc"
    PLUGIN.parent.mkdir(exist_ok=True)
    if not PLUGIN.exists() or PLUGIN.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++", "-std=c++17", "-O1",
                               "-fPIC", "-shared", "-I", str(ROOT / "include"), str(src), "-o", str(PLUGIN)])
    brt.lib()  # the runtime must be loaded (RTLD_GLOBAL) before the plug-in resolves its symbols
    brt.register_kernels_from_dynlib(PLUGIN)
    return PLUGIN


CUDA_PLUGIN = ROOT / "tests" / "cpp" / "_build" / "libcuda_plugin.so"
_cuda_plugin_registered = False


def cuda_plugin():
    """tests/cpp/cuda_plugin.cc: the kernel plug-in of the integration notes (an Impl class with the contract of
    the reference's reduce_impl.h, wrapped by CudaOpKernelWithWorkspace, calling the C ABI), built with g++ against
    this repo's headers and registered once"""
    global _cuda_plugin_registered
    src = ROOT / "tests" / "cpp" / "cuda_plugin.cc"
    CUDA_PLUGIN.parent.mkdir(exist_ok=True)
    if not CUDA_PLUGIN.exists() or CUDA_PLUGIN.stat().st_mtime < src.stat().st_mtime:
        cuda_inc = next((p for p in ("/usr/local/cuda/include", "/usr/local/cuda-12.9/include") if Path(p).exists()), None)
        assert cuda_inc, "no CUDA headers"
        lib_dir = ROOT / "byteir_b200" / "_lib"
        subprocess.check_call(["/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++", "-std=c++17", "-O1", "-fPIC",
                               "-shared", "-I", str(ROOT / "include"), "-I", cuda_inc, str(src), "-o", str(CUDA_PLUGIN),
                               "-L", str(lib_dir), "-lb200_kernels", f"-Wl,-rpath,{lib_dir}"])
    if not _cuda_plugin_registered:
        brt.lib()
        brt.register_kernels_from_dynlib(CUDA_PLUGIN)
        _cuda_plugin_registered = True
    return CUDA_PLUGIN


def test_cuda_kernel_plugin_builds_registers_and_its_key_loads():
    cuda_plugin()
    s = _cuda_session()
    s.load_from_memory(reduce_mlir("PluginReduceSumOp_f16_f16", "f16", (64, 512, 1024), (1024,), "dense<[0, 1]> : tensor<2xi64>"))
    assert s.arg_info(1).shape == (1024,)
    with pytest.raises(brt.BrtError, match="consecutive"):  # the plug-in's own check, raised from its constructor
        s.load_from_memory(reduce_mlir("PluginReduceSumOp_f16_f16", "f16", (4, 5, 6), (5,), "dense<[0, 2]> : tensor<2xi64>"))


ADD = """
module attributes {byre.container_module} {
  func.func @test_add(%arg0 : memref<100x32xf32, "cpu"> {byre.argname = "A", byre.argtype = 1: i32},
                      %arg1 : memref<100x32xf32, "cpu"> {byre.argname = "B", byre.argtype = 1: i32},
                      %arg2 : memref<100x32xf32, "cpu"> {byre.argname = "C", byre.argtype = 2: i32})
                      attributes {byre.entry_point} {
    // C = (A + B) + B through an intermediate
    %0 = memref.alloc() : memref<100x32xf32, "cpu">
    byre.compute @AddOp_f32f32_f32(%arg0, %arg1, %0) {device = "cpu", memory_effects = [1 : i32, 1 : i32, 2 : i32]} : memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">
    byre.compute @AddOp_f32f32_f32(%0, %arg1, %arg2) {device = "cpu"} : memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">, memref<100x32xf32, "cpu">
    return
  }
}
"""


def _ptr(a):
    return a.ctypes.data


def test_load_metadata_and_run_twice():
    s = brt.Session("cpu")
    s.load_from_memory(ADD)
    args = s.args()
    assert [a.name for a in args] == ["A", "B", "C"]
    assert [a.argtype for a in args] == [1, 1, 2]
    assert args[2].shape == (100, 32) and args[2].dtype == "f32" and args[2].space == "cpu"
    assert s.arg_offset("B") == 1 and s.arg_offset("nope") == -1
    req = s.new_request()
    req.enable_op_trace()
    a = np.random.default_rng(0).standard_normal((100, 32)).astype(np.float32)
    b = np.random.default_rng(1).standard_normal((100, 32)).astype(np.float32)
    c = np.zeros_like(a)
    req.bind_arg(0, _ptr(a)); req.bind_arg(1, _ptr(b)); req.bind_arg(2, _ptr(c))
    req.finish_io_binding()
    for _ in range(2):  # the reference's tests run twice on one RequestContext
        req.run(); req.sync()
        np.testing.assert_array_equal(c, (a + b) + b)
    assert req.op_trace() == ["AddOp_f32f32_f32"] * 4


def test_get_arg_allocates_and_owns():
    s = brt.Session("cpu")
    s.load_from_memory(ADD)
    req = s.new_request()
    ptrs = [req.get_arg(i) for i in range(3)]  # nothing bound: the context allocates
    assert len(set(ptrs)) == 3 and all(p % 256 == 0 for p in ptrs)
    n = 100 * 32
    views = [np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), (n,)) for p in ptrs]
    views[0][:] = 1.5; views[1][:] = 2.0
    req.run(); req.sync()
    assert np.all(views[2] == 5.5)
    assert req.get_arg(0) == ptrs[0]  # stable across calls
    # a later bind replaces the owned buffer
    mine = np.full(n, 3.0, np.float32)
    req.bind_arg(0, _ptr(mine))
    req.run(); req.sync()
    assert np.all(views[2] == 7.0)


ALIAS = """
module attributes {byre.container_module} {
  func.func @f(%arg0: memref<8xf32, "cpu"> {byre.argname = "In", byre.argtype = 1 : i32},
               %arg1: memref<4xf32, "cpu"> {byre.argname = "Out", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    %alloc = memref.alloc() : memref<64xi8, "cpu">
    %0 = "byre.alias"(%alloc) <{offset = 0 : i64}> {device = "cpu"} : (memref<64xi8, "cpu">) -> memref<4xf32, "cpu">
    %1 = "byre.alias"(%alloc) {offset = 16 : i64} : (memref<64xi8, "cpu">) -> memref<4xf32, "cpu">
    %2 = "byre.alias"(%arg0) <{offset = 4 : i64}> : (memref<8xf32, "cpu">) -> memref<4xf32, "cpu">
    %3 = "byre.alias"(%arg0) <{offset = 0 : i64}> : (memref<8xf32, "cpu">) -> memref<4xf32, "cpu">
    byre.compute @ScaleOp_f32_f32(%2, %0) {factor = 2.0 : f32} : memref<4xf32, "cpu">, memref<4xf32, "cpu">
    byre.compute @ScaleOp_f32_f32(%3, %1) {factor = 1.000000e+01 : f32, shift = 1 : i64} : memref<4xf32, "cpu">, memref<4xf32, "cpu">
    "byre.compute"(%0, %1, %arg1) {callee = "AddOp_f32f32_f32"} : (memref<4xf32, "cpu">, memref<4xf32, "cpu">, memref<4xf32, "cpu">) -> ()
    return
  }
}
"""


def test_alias_offsets_count_source_elements_and_generic_form():
    s = brt.Session("cpu")
    s.load_from_memory(ALIAS)
    req = s.new_request()
    x = np.arange(8, dtype=np.float32)
    out = np.zeros(4, np.float32)
    req.bind_arg(0, _ptr(x)); req.bind_arg(1, _ptr(out))
    req.run(); req.sync()
    # %2 = x[4:8] (offset in f32 elements), %3 = x[0:4]; %0/%1 live 16 bytes apart in one i8 block
    np.testing.assert_array_equal(out, x[4:8] * 2 + (x[0:4] * 10 + 1))


@pytest.mark.parametrize("bad", ["offset = 52 : i64}> {device = \"cpu\"}",  # 52 + 16 bytes > the 64-byte block
                                 "offset = -1 : i64}> {device = \"cpu\"}"])
def test_alias_that_does_not_fit_its_source_is_refused_at_load_time(bad):
    s = brt.Session("cpu")
    with pytest.raises(brt.BrtError, match="does not fit its source"):
        s.load_from_memory(ALIAS.replace("offset = 0 : i64}> {device = \"cpu\"}", bad))
    with pytest.raises(brt.BrtError, match="does not fit its source"):
        s.load_from_memory(ALIAS.replace("(%arg0) <{offset = 4 : i64}>", "(%arg0) <{offset = 5 : i64}>"))  # 5 + 4 > 8 elements


def test_unknown_op_is_reported_like_the_reference():
    s = brt.Session("cpu")
    with pytest.raises(brt.BrtError, match="No providers support Op NoSuchOp_f32"):
        s.load_from_memory(ADD.replace("@AddOp_f32f32_f32(%0", "@NoSuchOp_f32(%0"))


def test_syntax_error_names_the_line():
    bad = ADD.replace("memref.alloc() :", "memref.alloc( :")
    s = brt.Session("cpu")
    with pytest.raises(brt.BrtError, match=r"line 8: expected"):
        s.load_from_memory(bad)


def test_missing_entry_point_and_missing_allocator():
    s = brt.Session("cpu")
    with pytest.raises(brt.BrtError, match="byre.entry_point"):
        s.load_from_memory(ADD.replace("attributes {byre.entry_point}", ""))
    with pytest.raises(brt.BrtError, match='memory space "cuda"'):
        s.load_from_memory(ADD.replace('"cpu"', '"cuda"'))


def test_kernel_constructor_failure_surfaces_at_load():
    s = brt.Session("cpu")
    bad = ADD.replace('%arg2 : memref<100x32xf32, "cpu"> {byre.argname = "C"', '%arg2 : memref<100x31xf32, "cpu"> {byre.argname = "C"') \
             .replace('memref<100x32xf32, "cpu">\n    return', 'memref<100x31xf32, "cpu">\n    return')
    with pytest.raises(brt.BrtError, match="shape mismatch"):
        s.load_from_memory(bad)


def test_run_time_failure_is_a_status_and_the_context_stays_usable():
    text = ADD.replace("byre.compute @AddOp_f32f32_f32(%0, %arg1, %arg2)", "byre.compute @AlwaysFailOp(%0, %arg1, %arg2)")
    s = brt.Session("cpu")
    s.load_from_memory(text)
    req = s.new_request()
    with pytest.raises(brt.BrtError, match="injected failure"):
        req.run()
    with pytest.raises(brt.BrtError, match="injected failure"):
        req.run()  # still answers


def test_load_file_and_truncated_bytecode(tmp_path):
    p = tmp_path / "add.mlir"
    p.write_text(ADD)
    s = brt.Session("cpu")
    s.load(p)
    assert s.arg_num() == 3
    with pytest.raises(brt.BrtError, match="cannot open"):
        s.load(tmp_path / "missing.mlir")
    bc = tmp_path / "m.mlirbc"
    bc.write_bytes(b"ML\xefR\x01byre")
    with pytest.raises(brt.BrtError, match="bytecode"):
        s.load(bc)


def test_request_before_load_fails_cleanly():
    s = brt.Session("cpu")
    with pytest.raises(brt.BrtError, match="before a model is loaded"):
        s.new_request()


# ---- the CUDA provider's kernels parse their ops at load time: no GPU needed for that
def _cuda_session():
    return brt.Session("cuda")


REDUCE = """
module attributes {byre.container_module} {
  func.func @reduce(%arg0: memref<%INx%T, "cuda"> {byre.argname = "Input0", byre.argtype = 1 : i32},
                    %arg1: memref<%OUTx%OT, "cuda"> {byre.argname = "Output0", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    byre.compute @%KEY(%arg0, %arg1) {device = "cuda", dimensions = %DIMS, memory_effects = [1 : i32, 2 : i32]} : memref<%INx%T, "cuda">, memref<%OUTx%OT, "cuda">
    return
  }
}
"""


def reduce_mlir(key, t, in_shape, out_shape, dims, out_t=None):
    f = lambda sh: "x".join(str(d) for d in sh)
    return (REDUCE.replace("%IN", f(in_shape)).replace("%OUT", f(out_shape)).replace("%OT", out_t or t).replace("%T", t)
            .replace("%KEY", key).replace("%DIMS", dims))


@pytest.mark.parametrize("dims", ["dense<1> : tensor<1xi64>", "dense<[1]> : tensor<1xi64>", "[1 : i64]", "array<i64: 1>"])
def test_cuda_reduce_op_accepts_every_spelling_of_dimensions(dims):
    s = _cuda_session()
    s.load_from_memory(reduce_mlir("ReduceSumOp_f32_f32", "f32", (1024, 4096), (1024,), dims))
    assert s.arg_info(1).shape == (1024,)


def test_cuda_reduce_op_validates_shapes_and_consecutive_dims():
    s = _cuda_session()
    with pytest.raises(brt.BrtError, match="output shape"):
        s.load_from_memory(reduce_mlir("ReduceSumOp_f32_f32", "f32", (1024, 4096), (4096,), "dense<1> : tensor<1xi64>"))
    # dimensions that are not consecutive are reduced group by group (the reference stops at load time:
    # "Only consecutive dimensions ...", reduce_impl.h:40-42)
    s.load_from_memory(reduce_mlir("ReduceMaxOp_f16_f16", "f16", (4, 5, 6), (5,), "dense<[0, 2]> : tensor<2xi64>"))
    # a 16-bit sum may be delivered unrounded as f32; a max may not change the element type
    s.load_from_memory(reduce_mlir("ReduceSumOp_f16_f32", "f16", (4, 5, 6), (6,), "dense<[0, 1]> : tensor<2xi64>", "f32"))
    assert s.arg_info(1).dtype == "f32"
    with pytest.raises(brt.BrtError):
        s.load_from_memory(reduce_mlir("ReduceMaxOp_f16_f32", "f16", (4, 5, 6), (6,), "dense<[0, 1]> : tensor<2xi64>", "f32"))
    # reduced dimensions with only size-1 dimensions between them are one group (the reference, which drops the
    # size-1 dimension from the list and then finds 0, 1, 3 not consecutive, refuses this one too)
    s.load_from_memory(reduce_mlir("ReduceSumOp_f16_f16", "f16", (128, 2, 1, 21, 3), (3,), "dense<[0, 1, 2, 3]> : tensor<4xi64>"))
    # unsorted dims are fine (resnet18_fw_bw_host_cuda.mlir:178 has dense<[3, 2]>)
    s.load_from_memory(reduce_mlir("ReduceSumOp_f16_f16", "f16", (2, 3, 4, 5), (2, 3), "dense<[3, 2]> : tensor<2xi64>"))


def test_cuda_provider_registers_the_reference_keys_and_the_bf16_ones():
    for key, t, i, o, d in [("ReduceSumOp_f16_f16", "f16", (8, 8), (8,), "dense<1> : tensor<1xi64>"),
                            ("ReduceSumOp_f32_f32", "f32", (8, 8), (8,), "dense<1> : tensor<1xi64>"),
                            ("ReduceMaxOp_f32_f32", "f32", (8, 8), (8,), "dense<0> : tensor<1xi64>"),
                            ("ReduceMaxOp_f16_f16", "f16", (8, 8), (8,), "dense<0> : tensor<1xi64>"),
                            ("ReduceSumOp_bf16_bf16", "bf16", (8, 8), (8,), "dense<0> : tensor<1xi64>")]:
        _cuda_session().load_from_memory(reduce_mlir(key, t, i, o, d))


INDEX = """
module attributes {byre.container_module} {
  func.func @index(%arg0: memref<30522x128x%T, "cuda"> {byre.argname = "Table", byre.argtype = 1 : i32},
                   %arg1: memref<128x%I, "cuda"> {byre.argname = "Idx", byre.argtype = 1 : i32},
                   %arg2: memref<128x128x%T, "cuda"> {byre.argname = "Upd", byre.argtype = 1 : i32},
                   %arg3: memref<128x128x%T, "cuda"> {byre.argname = "Sel", byre.argtype = 2 : i32},
                   %arg4: memref<30522x128x%T, "cuda"> {byre.argname = "Put", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    byre.compute @IndexSelectOp_%T%I_%T(%arg0, %arg1, %arg3) {dim = 0 : i32} : memref<30522x128x%T, "cuda">, memref<128x%I, "cuda">, memref<128x128x%T, "cuda">
    byre.compute @IndexPutOp_%Ti64%T_%T(%arg0, %arg1, %arg2, %arg4) {dim = 0 : i32} : memref<30522x128x%T, "cuda">, memref<128x%I, "cuda">, memref<128x128x%T, "cuda">, memref<30522x128x%T, "cuda">
    return
  }
}
"""


def test_cuda_index_ops_load():
    for t in ("f32", "f16"):
        s = _cuda_session()
        s.load_from_memory(INDEX.replace("%T", t).replace("%I", "i64"))
        assert [a.name for a in s.args()] == ["Table", "Idx", "Upd", "Sel", "Put"]


TRANSPOSE = """
module attributes {byre.container_module} {
  func.func @t(%arg0: memref<10x20x30x40xf16, "cuda"> {byre.argname = "In", byre.argtype = 1 : i32},
               %arg1: memref<%OUTxf16, "cuda"> {byre.argname = "Out", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    byre.compute @TransposeOp_f16_f16(%arg0, %arg1) {permutation = dense<%PERM> : tensor<4xi64>} : memref<10x20x30x40xf16, "cuda">, memref<%OUTxf16, "cuda">
    return
  }
}
"""


def test_cuda_transpose_op_checks_the_permuted_shape():
    s = _cuda_session()
    s.load_from_memory(TRANSPOSE.replace("%OUT", "10x30x40x20").replace("%PERM", "[0, 2, 3, 1]"))
    s.load_from_memory(TRANSPOSE.replace("%OUT", "40x20x10x30").replace("%PERM", "[3, 1, 0, 2]"))  # any permutation
    with pytest.raises(brt.BrtError, match="permuted"):
        s.load_from_memory(TRANSPOSE.replace("%OUT", "10x30x40x20").replace("%PERM", "[0, 3, 1, 2]"))


CUSTOM = """
module attributes {byre.container_module} {
  func.func @c(%arg0 : memref<1x128x3x32xf16, "cuda"> {byre.argname = "Q", byre.argtype = 1: i32},
               %arg1 : memref<1x3x128xf32, "cuda"> {byre.argname = "Lse", byre.argtype = 2: i32}) attributes {byre.entry_point} {
    "byre.custom"(%arg0, %arg1) {callee = "custom", lib_path = "%LIB", api_name = "%API", version = "2.5.3", extra_args = [12288 : i64, 0.5 : f32, -1 : i64]} : (memref<1x128x3x32xf16, "cuda">, memref<1x3x128xf32, "cuda">) -> ()
    return
  }
}
"""


def test_custom_op_resolves_library_symbol_and_version():
    libfa = str(ROOT / "byteir_b200" / "_lib" / "libflash_attn.so")
    s = _cuda_session()
    s.load_from_memory(CUSTOM.replace("%LIB", libfa).replace("%API", "run_flash_attn_fwd"))
    with pytest.raises(brt.BrtError, match="Couldn't find function: no_such_api"):
        s.load_from_memory(CUSTOM.replace("%LIB", libfa).replace("%API", "no_such_api"))
    with pytest.raises(brt.BrtError, match="load failed"):
        s.load_from_memory(CUSTOM.replace("%LIB", "/nonexistent/libx.so").replace("%API", "run_flash_attn_fwd"))
    # bf16 operands pick the bf16 sibling of a flash-attention entry point
    s.load_from_memory(CUSTOM.replace("%LIB", libfa).replace("%API", "run_flash_attn_fwd").replace("xf16", "xbf16"))


def test_cuda_request_without_a_gpu_fails_with_a_status_not_a_crash():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    s = _cuda_session()
    s.load_from_memory(reduce_mlir("ReduceSumOp_f32_f32", "f32", (8, 8), (8,), "dense<1> : tensor<1xi64>"))
    with pytest.raises(brt.BrtError):
        s.new_request()


HOST_DEVICE = """
module attributes {byre.container_module} {
  func.func @main(%arg0: memref<1024x256xf32, "cpu"> {byre.argname = "A", byre.argtype = 1 : i32},
                  %arg1: memref<1024xf32, "cpu"> {byre.argname = "Sum", byre.argtype = 2 : i32},
                  %arg2: memref<3xf16, "cuda"> {byre.argname = "Three", byre.argtype = 2 : i32},
                  %arg3: memref<1001xf16, "cuda"> {byre.argname = "Halves", byre.argtype = 2 : i32},
                  %arg4: memref<37xi64, "cuda"> {byre.argname = "Sevens", byre.argtype = 2 : i32},
                  %arg5: memref<3xi1, "cuda"> {byre.argname = "Flags", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    %0 = memref.alloc() : memref<1024x256xf32, "cuda">
    %1 = memref.alloc() : memref<1024xf32, "cuda">
    byre.compute @cpu2cuda(%arg0, %0) {memory_effects = [1 : i32, 2 : i32]} : memref<1024x256xf32, "cpu">, memref<1024x256xf32, "cuda">
    byre.compute @ReduceSumOp_f32_f32(%0, %1) {dimensions = dense<1> : tensor<1xi64>, memory_effects = [1 : i32, 2 : i32]} : memref<1024x256xf32, "cuda">, memref<1024xf32, "cuda">
    byre.compute @cuda2cpu(%1, %arg1) {memory_effects = [1 : i32, 2 : i32]} : memref<1024xf32, "cuda">, memref<1024xf32, "cpu">
    byre.compute @FillOp(%arg2) {value = dense<[1.000000e+00, 2.000000e+00, 3.000000e+00]> : tensor<3xf16>} : memref<3xf16, "cuda">
    byre.compute @FillOp(%arg3) {value = dense<5.000000e-01> : tensor<1001xf16>} : memref<1001xf16, "cuda">
    byre.compute @FillOp(%arg4) {value = dense<7> : tensor<37xi64>} : memref<37xi64, "cuda">
    byre.compute @FillOp(%arg5) {value = dense<true> : tensor<3xi1>} : memref<3xi1, "cuda">
    return
  }
}
"""


def test_host_device_copies_and_fill_load():
    """cpu2cuda / cuda2cpu / FillOp are registered, take "cpu"-space memrefs in a CUDA session that also
    has the host allocator, and FillOp checks its constant against the tensor"""
    s = brt.Session("cuda", host_space=True)
    s.load_from_memory(HOST_DEVICE)
    assert [s.arg_info(i).space for i in range(6)] == ["cpu", "cpu", "cuda", "cuda", "cuda", "cuda"]
    assert s.arg_info(5).nbytes == 3  # i1 is stored one byte per element
    with pytest.raises(brt.BrtError, match="FillOp"):
        brt.Session("cuda", host_space=True).load_from_memory(
            HOST_DEVICE.replace("dense<[1.000000e+00, 2.000000e+00, 3.000000e+00]> : tensor<3xf16>",
                                "dense<[1.000000e+00, 2.000000e+00]> : tensor<2xf16>"))
    with pytest.raises(brt.BrtError, match="no allocator registered for memory space \"cpu\""):
        brt.Session("cuda").load_from_memory(HOST_DEVICE)  # a plain CUDA session has no host allocator


def test_compiler_written_modules_load_when_a_checkout_is_given():
    """With BYTEIR_CHECKOUT pointing at a checkout of the reference: its runtime fixtures written by the
    compiler (resnet18 forward / backward / both, 167 to 265 arguments, one arena with dozens of
    byre.alias views) and by hand (fill, cpu2cuda) load, once the ops outside this provider
    (PTX, cuDNN, cuBLAS kernels) are taken out of the text."""
    import os
    import re
    root = os.environ.get("BYTEIR_CHECKOUT")
    if not root or not (Path(root) / "runtime" / "test" / "test_files").is_dir():
        pytest.skip("BYTEIR_CHECKOUT is not set")
    ours = ("ReduceSumOp", "ReduceMaxOp", "IndexSelectOp", "IndexPutOp", "TransposeOp", "FillOp", "cpu2cuda", "cuda2cpu")
    files = {"resnet18_fw_host_cuda.mlir": 265, "resnet18_bw_host_cuda.mlir": 204, "resnet18_fw_bw_host_cuda.mlir": 167,
             "fill_cuda.mlir": 5, "custom_add_cpu2cuda.mlir": 3}
    for name, n_args in files.items():
        kept = []
        for line in (Path(root) / "runtime" / "test" / "test_files" / name).read_text().splitlines():
            m = re.search(r"byre\.compute @(\w+)\(", line)
            if m and not m.group(1).startswith(ours):
                continue
            kept.append(line)
        s = brt.Session("cuda", host_space=True)
        s.load_from_memory("\n".join(kept))
        assert len(s.args()) == n_args, name


def test_session_takes_device_memory_from_the_callers_functions():
    """Session(alloc_func, free_func): unbound arguments and intermediates come from the caller's
    allocator and go back to it (here host memory stands in for the device's); the reference's names
    of the binding answer too"""
    import ctypes
    live, sizes = {}, []

    def alloc(size):
        buf = ctypes.create_string_buffer(max(size, 1))
        live[ctypes.addressof(buf)] = buf
        sizes.append(size)
        return ctypes.addressof(buf)

    def free(ptr):
        del live[ptr]

    s = brt.Session("CUDA", alloc_func=alloc, free_func=free)
    s.load_from_memory(reduce_mlir("ReduceSumOp_f32_f32", "f32", (64, 32), (64,), "dense<1> : tensor<1xi64>"))
    assert s.get_input_arg_offsets() == [0] and s.get_output_arg_offsets() == [1]
    assert s.get_static_shape(0) == [64, 32] and s.get_data_type(1) == "f32"
    assert s.get_input_names() == ["Input0"] and s.get_output_names() == ["Output0"]
    # any non-null stream where there is no device (nothing is launched here); a real one where there is,
    # since closing the request waits for its stream
    import torch
    stream = torch.cuda.Stream().cuda_stream if torch.cuda.is_available() else 0x10
    req = s.new_request_context(stream)
    req.bind_args([(0, 0x1000)])
    req.finish_io_binding()             # the unbound output is allocated by the caller's function
    assert 64 * 4 in sizes and len(live) >= 1
    req.close()
    s.close()
    assert not live
    with pytest.raises(ValueError):
        brt.Session("cuda", alloc_func=alloc)


def test_damaged_text_is_an_error_not_a_crash():
    """400 random edits of valid modules (dropped, doubled and replaced characters, truncations): the
    loader answers with a Status or a loaded module, never with a fault"""
    rng = np.random.default_rng(7)
    alphabet = list('<>(){}[]"%@:,=x-+ \n') + list("0123456789abcdefmrt")
    sources = [ADD, HOST_DEVICE, reduce_mlir("ReduceSumOp_f32_f32", "f32", (64, 32), (64,), "dense<1> : tensor<1xi64>")]
    outcomes = {"ok": 0, "error": 0}
    for trial in range(400):
        text = list(sources[trial % len(sources)])
        for _ in range(int(rng.integers(1, 4))):
            pos = int(rng.integers(0, len(text)))
            kind = int(rng.integers(0, 4))
            if kind == 0:
                del text[pos]
            elif kind == 1:
                text.insert(pos, text[pos])
            elif kind == 2:
                text[pos] = alphabet[int(rng.integers(0, len(alphabet)))]
            else:
                del text[pos:]
        s = brt.Session("cuda", host_space=True) if trial % len(sources) else brt.Session("cpu")
        try:
            s.load_from_memory("".join(text))
            outcomes["ok"] += 1
        except brt.BrtError:
            outcomes["error"] += 1
        s.close()
    assert outcomes["error"] > 100  # most edits break the module
