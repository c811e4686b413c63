"""GPU tests through the drop-in boundary: a ByRE module (text, as byteir-opt
prints it) loaded into a brt Session with the CUDA provider, arguments bound to
device buffers, run on a CUDA stream, result compared with the CPU oracle.
The pattern of the reference's per-op tests (runtime/test/backends/cuda/providers/
default/kernel/*_test.cc): one-op module, run twice on one RequestContext."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from byteir_b200 import brt
from test_brt_host import HOST_DEVICE, INDEX, TRANSPOSE, reduce_mlir

pytestmark = pytest.mark.gpu


def _run(text, inputs, stream=True):
    """inputs: {arg name: numpy array}; returns {output name: numpy array}"""
    s = brt.Session("cuda")
    s.load_from_memory(text)
    req = s.new_request(torch.cuda.current_stream().cuda_stream if stream else None)
    held = {}
    for a in s.args():
        if a.argtype & 1:
            x = inputs[a.name]
            t = torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).cuda()
            assert t.numel() * t.element_size() == a.nbytes
            held[a.name] = t
            req.bind_arg(a.offset, t.data_ptr())
        else:
            t = torch.empty(a.nbytes, dtype=torch.uint8, device="cuda")
            held[a.name] = t
            req.bind_arg(a.offset, t.data_ptr())
    req.finish_io_binding()
    for _ in range(2):
        req.run()
        req.sync()
    torch.cuda.synchronize()
    out = {}
    np_dt = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "i64": np.int64}
    for a in s.args():
        if a.argtype & 2:
            out[a.name] = held[a.name].cpu().numpy().view(np_dt[a.dtype]).reshape(a.shape)
    req.close()
    s.close()
    return out


@pytest.mark.parametrize("stream", [True, False])
def test_reduce_sum_config1_through_session(stream):
    rng = np.random.default_rng(1234)
    x = rng.uniform(-1, 1, (1024, 4096)).astype(np.float32)
    out = _run(reduce_mlir("ReduceSumOp_f32_f32", "f32", (1024, 4096), (1024,), "dense<1> : tensor<1xi64>"),
               {"Input0": x}, stream)["Output0"]
    want = O.reduce("sum", x, 1024, 4096, 1)
    np.testing.assert_allclose(out, want, rtol=1e-5, atol=1e-5)


def test_reduce_multi_axis_f16_through_session():
    rng = np.random.default_rng(1235)
    x = rng.standard_normal((16, 128, 1024), dtype=np.float32).astype(np.float16)
    s = _run(reduce_mlir("ReduceSumOp_f16_f16", "f16", (16, 128, 1024), (1024,), "dense<[0, 1]> : tensor<2xi64>"),
             {"Input0": x})["Output0"]
    np.testing.assert_allclose(s.astype(np.float64), O.reduce("sum", x, 1, 16 * 128, 1024).astype(np.float64),
                               rtol=2e-2, atol=1e-2)
    m = _run(reduce_mlir("ReduceMaxOp_f16_f16", "f16", (16, 128, 1024), (16, 128), "dense<2> : tensor<1xi64>"),
             {"Input0": x})["Output0"]
    assert np.array_equal(m.reshape(-1).view(np.uint16), O.reduce("max", x, 16 * 128, 1024, 1).view(np.uint16))


@pytest.mark.parametrize("t,npdt", [("f32", np.float32), ("f16", np.float16)])
def test_index_select_and_put_through_session(t, npdt):
    rng = np.random.default_rng(7)
    table = rng.standard_normal((30522, 128)).astype(npdt)
    idx = rng.integers(0, 30522, 128).astype(np.int64)
    idx[5] = idx[9] = idx[77]  # duplicates
    upd = rng.standard_normal((128, 128)).astype(npdt)
    out = _run(INDEX.replace("%T", t).replace("%I", "i64"), {"Table": table, "Idx": idx, "Upd": upd})
    assert np.array_equal(out["Sel"], table[idx])
    want, _ = O.index_put_add(table, idx, upd)
    tol = 1e-5 if t == "f32" else 1e-3
    np.testing.assert_allclose(out["Put"].astype(np.float64), want.astype(np.float64), rtol=tol, atol=tol)


@pytest.mark.parametrize("perm", [(0, 2, 3, 1), (0, 3, 1, 2), (3, 1, 0, 2)])
def test_transpose_through_session(perm):
    x = np.random.default_rng(3).uniform(-1, 1, (10, 20, 30, 40)).astype(np.float16)
    out_shape = tuple(x.shape[p] for p in perm)
    text = TRANSPOSE.replace("%OUT", "x".join(map(str, out_shape))).replace("%PERM", str(list(perm)))
    out = _run(text, {"In": x})["Out"]
    assert np.array_equal(out, np.transpose(x, perm))


def test_get_arg_on_device_and_intermediates():
    """two chained ops through a planned intermediate, I/O allocated by the context"""
    text = """
module attributes {byre.container_module} {
  func.func @chain(%arg0: memref<64x256xf32, "cuda"> {byre.argname = "X", byre.argtype = 1 : i32},
                   %arg1: memref<64xf32, "cuda"> {byre.argname = "Y", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    %0 = memref.alloc() : memref<256x64xf32, "cuda">
    byre.compute @TransposeOp_f32_f32(%arg0, %0) {permutation = dense<[1, 0]> : tensor<2xi64>} : memref<64x256xf32, "cuda">, memref<256x64xf32, "cuda">
    byre.compute @ReduceMaxOp_f32_f32(%0, %arg1) {dimensions = dense<0> : tensor<1xi64>} : memref<256x64xf32, "cuda">, memref<64xf32, "cuda">
    return
  }
}
"""
    s = brt.Session("cuda")
    s.load_from_memory(text)
    req = s.new_request()
    x = np.random.default_rng(0).standard_normal((64, 256)).astype(np.float32)
    xin = req.get_arg(0)
    yout = req.get_arg(1)
    import ctypes as C
    cudart = C.CDLL("libcudart.so")
    cudart.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    assert cudart.cudaMemcpy(xin, x.ctypes.data, x.nbytes, 1) == 0
    req.run(); req.sync()
    y = np.empty(64, np.float32)
    assert cudart.cudaMemcpy(y.ctypes.data, yout, y.nbytes, 2) == 0
    assert np.array_equal(y, x.max(axis=1))
    assert s.arg_info(0).name == "X"


FLASH = """
module attributes {byre.container_module} {
  func.func @attn(%arg0 : memref<%QSHAPE, "cuda"> {byre.argname = "d_Out", byre.argtype = 1: i32},
                 %arg1 : memref<%QSHAPE, "cuda"> {byre.argname = "Q", byre.argtype = 1: i32},
                 %arg2 : memref<%QSHAPE, "cuda"> {byre.argname = "K", byre.argtype = 1: i32},
                 %arg3 : memref<%QSHAPE, "cuda"> {byre.argname = "V", byre.argtype = 1: i32},
                 %arg4 : memref<%QSHAPE, "cuda"> {byre.argname = "Out", byre.argtype = 2: i32},
                 %arg5 : memref<%LSHAPE, "cuda"> {byre.argname = "SoftmaxLse", byre.argtype = 2: i32},
                 %arg6 : memref<%QSHAPE, "cuda"> {byre.argname = "d_Q", byre.argtype = 2: i32},
                 %arg7 : memref<%QSHAPE, "cuda"> {byre.argname = "d_K", byre.argtype = 2: i32},
                 %arg8 : memref<%QSHAPE, "cuda"> {byre.argname = "d_V", byre.argtype = 2: i32},
                 %arg9 : memref<2xi64, "cuda"> {byre.argname = "RngState", byre.argtype = 2: i32},
                 %arg10 : memref<%LSHAPE, "cuda"> {byre.argname = "d_SoftmaxLse", byre.argtype = 2: i32},
                 %arg11 : memref<%ASHAPE, "cuda"> {byre.argname = "d_Q_accum", byre.argtype = 2: i32},
                 %arg12 : memref<1xf32, "cuda"> {byre.argname = "SoftmaxPtr", byre.argtype = 2: i32}) attributes {byre.entry_point} {
    "byre.custom"(%arg1, %arg2, %arg3, %arg9, %arg4, %arg5, %arg12) {callee = "custom", lib_path = "%LIB", api_name = "run_flash_attn_fwd", version = "2.5.3", extra_args = %EXTRA} : (memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<2xi64, "cuda">, memref<%QSHAPE, "cuda">, memref<%LSHAPE, "cuda">, memref<1xf32, "cuda">) -> ()
    "byre.custom"(%arg0, %arg1, %arg2, %arg3, %arg4, %arg5, %arg9, %arg6, %arg7, %arg8, %arg10, %arg11) {callee = "custom", lib_path = "%LIB", api_name = "run_flash_attn_bwd", version = "2.5.3", extra_args = %EXTRA} : (memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%LSHAPE, "cuda">, memref<2xi64, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%QSHAPE, "cuda">, memref<%LSHAPE, "cuda">, memref<%ASHAPE, "cuda">) -> ()
    return
  }
}
"""


@pytest.mark.parametrize("t", ["f16", "bf16"])
def test_flash_attn_fwd_bwd_custom_call_through_session(t):
    """the module of runtime/test/test_files/flash_attn_bwd.mlir, at head dim 128: forward then backward
    through byre.custom -> libflash_attn.so; bf16 memrefs select the bf16 entry points"""
    from pathlib import Path
    b, s, h, d = 1, 256, 3, 128
    lib = str(Path(__file__).resolve().parent.parent / "byteir_b200" / "_lib" / "libflash_attn.so")
    extra = [s * h * d] * 4 + [h * d] * 4 + [d] * 4 + [b, h, h, d, d]
    extra_s = "[" + ", ".join(f"{v} : i64" for v in extra) + f", {0.08838834764831845} : f32, " + \
        ", ".join(f"{v} : i64" for v in (s, s, s, s)) + ", 0.0 : f32, -1 : i64, 0 : i64]"
    text = (FLASH.replace("%QSHAPE", f"{b}x{s}x{h}x{d}x{t}").replace("%LSHAPE", f"{b}x{h}x{s}xf32")
            .replace("%ASHAPE", f"{b}x{h}x{s}x{d}xf32").replace("%LIB", lib).replace("%EXTRA", extra_s))
    rng = np.random.default_rng(21)
    mk = lambda: (rng.standard_normal((b, s, h, d), dtype=np.float32).astype(np.float16) if t == "f16"
                  else O.f32_to_bf16(rng.standard_normal((b, s, h, d), dtype=np.float32)))
    q, k, v, do = mk(), mk(), mk(), mk()
    out = _run(text, {"Q": q, "K": k, "V": v, "d_Out": do})
    scale = 0.08838834764831845
    wo, wl = O.flash_attn_fwd(q, k, v, scale, True)
    np.testing.assert_allclose(out["SoftmaxLse"], wl, rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(O.to_f32(out["Out"]), O.to_f32(wo), rtol=2e-2, atol=1e-2)
    wq, wk, wv = O.flash_attn_bwd(do, q, k, v, out["Out"], out["SoftmaxLse"], scale, True)
    for name, want in (("d_Q", wq), ("d_K", wk), ("d_V", wv)):
        np.testing.assert_allclose(O.to_f32(out[name]), O.to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)


def test_host_device_copies_and_fill_through_session():
    """the ops on either side of the compute ops in host-driven modules (the reference's
    custom_add_cpu2cuda.mlir and fill_cuda.mlir patterns): cpu2cuda, cuda2cpu, FillOp"""
    rng = np.random.default_rng(11)
    a_host = torch.from_numpy(rng.uniform(-1, 1, (1024, 256)).astype(np.float32)).pin_memory()
    sum_host = torch.zeros(1024, dtype=torch.float32).pin_memory()
    three = torch.zeros(3, dtype=torch.float16, device="cuda")
    halves = torch.zeros(1001, dtype=torch.float16, device="cuda")
    sevens = torch.zeros(37, dtype=torch.int64, device="cuda")
    flags = torch.zeros(3, dtype=torch.bool, device="cuda")
    s = brt.Session("cuda", host_space=True)
    s.load_from_memory(HOST_DEVICE)
    req = s.new_request(torch.cuda.current_stream().cuda_stream)
    for name, t in (("A", a_host), ("Sum", sum_host), ("Three", three), ("Halves", halves), ("Sevens", sevens),
                    ("Flags", flags)):
        info = s.arg_info(s.arg_offset(name))
        assert info.space == ("cpu" if not t.is_cuda else "cuda") and info.nbytes == t.numel() * t.element_size()
        req.bind_arg(info.offset, t.data_ptr())
    req.finish_io_binding()
    for _ in range(2):
        req.run()
        req.sync()
    torch.cuda.synchronize()
    want = O.reduce("sum", a_host.numpy(), 1024, 256, 1)
    np.testing.assert_allclose(sum_host.numpy(), want, rtol=1e-5, atol=1e-5)
    assert three.cpu().tolist() == [1.0, 2.0, 3.0]
    assert torch.all(halves == 0.5) and torch.all(sevens == 7) and torch.all(flags)
    req.close()
    s.close()


KVCACHE = """
module attributes {byre.container_module} {
  func.func @test_flash_attn_kvcache(%arg0 : memref<2x1x3x32xf16, "cuda"> {byre.argname = "Q", byre.argtype = 2: i32},
                 %arg1 : memref<2x128x3x32xf16, "cuda"> {byre.argname = "KCache", byre.argtype = 2: i32},
                 %arg2 : memref<2x128x3x32xf16, "cuda"> {byre.argname = "VCache", byre.argtype = 2: i32},
                 %arg3 : memref<2x1x3x32xf16, "cuda"> {byre.argname = "K", byre.argtype = 2: i32},
                 %arg4 : memref<2x1x3x32xf16, "cuda"> {byre.argname = "V", byre.argtype = 2: i32},
                 %arg5: memref<2xi32, "cuda"> {byre.argname = "SeqLenK", byre.argtype = 2: i32},
                 %arg6: memref<2x1x3x32xf16, "cuda"> {byre.argname = "Output", byre.argtype = 2: i32},
                 %arg7 : memref<2x3x1xf32, "cuda"> {byre.argname = "SoftmaxLse", byre.argtype = 2: i32}) attributes {byre.entry_point} {
    "byre.custom"(%arg0, %arg1, %arg2, %arg3, %arg4, %arg5, %arg6, %arg7) {callee = "custom", lib_path = "%LIB", api_name = "run_flash_attn_kvcache", version = "2.5.3", extra_args = [96 : i64, 12288 : i64, 12288 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 96 : i64, 32 : i64, 32 : i64, 32 : i64, 32 : i64, 32 : i64, 32 : i64, 2 : i64, 3 : i64, 3 : i64, 32 : i64, 32 : i64, 1 : i64, 0.5 : f32, 1 : i64, 128 : i64, 128 : i64, 128 : i64, -1 : i64, -1 : i64]} : (memref<2x1x3x32xf16, "cuda">, memref<2x128x3x32xf16, "cuda">, memref<2x128x3x32xf16, "cuda">, memref<2x1x3x32xf16, "cuda">, memref<2x1x3x32xf16, "cuda">, memref<2xi32, "cuda">, memref<2x1x3x32xf16, "cuda">, memref<2x3x1xf32, "cuda">) -> ()
    return
  }
}
"""


def test_flash_attn_kvcache_custom_call_through_session():
    """the module and the vectors of the reference's kv-cache test (runtime/test/test_files/
    flash_attn_kvcache.mlir, flash_attn_fwd_test.cc:183-330) through byre.custom -> libflash_attn.so"""
    from pathlib import Path
    root = Path(__file__).resolve().parent
    lib = str(root.parent / "byteir_b200" / "_lib" / "libflash_attn.so")
    g = np.load(root / "golden" / "flash_attn_kvcache_b2_s128_h3_d32_f16.npz")
    dev = {"Q": g["q"], "KCache": g["kcache"], "VCache": g["vcache"], "K": g["k"], "V": g["v"],
           "SeqLenK": g["cache_seqlens"], "Output": np.zeros((2, 1, 3, 32), np.float16),
           "SoftmaxLse": np.zeros((2, 3, 1), np.float32)}
    dev = {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in dev.items()}
    s = brt.Session("cuda")
    s.load_from_memory(KVCACHE.replace("%LIB", lib))
    req = s.new_request(torch.cuda.current_stream().cuda_stream)
    for a in s.args():
        assert a.nbytes == dev[a.name].numel() * dev[a.name].element_size()
        req.bind_arg(a.offset, dev[a.name].data_ptr())
    req.finish_io_binding()
    req.run()
    req.sync()
    torch.cuda.synchronize()
    assert np.array_equal(dev["KCache"].cpu().numpy(), g["kcache_out"])
    assert np.array_equal(dev["VCache"].cpu().numpy(), g["vcache_out"])
    got, want = dev["Output"].cpu().numpy().astype(np.float32), g["out"].astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=0)
    assert torch.isfinite(dev["SoftmaxLse"]).all()
    req.close()
    s.close()


def test_bytecode_module_runs_on_the_gpu(tmp_path):
    """a ByRE bytecode file (byre_serial 1.0.0): an arena, two views of it, a transpose into one, a column
    sum into the other, a max over the rows of the transpose; same results as the oracle"""
    from byre_bytecode_writer import write_module
    desc = {"name": "main",
            "args": [("X", 1, "f32", (64, 256), "cuda"), ("ColSum", 2, "f32", (64,), "cuda"), ("RowMax", 2, "f32", (64,), "cuda")],
            "ops": [("alloc", "i8", (65536 + 256,), "cuda"),
                    ("alias", 3, 0, "f32", (256, 64), "cuda"),
                    ("alias", 3, 65536, "f32", (64,), "cuda"),
                    ("compute", "TransposeOp_f32_f32", [0, 4], {"permutation": ("dense", "i64", (2,), [1, 0])}, [1, 2]),
                    ("compute", "ReduceSumOp_f32_f32", [4, 5], {"dimensions": ("dense", "i64", (1,), [0])}, [1, 2]),
                    ("copy", 5, 1, "cuda2cuda"),
                    ("compute", "ReduceMaxOp_f32_f32", [4, 2], {"dimensions": ("array", "i64", [0])}, [1, 2])]}
    path = tmp_path / "m.mlirbc"
    path.write_bytes(write_module(desc))
    s = brt.Session("cuda")
    s.load(str(path))
    x = np.random.default_rng(3).standard_normal((64, 256)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    col, row = torch.zeros(64, device="cuda"), torch.zeros(64, device="cuda")
    req = s.new_request(torch.cuda.current_stream().cuda_stream)
    for name, t in (("X", xd), ("ColSum", col), ("RowMax", row)):
        req.bind_arg(s.arg_offset(name), t.data_ptr())
    req.finish_io_binding()
    req.run()
    req.sync()
    torch.cuda.synchronize()
    np.testing.assert_allclose(col.cpu().numpy(), x.astype(np.float64).sum(axis=1), rtol=1e-5, atol=1e-4)
    assert np.array_equal(row.cpu().numpy(), x.max(axis=1))
    req.close()
    s.close()


def test_backend_run_and_profile_with_the_torch_allocator(tmp_path):
    """BRTBackend as the reference's users drive it: device memory from torch's caching allocator, torch's
    current stream, run / run_with_outputs / profile"""
    from byteir_b200.backend import BRTBackend
    path = tmp_path / "reduce.mlir"
    path.write_text(reduce_mlir("ReduceSumOp_f16_f16", "f16", (64, 512, 1024), (1024,), "dense<[0, 1]> : tensor<2xi64>"))
    be = BRTBackend("cuda", str(path))
    assert be.input_shapes == [[64, 512, 1024]] and be.output_dtypes == [torch.float16]
    x = torch.from_numpy(np.random.default_rng(5).uniform(-1, 1, (64, 512, 1024)).astype(np.float16)).cuda()
    want = O.reduce("sum", x.cpu().numpy(), 1, 64 * 512, 1024).reshape(-1).astype(np.float32)
    (out,) = be.run([x])
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=2e-2, atol=1e-2)
    out2 = torch.zeros(1024, dtype=torch.float16, device="cuda")
    be.run_with_outputs([x], [out2])
    assert torch.equal(out, out2)
    (out3,), ms = be.profile([x], warmup_trials=2, run_trials=5)
    assert torch.equal(out, out3) and 0 < ms < 50
    with pytest.raises(AssertionError):
        be.run([x.float()])


# ---- the exchange step and multi-group reductions through the boundary ---------------------------------------
SHARDED_SUM = """
module attributes {byre.container_module} {
  func.func @main(%arg0: memref<8x64x256xf16, "cuda"> {byre.argname = "X", byre.argtype = 1 : i32},
                  %arg1: memref<256xf16, "cuda"> {byre.argname = "Sum", byre.argtype = 2 : i32}) attributes {byre.entry_point} {
    %0 = memref.alloc() : memref<256xf32, "cuda">
    byre.compute @ReduceSumOp_f16_f32(%arg0, %0) {dimensions = dense<[0, 1]> : tensor<2xi64>, memory_effects = [1 : i32, 2 : i32]} : memref<8x64x256xf16, "cuda">, memref<256xf32, "cuda">
    byre.compute @nccl.AllReduce(%0, %arg1) {reduction = "sum", replica_group = [0], memory_effects = [1 : i32, 2 : i32]} : memref<256xf32, "cuda">, memref<256xf16, "cuda">
    return
  }
}
"""


@pytest.mark.parametrize("backend", ["peer", "callback"])
def test_sharded_sum_module_on_one_rank(backend):
    """a rank's module of the sum whose reduced axis is sharded: unrounded f32 partial sums, then nccl.AllReduce
    into an f16 target (rounded once).  World of one rank: the peer-memory kernel talks to its own inbox; the
    callback communicator copies send to recv on the request's stream and the op casts afterwards.  Either way the
    bits equal the unsharded ReduceSumOp_f16_f16."""
    from byteir_b200 import ops, _native as N
    rng = np.random.default_rng(41)
    x = rng.standard_normal((8, 64, 256), dtype=np.float32).astype(np.float16)
    xd = torch.from_numpy(x).cuda()
    out = torch.zeros(256, dtype=torch.float16, device="cuda")
    s = brt.DistributedSession(0, 1, device="cuda", device_id=0)
    s.load_from_memory(SHARDED_SUM)
    stream = torch.cuda.Stream()
    calls = []
    if backend == "peer":
        n = 256
        inbox = torch.zeros(N.lib().b200_sharded_sum_inbox_bytes(1, n) // 4, dtype=torch.float32, device="cuda")
        flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        s.set_allreduce_peer(n, [inbox.data_ptr()], [flags.data_ptr()], counter.data_ptr(), status.data_ptr())
    else:
        import ctypes as C
        cudart = C.CDLL("libcudart.so")
        cudart.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]

        def all_reduce(send, recv, n, dtype, op, group, st):
            calls.append((n, dtype, op, tuple(group), st))
            assert cudart.cudaMemcpyAsync(recv, send, n * 4, 3, st) == 0  # one rank: the sum is the vector itself
        s.set_allreduce(all_reduce)
    torch.cuda.synchronize()
    req = s.new_request(stream.cuda_stream)
    req.bind_arg(s.arg_offset("X"), xd.data_ptr())
    req.bind_arg(s.arg_offset("Sum"), out.data_ptr())
    req.finish_io_binding()
    for _ in range(3):
        req.run()
        req.sync()
    torch.cuda.synchronize()
    want = ops.reduce_sum(xd, [0, 1])
    assert torch.equal(out, want)
    np.testing.assert_allclose(out.float().cpu().numpy(), x.astype(np.float64).sum(axis=(0, 1)), rtol=2e-2, atol=1e-2)
    if backend == "peer":
        assert int(status.item()) == 0 and int(counter.item()) == 3
    else:
        assert calls[0] == (256, "f32", "sum", (0,), stream.cuda_stream)
    req.close()
    s.close()


@pytest.mark.parametrize("t,npdt", [("f32", np.float32), ("f16", np.float16)])
@pytest.mark.parametrize("shape,dims", [((6, 50, 36), (0, 2)), ((3, 4, 5, 16, 7), (0, 2, 3)), ((9, 1, 8, 20), (0, 1, 3))])
def test_reduce_over_dimensions_that_are_not_consecutive(shape, dims, t, npdt):
    """the reference refuses these at load time (reduce_impl.h:40-42); here the groups of consecutive dimensions
    are reduced one after the other, a 16-bit sum through f32 intermediates so that it is rounded once"""
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(npdt)
    out_shape = tuple(s for i, s in enumerate(shape) if i not in dims)
    dims_s = "dense<[" + ", ".join(map(str, dims)) + f"]> : tensor<{len(dims)}xi64>"
    s = _run(reduce_mlir(f"ReduceSumOp_{t}_{t}", t, shape, out_shape, dims_s), {"Input0": x})["Output0"]
    want = x.astype(np.float64).sum(axis=dims)
    tol = dict(rtol=1e-5, atol=1e-4) if t == "f32" else dict(rtol=2e-3, atol=2e-2)
    np.testing.assert_allclose(s.astype(np.float64), want, **tol)
    m = _run(reduce_mlir(f"ReduceMaxOp_{t}_{t}", t, shape, out_shape, dims_s), {"Input0": x})["Output0"]
    assert np.array_equal(m, x.max(axis=dims))


def test_cuda_kernel_plugin_runs():
    """the plug-in of the integration notes (tests/cpp/cuda_plugin.cc) on configuration 2's sum"""
    from test_brt_host import cuda_plugin
    cuda_plugin()
    x = np.random.default_rng(5).standard_normal((64, 512, 1024), dtype=np.float32).astype(np.float16)
    text = reduce_mlir("PluginReduceSumOp_f16_f16", "f16", x.shape, (1024,), "dense<[0, 1]> : tensor<2xi64>")
    got = _run(text, {"Input0": x})["Output0"]
    want = O.reduce("sum", x, 1, 64 * 512, 1024)
    np.testing.assert_allclose(got.astype(np.float64), want.astype(np.float64), rtol=2e-2, atol=1e-2)
    # the same kernels behind the built-in key: the same bits
    builtin = _run(reduce_mlir("ReduceSumOp_f16_f16", "f16", x.shape, (1024,), "dense<[0, 1]> : tensor<2xi64>"), {"Input0": x})["Output0"]
    assert np.array_equal(got.view(np.uint16), builtin.view(np.uint16))


def test_group_copy_from_bytecode_runs_on_the_gpu(tmp_path):
    from byre_bytecode_writer import write_module
    desc = {"name": "main",
            "args": [("A", 1, "f32", (1000,), "cuda"), ("B", 1, "f16", (33, 7), "cuda"), ("OutA", 2, "f32", (1000,), "cuda"),
                     ("OutB", 2, "f16", (33, 7), "cuda")],
            "ops": [("group_copy", [0, 1], [2, 3], "cuda2cuda")]}
    s = brt.Session("cuda")
    s.load_from_memory(write_module(desc))
    a = torch.randn(1000, device="cuda")
    b = torch.randn(33, 7, device="cuda").half()
    oa, ob = torch.zeros_like(a), torch.zeros_like(b)
    req = s.new_request(torch.cuda.current_stream().cuda_stream)
    for name, t in (("A", a), ("B", b), ("OutA", oa), ("OutB", ob)):
        req.bind_arg(s.arg_offset(name), t.data_ptr())
    req.finish_io_binding()
    req.enable_op_trace()
    req.run()
    req.sync()
    torch.cuda.synchronize()
    assert torch.equal(oa, a) and torch.equal(ob, b)
    assert req.op_trace() == ["cuda2cuda", "cuda2cuda"]
    req.close()
    s.close()


def test_the_references_own_attention_modules_run_unchanged(tmp_path, monkeypatch):
    """runtime/test/test_files/flash_attn_fwd.mlir and flash_attn_bwd.mlir, byte for byte (head dim 32, fp16, the
    library named by a path relative to the working directory, as the compiler writes it), with the reference's
    vectors: what flash_attn_fwd_test.cc and flash_attn_bwd_test.cc do"""
    from pathlib import Path
    golden = Path(__file__).resolve().parent / "golden"
    libdir = tmp_path / "test" / "test_files" / "external_libs"
    libdir.mkdir(parents=True)
    (libdir / "libflash_attn.so").symlink_to(golden.parent.parent / "byteir_b200" / "_lib" / "libflash_attn.so")
    monkeypatch.chdir(tmp_path)
    g = np.load(golden / "flash_attn_b1_s128_h3_d32_f16.npz")
    names = {"Q": "q", "K": "k", "V": "v", "d_Out": "dout"}
    for module in ("flash_attn_fwd.mlir", "flash_attn_bwd.mlir"):
        s = brt.Session("cuda")
        s.load(str(golden / module))
        req = s.new_request(torch.cuda.current_stream().cuda_stream)
        held = {}
        for a in s.args():
            if a.name in names:
                t = torch.from_numpy(g[names[a.name]]).cuda()
            else:
                t = torch.zeros(a.nbytes, dtype=torch.uint8, device="cuda")
            assert t.numel() * t.element_size() == a.nbytes
            held[a.name] = t
            req.bind_arg(a.offset, t.data_ptr())
        req.finish_io_binding()
        req.run()
        req.sync()
        torch.cuda.synchronize()
        view = lambda n: held[n].view(torch.float16).reshape(1, 128, 3, 32).cpu().numpy()
        key = lambda x: np.where(x.view(np.uint16) & 0x8000, -(x.view(np.uint16).astype(np.int32) & 0x7fff),
                                 x.view(np.uint16).astype(np.int32))
        assert np.abs(key(view("Out")) - key(g["out"])).max() <= 1
        if module == "flash_attn_bwd.mlir":
            for arg, name in (("d_Q", "dq"), ("d_K", "dk"), ("d_V", "dv")):
                np.testing.assert_allclose(view(arg).astype(np.float32), g[name].astype(np.float32), rtol=2e-2, atol=1e-2,
                                           err_msg=name)
        req.close()
        s.close()
