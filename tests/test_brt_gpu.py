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
from test_brt_host import INDEX, TRANSPOSE, reduce_mlir

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
