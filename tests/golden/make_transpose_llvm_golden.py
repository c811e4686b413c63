"""A transpose golden vector made by the reference's own CPU code.

runtime/test/test_files/LLJIT/transpose_32_64_64.ll is the LLVM IR the reference's compiler emitted for
compiler/test/E2E/Host/Transpose/00_Input.mlir: f32 [1, 32, 64, 64] -> permutation (0, 2, 3, 1), entry
_mlir_ciface_Unknown0(memref descriptor *in, memref descriptor *out), which the reference's CPU provider
runs through its LLVM JIT (runtime/test/backends/cpu/device/llvm_jit_test.cc:166-230); transpose_3_224_224.ll
is the same for f32 [1, 3, 224, 224].  This script runs that IR with llvmlite's JIT on the input 0, 1, 2, ... (every
element distinct and exact in f32, which pins a pure permutation completely, and the output compresses to
a few kilobytes) and stores what comes out in transpose_f32_1x32x64x64_perm0231.npz and
transpose_f32_1x3x224x224_perm0231.npz; tests/test_oracle.py
compares the oracle, and the GPU tests the kernel, with the stored output.

Run where a checkout of the reference is at hand (llvmlite is needed only here):
    python tests/golden/make_transpose_llvm_golden.py <path to the byteir checkout>
"""
import ctypes as C
import os
import sys
from pathlib import Path

import numpy as np

PERM = (0, 2, 3, 1)
CASES = [("transpose_32_64_64.ll", (1, 32, 64, 64)), ("transpose_3_224_224.ll", (1, 3, 224, 224))]


def make_input(shape):
    return np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)  # exact in f32


class MemRef4(C.Structure):
    _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_int64),
                ("sizes", C.c_int64 * 4), ("strides", C.c_int64 * 4)]


def descriptor(a):
    strides = [s // a.itemsize for s in a.strides]
    return MemRef4(a.ctypes.data, a.ctypes.data, 0, (C.c_int64 * 4)(*a.shape), (C.c_int64 * 4)(*strides))


def main():
    import llvmlite.binding as llvm
    ref = Path(sys.argv[1])
    llvm.initialize_native_target()
    llvm.initialize_native_asmprinter()
    llvm.initialize_native_asmparser()  # the IR holds inline assembly
    # ... and AVX in it: the target machine needs the host's vector features
    tm = llvm.Target.from_default_triple().create_target_machine(cpu=llvm.get_host_cpu_name(),
                                                                 features=llvm.get_host_cpu_features().flatten())
    keep = []  # engines and their modules stay alive until the end
    for file, shape in CASES:
        mod = llvm.parse_assembly((ref / "runtime/test/test_files/LLJIT" / file).read_text())
        mod.verify()
        engine = llvm.create_mcjit_compiler(mod, tm)
        engine.finalize_object()
        keep.append((mod, engine))
        fn = C.CFUNCTYPE(None, C.POINTER(MemRef4), C.POINTER(MemRef4))(engine.get_function_address("_mlir_ciface_Unknown0"))
        x = make_input(shape)
        out = np.full([shape[p] for p in PERM], -1.0, np.float32)
        dx, do = descriptor(x), descriptor(out)
        fn(C.byref(dx), C.byref(do))
        assert out.min() >= 0 and np.array_equal(np.sort(out.reshape(-1)), np.arange(out.size, dtype=np.float32))
        dst = Path(__file__).parent / ("transpose_f32_%s_perm0231.npz" % "x".join(str(v) for v in shape))
        # stored as differences along the flat output (a permutation of 0, 1, 2, ... is regular: they compress
        # to a few kilobytes); out = cumsum(delta)
        flat = out.reshape(-1).astype(np.int64)
        np.savez_compressed(dst, shape=np.array(shape), perm=np.array(PERM),
                            delta=np.diff(flat, prepend=0).astype(np.int32))
        print(dst, dst.stat().st_size, "bytes", flush=True)
    os._exit(0)  # two JIT engines with the same symbol names do not tear down cleanly; the files are written


if __name__ == "__main__":
    main()
