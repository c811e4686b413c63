"""Pack the reference's flash-attention golden vectors into one small .npz.

The reference stores them as text (space separated floats, one file per
tensor) under runtime/test/test_files/flash_attn_*.data; they were produced by
runtime/test/test_files/generate_flash_attn_ground_truth.py with the upstream
flash-attn package: b=1, seqlen=128, heads=3, head_dim=32, fp16, causal,
softmax scale 0.5.  The reference's own tests round these values to fp16 and
demand a bit-exact match (runtime/test/backends/cuda/providers/default/kernel/
flash_attn_fwd_test.cc:142), so fp16 is a lossless container for them.

The kv-cache vectors (flash_attn_kvcache_*.data, same generator script, lines 56-105)
go to a second file: b=2, cache of 128 rows with 64 in use, one new row, heads=3,
head_dim=32, fp16, scale 0.5; inputs q/k/v/kcache/vcache/cache_seqlens, outputs out
and the two updated caches.

It also copies the reference's one ByRE bytecode fixture (runtime/test/test_files/LLJIT/
Case0_v1_0_0/entry.mlirbc, 447 bytes, byre_serial 1.0.0 in an MLIR 17 container) to
byre_serial_v1_lljit_case0.mlirbc; its text twin is LLJIT/Case0/entry.mlir.  The compiler's own end-to-end
test holds the same module under another producer string (compiler/test/E2E/Host/Case0_Bytecode/
Output.mlirbc, 448 bytes): copied to byre_serial_v1_host_case0_bytecode.mlirbc.

The reference's three flash-attention test modules (runtime/test/test_files/flash_attn_fwd.mlir,
flash_attn_bwd.mlir, flash_attn_kvcache.mlir: a few lines of ByRE text each, with the packed
`extra_args` the compiler writes for the custom call) are copied as fixtures too, so that the GPU
tests run the reference's own modules, not restatements of them.

Run where a checkout of the reference is at hand:
    python tests/golden/make_flash_attn_golden.py <path to the byteir checkout>
"""
import sys
from pathlib import Path

import numpy as np

SHAPE = (1, 128, 3, 32)
NAMES = {
    "q": "flash_attn_inputs_q.data",
    "k": "flash_attn_inputs_k.data",
    "v": "flash_attn_inputs_v.data",
    "dout": "flash_attn_inputs_dout.data",
    "out": "flash_attn_fwd_outputs.data",
    "dq": "flash_attn_bwd_outputs_dq.data",
    "dk": "flash_attn_bwd_outputs_dk.data",
    "dv": "flash_attn_bwd_outputs_dv.data",
}


KV_NAMES = {  # key -> (file, shape)
    "q": ("flash_attn_kvcache_inputs_q.data", (2, 1, 3, 32)),
    "k": ("flash_attn_kvcache_inputs_k.data", (2, 1, 3, 32)),
    "v": ("flash_attn_kvcache_inputs_v.data", (2, 1, 3, 32)),
    "kcache": ("flash_attn_kvcache_inputs_kcache.data", (2, 128, 3, 32)),
    "vcache": ("flash_attn_kvcache_inputs_vcache.data", (2, 128, 3, 32)),
    "out": ("flash_attn_kvcache_outputs.data", (2, 1, 3, 32)),
    "kcache_out": ("flash_attn_kvcache_outputs_kcache.data", (2, 128, 3, 32)),
    "vcache_out": ("flash_attn_kvcache_outputs_vcache.data", (2, 128, 3, 32)),
}


def read_f16(path: Path, shape) -> np.ndarray:
    vals = np.array(path.read_text().split(), dtype=np.float64)
    assert vals.size == int(np.prod(shape)), (path.name, vals.size)
    f16 = vals.astype(np.float16)
    assert np.array_equal(f16.astype(np.float64), vals), path.name
    return f16.reshape(shape)


def kvcache(src: Path) -> None:
    arrays = {key: read_f16(src / fname, shape) for key, (fname, shape) in KV_NAMES.items()}
    lens = np.array((src / "flash_attn_kvcache_inputs_cache_seqlens.data").read_text().split(), dtype=np.int32)
    assert lens.shape == (2,)
    arrays["cache_seqlens"] = lens
    out = Path(__file__).with_name("flash_attn_kvcache_b2_s128_h3_d32_f16.npz")
    np.savez_compressed(out, **arrays)
    print("wrote", out, out.stat().st_size, "bytes")


def main(ref_root: str) -> None:
    src = Path(ref_root) / "runtime" / "test" / "test_files"
    kvcache(src)
    for name in ("flash_attn_fwd.mlir", "flash_attn_bwd.mlir", "flash_attn_kvcache.mlir"):
        text = (src / name).read_text()
        assert "byre.custom" in text and "libflash_attn.so" in text, name
        Path(__file__).with_name(name).write_text(text)
        print("copied", name, len(text), "bytes")
    bc = (src / "LLJIT" / "Case0_v1_0_0" / "entry.mlirbc").read_bytes()
    assert bc[:4] == b"ML\xefR"
    Path(__file__).with_name("byre_serial_v1_lljit_case0.mlirbc").write_bytes(bc)
    # the same module as the compiler's end-to-end test writes it (another producer string)
    bc2 = (src.parents[2] / "compiler" / "test" / "E2E" / "Host" / "Case0_Bytecode" / "Output.mlirbc").read_bytes()
    assert bc2[:4] == b"ML\xefR"
    Path(__file__).with_name("byre_serial_v1_host_case0_bytecode.mlirbc").write_bytes(bc2)
    arrays = {}
    for key, fname in NAMES.items():
        vals = np.array((src / fname).read_text().split(), dtype=np.float64)
        assert vals.size == int(np.prod(SHAPE)), (fname, vals.size)
        f16 = vals.astype(np.float16)
        # the text was printed from fp16 tensors: the round trip must be exact
        assert np.array_equal(f16.astype(np.float64), vals), fname
        arrays[key] = f16.reshape(SHAPE)
    out = Path(__file__).with_name("flash_attn_b1_s128_h3_d32_f16.npz")
    np.savez_compressed(out, **arrays)
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_flash_attn_golden.py <path to the byteir checkout>")
    main(sys.argv[1])
