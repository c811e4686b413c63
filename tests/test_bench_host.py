"""bench.py's host side without a GPU: the reference arm's line, the ByRE modules the end-to-end leg
loads, and the refusal to run the product arm without a CUDA device."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--only-primary"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["vs_baseline"] is None
    assert line["config"]["workload"] == "reduce_f16_64x512x1024_sum01_max2"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


def test_product_arm_refuses_to_run_without_a_cuda_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "3"], capture_output=True,
                         text=True, timeout=600, cwd=ROOT)
    assert out.returncode != 0
    assert "no CPU path" in (out.stderr + out.stdout)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_the_end_to_end_modules_of_configuration_2_load(world):
    """one upload of x, both ops of the configuration, two results; at N ranks the sum goes through nccl.AllReduce"""
    import bench
    from byteir_b200 import brt
    wl = bench.ReduceC2(0, world)
    text, binding = wl.plugin(None)
    s = brt.DistributedSession(0, world, device="cuda", device_id=0, host_space=True) if world > 1 else \
        brt.Session("cuda", host_space=True)
    s.load_from_memory(text)  # loading needs no device
    args = {a.name: a for a in s.args()}
    assert set(args) == set(binding) == {"X", "Sum", "Max"}
    assert args["X"].shape == (64, 512, 1024) and args["X"].space == "cpu" and args["X"].argtype == 1
    assert args["Sum"].shape == (1024,) and args["Max"].shape == (64, 512)
    assert ("nccl.AllReduce" in text) == (world > 1)
    assert wl.work() == 67_110_912 + 67_174_400  # the algorithmic bytes of the two ops
