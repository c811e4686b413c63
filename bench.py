#!/usr/bin/env python
"""Benchmark of the ByRE compute-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one pass of the named workload over one batch of seeded synthetic
input.  The default workload is the f16 [64, 512, 1024] multi-axis reduction
(ReduceSum over dims {0,1} + ReduceMax over dim 2); the others are selected with
--workload.  One JSON line is printed by rank 0.

  value     whole-job throughput with inputs resident in HBM, CUDA-event timed
  e2e       same metric with host buffers: pinned host -> device copy of the
            step's inputs, the op, device -> host copy of its result, all inside
            the timed region
  roofline  the dominant kernel's algorithmic bytes (or FLOPs) per launch over its
            own event-timed duration, against the measured peak
  cpu_baseline  the CPU oracle (a restatement of the reference's op semantics) on
            this host's cores, on a bounded sample of the same workload

Multi-GPU: one process per GPU (torchrun); every rank processes its own batch
(weak scaling).  Only the dim-0-sharded sum exchanges data: an NCCL all-reduce of
the f32 partial sums before the single rounding to f16.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, in bytes,
# from the ncu captures summarised under profiles/ (absent = not captured).  The attention
# figure was captured on B=1, H=16 (50.4 MB read + 1.0 MB written) and is scaled by the
# 16x more (batch, head) pairs of the bench workload; the writes of a launch mostly stay
# in L2 until after the kernel, so they under-count.
NCU_TRAFFIC = {
    "reduce_c2": 67.126e6 + 0.57e6,      # reduce_cols_kernel (profiles/cols_ncu_full.md)
    "gather": 62.25e6 + 24.40e6,         # gather_generic_kernel (profiles/gather_ncu_full.md)
    "scatter": 81.86e6 + 5.33e6,         # scatter_chunk_kernel alone (profiles/chunk_ncu_full.md)
    "attn": 16 * (50.40e6 + 0.98e6),     # flash_fwd_kernel<bf16> (profiles/flash_fwd_ncu_full.md)
    "decode": 452.36e6 + 4.24e6,         # decode_mma_kernel<128, bf16> (profiles/decode_ncu_full.md)
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons while the timed region runs"""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------
def zipf_indices(rng, n, rows, s=1.1):
    w = 1.0 / np.arange(1, rows + 1, dtype=np.float64) ** s
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n))
    return rng.permutation(rows)[np.minimum(ranks, rows - 1)].astype(np.int64)


class Workload:
    """One configuration: builds host inputs, runs a step on the GPU, and runs the
    same step on the CPU oracle."""
    name = ""
    unit = "GB/s"
    dtype = ""
    bound = "hbm"

    def work_per_step(self):  # algorithmic bytes (or FLOPs) of one step on one GPU
        raise NotImplementedError

    def end_batch(self):  # joins whatever a batch of pipelined steps left running beside the stream
        pass

    def dominant(self):  # (kernel name, algorithmic work per launch)
        raise NotImplementedError


class ReduceC2(Workload):
    """f16 [64, 512, 1024] N(0,1): ReduceSum dims {0,1} -> f16 [1024]; ReduceMax dim 2 -> f16 [64, 512]"""
    name = "reduce_f16_64x512x1024_sum01_max2"
    dtype = "f16 (f32 accumulate)"
    shape = (64, 512, 1024)
    SUM_BYTES = 64 * 512 * 1024 * 2 + 1024 * 2
    MAX_BYTES = 64 * 512 * 1024 * 2 + 64 * 512 * 2

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def host_inputs(self, n_buffers):
        rng = np.random.default_rng(1234 + 1 + 1000 * self.rank)
        return [rng.standard_normal(self.shape, dtype=np.float32).astype(np.float16) for _ in range(n_buffers)]

    def work_per_step(self):
        return self.SUM_BYTES + self.MAX_BYTES

    def launches_per_step(self):
        return 3 + (1 if self.world > 1 else 0)  # column pass, finalize, row max (+ exchange/cast kernel)

    def dominant(self):
        return "reduce_cols_kernel+reduce_finalize_kernel (ReduceSum dims {0,1})", self.SUM_BYTES

    def setup_gpu(self, torch, ops, xs):
        self.torch, self.ops = torch, ops
        self.out_sum = torch.empty(1024, dtype=torch.float16, device="cuda")
        self.out_max = torch.empty(64, 512, dtype=torch.float16, device="cuda")
        self.part = torch.empty(1024, dtype=torch.float32, device="cuda")
        from byteir_b200 import _native as N
        need = N.lib().b200_reduce_workspace_bytes(0, N.F16, 1, 64 * 512, 1024)
        self.ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
        self.exchange = "none"
        self.sharded = None
        if self.world > 1:
            self.exchange = "nccl all-reduce + cast"
            if os.environ.get("B200_EXCHANGE", "peer") == "peer":
                try:
                    self._setup_peer_exchange(torch, ops, N)
                    self.exchange = "b200_sharded_sum_finish (one kernel over NVLink peer memory)"
                except Exception as e:  # symmetric memory unavailable: keep NCCL
                    print(f"peer-memory exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)

    def _setup_peer_exchange(self, torch, ops, N):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        n = 1024
        inbox_bytes = N.lib().b200_sharded_sum_inbox_bytes(self.world, n)
        flag_off = (inbox_bytes + 255) // 256 * 256
        total = flag_off + 256
        buf = symm_mem.empty(total // 4, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier()  # every inbox and flag word is zero before anyone publishes
        self._symm = (buf, hdl)
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.sharded = ops.ShardedSum(self.rank, self.world, n, ptrs, [p + flag_off for p in ptrs],
                                      self.counter, self.status)
        self.side = torch.cuda.Stream()
        self.parts = [self.part, torch.empty_like(self.part)]
        self.xdone = [torch.cuda.Event(), torch.cuda.Event()]
        self.kstep = 0

    def step_gpu(self, x, dist=None, pipelined=False):
        ops = self.ops
        if self.world > 1 and self.sharded is not None:
            # The reduced axis (dim 0 of the global [64 * world, 512, 1024] tensor) is sharded.  The
            # exchange of the 4 KiB of f32 partials (one block, NVLink latency) runs on a side stream
            # beside the max reduction (whole GPU, HBM-bound).  Inside a batch of back-to-back steps
            # (pipelined) the step does not wait for its exchange: it overlaps the next step as well,
            # the partials alternate between two buffers, and end_batch() joins the side stream.
            torch = self.torch
            cur = torch.cuda.current_stream()
            k = self.kstep
            part = self.parts[k & 1]
            if k >= 2:
                cur.wait_event(self.xdone[k & 1])  # the exchange two steps back has read this buffer
            ops.reduce_sum_to_f32(x, [0, 1], out=part, workspace=self.ws)
            self.side.wait_stream(cur)
            with torch.cuda.stream(self.side):
                self.sharded(part, self.out_sum)
                self.xdone[k & 1].record(self.side)
            ops.reduce_max(x, [2], out=self.out_max)
            self.kstep = k + 1
            if not pipelined:
                self.end_batch()
        elif self.world > 1:
            # comparison path: NCCL all-reduce of the partials beside the max reduction, then the cast
            ops.reduce_sum_to_f32(x, [0, 1], out=self.part, workspace=self.ws)
            work = dist.all_reduce(self.part, async_op=True)
            ops.reduce_max(x, [2], out=self.out_max)
            work.wait()
            ops.cast_from_f32(self.part, self.torch.float16, out=self.out_sum)
        else:
            ops.reduce_sum(x, [0, 1], out=self.out_sum, workspace=self.ws)
            ops.reduce_max(x, [2], out=self.out_max)
        return self.out_sum, self.out_max

    def end_batch(self):
        if self.world > 1 and self.sharded is not None:
            self.torch.cuda.current_stream().wait_stream(self.side)
            self.kstep = 0

    def dominant_gpu(self, x):
        self.ops.reduce_sum(x, [0, 1], out=self.out_sum, workspace=self.ws)

    def result_bytes(self):
        return 1024 * 2 + 64 * 512 * 2

    def step_cpu(self, O, x):
        O.reduce("sum", x, 1, 64 * 512, 1024)
        O.reduce("max", x, 64 * 512, 1024, 1)

    def check(self, O, x, outs):
        s, m = (o.cpu().numpy() for o in outs)
        if self.world == 1:
            want = O.reduce("sum", x, 1, 64 * 512, 1024)
            np.testing.assert_allclose(s.astype(np.float64), want.astype(np.float64), rtol=2e-2, atol=1e-2)
        else:
            # the global tensor is [64 * world, 512, 1024]: rebuild every rank's first shard on this host
            total = O.reduce_sum_f64(x, 1, 64 * 512, 1024)
            for r in range(1, self.world):
                total = total + O.reduce_sum_f64(ReduceC2(r, self.world).host_inputs(1)[0], 1, 64 * 512, 1024)
            np.testing.assert_allclose(s.astype(np.float64), total, rtol=2e-2, atol=2e-2)
            if getattr(self, "status", None) is not None:
                assert int(self.status.item()) == 0, "the peer exchange timed out"
        wm = O.reduce("max", x, 64 * 512, 1024, 1)
        assert np.array_equal(m.reshape(-1).view(np.uint16), wm.view(np.uint16)), "ReduceMax not bit-exact"


class ReduceC1(Workload):
    """f32 [1024, 4096] U(-1,1): ReduceSum over the last dim"""
    name = "reduce_f32_1024x4096_sum1"
    dtype = "f32"
    shape = (1024, 4096)
    BYTES = 1024 * 4096 * 4 + 1024 * 4

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 1000 * self.rank)
        return [rng.uniform(-1, 1, self.shape).astype(np.float32) for _ in range(n)]

    def work_per_step(self):
        return self.BYTES

    def launches_per_step(self):
        return 1

    def dominant(self):
        return "reduce_rows_kernel (ReduceSum f32 rows)", self.BYTES

    def setup_gpu(self, torch, ops, xs):
        self.ops = ops
        self.out = torch.empty(1024, dtype=torch.float32, device="cuda")

    def step_gpu(self, x, dist=None):
        self.ops.reduce_sum(x, [1], out=self.out)
        return (self.out,)

    dominant_gpu = step_gpu

    def result_bytes(self):
        return 4096

    def step_cpu(self, O, x):
        O.reduce("sum", x, 1024, 4096, 1)

    def check(self, O, x, outs):
        want = O.reduce("sum", x, 1024, 4096, 1)
        np.testing.assert_allclose(outs[0].cpu().numpy(), want, rtol=1e-5, atol=1e-5)


class GatherC3(Workload):
    """IndexSelect: f16 table [1e6, 128] N(0, 0.02), 262144 int64 indices U[0, 1e6)"""
    name = "index_select_f16_1e6x128_idx262144"
    dtype = "f16 (byte copy)"
    ROWS, FEAT, N = 1_000_000, 128, 262_144
    BYTES = 262_144 * 8 + 2 * 262_144 * 128 * 2

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 2 + 1000 * self.rank)
        self.table = (rng.standard_normal((self.ROWS, self.FEAT), dtype=np.float32) * 0.02).astype(np.float16)
        return [rng.integers(0, self.ROWS, self.N).astype(np.int64) for _ in range(n)]

    def work_per_step(self):
        return self.BYTES

    def launches_per_step(self):
        return 1

    def dominant(self):
        return "gather_generic_kernel (256-byte rows: vector loads)", self.BYTES

    def setup_gpu(self, torch, ops, xs):
        self.ops = ops
        self.table_d = torch.from_numpy(self.table).cuda()
        self.out = torch.empty(self.N, self.FEAT, dtype=torch.float16, device="cuda")

    def step_gpu(self, idx, dist=None):
        self.ops.index_select(self.table_d, idx, 0, out=self.out)
        return (self.out,)

    dominant_gpu = step_gpu

    def result_bytes(self):
        return self.N * self.FEAT * 2

    def step_cpu(self, O, idx):
        O.index_select(self.table, idx, 0)

    def check(self, O, idx, outs):
        want, _ = O.index_select(self.table, idx, 0)
        assert np.array_equal(outs[0].cpu().numpy().view(np.uint16), want.view(np.uint16))


class ScatterC3(Workload):
    """IndexPut accumulate: f16 table [1e6, 128], updates [262144, 128] N(0,1), Zipf(1.1) indices"""
    name = "index_put_add_f16_1e6x128_zipf262144"
    dtype = "f16 (f32 accumulate)"
    ROWS, FEAT, N = 1_000_000, 128, 262_144
    BYTES = 2 * 1_000_000 * 128 * 2 + 262_144 * 128 * 2 + 262_144 * 8

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 3 + 1000 * self.rank)
        self.table = (rng.standard_normal((self.ROWS, self.FEAT), dtype=np.float32) * 0.02).astype(np.float16)
        self.upd = rng.standard_normal((self.N, self.FEAT), dtype=np.float32).astype(np.float16)
        return [zipf_indices(rng, self.N, self.ROWS) for _ in range(n)]

    def work_per_step(self):
        return self.BYTES

    def launches_per_step(self):
        return 1 + 9 + 2  # table copy, 3 radix passes x (hist, scan, scatter), chunk sums, span sums

    def dominant(self):
        return "copy_table_kernel + sort + scatter_chunk_kernel (whole op)", self.BYTES

    def setup_gpu(self, torch, ops, xs):
        self.ops = ops
        self.table_d = torch.from_numpy(self.table).cuda()
        self.upd_d = torch.from_numpy(self.upd).cuda()
        self.out = torch.empty_like(self.table_d)
        from byteir_b200 import _native as N
        need = N.lib().b200_index_put_workspace_bytes(N.F16, self.ROWS, self.N, self.FEAT)
        self.ws = torch.empty(need, dtype=torch.uint8, device="cuda")

    def step_gpu(self, idx, dist=None):
        self.ops.index_put_add(self.table_d, idx, self.upd_d, out=self.out, workspace=self.ws)
        return (self.out,)

    dominant_gpu = step_gpu

    def result_bytes(self):
        return self.ROWS * self.FEAT * 2

    def step_cpu(self, O, idx):
        O.index_put_add(self.table, idx, self.upd)

    def check(self, O, idx, outs):
        want, _ = O.index_put_add(self.table, idx, self.upd)
        g, w = outs[0].cpu().numpy().astype(np.float64), want.astype(np.float64)
        assert np.all(np.abs(g - w) <= 1e-3 * np.abs(w) + 1e-4)


class TransposeC4(Workload):
    """Transpose f16 [32, 128, 64, 64] perm (0,2,3,1) and bf16 [8192, 8192] 2-D"""
    name = "transpose_f16_32x128x64x64_p0231+bf16_8192x8192"
    dtype = "f16 / bf16 (byte copy)"
    BYTES_A = 2 * 32 * 128 * 64 * 64 * 2
    BYTES_B = 2 * 8192 * 8192 * 2

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 4 + 1000 * self.rank)
        out = []
        for _ in range(n):
            a = rng.uniform(-1, 1, (32, 128, 64, 64)).astype(np.float16)
            b = rng.integers(0, 65536, (8192, 8192), dtype=np.uint16)  # bf16 bit patterns; a byte copy
            out.append((a, b))
        return out

    def work_per_step(self):
        return self.BYTES_A + self.BYTES_B

    def launches_per_step(self):
        return 2

    def dominant(self):
        return "transpose_tma_kernel<2> (bf16 8192x8192)", self.BYTES_B

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        self.out_a = torch.empty(32, 64, 64, 128, dtype=torch.float16, device="cuda")
        self.out_b = torch.empty(8192, 8192, dtype=torch.bfloat16, device="cuda")

    def to_dev(self, torch, x):
        a, b = x
        return (torch.from_numpy(a).cuda(), torch.from_numpy(b.view(np.int16)).cuda().view(torch.bfloat16))

    def step_gpu(self, x, dist=None):
        a, b = x
        self.ops.transpose(a, (0, 2, 3, 1), out=self.out_a)
        self.ops.transpose(b, (1, 0), out=self.out_b)
        return self.out_a, self.out_b

    def dominant_gpu(self, x):
        self.ops.transpose(x[1], (1, 0), out=self.out_b)

    def result_bytes(self):
        return (self.BYTES_A + self.BYTES_B) // 2

    def step_cpu(self, O, x):
        O.transpose(x[0], (0, 2, 3, 1))
        O.transpose(x[1], (1, 0))

    def check(self, O, x, outs):
        a, b = x
        assert np.array_equal(outs[0].cpu().numpy().view(np.uint16), np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1))).view(np.uint16))
        assert np.array_equal(outs[1].view(self.torch.int16).cpu().numpy().view(np.uint16), np.ascontiguousarray(b.T))



class AttnC5(Workload):
    """FlashAttn fwd+bwd: bf16 Q,K,V,dO [B=8, S=4096, H=32, D=128] N(0,1), causal, scale 1/sqrt(128)"""
    name = "flash_attn_fwd_bwd_bf16_b8_s4096_h32_d128_causal"
    unit = "TFLOP/s"
    dtype = "bf16 (f32 accumulate)"
    bound = "tensor"
    B, S, H, D = 8, 4096, 32, 128
    FWD_FLOPS = 4 * 8 * 32 * 4096 * 4096 * 128 // 2
    BWD_FLOPS = FWD_FLOPS * 5 // 2

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def _gen(self, rng, shape):
        return rng.standard_normal(shape, dtype=np.float32)

    def host_inputs(self, n):
        import oracle_lib as O
        rng = np.random.default_rng(1234 + 5 + 1000 * self.rank)
        shape = (self.B, self.S, self.H, self.D)
        out = []
        for _ in range(min(n, 1)):  # 1 GiB of host data per set: one set, reused
            out.append(tuple(O.f32_to_bf16(self._gen(rng, shape)) for _ in range(4)))
        return out * n

    def work_per_step(self):
        return self.FWD_FLOPS + self.BWD_FLOPS

    def launches_per_step(self):
        return 4  # fwd, dot(dO,O), dK/dV, dQ

    def dominant(self):
        return "flash_fwd_kernel<bf16>", self.FWD_FLOPS

    def to_dev(self, torch, x):
        return tuple(torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16) for a in x)

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        q = xs[0][0]
        self.o = torch.empty_like(q)
        self.lse = torch.empty((self.B, self.H, self.S), dtype=torch.float32, device="cuda")
        self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(3))
        self.dsum = torch.empty((self.B, self.H, self.S), dtype=torch.float32, device="cuda")
        self.scale = 1.0 / float(np.sqrt(self.D))

    def step_gpu(self, x, dist=None):
        q, k, v, do = x
        self.ops.flash_attn_fwd(q, k, v, self.scale, True, out=self.o, lse=self.lse)
        self.ops.flash_attn_bwd(do, q, k, v, self.o, self.lse, self.scale, True, dq=self.dq, dk=self.dk,
                                dv=self.dv, d_softmax_sum=self.dsum)
        return self.o, self.dq, self.dk, self.dv

    def dominant_gpu(self, x):
        q, k, v, do = x
        self.ops.flash_attn_fwd(q, k, v, self.scale, True, out=self.o, lse=self.lse)

    def result_bytes(self):
        return 4 * self.B * self.S * self.H * self.D * 2

    # CPU: a bounded sample (one batch entry, 8 heads, 1024 positions) of the same op
    CPU_SAMPLE = (1, 1024, 8, 128)

    def cpu_sample_flops(self):
        b, s, h, d = self.CPU_SAMPLE
        return (4 * b * h * s * s * d // 2) * 7 // 2

    def step_cpu(self, O, x):
        b, s, h, d = self.CPU_SAMPLE
        q, k, v, do = (a[:b, :s, :h, :] for a in x)
        o, lse = O.flash_attn_fwd(q, k, v, self.scale, True)
        O.flash_attn_bwd(do, q, k, v, o, lse, self.scale, True)

    def check(self, O, x, outs):
        # one (batch, head) slice of the full-size result against the oracle, first 512 positions
        # (causal: the first rows depend only on the first keys)
        q, k, v, do = (np.ascontiguousarray(a[:1, :512, :2, :]) for a in x)
        o, lse = O.flash_attn_fwd(q, k, v, self.scale, True)
        got = outs[0][:1, :512, :2, :].contiguous().view(self.torch.int16).cpu().numpy().view(np.uint16)
        np.testing.assert_allclose(O.bf16_to_f32(got), O.bf16_to_f32(o), rtol=2e-2, atol=1e-2)


class DecodeKv(Workload):
    """Decode step over a kv cache: bf16 q [B=16, 1, H=32, D=128], caches [16, 8192, H_k=8, 128] N(0,1) with
    U[6144, 8190] rows in use, one new row appended per step, scale 1/sqrt(128)"""
    name = "flash_attn_kvcache_bf16_b16_h32_hk8_d128_cache8192"
    dtype = "bf16 (f32 accumulate)"
    B, H, HK, D, CAP = 16, 32, 8, 128, 8192
    l2_policy = "every step streams the 512 MiB of the two caches (L2 is 126 MiB)"

    def __init__(self, rank, world):
        self.rank, self.world = rank, world
        rng = np.random.default_rng(1234 + 6 + 1000 * rank)
        self.lens = rng.integers(6144, self.CAP - 1, self.B).astype(np.int32)
        self.rng = rng
        self.scale = 1.0 / float(np.sqrt(self.D))

    def host_inputs(self, n):
        import oracle_lib as O
        gen = lambda shape: O.f32_to_bf16(self.rng.standard_normal(shape, dtype=np.float32))
        if not hasattr(self, "kcache"):
            self.kcache = gen((self.B, self.CAP, self.HK, self.D))
            self.vcache = gen((self.B, self.CAP, self.HK, self.D))
        return [(gen((self.B, 1, self.H, self.D)), gen((self.B, 1, self.HK, self.D)), gen((self.B, 1, self.HK, self.D)))
                for _ in range(n)]

    def work_per_step(self):  # K and V rows in use, once each
        return int(2 * (self.lens.astype(np.int64) + 1).sum() * self.HK * self.D * 2)

    def launches_per_step(self):
        return 2  # split kernel, merge kernel

    def dominant(self):
        return "decode_mma_kernel<128, bf16>", self.work_per_step()

    def to_dev(self, torch, x):
        return tuple(torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16) for a in x)

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        self.kc, self.vc = self.to_dev(torch, (self.kcache, self.vcache))
        self.lens_d = torch.from_numpy(self.lens).cuda()
        self.o = torch.empty_like(xs[0][0])
        self.lse = torch.empty((self.B, self.H, 1), dtype=torch.float32, device="cuda")
        p = ops.kvcache_params(xs[0][0], self.kc, self.vc, xs[0][1], xs[0][2], self.o, self.scale, True)
        import ctypes as C
        from byteir_b200 import _native as N
        self.ws = torch.empty(max(16, N.lib().b200_flash_attn_kvcache_workspace_bytes(C.byref(p))), dtype=torch.uint8,
                              device="cuda")

    def step_gpu(self, x, dist=None):
        q, kn, vn = x
        self.ops.flash_attn_kvcache(q, self.kc, self.vc, kn, vn, self.lens_d, self.scale, True, out=self.o,
                                    lse=self.lse, workspace=self.ws)
        return self.o, self.lse

    dominant_gpu = step_gpu

    def result_bytes(self):
        return self.B * self.H * self.D * 2 + self.B * self.H * 4

    # CPU: two batch entries of the same step
    CPU_SAMPLE = (2, 8192, 8, 128)

    def cpu_sample_flops(self):  # bytes, like work_per_step
        return int(2 * (self.lens[:2].astype(np.int64) + 1).sum() * self.HK * self.D * 2)

    def step_cpu(self, O, x):
        q, kn, vn = (a[:2] for a in x)
        if not hasattr(self, "cpu_caches"):
            self.cpu_caches = (self.kcache[:2].copy(), self.vcache[:2].copy())
        O.flash_attn_kvcache(np.ascontiguousarray(q), self.cpu_caches[0], self.cpu_caches[1], kn, vn, self.lens[:2],
                             self.scale, True)

    def check(self, O, x, outs):
        # batch entry 3 against the oracle: output, LSE, and the appended cache rows
        b = 3
        q, kn, vn = (np.ascontiguousarray(a[b:b + 1]) for a in x)
        kc, vc = self.kcache[b:b + 1].copy(), self.vcache[b:b + 1].copy()
        o, lse = O.flash_attn_kvcache(q, kc, vc, kn, vn, self.lens[b:b + 1], self.scale, True)
        got = outs[0][b:b + 1].contiguous().view(self.torch.int16).cpu().numpy().view(np.uint16)
        np.testing.assert_allclose(O.bf16_to_f32(got), O.bf16_to_f32(o), rtol=2e-2, atol=1e-2)
        np.testing.assert_allclose(outs[1][b:b + 1].cpu().numpy(), lse, rtol=1e-3, atol=1e-3)
        row = int(self.lens[b])
        got_k = self.kc[b, row].contiguous().view(self.torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got_k, kc[0, row])


WORKLOADS = {"attn": AttnC5, "decode": DecodeKv, "reduce_c2": ReduceC2, "reduce_c1": ReduceC1, "gather": GatherC3, "scatter": ScatterC3,
             "transpose": TransposeC4}
METRIC = "HBM GB/s (algorithmic bytes / time) of the ByRE compute op"
METRIC_TENSOR = "flash-attn fwd+bwd TFLOP/s (algorithmic FLOPs / time)"


def metric_of(wl):
    return METRIC_TENSOR if wl.bound == "tensor" else METRIC


def rate(wl, work, seconds):
    """GB/s for byte work, TFLOP/s for FLOP work"""
    return work / seconds / (1e12 if wl.bound == "tensor" else 1e9)


def to_dev_default(torch, x):
    return torch.from_numpy(x).cuda()


def run_reference(args, rank, world, json_out):
    """The reference arm: the CPU restatement of the reference's op semantics on all
    host cores (the reference's own CPU pipeline needs LLVM/MLIR, which this
    image does not have)."""
    if rank != 0:
        return
    import oracle_lib as O
    wl = WORKLOADS[args.workload](0, 1)
    xs = wl.host_inputs(2)
    cores = O.lib().oracle_num_threads()
    for i in range(args.warmup):
        wl.step_cpu(O, xs[i % 2])
    t0 = time.perf_counter()
    for i in range(args.steps):
        wl.step_cpu(O, xs[i % 2])
    dt = (time.perf_counter() - t0) / args.steps
    cpu_work = wl.cpu_sample_flops() if hasattr(wl, "cpu_sample_flops") else wl.work_per_step()
    val = rate(wl, cpu_work, dt)
    json_out.write(json.dumps({
        "impl": "reference", "metric": metric_of(wl), "value": val, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded)",
        "config": {"workload": wl.name, "note": "CPU port of the reference op semantics; " + (
            f"each step a bounded sample {wl.CPU_SAMPLE} [B,S,H,D] of the workload" if hasattr(wl, "CPU_SAMPLE")
            else "one full batch per step")},
        "cpu_baseline": {"value": val, "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} steps on the host"},
        "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }) + "\n")
    json_out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="reduce_c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--attn-shape", default="", help="B,S,H override of the attention workload (profiling a small case)")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="dump every thread's Python stack and exit if the run takes longer than this many seconds")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.watchdog > 0:
        import faulthandler
        faulthandler.dump_traceback_later(args.watchdog, exit=True)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    # stdout carries exactly one JSON line: anything a library prints to file descriptor 1
    # (NCCL's version banner, for one) is sent to stderr instead
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    if args.impl == "reference":
        run_reference(args, rank, world, json_out)
        return

    import torch
    from byteir_b200 import ops  # fails loudly if the CUDA library is missing

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    wl = WORKLOADS[args.workload](rank, world)
    if args.workload == "attn" and args.attn_shape:
        wl.B, wl.S, wl.H = (int(v) for v in args.attn_shape.split(","))
        wl.FWD_FLOPS = 4 * wl.B * wl.H * wl.S * wl.S * wl.D // 2
        wl.BWD_FLOPS = wl.FWD_FLOPS * 5 // 2
        wl.name = f"flash_attn_fwd_bwd_bf16_b{wl.B}_s{wl.S}_h{wl.H}_d128_causal"
    per_buf = None
    xs_host = wl.host_inputs(1)
    # rotate over enough distinct inputs that together they exceed L2
    first = xs_host[0]
    per_buf = sum(a.nbytes for a in (first if isinstance(first, tuple) else (first,)))
    n_buf = max(2, -(-2 * L2_BYTES // per_buf)) if args.workload not in ("scatter", "transpose", "attn", "decode") else 2
    if args.workload == "attn":
        n_buf = 1  # one input set is 1 GiB, far beyond L2
    n_buf = min(n_buf, 8)
    xs_host = wl.host_inputs(n_buf)
    to_dev = getattr(wl, "to_dev", to_dev_default)
    xs = [to_dev(torch, x) for x in xs_host]
    wl.setup_gpu(torch, ops, xs)

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # correctness of what is about to be timed
    outs = wl.step_gpu(xs[0], dist)
    torch.cuda.synchronize()
    if rank == 0:
        import oracle_lib as O
        wl.check(O, xs_host[0], outs)

    for i in range(args.warmup):
        wl.step_gpu(xs[i % n_buf], dist)
    sync_all()

    # The timed region is launch-bound from Python (a step is tens of microseconds of
    # device time), so the K steps are captured once into a CUDA graph and the graph
    # replay is what is timed; --no-graph times eager launches instead.
    def capture(fn, count):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(g, stream=side):
            for i in range(count):
                fn(i)
        return g

    # a batch of K back-to-back steps: a workload with an exchange step may let it overlap the
    # next step (ReduceC2 at N > 1); the last call of the batch joins it
    pipelined = isinstance(wl, ReduceC2) and world > 1

    def batch_step(i):
        if pipelined:
            wl.step_gpu(xs[i % n_buf], dist, pipelined=True)
            if i == args.steps - 1:
                wl.end_batch()
        else:
            wl.step_gpu(xs[i % n_buf], dist)

    use_graph = not args.no_graph
    step_graph = None
    if use_graph:
        try:
            step_graph = capture(batch_step, args.steps)
            step_graph.replay()  # untimed: first replay uploads the graph
        except Exception as e:  # pragma: no cover - depends on the NCCL / driver combination
            print(f"graph capture failed ({e}); timing eager launches", file=sys.stderr)
            step_graph = None
            use_graph = False
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if step_graph is not None and world > 1:
        # Ranks leave the host barrier hundreds of microseconds apart, which is comparable to the whole
        # timed region.  One more untimed replay is queued right before the timed one: its last
        # exchange aligns the GPUs to within microseconds, and the timed K steps start from there.
        step_graph.replay()
    ev0.record()
    if step_graph is not None:
        step_graph.replay()
    else:
        for i in range(args.steps):
            batch_step(i)
    ev1.record()
    sync_all()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    value = rate(wl, wl.work_per_step() * world, ms_per_step * 1e-3)

    # dominant kernel alone: `reps` back-to-back launches over rotating inputs,
    # CUDA events around the batch (graph replay, so launch gaps are the device's own)
    dom_name, dom_work = wl.dominant()
    reps = max(args.steps, 20)
    for i in range(3):
        wl.dominant_gpu(xs[i % n_buf])
    torch.cuda.synchronize()
    dom_graph = capture(lambda i: wl.dominant_gpu(xs[i % n_buf]), reps) if use_graph else None
    if dom_graph is not None:
        dom_graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        ev0.record()
        if dom_graph is not None:
            dom_graph.replay()
        else:
            for i in range(reps):
                wl.dominant_gpu(xs[i % n_buf])
        ev1.record()
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1) / reps)
    dom_ms = float(np.median(times))
    clocks = sampler.stop() if rank == 0 else None

    # end to end with host buffers: pinned host -> device, op, device -> host
    pinned_in = []
    for x in xs_host[:2]:
        parts = x if isinstance(x, tuple) else (x,)
        pinned_in.append(tuple(torch.from_numpy(p.view(np.int16) if p.dtype == np.uint16 else p).pin_memory() for p in parts))
    dev_in = [tuple(torch.empty_like(p, device="cuda") for p in parts) for parts in pinned_in]
    outs = wl.step_gpu(xs[0], dist)
    pinned_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]

    def as_input(parts_dev, like):
        vals = []
        for d, l in zip(parts_dev, like if isinstance(like, tuple) else (like,)):
            vals.append(d.view(l.dtype) if d.dtype != l.dtype else d)
        return tuple(vals) if isinstance(like, tuple) else vals[0]

    def e2e_step(i):
        k = i % len(pinned_in)
        for src, dst in zip(pinned_in[k], dev_in[k]):
            dst.copy_(src, non_blocking=True)
        o = wl.step_gpu(as_input(dev_in[k], xs[0]), dist)
        for src, dst in zip(o, pinned_out):
            dst.copy_(src, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 20))
    for i in range(2):
        e2e_step(i)
    sync_all()
    ev0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    ev1.record()
    sync_all()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e_val = rate(wl, wl.work_per_step() * world, e2e_ms * 1e-3)
    h2d = sum(p.numel() * p.element_size() for p in pinned_in[0])
    d2h = sum(p.numel() * p.element_size() for p in pinned_out)

    def finish():
        # Tearing the NCCL group down while CUDA graphs that captured its collectives exist has
        # blocked; the graphs are dropped, the ranks meet once more, and the processes leave
        # without the group destructor.
        nonlocal step_graph, dom_graph
        step_graph = dom_graph = None
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        finish()
        return

    peaks = measured_peaks()
    achieved = rate(wl, dom_work, dom_ms * 1e-3)
    peak = peaks["bf16_tflops"] if wl.bound == "tensor" else peaks["hbm_gbs"]
    roofline = {"bound": wl.bound, "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": wl.unit,
                "frac": achieved / peak, "peak_source": peaks["source"], "us_per_launch": dom_ms * 1e3,
                "traffic": NCU_TRAFFIC.get(args.workload)}
    if wl.bound == "tensor":
        # `peak` is the burst figure (a GEMM timed alone).  The dominant kernel is timed as a batch of
        # back-to-back launches that runs into the power cap (see `clocks`), which is the regime of
        # the sustained figure, so that fraction is reported beside it.
        roofline["peak_sustained"] = peaks["bf16_tflops_sustained"]
        roofline["frac_of_sustained"] = achieved / peaks["bf16_tflops_sustained"]

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        import oracle_lib as O
        cores = O.lib().oracle_num_threads()
        wl.step_cpu(O, xs_host[0])
        t0 = time.perf_counter()
        n = 0
        while True:
            wl.step_cpu(O, xs_host[n % len(xs_host)])
            n += 1
            if time.perf_counter() - t0 > 10.0 or n >= 50:
                break
        dt = (time.perf_counter() - t0) / n
        cpu_work = wl.cpu_sample_flops() if hasattr(wl, "cpu_sample_flops") else wl.work_per_step()
        sample = (f"{n} steps on a {wl.CPU_SAMPLE} [B,S,H,D] slice of the workload" if hasattr(wl, "CPU_SAMPLE")
                  else f"{n} full steps of the same workload (about 10 s)")
        cpu = {"value": rate(wl, cpu_work, dt), "unit": wl.unit, "cores": cores, "kind": "port",
               "sample": sample, "ms_per_step": dt * 1e3}

    line = {
        "metric": metric_of(wl), "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic (seeded numpy Generator)",
        "config": {"workload": wl.name, "per_gpu_batch": wl.__doc__.strip(),
                   "l2_policy": getattr(wl, "l2_policy", None) or
                   f"inputs rotate over {n_buf} distinct buffers ({n_buf * per_buf / 2**20:.0f} MiB, L2 is 126 MiB)",
                   "launch": "CUDA graph replay of the K steps" if use_graph else "eager launches",
                   "exchange": getattr(wl, "exchange", "none"),
                   "parallelism": f"dp{world}"},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_val, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": wl.launches_per_step() * args.steps,
        "clocks": clocks,
    }
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
    finish()


if __name__ == "__main__":
    main()
