#!/usr/bin/env python
"""Benchmark of the ByRE compute-op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one pass of a workload over one batch of seeded synthetic input.  The line's own
numbers are the f16 [64, 512, 1024] multi-axis reduction (ReduceSum over dims {0,1} and
ReduceMax over dim 2, each on its own input buffer); `workloads` carries the same
measurements for every other configuration of the path, one op each.  `--workload NAME`
measures one of them alone (used for profiling).  One JSON line is printed by rank 0.

  value     whole-job throughput with inputs resident in HBM: K steps replayed as one CUDA
            graph, CUDA events around the replay, max over ranks, median of five replays
  e2e       the same metric through the plug-in boundary with HOST buffers: a ByRE module whose
            arguments live in the "cpu" space (cpu2cuda -> op -> cuda2cpu), loaded into a brt
            Session and run with Session::Run; pinned host -> device and device -> host copies
            are inside the timed region; two requests are in flight, each on its own stream, so
            that the upload of a step runs beside the download of the step before
  roofline  algorithmic bytes (or FLOPs) of the op over its own event-timed duration, against
            the measured peak; for the attention workloads also `alone`: single steps, each after
            a pause, which is the regime the burst peak was measured in (back-to-back steps run
            into the power cap)
  ref_gpu   the reference's own CUDA kernel launcher for the op (compiled for sm_100a into
            oracle/_ref/libref_kernels.so), timed the same way on the same inputs
  cpu_baseline  the CPU oracle (a restatement of the reference's op semantics) on this host's
            cores, on a bounded sample of the same workload
  in_place  (scatter only) the op with in == out: no table copy, against the bytes of the rows
            that some index names

Multi-GPU: one process per GPU (torchrun); every rank processes its own batch (weak scaling),
no exchange, except the sum whose reduced axis is itself sharded: one kernel over NVLink peer
memory adds the ranks' f32 partial sums before the single rounding to f16.
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
FLASH_LIB = ROOT / "byteir_b200" / "_lib" / "libflash_attn.so"
REF_LIB = ROOT / "oracle" / "_ref" / "libref_kernels.so"


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def captured_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's dominant kernel, written
    beside the profile summaries they were read from"""
    p = ROOT / "profiles" / "traffic.json"
    return json.loads(p.read_text()) if p.exists() else {}


class ClockSampler:
    """samples nvidia-smi clocks and throttle reasons while a timed region runs"""
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
# ByRE module text for the plug-in (end-to-end) leg
# ----------------------------------------------------------------------------
def memref(shape, elt, space):
    return "memref<" + "x".join([str(d) for d in shape] + [elt]) + f', "{space}">'


def byre_module(args, allocs, ops_):
    """args: [(name, argtype, shape, elt, space)]; allocs: [(shape, elt)] (device intermediates, named
    %0, %1, ...); ops_: text lines using %argN / %N"""
    lines = ["module attributes {byre.container_module} {", "  func.func @main("]
    arg_lines = []
    for i, (name, argtype, shape, elt, space) in enumerate(args):
        arg_lines.append(f'      %arg{i}: {memref(shape, elt, space)} {{byre.argname = "{name}", byre.argtype = {argtype} : i32}}')
    lines.append(",\n".join(arg_lines) + ") attributes {byre.entry_point} {")
    for i, (shape, elt) in enumerate(allocs):
        lines.append(f"    %{i} = memref.alloc() : {memref(shape, elt, 'cuda')}")
    lines += ["    " + o for o in ops_]
    lines += ["    return", "  }", "}"]
    return "\n".join(lines) + "\n"


def copy_op(kind, src, dst, shape, elt):
    s_space, d_space = ("cpu", "cuda") if kind == "cpu2cuda" else ("cuda", "cpu")
    return (f"byre.compute @{kind}({src}, {dst}) {{memory_effects = [1 : i32, 2 : i32]}} : "
            f"{memref(shape, elt, s_space)}, {memref(shape, elt, d_space)}")


def compute_op(key, operands, attrs, effects):
    ops_s = ", ".join(o for o, _ in operands)
    types = ", ".join(t for _, t in operands)
    eff = ", ".join(f"{e} : i32" for e in effects)
    a = (attrs + ", ") if attrs else ""
    return f"byre.compute @{key}({ops_s}) {{{a}memory_effects = [{eff}]}} : {types}"


def zipf_indices(rng, n, rows, s=1.1):
    w = 1.0 / np.arange(1, rows + 1, dtype=np.float64) ** s
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n))
    return rng.permutation(rows)[np.minimum(ranks, rows - 1)].astype(np.int64)


_HOST_CACHE = {}


def cached(key, make):
    if key not in _HOST_CACHE:
        _HOST_CACHE[key] = make()
    return _HOST_CACHE[key]


def bits_view(a):
    """torch has no uint16 arithmetic type: bf16 bit patterns travel as int16"""
    return a.view(np.int16) if a.dtype == np.uint16 else a


# ----------------------------------------------------------------------------
# workloads: one ByRE op (or one custom call pair) each
# ----------------------------------------------------------------------------
class Workload:
    """One configuration: host inputs, one step on the GPU through the C ABI, the same step on the CPU
    oracle, the ByRE module of the step with host-space arguments, and (where the reference has one)
    the reference's own GPU kernel for the step."""
    key = ""
    name = ""
    unit = "GB/s"
    dtype = ""
    bound = "hbm"
    kernel = ""
    launches = 1
    cpu_sample = None

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    N_BUF = 4  # distinct input sets a run rotates over (together beyond L2, or each beyond it alone)

    def to_dev(self, torch, x):
        return tuple(torch.from_numpy(bits_view(a)).cuda() for a in x)

    def end_batch(self):
        pass

    def cpu_work(self):
        return self.work()

    def plugin(self, torch):  # (module text, {arg name: ("in", input index) | ("out", output index) | ("dev", tensor)})
        return None

    def ref_gpu(self, ref, torch):  # (kernel name, callable(x) launching the reference kernel) or None
        return None

    def variants(self, torch):  # {key: (callable(x), algorithmic bytes or flops, note)}: the op in another form
        return {}

    def make_session(self, brt, local_rank):  # the session the plug-in leg loads the module into
        return brt.Session("cuda", device_id=local_rank, host_space=True)


class ReduceBase(Workload):
    """ReduceSumOp / ReduceMaxOp on one tensor"""
    op = "sum"
    shape = ()
    dims = ()
    t = "f16"

    def _np(self):
        return np.float32 if self.t == "f32" else np.float16

    def abc(self):
        import oracle_lib as O
        return O.reduce_abc(self.shape, list(self.dims))

    def out_shape(self):
        return tuple(s for i, s in enumerate(self.shape) if i not in self.dims)

    def work(self):
        es = 4 if self.t == "f32" else 2
        return int(np.prod(self.shape)) * es + int(np.prod(self.out_shape())) * es

    def setup_gpu(self, torch, ops, xs):
        self.torch, self.ops = torch, ops
        self.out = torch.empty(self.out_shape(), dtype=xs[0][0].dtype, device="cuda")
        from byteir_b200 import _native as N
        A, B, C = self.abc()
        need = N.lib().b200_reduce_workspace_bytes(0 if self.op == "sum" else 1, N.F32 if self.t == "f32" else N.F16, A, B, C)
        self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda") if need else None

    def step_gpu(self, x):
        fn = self.ops.reduce_sum if self.op == "sum" else self.ops.reduce_max
        fn(x[0], list(self.dims), out=self.out, workspace=self.ws)
        return (self.out,)

    def step_cpu(self, O, x):
        A, B, C = self.abc()
        O.reduce(self.op, x[0], A, B, C)

    def check(self, O, x, outs):
        A, B, C = self.abc()
        want = O.reduce(self.op, x[0], A, B, C)
        got = outs[0].cpu().numpy().reshape(-1)
        if self.op == "max":
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), "ReduceMax not bit-exact"
        elif self.t == "f32":
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
        else:
            np.testing.assert_allclose(got.astype(np.float64), want.astype(np.float64), rtol=2e-2, atol=1e-2)

    def plugin(self, torch):
        key = f"Reduce{'Sum' if self.op == 'sum' else 'Max'}Op_{self.t}_{self.t}"
        dims = ", ".join(str(d) for d in self.dims)
        attr = f"dimensions = dense<[{dims}]> : tensor<{len(self.dims)}xi64>"
        ins, outs = self.shape, self.out_shape()
        text = byre_module(
            [("X", 1, ins, self.t, "cpu"), ("Y", 2, outs, self.t, "cpu")], [(ins, self.t), (outs, self.t)],
            [copy_op("cpu2cuda", "%arg0", "%0", ins, self.t),
             compute_op(key, [("%0", memref(ins, self.t, "cuda")), ("%1", memref(outs, self.t, "cuda"))], attr, [1, 2]),
             copy_op("cuda2cpu", "%1", "%arg1", outs, self.t)])
        return text, {"X": ("in", 0), "Y": ("out", 0)}

    def ref_gpu(self, ref, torch):
        A, B, C = self.abc()
        # the reference sizes its f16 workspace with sizeof(half) although it stores f32 partials
        # (reduce_impl.h:77-79): sized here by the f32 rule so that the kernel stays in bounds
        ws = torch.empty(max(ref.ref_reduce_workspace_bytes(0, A, B, C), 16), dtype=torch.uint8, device="cuda")
        out = torch.empty_like(self.out)
        op, dt = (0 if self.op == "sum" else 1), (0 if self.t == "f32" else 1)

        def run(x):
            rc = ref.ref_reduce(op, dt, x[0].data_ptr(), out.data_ptr(), A, B, C, ws.data_ptr(),
                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
        return "kernel::call_reduce (reduction/kernels/reduction.cu)", run


class ReduceC1(ReduceBase):
    """f32 [1024, 4096] U(-1,1): ReduceSum over the last dim"""
    key, name, dtype, t = "reduce_c1", "reduce_f32_1024x4096_sum1", "f32", "f32"
    op, shape, dims = "sum", (1024, 4096), (1,)
    kernel = "reduce_short_rows_kernel<float, sum>"

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 1000 * self.rank)
        return [(rng.uniform(-1, 1, self.shape).astype(np.float32),) for _ in range(n)]

    N_BUF = 16


def c2_inputs(rank, n, shape=(64, 512, 1024)):
    def make():
        rng = np.random.default_rng(1234 + 1 + 1000 * rank)
        return [(rng.standard_normal(shape, dtype=np.float32).astype(np.float16),) for _ in range(n)]
    return cached(("c2", rank, n, shape), make)


class ReduceC2Sum(ReduceBase):
    """f16 [64, 512, 1024] N(0,1): ReduceSum over dims {0,1} (column reduction, f32 accumulate) -> f16 [1024]"""
    key, name, dtype = "reduce_c2_sum", "reduce_f16_64x512x1024_sum01", "f16 (f32 accumulate)"
    op, shape, dims = "sum", (64, 512, 1024), (0, 1)
    kernel = "reduce_cols_kernel + reduce_finalize_kernel"
    launches = 2

    def host_inputs(self, n):
        return c2_inputs(self.rank, n)

    N_BUF = 4


class ReduceC2Max(ReduceBase):
    """f16 [64, 512, 1024] N(0,1): ReduceMax over dim 2 (row reduction, bit-exact) -> f16 [64, 512]"""
    key, name, dtype = "reduce_c2_max", "reduce_f16_64x512x1024_max2", "f16"
    op, shape, dims = "max", (64, 512, 1024), (2,)
    kernel = "reduce_short_rows_kernel<half, max>"

    def host_inputs(self, n):
        return c2_inputs(self.rank, n)

    N_BUF = 4


class ReduceC2(Workload):
    """f16 [64, 512, 1024] N(0,1): ReduceSum dims {0,1} -> f16 [1024] and ReduceMax dim 2 -> f16 [64, 512]; under
    N ranks the global tensor is [64 N, 512, 1024], dim 0 sharded, so the sum ends with an exchange of partials"""
    key, name, dtype = "reduce_c2", "reduce_f16_64x512x1024_sum01_max2", "f16 (f32 accumulate)"
    kernel = "reduce_cols_kernel + reduce_finalize_kernel (ReduceSum dims {0,1})"

    def __init__(self, rank, world, rows0=64):
        super().__init__(rank, world)
        self.rows0 = rows0
        self.shape = (rows0, 512, 1024)
        self.SUM_BYTES = rows0 * 512 * 1024 * 2 + 1024 * 2
        self.MAX_BYTES = rows0 * 512 * 1024 * 2 + rows0 * 512 * 2
        self.launches = 3 + (1 if world > 1 else 0)  # column pass, second pass, row max (+ exchange kernel)

    def host_inputs(self, n):
        # a step reads two different buffers: (input of the sum, input of the max)
        xs = c2_inputs(self.rank, n, self.shape)
        half = max(1, n // 2)
        return [(xs[i][0], xs[(i + half) % n][0]) for i in range(n)]

    N_BUF = 4

    def work(self):
        return self.SUM_BYTES + self.MAX_BYTES

    def setup_gpu(self, torch, ops, xs):
        self.torch, self.ops = torch, ops
        self.out_sum = torch.empty(1024, dtype=torch.float16, device="cuda")
        self.out_max = torch.empty(self.rows0, 512, dtype=torch.float16, device="cuda")
        self.part = torch.empty(1024, dtype=torch.float32, device="cuda")
        from byteir_b200 import _native as N
        need = N.lib().b200_reduce_workspace_bytes(0, N.F16, 1, self.rows0 * 512, 1024)
        self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        self.exchange = "none"
        self.sharded = None
        if self.world > 1:
            self.exchange = "nccl all-reduce + cast"
            if os.environ.get("B200_EXCHANGE", "peer") in ("peer", "switch"):
                try:
                    self._setup_peer_exchange(torch, ops, N)
                    self.exchange = "b200_sharded_sum_finish (one kernel over NVLink peer memory)"
                    if os.environ.get("B200_EXCHANGE") == "switch":  # measurement: the sum taken inside the NVSwitch
                        buf, hdl = self._symm
                        mc = int(hdl.multicast_ptr)
                        if not mc:
                            raise RuntimeError("no multicast mapping of the symmetric buffer")
                        ptrs = [int(p) for p in hdl.buffer_ptrs]
                        self.sharded = ops.ShardedSumSwitch(self.rank, self.world, 1024, ptrs[self.rank], mc,
                                                            [p + self._flag_off for p in ptrs], self.counter, self.status)
                        self.exchange = "b200_sharded_sum_finish_nvls (multimem.ld_reduce through the NVSwitch)"
                except Exception as e:  # symmetric memory unavailable: keep NCCL
                    print(f"peer-memory exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)

    def _setup_peer_exchange(self, torch, ops, N):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        n = 1024
        inbox_bytes = N.lib().b200_sharded_sum_inbox_bytes(self.world, n)
        flag_off = (inbox_bytes + 255) // 256 * 256
        self._flag_off = flag_off
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
        # the reductions leave two block slots of their wave to the exchange kernels that run beside them (in a
        # batch of back-to-back steps the exchange of one step is still waiting for its peers when the next one starts)
        N.lib().b200_reduce_reserve_blocks(int(os.environ.get("B200_RESERVE_BLOCKS", "2")))
        # the exchange is one small block beside grids that fill the GPU: highest priority, so that it
        # never queues behind their blocks
        self.side = torch.cuda.Stream(priority=-1)
        self.parts = [self.part, torch.empty_like(self.part)]
        self.xdone = [torch.cuda.Event(), torch.cuda.Event()]
        self.kstep = 0

    def step_gpu(self, x, pipelined=False):
        import torch.distributed as dist
        ops = self.ops
        xs, xm = x
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
            ops.reduce_sum_to_f32(xs, [0, 1], out=part, workspace=self.ws)
            self.side.wait_stream(cur)
            with torch.cuda.stream(self.side):
                self.sharded(part, self.out_sum)
                self.xdone[k & 1].record(self.side)
            ops.reduce_max(xm, [2], out=self.out_max)
            self.kstep = k + 1
            if not pipelined:
                self.end_batch()
        elif self.world > 1:
            # comparison path: NCCL all-reduce of the partials beside the max reduction, then the cast
            ops.reduce_sum_to_f32(xs, [0, 1], out=self.part, workspace=self.ws)
            work = dist.all_reduce(self.part, async_op=True)
            ops.reduce_max(xm, [2], out=self.out_max)
            work.wait()
            ops.cast_from_f32(self.part, self.torch.float16, out=self.out_sum)
        else:
            ops.reduce_sum(xs, [0, 1], out=self.out_sum, workspace=self.ws)
            ops.reduce_max(xm, [2], out=self.out_max)
        return self.out_sum, self.out_max

    def end_batch(self):
        if self.world > 1 and self.sharded is not None:
            self.torch.cuda.current_stream().wait_stream(self.side)
            self.kstep = 0

    def step_cpu(self, O, x):
        O.reduce("sum", x[0], 1, self.rows0 * 512, 1024)
        O.reduce("max", x[1], self.rows0 * 512, 1024, 1)

    def check(self, O, x, outs):
        s, m = (o.cpu().numpy() for o in outs)
        if self.world == 1:
            want = O.reduce("sum", x[0], 1, self.rows0 * 512, 1024)
            np.testing.assert_allclose(s.astype(np.float64), want.astype(np.float64), rtol=2e-2, atol=1e-2)
        else:
            # the global tensor is [rows0 * world, 512, 1024]: rebuild every rank's first shard on this host
            total = O.reduce_sum_f64(x[0], 1, self.rows0 * 512, 1024)
            for r in range(1, self.world):
                other = ReduceC2(r, self.world, self.rows0).host_inputs(4)[0][0]
                total = total + O.reduce_sum_f64(other, 1, self.rows0 * 512, 1024)
            np.testing.assert_allclose(s.astype(np.float64), total, rtol=2e-2, atol=2e-2)
            if getattr(self, "status", None) is not None:
                assert int(self.status.item()) == 0, "the peer exchange timed out"
        wm = O.reduce("max", x[1], self.rows0 * 512, 1024, 1)
        assert np.array_equal(m.reshape(-1).view(np.uint16), wm.view(np.uint16)), "ReduceMax not bit-exact"

    def make_session(self, brt, local_rank):
        if self.world == 1:
            return super().make_session(brt, local_rank)
        # one rank of the job: the module's nccl.AllReduce runs on the one-kernel peer-memory sum, or on
        # torch.distributed's NCCL group (created once at start-up) when peer memory is not available
        torch = self.torch
        s = brt.DistributedSession(self.rank, self.world, device="cuda", device_id=local_rank, host_space=True)
        if self.sharded is not None:
            buf, hdl = self._symm
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            s.set_allreduce_peer(1024, ptrs, [p + self._flag_off for p in ptrs], self.counter.data_ptr(),
                                 self.status.data_ptr())
        else:
            import torch.distributed as dist

            class Dev:  # a raw device address as a tensor
                def __init__(self, ptr, n):
                    self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}

            def all_reduce(send, recv, n, dtype, op, group, stream):
                assert dtype == "f32" and op == "sum"
                r = torch.as_tensor(Dev(recv, n), device="cuda")
                r.copy_(torch.as_tensor(Dev(send, n), device="cuda"))
                dist.all_reduce(r)
            s.set_allreduce(all_reduce)
        return s

    def plugin(self, torch):
        # Configuration 2 is two ops on the SAME tensor x (sum over dims {0,1}, max over dim 2), so the module
        # takes x once: one upload, two ops, two results.  (The device-timed step above reads two different
        # buffers only so that its number does not ride on x still sitting in L2.)
        ins = self.shape
        if self.world > 1:
            group = ", ".join(str(r) for r in range(self.world))
            text = byre_module(
                [("X", 1, ins, "f16", "cpu"), ("Sum", 2, (1024,), "f16", "cpu"), ("Max", 2, (self.rows0, 512), "f16", "cpu")],
                [(ins, "f16"), ((1024,), "f32"), ((1024,), "f16"), ((self.rows0, 512), "f16")],
                [copy_op("cpu2cuda", "%arg0", "%0", ins, "f16"),
                 compute_op("ReduceSumOp_f16_f32", [("%0", memref(ins, "f16", "cuda")), ("%1", memref((1024,), "f32", "cuda"))],
                            "dimensions = dense<[0, 1]> : tensor<2xi64>", [1, 2]),
                 compute_op("nccl.AllReduce", [("%1", memref((1024,), "f32", "cuda")), ("%2", memref((1024,), "f16", "cuda"))],
                            f'reduction = "sum", replica_group = [{group}]', [1, 2]),
                 compute_op("ReduceMaxOp_f16_f16", [("%0", memref(ins, "f16", "cuda")), ("%3", memref((self.rows0, 512), "f16", "cuda"))],
                            "dimensions = dense<[2]> : tensor<1xi64>", [1, 2]),
                 copy_op("cuda2cpu", "%2", "%arg1", (1024,), "f16"),
                 copy_op("cuda2cpu", "%3", "%arg2", (self.rows0, 512), "f16")])
            return text, {"X": ("in", 0), "Sum": ("out", 0), "Max": ("out", 1)}
        text = byre_module(
            [("X", 1, ins, "f16", "cpu"), ("Sum", 2, (1024,), "f16", "cpu"), ("Max", 2, (self.rows0, 512), "f16", "cpu")],
            [(ins, "f16"), ((1024,), "f16"), ((self.rows0, 512), "f16")],
            [copy_op("cpu2cuda", "%arg0", "%0", ins, "f16"),
             compute_op("ReduceSumOp_f16_f16", [("%0", memref(ins, "f16", "cuda")), ("%1", memref((1024,), "f16", "cuda"))],
                        "dimensions = dense<[0, 1]> : tensor<2xi64>", [1, 2]),
             compute_op("ReduceMaxOp_f16_f16", [("%0", memref(ins, "f16", "cuda")), ("%2", memref((self.rows0, 512), "f16", "cuda"))],
                        "dimensions = dense<[2]> : tensor<1xi64>", [1, 2]),
             copy_op("cuda2cpu", "%1", "%arg1", (1024,), "f16"),
             copy_op("cuda2cpu", "%2", "%arg2", (self.rows0, 512), "f16")])
        return text, {"X": ("in", 0), "Sum": ("out", 0), "Max": ("out", 1)}

    def e2e_want(self, x):  # what the typed path computes when both ops read the module's one input
        return self.step_gpu((x[0], x[0]))


def c3_table(rank):
    def make():
        rng = np.random.default_rng(1234 + 2 + 1000 * rank)
        return (rng.standard_normal((1_000_000, 128), dtype=np.float32) * 0.02).astype(np.float16)
    return cached(("c3_table", rank), make)


class GatherC3(Workload):
    """IndexSelect: f16 table [1e6, 128] N(0, 0.02), 262144 int64 indices U[0, 1e6)"""
    key, name, dtype = "gather", "index_select_f16_1e6x128_idx262144", "f16 (byte copy)"
    kernel = "gather_rows_g4_kernel (tensor-map gather, 32-row tiles)"
    ROWS, FEAT, N = 1_000_000, 128, 262_144

    def host_inputs(self, n):
        self.table = c3_table(self.rank)
        rng = np.random.default_rng(1234 + 20 + 1000 * self.rank)
        return [(rng.integers(0, self.ROWS, self.N).astype(np.int64),) for _ in range(n)]

    N_BUF = 8

    def work(self):
        return self.N * 8 + 2 * self.N * self.FEAT * 2

    def setup_gpu(self, torch, ops, xs):
        self.ops = ops
        self.table_d = torch.from_numpy(self.table).cuda()
        self.out = torch.empty(self.N, self.FEAT, dtype=torch.float16, device="cuda")

    def step_gpu(self, x):
        self.ops.index_select(self.table_d, x[0], 0, out=self.out)
        return (self.out,)

    def step_cpu(self, O, x):
        O.index_select(self.table, x[0], 0)

    def check(self, O, x, outs):
        want, _ = O.index_select(self.table, x[0], 0)
        assert np.array_equal(outs[0].cpu().numpy().view(np.uint16), want.view(np.uint16))

    def plugin(self, torch):
        t, i, o = (self.ROWS, self.FEAT), (self.N,), (self.N, self.FEAT)
        text = byre_module(
            [("Table", 1, t, "f16", "cuda"), ("Idx", 1, i, "i64", "cpu"), ("Out", 2, o, "f16", "cpu")],
            [(i, "i64"), (o, "f16")],
            [copy_op("cpu2cuda", "%arg1", "%0", i, "i64"),
             compute_op("IndexSelectOp_f16i64_f16", [("%arg0", memref(t, "f16", "cuda")), ("%0", memref(i, "i64", "cuda")),
                                                     ("%1", memref(o, "f16", "cuda"))], "dim = 0 : i32", [1, 1, 2]),
             copy_op("cuda2cpu", "%1", "%arg2", o, "f16")])
        return text, {"Table": ("dev", self.table_d), "Idx": ("in", 0), "Out": ("out", 0)}

    def ref_gpu(self, ref, torch):
        out = torch.empty_like(self.out)

        def run(x):
            rc = ref.ref_index_select(2, self.table_d.data_ptr(), x[0].data_ptr(), out.data_ptr(), 1, self.ROWS, self.N,
                                      self.FEAT, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
        return "kernel::index_select (indexing/kernels/index_select.cu)", run


class ScatterC3(Workload):
    """IndexPut accumulate: f16 table [1e6, 128], updates [262144, 128] N(0,1), Zipf(1.1) indices, out of place"""
    key, name, dtype = "scatter", "index_put_add_f16_1e6x128_zipf262144", "f16 (f32 accumulate)"
    kernel = "copy_table_kernel beside the radix sort, scatter_chunk_staged_kernel, scatter_span_kernel (whole op)"
    launches = 1 + 5 + 2  # table copy; first histogram, 2 x (scan, scatter); accumulate, span
    ROWS, FEAT, N = 1_000_000, 128, 262_144

    def host_inputs(self, n):
        self.table = c3_table(self.rank)
        rng = np.random.default_rng(1234 + 3 + 1000 * self.rank)
        self.upd = rng.standard_normal((self.N, self.FEAT), dtype=np.float32).astype(np.float16)
        self._idx_host = [zipf_indices(rng, self.N, self.ROWS) for _ in range(n)]
        return [(x,) for x in self._idx_host]

    N_BUF = 2

    def work(self):
        return 2 * self.ROWS * self.FEAT * 2 + self.N * self.FEAT * 2 + self.N * 8

    def setup_gpu(self, torch, ops, xs):
        self.ops = ops
        self.table_d = torch.from_numpy(self.table).cuda()
        self.upd_d = torch.from_numpy(self.upd).cuda()
        self.out = torch.empty_like(self.table_d)
        from byteir_b200 import _native as N
        need = N.lib().b200_index_put_workspace_bytes(N.F16, self.ROWS, self.N, self.FEAT)
        self.ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        # the helper stream of the index sort is created outside any stream capture
        assert N.lib().b200_index_put_prepare(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0

    def step_gpu(self, x):
        self.ops.index_put_add(self.table_d, x[0], self.upd_d, out=self.out, workspace=self.ws)
        return (self.out,)

    def step_cpu(self, O, x):
        O.index_put_add(self.table, x[0], self.upd)

    def check(self, O, x, outs):
        want, _ = O.index_put_add(self.table, x[0], self.upd)
        g, w = outs[0].cpu().numpy().astype(np.float64), want.astype(np.float64)
        assert np.all(np.abs(g - w) <= 1e-3 * np.abs(w) + 1e-4)

    def plugin(self, torch):
        t, i, u = (self.ROWS, self.FEAT), (self.N,), (self.N, self.FEAT)
        text = byre_module(
            [("Table", 1, t, "f16", "cuda"), ("Idx", 1, i, "i64", "cpu"), ("Upd", 1, u, "f16", "cuda"),
             ("Out", 2, t, "f16", "cpu")],
            [(i, "i64"), (t, "f16")],
            [copy_op("cpu2cuda", "%arg1", "%0", i, "i64"),
             compute_op("IndexPutOp_f16i64f16_f16",
                        [("%arg0", memref(t, "f16", "cuda")), ("%0", memref(i, "i64", "cuda")), ("%arg2", memref(u, "f16", "cuda")),
                         ("%1", memref(t, "f16", "cuda"))], "dim = 0 : i32", [1, 1, 1, 2]),
             copy_op("cuda2cpu", "%1", "%arg3", t, "f16")])
        return text, {"Table": ("dev", self.table_d), "Idx": ("in", 0), "Upd": ("dev", self.upd_d), "Out": ("out", 0)}

    def variants(self, torch):
        # in place (in == out): no table copy; the algorithmic bytes are the rows some index names, read and
        # written once, the updates and the indices
        inplace = self.table_d.clone()
        rows_named = [int(np.unique(x).size) for x in self._idx_host]  # counted on the host
        u = int(np.median(rows_named))
        work = 2 * u * self.FEAT * 2 + self.N * self.FEAT * 2 + self.N * 8

        def run(x):
            self.ops.index_put_add(inplace, x[0], self.upd_d, out=inplace, workspace=self.ws)
        return {"in_place": (run, work, f"in == out; {u} distinct rows named (median over the index lists)")}

    def ref_gpu(self, ref, torch):
        # the reference's IndexPut is f32 only (index_put.cu:57-59): both sides are timed on an f32 copy of the
        # same table, indices and updates
        t32, u32 = self.table_d.float(), self.upd_d.float()
        out32 = torch.empty_like(t32)
        from byteir_b200 import _native as N
        ws = torch.empty(N.lib().b200_index_put_workspace_bytes(N.F32, self.ROWS, self.N, self.FEAT), dtype=torch.uint8,
                         device="cuda")

        def run(x):
            rc = ref.ref_index_put_f32(t32.data_ptr(), x[0].data_ptr(), u32.data_ptr(), out32.data_ptr(), self.N, self.FEAT,
                                       self.ROWS * self.FEAT, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0

        def ours(x):
            self.ops.index_put_add(t32, x[0], u32, out=out32, workspace=ws)
        return "kernel::index_put<float, true> on an f32 copy of the inputs (indexing/kernels/index_put.cu)", run, ours


class Transpose4D(Workload):
    """Transpose f16 [32, 128, 64, 64] U(-1,1), perm (0,2,3,1)"""
    key, name, dtype = "transpose_4d", "transpose_f16_32x128x64x64_p0231", "f16 (byte copy)"
    kernel = "transpose_tma_kernel<4>"
    SHAPE, PERM = (32, 128, 64, 64), (0, 2, 3, 1)

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 4 + 1000 * self.rank)
        return [(rng.uniform(-1, 1, self.SHAPE).astype(np.float16),) for _ in range(n)]

    def work(self):
        return 2 * int(np.prod(self.SHAPE)) * 2

    def out_shape(self):
        return tuple(self.SHAPE[p] for p in self.PERM)

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        self.out = torch.empty(self.out_shape(), dtype=xs[0][0].dtype, device="cuda")

    def step_gpu(self, x):
        self.ops.transpose(x[0], self.PERM, out=self.out)
        return (self.out,)

    def step_cpu(self, O, x):
        O.transpose(x[0], self.PERM)

    def check(self, O, x, outs):
        got = outs[0].view(self.torch.int16).cpu().numpy().view(np.uint16)
        want = np.ascontiguousarray(np.transpose(x[0], self.PERM)).view(np.uint16)
        assert np.array_equal(got, want)

    ELT = "f16"

    def plugin(self, torch):
        i, o = self.SHAPE, self.out_shape()
        perm = ", ".join(str(p) for p in self.PERM)
        text = byre_module(
            [("In", 1, i, self.ELT, "cpu"), ("Out", 2, o, self.ELT, "cpu")], [(i, self.ELT), (o, self.ELT)],
            [copy_op("cpu2cuda", "%arg0", "%0", i, self.ELT),
             compute_op(f"TransposeOp_{self.ELT}_{self.ELT}",
                        [("%0", memref(i, self.ELT, "cuda")), ("%1", memref(o, self.ELT, "cuda"))],
                        f"permutation = dense<[{perm}]> : tensor<{len(self.PERM)}xi64>", [1, 2]),
             copy_op("cuda2cpu", "%1", "%arg1", o, self.ELT)])
        return text, {"In": ("in", 0), "Out": ("out", 0)}


class Transpose2D(Transpose4D):
    """Transpose bf16 [8192, 8192] (random bit patterns: a byte copy)"""
    key, name, dtype = "transpose_2d", "transpose_bf16_8192x8192", "bf16 (byte copy)"
    kernel = "transpose_tma_kernel<2>"
    SHAPE, PERM, ELT = (8192, 8192), (1, 0), "bf16"

    def host_inputs(self, n):
        rng = np.random.default_rng(1234 + 40 + 1000 * self.rank)
        return [(rng.integers(0, 65536, self.SHAPE, dtype=np.uint16),) for _ in range(n)]

    N_BUF = 2

    def to_dev(self, torch, x):
        return (torch.from_numpy(x[0].view(np.int16)).cuda().view(torch.bfloat16),)

    def ref_gpu(self, ref, torch):
        out = torch.empty_like(self.out)

        def run(x):  # the reference has f16 and f32 only: the same bits as f16, which is the same byte copy
            rc = ref.ref_transpose2d(1, x[0].data_ptr(), out.data_ptr(), 8192, 8192,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
        return "kernel::transpose_naive_2d<half> on the same bits (tensor_manipulate/kernels/transpose.cu)", run


def attn_inputs(rank, shape):
    def make():
        import oracle_lib as O
        rng = np.random.default_rng(1234 + 5 + 1000 * rank)
        return tuple(O.f32_to_bf16(rng.standard_normal(shape, dtype=np.float32)) for _ in range(4))
    return cached(("attn", rank, shape), make)


class AttnFwd(Workload):
    """FlashAttn forward: bf16 Q,K,V [B=8, S=4096, H=32, D=128] N(0,1), causal, scale 1/sqrt(128)"""
    key, name = "attn_fwd", "flash_attn_fwd_bf16_b8_s4096_h32_d128_causal"
    unit, dtype, bound = "TFLOP/s", "bf16 (f32 accumulate)", "tensor"
    kernel = "flash_fwd_kernel<bf16>"
    B, S, H, D = 8, 4096, 32, 128
    with_bwd = False
    cpu_sample = (1, 1024, 8, 128)

    def __init__(self, rank, world):
        super().__init__(rank, world)
        self.scale = 1.0 / float(np.sqrt(self.D))

    def fwd_flops(self):
        return 4 * self.B * self.H * self.S * self.S * self.D // 2

    def work(self):
        return self.fwd_flops() * (7 if self.with_bwd else 2) // 2

    def cpu_work(self):
        b, s, h, d = self.cpu_sample
        return (4 * b * h * s * s * d // 2) * (7 if self.with_bwd else 2) // 2

    def host_inputs(self, n):
        return [attn_inputs(self.rank, (self.B, self.S, self.H, self.D))] * n

    N_BUF = 1

    def to_dev(self, torch, x):
        return tuple(torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16) for a in x)

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        q = xs[0][0]
        self.o = torch.empty_like(q)
        self.lse = torch.empty((self.B, self.H, self.S), dtype=torch.float32, device="cuda")
        if self.with_bwd:
            self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(3))
            self.dsum = torch.empty((self.B, self.H, self.S), dtype=torch.float32, device="cuda")

    def step_gpu(self, x):
        q, k, v, do = x
        self.ops.flash_attn_fwd(q, k, v, self.scale, True, out=self.o, lse=self.lse)
        if not self.with_bwd:
            return self.o, self.lse
        self.ops.flash_attn_bwd(do, q, k, v, self.o, self.lse, self.scale, True, dq=self.dq, dk=self.dk, dv=self.dv,
                                d_softmax_sum=self.dsum)
        return self.o, self.lse, self.dq, self.dk, self.dv

    def step_cpu(self, O, x):
        b, s, h, d = self.cpu_sample
        q, k, v, do = (a[:b, :s, :h, :] for a in x)
        o, lse = O.flash_attn_fwd(q, k, v, self.scale, True)
        if self.with_bwd:
            O.flash_attn_bwd(do, q, k, v, o, lse, self.scale, True)

    def check(self, O, x, outs):
        # Two heads of the last batch entry at the full sequence length against the oracle: forward, and
        # (backward) dQ / dK / dV differentiated from the device's own O and LSE.
        b, hs = self.B - 1, slice(self.H - 2, self.H)
        q, k, v, do = (np.ascontiguousarray(a[b:b + 1, :, hs, :]) for a in x)
        o, lse = O.flash_attn_fwd(q, k, v, self.scale, True)
        host = lambda t: t[b:b + 1, :, hs, :].contiguous().view(self.torch.int16).cpu().numpy().view(np.uint16)
        got_o = host(outs[0])
        got_lse = outs[1][b:b + 1, hs, :].contiguous().cpu().numpy()
        np.testing.assert_allclose(got_lse, lse, rtol=1e-3, atol=1e-3)
        np.testing.assert_allclose(O.bf16_to_f32(got_o), O.bf16_to_f32(o), rtol=2e-2, atol=1e-2)
        if self.with_bwd:
            wq, wk, wv = O.flash_attn_bwd(do, q, k, v, got_o, got_lse, self.scale, True)
            for name, got, want in (("dq", outs[2], wq), ("dk", outs[3], wk), ("dv", outs[4], wv)):
                np.testing.assert_allclose(O.bf16_to_f32(host(got)), O.bf16_to_f32(want), rtol=2e-2, atol=1e-2, err_msg=name)

    def plugin(self, torch):
        b, s, h, d = self.B, self.S, self.H, self.D
        qs, ls, acc = (b, s, h, d), (b, h, s), (b, h, s, d)
        extra = [s * h * d] * 4 + [h * d] * 4 + [d] * 4 + [b, h, h, d, d]
        extra_s = ("[" + ", ".join(f"{v} : i64" for v in extra) + f", {self.scale!r} : f32, "
                   + ", ".join(f"{v} : i64" for v in (s, s, s, s)) + ", 0.0 : f32, -1 : i64, 0 : i64]")
        mq, ml = memref(qs, "bf16", "cuda"), memref(ls, "f32", "cuda")
        custom = lambda api, operands: (
            '"byre.custom"(' + ", ".join(o for o, _ in operands) + ') {callee = "custom", lib_path = "' + str(FLASH_LIB)
            + f'", api_name = "{api}", version = "2.5.3", extra_args = {extra_s}}} : ('
            + ", ".join(t for _, t in operands) + ") -> ()")
        names_in = ["Q", "K", "V"] + (["dOut"] if self.with_bwd else [])
        args = [(n, 1, qs, "bf16", "cpu") for n in names_in] + [("Out", 2, qs, "bf16", "cpu"), ("Lse", 2, ls, "f32", "cpu")]
        n_in = len(names_in)
        # device intermediates: %0..%3 q k v dout | %4 out %5 lse | %6 rng %7 softmax_ptr | %8..%10 dq dk dv %11 dsum %12 dq_accum
        allocs = [(qs, "bf16")] * 4 + [(qs, "bf16"), (ls, "f32"), ((2,), "i64"), ((1,), "f32")]
        body = [copy_op("cpu2cuda", f"%arg{i}", f"%{i}", qs, "bf16") for i in range(n_in)]
        body.append(custom("run_flash_attn_fwd", [("%0", mq), ("%1", mq), ("%2", mq), ("%6", memref((2,), "i64", "cuda")), ("%4", mq),
                                                  ("%5", ml), ("%7", memref((1,), "f32", "cuda"))]))
        bind = {n: ("in", i) for i, n in enumerate(names_in)}
        bind.update({"Out": ("out", 0), "Lse": ("out", 1)})
        if self.with_bwd:
            args += [("dQ", 2, qs, "bf16", "cpu"), ("dK", 2, qs, "bf16", "cpu"), ("dV", 2, qs, "bf16", "cpu")]
            allocs += [(qs, "bf16")] * 3 + [(ls, "f32"), (acc, "f32")]
            body.append(custom("run_flash_attn_bwd",
                               [("%3", mq), ("%0", mq), ("%1", mq), ("%2", mq), ("%4", mq), ("%5", ml), ("%6", memref((2,), "i64", "cuda")),
                                ("%8", mq), ("%9", mq), ("%10", mq), ("%11", ml), ("%12", memref(acc, "f32", "cuda"))]))
            bind.update({"dQ": ("out", 2), "dK": ("out", 3), "dV": ("out", 4)})
        body.append(copy_op("cuda2cpu", "%4", f"%arg{n_in}", qs, "bf16"))
        body.append(copy_op("cuda2cpu", "%5", f"%arg{n_in + 1}", ls, "f32"))
        if self.with_bwd:
            body += [copy_op("cuda2cpu", f"%{8 + j}", f"%arg{n_in + 2 + j}", qs, "bf16") for j in range(3)]
        return byre_module(args, allocs, body), bind


class AttnFwdBwd(AttnFwd):
    """FlashAttn fwd+bwd: bf16 Q,K,V,dO [B=8, S=4096, H=32, D=128] N(0,1), causal, scale 1/sqrt(128)"""
    key, name = "attn_fwd_bwd", "flash_attn_fwd_bwd_bf16_b8_s4096_h32_d128_causal"
    kernel = "flash_fwd_kernel, bwd_dot_do_o_kernel, flash_bwd_kernel<dK/dV>, flash_bwd_kernel<dQ> (whole step)"
    launches = 4
    with_bwd = True


class DecodeKv(Workload):
    """Decode step over a kv cache: bf16 q [B=16, 1, H=32, D=128], caches [16, 8192, H_k=8, 128] N(0,1) with
    U[6144, 8190] rows in use, one new row appended per step, scale 1/sqrt(128)"""
    key, name, dtype = "decode", "flash_attn_kvcache_bf16_b16_h32_hk8_d128_cache8192", "bf16 (f32 accumulate)"
    kernel = "decode_mma_kernel<128, bf16> + merge"
    launches = 2
    B, H, HK, D, CAP = 16, 32, 8, 128, 8192

    def __init__(self, rank, world):
        super().__init__(rank, world)
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

    N_BUF = 2

    def work(self):  # K and V rows in use, once each
        return int(2 * (self.lens.astype(np.int64) + 1).sum() * self.HK * self.D * 2)

    def cpu_work(self):
        return int(2 * (self.lens[:2].astype(np.int64) + 1).sum() * self.HK * self.D * 2)

    def to_dev(self, torch, x):
        return tuple(torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16) for a in x)

    def setup_gpu(self, torch, ops, xs):
        self.ops, self.torch = ops, torch
        self.kc, self.vc = self.to_dev(torch, (self.kcache, self.vcache))
        self.lens_d = torch.from_numpy(self.lens).cuda()
        self.o = torch.empty_like(xs[0][0])
        self.lse = torch.empty((self.B, self.H, 1), dtype=torch.float32, device="cuda")
        p = ops.kvcache_params(xs[0][0], self.kc, self.vc, xs[0][1], xs[0][2], self.o, self.scale, True)
        from byteir_b200 import _native as N
        self.ws = torch.empty(max(16, N.lib().b200_flash_attn_kvcache_workspace_bytes(ctypes.byref(p))), dtype=torch.uint8,
                              device="cuda")

    def step_gpu(self, x):
        q, kn, vn = x
        self.ops.flash_attn_kvcache(q, self.kc, self.vc, kn, vn, self.lens_d, self.scale, True, out=self.o,
                                    lse=self.lse, workspace=self.ws)
        return self.o, self.lse

    cpu_sample = "two of the sixteen batch entries"

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

    def plugin(self, torch):
        b, h, hk, d, cap = self.B, self.H, self.HK, self.D, self.CAP
        qs, cs, ns, ls = (b, 1, h, d), (b, cap, hk, d), (b, 1, hk, d), (b, h, 1)
        ints = [h * d, cap * hk * d, cap * hk * d, hk * d, hk * d, h * d,      # batch strides q k v knew vnew o
                h * d, hk * d, hk * d, hk * d, hk * d, h * d,                  # row strides
                d, d, d, d, d, d,                                              # head strides
                b, h, hk, d, d, 1]                                             # b h h_k d d_rounded seqlen_knew
        extra_s = ("[" + ", ".join(f"{v} : i64" for v in ints) + f", {self.scale!r} : f32, "
                   + ", ".join(f"{v} : i64" for v in (1, cap, 128, cap, -1, 0)) + "]")
        ops_ = [("%0", memref(qs, "bf16", "cuda")), ("%arg3", memref(cs, "bf16", "cuda")), ("%arg4", memref(cs, "bf16", "cuda")),
                ("%1", memref(ns, "bf16", "cuda")), ("%2", memref(ns, "bf16", "cuda")), ("%arg5", memref((b,), "i32", "cuda")),
                ("%3", memref(qs, "bf16", "cuda")), ("%4", memref(ls, "f32", "cuda"))]
        custom = ('"byre.custom"(' + ", ".join(o for o, _ in ops_) + ') {callee = "custom", lib_path = "' + str(FLASH_LIB)
                  + f'", api_name = "run_flash_attn_kvcache", version = "2.5.3", extra_args = {extra_s}}} : ('
                  + ", ".join(t for _, t in ops_) + ") -> ()")
        text = byre_module(
            [("Q", 1, qs, "bf16", "cpu"), ("KNew", 1, ns, "bf16", "cpu"), ("VNew", 1, ns, "bf16", "cpu"),
             ("KCache", 2, cs, "bf16", "cuda"), ("VCache", 2, cs, "bf16", "cuda"), ("SeqLenK", 1, (b,), "i32", "cuda"),
             ("Out", 2, qs, "bf16", "cpu"), ("Lse", 2, ls, "f32", "cpu")],
            [(qs, "bf16"), (ns, "bf16"), (ns, "bf16"), (qs, "bf16"), (ls, "f32")],
            [copy_op("cpu2cuda", "%arg0", "%0", qs, "bf16"), copy_op("cpu2cuda", "%arg1", "%1", ns, "bf16"),
             copy_op("cpu2cuda", "%arg2", "%2", ns, "bf16"), custom,
             copy_op("cuda2cpu", "%3", "%arg6", qs, "bf16"), copy_op("cuda2cpu", "%4", "%arg7", ls, "f32")])
        return text, {"Q": ("in", 0), "KNew": ("in", 1), "VNew": ("in", 2), "KCache": ("dev", self.kc), "VCache": ("dev", self.vc),
                      "SeqLenK": ("dev", self.lens_d), "Out": ("out", 0), "Lse": ("out", 1)}


PRIMARY = ReduceC2
ITEMS = [ReduceC1, ReduceC2Sum, ReduceC2Max, GatherC3, ScatterC3, Transpose4D, Transpose2D, AttnFwd, AttnFwdBwd, DecodeKv]
WORKLOADS = {c.key: c for c in [PRIMARY] + ITEMS}
METRIC = "HBM GB/s (algorithmic bytes / time) of the ByRE compute op"
METRIC_TENSOR = "flash-attn TFLOP/s (algorithmic FLOPs / time)"


def metric_of(wl):
    return METRIC_TENSOR if wl.bound == "tensor" else METRIC


def rate(wl, work, seconds):
    """GB/s for byte work, TFLOP/s for FLOP work"""
    return work / seconds / (1e12 if wl.bound == "tensor" else 1e9)


# ----------------------------------------------------------------------------
# the reference arm and the CPU legs
# ----------------------------------------------------------------------------
def oracle_with_all_cores():
    """the CPU oracle with as many OpenMP threads as this process may run on (a launcher may have exported
    OMP_NUM_THREADS=1 for its ranks)"""
    import oracle_lib as O
    cores = host_cores()
    O.lib().oracle_set_num_threads(cores)
    return O, O.lib().oracle_num_threads()


def time_cpu(wl, O, xs_host, seconds, max_steps=50):
    wl.step_cpu(O, xs_host[0])
    t0 = time.perf_counter()
    n = 0
    while True:
        wl.step_cpu(O, xs_host[n % len(xs_host)])
        n += 1
        if time.perf_counter() - t0 > seconds or n >= max_steps:
            break
    return (time.perf_counter() - t0) / n, n


def sample_text(wl, n):
    if wl.cpu_sample is None:
        return f"{n} full steps of the same workload"
    if isinstance(wl.cpu_sample, tuple):
        return f"{n} steps on a {wl.cpu_sample} [B,S,H,D] slice of the workload"
    return f"{n} steps on {wl.cpu_sample}"


def run_reference(args, rank, world, json_out):
    """The reference arm: the CPU restatement of the reference's op semantics on all host cores (the
    reference's own CPU pipeline needs LLVM/MLIR, which this image does not have)."""
    if rank != 0:
        return
    O, cores = oracle_with_all_cores()
    wl = WORKLOADS[args.workload](0, 1)
    xs = wl.host_inputs(wl.N_BUF)
    for i in range(args.warmup):
        wl.step_cpu(O, xs[i % len(xs)])
    t0 = time.perf_counter()
    for i in range(args.steps):
        wl.step_cpu(O, xs[i % len(xs)])
    dt = (time.perf_counter() - t0) / args.steps
    val = rate(wl, wl.cpu_work(), dt)
    others = {}
    if args.workload == PRIMARY.key and not args.only_primary:
        for cls in ITEMS:
            w = cls(0, 1)
            dts, n = time_cpu(w, O, w.host_inputs(2), 3.0, 20)
            others[w.key] = {"workload": w.name, "value": rate(w, w.cpu_work(), dts), "unit": w.unit,
                             "ms_per_step": dts * 1e3, "sample": sample_text(w, n)}
    json_out.write(json.dumps({
        "impl": "reference", "metric": metric_of(wl), "value": val, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded numpy Generator)",
        "config": {"workload": wl.name, "note": "CPU port of the reference op semantics on the host cores; "
                   + sample_text(wl, args.steps)},
        "cpu_baseline": {"value": val, "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": sample_text(wl, args.steps)},
        "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "workloads": others or None,
    }) + "\n")
    json_out.flush()


# ----------------------------------------------------------------------------
# GPU measurement of one workload
# ----------------------------------------------------------------------------
class Bench:
    def __init__(self, args, torch, dist, rank, world, local_rank):
        self.args, self.torch, self.dist = args, torch, dist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        self.peaks = measured_peaks()
        self.traffic = captured_traffic()
        self.ev0 = torch.cuda.Event(enable_timing=True)
        self.ev1 = torch.cuda.Event(enable_timing=True)
        self._ref = None

    def sync_all(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.dist is None:
            return ms
        t = self.torch.tensor([ms], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def capture(self, fn, count):
        torch = self.torch
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.graph(g, stream=side):
            for i in range(count):
                fn(i)
        return g

    def timed_replays(self, step, steps, replays, align=False):
        """`replays` timed regions of exactly `steps` steps each: barrier + synchronize on both sides, CUDA
        events around the region, max over ranks; returns ms per step of every region"""
        graph = None
        if not self.args.no_graph:
            try:
                graph = self.capture(step, steps)
                graph.replay()  # untimed: the first replay uploads the graph
            except Exception as e:  # pragma: no cover - depends on the NCCL / driver combination
                print(f"graph capture failed ({e}); timing eager launches", file=sys.stderr)
                graph = None
        out = []
        for _ in range(replays):
            self.sync_all()
            if graph is not None and align:
                # Ranks leave the host barrier hundreds of microseconds apart, which is comparable to the
                # whole timed region.  One more untimed replay is queued right before the timed one: its
                # last exchange aligns the GPUs to within microseconds, and the timed steps start there.
                graph.replay()
            self.ev0.record()
            if graph is not None:
                graph.replay()
            else:
                for i in range(steps):
                    step(i)
            self.ev1.record()
            self.sync_all()
            out.append(self.max_over_ranks(self.ev0.elapsed_time(self.ev1)) / steps)
        return out, graph

    def ref_lib(self):
        if self._ref is None and REF_LIB.exists():
            lib = ctypes.CDLL(str(REF_LIB))
            C = ctypes
            lib.ref_reduce_workspace_bytes.restype = C.c_size_t
            lib.ref_reduce_workspace_bytes.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t]
            lib.ref_reduce.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                       C.c_void_p, C.c_void_p]
            lib.ref_index_select.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [C.c_void_p]
            lib.ref_index_put_f32.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p]
            lib.ref_transpose2d.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
            self._ref = lib
        return self._ref

    def measure(self, wl, steps, replays, primary, light=False):
        torch, args, rank, world = self.torch, self.args, self.rank, self.world
        from byteir_b200 import ops
        n_buf = wl.N_BUF
        xs_host = wl.host_inputs(n_buf)
        per_buf = sum(a.nbytes for a in xs_host[0])
        xs = [wl.to_dev(torch, x) for x in xs_host]
        wl.setup_gpu(torch, ops, xs)
        pipelined = isinstance(wl, ReduceC2) and world > 1

        # correctness of what is about to be timed
        outs = wl.step_gpu(xs[0])
        torch.cuda.synchronize()
        O = None
        if rank == 0:
            import oracle_lib as O
            wl.check(O, xs_host[0], outs)
        for i in range(args.warmup):
            wl.step_gpu(xs[i % n_buf])
        self.sync_all()

        def step(i):
            if pipelined:
                wl.step_gpu(xs[i % n_buf], pipelined=True)
                if i == steps - 1:
                    wl.end_batch()
            else:
                wl.step_gpu(xs[i % n_buf])

        sampler = ClockSampler(self.local_rank)
        if rank == 0:
            sampler.start()
        per_step, graph = self.timed_replays(step, steps, replays, align=pipelined)
        clocks = sampler.stop() if rank == 0 else None
        ms = float(np.median(per_step))
        entry = {
            "workload": wl.name, "value": rate(wl, wl.work() * world, ms * 1e-3), "unit": wl.unit, "ms_per_step": ms,
            "steps": steps,
            "replays": {"n": len(per_step), "median_ms_per_step": ms, "min_ms_per_step": float(min(per_step)),
                        "max_ms_per_step": float(max(per_step))},
            "dtype": wl.dtype, "gpu_launches": wl.launches * steps, "clocks": clocks,
            "l2_policy": f"inputs rotate over {n_buf} distinct buffers of {per_buf / 2**20:.0f} MiB (L2 is 126 MiB)"
            if n_buf > 1 else f"one input set of {per_buf / 2**20:.0f} MiB per step (L2 is 126 MiB)",
        }

        if light:
            del graph
            return entry

        # roofline: the op's own duration.  For a one-op workload that is the step itself; the combined
        # step reports its column sum, timed alone in the same way.
        peak = self.peaks["bf16_tflops"] if wl.bound == "tensor" else self.peaks["hbm_gbs"]
        if primary and isinstance(wl, ReduceC2):
            dom = ReduceC2Sum(rank, world)
            dom_xs = [(x[0],) for x in xs]
            dom.setup_gpu(torch, ops, dom_xs)
            dom_step = lambda i: dom.step_gpu(dom_xs[i % n_buf])
            for i in range(3):
                dom_step(i)
            dom_ms_all, _ = self.timed_replays(dom_step, max(steps, 20), replays)
            dom_ms, dom_work, dom_name, dom_key = float(np.median(dom_ms_all)), dom.work(), dom.kernel, dom.key
        else:
            dom_ms, dom_work, dom_name, dom_key = ms, wl.work(), wl.kernel, wl.key
        achieved = rate(wl, dom_work, dom_ms * 1e-3)
        entry["roofline"] = {"bound": wl.bound, "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": wl.unit,
                             "frac": achieved / peak, "peak_source": self.peaks["source"], "us_per_launch": dom_ms * 1e3,
                             "traffic": self.traffic.get(dom_key)}
        if wl.bound == "tensor":
            # `peak` is the burst figure (a GEMM timed alone).  A batch of back-to-back launches runs into
            # the power cap (see `clocks`), the regime of the sustained figure, reported beside it.
            entry["roofline"]["peak_sustained"] = self.peaks["bf16_tflops_sustained"]
            entry["roofline"]["frac_of_sustained"] = achieved / self.peaks["bf16_tflops_sustained"]
            # ... and the step timed in short bursts, the regime of the burst figure: after a pause that lets
            # the GPU cool, one untimed step and three timed ones; median of five such bursts
            alone = []
            for i in range(5):
                torch.cuda.synchronize()
                time.sleep(0.25)
                wl.step_gpu(xs[i % n_buf])  # untimed: brings the clocks back up after the pause
                self.ev0.record()
                for j in range(3):
                    wl.step_gpu(xs[(i + j) % n_buf])
                self.ev1.record()
                torch.cuda.synchronize()
                alone.append(self.ev0.elapsed_time(self.ev1) / 3)
            alone_ms = self.max_over_ranks(float(np.median(alone)))
            a_rate = rate(wl, wl.work() * world, alone_ms * 1e-3)
            entry["roofline"]["alone"] = {"ms_per_step": alone_ms, "achieved": a_rate / world, "frac": a_rate / world / peak}

        # the reference's own GPU kernel on the same inputs
        entry["ref_gpu"] = None
        ref = self.ref_lib()
        spec = wl.ref_gpu(ref, torch) if ref is not None else None
        if spec is not None:
            ref_name, ref_run = spec[0], spec[1]
            ours_run = spec[2] if len(spec) > 2 else None
            reps = max(3, min(steps, 10))
            for i in range(2):
                ref_run(xs[i % n_buf])
            torch.cuda.synchronize()
            ref_ms_all, _ = self.timed_replays(lambda i: ref_run(xs[i % n_buf]), reps, 3)
            ref_ms = float(np.median(ref_ms_all))
            ours_ms = ms
            if ours_run is not None:
                for i in range(2):
                    ours_run(xs[i % n_buf])
                ours_all, _ = self.timed_replays(lambda i: ours_run(xs[i % n_buf]), reps, 3)
                ours_ms = float(np.median(ours_all))
            entry["ref_gpu"] = {"kernel": ref_name, "ms_per_step": ref_ms, "ours_ms_per_step": ours_ms,
                                "x_over_ref_gpu": ref_ms / ours_ms}

        # the same op in another form (the in-place scatter-add), timed the same way
        for vkey, (vrun, vwork, vnote) in wl.variants(torch).items():
            for i in range(2):
                vrun(xs[i % n_buf])
            v_all, _ = self.timed_replays(lambda i: vrun(xs[i % n_buf]), max(3, min(steps, 10)), 3)
            v_ms = float(np.median(v_all))
            v_rate = rate(wl, vwork, v_ms * 1e-3)
            entry[vkey] = {"ms_per_step": v_ms, "value": v_rate, "unit": wl.unit, "frac": v_rate / peak, "work": vwork,
                           "note": vnote}

        entry["e2e"] = self.e2e(wl, xs_host, xs, outs)

        entry["cpu_baseline"] = None
        if world == 1 and not args.no_cpu_baseline and rank == 0:
            O, cores = oracle_with_all_cores()
            dt, n = time_cpu(wl, O, xs_host, 10.0 if primary else 4.0)
            entry["cpu_baseline"] = {"value": rate(wl, wl.cpu_work(), dt), "unit": wl.unit, "cores": cores, "kind": "port",
                                     "sample": sample_text(wl, n), "ms_per_step": dt * 1e3}
        del graph
        return entry

    def e2e(self, wl, xs_host, xs, outs):
        """The step through the plug-in boundary with host buffers: a ByRE module with "cpu"-space arguments
        run by Session::Run (cpu2cuda, the op, cuda2cpu), timed with CUDA events on the request's stream."""
        torch, world = self.torch, self.world
        # a stream of its own: the handle of torch's default stream is 0, which the request would take for
        # "no stream given" and replace by a queue of its own, outside the timed region
        if not hasattr(self, "e2e_stream"):
            self.e2e_stream = torch.cuda.Stream()
        self.e2e_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.e2e_stream):
            out = self._e2e(wl, xs_host, xs, outs)
        torch.cuda.current_stream().wait_stream(self.e2e_stream)
        return out

    def _e2e(self, wl, xs_host, xs, outs):
        torch, world = self.torch, self.world
        steps = 3 if wl.bound == "tensor" or wl.work() > (1 << 29) else max(3, min(self.args.steps, 10))
        pinned_in = [tuple(torch.from_numpy(bits_view(p)).pin_memory() for p in x) for x in xs_host[:2]]
        if len(pinned_in) == 1:
            pinned_in = pinned_in * 2
        pinned_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        pinned_outs = [pinned_out, [torch.empty_like(o).pin_memory() for o in pinned_out]]
        h2d = sum(p.numel() * p.element_size() for p in pinned_in[0])
        d2h = sum(p.numel() * p.element_size() for p in pinned_out)
        spec = wl.plugin(torch)
        cur = torch.cuda.current_stream()
        streams = [cur, cur]
        if spec is not None:
            from byteir_b200 import brt
            text, binding = spec
            session = wl.make_session(brt, self.local_rank)
            session.load_from_memory(text)
            # Two requests in flight, each on a stream of its own: the upload of one step runs beside the
            # download of the step before (the bus is full duplex), as a serving loop would double-buffer.
            # A module with an exchange keeps one stream: its protocol is one call chain per rank.
            # Only where both directions carry megabytes: two uploads side by side share one copy engine and
            # measured slower than one after the other (reductions 51 -> 41 GB/s), and a step that moves
            # kilobytes (the decode step) gains nothing from a second stream.
            up = sum(a.nbytes for a in session.args() if binding[a.name][0] == "in")
            down = sum(a.nbytes for a in session.args() if binding[a.name][0] == "out")
            if min(up, down) * 5 >= max(up, down) and min(up, down) >= (8 << 20) and not (world > 1 and isinstance(wl, ReduceC2)):
                streams = [torch.cuda.Stream(), torch.cuda.Stream()]
            reqs = []
            for k in range(2):
                req = session.new_request(streams[k].cuda_stream)
                used_in = set()
                for a in session.args():
                    kind, what = binding[a.name]
                    t = pinned_in[k][what] if kind == "in" else pinned_outs[k][what] if kind == "out" else what
                    if kind == "in":
                        used_in.add(what)
                    assert a.nbytes == t.numel() * t.element_size(), (a.name, a.nbytes)
                    req.bind_arg(a.offset, t.data_ptr())
                req.finish_io_binding()
                reqs.append(req)
            h2d = sum(pinned_in[0][i].numel() * pinned_in[0][i].element_size() for i in used_in)
            d2h = sum(pinned_out[w].numel() * pinned_out[w].element_size() for kind, w in binding.values() if kind == "out")
            run = lambda i: reqs[i % 2].run()
            path = "ByRE module with host-space arguments through brt Session::Run (libbrt_b200.so)"
        else:
            dev_in = [tuple(torch.empty_like(p, device="cuda") for p in parts) for parts in pinned_in]

            def run(i):
                k = i % 2
                for src, dst in zip(pinned_in[k], dev_in[k]):
                    dst.copy_(src, non_blocking=True)
                o = wl.step_gpu(tuple(d.view(x.dtype) for d, x in zip(dev_in[k], xs[0])))
                for src, dst in zip(o, pinned_out):
                    dst.copy_(src, non_blocking=True)
            path = "typed C ABI with explicit pinned copies"

        def batch(count):  # `count` steps between two points of the current stream
            for st in streams:
                if st is not cur:
                    st.wait_stream(cur)
            for i in range(count):
                run(i)
            for st in streams:
                if st is not cur:
                    cur.wait_stream(st)
        # Warm-up, then a timed region of at least ~20 ms: the first copies after the bus was idle run at two
        # thirds of the rate (measured: 16 MiB uploads 38 GB/s in the first ten, 50 GB/s over fifty), which a
        # region of ten small steps would mostly consist of.
        self.sync_all()
        self.ev0.record()
        batch(2)
        self.ev1.record()
        self.sync_all()
        est = max(self.max_over_ranks(self.ev0.elapsed_time(self.ev1)) / 2, 1e-3)
        steps = int(min(100, max(steps, round(20.0 / est))))
        batch(int(min(50, max(2, round(10.0 / est)))))
        self.sync_all()
        self.ev0.record()
        batch(steps)
        self.ev1.record()
        self.sync_all()
        ms = self.max_over_ranks(self.ev0.elapsed_time(self.ev1)) / steps
        if spec is not None:
            # what comes back through the boundary is what the typed path computes on the same input
            reqs[0].run()
            reqs[0].sync()
            want = wl.e2e_want(xs[0]) if hasattr(wl, "e2e_want") else wl.step_gpu(xs[0])
            torch.cuda.synchronize()
            for kind, w in binding.values():
                if kind == "out":
                    a, b = pinned_out[w].reshape(-1)[:65536], want[w].reshape(-1)[:65536].cpu()
                    if world > 1 and isinstance(wl, ReduceC2):  # an NCCL all-reduce may add the ranks in another order
                        assert torch.allclose(a.float(), b.float(), rtol=2e-2, atol=2e-2), f"{wl.key}: paths differ"
                    else:
                        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), f"{wl.key}: plug-in path and typed path differ"
            for r in reqs:
                r.close()
            session.close()
        out = {"value": rate(wl, wl.work() * world, ms * 1e-3), "unit": wl.unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms, "steps": steps, "path": path,
               "requests_in_flight": 2 if streams[0] is not cur else 1}
        if isinstance(wl, ReduceC2):
            out["note"] = "the module takes x once and runs both ops of the configuration on it (one upload per step)"
        return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=PRIMARY.key, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only-primary", action="store_true", help="skip the `workloads` entries of the other configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--attn-shape", default="", help="B,S,H override of the attention workloads (profiling a small case)")
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
    from byteir_b200 import ops  # noqa: F401  fails loudly if the CUDA library is missing

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.attn_shape:
        b, s, h = (int(v) for v in args.attn_shape.split(","))
        for cls in (AttnFwd, AttnFwdBwd):
            cls.B, cls.S, cls.H = b, s, h
            cls.name = cls.name.replace("b8_s4096_h32", f"b{b}_s{s}_h{h}")

    bench = Bench(args, torch, dist, rank, world, local_rank)
    wl = WORKLOADS[args.workload](rank, world)
    top = bench.measure(wl, args.steps, 5, primary=True)

    strong = None
    if world > 1 and args.workload == PRIMARY.key and 64 % world == 0:
        # the fixed [64, 512, 1024] tensor split over the ranks (strong scaling), beside the weak-scaling value
        strong = bench.measure(ReduceC2(rank, world, rows0=64 // world), args.steps, 5, primary=False, light=True)

    others = None
    if args.workload == PRIMARY.key and not args.only_primary:
        others = {}
        sub_steps = max(3, min(args.steps, 20))
        for cls in ITEMS:
            if cls is DecodeKv:  # the attention inputs (1 GiB of host memory) are no longer needed
                _HOST_CACHE.pop(("attn", rank, (AttnFwd.B, AttnFwd.S, AttnFwd.H, AttnFwd.D)), None)
            w = cls(rank, world)
            t0 = time.perf_counter()
            others[w.key] = bench.measure(w, sub_steps, 5, primary=False)
            others[w.key]["bench_seconds"] = time.perf_counter() - t0
            del w
            torch.cuda.empty_cache()

    def finish():
        # Tearing the NCCL group down while CUDA graphs that captured its collectives exist has
        # blocked; the ranks meet once more, and the processes leave without the group destructor.
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

    line = {
        "metric": metric_of(wl), "value": top["value"], "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": top["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded numpy Generator)",
        "config": {"workload": wl.name, "per_gpu_batch": " ".join(wl.__doc__.split()),
                   "l2_policy": top["l2_policy"] + ("; the sum and the max of a step read different buffers"
                                                    if isinstance(wl, ReduceC2) else ""),
                   "launch": "eager launches" if args.no_graph else "CUDA graph replay of the K steps, median of 5 replays",
                   "exchange": getattr(wl, "exchange", "none"),
                   "scaling_note": "weak: every rank holds a full per-GPU batch, so the global tensor grows with N"
                   + ("; `strong` is the fixed tensor split N ways" if strong else ""),
                   "parallelism": f"dp{world}"},
        "replays": top["replays"], "roofline": top["roofline"], "cpu_baseline": top["cpu_baseline"], "ref_gpu": top["ref_gpu"],
        "e2e": top["e2e"], "gpu_launches": top["gpu_launches"], "clocks": top["clocks"],
        "strong": strong, "workloads": others,
    }
    if "in_place" in top:
        line["in_place"] = top["in_place"]
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
    finish()


if __name__ == "__main__":
    main()
