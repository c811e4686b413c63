"""The exchange step of the hot path on CPU ranks, through the plug-in boundary: every rank is a
brt DistributedSession that loads its own ByRE module (the reference's Distributed/all_reduce.mlir with
host-space memrefs) and runs `nccl.AllReduce` on the communicator the host program hands it.  Two forms:
ranks as threads of one process with a hand-made communicator, and ranks as two gloo processes whose
communicator is torch.distributed's process group, created once.  The classes under test are the product's
(DistributedSession, the AllReduce op kernel, DistributedBackendCallback); the oracle is numpy."""
import ctypes as C
import os
import sys
import threading
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

# runtime/test/test_files/Distributed/all_reduce.mlir (loose spacing kept), memrefs moved to the host space,
# the group rewritten to the ranks of the test
ALL_REDUCE = """
module attributes {byre.container_module} {
  func.func @test_all_reduce(%arg0 : memref<%Nx%T, "%SPACE"> {byre.argname = "in0", byre.argtype = 1: i32},
                             %arg1 : memref<%Nx%OT, "%SPACE"> {byre.argname = "out", byre.argtype = 2: i32}) attributes {byre.entry_point} {
    byre.compute @nccl.AllReduce(%arg0, %arg1) { reduction = "%OP" , replica_group = [%GROUP]} : memref<%Nx%T, "%SPACE">, memref<%Nx%OT, "%SPACE">
    return
  }
}
"""

NP_DT = {"f32": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64}


def module(n, t="f32", op="sum", group=(0, 1), space="cpu", out_t=None):
    return (ALL_REDUCE.replace("%N", str(n)).replace("%OT", out_t or t).replace("%T", t).replace("%OP", op)
            .replace("%GROUP", " ,".join(str(g) for g in group)).replace("%SPACE", space))


def host_array(ptr, n, dtype):
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(np.ctypeslib.as_ctypes_type(NP_DT[dtype]))), (n,))


class ThreadComm:
    """a communicator for ranks that are threads: a slot per rank and a barrier"""

    def __init__(self, world):
        self.world = world
        self.slots = [None] * world
        self.barrier = threading.Barrier(world, timeout=30)
        self.calls = []

    def all_reduce(self, rank):
        def fn(send, recv, n, dtype, op, group, stream):
            assert stream is None, "host buffers carry no stream"
            self.calls.append((rank, n, dtype, op, tuple(group)))
            self.slots[rank] = host_array(send, n, dtype).copy()
            self.barrier.wait()
            ranks = group or range(self.world)
            stack = np.stack([self.slots[r] for r in ranks])
            host_array(recv, n, dtype)[:] = {"sum": stack.sum(0), "max": stack.max(0), "min": stack.min(0)}[op]
            self.barrier.wait()  # nobody overwrites a slot that a peer still reads
        return fn


def _run_rank(brt, rank, world, text, x, out, comm, errors):
    try:
        s = brt.DistributedSession(rank, world, device="cpu")
        assert (s.rank, s.nranks) == (rank, world)
        s.load_from_memory(text)
        s.set_allreduce(comm.all_reduce(rank))
        req = s.new_request()
        req.bind_arg(s.arg_offset("in0"), x.ctypes.data)
        req.bind_arg(s.arg_offset("out"), out.ctypes.data)
        req.finish_io_binding()
        for _ in range(2):  # the reference's tests run every module twice on one context
            req.run()
            req.sync()
        req.close()
        s.close()
    except Exception as e:  # pragma: no cover - reported by the test body
        errors.append((rank, e))
        comm.barrier.abort()


@pytest.mark.parametrize("op", ["sum", "max", "min"])
@pytest.mark.parametrize("world", [2, 3])
def test_all_reduce_module_on_thread_ranks(world, op):
    from byteir_b200 import brt
    rng = np.random.default_rng(world)
    xs = [rng.standard_normal(4).astype(np.float32) for _ in range(world)]
    outs = [np.zeros(4, np.float32) for _ in range(world)]
    comm, errors = ThreadComm(world), []
    text = module(4, "f32", op, range(world))
    threads = [threading.Thread(target=_run_rank, args=(brt, r, world, text, xs[r], outs[r], comm, errors))
               for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    want = {"sum": np.sum, "max": np.max, "min": np.min}[op](np.stack(xs), axis=0)
    for r in range(world):
        np.testing.assert_allclose(outs[r], want, rtol=1e-6)
    assert (0, 4, "f32", op, tuple(range(world))) in comm.calls  # attributes reach the communicator as written


def test_all_reduce_without_a_communicator_and_with_a_failing_one():
    from byteir_b200 import brt
    x, out = np.ones(4, np.float32), np.zeros(4, np.float32)

    def bound(session):
        req = session.new_request()
        req.bind_arg(0, x.ctypes.data)
        req.bind_arg(1, out.ctypes.data)
        req.finish_io_binding()
        return req

    plain = brt.Session("cpu")  # an ordinary session has no communicator to hand to the op
    plain.load_from_memory(module(4))
    with pytest.raises(brt.BrtError, match="communicator"):
        bound(plain).run()
    s = brt.DistributedSession(0, 1, device="cpu")
    s.load_from_memory(module(4, group=(0,)))
    with pytest.raises(brt.BrtError, match="communicator"):
        bound(s).run()

    def broken(*_):
        raise RuntimeError("link down")
    s.set_allreduce(broken)
    with pytest.raises(brt.BrtError, match="callback failed"):
        bound(s).run()
    assert isinstance(s.allreduce_error, RuntimeError)
    with pytest.raises(brt.BrtError, match="not a distributed session"):
        brt._check(brt.lib().brt_session_set_allreduce_callback(plain._h, None, None))


def test_all_reduce_op_checks_its_module():
    from byteir_b200 import brt
    s = brt.DistributedSession(1, 4, device="cuda", device_id=0)  # loading needs no device
    # the reference's own fixture text, device memrefs, group [1, 2, 3]
    s.load_from_memory(module(4, group=(1, 2, 3), space="cuda"))
    assert [a.name for a in s.args()] == ["in0", "out"]
    with pytest.raises(brt.BrtError, match="unknown reduction"):
        s.load_from_memory(module(4, op="prod", space="cuda"))
    with pytest.raises(brt.BrtError, match="element types differ"):
        s.load_from_memory(module(4, t="f16", out_t="f32", space="cuda"))
    s.load_from_memory(module(1024, t="f32", out_t="f16", space="cuda"))  # the sum of partials, rounded once
    s.load_from_memory(module(1024, t="f32", out_t="bf16", space="cuda"))
    with pytest.raises(brt.BrtError, match="not one of 2 ranks"):
        brt.DistributedSession(2, 2, device="cpu")


# ---- ranks as gloo processes ---------------------------------------------------------------------------
def _gloo_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    from byteir_b200 import brt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # the communicator, created once
    try:
        ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
        calls = []

        def all_reduce(send, recv, n, dtype, op, group, stream):
            calls.append((n, dtype, op, tuple(group)))
            t = torch.from_numpy(host_array(recv, n, dtype))
            t.copy_(torch.from_numpy(host_array(send, n, dtype)))
            dist.all_reduce(t, op=ops[op])

        rng = np.random.default_rng(7 + rank)
        n = 1024  # the f32 partial sums of the sharded column reduction
        x = rng.standard_normal(n).astype(np.float32)
        ok = True
        for op in ("sum", "max"):
            s = brt.DistributedSession(rank, world, device="cpu")
            s.load_config([_write(module(n, "f32", op, range(world)), r, op) for r in range(world)])
            s.set_allreduce(all_reduce)
            out = np.zeros(n, np.float32)
            req = s.new_request()
            req.bind_arg(s.arg_offset("in0"), x.ctypes.data)
            req.bind_arg(s.arg_offset("out"), out.ctypes.data)
            req.finish_io_binding()
            req.run()
            req.sync()
            every = [torch.empty(n) for _ in range(world)]
            dist.all_gather(every, torch.from_numpy(x))
            stack = np.stack([e.numpy() for e in every])
            want = stack.sum(0) if op == "sum" else stack.max(0)
            ok = ok and np.allclose(out, want, rtol=1e-6, atol=1e-6)
            req.close()
            s.close()
        ok = ok and calls == [(n, "f32", "sum", tuple(range(world))), (n, "f32", "max", tuple(range(world)))]
        if rank == 0:
            q.put(bool(ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _write(text, rank, tag):
    import tempfile
    d = Path(tempfile.gettempdir()) / f"byre_all_reduce_{os.getpid()}"  # a directory per rank process
    d.mkdir(exist_ok=True)
    p = d / f"rank{rank}_{tag}.mlir"
    p.write_text(text)
    return str(p)


def test_all_reduce_module_on_two_gloo_processes():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True
