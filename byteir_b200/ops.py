"""Host-side mirror of the ByRE compute ops of the default CUDA provider, over
torch CUDA tensors.  torch supplies device memory and the current stream only;
every op runs the sm_100a kernels through the C ABI.

Semantics follow the reference op kernels
(runtime/lib/backends/cuda/providers/default/{reduction,indexing,
tensor_manipulate}): ReduceSumOp / ReduceMaxOp with a `dimensions` attribute
(consecutive dims), IndexSelectOp / IndexPutOp with `dim`, TransposeOp with
`permutation`.
"""
import ctypes as C

import torch

from . import _native as N

_DT = {torch.float32: N.F32, torch.float16: N.F16, torch.bfloat16: N.BF16}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported element type {t.dtype}") from None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise ValueError("byteir_b200 ops take CUDA tensors; there is no CPU path")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous (ByRE memrefs are)")


def reduce_abc(shape, dimensions):
    """A x B x C view of reduce_impl.h:28-59.  Dimensions of size 1 are taken out of the shape first, so
    that reduced dimensions with only such dimensions between them count as consecutive."""
    keep = [i for i, s in enumerate(shape) if s != 1]
    renumber = {d: k for k, d in enumerate(keep)}
    dims = sorted({renumber[d] for d in dimensions if shape[d] != 1})
    if not dims:
        n = 1
        for s in shape:
            n *= s
        return 0, 0, n
    shape = [shape[i] for i in keep]
    for a, b in zip(dims, dims[1:]):
        if b - a != 1:
            raise ValueError("Only consecutive dimensions reduction is supported")
    A = B = Cc = 1
    for s in shape[:dims[0]]:
        A *= s
    for d in dims:
        B *= shape[d]
    for s in shape[dims[-1] + 1:]:
        Cc *= s
    return A, B, Cc


class _NoWorkspace:
    @staticmethod
    def data_ptr():
        return None

    @staticmethod
    def numel():
        return 0


def _workspace(nbytes, device):
    if int(nbytes) == 0:
        return _NoWorkspace
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def _reduce(op, x, dimensions, out=None, workspace=None):
    _need_cuda(x)
    A, B, Cc = reduce_abc(tuple(x.shape), list(dimensions))
    out_shape = [s for i, s in enumerate(x.shape) if i not in set(dimensions)]
    if out is None:
        out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
    need = N.lib().b200_reduce_workspace_bytes(op, _dt(x), A, B, Cc)
    if workspace is None:
        workspace = _workspace(need, x.device)
    rc = N.lib().b200_reduce(op, _dt(x), x.data_ptr(), out.data_ptr(), A, B, Cc,
                             workspace.data_ptr(), workspace.numel(), _stream())
    N.check(rc, "b200_reduce")
    return out


def reduce_sum(x, dimensions, out=None, workspace=None):
    return _reduce(N.REDUCE_SUM, x, dimensions, out, workspace)


def reduce_max(x, dimensions, out=None, workspace=None):
    return _reduce(N.REDUCE_MAX, x, dimensions, out, workspace)


def reduce_sum_to_f32(x, dimensions, out=None, workspace=None):
    """Unrounded f32 partial of a sum (the operand of a later all-reduce)."""
    _need_cuda(x)
    A, B, Cc = reduce_abc(tuple(x.shape), list(dimensions))
    if out is None:
        out = torch.empty(A * Cc, dtype=torch.float32, device=x.device)
    need = N.lib().b200_reduce_workspace_bytes(N.REDUCE_SUM, _dt(x), A, B, Cc)
    if workspace is None:
        workspace = _workspace(need, x.device)
    rc = N.lib().b200_reduce_sum_to_f32(_dt(x), x.data_ptr(), out.data_ptr(), A, B, Cc,
                                        workspace.data_ptr(), workspace.numel(), _stream())
    N.check(rc, "b200_reduce_sum_to_f32")
    return out


def cast_from_f32(x, dtype, out=None):
    _need_cuda(x)
    if out is None:
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
    N.check(N.lib().b200_cast_from_f32(_DT[dtype], x.data_ptr(), out.data_ptr(), x.numel(), _stream()),
            "b200_cast_from_f32")
    return out


def index_select(x, index, dim, out=None, status=None, path=0):
    _need_cuda(x, index)
    if index.dtype not in (torch.int64, torch.int32, torch.uint32):
        raise TypeError("index must be i64 or ui32")
    shape = tuple(x.shape)
    A = 1
    for s in shape[:dim]:
        A *= s
    Cc = 1
    for s in shape[dim + 1:]:
        Cc *= s
    IB, OB = shape[dim], index.numel()
    if out is None:
        out = torch.empty(shape[:dim] + (OB,) + shape[dim + 1:], dtype=x.dtype, device=x.device)
    rc = N.lib().b200_index_select_path(path, x.element_size(), index.element_size(), x.data_ptr(),
                                        index.data_ptr(), out.data_ptr(), A, IB, OB, Cc,
                                        status.data_ptr() if status is not None else None, _stream())
    N.check(rc, "b200_index_select")
    return out


def index_put_add(x, index, update, dim=0, out=None, workspace=None, status=None):
    """out = x; out[index[i], ...] += update[i, ...] (IndexPutOp, accumulate)."""
    _need_cuda(x, index, update)
    if index.dtype != torch.int64:
        raise TypeError("index must be i64")
    rows = 1
    for s in x.shape[:dim + 1]:
        rows *= s
    feature = 1
    for s in x.shape[dim + 1:]:
        feature *= s
    n = index.numel()
    if out is None:
        out = torch.empty_like(x)
    need = N.lib().b200_index_put_workspace_bytes(_dt(x), rows, n, feature)
    if workspace is None:
        workspace = _workspace(need, x.device)
    rc = N.lib().b200_index_put_add(_dt(x), x.data_ptr(), index.data_ptr(), update.data_ptr(),
                                    out.data_ptr(), rows, n, feature, workspace.data_ptr(),
                                    workspace.numel(), status.data_ptr() if status is not None else None,
                                    _stream())
    N.check(rc, "b200_index_put_add")
    return out


def transpose(x, permutation, out=None):
    _need_cuda(x)
    perm = list(permutation)
    if out is None:
        out = torch.empty([x.shape[p] for p in perm], dtype=x.dtype, device=x.device)
    shape = (C.c_int64 * x.dim())(*x.shape)
    p = (C.c_int64 * x.dim())(*perm)
    N.check(N.lib().b200_permute(x.element_size(), x.data_ptr(), out.data_ptr(), x.dim(), shape, p, _stream()),
            "b200_permute")
    return out


def transpose_batched(x, out=None, path=0):
    """[batch, rows, cols] -> [batch, cols, rows]"""
    _need_cuda(x)
    b, r, c = x.shape
    if out is None:
        out = torch.empty((b, c, r), dtype=x.dtype, device=x.device)
    N.check(N.lib().b200_transpose_batched_path(path, x.element_size(), x.data_ptr(), out.data_ptr(), b, r, c, _stream()),
            "b200_transpose_batched")
    return out


def _attn_params(q, k, v, o, scale, causal, window):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    p = N.FlashAttnParams()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1), q.stride(2)
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
    p.v_batch_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = o.stride(0), o.stride(1), o.stride(2)
    p.b, p.h, p.h_k, p.d = b, h, hk, d
    p.d_rounded = -(-d // 32) * 32
    p.softmax_scale = scale
    p.seqlen_q, p.seqlen_k = sq, sk
    p.seqlen_q_rounded, p.seqlen_k_rounded = -(-sq // 128) * 128, -(-sk // 128) * 128
    p.p_dropout = 0.0
    p.window_size_left = window[0]
    p.window_size_right = 0 if causal else window[1]
    return p


def flash_attn_fwd(q, k, v, softmax_scale, causal=True, window=(-1, -1), out=None, lse=None):
    """q, k, v: [B, S, H, D] (last dim contiguous), f16 or bf16.  Returns (out, softmax_lse[B, H, Sq])."""
    for t in (q, k, v):
        if not t.is_cuda or t.stride(-1) != 1:
            raise ValueError("q, k, v must be CUDA tensors with a contiguous last dim")
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((q.shape[0], q.shape[2], q.shape[1]), dtype=torch.float32, device=q.device)
    p = _attn_params(q, k, v, out, softmax_scale, causal, window)
    rc = N.lib().b200_flash_attn_fwd(_dt(q), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                     lse.data_ptr(), C.byref(p), _stream())
    N.check(rc, "b200_flash_attn_fwd")
    return out, lse


def flash_attn_bwd(dout, q, k, v, out, lse, softmax_scale, causal=True, window=(-1, -1),
                   dq=None, dk=None, dv=None, d_softmax_sum=None):
    """Gradients of flash_attn_fwd.  Returns (dq, dk, dv); dq/dk/dv share the strides of q/k/v."""
    for t in (dout, q, k, v, out):
        if not t.is_cuda or t.stride(-1) != 1:
            raise ValueError("tensors must be CUDA tensors with a contiguous last dim")
    if dout.stride() != out.stride():
        raise ValueError("dout must share out's strides")
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    p = _attn_params(q, k, v, out, softmax_scale, causal, window)
    if d_softmax_sum is None:
        d_softmax_sum = torch.empty((q.shape[0], q.shape[2], p.seqlen_q_rounded), dtype=torch.float32,
                                    device=q.device)
    rc = N.lib().b200_flash_attn_bwd(_dt(q), dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                     out.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                     dv.data_ptr(), d_softmax_sum.data_ptr(), None, C.byref(p), _stream())
    N.check(rc, "b200_flash_attn_bwd")
    return dq, dk, dv


def kvcache_params(q, kcache, vcache, knew, vnew, out, softmax_scale, causal=True, window=(-1, -1)):
    """The packed arguments of run_flash_attn_kvcache for tensors laid out [B, S, H, D]."""
    p = N.FlashKvCacheParams()
    for name, t in (("q", q), ("k", kcache), ("v", vcache), ("knew", knew), ("vnew", vnew), ("o", out)):
        bs, rs, hs = (t.stride(0), t.stride(1), t.stride(2)) if t is not None else (0, 0, 0)
        setattr(p, name + "_batch_stride", bs)
        setattr(p, name + "_row_stride", rs)
        setattr(p, name + "_head_stride", hs)
    p.b, p.seqlen_q, p.h, p.d = q.shape
    p.seqlen_k, p.h_k = kcache.shape[1], kcache.shape[2]
    p.seqlen_knew = knew.shape[1] if knew is not None else 0
    p.d_rounded = (p.d + 31) // 32 * 32
    p.seqlen_q_rounded = (p.seqlen_q + 127) // 128 * 128
    p.seqlen_k_rounded = (p.seqlen_k + 127) // 128 * 128
    p.softmax_scale = softmax_scale
    p.window_size_left = window[0]
    p.window_size_right = 0 if causal else window[1]
    return p


def flash_attn_kvcache(q, kcache, vcache, knew=None, vnew=None, seqlens_k=None, softmax_scale=None,
                       causal=True, window=(-1, -1), out=None, lse=None, workspace=None):
    """One decode step: append knew/vnew [B, S_new, H_k, D] to the caches [B, S_max, H_k, D] at row
    seqlens_k[b] (i32 [B]; None = the cache is full and nothing is appended) and attend q [B, Sq, H, D]
    to the rows in use.  The caches are updated in place.  Returns (out, softmax_lse[B, H, Sq])."""
    for t in (q, kcache, vcache, knew, vnew):
        if t is not None and (not t.is_cuda or t.stride(-1) != 1):
            raise ValueError("tensors must be CUDA tensors with a contiguous last dim")
    if seqlens_k is not None and (seqlens_k.dtype != torch.int32 or not seqlens_k.is_contiguous()):
        raise ValueError("seqlens_k must be a contiguous int32 tensor")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((q.shape[0], q.shape[2], q.shape[1]), dtype=torch.float32, device=q.device)
    p = kvcache_params(q, kcache, vcache, knew, vnew, out, softmax_scale, causal, window)
    ptr = lambda t: t.data_ptr() if t is not None else None
    rc = N.lib().b200_flash_attn_kvcache(_dt(q), q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), ptr(knew),
                                         ptr(vnew), ptr(seqlens_k), out.data_ptr(), lse.data_ptr(), C.byref(p),
                                         ptr(workspace), workspace.numel() * workspace.element_size()
                                         if workspace is not None else 0, _stream())
    N.check(rc, "b200_flash_attn_kvcache")
    return out, lse


class ShardedSum:
    """Exchange step of a sum whose reduced axis is sharded over ranks (one kernel over NVLink peer
    memory instead of all-reduce + cast).  `peer_inbox` / `peer_flags`: device addresses per rank of
    memory all ranks can write (e.g. from torch symmetric memory), `counter`: a zeroed device uint32."""

    def __init__(self, rank, world, n, peer_inbox, peer_flags, counter, status=None):
        self.rank, self.world, self.n = rank, world, n
        self._inbox = (C.c_void_p * world)(*peer_inbox)
        self._flags = (C.c_void_p * world)(*peer_flags)
        self._counter, self._status = counter, status

    def __call__(self, partial, out):
        rc = N.lib().b200_sharded_sum_finish(
            _dt(out), partial.data_ptr(), self._inbox, self._flags, self.rank, self.world, self.n,
            self._counter.data_ptr(), out.data_ptr(),
            self._status.data_ptr() if self._status is not None else None, _stream())
        N.check(rc, "b200_sharded_sum_finish")
        return out


class ShardedSumSwitch:
    """The same exchange with the sum taken inside the NVSwitch (multimem.ld_reduce over a multicast
    mapping of symmetric memory).  `own_slots`: this rank's float[2][n] in symmetric memory;
    `multicast_slots`: the multicast address of the same range; `peer_flags`, `counter` as above."""

    def __init__(self, rank, world, n, own_slots, multicast_slots, peer_flags, counter, status=None):
        self.rank, self.world, self.n = rank, world, n
        self._own, self._mc = own_slots, multicast_slots
        self._flags = (C.c_void_p * world)(*peer_flags)
        self._counter, self._status = counter, status

    def __call__(self, partial, out):
        rc = N.lib().b200_sharded_sum_finish_nvls(
            _dt(out), partial.data_ptr(), self._own, self._mc, self._flags, self.rank, self.world, self.n,
            self._counter.data_ptr(), out.data_ptr(),
            self._status.data_ptr() if self._status is not None else None, _stream())
        N.check(rc, "b200_sharded_sum_finish_nvls")
        return out
