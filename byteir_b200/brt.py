"""Python door onto the brt host runtime (libbrt_b200.so) through its C API
(include/brt_c_api.h).  Usage follows the reference's `brt.Session`
(runtime/python/src/module.cc): create a session for a device, load a ByRE
module, make a request, bind or fetch argument buffers, run, sync.
"""
import ctypes as C
from pathlib import Path

from ._native import LIB_DIR

# brt::DTypeEnum (include/brt/core/framework/dtype.h)
DTYPE_NAMES = {1: "f32", 2: "i32", 3: "i64", 4: "ui8", 5: "ui32", 6: "f16", 7: "bf16", 8: "f64", 9: "i1",
               11: "i8", 12: "i16", 13: "ui16", 14: "ui64"}

_vp, _i64, _int, _sz, _cp = C.c_void_p, C.c_int64, C.c_int, C.c_size_t, C.c_char_p

SIGNATURES = {
    "brt_last_error": (_cp, []),
    "brt_register_kernels_from_dynlib": (_int, [_cp]),
    "brt_session_create": (_vp, []),
    "brt_session_destroy": (None, [_vp]),
    "brt_session_create_distributed": (_vp, [_int, _int]),
    "brt_session_set_allreduce_callback": (_int, [_vp, _vp, _vp]),
    "brt_session_set_allreduce_peer": (_int, [_vp, C.c_uint64, C.POINTER(_vp), C.POINTER(_vp), _vp, _vp]),
    "brt_session_add_cpu": (_int, [_vp]),
    "brt_session_add_cuda": (_int, [_vp, _int]),
    "brt_session_add_cuda_external": (_int, [_vp, _int, _vp, _vp]),
    "brt_session_load": (_int, [_vp, _cp]),
    "brt_session_load_from_memory": (_int, [_vp, _cp]),
    "brt_session_load_buffer": (_int, [_vp, _cp, _sz]),
    "brt_session_arg_num": (_i64, [_vp]),
    "brt_session_arg_offset": (_int, [_vp, _cp]),
    "brt_session_arg_info": (_int, [_vp, _i64, C.POINTER(_int), C.POINTER(_int), C.POINTER(_i64), _cp, _sz,
                                    C.POINTER(_int), _cp, _sz]),
    "brt_request_create": (_vp, [_vp, _vp]),
    "brt_request_destroy": (None, [_vp]),
    "brt_request_bind_arg": (_int, [_vp, _i64, _vp]),
    "brt_request_get_arg": (_vp, [_vp, _i64]),
    "brt_request_finish_io_binding": (_int, [_vp]),
    "brt_session_run": (_int, [_vp, _vp]),
    "brt_request_sync": (_int, [_vp]),
    "brt_request_enable_op_trace": (_int, [_vp]),
    "brt_request_op_trace": (_i64, [_vp, _cp, _sz]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = LIB_DIR / "libbrt_b200.so"
        if not path.exists():
            raise ImportError(f"{path} is missing: build it with `python -m byteir_b200.build`")
        h = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


class BrtError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise BrtError(lib().brt_last_error().decode(errors="replace"))


def register_kernels_from_dynlib(path):
    _check(lib().brt_register_kernels_from_dynlib(str(path).encode()))


class ArgInfo:
    def __init__(self, offset, name, dtype, shape, space, argtype):
        self.offset, self.name, self.dtype, self.shape, self.space, self.argtype = offset, name, dtype, shape, space, argtype

    @property
    def nbytes(self):
        n = {"f32": 4, "i32": 4, "ui32": 4, "i64": 8, "ui64": 8, "f64": 8, "f16": 2, "bf16": 2, "i16": 2,
             "ui16": 2, "i8": 1, "ui8": 1, "i1": 1}[self.dtype]
        for s in self.shape:
            n *= s
        return n

    def __repr__(self):
        return f"ArgInfo({self.offset}, {self.name!r}, {self.dtype}, {self.shape}, {self.space!r}, type={self.argtype})"


_ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_size_t)
_FREE_FN = C.CFUNCTYPE(None, C.c_void_p)


class Session:
    """device: "cuda" (default CUDA provider + CUDA allocators) or "cpu" (any case, as the reference's
    binding takes "CUDA" / "CPU"); host_space=True adds the CPU allocator and provider to a CUDA session,
    for modules with memrefs in the "cpu" space (cpu2cuda / cuda2cpu copies).  alloc_func(size) -> address
    and free_func(address) make the session take its device memory (unbound arguments, intermediates,
    weights) from the caller, e.g. torch.cuda.caching_allocator_alloc / caching_allocator_delete, as the
    reference's Session(device, alloc_func, free_func) does (runtime/python/src/module.cc:340-376)."""

    def __init__(self, device="cuda", device_id=0, host_space=False, alloc_func=None, free_func=None):
        device = device.lower()
        self._h = self._create()
        if not self._h:
            raise BrtError(lib().brt_last_error().decode())
        if (alloc_func is None) != (free_func is None):
            raise ValueError("alloc_func and free_func come together")
        if device == "cuda":
            if alloc_func is not None:
                # the C side keeps the two function pointers for the session's life: so must Python
                self._alloc = _ALLOC_FN(lambda size: int(alloc_func(size)) or None)
                self._free = _FREE_FN(lambda ptr: free_func(ptr or 0))
                _check(lib().brt_session_add_cuda_external(self._h, device_id, C.cast(self._alloc, C.c_void_p),
                                                           C.cast(self._free, C.c_void_p)))
            else:
                _check(lib().brt_session_add_cuda(self._h, device_id))
            if host_space:
                _check(lib().brt_session_add_cpu(self._h))
        elif device == "cpu":
            _check(lib().brt_session_add_cpu(self._h))
        else:
            raise ValueError(device)

    def _create(self):
        return lib().brt_session_create()

    def close(self):
        if self._h:
            lib().brt_session_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load(self, path):
        _check(lib().brt_session_load(self._h, str(path).encode()))

    def load_from_memory(self, text):
        """ByRE text (str), or ByRE text / bytecode as bytes"""
        if isinstance(text, (bytes, bytearray)):
            _check(lib().brt_session_load_buffer(self._h, bytes(text), len(text)))
        else:
            _check(lib().brt_session_load_from_memory(self._h, text.encode()))

    def arg_num(self):
        return lib().brt_session_arg_num(self._h)

    def arg_offset(self, name):
        return lib().brt_session_arg_offset(self._h, name.encode())

    def arg_info(self, offset):
        dt, rank, at = _int(), _int(), _int()
        shape = (_i64 * 8)()
        space, name = C.create_string_buffer(32), C.create_string_buffer(128)
        _check(lib().brt_session_arg_info(self._h, offset, C.byref(dt), C.byref(rank), shape, space, 32,
                                          C.byref(at), name, 128))
        return ArgInfo(offset, name.value.decode(), DTYPE_NAMES.get(dt.value, str(dt.value)),
                       tuple(shape[i] for i in range(rank.value)), space.value.decode(), at.value)

    def args(self):
        return [self.arg_info(i) for i in range(self.arg_num())]

    def new_request(self, cuda_stream=None):
        return Request(self, cuda_stream)

    # ---- the names of the reference's binding (runtime/python/src/module.cc:377-421)
    new_request_context = new_request

    def get_input_arg_offsets(self):
        return [a.offset for a in self.args() if a.argtype & 1]

    def get_output_arg_offsets(self):
        return [a.offset for a in self.args() if a.argtype & 2]

    def get_weight_arg_offsets(self):
        return [a.offset for a in self.args() if a.argtype & 4]

    def get_static_shape(self, offset):
        return list(self.arg_info(offset).shape)

    def get_data_type(self, offset):
        """the element type's name: "f32", "f16", "bf16", "i64", ..."""
        return self.arg_info(offset).dtype

    def get_input_names(self):
        return [a.name for a in self.args() if a.argtype & 1]

    def get_output_names(self):
        return [a.name for a in self.args() if a.argtype & 2]


REDUCE_OP_NAMES = {0: "sum", 1: "max", 2: "min"}
_ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int, C.c_int,
                            C.POINTER(C.c_int64), C.c_uint64, C.c_void_p)


class DistributedSession(Session):
    """One rank of `nranks` (the reference's DistributedSession, runtime/include/brt/core/distributed/
    distributed_session.h:44-82): every rank loads its own module; `nccl.AllReduce` ops run on the
    communicator given with set_allreduce (a function of this program that runs one all-reduce on the
    process group it created once) or set_allreduce_peer (the one-kernel sum over NVLink peer memory)."""

    def __init__(self, rank, nranks, device="cuda", device_id=None, host_space=False, alloc_func=None, free_func=None):
        self.rank, self.nranks = rank, nranks
        super().__init__(device, rank if device_id is None else device_id, host_space, alloc_func, free_func)

    def _create(self):
        return lib().brt_session_create_distributed(self.rank, self.nranks)

    def load_config(self, config):
        """config[rank] is this rank's module file"""
        self.load(config[self.rank])

    def set_allreduce(self, fn):
        """fn(send, recv, length, dtype, op, group, stream): addresses as int, dtype as "f32" / "f16" / ...,
        op "sum" / "max" / "min", group a list of ranks (empty: all), stream a CUDA stream handle or None for
        host buffers.  It enqueues (device) or completes (host) one all-reduce; an exception fails the run."""
        def thunk(_user, send, recv, length, dtype, op, group, group_len, stream):
            try:
                fn(send, recv, int(length), DTYPE_NAMES.get(dtype, str(dtype)), REDUCE_OP_NAMES.get(op, str(op)),
                   [int(group[i]) for i in range(group_len)], stream)
                return 0
            except Exception as e:  # the C side turns the code into a failed Status
                self.allreduce_error = e
                return 1
        self._allreduce = _ALLREDUCE_FN(thunk)  # kept alive as long as the session
        _check(lib().brt_session_set_allreduce_callback(self._h, C.cast(self._allreduce, C.c_void_p), None))

    def set_allreduce_peer(self, capacity, peer_inbox, peer_flags, epoch_counter, status=None):
        """peer_inbox / peer_flags: device addresses per rank (memory every rank has mapped, zeroed once);
        epoch_counter: address of a zeroed device uint32; status: address of a device int, or None"""
        inbox = (C.c_void_p * self.nranks)(*peer_inbox)
        flags = (C.c_void_p * self.nranks)(*peer_flags)
        _check(lib().brt_session_set_allreduce_peer(self._h, capacity, inbox, flags, epoch_counter, status))


class Request:
    def __init__(self, session, cuda_stream=None):
        self._s = session
        self._h = lib().brt_request_create(session._h, cuda_stream)
        if not self._h:
            raise BrtError(lib().brt_last_error().decode())

    def close(self):
        if self._h:
            lib().brt_request_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def bind_args(self, offset_and_ptr):
        for offset, ptr in offset_and_ptr:
            self.bind_arg(offset, ptr)

    def bind_arg(self, offset, ptr):
        _check(lib().brt_request_bind_arg(self._h, offset, ptr))

    def get_arg(self, offset):
        p = lib().brt_request_get_arg(self._h, offset)
        if not p:
            raise BrtError(lib().brt_last_error().decode())
        return p

    def finish_io_binding(self):
        _check(lib().brt_request_finish_io_binding(self._h))

    def run(self):
        _check(lib().brt_session_run(self._s._h, self._h))

    def sync(self):
        _check(lib().brt_request_sync(self._h))

    def enable_op_trace(self):
        _check(lib().brt_request_enable_op_trace(self._h))

    def op_trace(self):
        n = lib().brt_request_op_trace(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        lib().brt_request_op_trace(self._h, buf, n + 1)
        return [k for k in buf.value.decode().split(";") if k]
