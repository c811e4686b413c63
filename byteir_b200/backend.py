"""BRTBackend: the class the reference's users and its numerical tests drive the runtime with
(runtime/python/brt/backend.py:14-141) - load a ByRE module, then run(inputs) -> outputs or
profile(inputs) -> (outputs, ms per run).  The session takes its device memory from torch's caching
allocator and runs on torch's current stream, as the reference's class does."""
import time

import torch

from . import brt

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f64": torch.float64,
               "i64": torch.int64, "i32": torch.int32, "i16": torch.int16, "i8": torch.int8, "ui8": torch.uint8,
               "i1": torch.bool}


class BRTBackend:
    def __init__(self, device, byre_file_path):
        device = device.lower()
        if device == "cuda":
            from torch.cuda.memory import caching_allocator_alloc, caching_allocator_delete
            self.session = brt.Session("cuda", alloc_func=caching_allocator_alloc, free_func=caching_allocator_delete)
            stream = torch.cuda.current_stream().cuda_stream
        else:
            self.session = brt.Session("cpu")
            stream = None
        self.session.load(byre_file_path)
        self.req = self.session.new_request_context(stream)
        self.device = device
        # shapes are static: cache them with the element types
        self.input_arg_offsets = self.session.get_input_arg_offsets()
        self.input_shapes = [self.session.get_static_shape(o) for o in self.input_arg_offsets]
        self.input_dtypes = [TORCH_DTYPE[self.session.get_data_type(o)] for o in self.input_arg_offsets]
        self.output_arg_offsets = self.session.get_output_arg_offsets()
        self.output_shapes = [self.session.get_static_shape(o) for o in self.output_arg_offsets]
        self.output_dtypes = [TORCH_DTYPE[self.session.get_data_type(o)] for o in self.output_arg_offsets]

    @staticmethod
    def _check_shape_dtype(tensors, shapes, dtypes):
        assert len(tensors) == len(shapes) == len(dtypes)
        for tensor, shape, dtype in zip(tensors, shapes, dtypes):
            assert list(shape) == list(tensor.shape), (shape, tuple(tensor.shape))
            assert dtype == tensor.dtype, (dtype, tensor.dtype)
            assert tensor.is_contiguous()

    def _new_outputs(self):
        return [torch.empty(shape, dtype=dtype, device=self.device)
                for shape, dtype in zip(self.output_shapes, self.output_dtypes)]

    def _bind(self, inputs, outputs):
        self.req.bind_args([(o, t.data_ptr()) for o, t in zip(self.input_arg_offsets, inputs)])
        self.req.bind_args([(o, t.data_ptr()) for o, t in zip(self.output_arg_offsets, outputs)])
        self.req.finish_io_binding()

    def _time(self, warmup_trials, run_trials):
        for _ in range(warmup_trials):
            self.req.run()
            self.req.sync()
        start = time.time()
        for _ in range(run_trials):
            self.req.run()
            self.req.sync()
        return (time.time() - start) * 1000 / run_trials

    def run(self, inputs, check=True):
        if check:
            self._check_shape_dtype(inputs, self.input_shapes, self.input_dtypes)
        outputs = self._new_outputs()
        self.run_with_outputs(inputs, outputs, check=False)
        return outputs

    def run_with_outputs(self, inputs, outputs, check=True):
        if check:
            self._check_shape_dtype(inputs, self.input_shapes, self.input_dtypes)
            self._check_shape_dtype(outputs, self.output_shapes, self.output_dtypes)
        self._bind(inputs, outputs)
        self.req.run()
        self.req.sync()

    def profile(self, inputs, check=True, warmup_trials=10, run_trials=50):
        if check:
            self._check_shape_dtype(inputs, self.input_shapes, self.input_dtypes)
        outputs = self._new_outputs()
        self._bind(inputs, outputs)
        return outputs, self._time(warmup_trials, run_trials)

    def profile_with_outputs(self, inputs, outputs, check=True, warmup_trials=10, run_trials=50):
        if check:
            self._check_shape_dtype(inputs, self.input_shapes, self.input_dtypes)
            self._check_shape_dtype(outputs, self.output_shapes, self.output_dtypes)
        self._bind(inputs, outputs)
        return self._time(warmup_trials, run_trials)
