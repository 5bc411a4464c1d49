"""ctypes mirror of the generic call structs of include/quixicore_cuda.h (qx_tensor_view,
qx_attribute, qx_kernel_call) and a builder that fills them from torch CUDA tensors, for callers
that want the contract-style `qx_cuda_dispatch(op_name, call)` door instead of the typed entries.
The layouts equal include/quixicore/contract/kernel_abi.hpp:66-107 of the reference (one-byte
enumerations): TensorView 40 bytes, Attribute 48, KernelCall 80."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_DTYPE = {torch.bool: 1, torch.int8: 2, torch.uint8: 3, torch.int16: 4, torch.int32: 6,
          torch.int64: 8, torch.float16: 10, torch.bfloat16: 11, torch.float32: 12,
          torch.float64: 13}
MEMORY_DEVICE = 2
ATTR_BOOL, ATTR_I64, ATTR_F64, ATTR_STRING, ATTR_BYTES = range(5)


class TensorView(C.Structure):
    _fields_ = [("data", C.c_void_p), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("rank", C.c_size_t), ("dtype", C.c_uint8),
                ("memory_space", C.c_uint8), ("flags", C.c_uint32)]


class Attribute(C.Structure):
    _fields_ = [("name", C.c_char_p), ("kind", C.c_uint8), ("data", C.c_void_p),
                ("size", C.c_size_t), ("i64", C.c_int64), ("f64", C.c_double)]


class KernelCallStruct(C.Structure):
    _fields_ = [("inputs", C.POINTER(TensorView)), ("input_count", C.c_size_t),
                ("outputs", C.POINTER(TensorView)), ("output_count", C.c_size_t),
                ("attributes", C.POINTER(Attribute)), ("attribute_count", C.c_size_t),
                ("backend_context", C.c_void_p), ("stream", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_size", C.c_size_t)]


class KernelCall:
    """Owns the ctypes storage of one qx_kernel_call built from torch tensors.
    `inputs` may contain None for an absent optional tensor."""

    def __init__(self, inputs, outputs, attrs=None, stream=None):
        self._keep = []
        self._in = (TensorView * max(len(inputs), 1))()
        self._out = (TensorView * max(len(outputs), 1))()
        for i, t in enumerate(inputs):
            self._fill(self._in[i], t)
        for i, t in enumerate(outputs):
            self._fill(self._out[i], t)
        attrs = attrs or {}
        self._attr = (Attribute * max(len(attrs), 1))()
        for i, (k, v) in enumerate(attrs.items()):
            a = self._attr[i]
            a.name = k.encode()
            if isinstance(v, bool):
                a.kind, a.i64 = ATTR_BOOL, int(v)
            elif isinstance(v, int):
                a.kind, a.i64 = ATTR_I64, v
            elif isinstance(v, float):
                a.kind, a.f64 = ATTR_F64, v
            else:
                buf = C.create_string_buffer(str(v).encode())
                self._keep.append(buf)
                a.kind, a.data, a.size = ATTR_STRING, C.cast(buf, C.c_void_p), len(buf) - 1
        s = KernelCallStruct()
        s.inputs, s.input_count = self._in, len(inputs)
        s.outputs, s.output_count = self._out, len(outputs)
        s.attributes, s.attribute_count = self._attr, len(attrs)
        s.backend_context = None
        s.stream = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        s.workspace, s.workspace_size = None, 0
        self.struct = s

    def _fill(self, view: TensorView, t):
        if t is None:
            view.data, view.rank = None, 0
            return
        shape = (C.c_int64 * max(t.dim(), 1))(*t.shape)
        strides = (C.c_int64 * max(t.dim(), 1))(*t.stride())
        self._keep += [shape, strides, t]
        view.data, view.shape, view.strides, view.rank = t.data_ptr(), shape, strides, t.dim()
        view.dtype = _DTYPE.get(t.dtype, 0)
        view.memory_space = MEMORY_DEVICE if t.is_cuda else 1
        view.flags = 2 if t.is_contiguous() else 0

    def set_workspace(self, ws: torch.Tensor):
        self._keep.append(ws)
        self.struct.workspace, self.struct.workspace_size = ws.data_ptr(), ws.numel() * ws.element_size()

    def ref(self):
        return C.cast(C.pointer(self.struct), C.c_void_p)


def dispatch(op_name: str, call: KernelCall) -> None:
    _lib.check(_lib.lib().qx_cuda_dispatch(op_name.encode(), call.ref()))
