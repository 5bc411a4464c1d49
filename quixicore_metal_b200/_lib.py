"""ctypes loader for libquixicore_cuda.so.  Fails loudly: there is no Python or CPU fallback."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libquixicore_cuda.so")

# qx_dtype values of include/quixicore_cuda.h
DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 10, 11, 12
DTYPE_U8, DTYPE_I32 = 3, 6
OUT_QUANT = {None: 0, "fp8": 1, "int8": 2, "mxfp8": 3}

STATUS_NAMES = ["ok", "invalid_argument", "invalid_shape", "unsupported_dtype", "unsupported_format",
                "unsupported_layout", "insufficient_workspace", "adapter_not_wired",
                "not_implemented", "runtime_error"]


class Status(C.Structure):
    # kernel_abi.hpp:22-26: a one-byte status code, then two pointers (24 bytes)
    _fields_ = [("code", C.c_uint8), ("operation", C.c_char_p), ("detail", C.c_char_p)]


class BaseQPlanes(C.Structure):
    # qx_base_q_planes: device pointers of the code / scale / bias planes
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p)]


class BaseQDescriptor(C.Structure):
    # qx_base_q_desc
    _fields_ = [("bits", C.c_int32), ("group_size", C.c_int32), ("scale_dtype", C.c_char_p),
                ("symmetric", C.c_int32), ("layout", C.c_char_p)]


class QxError(RuntimeError):
    """A non-ok qx_status; `.code` is the status name of the contract ABI."""

    def __init__(self, st: Status):
        self.code = STATUS_NAMES[st.code] if 0 <= st.code < len(STATUS_NAMES) else str(st.code)
        op = (st.operation or b"").decode()
        detail = (st.detail or b"").decode()
        super().__init__(f"{op}: {detail}")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m quixicore_metal_b200.build` "
            "(needs nvcc). This backend has no fallback path.")
    L = C.CDLL(LIB_PATH)
    vp, i64, i32, u32, f64, sz = C.c_void_p, C.c_int64, C.c_int, C.c_uint32, C.c_double, C.c_size_t
    cs = C.c_char_p
    L.qx_cuda_decode_linear_epilogue.restype = Status
    L.qx_cuda_decode_linear_epilogue.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, cs, i32, i32, i32, i32,
                                                 i32, vp, vp, vp, sz]
    L.qx_cuda_decode_linear_partial.restype = Status
    L.qx_cuda_decode_linear_partial.argtypes = [vp, vp, vp, vp, i64, i64, i64, cs, i32, vp, sz]
    L.qx_cuda_decode_swiglu.restype = Status
    L.qx_cuda_decode_swiglu.argtypes = [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, cs, i32, i32, i32, vp, vp, vp, sz]
    L.qx_cuda_projection_workspace_bytes.restype = sz
    L.qx_cuda_projection_workspace_bytes.argtypes = [i64, i64, i64, cs, i32, i32]
    L.qx_cuda_quantize_per_token.restype = Status
    L.qx_cuda_quantize_per_token.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32]
    L.qx_cuda_quantize_mxfp8_rows.restype = Status
    L.qx_cuda_quantize_mxfp8_rows.argtypes = [vp, vp, vp, i64, i64, i32]
    L.qx_cuda_lm_head_workspace_bytes.restype = sz
    L.qx_cuda_lm_head_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    L.qx_cuda_lm_head_sample_q.restype = Status
    L.qx_cuda_lm_head_sample_q.argtypes = [vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, cs, i32, i32, i32, f64, u32, f64]
    L.qx_cuda_lm_head_sample_q_noalloc.restype = Status
    L.qx_cuda_lm_head_sample_q_noalloc.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, cs, i32, i32, i32, f64, u32, f64]
    L.qx_cuda_lm_head_dense_workspace_bytes.restype = sz
    L.qx_cuda_lm_head_dense_workspace_bytes.argtypes = [i64, i64, i32, i32]
    L.qx_cuda_lm_head_sample_dense.restype = Status
    L.qx_cuda_lm_head_sample_dense.argtypes = [vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, i32, i32, i32, f64, u32]
    L.qx_cuda_sample_logits.restype = Status
    L.qx_cuda_sample_logits.argtypes = [vp, vp, vp, i64, i64, i32, i32, i32, f64, f64, u32]
    L.qx_cuda_rms_norm_add.restype = Status
    L.qx_cuda_rms_norm_add.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, f64, i32, f64, i32, i32]
    L.qx_cuda_silu_mul_quant.restype = Status
    L.qx_cuda_silu_mul_quant.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, i32, f64, f64, i32, i32, i32]
    L.qx_cuda_qgemm_workspace_bytes.restype = sz
    L.qx_cuda_qgemm_workspace_bytes.argtypes = [i64, i64, i64, cs, i32]
    L.qx_cuda_qgemm.restype = Status
    L.qx_cuda_qgemm.argtypes = [vp, vp, vp, vp, i64, i64, i64, cs, i32, vp, sz]
    L.qx_cuda_quantized_embedding.restype = Status
    L.qx_cuda_quantized_embedding.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, cs, f64, i32, i32]
    pp = C.POINTER(BaseQPlanes)
    dp = C.POINTER(BaseQDescriptor)
    L.qx_cuda_base_q_workspace_bytes.restype = sz
    L.qx_cuda_base_q_workspace_bytes.argtypes = [i64, i64, i64, i32]
    L.qx_cuda_base_qdequant.restype = Status
    L.qx_cuda_base_qdequant.argtypes = [vp, pp, dp, vp, i64, i64, i32]
    L.qx_cuda_base_qembedding.restype = Status
    L.qx_cuda_base_qembedding.argtypes = [vp, pp, dp, vp, vp, i64, i64, i64, i32]
    L.qx_cuda_base_qgemm.restype = Status
    L.qx_cuda_base_qgemm.argtypes = [vp, pp, dp, vp, vp, i64, i64, i64, i32, vp, sz]
    L.qx_cuda_base_qgemv_qkv.restype = Status
    L.qx_cuda_base_qgemv_qkv.argtypes = [vp, pp, pp, pp, dp, vp, vp, vp, vp, i64, i64, i64, i64, i32, vp, sz]
    L.qx_cuda_base_qgemv_swiglu.restype = Status
    L.qx_cuda_base_qgemv_swiglu.argtypes = [vp, pp, pp, dp, vp, vp, i64, i64, i32, vp, sz]
    L.qx_cuda_base_qlm_head_argmax.restype = Status
    L.qx_cuda_base_qlm_head_argmax.argtypes = [vp, pp, dp, vp, vp, i64, i64, i64, i32, vp, sz]
    L.qx_cuda_base_qmoe.restype = Status
    L.qx_cuda_base_qmoe.argtypes = [vp, pp, dp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz]
    L.qx_cuda_peer_push.restype = Status
    L.qx_cuda_peer_push.argtypes = [vp, vp, sz, C.POINTER(vp), C.POINTER(vp), i32, i32, i32, vp]
    L.qx_cuda_lm_head_sample_sharded.restype = Status
    L.qx_cuda_lm_head_sample_sharded.argtypes = [vp, vp, vp, vp, vp, vp, i64, C.POINTER(vp), C.POINTER(vp), vp, vp,
                                                 C.POINTER(vp), vp,
                                                 i32, i32, i32, i32, vp, sz, i64, i64, i64, i64, i64, cs, i32,
                                                 i32, i32, f64, u32, f64]
    L.qx_cuda_peer_gather.restype = Status
    L.qx_cuda_peer_gather.argtypes = [vp, vp, i64, C.POINTER(vp), i32, i32, i32, i32, vp]
    L.qx_cuda_peer_gather_local.restype = Status
    L.qx_cuda_peer_gather_local.argtypes = [vp, C.POINTER(vp), i64, C.POINTER(vp), i32, i32, i32, C.POINTER(vp)]
    L.qx_cuda_peer_allreduce.restype = Status
    L.qx_cuda_peer_allreduce.argtypes = [vp, vp, vp, vp, i64, C.POINTER(vp), i32, i32, vp, vp, vp, i32, i32]
    L.qx_cuda_peer_allreduce_local.restype = Status
    L.qx_cuda_peer_allreduce_local.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), i64, C.POINTER(vp), i32,
                                               C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), i32, i32]
    L.qx_cuda_peer_wait.restype = Status
    L.qx_cuda_peer_wait.argtypes = [vp, vp, i32, i32, i32, i32, vp]
    L.qx_cuda_lm_head_masked_workspace_bytes.restype = sz
    L.qx_cuda_lm_head_masked_workspace_bytes.argtypes = [i64, i64, i64, i32]
    L.qx_cuda_lm_head_masked.restype = Status
    L.qx_cuda_lm_head_masked.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, cs, i32, i32, i32]
    L.qx_cuda_lm_head_candidates.restype = Status
    L.qx_cuda_lm_head_candidates.argtypes = [vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, sz, i64, i64, i64, cs, i32, i32]
    L.qx_cuda_lm_head_beam_workspace_bytes.restype = sz
    L.qx_cuda_lm_head_beam_workspace_bytes.argtypes = [i64, i64, i64, i32]
    L.qx_cuda_lm_head_beam_advance.restype = Status
    L.qx_cuda_lm_head_beam_advance.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i32, i64, i64, cs, i32]
    L.qx_cuda_lm_head_shard_candidates.restype = i64
    L.qx_cuda_lm_head_shard_candidates.argtypes = [i32, i32, i64]
    L.qx_cuda_lm_head_shard_workspace_bytes.restype = sz
    L.qx_cuda_lm_head_shard_workspace_bytes.argtypes = [i64, i64, i64, i32, i32]
    L.qx_cuda_lm_head_shard_partials_q.restype = Status
    L.qx_cuda_lm_head_shard_partials_q.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i64, i64, i64, cs, i32, i32, i32, f64, u32]
    L.qx_cuda_lm_head_shard_reduce.restype = Status
    L.qx_cuda_lm_head_shard_reduce.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, f64, u32, f64]
    L.qx_cuda_format_info.restype = i32
    L.qx_cuda_format_info.argtypes = [cs, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.qx_cuda_launch_count.restype = C.c_uint64
    L.qx_cuda_launch_count.argtypes = []
    L.qx_cuda_device_error.restype = i32
    L.qx_cuda_device_error.argtypes = []
    L.qx_cuda_set_option.restype = i32
    L.qx_cuda_set_option.argtypes = [cs, i32]
    L.qx_cuda_scratch_alloc_count.restype = C.c_uint64
    L.qx_cuda_scratch_alloc_count.argtypes = []
    L.qx_cuda_version.restype = cs
    L.qx_cuda_version.argtypes = []
    L.qx_cuda_dispatch.restype = Status
    L.qx_cuda_dispatch.argtypes = [cs, vp]
    L.qx_cuda_workspace_bytes.restype = sz
    L.qx_cuda_workspace_bytes.argtypes = [cs, vp]
    _lib = L
    return L


def check(st: Status) -> None:
    if st.code != 0:
        raise QxError(st)


def set_option(name: str, value: int) -> None:
    """Chooses between equivalent device paths (see qx_cuda_set_option in the header)."""
    if not lib().qx_cuda_set_option(name.encode(), int(value)):
        raise ValueError(f"unknown option or value: {name}={value}")


def launch_count() -> int:
    return int(lib().qx_cuda_launch_count())
