"""quixicore_metal_b200: B200-native (sm_100a) kernels for QuixiCore's quantized decode
projections - `decode_linear_epilogue`, `decode_swiglu`, fused `lm_head_sample` - behind the
reference's operator names.

    from quixicore_metal_b200 import tk          # tk.decode_linear_epilogue(x, Wq, format="q4_0", ...)
    from quixicore_metal_b200 import tk_torch    # the positional binding layer the router calls

The compute lives in csrc/ (hand-written CUDA) behind the C ABI of include/quixicore_cuda.h.
"""
from . import _lib  # noqa: F401

__all__ = ["tk", "tk_torch", "native_loaded"]


def native_loaded() -> bool:
    """True once libquixicore_cuda.so is loaded in this process (raises if it cannot be)."""
    _lib.lib()
    return True


def __getattr__(name):
    if name in ("tk", "tk_torch", "parallel"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
