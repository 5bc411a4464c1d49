"""quixicore_metal_b200: B200-native (sm_100a) kernels for QuixiCore's quantized decode
projections - `decode_linear_epilogue`, `decode_swiglu`, fused `lm_head_sample` - behind the
reference's operator names.

    from quixicore_metal_b200 import tk          # tk.decode_linear_epilogue(x, Wq, format="q4_0", ...)
    from quixicore_metal_b200 import tk_torch    # the positional binding layer the router calls

The compute lives in csrc/ (hand-written CUDA) behind the C ABI of include/quixicore_cuda.h.
"""
from . import _lib  # noqa: F401

__all__ = ["tk", "tk_torch", "native_loaded", "install_as_tk_torch"]


def native_loaded() -> bool:
    """True once libquixicore_cuda.so is loaded in this process (raises if it cannot be)."""
    _lib.lib()
    return True


def install_as_tk_torch():
    """Registers this package's binding as the top-level module `tk_torch`.

    The reference's router resolves torch tensors with a bare `import tk_torch`
    (bindings/python/tk/__init__.py:25-30).  On a CUDA host there is no MPS build of that module;
    after this call the import yields this backend, so the unmodified reference `tk` serves
    `tk.decode_linear_epilogue / decode_swiglu / lm_head_sample` on CUDA tensors from here.
    Returns the module.  A different `tk_torch` that is already imported is left alone and raises."""
    import importlib
    import sys
    mod = importlib.import_module(f"{__name__}.tk_torch")
    cur = sys.modules.get("tk_torch")
    if cur is not None and cur is not mod:
        raise ImportError("another module named tk_torch is already imported")
    sys.modules["tk_torch"] = mod
    return mod


def __getattr__(name):
    if name in ("tk", "tk_torch", "parallel"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
