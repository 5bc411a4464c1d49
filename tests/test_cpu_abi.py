"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and
its argument validation answers with the contract's status codes before any device is touched."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from quixicore_metal_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from quixicore_metal_b200 import build
        build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(L):
    header = open(os.path.join(ROOT, "include", "quixicore_cuda.h")).read()
    names = sorted(set(re.findall(r"\b(qx_cuda_\w+)\s*\(", header)))
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/quixicore_cuda.h but not exported"
    assert L.qx_cuda_version().startswith(b"quixicore-b200")


def test_format_table(L):
    want = {"q4_0": (32, 18), "q8_0": (32, 34), "q6_K": (256, 210), "mxfp8": (32, 33),
            "nvfp4": (16, 9), "mxfp4": (32, 17)}
    for name, (bk, bb) in want.items():
        a, b = C.c_int(), C.c_int()
        assert L.qx_cuda_format_info(name.encode(), C.byref(a), C.byref(b)) == 1
        assert (a.value, b.value) == (bk, bb)
    assert L.qx_cuda_format_info(b"q5_1", None, None) == 0


def _code(st):
    from quixicore_metal_b200 import _lib
    return _lib.STATUS_NAMES[st.code]


def test_projection_validation_status_codes(L):
    from quixicore_metal_b200 import _lib
    p = 0x1000   # never dereferenced: validation fails first
    f32, bf16 = _lib.DTYPE_F32, _lib.DTYPE_BF16
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q5_1", f32, 0, 0, 0)
    assert _code(st) == "unsupported_format" and b"format must be" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", f32, 3, 0, 0)
    assert _code(st) == "invalid_argument" and b"activation" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 48, 8, b"q4_0", f32, 0, 0, 0)
    assert _code(st) == "invalid_shape"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 0, 64, 8, b"q4_0", f32, 0, 0, 0)
    assert _code(st) == "invalid_shape"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", _lib.DTYPE_I32, 0, 0, 0)
    assert _code(st) == "unsupported_dtype"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 1, 0)
    assert _code(st) == "invalid_argument" and b"bias" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, None, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0)
    assert _code(st) == "invalid_argument"
    st = L.qx_cuda_decode_swiglu(None, p, p, None, None, None, p, 1, 64, 8, b"q4_0", bf16, 0)
    assert _code(st) == "invalid_argument" and b"identical shapes" in st.detail
    st = L.qx_cuda_decode_swiglu(None, p, p, p, p, None, p, 1, 64, 8, b"q4_0", bf16, 1)
    assert _code(st) == "invalid_argument" and b"biases" in st.detail
    st = L.qx_cuda_quantize_mxfp8_rows(None, p, p, 4, 48, bf16)
    assert _code(st) == "invalid_shape"
    st = L.qx_cuda_quantize_per_token(None, p, p, p, 4, 48, bf16, 2)
    assert _code(st) == "invalid_argument"


def test_lm_head_validation_status_codes(L):
    from quixicore_metal_b200 import _lib
    p, bf16 = 0x1000, _lib.DTYPE_BF16

    def call(T=2, V=512, K=64, fmt=b"q8_0", mode=0, k=0, temp=1.0, top_p=0.9, ws=p, ws_bytes=1 << 30):
        return L.qx_cuda_lm_head_sample_q(None, p, p, None, p, ws, ws_bytes, T, V, K, fmt, bf16, mode, k, temp, 0, top_p)
    assert _code(call(mode=4)) == "invalid_argument"
    assert _code(call(temp=0.0)) == "invalid_argument"
    assert _code(call(fmt=b"q2_K")) == "unsupported_format"
    assert _code(call(K=48)) == "invalid_shape"
    assert _code(call(mode=2, k=65)) == "invalid_argument"
    assert _code(call(mode=2, k=0)) == "invalid_argument"
    assert _code(call(mode=2, k=40, V=32)) == "invalid_argument"
    assert _code(call(mode=3, k=8, top_p=0.0)) == "invalid_argument"
    assert _code(call(mode=3, k=8, ws_bytes=16)) == "insufficient_workspace"
    need = L.qx_cuda_lm_head_workspace_bytes(64, 128256, 3, 32)
    assert need == 2 * 64 * 501 * 32 * 4 + 64 * 501 * 4 + 0 or need >= 2 * 64 * 501 * 32 * 4
    st = L.qx_cuda_lm_head_shard_partials_q(None, p, p, None, p, p, p, p, 1 << 30, 2, 512, 64, 100, 2, b"q8_0", bf16, 0, 0, 1.0, 0)
    assert _code(st) == "invalid_argument" and b"multiple of 256" in st.detail
    st = L.qx_cuda_lm_head_shard_partials_q(None, p, p, None, p, p, p, p, 1 << 30, 2, 512, 64, 256, 1, b"q8_0", bf16, 0, 0, 1.0, 0)
    assert _code(st) == "invalid_argument" and b"max_tiles" in st.detail
    st = L.qx_cuda_lm_head_sample_q_noalloc(None, p, p, None, p, 64, 128256, 4096, b"q8_0", bf16, 3, 32, 0.8, 1, 0.9)
    assert _code(st) == "insufficient_workspace"


def test_generic_dispatch_validation(L):
    from quixicore_metal_b200 import capi
    st = L.qx_cuda_dispatch(None, None)
    assert _code(st) == "invalid_argument"
    empty = capi.KernelCallStruct()
    st = L.qx_cuda_dispatch(b"flash_attention", C.byref(empty))
    assert _code(st) == "not_implemented" and st.operation == b"flash_attention"
    st = L.qx_cuda_dispatch(b"decode_linear_epilogue", C.byref(empty))
    assert _code(st) == "invalid_argument"
    assert L.qx_cuda_workspace_bytes(b"decode_swiglu", C.byref(empty)) == 0


def test_no_cpu_fallback_without_a_device(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from quixicore_metal_b200 import _lib
    p = 0x1000
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", _lib.DTYPE_BF16, 0, 0, 0)
    assert _code(st) == "runtime_error" and b"no CPU fallback" in st.detail
    x = torch.zeros(1, 64)
    w = torch.zeros(8, 2, 18, dtype=torch.uint8)
    from quixicore_metal_b200 import tk
    with pytest.raises(RuntimeError, match="x must be non-empty"):
        tk.decode_linear_epilogue(x, w, format="q4_0")        # CPU tensors are refused, not emulated


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from quixicore_metal_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.lib()
