"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, and
its argument validation answers with the contract's status codes before any device is touched."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout, when it sits beside this repository (absent on a GPU machine: those checks skip)
_REF_ROOT = os.environ.get("QX_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


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
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q5_1", f32, 0, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "unsupported_format" and b"format must be" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", f32, 3, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_argument" and b"activation" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 48, 8, b"q4_0", f32, 0, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_shape"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 0, 64, 8, b"q4_0", f32, 0, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_shape"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", _lib.DTYPE_I32, 0, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "unsupported_dtype"
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 1, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_argument" and b"bias" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, None, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_argument"
    st = L.qx_cuda_decode_swiglu(None, p, p, None, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, None, None, None, 0)
    assert _code(st) == "invalid_argument" and b"identical shapes" in st.detail
    st = L.qx_cuda_decode_swiglu(None, p, p, p, p, None, p, 1, 64, 8, b"q4_0", bf16, 1, 0, None, None, None, 0)
    assert _code(st) == "invalid_argument" and b"biases" in st.detail
    st = L.qx_cuda_quantize_mxfp8_rows(None, p, p, 4, 48, bf16)
    assert _code(st) == "invalid_shape"
    # output quantisation arguments
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0, 4, p, p, None, 0)
    assert _code(st) == "invalid_argument" and b"output_quant" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0, 1, None, p, None, 0)
    assert _code(st) == "invalid_argument" and b"out_codes" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0, 2, p, None, None, 0)
    assert _code(st) == "invalid_argument" and b"out_scale" in st.detail
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", bf16, 0, 0, 0, 3, p, None, None, 0)
    assert _code(st) == "invalid_shape" and b"multiple of 32" in st.detail
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
    need = L.qx_cuda_lm_head_workspace_bytes(64, 128256, 4096, 3, 32)
    # partials (values, ids, tile lses) + flags + prepared hidden rows + row scales at the least
    assert need >= 2 * 64 * 501 * 32 * 4 + 64 * 501 * 4 + 1024 + 64 * 4096 * 2 + 64 * 4
    assert L.qx_cuda_lm_head_workspace_bytes(0, 128256, 4096, 3, 32) == 0
    st = L.qx_cuda_lm_head_shard_partials_q(None, p, p, None, p, p, p, p, 1 << 30, 2, 512, 64, 100, 2, b"q8_0", bf16, 0, 0, 1.0, 0)
    assert _code(st) == "invalid_argument" and b"multiple of 256" in st.detail
    st = L.qx_cuda_lm_head_shard_partials_q(None, p, p, None, p, p, p, p, 1 << 30, 2, 512, 64, 256, 1, b"q8_0", bf16, 0, 0, 1.0, 0)
    assert _code(st) == "invalid_argument" and b"max_tiles" in st.detail
    st = L.qx_cuda_lm_head_sample_q_noalloc(None, p, p, None, p, 64, 128256, 4096, b"q8_0", bf16, 3, 32, 0.8, 1, 0.9)
    assert _code(st) == "insufficient_workspace"
    # the built-in array also has to hold the prepared hidden rows: a wide K alone exceeds it
    st = L.qx_cuda_lm_head_sample_q_noalloc(None, p, p, None, p, 64, 1024, 65536, b"q8_0", bf16, 0, 0, 0.8, 1, 0.9)
    assert _code(st) == "insufficient_workspace"


def test_peer_exchange_validation_status_codes(L):
    """The peer-store entries refuse bad arguments with the contract's codes before a device is touched."""
    from quixicore_metal_b200 import _lib
    p, bf16 = 0x1000, _lib.DTYPE_BF16
    two = (C.c_void_p * 2)(p, p)

    def allreduce(n=8192, world=2, rank=0, dtype=bf16, timeout=100, src=p, bufs=two):
        return L.qx_cuda_peer_allreduce(None, src, p, p, n, bufs, world, rank, p, p, p, dtype, timeout)
    assert _code(allreduce(src=None)) == "invalid_argument"
    assert _code(allreduce(bufs=None)) == "invalid_argument"
    assert _code(allreduce(world=17)) == "invalid_argument"
    assert _code(allreduce(rank=2)) == "invalid_argument"
    assert _code(allreduce(n=0)) == "invalid_shape"
    assert _code(allreduce(n=7)) == "invalid_shape"
    assert _code(allreduce(dtype=99)) == "unsupported_dtype"
    assert _code(allreduce(timeout=0)) == "invalid_argument"
    assert _code(allreduce(timeout=20000)) == "invalid_argument"

    def gather(slot=64, world=2, rank=0, step=1, timeout=100, buf=p, words=two):
        return L.qx_cuda_peer_gather(None, buf, slot, words, world, rank, step, timeout, p)
    assert _code(gather(buf=None)) == "invalid_argument"
    assert _code(gather(words=None)) == "invalid_argument"
    assert _code(gather(world=0)) == "invalid_argument"
    assert _code(gather(rank=-1)) == "invalid_argument"
    assert _code(gather(slot=0)) == "invalid_shape"
    assert _code(gather(slot=3)) == "invalid_shape"
    assert _code(gather(timeout=0)) == "invalid_argument"
    # the sharded LM-head call checks its slot geometry first
    st = L.qx_cuda_lm_head_sample_sharded(None, p, p, None, p, p, 6, None, None, None, None, None, p, 2, 0, 1, 100, p, 1 << 30,
                                          2, 512, 64, 0, 2, b"q8_0", bf16, 0, 0, 1.0, 0, 0.9)
    assert _code(st) == "invalid_shape" and b"slot_stride" in st.detail
    st = L.qx_cuda_lm_head_sample_sharded(None, p, p, None, p, p, 64, None, None, None, None, None, p, 2, 5, 1, 100, p, 1 << 30,
                                          2, 512, 64, 0, 2, b"q8_0", bf16, 0, 0, 1.0, 0, 0.9)
    assert _code(st) == "invalid_argument"


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


def test_projection_workspace_query(L):
    from quixicore_metal_b200 import _lib
    bf16, f32 = _lib.DTYPE_BF16, _lib.DTYPE_F32
    # batch 1, K = 8192: the prepared f16 activations (16 KB) + row scales, 256-byte granules
    assert L.qx_cuda_projection_workspace_bytes(1, 8192, 28672, b"nvfp4", bf16, 0) == 8192 * 2 + 256
    # fp32 activations take the generic kernel: no scratch
    assert L.qx_cuda_projection_workspace_bytes(1, 8192, 28672, b"nvfp4", f32, 0) == 0
    # 64 rows on the tcgen05 pipeline: one 64-row operand image
    assert L.qx_cuda_projection_workspace_bytes(64, 8192, 28672, b"nvfp4", bf16, 0) >= 64 * 8192 * 2
    assert L.qx_cuda_projection_workspace_bytes(1, 8192, 28672, b"q5_1", bf16, 0) == 0


def test_options(L):
    assert L.qx_cuda_set_option(b"stream_passes", 2) == 1
    assert L.qx_cuda_set_option(b"stream_passes", 1) == 1
    assert L.qx_cuda_set_option(b"stream_passes", 7) == 0
    assert L.qx_cuda_set_option(b"no_such_option", 1) == 0


# ---- layout of the generic call structs against the contract header they stand in for ----------
def test_struct_layout_equals_kernel_abi():
    """Sizes and offsets of include/quixicore/contract/kernel_abi.hpp:22-107 on LP64 (one-byte
    enumerations): the ctypes mirrors must agree with them, field by field."""
    from quixicore_metal_b200 import _lib, capi
    TV, AT, KC, ST = capi.TensorView, capi.Attribute, capi.KernelCallStruct, _lib.Status
    assert C.sizeof(ST) == 24 and ST.code.offset == 0 and ST.code.size == 1
    assert ST.operation.offset == 8 and ST.detail.offset == 16
    assert C.sizeof(TV) == 40
    assert (TV.data.offset, TV.shape.offset, TV.strides.offset, TV.rank.offset) == (0, 8, 16, 24)
    assert (TV.dtype.offset, TV.memory_space.offset, TV.flags.offset) == (32, 33, 36)
    assert C.sizeof(AT) == 48
    assert (AT.name.offset, AT.kind.offset, AT.data.offset, AT.size.offset, AT.i64.offset, AT.f64.offset) == \
        (0, 8, 16, 24, 32, 40) and AT.kind.size == 1
    assert C.sizeof(KC) == 80
    assert [getattr(KC, f).offset for f, _ in KC._fields_] == [0, 8, 16, 24, 32, 40, 48, 56, 64, 72]


_LAYOUT_CHECK = r"""
#include <cstddef>
#include "quixicore_cuda.h"
#ifdef WITH_REFERENCE
#include "quixicore/contract/kernel_abi.hpp"
namespace r = quixicore::contract;
#define SAME(T, U, f) static_assert(offsetof(T, f) == offsetof(U, f), #f)
static_assert(sizeof(qx_status) == sizeof(r::Status), "Status");
SAME(qx_status, r::Status, code); SAME(qx_status, r::Status, operation); SAME(qx_status, r::Status, detail);
static_assert(sizeof(qx_tensor_view) == sizeof(r::TensorView), "TensorView");
SAME(qx_tensor_view, r::TensorView, data); SAME(qx_tensor_view, r::TensorView, shape);
SAME(qx_tensor_view, r::TensorView, strides); SAME(qx_tensor_view, r::TensorView, rank);
SAME(qx_tensor_view, r::TensorView, dtype); SAME(qx_tensor_view, r::TensorView, memory_space);
SAME(qx_tensor_view, r::TensorView, flags);
static_assert(sizeof(qx_attribute) == sizeof(r::Attribute), "Attribute");
SAME(qx_attribute, r::Attribute, name); SAME(qx_attribute, r::Attribute, kind); SAME(qx_attribute, r::Attribute, data);
SAME(qx_attribute, r::Attribute, size); SAME(qx_attribute, r::Attribute, i64); SAME(qx_attribute, r::Attribute, f64);
static_assert(sizeof(qx_kernel_call) == sizeof(r::KernelCall), "KernelCall");
SAME(qx_kernel_call, r::KernelCall, inputs); SAME(qx_kernel_call, r::KernelCall, outputs);
SAME(qx_kernel_call, r::KernelCall, attributes); SAME(qx_kernel_call, r::KernelCall, backend_context);
SAME(qx_kernel_call, r::KernelCall, stream); SAME(qx_kernel_call, r::KernelCall, workspace);
SAME(qx_kernel_call, r::KernelCall, workspace_size);
static_assert((int)QX_RUNTIME_ERROR == (int)r::StatusCode::runtime_error, "status codes");
static_assert((int)QX_DTYPE_PACKED == (int)r::DType::packed && (int)QX_DTYPE_BF16 == (int)r::DType::bf16, "dtypes");
static_assert((int)QX_MEMORY_SHARED == (int)r::MemorySpace::shared, "memory spaces");
static_assert((int)QX_ATTR_BYTES == (int)r::AttributeKind::bytes, "attribute kinds");
static_assert((int)QX_TENSOR_OPTIONAL == (int)r::tensor_optional, "tensor flags");
#endif
static_assert(sizeof(qx_status) == 24 && offsetof(qx_status, operation) == 8, "qx_status");
static_assert(sizeof(qx_tensor_view) == 40 && offsetof(qx_tensor_view, dtype) == 32 &&
              offsetof(qx_tensor_view, memory_space) == 33 && offsetof(qx_tensor_view, flags) == 36, "qx_tensor_view");
static_assert(sizeof(qx_attribute) == 48 && offsetof(qx_attribute, data) == 16, "qx_attribute");
static_assert(sizeof(qx_kernel_call) == 80, "qx_kernel_call");
int main() { return 0; }
"""


def test_header_layout_static_asserts(tmp_path):
    """Compiles the C header with static_asserts on its own layout and, when the reference checkout
    is on this machine, beside the contract header it mirrors."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++")
    src = tmp_path / "layout.cpp"
    src.write_text(_LAYOUT_CHECK)
    ref_inc = os.path.join(_REF_ROOT, "include")
    cmd = [gxx, "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)]
    if os.path.exists(os.path.join(ref_inc, "quixicore", "contract", "kernel_abi.hpp")):
        cmd += ["-DWITH_REFERENCE", "-I", ref_inc]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    # and as plain C
    csrc = tmp_path / "layout.c"
    csrc.write_text('#include "quixicore_cuda.h"\nint main(void) { return (int)sizeof(qx_kernel_call) - 80; }\n')
    gcc = shutil.which("gcc")
    p = subprocess.run([gcc, "-std=c11", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(csrc)],
                       capture_output=True, text=True)
    assert p.returncode == 0, p.stderr


# ---- the Python binding against the reference module it replaces --------------------------------
_REF_TK_TORCH = os.path.join(_REF_ROOT, "bindings", "pytorch_mps", "tk_torch", "__init__.py")
# (name, positional parameters with defaults) of bindings/pytorch_mps/tk_torch/__init__.py:932-958,
# :1620-1637, :1738-1745, kept here so the check also runs where the reference checkout is absent
_BQ_TAIL = ["bits", "group_size", "scale_dtype='bf16'", "symmetric=False", "layout='metal'"]
_SIGNATURES = {
    "decode_linear_epilogue": ["x", "weight", "bias", "residual", "format=''", "activation=0",
                               "use_bias=False", "use_residual=False"],
    "decode_swiglu": ["x", "gate_weight", "up_weight", "gate_bias", "up_bias", "format=''", "use_bias=False"],
    "lm_head_sample": ["h", "W", "bias", "mode", "k", "temperature", "seed"],
    "lm_head_sample_q": ["h", "Wq", "bias", "V", "K", "fmt", "mode", "topk", "temperature", "seed", "top_p=0.0"],
    "lm_head_beam_advance": ["h", "Wq", "bias", "cum_log_probs", "beam_width", "fmt='q4_0'"],
    "lm_head_masked": ["h", "W", "bias", "allow_mask", "format=''", "topk=1", "normalize_allowed=True"],
    "lm_head_candidates": ["h", "W", "bias", "candidate_ids", "offsets", "format=''", "topk=1"],
    "qgemm": ["wq", "x", "format='q8_0'"],
    "qgemv": ["wq", "x", "format='q8_0'"],
    "dequant_gather": ["table", "ids", "format", "scale=1.0"],
    "quantized_embedding": ["table", "ids", "add", "format", "scale=1.0", "use_add=False", "output_dtype='float16'"],
    "rms_norm_add": ["x", "residual", "weight", "eps=1e-05"],
    "rms_norm_add_fp8": ["x", "residual", "weight", "eps=1e-05", "scale=None"],
    "rms_norm_add_per_block": ["x", "residual", "weight", "eps=1e-05", "int8=False", "ue8m0=False"],
    "silu_mul_quant_fp8": ["x", "gate", "act='swiglu'", "alpha=1.702", "limit=7.0"],
    "silu_mul_quant_int8": ["x", "gate", "act='swiglu'", "alpha=1.702", "limit=7.0"],
    "silu_mul_quant_fp8_group": ["x", "gate", "group_size=128", "ue8m0=False", "act='swiglu'", "alpha=1.702", "limit=7.0"],
    "quantize_per_token_fp8": ["x"],
    "quantize_per_token_int8": ["x"],
    "argmax_sample": ["logits"],
    "sample_categorical": ["logits", "temperature=1.0", "seed=0"],
    "top_k_sample": ["logits", "k", "temperature=1.0", "seed=0"],
    "top_p_sample": ["logits", "p", "temperature=1.0", "seed=0"],
    "base_qdequant": ["codes", "scales", "biases", *_BQ_TAIL, "output_dtype='float16'"],
    "base_qembedding": ["codes", "scales", "biases", "ids", *_BQ_TAIL, "output_dtype='float16'"],
    "base_qgemv": ["codes", "scales", "biases", "x", *_BQ_TAIL],
    "base_qgemm": ["codes", "scales", "biases", "x", *_BQ_TAIL],
    "base_qgemv_qkv": ["q_codes", "q_scales", "q_biases", "k_codes", "k_scales", "k_biases", "v_codes", "v_scales",
                       "v_biases", "x", *_BQ_TAIL],
    "base_qgemv_swiglu": ["gate_codes", "gate_scales", "gate_biases", "up_codes", "up_scales", "up_biases", "x",
                          *_BQ_TAIL],
    "base_qlm_head_argmax": ["codes", "scales", "biases", "x", *_BQ_TAIL],
    "base_qmoe_gemm": ["codes", "scales", "biases", "input", "expert_of_tile", *_BQ_TAIL],
    "base_qmoe_swiglu": ["codes", "scales", "biases", "input", "expert_of_tile", *_BQ_TAIL],
}


def _positional_signature(fn_node):
    import ast
    a = fn_node.args
    names = [x.arg for x in a.args]
    defaults = [None] * (len(names) - len(a.defaults)) + [ast.literal_eval(d) for d in a.defaults]
    return [n if d is None and i < len(names) - len(a.defaults) else f"{n}={d!r}"
            for i, (n, d) in enumerate(zip(names, defaults))]


def _module_signatures(path):
    import ast
    tree = ast.parse(open(path).read())
    return {n.name: _positional_signature(n) for n in tree.body
            if isinstance(n, ast.FunctionDef) and n.name in _SIGNATURES}


def test_tk_torch_signatures_equal_the_reference_module():
    """Same names, positional parameters and defaults as the reference's PyTorch binding, so its
    router can call this module unchanged (keyword-only additions here do not disturb that)."""
    ours = _module_signatures(os.path.join(ROOT, "quixicore_metal_b200", "tk_torch.py"))
    for name, want in _SIGNATURES.items():
        assert name in ours, f"tk_torch.{name} is missing"
        assert ours[name] == want, (name, ours[name], want)
    if os.path.exists(_REF_TK_TORCH):
        ref = _module_signatures(_REF_TK_TORCH)
        for name, want in _SIGNATURES.items():
            assert ref[name] == want, ("the pinned signature table is out of date", name, ref[name])


def test_install_routes_the_reference_router_here():
    """After install_as_tk_torch() an `import tk_torch` - what the reference's router does for torch
    tensors (bindings/python/tk/__init__.py:25-30) - yields this backend."""
    import sys
    import quixicore_metal_b200 as q
    saved = sys.modules.pop("tk_torch", None)
    try:
        q.install_as_tk_torch()
        import tk_torch
        assert tk_torch is q.tk_torch
        ref_py = os.path.join(_REF_ROOT, "bindings", "python")
        if os.path.exists(os.path.join(ref_py, "tk", "__init__.py")):
            sys.path.insert(0, ref_py)
            try:
                saved_tk = sys.modules.pop("tk", None)
                import tk as ref_tk
                assert ref_tk._torch() is q.tk_torch
            finally:
                sys.path.remove(ref_py)
                sys.modules.pop("tk", None)
                if saved_tk is not None:
                    sys.modules["tk"] = saved_tk
    finally:
        sys.modules.pop("tk_torch", None)
        if saved is not None:
            sys.modules["tk_torch"] = saved


def test_tensors_on_different_devices_are_refused():
    """The device check runs before anything touches a pointer; two stand-in devices are enough."""
    from quixicore_metal_b200 import tk_torch

    class FakeTensor:
        def __init__(self, index):
            self.device = ("cuda", index)

    a, b = FakeTensor(0), FakeTensor(1)
    tk_torch._same_device("decode_linear_epilogue", a, FakeTensor(0), None)
    with pytest.raises(RuntimeError, match="same device"):
        tk_torch._same_device("decode_linear_epilogue", a, FakeTensor(0), b)
    with pytest.raises(RuntimeError, match="same device"):
        tk_torch._same_device("lm_head_sample_q", a, b)


def test_no_cpu_fallback_without_a_device(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from quixicore_metal_b200 import _lib
    p = 0x1000
    st = L.qx_cuda_decode_linear_epilogue(None, p, p, None, None, p, 1, 64, 8, b"q4_0", _lib.DTYPE_BF16, 0, 0, 0, 0, None, None, None, 0)
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
