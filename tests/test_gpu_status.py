"""Runs after the kernel parity files: no bounded device-side wait may have expired."""
import pytest

pytestmark = pytest.mark.gpu


def test_device_error_flag_is_clear():
    import torch
    from quixicore_metal_b200 import _lib
    torch.cuda.synchronize()
    assert _lib.lib().qx_cuda_device_error() == 0
