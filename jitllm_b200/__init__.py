"""jitllm_b200 -- B200-native quantized matmul behind jitllm's operator surface.

The product is libjitllm_b200.so (hand-written CUDA for sm_100a, C ABI in
include/jitllm_b200.h). This package is the thin host layer used by the tests,
the benchmark and Python callers: a ctypes binding (`_lib`) and a mirror of the
reference's `nn.Device` operator interface (`device.Device`).
"""
from ._lib import (ACT_SILU, ACT_SWIGLU_OAI, BF16, DECLINED, DT_BF16, DT_F16, DT_F32, F16, F32, K_AUTO,
                   K_MMA, K_SIMT, K_TC5, MXFP4, OK, Q4_0, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, row_bytes)
from .device import Device, DeviceError, Weight

__all__ = ["Device", "DeviceError", "Weight", "Q4_K", "Q8_0", "MXFP4", "Q4_0", "Q5_0", "Q5_1", "Q5_K", "Q6_K", "F32", "F16", "BF16", "row_bytes",
           "K_AUTO", "K_SIMT", "K_MMA", "K_TC5", "DT_F32", "DT_F16", "DT_BF16", "OK", "DECLINED",
           "ACT_SILU", "ACT_SWIGLU_OAI"]
