"""B200-native (sm_100a) quantized transformer-decode backend: Python host mirror of the
reference's operator surface over the C ABI of `libb200backend.so`."""
from .backend import (ACT_NONE, ACT_RELU, ACT_SILU, ACT_SILU_GATE, BF16, F32, FP8_E4M3, I8, I32, U32, Backend,
                      BackendError, DeviceBuffer)

__all__ = ["Backend", "DeviceBuffer", "BackendError", "ACT_NONE", "ACT_RELU", "ACT_SILU", "ACT_SILU_GATE",
           "F32", "BF16", "I8", "FP8_E4M3", "I32", "U32"]
