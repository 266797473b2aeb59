"""Host-side mirror of the reference's operator surface for the quantized decode path.

`Backend` plays the role of `CudaBackendOps` + `MemoryOps` for this path
(crates/tensor-core/src/backend_ops.rs:1275, crates/tensor-core/src/buffer.rs:389): the
method names and argument meaning follow the trait methods they stand for, and every
method is a thin call into the C ABI of `libb200backend.so`.  Nothing here computes.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from ._lib import BackendError, check, lib

# b200_activation
ACT_NONE, ACT_RELU, ACT_SILU, ACT_SILU_GATE = 0, 1, 2, 3
# b200_dtype
F32, BF16, I8, FP8_E4M3, I32, U32 = 0, 1, 2, 3, 4, 5


class DeviceBuffer:
    """Device-resident buffer handle (the reference's `DeviceBuffer<T>`,
    crates/tensor-core/src/buffer.rs:145-207).  Owned by the backend that made it."""

    def __init__(self, backend: "Backend", handle: int, nbytes: int, shape=None, dtype=None):
        self.backend = backend
        self.handle = C.c_void_p(handle)
        self.nbytes = nbytes
        self.shape = tuple(shape) if shape is not None else (nbytes,)
        self.dtype = np.dtype(dtype) if dtype is not None else np.dtype(np.uint8)

    def numpy(self) -> np.ndarray:
        return self.backend.download(self)

    def release(self) -> None:
        if self.handle is not None and self.backend._ctx is not None:
            lib().b200_release(self.backend._ctx, self.handle)
        self.handle = None

    @property
    def device_ptr(self) -> int:
        return lib().b200_buf_device_ptr(self.handle) or 0


class Backend:
    """One context per CUDA ordinal: single stream, enqueue-only ops, `download` is the sync point."""

    def __init__(self, ordinal: int = 0):
        self._ctx = None
        ctx = C.c_void_p()
        check(lib().b200_ctx_create(ordinal, C.byref(ctx)))
        self._ctx = ctx
        self.ordinal = ordinal

    def close(self) -> None:
        if self._ctx is not None:
            lib().b200_ctx_destroy(self._ctx)
            self._ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------- MemoryOps
    def alloc_zeroed(self, shape, dtype=np.float32) -> DeviceBuffer:
        dtype = np.dtype(dtype)
        nbytes = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
        h = C.c_void_p()
        check(lib().b200_alloc_zeroed(self._ctx, nbytes, C.byref(h)))
        return DeviceBuffer(self, h.value or 0, nbytes, shape, dtype)

    def upload(self, array: np.ndarray) -> DeviceBuffer:
        a = np.ascontiguousarray(array)
        h = C.c_void_p()
        check(lib().b200_upload(self._ctx, a.ctypes.data_as(C.c_void_p), a.nbytes, C.byref(h)))
        return DeviceBuffer(self, h.value or 0, a.nbytes, a.shape, a.dtype)

    def upload_into(self, array: np.ndarray, dst: DeviceBuffer, offset_bytes: int = 0) -> None:
        a = np.ascontiguousarray(array)
        check(lib().b200_upload_into(self._ctx, a.ctypes.data_as(C.c_void_p), a.nbytes, dst.handle, offset_bytes))

    def download(self, buf: DeviceBuffer, shape=None, dtype=None, offset_bytes: int = 0) -> np.ndarray:
        dtype = np.dtype(dtype) if dtype is not None else buf.dtype
        shape = tuple(shape) if shape is not None else buf.shape
        out = np.empty(shape, dtype=dtype)
        check(lib().b200_download(self._ctx, buf.handle, offset_bytes, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def synchronize_device(self) -> None:
        check(lib().b200_synchronize(self._ctx))

    @property
    def poisoned(self) -> bool:
        return bool(lib().b200_ctx_is_poisoned(self._ctx))

    @property
    def stream(self) -> int:
        return lib().b200_ctx_stream(self._ctx) or 0

    def timer_start(self) -> None:
        """Starts the CUDA-event stopwatch on this context's stream."""
        check(lib().b200_timer_start(self._ctx))

    def timer_stop(self) -> float:
        """Waits for the stream and returns the device milliseconds since timer_start()."""
        ms = C.c_float()
        check(lib().b200_timer_stop(self._ctx, C.byref(ms)))
        return float(ms.value)

    def gemm_tuning(self, tile_n: int = 0, splits: int = 0) -> None:
        check(lib().b200_gemm_tuning(self._ctx, tile_n, splits))

    def gemm_plan_info(self, m: int, n: int, k: int, gated: bool = False, fused: bool = True) -> dict:
        """Which kernel form a GEMM of this shape takes (nothing is launched)."""
        buf = (C.c_int32 * 6)()
        check(lib().b200_gemm_plan_info(self._ctx, m, n, k, int(gated), int(fused), buf))
        return dict(zip(["tile", "splits", "cluster", "persistent", "ctas", "stages"], list(buf)))

    def gemm_phase_stamps(self, m: int, n: int, k: int, fused: bool = False, iters: int = 50) -> dict:
        """Profiling aid: where the time of one decode-shaped GEMM launch goes (see b200_gemm_phase_stamps)."""
        stamps = (C.c_uint64 * 9)()
        loop_us, alone_us = C.c_float(), C.c_float()
        info = (C.c_int32 * 6)()
        check(lib().b200_gemm_phase_stamps(self._ctx, m, n, k, int(fused), iters, stamps, C.byref(loop_us), C.byref(alone_us), info))
        names = ["entry", "setup", "dep_wait", "loads_issued", "first_tile", "mma_issued", "acc_ready", "stored", "exit"]
        return {"m": m, "n": n, "k": k, "fused": bool(fused), "tile": info[0], "splits": info[1], "cluster": info[2],
                "stages": info[5], "loop_us_per_launch": round(float(loop_us.value), 2), "alone_us": round(float(alone_us.value), 2),
                "stamps_ns": dict(zip(names, [int(x) for x in stamps]))}

    def memory_info(self):
        """(free, total) device memory in bytes."""
        free, total = C.c_size_t(), C.c_size_t()
        check(lib().b200_memory_info(self._ctx, C.byref(free), C.byref(total)))
        return int(free.value), int(total.value)

    def recover(self) -> None:
        """In-place recovery of a poisoned context (`invalidate` of the reference's ordinal state machine)."""
        check(lib().b200_ctx_recover(self._ctx))

    # ------------------------------------------------------------- QuantOps
    def quantize_i8_per_row(self, x: DeviceBuffer, rows: int, cols: int):
        """Symmetric int8 with one scale per row (per output channel for weights [n, k], per token
        for activations [m, k]).  Returns (q int8 [rows, cols], scale f32 [rows])."""
        q = self.alloc_zeroed((rows, cols), np.int8)
        s = self.alloc_zeroed((rows,), np.float32)
        check(lib().b200_quantize_i8_per_row(self._ctx, x.handle, 0, rows, cols, q.handle, 0, s.handle, 0))
        return q, s

    def dequantize_i8_per_row(self, q: DeviceBuffer, scale: DeviceBuffer, rows: int, cols: int) -> DeviceBuffer:
        x = self.alloc_zeroed((rows, cols), np.float32)
        check(lib().b200_dequantize_i8_per_row(self._ctx, q.handle, 0, scale.handle, 0, rows, cols, x.handle, 0))
        return x

    def quantize_fp8_e4m3_per_tensor(self, x: DeviceBuffer, numel: int):
        q = self.alloc_zeroed((numel,), np.uint8)
        s = self.alloc_zeroed((1,), np.float32)
        check(lib().b200_quantize_fp8_e4m3_per_tensor(self._ctx, x.handle, 0, numel, q.handle, 0, s.handle, 0))
        return q, s

    def gemm_i8_s32(self, a: DeviceBuffer, w: DeviceBuffer, m: int, n: int, k: int) -> DeviceBuffer:
        acc = self.alloc_zeroed((m, n), np.int32)
        check(lib().b200_gemm_i8_s32(self._ctx, a.handle, 0, w.handle, 0, m, n, k, acc.handle, 0))
        return acc

    def gemm_q8_scaled(self, op_dtype: int, a: DeviceBuffer, a_scale: DeviceBuffer, a_scale_per_row: bool,
                       w: DeviceBuffer, w_scale: DeviceBuffer, w_scale_per_row: bool, m: int, n: int, k: int,
                       bias: Optional[DeviceBuffer] = None, activation: int = ACT_NONE,
                       residual: Optional[DeviceBuffer] = None, out_dtype: int = F32,
                       w_off: int = 0, w_scale_off: int = 0, bias_off: int = 0) -> DeviceBuffer:
        n_out = n // 2 if activation == ACT_SILU_GATE else n
        out = self.alloc_zeroed((m, n_out), np.float32 if out_dtype == F32 else np.uint16)
        check(lib().b200_gemm_q8_scaled(
            self._ctx, op_dtype, a.handle, 0, a_scale.handle, 0, int(a_scale_per_row), w.handle, w_off,
            w_scale.handle, w_scale_off, int(w_scale_per_row), bias.handle if bias else None, bias_off, activation,
            residual.handle if residual else None, 0, m, n, k, out_dtype, out.handle, 0))
        return out

    # ------------------------------------------------------------- QuantOps, block-scale contract
    def quantize_i8_block(self, x: DeviceBuffer, rows: int, cols: int, scales_block_major: bool = False, block_len: int = 128):
        """One power-of-two scale per 128 values of a row (the reference's proposed contract).  Returns
        (q int8 [rows, cols], delta f32 [rows, nb] or [nb, rows])."""
        nb = -(-cols // 128)
        q = self.alloc_zeroed((rows, cols), np.int8)
        d = self.alloc_zeroed((nb, rows) if scales_block_major else (rows, nb), np.float32)
        check(lib().b200_quantize_i8_block(self._ctx, x.handle, 0, rows, cols, block_len, int(scales_block_major), q.handle, 0,
                                           d.handle, 0))
        return q, d

    def dequantize_i8_block(self, q: DeviceBuffer, delta: DeviceBuffer, rows: int, cols: int,
                            scales_block_major: bool = False, block_len: int = 128) -> DeviceBuffer:
        x = self.alloc_zeroed((rows, cols), np.float32)
        check(lib().b200_dequantize_i8_block(self._ctx, q.handle, 0, delta.handle, 0, rows, cols, block_len,
                                             int(scales_block_major), x.handle, 0))
        return x

    def gemm_i8_block_scaled(self, a: DeviceBuffer, a_delta: DeviceBuffer, w: DeviceBuffer, w_delta: DeviceBuffer, m: int,
                             n: int, k: int, block_len: int = 128) -> DeviceBuffer:
        """`gemm_i8_s32_scaled` of the proposed QuantOps: a_delta [m, nb], w_delta [nb, n]; f32 [m, n]."""
        out = self.alloc_zeroed((m, n), np.float32)
        check(lib().b200_gemm_i8_block_scaled(self._ctx, a.handle, 0, a_delta.handle, 0, w.handle, 0, w_delta.handle, 0, m, n, k,
                                              block_len, out.handle, 0))
        return out

    def quant_check(self) -> None:
        """Synchronises; raises InvalidArgument when a block-scale call met a non-finite input or result."""
        check(lib().b200_quant_check(self._ctx))

    # ------------------------------------------------------------- BackendOps (quantized linear)
    def linear_forward_device_into(self, a: DeviceBuffer, m: int, k: int, w_q: DeviceBuffer, w_off: int,
                                   w_scale: DeviceBuffer, w_scale_off: int, bias: Optional[DeviceBuffer],
                                   bias_off: int, n: int, activation: int, out: DeviceBuffer,
                                   residual: Optional[DeviceBuffer] = None) -> None:
        """`linear_forward_device_into_tracked` for int8 per-channel weights
        (crates/tensor-core/src/backend_ops.rs:4350-4366): writes all outputs into `out`."""
        check(lib().b200_linear_w8a8(self._ctx, a.handle, 0, m, k, w_q.handle, w_off, w_scale.handle, w_scale_off,
                                     bias.handle if bias else None, bias_off, n, activation,
                                     residual.handle if residual else None, 0, out.handle, 0))

    def linear_forward_device(self, a: DeviceBuffer, m: int, k: int, w_q: DeviceBuffer, w_scale: DeviceBuffer,
                              bias: Optional[DeviceBuffer], n: int, activation: int = ACT_NONE,
                              residual: Optional[DeviceBuffer] = None) -> DeviceBuffer:
        """`linear_forward_device` (crates/tensor-core/src/backend_ops.rs:4296-4309), allocating the output."""
        n_out = n // 2 if activation == ACT_SILU_GATE else n
        out = self.alloc_zeroed((m, n_out), np.float32)
        self.linear_forward_device_into(a, m, k, w_q, 0, w_scale, 0, bias, 0, n, activation, out, residual)
        return out


    def linear_fp8_forward_device(self, a: DeviceBuffer, m: int, k: int, w_fp8: DeviceBuffer, w_scale: DeviceBuffer,
                                  bias: Optional[DeviceBuffer], n: int, activation: int = ACT_NONE,
                                  residual: Optional[DeviceBuffer] = None, out_dtype: int = F32, w_off: int = 0,
                                  w_scale_off: int = 0, bias_off: int = 0) -> DeviceBuffer:
        """`linear_forward_device` with E4M3 weights (one scale) and the f32 activation quantised per tensor on
        the device (crates/tensor-core/src/low_precision.rs:193-249 is the f16 / bf16 ancestor)."""
        n_out = n // 2 if activation == ACT_SILU_GATE else n
        out = self.alloc_zeroed((m, n_out), np.float32 if out_dtype == F32 else np.uint16)
        check(lib().b200_linear_fp8(self._ctx, a.handle, 0, m, k, w_fp8.handle, w_off, w_scale.handle, w_scale_off,
                                    bias.handle if bias else None, bias_off, n, activation,
                                    residual.handle if residual else None, 0, out_dtype, out.handle, 0))
        return out


__all__ = ["Backend", "DeviceBuffer", "BackendError", "ACT_NONE", "ACT_RELU", "ACT_SILU", "ACT_SILU_GATE",
           "F32", "BF16", "I8", "FP8_E4M3", "I32", "U32"]
