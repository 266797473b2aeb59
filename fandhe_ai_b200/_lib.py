"""ctypes loader of `libb200backend.so`.

The shared library is the product; nothing in this package computes on the CPU.
Loading fails loudly when the library has not been built (`python -m fandhe_ai_b200.build`).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libb200backend.so"

_lib = None


class BackendError(RuntimeError):
    """Mirror of the reference's `BackendError` (crates/tensor-core/src/device.rs:225-371):
    `kind` is the variant name, `status` the C-ABI code."""

    def __init__(self, status: int, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.status = status
        self.kind = kind
        self.message = message


def lib() -> C.CDLL:
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m fandhe_ai_b200.build` "
                "(this backend has no CPU or PyTorch fallback)"
            )
        _lib = C.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


def check(status: int) -> None:
    if status != 0:
        l = lib()
        raise BackendError(status, l.b200_status_name(status).decode(), l.b200_last_error().decode())


class PagedKvLayoutC(C.Structure):
    """b200_paged_kv_layout"""
    _fields_ = [("num_blocks", C.c_uint64), ("block_size", C.c_uint64), ("embed_dim", C.c_uint64),
                ("dtype", C.c_int32)]


class PagedAttentionArgsC(C.Structure):
    """b200_paged_attention_args"""
    _fields_ = [("layout", PagedKvLayoutC), ("batch", C.c_uint64), ("l_new", C.c_uint64), ("num_heads", C.c_uint64),
                ("num_kv_heads", C.c_uint64), ("max_blocks_per_seq", C.c_uint64), ("scale", C.c_float)]


class PagedAttentionPlanC(C.Structure):
    """b200_paged_attention_plan"""
    _fields_ = [("out_numel", C.c_uint64), ("s_max", C.c_uint64), ("query_rows", C.c_uint64),
                ("workspace_elems", C.c_uint64)]


class DecoderConfigC(C.Structure):
    """b200_decoder_config"""
    _fields_ = [("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("vocab", C.c_int32), ("rms_eps", C.c_float),
                ("rope_theta", C.c_float), ("max_batch", C.c_int32), ("max_seq_len", C.c_int32),
                ("block_size", C.c_int32), ("num_blocks", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
                ("use_graph", C.c_int32), ("tp_exact_int8", C.c_int32), ("act_fp8", C.c_int32)]


_P = C.c_void_p
_SZ = C.c_size_t
_I32 = C.c_int32
_I64 = C.c_int64
_U64 = C.c_uint64

# name -> (restype, argtypes); every symbol declared in include/b200_backend.h
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_status_name": (C.c_char_p, [_I32]),
    "b200_ctx_create": (_I32, [_I32, C.POINTER(_P)]),
    "b200_ctx_destroy": (_I32, [_P]),
    "b200_synchronize": (_I32, [_P]),
    "b200_ctx_is_poisoned": (_I32, [_P]),
    "b200_ctx_generation": (C.c_uint64, [_P]),
    "b200_ctx_stream": (_P, [_P]),
    "b200_ctx_recover": (_I32, [_P]),
    "b200_test_inject_probe_failures": (_I32, [_P, _I32]),
    "b200_test_poison": (_I32, [_P]),
    "b200_test_mark_capturing": (_I32, [_P, _I32]),
    "b200_memory_info": (_I32, [_P, C.POINTER(_SZ), C.POINTER(_SZ)]),
    "b200_gemm_tuning": (_I32, [_P, _I32, _I32]),
    "b200_gemm_plan_info": (_I32, [_P, _I64, _I64, _I64, _I32, _I32, _P]),
    "b200_alloc_zeroed": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "b200_upload": (_I32, [_P, _P, _SZ, C.POINTER(_P)]),
    "b200_upload_into": (_I32, [_P, _P, _SZ, _P, _SZ]),
    "b200_download": (_I32, [_P, _P, _SZ, _P, _SZ]),
    "b200_release": (_I32, [_P, _P]),
    "b200_buf_bytes": (_SZ, [_P]),
    "b200_buf_device_ptr": (_P, [_P]),
    "b200_quantize_i8_per_row": (_I32, [_P, _P, _SZ, _I64, _I64, _P, _SZ, _P, _SZ]),
    "b200_dequantize_i8_per_row": (_I32, [_P, _P, _SZ, _P, _SZ, _I64, _I64, _P, _SZ]),
    "b200_quantize_fp8_e4m3_per_tensor": (_I32, [_P, _P, _SZ, _I64, _P, _SZ, _P, _SZ]),
    "b200_gemm_i8_s32": (_I32, [_P, _P, _SZ, _P, _SZ, _I64, _I64, _I64, _P, _SZ]),
    "b200_gemm_q8_scaled": (_I32, [_P, _I32, _P, _SZ, _P, _SZ, _I32, _P, _SZ, _P, _SZ, _I32, _P, _SZ, _I32,
                                   _P, _SZ, _I64, _I64, _I64, _I32, _P, _SZ]),
    "b200_validate_paged_kv_append": (_I32, [_U64, _U64, _U64, _U64, _P, _U64, C.POINTER(PagedKvLayoutC),
                                             C.POINTER(_U64)]),
    "b200_validate_paged_attention": (_I32, [_U64, _U64, _U64, _P, _U64, _P, _U64, C.POINTER(PagedAttentionArgsC),
                                             C.POINTER(PagedAttentionPlanC)]),
    "b200_paged_kv_append": (_I32, [_P, _P, _SZ, _P, _SZ, _P, _P, _P, _U64, C.POINTER(PagedKvLayoutC)]),
    "b200_paged_attention_forward": (_I32, [_P, _P, _SZ, _P, _P, _P, _U64, _P, _U64, C.POINTER(PagedAttentionArgsC),
                                            _P, _SZ]),
    "b200_paged_attention_forward_resident": (_I32, [_P, _P, _SZ, _P, _P, _P, _P, _U64,
                                                     C.POINTER(PagedAttentionArgsC), _P, _SZ]),
    "b200_paged_attention_forward_noalloc": (_I32, [_P, _P, _SZ, _P, _P, _P, _P, _U64,
                                                    C.POINTER(PagedAttentionArgsC), _P, _SZ]),
    "b200_paged_attention_tuning": (_I32, [_P, _I32]),
    "b200_block_table_create": (_I32, [_U64, _U64, C.POINTER(_P)]),
    "b200_block_table_destroy": (None, [_P]),
    "b200_block_table_extend_for_append": (_I32, [_P, _U64, _U64, _P, _U64, C.POINTER(_U64)]),
    "b200_block_table_flatten": (_I32, [_P, _U64, _P, _U64]),
    "b200_block_table_rewind_to": (_I32, [_P, _U64]),
    "b200_block_table_clear": (None, [_P]),
    "b200_block_table_seq_len": (_U64, [_P]),
    "b200_block_table_free_blocks": (_U64, [_P]),
    "b200_block_table_used_blocks": (_U64, [_P]),
    "b200_block_table_batch": (_I64, [_P]),
    "b200_decoder_create": (_I32, [_P, C.POINTER(DecoderConfigC), C.POINTER(_P)]),
    "b200_decoder_destroy": (_I32, [_P]),
    "b200_decoder_load_tensor": (_I32, [_P, _I32, _I32, _P, _I64, _I64]),
    "b200_decoder_load_tensor_i8": (_I32, [_P, _I32, _I32, _P, _P, _I64, _I64]),
    "b200_decoder_load_safetensors": (_I32, [_P, C.c_char_p]),
    "b200_decoder_load_safetensors_bytes": (_I32, [_P, _P, _SZ]),
    "b200_safetensors_validate": (_I32, [_P, _SZ, C.POINTER(_U64)]),
    "b200_decoder_init_random": (_I32, [_P, _U64, C.c_float]),
    "b200_nccl_unique_id": (_I32, [_P]),
    "b200_decoder_init_tp": (_I32, [_P, _P]),
    "b200_decoder_tp_exchange": (_I32, [_P]),
    "b200_selftest_peer_wait": (_I32, [_P]),
    "b200_selftest_tp_finish": (_I32, [_P, _I32, _I32, _I32, _I32, _P, _P, _P, C.c_float, _P, _P, _P, _P]),
    "b200_selftest_tp_scatter": (_I32, [_P, _I32, _I32, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P, _P, C.c_float, _P, _P, _P, _P]),
    "b200_gemm_phase_stamps": (_I32, [_P, C.c_int64, C.c_int64, C.c_int64, _I32, _I32, _P, _P, _P, _P]),
    "b200_decoder_batch": (_I32, [_P]),
    "b200_sampling_weights": (_I32, [_P, C.c_int64, C.c_int64, _I32, _I32, C.c_float, _P]),
    "b200_decoder_sampling_weights": (_I32, [_P, _I32, _I32, C.c_float, _P, C.c_uint64]),
    "b200_decoder_step_rows": (_I32, [_P, _P, _P, _P]),
    "b200_decoder_row_restart": (_I32, [_P, _I32, _I32]),
    "b200_scheduler_create": (_I32, [_P, _I32, _I32, _I32, _P]),
    "b200_scheduler_destroy": (None, [_P]),
    "b200_scheduler_submit": (_I32, [_P, _P, _I32, _I32, _P]),
    "b200_scheduler_queued_len": (_I32, [_P]),
    "b200_scheduler_active_len": (_I32, [_P]),
    "b200_scheduler_finished_len": (_I32, [_P]),
    "b200_scheduler_step": (_I32, [_P, _P]),
    "b200_scheduler_plan_step": (_I32, [_P, _P, _P, _P, _P, _P, _P]),
    "b200_scheduler_commit_step": (_I32, [_P, _P, _P]),
    "b200_scheduler_failed_len": (_I32, [_P]),
    "b200_scheduler_take_failed": (_I32, [_P, _P, _P, _P, _I32, _P]),
    "b200_scheduler_configure": (_I32, [_P, _I32, _I32]),
    "b200_decoder_prefill": (_I32, [_P, _I32, _I32, _P, _I32]),
    "b200_decoder_vocab": (_I32, [_P]),
    "b200_scheduler_take_finished": (_I32, [_P, _P, _P, _I32, _P]),
    "b200_decoder_begin": (_I32, [_P, _I32, _P, _P]),
    "b200_decoder_fill_cache_random": (_I32, [_P, _U64, C.c_float]),
    "b200_decoder_step": (_I32, [_P, _P, _P]),
    "b200_decoder_logits": (_I32, [_P, _P, _U64]),
    "b200_decoder_generate": (_I32, [_P, _P, _I32, _I32, _I32, _P]),
    "b200_decoder_shard_plan": (_I32, [C.POINTER(DecoderConfigC), _I32, C.POINTER(_I64), C.POINTER(_I64), _P,
                                       C.POINTER(_I32), C.POINTER(_I64), C.POINTER(_I64)]),
    "b200_decoder_launches_per_step": (_U64, [_P]),
    "b200_decoder_weight_bytes": (_U64, [_P]),
    "b200_decoder_plan_info": (_I32, [_P, _P]),
    "b200_timer_start": (_I32, [_P]),
    "b200_timer_stop": (_I32, [_P, C.POINTER(C.c_float)]),
    "b200_decoder_time_attention": (_I32, [_P, _I32, C.POINTER(C.c_float), C.POINTER(_U64)]),
    "b200_quantize_i8_block": (_I32, [_P, _P, _SZ, _I64, _I64, _I64, _I32, _P, _SZ, _P, _SZ]),
    "b200_dequantize_i8_block": (_I32, [_P, _P, _SZ, _P, _SZ, _I64, _I64, _I64, _I32, _P, _SZ]),
    "b200_gemm_i8_block_scaled": (_I32, [_P, _P, _SZ, _P, _SZ, _P, _SZ, _P, _SZ, _I64, _I64, _I64, _I64, _P, _SZ]),
    "b200_quant_check": (_I32, [_P]),
    "b200_linear_fp8": (_I32, [_P, _P, _SZ, _I64, _I64, _P, _SZ, _P, _SZ, _P, _SZ, _I64, _I32, _P, _SZ, _I32, _P, _SZ]),
    "b200_linear_w8a8": (_I32, [_P, _P, _SZ, _I64, _I64, _P, _SZ, _P, _SZ, _P, _SZ, _I64, _I32, _P, _SZ, _P, _SZ]),
}


def _declare(l: C.CDLL) -> None:
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(l, name)
        fn.restype = res
        fn.argtypes = args
