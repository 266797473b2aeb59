"""Host mirror of the decode driver: `BlockTable` (the reference's host page table,
crates/autodiff/src/nn/paged_kv.rs:158-364) and `Decoder` (the quantized Llama-style stack driven
like `generate()`, crates/autodiff/src/generate/mod.rs:500-613).  Both are thin ctypes views of the
C++ objects inside `libb200backend.so`."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import DecoderConfigC, check, lib
from .backend import Backend

W_EMBED, W_ATTN_NORM, W_QKV, W_O, W_MLP_NORM, W_GATE_UP, W_DOWN, W_FINAL_NORM, W_LM_HEAD = range(9)


class BlockTable:
    """LIFO free stack + fresh counter, row-major slot mapping, sentinel-padded flattening."""

    def __init__(self, max_blocks: int, block_size: int):
        self._h = C.c_void_p()
        check(lib().b200_block_table_create(max_blocks, block_size, C.byref(self._h)))
        self.max_blocks = max_blocks
        self.block_size = block_size

    def __del__(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            lib().b200_block_table_destroy(self._h)
            self._h = None

    def extend_for_append(self, batch: int, l_new: int) -> list[int]:
        cap = max(1, batch * l_new)
        buf = (C.c_uint32 * cap)()
        n = C.c_uint64()
        check(lib().b200_block_table_extend_for_append(self._h, batch, l_new, buf, cap, C.byref(n)))
        return list(buf[: n.value])

    def flatten_tables(self, max_blocks_per_seq: int) -> np.ndarray:
        b = max(self.batch or 0, 0)
        out = np.empty((b, max_blocks_per_seq), np.uint32)
        check(lib().b200_block_table_flatten(self._h, max_blocks_per_seq, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def rewind_to(self, new_len: int) -> None:
        check(lib().b200_block_table_rewind_to(self._h, new_len))

    def clear(self) -> None:
        lib().b200_block_table_clear(self._h)

    @property
    def seq_len(self) -> int:
        return int(lib().b200_block_table_seq_len(self._h))

    @property
    def num_free_blocks(self) -> int:
        return int(lib().b200_block_table_free_blocks(self._h))

    @property
    def num_used_blocks(self) -> int:
        return int(lib().b200_block_table_used_blocks(self._h))

    @property
    def batch(self):
        b = int(lib().b200_block_table_batch(self._h))
        return None if b < 0 else b


SAMPLE_GREEDY, SAMPLE_TEMPERATURE, SAMPLE_TOP_K = 0, 1, 2


def sampling_weights(logits, strategy: int, k: int = 0, temperature: float = 1.0) -> np.ndarray:
    """Host rows of logits [rows, vocab] -> the reference's sampling weights (see Decoder.sampling_weights)."""
    x = np.ascontiguousarray(logits, dtype=np.float32)
    rows, vocab = x.shape
    out = np.empty((rows, vocab), np.float32)
    check(lib().b200_sampling_weights(x.ctypes.data_as(C.c_void_p), rows, vocab, strategy, k, C.c_float(temperature),
                                      out.ctypes.data_as(C.c_void_p)))
    return out


@dataclass
class DecoderConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_batch: int = 32
    max_seq_len: int = 256
    block_size: int = 16
    num_blocks: int = 0          # 0: enough for max_batch rows of max_seq_len tokens
    tp_rank: int = 0
    tp_size: int = 1
    use_graph: int = 1
    tp_exact_int8: int = 0       # tensor parallel: one global per-token scale + int32 all-reduce (results independent of tp_size)
    act_fp8: int = 0             # 1: E4M3 weights and activations, f32 accumulation (the FP8 x FP8 form of the decoder)

    def to_c(self) -> DecoderConfigC:
        nb = self.num_blocks or self.max_batch * -(-self.max_seq_len // self.block_size)
        return DecoderConfigC(self.n_layers, self.d_model, self.n_heads, self.n_kv_heads, self.head_dim, self.d_ff,
                              self.vocab, self.rms_eps, self.rope_theta, self.max_batch, self.max_seq_len,
                              self.block_size, nb, self.tp_rank, self.tp_size, self.use_graph, self.tp_exact_int8, self.act_fp8)


def shard_plan(cfg: DecoderConfig, which: int) -> dict:
    """Rows and columns of full weight matrix `which` that rank cfg.tp_rank keeps (host arithmetic only)."""
    cc = cfg.to_c()
    rows, cols, c0, cn = C.c_int64(), C.c_int64(), C.c_int64(), C.c_int64()
    n = C.c_int32()
    rr = (C.c_int64 * 6)()
    check(lib().b200_decoder_shard_plan(C.byref(cc), which, C.byref(rows), C.byref(cols), rr, C.byref(n), C.byref(c0),
                                        C.byref(cn)))
    return {"rows": rows.value, "cols": cols.value, "col_start": c0.value, "col_count": cn.value,
            "row_ranges": [(rr[2 * i], rr[2 * i + 1]) for i in range(n.value)]}


def nccl_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    check(lib().b200_nccl_unique_id(buf))
    return bytes(buf)


class Decoder:
    def __init__(self, be: Backend, cfg: DecoderConfig):
        self.be = be
        self.cfg = cfg
        self._h = C.c_void_p()
        cc = cfg.to_c()
        check(lib().b200_decoder_create(be._ctx, C.byref(cc), C.byref(self._h)))

    def close(self) -> None:
        if self._h is not None and self._h.value:
            lib().b200_decoder_destroy(self._h)
        self._h = None

    def load_tensor(self, which: int, layer: int, array) -> None:
        a = np.ascontiguousarray(array, dtype=np.float32)
        if a.ndim == 1:
            a = a.reshape(1, -1)
        check(lib().b200_decoder_load_tensor(self._h, which, layer, a.ctypes.data_as(C.c_void_p), a.shape[0], a.shape[1]))

    def load_weights(self, weights: dict) -> None:
        """weights: {"embed", "final_norm", "lm_head", "layers": [{"attn_norm","wqkv","wo","mlp_norm","wgu","wdown"}]}"""
        self.load_tensor(W_EMBED, 0, weights["embed"])
        self.load_tensor(W_FINAL_NORM, 0, weights["final_norm"])
        self.load_tensor(W_LM_HEAD, 0, weights["lm_head"])
        for l, lw in enumerate(weights["layers"]):
            self.load_tensor(W_ATTN_NORM, l, lw["attn_norm"])
            self.load_tensor(W_QKV, l, lw["wqkv"])
            self.load_tensor(W_O, l, lw["wo"])
            self.load_tensor(W_MLP_NORM, l, lw["mlp_norm"])
            self.load_tensor(W_GATE_UP, l, lw["wgu"])
            self.load_tensor(W_DOWN, l, lw["wdown"])

    def load_safetensors(self, path) -> None:
        """Loads every tensor from a safetensors file (int8 payloads with per-row scales, or f32 tensors)."""
        check(lib().b200_decoder_load_safetensors(self._h, str(path).encode()))

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        check(lib().b200_decoder_init_random(self._h, seed, std))

    def init_tp(self, unique_id: bytes) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(lib().b200_decoder_init_tp(self._h, buf))

    @property
    def tp_exchange(self) -> bool:
        """True when the row-parallel outputs are finished over the ranks' mapped exchange blocks (one kernel
        with peer loads and stores) instead of ncclAllReduce."""
        return bool(lib().b200_decoder_tp_exchange(self._h))

    @property
    def tp_exchange_mode(self) -> int:
        """0: ncclAllReduce; 1: finish kernel that loads the peers' partials; 2: the GEMMs store their partial rows
        into the owner's block and the finish kernel reads local memory only."""
        return int(lib().b200_decoder_tp_exchange(self._h))

    def begin(self, batch: int, max_total_lens, start_lens=None) -> None:
        mt = np.ascontiguousarray(max_total_lens, dtype=np.int32)
        sl = np.ascontiguousarray(start_lens, dtype=np.int32) if start_lens is not None else None
        check(lib().b200_decoder_begin(self._h, batch, sl.ctypes.data_as(C.c_void_p) if sl is not None else None,
                                       mt.ctypes.data_as(C.c_void_p)))
        self._batch = batch

    def fill_cache_random(self, seed: int = 1, std: float = 1.0) -> None:
        check(lib().b200_decoder_fill_cache_random(self._h, seed, std))

    def prefill(self, ids, row0: int = 0) -> None:
        """Multi-token prefill: ids [count, l_new] for the rows [row0, row0 + count); nothing is sampled."""
        a = np.ascontiguousarray(ids, dtype=np.int32)
        count, l_new = a.shape
        check(lib().b200_decoder_prefill(self._h, row0, count, a.ctypes.data_as(C.c_void_p), l_new))

    def step(self, ids=None, want_next: bool = True):
        ids_c = np.ascontiguousarray(ids, dtype=np.int32) if ids is not None else None
        nxt = np.empty(self._batch, np.int32) if want_next else None
        check(lib().b200_decoder_step(self._h, ids_c.ctypes.data_as(C.c_void_p) if ids_c is not None else None,
                                      nxt.ctypes.data_as(C.c_void_p) if nxt is not None else None))
        return nxt

    def step_raw(self, ids_ptr, next_ptr) -> None:
        """step() on caller-owned int32 buffers (no allocation in the timed loop)."""
        check(lib().b200_decoder_step(self._h, ids_ptr, next_ptr))

    def logits(self) -> np.ndarray:
        out = np.empty((self._batch, self.cfg.vocab), np.float32)
        check(lib().b200_decoder_logits(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def sampling_weights(self, strategy: int, k: int = 0, temperature: float = 1.0) -> np.ndarray:
        """[batch, vocab] f32 weights of the last step's logits, as the reference's sample_step builds them before
        it draws (crates/autodiff/src/generate/mod.rs:382-455); the draw stays with the caller's generator."""
        out = np.empty((self._batch, self.cfg.vocab), np.float32)
        check(lib().b200_decoder_sampling_weights(self._h, strategy, k, C.c_float(temperature),
                                                  out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def generate(self, prompt, max_length: int) -> np.ndarray:
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        batch, t = p.shape
        out = np.empty((batch, max_length), np.int32)
        check(lib().b200_decoder_generate(self._h, p.ctypes.data_as(C.c_void_p), batch, t, max_length,
                                          out.ctypes.data_as(C.c_void_p)))
        self._batch = batch
        return out

    def time_attention(self, iters: int = 32):
        """(mean ms of one decode-attention launch alone, its algorithmic bytes)."""
        ms = C.c_float()
        nbytes = C.c_uint64()
        check(lib().b200_decoder_time_attention(self._h, iters, C.byref(ms), C.byref(nbytes)))
        return float(ms.value), int(nbytes.value)

    @property
    def launches_per_step(self) -> int:
        return int(lib().b200_decoder_launches_per_step(self._h))

    @property
    def weight_bytes(self) -> int:
        return int(lib().b200_decoder_weight_bytes(self._h))

    def plan_info(self) -> dict:
        buf = (C.c_int32 * 10)()
        check(lib().b200_decoder_plan_info(self._h, buf))
        k = ["qkv_tile", "qkv_splits", "o_tile", "o_splits", "gu_tile", "gu_splits", "down_tile", "down_splits",
             "attn_chunk_blocks", "attn_max_chunks"]
        return dict(zip(k, list(buf)))


def write_safetensors(path, tensors: dict) -> None:
    """Writes {name: numpy array} (float32 / int8 / any dtype of the format) as a safetensors file: 8-byte little-endian
    header length, JSON header, contiguous data.  For tests and for exporting quantised weights."""
    import json

    names = {"float32": "F32", "int8": "I8", "uint8": "U8", "float16": "F16", "int32": "I32", "int64": "I64",
             "float64": "F64", "bool": "BOOL", "uint16": "U16"}
    header, blobs, at = {}, [], 0
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr)
        raw = a.tobytes()
        header[name] = {"dtype": names[str(a.dtype)], "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(len(text).to_bytes(8, "little"))
        f.write(text)
        for raw in blobs:
            f.write(raw)

