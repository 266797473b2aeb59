"""CPU restatement of the quantized Llama-style decoder (TEST INFRASTRUCTURE ONLY, like oracle.py).

PARITY UNPINNED: the reference has no RoPE, SwiGLU layer, Llama model, int8 path or tensor parallelism;
the wiring below is this project's definition, built from the pieces the reference does pin (RMSNorm
with an f64 sum of squares, the two-branch SiLU, the sequential paged attention, first-max greedy
sampling) and the quantisation rule of the benchmark text.  One token row at a time goes through

    h = embed[id]
    per layer:  xq, sx = quant(rmsnorm(h) * attn_norm)
                qkv    = acc(xq, Wqkv) * (sx * s_w)            -> RoPE on q, k -> k, v appended as bf16
                a      = paged_attention(q, cache)              (f32 math on bf16 K/V)
                h     += sum_r acc(quant_r(a_r), Wo_r) * (sa_r * s_w)     (r: tensor-parallel rank, ascending)
                xq, sx = quant(rmsnorm(h) * mlp_norm)
                f      = silu(gate) * up,   gate/up = acc(xq, Wgu) * (sx * s_w)
                h     += sum_r acc(quant_r(f_r), Wdown_r) * (sf_r * s_w)
    logits = acc(quant(rmsnorm(h) * final_norm), Wlm) * (sx * s_w);  next = first argmax
"""
from __future__ import annotations

import numpy as np

from . import oracle as O


def make_weights(cfg: dict, seed: int = 0, std: float = 0.02) -> dict:
    """Random-init weights N(0, std^2) (norm weights 1), f32, full (unsharded) shapes."""
    rng = np.random.default_rng(seed)
    d, dh, hq, hkv, f, v = cfg["d_model"], cfg["head_dim"], cfg["n_heads"], cfg["n_kv_heads"], cfg["d_ff"], cfg["vocab"]

    def n(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32)

    w = {"embed": n(v, d), "final_norm": np.ones(d, np.float32), "lm_head": n(v, d), "layers": []}
    for _ in range(cfg["n_layers"]):
        w["layers"].append({"attn_norm": np.ones(d, np.float32), "wqkv": n((hq + 2 * hkv) * dh, d), "wo": n(d, hq * dh),
                            "mlp_norm": np.ones(d, np.float32), "wgu": n(2 * f, d), "wdown": n(d, f)})
    return w


def wide_shape(n: int, rows: int = 1, sm_count: int = 148):
    """Launch shape the decode driver picks for a row of n columns owned by one CTA: (groups of four columns per
    thread, threads), or None when the row is too wide (restates wide_shape() of csrc/decode_rows.cu)."""
    if n <= 0 or n % 4:
        return None
    groups = n // 4
    v = -(-groups // 1024)
    if v > 4:
        return None
    if v == 3:
        v = 4
    while rows > sm_count and v < 4 and groups // (2 * v) >= 256:
        v *= 2
    return v, (-(-groups // v) + 31) // 32 * 32


def pick_cluster(n: int):
    """Column chunks (one 256-thread CTA each) of the cluster kernels for a row of n columns, or None
    (restates pick_cluster() of csrc/decode_rows.cu)."""
    cl = 8
    while cl >= 1:
        if n % (cl * 4) == 0 and n // cl <= 2048 and not (cl > 1 and n // cl < 512):
            return cl
        cl //= 2
    return None


class DecoderRef:
    """exact=False: the sequential definition (reference order of every reduction, libm exp).
    exact=True: every floating-point reduction in the order of the CUDA kernels and their exponential, so that
    logits and greedy ids can be compared bit for bit with the device (shapes that run on the general attention
    kernel only: head_dim other than 128, or blocks other than 16 tokens); the integer GEMMs go through BLAS."""

    def __init__(self, cfg: dict, weights: dict, tp: int = 1, exact: bool = False, sm_count: int = 148, fp8: bool = False):
        """fp8=True: the FP8 x FP8 form - weights and activations as E4M3 codes under per-row scales amax / 448,
        products accumulated in f32 (ascending k, one fma per product); everything else unchanged."""
        self.cfg = cfg
        self.tp = tp
        self.w = weights
        self.exact = exact
        self.sm_count = sm_count
        self.fp8 = fp8
        self._qrow = O.quantize_fp8_per_row if fp8 else O.quantize_i8_per_row
        if fp8 and exact:
            raise ValueError("the tensor core's f32 accumulation order is not restated")
        self.q = {"lm_head": self._qrow(weights["lm_head"]), "layers": []}
        for lw in weights["layers"]:
            self.q["layers"].append({k: self._qrow(lw[k]) for k in ("wqkv", "wo", "wgu", "wdown")})
        self.blas = None
        if exact:
            if tp != 1:
                raise ValueError("exact order is defined for one rank")
            if cfg["head_dim"] == 128 and cfg.get("block_size", 16) == 16:
                raise ValueError("this shape runs on the tensor-core attention kernel, whose summation order is not restated")
            if pick_cluster(cfg["d_model"]) is None or wide_shape(cfg["d_model"]) is None or wide_shape(cfg["d_ff"]) is None:
                raise ValueError("row width outside the restated kernels")
            self.blas = {"lm_head": O.int8_weight_for_blas(self.q["lm_head"][0]),
                         "layers": [{k: O.int8_weight_for_blas(v[0]) for k, v in lq.items()} for lq in self.q["layers"]]}
        self.cos, self.sin = O.rope_table(cfg["max_seq_len"], cfg["head_dim"], cfg.get("rope_theta", 10000.0))
        self.k = None

    def _acc(self, xq, lq_entry, blas_entry):
        if self.fp8:
            return O.gemm_fp8_f32(xq, lq_entry[0])
        return O.gemm_i8_s32_blas(xq, blas_entry) if blas_entry is not None else O.gemm_i8_s32(xq, lq_entry[0])

    def _norm(self, h, w, eps, first: bool):
        """RMSNorm of the rows of h: `first` is the embedding kernel (a cluster of 256-thread CTAs per row), the
        others are the one-wide-CTA-per-row kernels."""
        if not self.exact:
            return O.rmsnorm(h, w, eps)
        d = h.shape[1]
        if first:
            return O.rmsnorm_kernel_order(h, w, eps, 1, 256, pick_cluster(d))
        vpt, threads = wide_shape(d, h.shape[0], self.sm_count)
        return O.rmsnorm_kernel_order(h, w, eps, 0, threads, vpt)

    def begin(self, batch: int):
        c = self.cfg
        ekv = c["n_kv_heads"] * c["head_dim"]
        self.bs = c.get("block_size", 16)
        self.mbps = -(-c["max_seq_len"] // self.bs)
        nblk = batch * self.mbps
        self.nblk = nblk
        self.k = [np.zeros((nblk * self.bs, ekv), np.uint16) for _ in range(c["n_layers"])]
        self.v = [np.zeros((nblk * self.bs, ekv), np.uint16) for _ in range(c["n_layers"])]
        self.tables = np.arange(nblk, dtype=np.uint32).reshape(batch, self.mbps)
        self.seq = np.zeros(batch, np.int64)
        self.batch = batch

    def _row_parallel(self, x, wq, ws, h):
        """h + sum over ranks (ascending) of acc(quant_r(x_r), W_r) * (s_r * s_w); x: [M, K]."""
        tp = self.tp
        k = x.shape[1] // tp
        total = None
        for r in range(tp):
            xq, sx = self._qrow(x[:, r * k:(r + 1) * k])
            wr = np.ascontiguousarray(wq[:, r * k:(r + 1) * k])
            acc = O.gemm_fp8_f32(xq, wr) if self.fp8 else O.gemm_i8_s32(xq, wr)
            y = O.epilogue_scaled(acc, sx, True, ws, True)
            total = y if total is None else (total + y).astype(np.float32)
        return (total + h).astype(np.float32)

    def step(self, ids):
        """One token per row; returns (logits [B, V], next ids [B])."""
        c = self.cfg
        d, dh, hq, hkv, f = c["d_model"], c["head_dim"], c["n_heads"], c["n_kv_heads"], c["d_ff"]
        eps = c.get("rms_eps", 1e-5)
        b = self.batch
        ids = np.asarray(ids)
        h = self.w["embed"][ids].astype(np.float32)
        pos = self.seq.copy()
        attention = O.paged_attention_kernel_order if self.exact else O.paged_attention
        for l, (lw, lq) in enumerate(zip(self.w["layers"], self.q["layers"])):
            lb = self.blas["layers"][l] if self.blas else {}
            xn = self._norm(h, lw["attn_norm"], eps, first=(l == 0))
            xq, sx = self._qrow(xn)
            qkv = O.epilogue_scaled(self._acc(xq, lq["wqkv"], lb.get("wqkv")), sx, True, lq["wqkv"][1], True)
            q = np.empty((b, hq * dh), np.float32)
            k_new = np.empty((b, hkv * dh), np.float32)
            for r in range(b):
                q[r] = O.rope_apply(qkv[r, : hq * dh], hq, dh, self.cos[pos[r]], self.sin[pos[r]])
                k_new[r] = O.rope_apply(qkv[r, hq * dh:(hq + hkv) * dh], hkv, dh, self.cos[pos[r]], self.sin[pos[r]])
            v_new = np.ascontiguousarray(qkv[:, (hq + hkv) * dh:])
            slots = [int(self.tables[r, pos[r] // self.bs]) * self.bs + int(pos[r] % self.bs) for r in range(b)]
            O.paged_kv_append(k_new, v_new, self.k[l], self.v[l], slots, hkv * dh, True)
            a = attention(q.reshape(b, 1, -1), self.k[l], self.v[l], self.tables, pos + 1, batch=b, l_new=1,
                          num_q_heads=hq, num_kv_heads=hkv, head_dim=dh, block_size=self.bs,
                          num_blocks=self.nblk, max_blocks_per_seq=self.mbps,
                          scale=float(np.float32(1.0) / np.sqrt(np.float32(dh))), kv_bf16=True).reshape(b, -1)
            if self.exact:
                aq, sa = self._qrow(a)
                h = (O.epilogue_scaled(self._acc(aq, lq["wo"], lb["wo"]), sa, True, lq["wo"][1], True) + h).astype(np.float32)
            else:
                h = self._row_parallel(a, *lq["wo"], h)
            xn = self._norm(h, lw["mlp_norm"], eps, first=False)
            xq, sx = self._qrow(xn)
            acc = self._acc(xq, lq["wgu"], lb.get("wgu"))
            if self.exact:
                act = O.epilogue_det(acc, sx, lq["wgu"][1], act=O.ACT_SILU_GATE)
                fq, sf = self._qrow(act)
                h = (O.epilogue_scaled(self._acc(fq, lq["wdown"], lb["wdown"]), sf, True, lq["wdown"][1], True) + h).astype(np.float32)
            else:
                act = O.epilogue_scaled(acc, sx, True, lq["wgu"][1], True, act=O.ACT_SILU_GATE)
                h = self._row_parallel(act, *lq["wdown"], h)
        self.seq += 1
        xn = self._norm(h, self.w["final_norm"], eps, first=False)
        xq, sx = self._qrow(xn)
        logits = O.epilogue_scaled(self._acc(xq, self.q["lm_head"], self.blas["lm_head"] if self.blas else None), sx, True,
                                   self.q["lm_head"][1], True)
        nxt = np.argmax(logits, axis=1).astype(np.int32) if self.exact else \
            np.array([O.greedy_argmax(logits[r]) for r in range(b)], np.int32)
        return logits, nxt

    def prefill(self, ids):
        """ids [B, L]: every row consumes L tokens in one pass over B * L token rows (row m = b * L + i): the K / V of
        all of them are appended and row (b, i) attends to the keys j <= seq_len - L + i, the reference's mask rule
        (crates/backend-cpu/src/paged_kv.rs:137-140).  Nothing is sampled.  The arithmetic per token row is that of
        step(); in kernel order the launch shape of the row kernels follows the number of token rows."""
        c = self.cfg
        d, dh, hq, hkv, f = c["d_model"], c["head_dim"], c["n_heads"], c["n_kv_heads"], c["d_ff"]
        eps = c.get("rms_eps", 1e-5)
        ids = np.asarray(ids)
        b, L = ids.shape
        assert b == self.batch
        m = b * L
        h = self.w["embed"][ids.reshape(-1)].astype(np.float32)
        pos = (self.seq[:, None] + np.arange(L)[None, :]).reshape(-1)
        row_of = np.repeat(np.arange(b), L)
        attention = O.paged_attention_kernel_order if self.exact else O.paged_attention
        for l, (lw, lq) in enumerate(zip(self.w["layers"], self.q["layers"])):
            lb = self.blas["layers"][l] if self.blas else {}
            xn = self._norm(h, lw["attn_norm"], eps, first=(l == 0))
            xq, sx = self._qrow(xn)
            qkv = O.epilogue_scaled(self._acc(xq, lq["wqkv"], lb.get("wqkv")), sx, True, lq["wqkv"][1], True)
            q = np.empty((m, hq * dh), np.float32)
            k_new = np.empty((m, hkv * dh), np.float32)
            for r in range(m):
                q[r] = O.rope_apply(qkv[r, : hq * dh], hq, dh, self.cos[pos[r]], self.sin[pos[r]])
                k_new[r] = O.rope_apply(qkv[r, hq * dh:(hq + hkv) * dh], hkv, dh, self.cos[pos[r]], self.sin[pos[r]])
            v_new = np.ascontiguousarray(qkv[:, (hq + hkv) * dh:])
            slots = [int(self.tables[row_of[r], pos[r] // self.bs]) * self.bs + int(pos[r] % self.bs) for r in range(m)]
            O.paged_kv_append(k_new, v_new, self.k[l], self.v[l], slots, hkv * dh, True)
            if l + 1 == len(self.w["layers"]):
                break               # the last layer's K / V rows are in the cache: nothing else of the pass is used
            a = attention(q.reshape(b, L, -1), self.k[l], self.v[l], self.tables, self.seq + L, batch=b, l_new=L,
                          num_q_heads=hq, num_kv_heads=hkv, head_dim=dh, block_size=self.bs,
                          num_blocks=self.nblk, max_blocks_per_seq=self.mbps,
                          scale=float(np.float32(1.0) / np.sqrt(np.float32(dh))), kv_bf16=True).reshape(m, -1)
            aq, sa = self._qrow(a)
            h = (O.epilogue_scaled(self._acc(aq, lq["wo"], lb.get("wo")), sa, True, lq["wo"][1], True) + h).astype(np.float32)
            xn = self._norm(h, lw["mlp_norm"], eps, first=False)
            xq, sx = self._qrow(xn)
            acc = self._acc(xq, lq["wgu"], lb.get("wgu"))
            if self.exact:
                act = O.epilogue_det(acc, sx, lq["wgu"][1], act=O.ACT_SILU_GATE)
            else:
                act = O.epilogue_scaled(acc, sx, True, lq["wgu"][1], True, act=O.ACT_SILU_GATE)
            fq, sf = self._qrow(act)
            h = (O.epilogue_scaled(self._acc(fq, lq["wdown"], lb.get("wdown")), sf, True, lq["wdown"][1], True) + h).astype(np.float32)
        self.seq += L

    def generate(self, prompt, max_length: int):
        """Greedy generate: returns (ids [B, max_length], logits of every step that sampled a token)."""
        prompt = np.asarray(prompt, np.int32)
        b, t = prompt.shape
        self.begin(b)
        out = np.zeros((b, max_length), np.int32)
        out[:, :t] = prompt
        all_logits = []
        for step in range(max_length - 1):
            logits, nxt = self.step(out[:, step])
            if step >= t - 1:
                out[:, step + 1] = nxt
                all_logits.append(logits)
        return out, all_logits
