"""Worker of the tensor-parallel GPU test: launched once per rank by torch.distributed.run.

Every rank builds the same full weights, keeps its shard inside a tensor-parallel decoder, and the ranks
decode a few tokens together.  Rank 0 compares the logits of every step with the CPU decoder restatement run
with the same tensor-parallel degree (per-rank activation scales at the row-parallel projections), and with
a single-GPU decoder for reference.  Prints one line starting with TP_OK or TP_FAIL."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def main():
    import torch.distributed as dist

    from fandhe_ai_b200 import Backend
    from fandhe_ai_b200.decoder import Decoder, DecoderConfig, nccl_unique_id
    from oracle import oracle as O
    from oracle.decoder_ref import DecoderRef, make_weights

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if os.environ.get("B200_TP_EXACT") == "1":
        return exact_mode(dist, rank, world, local)
    cfg = dict(n_layers=2, d_model=512, n_heads=8, n_kv_heads=4, head_dim=128, d_ff=1024, vocab=2048, max_seq_len=48)
    weights = make_weights(cfg, seed=5)
    batch, steps = 4, 10
    be = Backend(local)
    fp8 = os.environ.get("B200_TP_FP8") == "1"      # the FP8 x FP8 form of the decoder under tensor parallelism
    dc = DecoderConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                       cfg["vocab"], max_batch=batch, max_seq_len=cfg["max_seq_len"], tp_rank=rank, tp_size=world,
                       act_fp8=1 if fp8 else 0)
    dec = Decoder(be, dc)
    obj = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(obj, src=0)
    dec.init_tp(obj[0])
    dec.load_weights(weights)
    dec.begin(batch, [steps + 1] * batch)
    rng = np.random.default_rng(9)
    all_ids = rng.integers(0, cfg["vocab"], (steps, batch)).astype(np.int32)
    got = []
    for t in range(steps):
        dec.step(all_ids[t])
        got.append(dec.logits())
    exchange = dec.tp_exchange_mode   # 2: scattered by the GEMMs, 1: pulled by the finish kernel, 0: ncclAllReduce
    dec.close()
    ok, msg = True, ""
    if rank == 0:
        ref = DecoderRef(cfg, weights, tp=world, fp8=fp8)
        ref.begin(batch)
        worst = 0.0
        for t in range(steps):
            lr, _ = ref.step(all_ids[t])
            worst = max(worst, float(np.abs(got[t] - lr).max() / np.abs(lr).max()))
            if not np.all(np.isfinite(got[t])):
                ok = False
        # the cross-rank f32 sum may run in another order (NCCL's) and a last-bit difference can flip an int8 code
        # downstream (1/127 of a row maximum), so the bound is quantisation noise, not 1e-3
        if worst > (4e-2 if fp8 else 2e-2):     # one E4M3 code is a far larger step than one int8 code
            ok = False
        msg = f"exchange={int(exchange)} worst |dlogit| / max|logit| vs the CPU decoder at tp={world}: {worst:.3e}"
    be.close()
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    if rank == 0:
        print(("TP_OK " if ok else "TP_FAIL ") + msg, flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


def exact_mode(dist, rank, world, local):
    """tp_exact_int8: rows split over the ranks are quantised under one scale (row maximum merged over the ranks) and the
    int32 partial sums are all-reduced, so the logits must be those of ONE GPU, bit for bit: compared with the
    kernel-order CPU decoder without any tensor parallelism (head_dim 64: the general attention kernel)."""
    from fandhe_ai_b200 import Backend
    from fandhe_ai_b200.decoder import Decoder, DecoderConfig, nccl_unique_id
    from oracle.decoder_ref import DecoderRef, make_weights

    cfg = dict(n_layers=2, d_model=512, n_heads=8, n_kv_heads=4, head_dim=64, d_ff=1024, vocab=2048, max_seq_len=48)
    weights = make_weights(cfg, seed=15)
    batch, steps = 4, 10
    be = Backend(local)
    dc = DecoderConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                       cfg["vocab"], max_batch=batch, max_seq_len=cfg["max_seq_len"], tp_rank=rank, tp_size=world,
                       tp_exact_int8=1)
    dec = Decoder(be, dc)
    obj = [nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(obj, src=0)
    dec.init_tp(obj[0])
    dec.load_weights(weights)
    prompt = np.random.default_rng(19).integers(0, cfg["vocab"], (batch, 5)).astype(np.int32)
    got_ids = dec.generate(prompt, 5 + steps)
    got_logits = dec.logits()
    dec.close()
    be.close()
    ok, msg = True, ""
    if rank == 0:
        want_ids, logits = DecoderRef(cfg, weights, exact=True).generate(prompt, 5 + steps)
        ok = bool(np.array_equal(got_ids, want_ids) and np.array_equal(got_logits, logits[-1]))
        msg = f"exact tp={world}: ids equal {np.array_equal(got_ids, want_ids)}, last logits max |d| {float(np.abs(got_logits - logits[-1]).max()):.3e}"
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    if rank == 0:
        print(("TP_OK " if ok else "TP_FAIL ") + msg, flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
