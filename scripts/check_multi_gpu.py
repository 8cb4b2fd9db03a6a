#!/usr/bin/env python
"""Equivalence of the parallel modes on N GPUs of one node (launch with torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        scripts/check_multi_gpu.py [--out result.json]

A small model is trained for a few steps on the same global batch under: replicated weights with the library
all-reduce (the yardstick), the own peer-memory all-reduce, the sharded optimizer (ZeRO-1), sharded parameters
(ZeRO-3), and expert parallelism over all ranks (alone, with ZeRO-1, with recomputation).  Losses and gradient
norms of every variant must follow the yardstick, full master weights too where they can be assembled, and the
ranks must agree bit for bit.  Rank 0 prints one JSON line (and writes it to --out); exit code 1 on a mismatch.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def cfg(mtype: str, experts: int) -> dict:
    m = dict(type=mtype, vocab_size=2048, hidden_size=256, num_hidden_layers=3, head_dim=128, num_attention_heads=4,
             num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False, num_experts=experts,
             num_experts_per_tok=2, moe_intermediate_size=128, router_aux_loss_coef=0.01)
    return {"model": m}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from moe_b200.models import build_model
    from moe_b200.ops import gemm as G
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    tcfg = TrainingConfig(learning_rate=1e-3, warmup_steps=0, max_steps=10, batch_size=2, gradient_accumulation=1,
                          lr_scheduler="constant")
    g = torch.Generator().manual_seed(0)
    data = [torch.randint(0, 2048, (2 * world, 128), generator=g) for _ in range(a.steps)]
    variants = [("replicated-nccl", dict(comm="nccl", overlap_grad_reduce=False), False, False),
                ("replicated-peer", dict(comm="p2p"), False, False),
                ("zero1", dict(comm="p2p", shard_optimizer=True), False, False),
                ("fsdp", dict(shard_params=True), False, False),
                ("ep", dict(comm="p2p", overlap_grad_reduce=False), True, False),
                ("ep+zero1+recompute", dict(comm="p2p", overlap_grad_reduce=False, shard_optimizer=True), True, True)]
    report, ok = {}, True
    for mtype in ("standard_moe", "global_moe"):
        experts = max(8, world) if mtype == "standard_moe" else 2 * max(8, world)
        ref = None
        for name, kw, ep, ckpt in variants:
            model, _ = build_model(cfg(mtype, experts), seed=5, device=f"cuda:{local}", ep=(rank, world) if ep else None)
            tr = Trainer(model, dataclasses.replace(tcfg, gradient_checkpointing=ckpt), **kw)
            losses, norms = [], []
            for b in data:
                mine = b[rank * 2:(rank + 1) * 2]
                r = tr.train_step({"input_ids": mine, "labels": mine})
                # the yardstick's loss is per rank; compare the mean over ranks
                l = r.ce_loss.detach().float().clone()
                dist.all_reduce(l)
                losses.append(float(l) / world)
                norms.append(float(r.grad_norm))
            torch.cuda.synchronize()
            G.check_status()
            full = None if ep else tr.engine.full_master().detach().clone()
            if full is not None:  # ranks agree bit for bit
                other = full.clone()
                dist.broadcast(other, src=0)
                same = bool(torch.equal(other, full))
                flag = torch.tensor([int(same)], device=full.device)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                ok &= bool(flag.item())
            ent = {"ce": [round(x, 5) for x in losses], "grad_norm": [round(x, 5) for x in norms]}
            if ref is None:
                ref = (losses, norms, full)
            else:
                ent["max_rel_ce_diff"] = max(abs(x - y) / abs(y) for x, y in zip(losses, ref[0]))
                ent["max_rel_norm_diff"] = max(abs(x - y) / abs(y) for x, y in zip(norms, ref[1]))
                good = ent["max_rel_ce_diff"] < 1e-2 and ent["max_rel_norm_diff"] < 5e-2
                if full is not None and ref[2] is not None:
                    d = (full - ref[2]).abs()
                    ent["weights_max_abs_diff"] = float(d.max())
                    ent["weights_frac_gt_2e-4"] = float((d > 2e-4).float().mean())
                    good &= ent["weights_max_abs_diff"] < 5e-3 and ent["weights_frac_gt_2e-4"] < 2e-2
                ent["ok"] = bool(good)
                ok &= good
            report[f"{mtype}/{name}"] = ent
            del tr, model
            dist.barrier()
    out = {"world": world, "ok": bool(ok), "variants": report}
    if rank == 0:
        print(json.dumps(out), flush=True)
        if a.out:
            os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
            with open(a.out, "w") as f:
                json.dump(out, f, indent=1)
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
