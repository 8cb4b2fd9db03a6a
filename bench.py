#!/usr/bin/env python
"""Headline benchmark: whole-job training tokens/s of the XS standard MoE (bf16) on N B200s.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference stack, same metric

A step is one optimizer step: forward, backward, gradient average over ranks, clip, AdamW.
Two timed regions of K steps each (CUDA events, barrier + synchronize on both sides, max over ranks):
  * `value`: inputs already on the device, no host read-back inside the region;
  * `e2e`  : through `Trainer.train_step`, each step copying its inputs from pinned host memory
             and reading the loss back to the host.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKS = None  # the reference publishes no throughput for a named config


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="xs_standard", help="name under configs/bench/")
    ap.add_argument("--batch", type=int, default=None, help="override per-GPU micro-batch")
    ap.add_argument("--seq", type=int, default=None, help="override sequence length")
    ap.add_argument("--no-overlap", action="store_true", help="reduce gradients after backward, not during")
    ap.add_argument("--ep", action="store_true", help="shard the experts over all ranks (expert parallelism)")
    ap.add_argument("--no-ep", action="store_true", help="keep every expert on every rank even if the config shards them")
    ap.add_argument("--ep-local", action="store_true",
                    help="diagnostic, one GPU: run the expert-parallel code path with a single rank (every row is "
                         "'sent' to the rank itself), which isolates the local cost of that path")
    ap.add_argument("--no-zero", action="store_true",
                    help="replicate Adam moments and the update on every rank (default for N > 1: sharded, ZeRO-1)")
    ap.add_argument("--fsdp", action="store_true",
                    help="shard parameters, gradients and optimizer state (ZeRO-3) instead of ZeRO-1")
    ap.add_argument("--stub-comm", action="store_true",
                    help="measurement aid: every rank talks to its own buffers (no NVLink traffic, no waits); "
                         "step time minus this run's step time is the exposed communication")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timed regions: one more eager step with CUDA-event marks around the bucket "
                         "reduces, AdamW and the parameter barrier on every rank (printed under `timeline`)")
    ap.add_argument("--layers", type=int, default=None, help="override num_hidden_layers (shape debugging only)")
    ap.add_argument("--checkpoint", action="store_true", help="recompute each decoder layer in backward")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly (no whole-step CUDA graph)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of this rank's GPU while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = f"/tmp/bench_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=self.fh,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx = float(f[2])
                except ValueError:
                    continue
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


def dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return rank, local, world


def timed_region(fn, steps: int, world: int, local: int):
    """Barrier + synchronize, K calls of fn(i) between CUDA events, synchronize; max over ranks (ms)."""
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = torch.tensor([s.elapsed_time(e)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item(), clocks


def load_bench_config(name: str, batch, seq) -> dict:
    import yaml

    with open(os.path.join(ROOT, "configs", "bench", f"{name}.yaml")) as f:
        cfg = yaml.safe_load(f)
    if batch:
        cfg["training"]["batch_size"] = batch
    if seq:
        cfg["data"]["seq_len"] = seq
    return cfg


def make_batches(n: int, batch: int, seq: int, vocab: int, rank: int, seed: int):
    """Uniform-random token ids in pinned host memory, a different batch per step and rank."""
    import torch

    g = torch.Generator().manual_seed(seed * 1000 + rank)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (batch, seq), generator=g, dtype=torch.int64)
        out.append(ids.pin_memory())
    return out


def run_ours(args) -> dict:
    import torch

    from moe_b200.models import build_model
    from moe_b200.ops import _ext
    from moe_b200.ops import gemm as G
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    if args.stub_comm:
        os.environ["MOE_B200_COMM_STUB"] = "1"
    rank, local, world = dist_setup(args.gpus)
    cfg = load_bench_config(args.config, args.batch, args.seq)
    if args.checkpoint:
        cfg["training"]["gradient_checkpointing"] = True
    if args.layers:
        cfg["model"]["num_hidden_layers"] = args.layers
    tcfg = TrainingConfig.from_dict(cfg["training"])
    B, S = tcfg.batch_size, cfg["data"]["seq_len"]
    V = cfg["model"]["vocab_size"]
    ep_size = int(cfg.get("parallel", {}).get("ep_size", 1) or 1)
    if ep_size < 0 or args.ep:
        ep_size = world
    if args.no_ep:
        ep_size = 1
    ep = (rank % ep_size, ep_size) if ep_size > 1 else None
    if ep is not None and ep_size != world:
        raise SystemExit("bench.py runs expert parallelism over all ranks (ep_size == number of GPUs)")
    model, mcfg = build_model(cfg, seed=42, device=f"cuda:{local}", ep=ep)
    trainer = Trainer(model, tcfg, is_moe=cfg["model"]["type"] != "dense", overlap_grad_reduce=not args.no_overlap,
                      cuda_graph=not args.no_graph,
                      shard_optimizer=(not args.no_zero) and world > 1 and not args.fsdp, shard_params=args.fsdp)
    if args.ep_local:
        if world != 1:
            raise SystemExit("--ep-local is a one-GPU diagnostic")
        import torch.distributed as dist

        from moe_b200.parallel.ep import EPContext

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local))
        trainer.ep = EPContext(model.config.num_experts, None, trainer.device)
        for name, p in model.named_parameters():
            if name.endswith("gate_up_proj"):
                p._ep = trainer.ep
        trainer.engine.end_step_hooks.append(trainer.ep.end_step)
    n_params = sum(p.numel() * (ep_size if getattr(p, "_ep_shard", None) else 1) for p in model.parameters())
    K, W = args.steps, args.warmup
    host = make_batches(W + 2 * K, B, S, V, rank, cfg["data"].get("seed", 0))
    # ---- warm-up (untimed); with the CUDA graph on, the first two steps run eagerly, the third captures
    for i in range(W):
        r = trainer.train_step({"input_ids": host[i], "labels": host[i]})
    torch.cuda.synchronize()
    # ---- region 1: device-resident inputs, no host read-back
    dev_batches = [b.cuda(non_blocking=True) for b in host[W:W + K]]
    torch.cuda.synchronize()
    l0 = _ext.launch_count()
    last = {}

    def step_dev(i):
        last["r"] = trainer.train_step({"input_ids": dev_batches[i], "labels": dev_batches[i]})

    ms, clocks = timed_region(step_dev, K, world, local)
    launches = _ext.launch_count() - l0
    loss_dev = float(last["r"].loss.item())
    # ---- region 2: end to end through the public API (H2D of inputs + D2H of the loss every step)
    losses = []

    def step_e2e(i):
        b = host[W + K + i]
        r = trainer.train_step({"input_ids": b, "labels": b})
        losses.append(float(r.loss.item()))

    ms_e2e, clocks_e2e = timed_region(step_e2e, K, world, local)
    G.check_status()
    timeline = None
    if args.timeline:
        import torch.distributed as dist

        trainer.use_graph = False
        b = host[W]
        trainer.train_step({"input_ids": b, "labels": b})  # eager path warm
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        trainer.engine.start_timeline()
        trainer.train_step({"input_ids": b, "labels": b})
        mine = trainer.engine.timeline_report()
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, mine)
        else:
            gathered = [mine]
        timeline = {f"rank{r}": t for r, t in enumerate(gathered)}
    tokens = B * S * world * K
    value = tokens / (ms / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    par = f"dp{world}" + (f"+ep{ep_size}" if ep else "")
    if getattr(trainer.engine, "sharded_params", False):
        par += ", parameters, gradients and Adam state sharded over the ranks (ZeRO-3)"
    elif trainer.engine.sharded:
        par += ", Adam state and update sharded over the ranks (ZeRO-1)"
    return {
        "metric": "train_tokens_per_sec", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / BASELINE_TOKS) if BASELINE_TOKS else None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{args.config} ({cfg['model']['type']}, H{mcfg.hidden_size} L{mcfg.num_hidden_layers} "
                            f"E{getattr(mcfg, 'num_experts', 0)} top{getattr(mcfg, 'num_experts_per_tok', 0)})",
                   "params": n_params, "global_batch": B * world, "micro_batch_per_gpu": B, "seq_len": S,
                   "parallelism": par, "optimizer": "AdamW, clip 1.0, warmup+cosine",
                   "activation_checkpointing": bool(tcfg.gradient_checkpointing),
                   "l2": "per-step working set (GBs of weights and activations, 1.2 GB of logits per chunk) is far larger than "
                         "the 126 MB L2; no explicit flush"},
        "e2e": {"value": e2e, "unit": "tok/s", "ms_per_step": ms_e2e / K, "h2d_bytes_per_step": B * S * 8,
                "d2h_bytes_per_step": 4, "clocks": clocks_e2e},
        "gpu_launches": launches, "clocks": clocks, "loss_last": loss_dev, "loss_e2e_last": losses[-1],
        **({"comm_stubbed": True} if args.stub_comm else {}), **({"timeline": timeline} if timeline else {}),
        # rank 0's loss of every end-to-end step (same synthetic token stream in both arms)
        "losses_e2e": [round(x, 4) for x in losses[:256]],
    }


def run_reference(args) -> dict:
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "src")):
        return {"impl": "reference", "unavailable": "baseline/_ref is missing (reference not installed on this box)"}
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import run_reference as rr

    return rr.run(args, ROOT, dist_setup, timed_region, make_batches, load_bench_config)


def main():
    args = parse_args()
    try:
        res = run_ours(args) if args.impl == "ours" else run_reference(args)
    except SystemExit:
        raise
    except Exception as e:  # a failed reference arm must still exit 0 with its one line
        if args.impl == "reference":
            res = {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
        else:
            raise
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(res), flush=True)
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
