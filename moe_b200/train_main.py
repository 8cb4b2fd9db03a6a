"""Pretraining entry point (`train.py` of the reference, `:330-709`), without Accelerate.

    python train.py --config configs/scaling/xs_standard.yaml [--resume DIR | --auto_resume]
                    [--data_dir D] [--output_dir O] [--max_checkpoints N] [--seed S] [--device cpu|cuda]

One process per GPU (launch with torchrun or `scripts/train.sh`); `--device cpu` runs the
plain-PyTorch path with the gloo backend.  Flags, YAML schema, stdout line, metric keys and the
`checkpoint-N/` + `meta.json` layout follow the reference.  The configured `max_steps` /
`warmup_steps` are optimizer steps (the reference multiplies both by the number of processes).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import yaml

from .models import build_model, load_config
from .models.load_balancing import seq_load_balancing_loss_func
from .trainer import Trainer
from .utils.bias_update import bias_alpha_schedule, get_selected_experts_for_seq_aux, update_expert_biases
from .utils.checkpoint import (cleanup_checkpoints, find_latest_checkpoint, load_checkpoint, read_meta,
                               save_checkpoint)
from .utils.logging import MetricsLogger, format_step_line, rank_banner
from .utils.routing_stats import accumulate_expert_counts, compute_routing_stats
from .utils.training import TrainingConfig, count_parameters
from .utils.watchdog import StepWatchdog

_DATA_KEYS = {"data_dir", "text_column", "seq_len", "tokenizer_name", "num_workers", "source", "seed",
              "reference_double_shift", "prefetch"}
_PARALLEL_KEYS = {"mode", "ep_size", "bucket_mb", "overlap", "cuda_graph"}
_TOP_KEYS = {"experiment_name", "model", "training", "data", "checkpoint", "parallel"}


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--config", required=True)
    p.add_argument("--resume", default=None, help="Path to checkpoint directory")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--auto_resume", action="store_true", help="Resume from the newest checkpoint in output_dir")
    p.add_argument("--data_dir", default=None, help="Override data.data_dir")
    p.add_argument("--output_dir", default=None, help="Override training.output_dir")
    p.add_argument("--max_checkpoints", type=int, default=0, help="Checkpoints to keep (0 = all)")
    p.add_argument("--device", default=None, choices=["cpu", "cuda"], help="default: cuda when available")
    p.add_argument("--max_steps", type=int, default=None, help="Override training.max_steps")
    p.add_argument("--parallel_mode", default=None, choices=["ddp", "zero", "fsdp"],
                   help="Override parallel.mode (the reference picks between its DDP and FSDP launcher files)")
    p.add_argument("--profile", action="store_true",
                   help="NVTX ranges per step and per phase (attn, moe, lce, comm); runs eagerly, without the CUDA graph")
    return p.parse_args(argv)


def validate_config(cfg: dict) -> None:
    unknown = set(cfg) - _TOP_KEYS
    if unknown:
        raise ValueError(f"unknown top-level config keys: {sorted(unknown)}")
    bad = set(cfg.get("data", {})) - _DATA_KEYS
    if bad:
        raise ValueError(f"unknown data config keys: {sorted(bad)}")
    bad = set(cfg.get("parallel", {})) - _PARALLEL_KEYS
    if bad:
        raise ValueError(f"unknown parallel config keys: {sorted(bad)}")


def init_distributed(device: str) -> tuple[int, int, int]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device == "cuda":
        torch.cuda.set_device(local)  # before any NCCL work
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device == "cuda":
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    return rank, local, world


def build_dataset(dcfg: dict, vocab: int, rank: int, world: int):
    source = dcfg.get("source", "parquet")
    if source == "synthetic":
        from .data import SyntheticConfig, SyntheticTokenDataset

        return SyntheticTokenDataset(SyntheticConfig(vocab_size=vocab, seq_len=dcfg.get("seq_len", 2048),
                                                     seed=dcfg.get("seed", 0)), rank, world)
    from transformers import AutoTokenizer

    from .data import DataConfig, StatefulParquetDataset

    tok = AutoTokenizer.from_pretrained(dcfg.get("tokenizer_name", "gpt2"))
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    dc = DataConfig(data_dir=dcfg["data_dir"], text_column=dcfg.get("text_column", "text"),
                    seq_len=dcfg.get("seq_len", 2048), tokenizer_name=dcfg.get("tokenizer_name", "gpt2"),
                    num_workers=dcfg.get("num_workers", 4),
                    reference_double_shift=dcfg.get("reference_double_shift", False),
                    prefetch=dcfg.get("prefetch", 2 if dcfg.get("num_workers", 0) else 0))
    return StatefulParquetDataset(dc, tok, rank=rank, world_size=world)


class BatchIterator:
    """Stacks `batch_size` samples into pinned `[B, S]` tensors; restarts the dataset when exhausted."""

    def __init__(self, dataset, batch_size: int, pin: bool):
        self.dataset, self.bs, self.pin = dataset, batch_size, pin
        self.it = iter(dataset)

    def next(self) -> dict:
        ids, labels = [], []
        while len(ids) < self.bs:
            try:
                s = next(self.it)
            except StopIteration:
                self.it = iter(self.dataset)
                continue
            ids.append(s["input_ids"])
            labels.append(s["labels"])
        out = {"input_ids": torch.stack(ids), "labels": torch.stack(labels)}
        if self.pin:
            out = {k: v.pin_memory() for k, v in out.items()}
        return out


def main(argv=None) -> None:
    args = parse_args(argv)
    cfg = load_config(args.config)
    validate_config(cfg)
    tdict = dict(cfg["training"])
    ddict = dict(cfg.get("data", {}))
    if args.data_dir:
        ddict["data_dir"] = args.data_dir
    if args.output_dir:
        tdict["output_dir"] = args.output_dir
    if args.max_steps is not None:
        tdict["max_steps"] = args.max_steps
    tcfg = TrainingConfig.from_dict(tdict)
    if args.parallel_mode:
        cfg.setdefault("parallel", {})["mode"] = args.parallel_mode
    resume_from = args.resume or cfg.get("checkpoint", {}).get("resume_from")
    if args.auto_resume and not resume_from:
        resume_from = find_latest_checkpoint(tcfg.output_dir)
    wandb_run_id = read_meta(resume_from).get("wandb_run_id") if resume_from else None

    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    rank, local, world = init_distributed(device)
    dev = torch.device("cuda", local) if device == "cuda" else torch.device("cpu")
    main_proc = rank == 0
    print(rank_banner(rank, local, world, dev), flush=True)
    if resume_from and main_proc:
        print(f"Will resume from: {resume_from}")

    mtype = cfg["model"]["type"]
    is_dense = mtype == "dense"
    is_global = mtype in ("global_moe", "deepseek_global_moe")
    # every rank builds identical weights from --seed (the reference reaches the same state through
    # DDP's initial broadcast of rank 0's weights); the data / dropout RNG is seeded per rank
    pcfg0 = cfg.get("parallel", {})
    ep_size = int(pcfg0.get("ep_size", 1) or 1)
    if ep_size < 0:
        ep_size = world
    if ep_size > 1 and (device != "cuda" or ep_size != world):
        raise ValueError("parallel.ep_size must be 1, -1 or the number of ranks, and needs CUDA")
    model, mcfg = build_model(cfg, seed=args.seed, device=dev, ep=(rank, ep_size) if ep_size > 1 else None)
    torch.manual_seed(args.seed + rank)
    params = count_parameters(model)
    expert_params = sum(p.numel() for n, p in model.named_parameters() if "gate_up_proj" in n or "down_proj" in n)
    bias_rate = cfg["model"].get("bias_update_rate", 0.0) or 0.0
    bias_interp = cfg["model"].get("bias_interpolation", False)
    seq_coef = cfg["model"].get("seq_aux_loss_coef", 0.0) or 0.0
    pcfg = cfg.get("parallel", {})
    # "ddp": everything replicated; "zero": Adam moments and the update sharded over the ranks (ZeRO-1), new bf16
    # weights stored to every rank by the update kernel; "fsdp": parameters, gradients and optimizer state
    # sharded, each layer's weights pulled from the peers right before use (ZeRO-3)
    # Defaults are what `bench.py` measures: sharded optimizer on more than one GPU, whole-step CUDA graph.
    pmode = str(pcfg.get("mode", "zero" if (world > 1 and device == "cuda") else "ddp")).lower()
    if pmode not in ("ddp", "zero", "fsdp"):
        raise ValueError(f"parallel.mode={pcfg.get('mode')!r}: expected ddp, zero or fsdp")
    shard_opt = pmode == "zero" and world > 1 and device == "cuda"
    shard_par = pmode == "fsdp" and device == "cuda"
    if pmode == "fsdp" and device != "cuda":
        raise ValueError("parallel.mode: fsdp needs CUDA (parameters are pulled over NVLink peer memory)")
    use_graph = bool(pcfg.get("cuda_graph", True)) and device == "cuda" and not args.profile
    if main_proc:
        print(f"\n{'=' * 60}\n  Model     : {mtype}\n  Params    : {params['total'] / 1e9:.3f}B total  |  "
              f"{expert_params / 1e9:.3f}B expert\n  Dist type : {('FSDP (ZeRO-3)' if shard_par else 'ZeRO-1' if shard_opt else 'DDP') if world > 1 else 'single'} ({device})\n"
              f"  Precision : {'bf16 compute, fp32 master' if device == 'cuda' else 'fp32'}\n  GPUs      : {world}\n"
              f"{'=' * 60}\n", flush=True)

    if args.profile:
        from .utils import profiling

        profiling.enable()
    trainer = Trainer(model, tcfg, is_moe=not is_dense, overlap_grad_reduce=pcfg.get("overlap", True),
                      shard_optimizer=shard_opt, shard_params=shard_par, cuda_graph=use_graph)
    trainer.engine.broadcast_parameters(0)
    dataset = build_dataset(ddict, cfg["model"]["vocab_size"], rank, world)
    if resume_from:
        step, ds_state = load_checkpoint(trainer, resume_from)
        if main_proc:
            print(f"Resumed from step {step}")
        if ds_state:
            dataset.set_state(ds_state)
    batches = BatchIterator(dataset, tcfg.batch_size, pin=device == "cuda")
    logger = MetricsLogger(tcfg.output_dir, tcfg.wandb_project, tcfg.wandb_run_name, wandb_run_id,
                           config={**cfg["model"], **tdict}, enabled=main_proc)
    wandb_run_id = logger.run_id or wandb_run_id
    os.makedirs(tcfg.output_dir, exist_ok=True)
    watchdog = StepWatchdog(factor=20.0, min_seconds=120.0).start()
    t0 = time.perf_counter()
    tokens_seen = 0
    count_accum = None
    if main_proc:
        print(f"Starting training from step {trainer.global_step}", flush=True)
    use_events = device == "cuda"

    while trainer.global_step < tcfg.max_steps:
        micro = [batches.next() for _ in range(tcfg.gradient_accumulation)]
        if use_events:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if args.profile and use_events:
            torch.cuda.nvtx.range_push(f"step{trainer.global_step}")
        res = trainer.train_step(micro)
        if args.profile and use_events:
            torch.cuda.nvtx.range_pop()
        step_before = trainer.global_step - 1
        bias_stats = {}
        if bias_rate > 0:
            alpha = bias_alpha_schedule(step_before) if (is_global and bias_interp) else 0.0
            bias_stats = update_expert_biases(model, bias_rate, None, is_global=is_global, alpha=alpha)
            bias_stats["routing/bias_alpha"] = alpha
        if use_events:
            ev1.record()
        gstep = trainer.global_step
        tokens_seen += res.tokens  # all micro-batches of all ranks (the reference counts one micro-batch)
        watchdog.beat()

        if gstep % tcfg.log_every == 0:
            step_ms = None
            if use_events:
                ev1.synchronize()
                t_ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
                if world > 1:
                    dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
                step_ms = float(t_ms.item())
            if main_proc:
                vals = torch.stack([res.loss.float(), _z(res.aux_loss, dev), _z(res.seq_aux_loss, dev),
                                    res.grad_norm.float().reshape(())]).cpu().tolist()
                total, aux, seq_aux, gn = vals
                ce = total - getattr(model, "router_aux_loss_coef", 0.0) * aux - seq_coef * seq_aux
                elapsed = time.perf_counter() - t0
                tps = tokens_seen / elapsed
                log = {"train/ce_loss": ce, "train/aux_loss": aux, "train/seq_aux_loss": seq_aux,
                       "train/grad_norm": gn, "train/lr": res.lr, "train/tokens_per_sec": tps,
                       "train/tokens_seen_B": tokens_seen / 1e9}
                if step_ms is not None:
                    log["train/step_ms_max"] = step_ms
                    log["train/tokens_per_sec_device"] = res.tokens / (step_ms / 1e3)
                print(format_step_line(gstep, total, ce, aux, seq_aux, res.lr, tps, gn), flush=True)
                log.update(bias_stats)
                logger.log(log, gstep)

        if res.router_logits is not None:
            if res.router_stats is not None:  # the router kernels already counted
                c = res.router_stats.expert_counts()
                count_accum = {l: (count_accum[l] + c[l] if count_accum else c[l].clone()) for l in range(c.shape[0])}
            else:
                sel = get_selected_experts_for_seq_aux(model) if mtype.startswith("deepseek") is False else None
                count_accum = accumulate_expert_counts(res.router_logits, mcfg.num_experts_per_tok, count_accum,
                                                       selected_experts=sel)
            if gstep % tcfg.routing_log_every == 0:
                _routing_snapshot(res, count_accum, mcfg, is_global, tcfg, gstep, world, main_proc, logger)
                count_accum = None

        if gstep % tcfg.save_every == 0:
            save_checkpoint(trainer, gstep, tcfg.output_dir, dataset.get_state(), wandb_run_id)
            if args.max_checkpoints > 0 and main_proc:
                cleanup_checkpoints(tcfg.output_dir, args.max_checkpoints)

    save_checkpoint(trainer, trainer.global_step, tcfg.output_dir, dataset.get_state(), wandb_run_id)
    if args.max_checkpoints > 0 and main_proc:
        cleanup_checkpoints(tcfg.output_dir, args.max_checkpoints)
    watchdog.stop()
    logger.close()
    if device == "cuda":
        from .ops import gemm as G

        G.check_status()
    if main_proc:
        print("Training complete.", flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def _z(t, dev):
    return t.float().reshape(()) if isinstance(t, torch.Tensor) else torch.zeros((), device=dev)


def _routing_snapshot(res, count_accum, mcfg, is_global, tcfg, gstep, world, main_proc, logger) -> None:
    """All-reduce the accumulated per-layer counts in one [L, E] tensor, then rank 0 writes the stats,
    the JSON snapshot and (when a rasteriser is available) the PNG plots."""
    from .utils.routing_plots import plot_routing_snapshot

    keys = sorted(count_accum)
    if world > 1 and keys:
        stacked = torch.stack([count_accum[k] for k in keys])
        dist.all_reduce(stacked, op=dist.ReduceOp.SUM)
        for k, row in zip(keys, stacked.unbind(0)):
            count_accum[k] = row
    hs = res.router_stats
    # statistics of the last micro-batch of every rank, summed over the ranks (a collective)
    rstats = compute_routing_stats(res.router_logits, mcfg.num_experts_per_tok, is_global=is_global,
                                   counts=None if hs is None else hs.expert_counts(),
                                   margins=None if hs is None else hs.margin, reduce_ranks=world > 1)
    if not main_proc:
        return
    logger.log({k: v for k, v in rstats.items() if not k.startswith("_hist/")}, gstep)
    rdir = os.path.join(tcfg.output_dir, "routing_logs")
    os.makedirs(rdir, exist_ok=True)
    snap = {"step": gstep, "layers": {}, "global_pool": None}
    mat = torch.stack([count_accum[k] for k in keys]).cpu() if keys else None
    for i, k in enumerate(keys):
        c = mat[i]
        tot = float(c.sum())
        snap["layers"][k] = {"token_counts": c.tolist(),
                             "token_fracs": (c / tot).tolist() if tot > 0 else [0.0] * c.numel()}
    if is_global and len(keys) > 1:
        pool = mat.sum(0)
        ptot = float(pool.sum())
        snap["global_pool"] = {"token_counts": pool.tolist(), "token_fracs": (pool / ptot).tolist() if ptot > 0 else [],
                               "layer_usage_count": (mat > 0).float().sum(0).tolist(), "num_layers": mat.shape[0]}
    with open(os.path.join(rdir, f"step_{gstep:08d}.json"), "w") as f:
        json.dump(snap, f)
    plot_routing_snapshot(snap, rdir, gstep)


if __name__ == "__main__":
    main()
