"""Checkpoints: `output_dir/checkpoint-{step}/` with `meta.json`, newest-first discovery and
keep-last-N pruning (`train.py:254-323` of the reference).

Inside a checkpoint directory: `model.safetensors` (HF parameter names, fp32 masters; buffers such
as `expert_bias` included), `optimizer.bin` (AdamW moments by parameter name + step),
`scheduler.bin`, `random_states_{rank}.pkl` (per-rank RNG) and `dataset_state_{rank}.json`
(per-rank data position).  `meta.json` = `{step, dataset_state (rank 0's), wandb_run_id, world_size}`.
A save goes to `checkpoint-{step}.tmp` and is renamed when complete, so an interrupted save never
shadows the previous checkpoint.  State is stored by name, not by rank, so a run can resume on a
different number of data-parallel ranks.
"""
from __future__ import annotations

import json
import os
import pickle
import random
import re
import shutil

import numpy as np
import torch
import torch.distributed as dist

_PAT = re.compile(r"^checkpoint-(\d+)$")


def _list(output_dir: str) -> list[tuple[int, str]]:
    out = []
    if not os.path.isdir(output_dir):
        return out
    for entry in os.listdir(output_dir):
        m = _PAT.match(entry)
        path = os.path.join(output_dir, entry)
        if m and os.path.isdir(path):
            out.append((int(m.group(1)), path))
    out.sort(key=lambda x: x[0])
    return out


def find_latest_checkpoint(output_dir: str) -> str | None:
    c = _list(output_dir)
    return c[-1][1] if c else None


def cleanup_checkpoints(output_dir: str, max_keep: int) -> None:
    if max_keep <= 0:
        return
    c = _list(output_dir)
    while len(c) > max_keep:
        _, path = c.pop(0)
        shutil.rmtree(path)


def _rank_world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _rng_state() -> dict:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def _set_rng_state(st: dict) -> None:
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def save_checkpoint(trainer, step: int, output_dir: str, dataset_state: dict | None = None,
                    wandb_run_id: str | None = None, scheduler_state: dict | None = None) -> str:
    """All ranks call this.  Rank 0 writes the shared files; every rank writes its RNG and data state."""
    from safetensors.torch import save_file

    rank, world = _rank_world()
    final = os.path.join(output_dir, f"checkpoint-{step}")
    tmp = final + ".tmp"
    if rank == 0:
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp, exist_ok=True)
    _barrier()
    # expert-parallel shards are gathered into whole banks (all ranks take part), so the files do
    # not depend on the expert-parallel size of the run that wrote them
    shards = {n: getattr(p, "_ep_shard", None) for n, p in trainer.model.named_parameters()}
    trainer.engine.sync_master()  # sharded optimizer: every rank's fp32 weights brought up to date first
    sd = {}
    seen = {}
    for k, v in trainer.engine.model_state_dict().items():
        t = _gather_full(v.detach(), shards.get(k))
        key = (v.data_ptr(), tuple(v.shape))
        if key in seen:  # tied weights: safetensors refuses shared storage
            t = t.clone()
        seen[key] = k
        sd[k] = t
    opt = trainer.engine.optimizer_state_dict()
    for name, st in opt["state"].items():
        if shards.get(name) is not None:
            dev = trainer.engine.device
            st["exp_avg"] = _gather_full(st["exp_avg"].to(dev), shards[name])
            st["exp_avg_sq"] = _gather_full(st["exp_avg_sq"].to(dev), shards[name])
    if rank == 0:
        save_file(sd, os.path.join(tmp, "model.safetensors"), metadata={"format": "pt"})
        torch.save(opt, os.path.join(tmp, "optimizer.bin"))
        torch.save(scheduler_state or {"last_epoch": trainer.global_step}, os.path.join(tmp, "scheduler.bin"))
    with open(os.path.join(tmp, f"random_states_{rank}.pkl"), "wb") as f:
        pickle.dump(_rng_state(), f)
    if dataset_state is not None:
        with open(os.path.join(tmp, f"dataset_state_{rank}.json"), "w") as f:
            json.dump(dataset_state, f)
    _barrier()
    if rank == 0:
        meta = {"step": step, "world_size": world}
        if dataset_state:
            meta["dataset_state"] = dataset_state
        if wandb_run_id:
            meta["wandb_run_id"] = wandb_run_id
        with open(os.path.join(tmp, "meta.json"), "w") as f:
            json.dump(meta, f)
        if os.path.isdir(final):
            shutil.rmtree(final)
        os.rename(tmp, final)
    _barrier()
    return final


def _gather_full(t: torch.Tensor, shard) -> torch.Tensor:
    if shard is None or not (dist.is_available() and dist.is_initialized()):
        return t.cpu().contiguous()
    parts = [torch.empty_like(t) for _ in range(shard[1])]
    dist.all_gather(parts, t.contiguous())
    return torch.cat(parts, dim=0).cpu()


def _slice_for(p: torch.Tensor, full: torch.Tensor) -> torch.Tensor:
    shard = getattr(p, "_ep_shard", None)
    if shard is None or full.shape == p.shape:
        return full
    n = p.shape[0]
    return full[shard[0] * n:(shard[0] + 1) * n]


def read_meta(ckpt_dir: str) -> dict:
    p = os.path.join(ckpt_dir, "meta.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return {}


def load_checkpoint(trainer, resume_from: str, strict: bool = True) -> tuple[int, dict | None]:
    """Restores parameters, AdamW state, step counter, RNG; returns (step, this rank's dataset state)."""
    from safetensors.torch import load_file

    rank, world = _rank_world()
    mpath = os.path.join(resume_from, "model.safetensors")
    if os.path.exists(mpath):
        sd = load_file(mpath)
        if getattr(trainer.model.config, "tie_word_embeddings", False) and "lm_head.weight" not in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        params = dict(trainer.model.named_parameters())
        sd = {k: (_slice_for(params[k], v) if k in params else v) for k, v in sd.items()}
        trainer.engine.load_model_state_dict(sd, strict=strict)
    opath = os.path.join(resume_from, "optimizer.bin")
    if os.path.exists(opath):
        opt = torch.load(opath, map_location="cpu", weights_only=False)
        params = dict(trainer.model.named_parameters())
        for name, st in opt["state"].items():
            if name in params:
                st["exp_avg"] = _slice_for(params[name], st["exp_avg"])
                st["exp_avg_sq"] = _slice_for(params[name], st["exp_avg_sq"])
        trainer.engine.load_optimizer_state_dict(opt)
    meta = read_meta(resume_from)
    step = int(meta.get("step", 0))
    spath = os.path.join(resume_from, "scheduler.bin")
    if os.path.exists(spath):
        step = int(torch.load(spath, map_location="cpu", weights_only=False).get("last_epoch", step))
    trainer.global_step = step
    rpath = os.path.join(resume_from, f"random_states_{rank}.pkl")
    if os.path.exists(rpath) and meta.get("world_size", world) == world:
        with open(rpath, "rb") as f:
            _set_rng_state(pickle.load(f))
    ds = None
    dpath = os.path.join(resume_from, f"dataset_state_{rank}.json")
    if os.path.exists(dpath) and meta.get("world_size", world) == world:
        with open(dpath) as f:
            ds = json.load(f)
    elif rank == 0 or meta.get("world_size", world) != world:
        ds = meta.get("dataset_state")
    return step, ds
