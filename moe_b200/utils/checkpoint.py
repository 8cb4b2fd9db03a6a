"""Checkpoints: `output_dir/checkpoint-{step}/` with `meta.json`, newest-first discovery and
keep-last-N pruning (`train.py:254-323` of the reference).

Inside a checkpoint directory: `model.safetensors` (HF parameter names, fp32 masters; buffers such
as `expert_bias` included), `optimizer.bin` (AdamW moments by parameter name + step),
`scheduler.bin`, `random_states_{rank}.pkl` (per-rank RNG) and `dataset_state_{rank}.json`
(per-rank data position).  `meta.json` = `{step, dataset_state (rank 0's), wandb_run_id, world_size}`.
A save goes to `checkpoint-{step}.tmp` and is renamed when complete, so an interrupted save never
shadows the previous checkpoint.  State is stored by name, not by rank, so a run can resume on a
different number of data-parallel ranks.

Runs whose state is sharded (sharded optimizer, sharded parameters, expert parallelism) write the sharded
payload of `sharded_state.py` instead of `model.safetensors` + `optimizer.bin`: every rank writes only the
slices it owns (`state-{rank}.safetensors`), rank 0 adds `index.json` and `extra.bin` (buffers, step, lr), and
nothing of the size of the model ever passes through one process.  `consolidate()` turns such a directory
into a plain `model.safetensors` on the CPU.
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


def _gather_objects(obj):
    rank, world = _rank_world()
    if world == 1:
        return [obj]
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def _save_sharded(trainer, tmp: str, rank: int, world: int) -> None:
    from . import sharded_state as ss

    eng = trainer.engine
    metas = ss.metas_from_engine(eng)
    part = ss.write_shard(tmp, rank, metas, eng.export_state_ranges())
    # full shapes of expert banks are the same on every rank; rank 0's metas name every tensor
    parts = _gather_objects(part)
    if rank == 0:
        ss.write_index(tmp, parts, metas, world)
        params = {n for n, _ in trainer.model.named_parameters()}
        buffers = {k: v.detach().cpu() for k, v in trainer.model.state_dict().items() if k not in params}
        torch.save({"buffers": buffers, "step": eng.step_count, "lr": eng.lr}, os.path.join(tmp, "extra.bin"))


def _load_sharded(trainer, resume_from: str, strict: bool) -> None:
    from . import sharded_state as ss

    eng = trainer.engine
    rd = ss.ShardReader(resume_from)
    rd.fill(ss.metas_from_engine(eng), eng.import_state_ranges(), strict=strict)
    extra = torch.load(os.path.join(resume_from, "extra.bin"), map_location="cpu", weights_only=False)
    own = dict(trainer.model.named_buffers())
    for k, v in extra.get("buffers", {}).items():
        if k in own:
            own[k].copy_(v)
    eng.step_count = int(extra.get("step", 0))
    eng.lr = float(extra.get("lr", eng.lr))
    eng.after_state_import()


def save_checkpoint(trainer, step: int, output_dir: str, dataset_state: dict | None = None,
                    wandb_run_id: str | None = None, scheduler_state: dict | None = None,
                    sharded: bool | None = None) -> str:
    """All ranks call this.  Rank 0 writes the shared files; every rank writes its RNG and data state.
    `sharded` (default: whenever the engine shards optimizer state, parameters or experts) selects the
    per-rank payload described in the module docstring."""
    from safetensors.torch import save_file

    rank, world = _rank_world()
    final = os.path.join(output_dir, f"checkpoint-{step}")
    tmp = final + ".tmp"
    if rank == 0:
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp, exist_ok=True)
    _barrier()
    eng = trainer.engine
    if sharded is None:
        sharded = bool(getattr(eng, "sharded", False) or getattr(eng, "sharded_params", False)
                       or getattr(eng, "has_ep", False))
    if sharded:
        _save_sharded(trainer, tmp, rank, world)
        if rank == 0:
            torch.save(scheduler_state or {"last_epoch": trainer.global_step}, os.path.join(tmp, "scheduler.bin"))
        return _finish_save(tmp, final, rank, world, step, dataset_state, wandb_run_id)
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
    return _finish_save(tmp, final, rank, world, step, dataset_state, wandb_run_id)


def _finish_save(tmp, final, rank, world, step, dataset_state, wandb_run_id) -> str:
    """Per-rank RNG / data position, then `meta.json` and the atomic rename by rank 0."""
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


def consolidate(ckpt_dir: str, out_path: str | None = None) -> str:
    """`model.safetensors` with whole tensors from a sharded checkpoint directory (CPU only)."""
    from . import sharded_state as ss

    return ss.consolidate(ckpt_dir, out_path)


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
    if os.path.exists(os.path.join(resume_from, "index.json")):
        _load_sharded(trainer, resume_from, strict)
    elif os.path.exists(mpath):
        sd = load_file(mpath)
        if getattr(trainer.model.config, "tie_word_embeddings", False) and "lm_head.weight" not in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        params = dict(trainer.model.named_parameters())
        sd = {k: (_slice_for(params[k], v) if k in params else v) for k, v in sd.items()}
        trainer.engine.load_model_state_dict(sd, strict=strict)
    opath = os.path.join(resume_from, "optimizer.bin")
    if os.path.exists(opath) and not os.path.exists(os.path.join(resume_from, "index.json")):
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
