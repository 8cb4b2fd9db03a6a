"""Sharded checkpoint payload: every rank writes the slices of the training state it owns, by name.

The reference's FSDP recipe asks for `SHARDED_STATE_DICT` (`accelerate_configs/fsdp_8gpu.yaml:11`) because a
30 B-parameter model (fp32 masters + two Adam moments = 366 GB) cannot pass through one process.  Here a
checkpoint directory holds

* `state-{rank:05d}.safetensors`: 1-D fp32 pieces keyed `"{kind}|{name}|{start}"`, kind `p` (master value),
  `m` / `v` (Adam moments), `start` = first element of the piece inside the FULL tensor `name` (flattened;
  for an expert bank the full tensor spans the experts of all expert-parallel ranks);
* `index.json`: per tensor its full shape and, per kind, the list of `[start, stop, rank]` pieces.

Pieces are addressed by parameter name and element range, not by rank, so a run with another number of ranks,
another expert-parallel size or another sharding mode reads exactly the ranges it needs from whichever
files hold them.  The functions below know nothing about process groups: `checkpoint.py` drives them.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch

FORMAT = "moe_b200-sharded-1"


@dataclass
class TensorMeta:
    """One parameter in the engine's flat layout."""
    name: str
    offset: int            # first flat index
    numel: int             # local number of elements
    full_shape: tuple      # shape of the whole tensor (all expert-parallel shards together)
    global_start: int = 0  # flat position of the local tensor inside the whole tensor


def metas_from_engine(engine) -> list[TensorMeta]:
    out = []
    for s in engine.slots:
        shard = getattr(s.param, "_ep_shard", None)
        shape = tuple(s.param.shape)
        if shard is not None:
            r, n = shard
            out.append(TensorMeta(s.name, s.offset, s.numel, (shape[0] * n, *shape[1:]), r * s.numel))
        else:
            out.append(TensorMeta(s.name, s.offset, s.numel, shape, 0))
    return out


def _pieces(metas: list[TensorMeta], lo: int, hi: int):
    """Cut the flat range [lo, hi) at parameter borders: yields (meta, local_start, local_stop)."""
    for m in metas:
        a, b = max(lo, m.offset), min(hi, m.offset + m.numel)
        if b > a:
            yield m, a - m.offset, b - m.offset


def write_shard(ckpt_dir: str, rank: int, metas: list[TensorMeta], ranges) -> dict:
    """`ranges`: iterable of (kind, flat_lo, flat_hi, tensor1d covering that range).  Writes this rank's file
    and returns its part of the index: {name: {kind: [[start, stop, rank], ...]}}."""
    from safetensors.torch import save_file

    tensors, index = {}, {}
    for kind, lo, hi, t in ranges:
        for m, a, b in _pieces(metas, lo, hi):
            gs = m.global_start + a
            piece = t[(m.offset + a) - lo:(m.offset + b) - lo].detach().to(torch.float32).cpu().contiguous().clone()
            tensors[f"{kind}|{m.name}|{gs}"] = piece
            index.setdefault(m.name, {}).setdefault(kind, []).append([gs, gs + (b - a), rank])
    if not tensors:  # safetensors refuses an empty file
        tensors["_empty"] = torch.zeros(1)
    save_file(tensors, os.path.join(ckpt_dir, f"state-{rank:05d}.safetensors"))
    return index


def write_index(ckpt_dir: str, parts: list[dict], metas: list[TensorMeta], world: int, extra: dict | None = None) -> None:
    tensors = {}
    for m in metas:
        tensors[m.name] = {"shape": list(m.full_shape), "pieces": {}}
    for part in parts:
        for name, kinds in part.items():
            ent = tensors.setdefault(name, {"shape": None, "pieces": {}})
            for kind, lst in kinds.items():
                ent["pieces"].setdefault(kind, []).extend(lst)
    for ent in tensors.values():
        for lst in ent["pieces"].values():
            lst.sort()
    with open(os.path.join(ckpt_dir, "index.json"), "w") as f:
        json.dump({"format": FORMAT, "world_size": world, "tensors": tensors, **(extra or {})}, f)


def is_sharded(ckpt_dir: str) -> bool:
    return os.path.exists(os.path.join(ckpt_dir, "index.json"))


class ShardReader:
    """Reads element ranges of named tensors from a sharded checkpoint directory."""

    def __init__(self, ckpt_dir: str):
        with open(os.path.join(ckpt_dir, "index.json")) as f:
            self.index = json.load(f)
        if self.index.get("format") != FORMAT:
            raise ValueError(f"{ckpt_dir}: not a {FORMAT} checkpoint")
        self.dir = ckpt_dir
        self._files: dict = {}

    def _file(self, rank: int):
        from safetensors import safe_open

        f = self._files.get(rank)
        if f is None:
            f = safe_open(os.path.join(self.dir, f"state-{rank:05d}.safetensors"), framework="pt", device="cpu")
            self._files[rank] = f
        return f

    def has(self, name: str, kind: str) -> bool:
        return bool(self.index["tensors"].get(name, {}).get("pieces", {}).get(kind))

    def shape(self, name: str):
        return tuple(self.index["tensors"][name]["shape"])

    def read(self, name: str, kind: str, start: int, stop: int, out: torch.Tensor) -> None:
        """out[:stop - start] = elements [start, stop) of the flattened full tensor; raises when a part of the
        range is in no file (a truncated or incomplete checkpoint must not load silently)."""
        pieces = self.index["tensors"].get(name, {}).get("pieces", {}).get(kind, [])
        covered = start
        for gs, ge, rank in pieces:
            if ge <= covered or gs >= stop:
                continue
            if gs > covered:
                break
            a, b = max(gs, covered), min(ge, stop)
            src = self._file(rank).get_slice(f"{kind}|{name}|{gs}")[a - gs:b - gs]
            out[a - start:b - start].copy_(src)
            covered = b
            if covered >= stop:
                break
        if covered < stop:
            raise KeyError(f"checkpoint has no data for {kind}|{name} elements [{covered}, {stop})")

    def fill(self, metas: list[TensorMeta], ranges, strict: bool = True) -> None:
        """`ranges`: iterable of (kind, flat_lo, flat_hi, destination tensor1d covering that range)."""
        for kind, lo, hi, dst in ranges:
            for m, a, b in _pieces(metas, lo, hi):
                if not self.has(m.name, kind):
                    if strict and kind == "p":
                        raise KeyError(f"checkpoint has no tensor {m.name}")
                    continue
                buf = torch.empty(b - a, dtype=torch.float32)
                self.read(m.name, kind, m.global_start + a, m.global_start + b, buf)
                dst[(m.offset + a) - lo:(m.offset + b) - lo].copy_(buf)


def consolidate(ckpt_dir: str, out_path: str | None = None) -> str:
    """Assemble `model.safetensors` (whole fp32 tensors under their HuggingFace names) from the shards of a
    checkpoint directory, on the CPU, one tensor at a time."""
    from safetensors.torch import save_file

    rd = ShardReader(ckpt_dir)
    sd = {}
    for name, ent in rd.index["tensors"].items():
        if not rd.has(name, "p"):
            continue
        shape = tuple(ent["shape"])
        n = 1
        for d in shape:
            n *= d
        buf = torch.empty(n, dtype=torch.float32)
        rd.read(name, "p", 0, n, buf)
        sd[name] = buf.view(shape)
    extra = os.path.join(ckpt_dir, "extra.bin")
    if os.path.exists(extra):
        for k, v in torch.load(extra, map_location="cpu", weights_only=False).get("buffers", {}).items():
            sd[k] = v
    out_path = out_path or os.path.join(ckpt_dir, "model.safetensors")
    save_file(sd, out_path, metadata={"format": "pt"})
    return out_path
