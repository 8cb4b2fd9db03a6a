"""Sharded checkpoint payload: every rank writes the slices it owns, a loader with another number of ranks or
another slicing reads the ranges it needs by name."""
import os

import pytest
import torch

from helpers import tiny_cfg
from moe_b200.data import SyntheticConfig, SyntheticTokenDataset
from moe_b200.models import build_model
from moe_b200.trainer import Trainer
from moe_b200.utils import sharded_state as ss
from moe_b200.utils.checkpoint import consolidate, find_latest_checkpoint, load_checkpoint, save_checkpoint
from moe_b200.utils.training import TrainingConfig


def make_trainer(seed=0, **kw):
    model, _ = build_model(tiny_cfg("deepseek_global_moe", **kw), seed=seed)
    tcfg = TrainingConfig(learning_rate=1e-2, warmup_steps=2, max_steps=20, batch_size=2, gradient_accumulation=1)
    return Trainer(model, tcfg)


def steps(tr, ds_state, n):
    ds = SyntheticTokenDataset(SyntheticConfig(256, 16, 0))
    if ds_state:
        ds.set_state(ds_state)
    it = iter(ds)
    out = []
    for _ in range(n):
        b = torch.stack([next(it)["input_ids"] for _ in range(2)])
        out.append(tr.train_step({"input_ids": b, "labels": b}).loss.item())
    return out, ds.get_state()


def test_sharded_save_resume_is_bit_exact_and_consolidates(tmp_path):
    full, _ = steps(make_trainer(), None, 6)
    tr = make_trainer()
    first, st = steps(tr, None, 3)
    path = save_checkpoint(tr, 3, str(tmp_path), st, sharded=True)
    files = set(os.listdir(path))
    assert {"index.json", "state-00000.safetensors", "extra.bin", "meta.json", "scheduler.bin"} <= files
    assert "model.safetensors" not in files
    tr2 = make_trainer(seed=99)  # different initial weights: everything must come from the files
    step, st2 = load_checkpoint(tr2, find_latest_checkpoint(str(tmp_path)))
    assert step == 3 and tr2.engine.step_count == 3
    rest, _ = steps(tr2, st2, 3)
    assert first + rest == full
    # whole tensors under their HuggingFace names, for tools that expect a plain state dict
    from safetensors.torch import load_file

    sd = load_file(consolidate(path))
    for n, p in tr.model.named_parameters():
        assert torch.equal(sd[n], p.detach()), n
    assert "model.layers.0.mlp.gate.expert_bias" in sd


class _FakeEngine:
    """A flat layout of three tensors, the middle one an expert bank split over `ep` ranks along its first
    dimension, the rest sliced evenly over `world` ranks (what a sharded optimizer or ZeRO-3 engine does)."""

    def __init__(self, rank, world, ep):
        self.rank, self.world = rank, world
        self.shapes = {"a.weight": (6, 8), "bank": (8 // ep, 5), "z.weight": (16,)}
        self.ep = {"bank": (rank % ep, ep)}
        self.metas, off = [], 0
        for n, shp in self.shapes.items():
            numel = int(torch.tensor(shp).prod())
            if n in self.ep:
                r, e = self.ep[n]
                self.metas.append(ss.TensorMeta(n, off, numel, (shp[0] * e, *shp[1:]), r * numel))
            else:
                self.metas.append(ss.TensorMeta(n, off, numel, shp, 0))
            off += numel + 3  # padding between tensors, as alignment leaves it
        self.total = off
        self.buf = {k: torch.zeros(off) for k in "pmv"}

    def truth(self, kind, name, gidx):
        return {"p": 1.0, "m": 2.0, "v": 3.0}[kind] * 1000 + hash(name) % 97 + gidx.float() * 0.25

    def fill_truth(self):
        for m in self.metas:
            g = torch.arange(m.numel) + m.global_start
            for k in "pmv":
                self.buf[k][m.offset:m.offset + m.numel] = self.truth(k, m.name, g)

    def ranges(self, export):
        out = []
        for m in self.metas:
            if m.name in self.ep:  # each expert-parallel rank has its own experts; replicas beyond `ep` skip
                if export and self.rank >= self.ep[m.name][1]:
                    continue
                lo, hi = m.offset, m.offset + m.numel
            else:  # even slices over the ranks
                per = (m.numel + self.world - 1) // self.world
                lo = m.offset + min(per * self.rank, m.numel)
                hi = m.offset + min(per * (self.rank + 1), m.numel)
                if not export:
                    lo, hi = m.offset, m.offset + m.numel  # a loader may want more than it would write
            if hi > lo:
                for k in "pmv":
                    out.append((k, lo, hi, self.buf[k][lo:hi]))
        return out


@pytest.mark.parametrize("w_save,ep_save,w_load,ep_load", [(2, 2, 1, 1), (2, 1, 4, 4), (4, 2, 2, 1), (1, 1, 8, 8)])
def test_resharding_by_name_and_range(tmp_path, w_save, ep_save, w_load, ep_load):
    d = str(tmp_path)
    parts, metas0 = [], None
    for r in range(w_save):
        e = _FakeEngine(r, w_save, ep_save)
        e.fill_truth()
        parts.append(ss.write_shard(d, r, e.metas, e.ranges(export=True)))
        metas0 = metas0 or e.metas
    ss.write_index(d, parts, metas0, w_save)
    rd = ss.ShardReader(d)
    assert rd.shape("bank") == (8, 5)
    for r in range(w_load):
        e = _FakeEngine(r, w_load, ep_load)
        rd.fill(e.metas, e.ranges(export=False))
        for m in e.metas:
            g = torch.arange(m.numel) + m.global_start
            for k in "pmv":
                assert torch.equal(e.buf[k][m.offset:m.offset + m.numel], e.truth(k, m.name, g)), (r, m.name, k)


def test_missing_piece_is_an_error(tmp_path):
    d = str(tmp_path)
    e = _FakeEngine(0, 2, 1)  # rank 1 never wrote its file: half of every tensor is missing
    e.fill_truth()
    ss.write_index(d, [ss.write_shard(d, 0, e.metas, e.ranges(export=True))], e.metas, 2)
    with pytest.raises(KeyError):
        ss.ShardReader(d).fill(_FakeEngine(0, 1, 1).metas, _FakeEngine(0, 1, 1).ranges(export=False))


def _gloo_worker(rank, world, port, out_dir):
    import sys

    import torch.distributed as dist

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tr = make_trainer(seed=3)
    g = torch.Generator().manual_seed(0)
    for _ in range(2):
        b = torch.randint(0, 256, (4, 16), generator=g)[rank * 2:(rank + 1) * 2]
        tr.train_step({"input_ids": b, "labels": b})
    save_checkpoint(tr, 2, out_dir, {"sample_idx": 4 + rank}, sharded=True)
    if rank == 0:
        torch.save({"p": tr.engine.p32.clone(), "m": tr.engine.m.clone()}, os.path.join(out_dir, "truth.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_write_one_process_reads(tmp_path):
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_gloo_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    path = find_latest_checkpoint(str(tmp_path))
    assert {"state-00000.safetensors", "state-00001.safetensors", "dataset_state_1.json"} <= set(os.listdir(path))
    tr = make_trainer(seed=50)
    step, ds = load_checkpoint(tr, path)  # other world size: rank 0's data position from meta.json
    truth = torch.load(tmp_path / "truth.pt")
    assert step == 2 and ds == {"sample_idx": 4}
    assert torch.equal(tr.engine.p32, truth["p"]) and torch.equal(tr.engine.m, truth["m"])
