"""Checkpoint layout / auto-resume / pruning, exact training resume, and the data layer
(reference tests/test_auto_resume.py, test_checkpoint_resume.py, test_parquet_*.py)."""
import json
import os
import random

import pytest
import torch

from helpers import tiny_cfg
from moe_b200.data import DataConfig, StatefulParquetDataset, SyntheticConfig, SyntheticTokenDataset
from moe_b200.models import build_model
from moe_b200.trainer import Trainer
from moe_b200.utils.checkpoint import (cleanup_checkpoints, find_latest_checkpoint, load_checkpoint, read_meta,
                                       save_checkpoint)
from moe_b200.utils.training import TrainingConfig, build_lr_scheduler, build_optimizer, lr_factor


def fake_ckpt(root, step, **meta):
    d = os.path.join(root, f"checkpoint-{step}")
    os.makedirs(d)
    with open(os.path.join(d, "meta.json"), "w") as f:
        json.dump({"step": step, **meta}, f)
    return d


def test_find_latest_and_cleanup(tmp_path):
    root = str(tmp_path)
    assert find_latest_checkpoint(os.path.join(root, "missing")) is None
    assert find_latest_checkpoint(root) is None
    for s in (100, 20, 3000):
        fake_ckpt(root, s)
    os.makedirs(os.path.join(root, "checkpoint-abc"))
    os.makedirs(os.path.join(root, "checkpoint-5000.tmp"))
    open(os.path.join(root, "checkpoint-9999"), "w").close()  # a file, not a directory
    assert find_latest_checkpoint(root).endswith("checkpoint-3000")
    cleanup_checkpoints(root, 0)
    assert len([d for d in os.listdir(root) if d.startswith("checkpoint-")]) == 6
    cleanup_checkpoints(root, 2)
    assert sorted(d for d in os.listdir(root) if d[11:].isdigit() and os.path.isdir(os.path.join(root, d))) == \
        ["checkpoint-100", "checkpoint-3000"]
    assert os.path.isdir(os.path.join(root, "checkpoint-abc"))


def make_trainer(seed=0, mtype="deepseek_global_moe", **kw):
    model, _ = build_model(tiny_cfg(mtype, **kw), seed=seed)
    tcfg = TrainingConfig(learning_rate=1e-2, warmup_steps=2, max_steps=20, batch_size=2, gradient_accumulation=1,
                          weight_decay=0.1)
    return Trainer(model, tcfg), tcfg


def test_save_layout_and_meta(tmp_path):
    tr, _ = make_trainer()
    ds = SyntheticTokenDataset(SyntheticConfig(256, 16, 0))
    it = iter(ds)
    tr.train_step({k: v[None] for k, v in next(it).items()})
    path = save_checkpoint(tr, 1, str(tmp_path), ds.get_state(), wandb_run_id="abc123")
    assert path.endswith("checkpoint-1") and not os.path.exists(path + ".tmp")
    files = set(os.listdir(path))
    assert {"model.safetensors", "optimizer.bin", "scheduler.bin", "random_states_0.pkl", "dataset_state_0.json",
            "meta.json"} <= files
    meta = read_meta(path)
    assert meta["step"] == 1 and meta["wandb_run_id"] == "abc123" and meta["dataset_state"] == {"sample_idx": 1}
    from safetensors.torch import load_file

    sd = load_file(os.path.join(path, "model.safetensors"))
    assert "model.global_experts.gate_up_proj" in sd and "model.layers.0.mlp.gate.expert_bias" in sd
    assert sd["model.embed_tokens.weight"].dtype == torch.float32


@pytest.mark.parametrize("tied", [False, True])
def test_resume_is_bit_exact(tmp_path, tied):
    def run(n_first, n_total, resume):
        tr, _ = make_trainer(tie_word_embeddings=tied)
        ds = SyntheticTokenDataset(SyntheticConfig(256, 16, 0))
        losses = []
        if resume:
            step, st = load_checkpoint(tr, find_latest_checkpoint(str(tmp_path)))
            ds.set_state(st)
            assert step == n_first and tr.global_step == n_first and tr.engine.step_count == n_first
        it = iter(ds)
        while tr.global_step < (n_total if resume or n_first is None else n_first):
            b = torch.stack([next(it)["input_ids"] for _ in range(2)])
            r = tr.train_step({"input_ids": b, "labels": b})
            losses.append(r.loss.item())
            from moe_b200.utils.bias_update import update_expert_biases

            update_expert_biases(tr.model, 1e-3, None, is_global=True, alpha=0.5)
        if not resume and n_first is not None:
            save_checkpoint(tr, tr.global_step, str(tmp_path), ds.get_state())
        return losses, [p.detach().clone() for p in tr.model.parameters()], tr

    full, pfull, _ = run(None, 6, False)
    first, _, _ = run(3, 6, False)
    rest, pres, tr = run(3, 6, True)
    assert first == full[:3]
    assert rest == full[3:]
    for a, b in zip(pfull, pres):
        assert torch.equal(a, b)
    assert tr.current_lr() == 1e-2 * lr_factor(6, tr.cfg)


def test_interrupted_save_keeps_previous_checkpoint(tmp_path, monkeypatch):
    tr, _ = make_trainer()
    save_checkpoint(tr, 1, str(tmp_path))
    import moe_b200.utils.checkpoint as ck

    def boom(*a, **k):
        raise RuntimeError("disk full")

    monkeypatch.setattr(torch, "save", boom)
    with pytest.raises(RuntimeError):
        ck.save_checkpoint(tr, 2, str(tmp_path))
    assert find_latest_checkpoint(str(tmp_path)).endswith("checkpoint-1")


def test_truncated_checkpoint_is_reported(tmp_path):
    tr, _ = make_trainer()
    path = save_checkpoint(tr, 1, str(tmp_path))
    with open(os.path.join(path, "model.safetensors"), "r+b") as f:
        f.truncate(100)
    with pytest.raises(Exception):
        load_checkpoint(tr, path)


def test_lr_schedule_and_scheduler_resume():
    cfg = TrainingConfig(learning_rate=1.0, warmup_steps=10, max_steps=110, min_lr_ratio=0.1, lr_scheduler="cosine")
    assert lr_factor(0, cfg) == 0 and lr_factor(5, cfg) == 0.5 and lr_factor(10, cfg) == 1.0
    assert abs(lr_factor(60, cfg) - 0.55) < 1e-9 and abs(lr_factor(110, cfg) - 0.1) < 1e-9
    assert abs(lr_factor(500, cfg) - 0.1) < 1e-9
    cfg.lr_scheduler = "linear"
    assert abs(lr_factor(60, cfg) - 0.55) < 1e-9
    cfg.lr_scheduler = "constant"
    assert lr_factor(60, cfg) == 1.0
    cfg.lr_scheduler = "cosine"
    model, _ = build_model(tiny_cfg("dense"), seed=0)
    opt = build_optimizer(model, cfg)
    sch = build_lr_scheduler(opt, cfg)
    for _ in range(7):
        sch.step()
    st = sch.state_dict()
    opt2 = build_optimizer(model, cfg)
    sch2 = build_lr_scheduler(opt2, cfg)
    sch2.load_state_dict(st)  # restored, not re-advanced
    assert sch2.get_last_lr() == sch.get_last_lr() == [0.7, 0.7]


def test_optimizer_groups_follow_reference_rule():
    model, _ = build_model(tiny_cfg("deepseek_standard_moe"), seed=0)
    opt = build_optimizer(model, TrainingConfig(weight_decay=0.1))
    decay, nodecay = opt.param_groups
    assert decay["weight_decay"] == 0.1 and nodecay["weight_decay"] == 0.0
    names = {id(p): n for n, p in model.named_parameters()}
    dn = {names[id(p)] for p in decay["params"]}
    nn_ = {names[id(p)] for p in nodecay["params"]}
    assert "model.embed_tokens.weight" in dn and "lm_head.weight" in dn
    assert "model.layers.0.mlp.gate.weight" in dn and "model.layers.0.mlp.experts.gate_up_proj" in dn
    assert all("norm" in n for n in nn_) and len(nn_) == 2 * 4 + 1


# ------------------------------------------------------------------------- data
class Tok:
    eos_token_id = 1

    def encode(self, t, add_special_tokens=False):
        return [2 + (ord(c) % 50) for c in t]


@pytest.fixture()
def parquet_dir(tmp_path):
    import pandas as pd

    r = random.Random(0)
    for i in range(4):
        rows = ["".join(chr(97 + r.randrange(26)) for _ in range(r.randrange(5, 90))) for _ in range(30)]
        rows[3] = ""  # empty rows are skipped
        pd.DataFrame({"text": rows}).to_parquet(tmp_path / f"shard{i}.parquet")
    return str(tmp_path)


def test_parquet_windows_overlap_by_one_token_and_label_modes(parquet_dir):
    ds = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32), Tok())
    s = [x for x in ds]
    assert all(x["input_ids"].shape == (32,) for x in s)
    assert torch.equal(s[0]["labels"], s[0]["input_ids"])
    ds2 = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32, reference_double_shift=True), Tok())
    s2 = [x for x in ds2]
    assert torch.equal(s2[0]["labels"][:-1], s2[0]["input_ids"][1:])
    assert s2[0]["labels"][-1] == s2[1]["input_ids"][0]  # windows slide by seq_len with one token of overlap


def test_parquet_resume_exact_including_file_boundaries(parquet_dir):
    cfg = DataConfig(data_dir=parquet_dir, seq_len=32)
    full = [x["input_ids"] for x in StatefulParquetDataset(cfg, Tok())]
    for cut in range(1, len(full), max(1, len(full) // 12)):
        ds = StatefulParquetDataset(cfg, Tok())
        it = iter(ds)
        for _ in range(cut):
            next(it)
        st = json.loads(json.dumps(ds.get_state()))  # JSON round trip, as in meta.json
        ds2 = StatefulParquetDataset(cfg, Tok())
        ds2.set_state(st)
        rest = [x["input_ids"] for x in ds2]
        assert len(rest) == len(full) - cut and all(torch.equal(a, b) for a, b in zip(rest, full[cut:])), cut


def test_parquet_sharding_is_disjoint_and_seeded(parquet_dir):
    cfg = DataConfig(data_dir=parquet_dir, seq_len=32)
    files = [StatefulParquetDataset(cfg, Tok(), rank=r, world_size=4).files for r in range(4)]
    assert sorted(sum(files, [])) == sorted(StatefulParquetDataset(cfg, Tok()).files)
    assert all(len(f) == 1 for f in files)
    state = random.getstate()
    a = StatefulParquetDataset(cfg, Tok(), seed=42).files
    assert random.getstate() == state  # global RNG untouched
    assert a == StatefulParquetDataset(cfg, Tok(), seed=42).files
    with pytest.raises(FileNotFoundError):
        StatefulParquetDataset(DataConfig(data_dir=os.path.join(parquet_dir, "none")), Tok())


def test_parquet_prefetch_thread_same_stream_and_state(parquet_dir):
    base = [x["input_ids"] for x in StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32), Tok())]
    ds = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32, prefetch=8), Tok())
    it = iter(ds)
    got = [next(it)["input_ids"] for _ in range(5)]
    st = ds.get_state()  # position of the sample handed out, not of the read-ahead
    ds2 = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32), Tok())
    ds2.set_state(st)
    rest = [x["input_ids"] for x in ds2]
    assert all(torch.equal(a, b) for a, b in zip(got + rest, base)) and len(got) + len(rest) == len(base)


def test_parquet_prefetch_state_at_every_position_including_file_ends(parquet_dir):
    """With a read-ahead worker the saved position is that of the sample handed out, at every cut: the worker
    reaching the end of a file (or of all files) while earlier samples still sit in the queue must not move it."""
    import time

    base = [x["input_ids"] for x in StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32), Tok())]
    for cut in range(1, len(base) + 1):
        ds = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32, prefetch=2), Tok())
        it = iter(ds)
        got = [next(it)["input_ids"] for _ in range(cut)]
        time.sleep(0.002)  # let the worker run ahead (across a file boundary where one is near)
        st = json.loads(json.dumps(ds.get_state()))
        it.close()
        ds2 = StatefulParquetDataset(DataConfig(data_dir=parquet_dir, seq_len=32), Tok())
        ds2.set_state(st)
        rest = [x["input_ids"] for x in ds2]
        assert len(got) + len(rest) == len(base), cut
        assert all(torch.equal(a, b) for a, b in zip(got + rest, base)), cut


def test_synthetic_stream_is_reproducible_and_rank_dependent():
    a = SyntheticTokenDataset(SyntheticConfig(1000, 8, 3), rank=0)
    b = SyntheticTokenDataset(SyntheticConfig(1000, 8, 3), rank=1)
    ia, ib = iter(a), iter(b)
    xa = [next(ia)["input_ids"] for _ in range(3)]
    assert not torch.equal(xa[0], next(ib)["input_ids"])
    c = SyntheticTokenDataset(SyntheticConfig(1000, 8, 3), rank=0, world_size=8)
    c.set_state({"sample_idx": 2})
    assert torch.equal(next(iter(c))["input_ids"], xa[2])
    assert a.get_state() == {"sample_idx": 3} and xa[0].max() < 1000
