"""Multi-process data parallelism on CPU (gloo, world_size 2): gradient averaging equals the single
process run on the concatenated batch, ranks stay bit-identical, `train.py` runs end to end under
torchrun-style environment variables, and a rank that dies is noticed as an error, not a hang."""
import os
import socket
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import tiny_cfg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ddp_worker(rank, world, port, out_dir, mtype):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from moe_b200.models import build_model
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    torch.manual_seed(100 + rank)  # different global RNG per rank must not matter: weights come from `seed`
    model, _ = build_model(tiny_cfg(mtype), seed=7)
    tr = Trainer(model, TrainingConfig(learning_rate=1e-2, warmup_steps=0, max_steps=10, batch_size=2,
                                       gradient_accumulation=1, lr_scheduler="constant"))
    tr.engine.broadcast_parameters(0)
    g = torch.Generator().manual_seed(0)
    full = [torch.randint(0, 256, (4, 16), generator=g) for _ in range(3)]
    for b in full:
        mine = b[rank * 2:(rank + 1) * 2]
        r = tr.train_step({"input_ids": mine, "labels": mine})
    torch.save({"p": tr.engine.p32.clone(), "norm": float(r.grad_norm)}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mtype", ["dense", "standard_moe"])
def test_ddp_two_ranks_match_single_process(tmp_path, mtype):
    port = free_port()
    mp.spawn(_ddp_worker, args=(2, port, str(tmp_path), mtype), nprocs=2, join=True)
    a = torch.load(tmp_path / "rank0.pt")
    b = torch.load(tmp_path / "rank1.pt")
    assert torch.equal(a["p"], b["p"]) and a["norm"] == b["norm"]
    if mtype != "dense":
        return  # the Switch loss uses per-rank statistics, so only rank agreement is exact for MoE
    from moe_b200.models import build_model
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    model, _ = build_model(tiny_cfg(mtype), seed=7)
    tr = Trainer(model, TrainingConfig(learning_rate=1e-2, warmup_steps=0, max_steps=10, batch_size=4,
                                       gradient_accumulation=1, lr_scheduler="constant"))
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        bt = torch.randint(0, 256, (4, 16), generator=g)
        tr.train_step({"input_ids": bt, "labels": bt})
    # Adam normalises the update, so float-summation-order noise in tiny gradients is amplified to ~lr
    diff = (tr.engine.p32 - a["p"]).abs()
    assert diff.max() < 2.5e-2 and (diff > 1e-4).float().mean() < 1e-3


def test_gradient_accumulation_equals_large_batch():
    from moe_b200.models import build_model
    from moe_b200.trainer import Trainer
    from moe_b200.utils.training import TrainingConfig

    g = torch.Generator().manual_seed(0)
    bt = torch.randint(0, 256, (4, 16), generator=g)
    res = []
    for accum in (1, 2):
        model, _ = build_model(tiny_cfg("dense"), seed=3)
        tr = Trainer(model, TrainingConfig(learning_rate=1e-2, warmup_steps=0, max_steps=5, batch_size=4 // accum,
                                           gradient_accumulation=accum, lr_scheduler="constant"))
        mbs = [{"input_ids": c, "labels": c} for c in bt.chunk(accum)]
        tr.train_step(mbs)
        res.append(tr.engine.p32.clone())
    assert torch.allclose(res[0], res[1], atol=2e-6)


def _run_train(nproc, out_dir, extra=(), env_extra=None, timeout=300):
    port = free_port()
    procs = []
    for rank in range(nproc):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(nproc), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", WANDB_MODE="disabled")
        env.update(env_extra or {})
        cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--config",
               os.path.join(ROOT, "configs", "bench", "tiny_cpu.yaml"), "--device", "cpu", "--output_dir", out_dir,
               *extra]
        procs.append(subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o))
    return outs


def test_train_py_two_rank_gloo_run_and_resume(tmp_path):
    out = str(tmp_path / "run")
    outs = _run_train(2, out, extra=["--max_steps", "4", "--max_checkpoints", "2"])
    assert all(rc == 0 for rc, _ in outs), outs[0][1][-2000:]
    log0 = outs[0][1]
    assert "step      4" in log0 and "Training complete." in log0
    import math
    import re

    ce = float(re.search(r"step\s+1\s+loss=\S+\s+ce=(\S+)", log0).group(1))
    assert abs(ce - math.log(151936)) < 0.15
    assert os.path.isdir(os.path.join(out, "checkpoint-4"))
    assert {"dataset_state_0.json", "dataset_state_1.json", "random_states_1.pkl"} <= set(
        os.listdir(os.path.join(out, "checkpoint-4")))
    outs = _run_train(2, out, extra=["--max_steps", "6", "--auto_resume"])
    assert all(rc == 0 for rc, _ in outs), outs[0][1][-2000:]
    assert "Resumed from step 4" in outs[0][1] and "step      6" in outs[0][1] and "step      4 " not in outs[0][1]


def _failing_worker(rank, world, port, out_dir):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)  # one good step together
    if rank == 1:
        os._exit(17)  # dies between steps, with no collective in flight
    t0 = time.time()
    try:
        dist.all_reduce(t)
        outcome = "completed"
    except Exception as e:  # gloo reports the lost peer / the timeout as an error
        outcome = f"error:{type(e).__name__}"
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")


def test_dead_rank_is_an_error_not_a_hang(tmp_path):
    port = free_port()
    ctx = mp.spawn(_failing_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 60
    while time.time() < deadline and not (tmp_path / "rank0.txt").exists():
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
    assert (tmp_path / "rank0.txt").exists(), "rank 0 hung on the collective"
    outcome, secs = (tmp_path / "rank0.txt").read_text().split()
    assert outcome.startswith("error:") and float(secs) < 30
