"""Run logging: the reference's stdout line and wandb keys (`train.py:601-619`), plus a JSONL metrics
file that is always written (there is no network on the training boxes; wandb is optional)."""
from __future__ import annotations

import json
import os
import socket
import time


def format_step_line(step: int, total: float, ce: float, aux: float, seq_aux: float, lr: float, tok_per_sec: float,
                     grad_norm: float) -> str:
    return (f"step {step:6d}  loss={total:.4f}  ce={ce:.4f}  aux={aux:.4f}  seq_aux={seq_aux:.4f}  "
            f"lr={lr:.2e}  tok/s={tok_per_sec / 1e3:.1f}k  |g|={grad_norm:.3f}")


def rank_banner(rank: int, local_rank: int, world: int, device) -> str:
    return (f"[rank {rank}] host={socket.gethostname()} local_rank={local_rank} "
            f"num_processes={world} device={device}")


class MetricsLogger:
    """Rank-0 sink for scalar metrics: JSONL always, wandb when a project is configured and importable."""

    def __init__(self, output_dir: str, project: str | None = None, run_name: str | None = None,
                 run_id: str | None = None, config: dict | None = None, enabled: bool = True):
        self.enabled = enabled
        self.run_id = run_id
        self._wandb = None
        self._fh = None
        if not enabled:
            return
        os.makedirs(output_dir, exist_ok=True)
        self._fh = open(os.path.join(output_dir, "metrics.jsonl"), "a")
        if project and os.environ.get("WANDB_MODE", "") != "disabled":
            try:
                import wandb

                kw = {"project": project, "name": run_name, "config": config or {}}
                if run_id:
                    kw.update(id=run_id, resume="must")
                if not os.environ.get("WANDB_API_KEY"):
                    os.environ.setdefault("WANDB_MODE", "offline")
                self._wandb = wandb.init(**kw)
                self.run_id = self._wandb.id
            except Exception as e:  # logging must never stop training
                print(f"[logging] wandb unavailable ({type(e).__name__}: {e}); JSONL only", flush=True)

    def log(self, metrics: dict, step: int) -> None:
        if not self.enabled:
            return
        rec = {"step": step, "time": time.time()}
        rec.update({k: v for k, v in metrics.items() if not k.startswith("_hist/")})
        self._fh.write(json.dumps(rec) + "\n")
        self._fh.flush()
        if self._wandb is not None:
            try:
                self._wandb.log({k: v for k, v in metrics.items() if not k.startswith("_")}, step=step)
            except Exception:
                pass

    def close(self) -> None:
        if self._fh:
            self._fh.close()
            self._fh = None
        if self._wandb is not None:
            try:
                self._wandb.finish()
            except Exception:
                pass
