"""Cluster launcher: what the reference's `modal_train.py:32-157` sets up, as data plus two small drivers.

* `ClusterSpec`: nodes, GPUs per node, time limit, retry budget, the two volumes (`/data` for parquet shards,
  `/checkpoints` for run outputs), the container image recipe (CUDA base, RDMA libraries, Python packages,
  which parts of this repository to ship) and the NCCL environment.
* `supervise(...)`: the fail-stop + auto-resume loop without any cloud service: run one node's share of the job
  in a child process and start it again (always with `--auto_resume`) when it exits non-zero, up to
  `max_retries` times.  The step watchdog exits with code 75 when a step hangs, a dead peer ends NCCL
  collectives with an error: both land here.  This is the role `retries=10` plays on Modal.
* `build_modal_app(spec)`: the same cluster as a Modal app (image, volumes, secrets, `retries`, `clustered(size,
  rdma=True)`, a downloader function for the data volume), for machines where the `modal` package exists.
"""
from __future__ import annotations

import os
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parent.parent


@dataclass
class ClusterSpec:
    n_nodes: int = 2
    gpus_per_node: int = 8
    gpu_type: str = "B200"
    timeout_hours: int = 24
    max_checkpoints: int = 3
    max_retries: int = 10
    retry_initial_delay: float = 0.0
    config_file: str = "configs/scaling/xs_standard.yaml"
    master_port: int = 1234
    data_volume: str = "moe-training-data"
    ckpt_volume: str = "moe-checkpoints"
    data_mount: str = "/data"
    ckpt_mount: str = "/checkpoints"
    app_name: str = "moe-training"
    secrets: tuple = ("huggingface-secret", "wandb-secret")
    base_image: str = "nvidia/cuda:12.9.0-devel-ubuntu22.04"
    python_version: str = "3.12"
    apt_packages: tuple = ("curl", "git", "libibverbs-dev", "libibverbs1", "libhwloc15", "libnl-route-3-200")
    pip_packages: tuple = ("torch>=2.8.0", "numpy", "pyarrow>=15.0.0", "pandas>=2.0.0", "pyyaml>=6.0",
                           "safetensors", "tokenizers>=0.19.0", "transformers>=5.0.0", "huggingface-hub>=0.20.0",
                           "python-dotenv>=1.0.0", "wandb>=0.17.0", "ninja")
    ship: tuple = ("train.py", "moe_b200", "csrc", "configs", "scripts", "__graft_entry__.py")
    remote_root: str = "/root/moe"
    env: dict = field(default_factory=lambda: {"NCCL_NVLS_ENABLE": "1", "CUDA_DEVICE_MAX_CONNECTIONS": "1"})

    def experiment_name(self, config: str | None = None, root: Path | None = None) -> str:
        import yaml

        with open((root or REPO_ROOT) / (config or self.config_file)) as f:
            return (yaml.safe_load(f) or {}).get("experiment_name", "default")

    def train_args(self, config: str | None = None, root: str | None = None) -> list[str]:
        """Arguments of `train.py` on a cluster node: data and checkpoints on the volumes, always auto-resume."""
        cfg = config or self.config_file
        base = root or str(REPO_ROOT)
        name = self.experiment_name(cfg)
        return ["--config", f"{base}/{cfg}", "--auto_resume", "--data_dir", f"{self.data_mount}/parquet",
                "--output_dir", f"{self.ckpt_mount}/{name}", "--max_checkpoints", str(self.max_checkpoints)]

    def node_command(self, node_rank: int, master_addr: str, config: str | None = None,
                     root: str | None = None) -> list[str]:
        """One node's torchrun invocation (`modal_train.py:143-157`)."""
        base = root or str(REPO_ROOT)
        return [sys.executable, "-m", "torch.distributed.run", f"--nnodes={self.n_nodes}", f"--node-rank={node_rank}",
                f"--nproc-per-node={self.gpus_per_node}", f"--master-addr={master_addr}",
                f"--master-port={self.master_port}", f"{base}/train.py", *self.train_args(config, root)]


def supervise(cmd: list[str], max_retries: int = 10, initial_delay: float = 0.0, env: dict | None = None,
              log=print, run=subprocess.call, sleep=time.sleep) -> int:
    """Run `cmd` until it exits 0, restarting it after a non-zero exit at most `max_retries` times (the delay
    doubles from `initial_delay`).  Returns the last exit code.  The command has to resume by itself
    (`--auto_resume`), which the cluster's `train_args` guarantee."""
    delay = initial_delay
    full_env = dict(os.environ)
    full_env.update(env or {})
    rc = 0
    for attempt in range(max_retries + 1):
        rc = run(cmd, env=full_env)
        if rc == 0:
            return 0
        if attempt == max_retries:
            break
        log(f"[supervise] exit code {rc}; restart {attempt + 1} of {max_retries}"
            + (" (a step exceeded its time limit)" if rc == 75 else ""))
        if delay > 0:
            sleep(delay)
            delay *= 2
    log(f"[supervise] giving up after {max_retries} restarts, last exit code {rc}")
    return rc


def run_node(spec: ClusterSpec, node_rank: int, master_addr: str, config: str | None = None) -> int:
    """One node of a bare-metal cluster under supervision."""
    return supervise(spec.node_command(node_rank, master_addr, config), spec.max_retries, spec.retry_initial_delay,
                     env=spec.env)


def build_modal_app(spec: ClusterSpec | None = None):
    """(app, train, download_data) for `modal run`: needs the `modal` package."""
    import modal
    import modal.experimental

    spec = spec or ClusterSpec()
    image = modal.Image.from_registry(spec.base_image, add_python=spec.python_version)
    image = image.apt_install(*spec.apt_packages).pip_install(*spec.pip_packages)
    for item in spec.ship:
        src = REPO_ROOT / item
        if src.is_dir():
            image = image.add_local_dir(str(src), remote_path=f"{spec.remote_root}/{item}")
        elif src.exists():
            image = image.add_local_file(str(src), remote_path=f"{spec.remote_root}/{item}")
    data_volume = modal.Volume.from_name(spec.data_volume, create_if_missing=True)
    ckpt_volume = modal.Volume.from_name(spec.ckpt_volume, create_if_missing=True)
    app = modal.App(spec.app_name, image=image, secrets=[modal.Secret.from_name(s) for s in spec.secrets],
                    volumes={spec.data_mount: data_volume, spec.ckpt_mount: ckpt_volume})

    @app.function(gpu=f"{spec.gpu_type}:{spec.gpus_per_node}", timeout=60 * 60 * spec.timeout_hours,
                  retries=modal.Retries(initial_delay=spec.retry_initial_delay, max_retries=spec.max_retries),
                  experimental_options={"efa_enabled": True})
    @modal.experimental.clustered(size=spec.n_nodes, rdma=True)
    def train(config: str = spec.config_file):
        info = modal.experimental.get_cluster_info()
        os.environ.update(spec.env)
        sys.path.insert(0, spec.remote_root)
        cmd = spec.node_command(info.rank, info.container_ips[0], config, root=spec.remote_root)
        rc = subprocess.call(cmd)  # Modal's own retries restart the cluster; auto-resume continues the run
        if rc != 0:
            raise RuntimeError(f"training exited with code {rc}")

    @app.function(timeout=60 * 60 * 6)
    def download_data(max_shards: int | None = None, workers: int = 32):
        sys.path.insert(0, f"{spec.remote_root}/scripts")
        import download_data as dd

        argv = ["--out_dir", f"{spec.data_mount}/parquet", "--workers", str(workers)]
        if max_shards is not None:
            argv += ["--max_shards", str(max_shards)]
        rc = dd.main(argv)
        data_volume.commit()
        if rc != 0:
            raise RuntimeError("some shards failed to download")

    return app, train, download_data
