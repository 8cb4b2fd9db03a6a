"""Launch helpers.

`run(...)` starts `torch.distributed.run` (torchrun) in-process from keyword arguments, the
service the reference's `torchrun_util/torchrun.py:4-14` provides (it rebuilds torchrun's argparse
parser through pydantic; here the keywords are turned into the command line directly, and
`PET_*` environment variables keep working because torchrun's own parser reads them).

`multinode_env(...)` sets the environment the reference's cluster launcher sets before calling
torchrun (`modal_train.py:112-157`): NVLS on, one device work queue, master address / port.
"""
from __future__ import annotations

import os
from typing import Any, Sequence


def build_argv(training_script: str, training_script_args: Sequence[str] = (), **kwargs: Any) -> list[str]:
    """`nproc_per_node=8, master_addr="10.0.0.1"` -> `["--nproc-per-node=8", "--master-addr=10.0.0.1", script, ...]`."""
    argv: list[str] = []
    for k, v in kwargs.items():
        if v is None or v is False:
            continue
        flag = "--" + k.replace("_", "-")
        if v is True:
            argv.append(flag)
        else:
            argv.append(f"{flag}={v}")
    return argv + [training_script, *[str(a) for a in training_script_args]]


def run(training_script: str, training_script_args: Sequence[str] = (), **kwargs: Any) -> None:
    """Run torchrun with the given options in this process; returns when all workers have exited."""
    from torch.distributed.run import get_args_parser, run as torchrun

    kwargs.setdefault("master_addr", os.environ.get("MASTER_ADDR", "127.0.0.1"))
    args = get_args_parser().parse_args(build_argv(training_script, training_script_args, **kwargs))
    torchrun(args)


def multinode_env(master_addr: str, master_port: int = 1234, nvls: bool = True) -> dict[str, str]:
    env = {"MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port), "CUDA_DEVICE_MAX_CONNECTIONS": "1",
           "NCCL_NVLS_ENABLE": "1" if nvls else "0"}
    os.environ.update(env)
    return env


def train_cluster(config: str, node_rank: int, nnodes: int, master_addr: str, nproc_per_node: int = 8,
                  output_dir: str | None = None, max_checkpoints: int = 3, master_port: int = 1234) -> None:
    """One node's share of a multi-node run: the same torchrun invocation the reference's cluster
    launcher makes, always with auto-resume so that a restarted job continues from the newest checkpoint."""
    multinode_env(master_addr, master_port)
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    targs = ["--config", config, "--auto_resume", "--max_checkpoints", str(max_checkpoints)]
    if output_dir:
        targs += ["--output_dir", output_dir]
    run(os.path.join(here, "train.py"), targs, nnodes=nnodes, node_rank=node_rank, nproc_per_node=nproc_per_node,
        master_addr=master_addr, master_port=master_port)
