"""Launch helpers.

`run(...)` starts `torch.distributed.run` (torchrun) in-process from keyword arguments, the
service the reference's `torchrun_util/torchrun.py:4-14` provides: the keywords are validated against a
pydantic model derived from torchrun's own argparse parser (`options_model()`), turned back into a command
line and parsed by torchrun's parser, so `PET_*` environment variables keep working.

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


_OPTIONS_MODEL = None


def options_model():
    """A pydantic model of torchrun's options, derived from its own argparse parser (one field per option, the
    parser's type and default; unknown names are rejected, values are validated / coerced).  The reference gets
    the same service from `torchrun_util/argparse_to_pydantic.py:9-63`; `TorchrunOptions(**kw).to_argv()` gives the
    command line back."""
    global _OPTIONS_MODEL
    if _OPTIONS_MODEL is not None:
        return _OPTIONS_MODEL
    import argparse

    from pydantic import ConfigDict, create_model
    from torch.distributed.run import get_args_parser

    fields: dict[str, tuple] = {}
    flags: dict[str, tuple[str, bool]] = {}
    for act in get_args_parser()._actions:
        if not act.option_strings or isinstance(act, argparse._HelpAction):
            continue  # positionals (script and its arguments) are passed separately
        long = max(act.option_strings, key=len)
        is_flag = act.nargs == 0
        if is_flag:
            typ: Any = bool
        elif act.type in (int, float, str):
            typ = act.type
        else:
            typ = str  # options with custom converters (e.g. "auto" or a number) stay strings for the parser
        default = act.default if act.default is not argparse.SUPPRESS else None
        if default is not None and not is_flag and not isinstance(default, typ):
            typ = Any  # environment-backed defaults of another type: accept what the parser accepts
        fields[act.dest] = (typ | None if typ is not Any else Any, default)
        flags[act.dest] = (long, is_flag)

    def to_argv(self, training_script: str, training_script_args: Sequence[str] = ()) -> list[str]:
        argv = []
        for name, (flag, is_flag) in flags.items():
            v = getattr(self, name)
            if v is None or v == type(self).model_fields[name].default:
                continue
            if is_flag:
                if v:
                    argv.append(flag)
            else:
                argv.append(f"{flag}={v}")
        return argv + [training_script, *[str(a) for a in training_script_args]]

    model = create_model("TorchrunOptions", __config__=ConfigDict(extra="forbid", coerce_numbers_to_str=True), **fields)
    model.to_argv = to_argv
    _OPTIONS_MODEL = model
    return model


def run(training_script: str, training_script_args: Sequence[str] = (), **kwargs: Any) -> None:
    """Run torchrun with the given options in this process; returns when all workers have exited."""
    from torch.distributed.run import get_args_parser, run as torchrun

    kwargs.setdefault("master_addr", os.environ.get("MASTER_ADDR", "127.0.0.1"))
    opts = options_model()(**kwargs)  # typo'd or mistyped options fail here, with pydantic's message
    args = get_args_parser().parse_args(opts.to_argv(training_script, training_script_args))
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
