"""Cluster launcher: the restart loop on real child processes, the node command, and the Modal app built
against a fake `modal` package that records what it is asked for."""
import sys
import types

from moe_b200.cluster import ClusterSpec, build_modal_app, supervise


def test_supervise_restarts_until_success(tmp_path):
    counter = tmp_path / "n"
    prog = ("import sys, pathlib; p = pathlib.Path(sys.argv[1]); n = int(p.read_text()) if p.exists() else 0; "
            "p.write_text(str(n + 1)); sys.exit(0 if n >= 2 else (75 if n == 0 else 1))")
    logs = []
    rc = supervise([sys.executable, "-c", prog, str(counter)], max_retries=5, log=logs.append)
    assert rc == 0 and counter.read_text() == "3"
    assert len(logs) == 2 and "time limit" in logs[0]


def test_supervise_gives_up_after_the_retry_budget():
    calls, sleeps = [], []
    rc = supervise(["x"], max_retries=3, initial_delay=1.0, run=lambda c, env: calls.append(c) or 7,
                   sleep=sleeps.append, log=lambda s: None)
    assert rc == 7 and len(calls) == 4 and sleeps == [1.0, 2.0, 4.0]


def test_node_command_uses_volumes_and_auto_resume():
    spec = ClusterSpec(n_nodes=2, gpus_per_node=8)
    cmd = spec.node_command(1, "10.0.0.1")
    joined = " ".join(cmd)
    assert "--nnodes=2" in cmd and "--node-rank=1" in cmd and "--nproc-per-node=8" in cmd
    assert "--master-addr=10.0.0.1" in cmd and "--master-port=1234" in cmd
    assert "--auto_resume" in cmd and "--data_dir /data/parquet" in joined and "--max_checkpoints 3" in joined
    assert f"--output_dir /checkpoints/{spec.experiment_name()}" in joined


class _Rec:
    def __init__(self, log, name):
        self._log, self._name = log, name

    def __getattr__(self, item):
        def call(*a, **k):
            self._log.append((f"{self._name}.{item}", a, k))
            return self
        return call


def test_modal_app_matches_the_cluster_spec(monkeypatch):
    log = []
    modal = types.ModuleType("modal")
    exp = types.ModuleType("modal.experimental")
    modal.experimental = exp
    modal.Image = types.SimpleNamespace(from_registry=lambda tag, add_python=None: log.append(("image", tag, add_python)) or _Rec(log, "image"))
    modal.Volume = types.SimpleNamespace(from_name=lambda n, create_if_missing=False: ("volume", n))
    modal.Secret = types.SimpleNamespace(from_name=lambda n: ("secret", n))
    modal.Retries = lambda initial_delay, max_retries: ("retries", initial_delay, max_retries)

    class App:
        def __init__(self, name, **kw):
            log.append(("app", name, kw))

        def function(self, **kw):
            log.append(("function", kw))
            return lambda f: f

    modal.App = App
    exp.clustered = lambda size, rdma: (log.append(("clustered", size, rdma)) or (lambda f: f))
    monkeypatch.setitem(sys.modules, "modal", modal)
    monkeypatch.setitem(sys.modules, "modal.experimental", exp)
    spec = ClusterSpec()
    app, train, download = build_modal_app(spec)
    assert ("clustered", 2, True) in log
    fn = [e for e in log if e[0] == "function"][0][1]
    assert fn["gpu"] == "B200:8" and fn["retries"] == ("retries", 0.0, 10) and fn["timeout"] == 24 * 3600
    appkw = [e for e in log if e[0] == "app"][0][2]
    assert appkw["volumes"] == {"/data": ("volume", "moe-training-data"), "/checkpoints": ("volume", "moe-checkpoints")}
    assert ("secret", "huggingface-secret") in appkw["secrets"]
    assert any(e[0] == "image.apt_install" and "libibverbs1" in e[1] for e in log)
    assert callable(train) and callable(download)


def test_torchrun_options_model_validates_and_round_trips():
    """The typed model of torchrun's options (built from torchrun's own parser): unknown and mistyped options
    are rejected before anything starts, and the generated command line parses back to the same values."""
    import pytest
    from torch.distributed.run import get_args_parser

    from moe_b200 import launch

    model = launch.options_model()
    opts = model(nproc_per_node="8", nnodes=2, node_rank=1, master_addr="10.0.0.1", master_port=1234)
    argv = opts.to_argv("train.py", ["--config", "x.yaml", "--auto_resume"])
    assert argv[-4:] == ["train.py", "--config", "x.yaml", "--auto_resume"] and "--nproc-per-node=8" in argv
    args = get_args_parser().parse_args(argv)
    assert (args.nnodes, args.node_rank, args.master_addr, args.master_port) == ("2", 1, "10.0.0.1", 1234)
    assert args.training_script == "train.py" and args.training_script_args == ["--config", "x.yaml", "--auto_resume"]
    assert "--standalone" in model(standalone=True).to_argv("t.py") and model().to_argv("t.py") == ["t.py"]
    with pytest.raises(Exception):
        model(nproc_pernode=8)  # misspelt option
    with pytest.raises(Exception):
        model(master_port="not-a-port")
