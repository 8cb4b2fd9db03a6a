"""`python -m moe_b200.cluster_node --node_rank R --master_addr A [--config C] [--nnodes N]`: one node of a
multi-node run under the restart loop of `moe_b200.cluster.supervise`."""
from __future__ import annotations

import argparse
import sys

from .cluster import ClusterSpec, run_node


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--node_rank", type=int, required=True)
    p.add_argument("--master_addr", required=True)
    p.add_argument("--config", default=None)
    p.add_argument("--nnodes", type=int, default=None)
    p.add_argument("--gpus_per_node", type=int, default=None)
    p.add_argument("--max_retries", type=int, default=None)
    p.add_argument("--data_mount", default=None)
    p.add_argument("--ckpt_mount", default=None)
    a = p.parse_args(argv)
    spec = ClusterSpec()
    for k, v in (("n_nodes", a.nnodes), ("gpus_per_node", a.gpus_per_node), ("max_retries", a.max_retries),
                 ("data_mount", a.data_mount), ("ckpt_mount", a.ckpt_mount)):
        if v is not None:
            setattr(spec, k, v)
    return run_node(spec, a.node_rank, a.master_addr, a.config)


if __name__ == "__main__":
    sys.exit(main())
