"""`modal run modal_train.py [--config configs/...yaml]`: the cluster of `moe_b200.cluster.ClusterSpec` as a
Modal app (2 nodes x 8 B200 by default, data and checkpoint volumes, 10 retries with auto-resume), and
`modal run modal_train.py::download_data` to fill the data volume.  Needs the `modal` package; on a plain
cluster use `python -m moe_b200.cluster_node` on every node instead."""
from moe_b200.cluster import ClusterSpec, build_modal_app

SPEC = ClusterSpec()
try:
    app, train, download_data = build_modal_app(SPEC)
except ImportError:  # importable without Modal: the spec is still usable
    app = train = download_data = None

if app is not None:
    @app.local_entrypoint()
    def main(config: str = SPEC.config_file):
        train.remote(config)
