"""Diagnostics a user runs by hand (`python -m moe_b200.diagnostics.<name>`), on synthetic data by default so
that they work offline: `compare_steps` (step-by-step loss table), `tiny_global_vs_perlayer`, `audit` (pipeline
checks) and `studies` (the research studies: long comparison with CSV, hidden-state similarity, identical-loss
checks, seed vs layout, dense vs MoE, learning-rate sweep, kernels vs plain ops, large-shape check, corpus vs
random tokens) on the shared `harness`."""
