"""Diagnostics a user runs by hand (`python -m moe_b200.diagnostics.<name>`): the capabilities of the
reference's `scripts/compare_training_steps.py`, `scripts/debug_tiny_global_vs_perlayer.py` and
`scripts/full_audit.py`, on synthetic data so that they work offline."""
