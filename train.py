#!/usr/bin/env python
"""Pretraining entry point; see `moe_b200/train_main.py`.

    ./scripts/train.sh configs/scaling/xs_standard.yaml
    python train.py --config configs/bench/tiny_cpu.yaml --device cpu
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from moe_b200.train_main import main  # noqa: E402
# names that the reference's tests and scripts import from `train`
from moe_b200.models import build_model, load_config  # noqa: E402,F401
from moe_b200.utils.bias_update import (bias_alpha_schedule, get_selected_experts_for_seq_aux,  # noqa: E402,F401
                                        update_expert_biases)
from moe_b200.utils.checkpoint import (cleanup_checkpoints, find_latest_checkpoint, load_checkpoint,  # noqa: E402,F401
                                       save_checkpoint)

if __name__ == "__main__":
    main()
