"""Reference arm of `bench.py`: the unmodified reference package (`baseline/_ref/src`, installed
from the reference tree) driven through its own model classes and training utilities.

What is the reference's and what is not:
  * from the reference, unchanged: `StandardMoEModel` / `GlobalMoEForCausalLM` (+ HF Qwen3-MoE
    underneath), `build_optimizer`, `build_lr_scheduler`, `get_grad_norm`, the Liger monkey-patch
    applied before the models are imported, the cuBLASLt preference, the `grouped_mm` experts
    implementation with its `eager` fallback, bf16 autocast, clip at `max_grad_norm`;
  * substituted, because the reference's `train.py` cannot start offline (it imports `accelerate`,
    which this image does not have, downloads a tokenizer and needs parquet shards): the loop
    body of `train.py:546-572` is restated here with torch DDP in place of Accelerate's wrapper
    and synthetic uniform-random token ids in place of the parquet stream.
"""
from __future__ import annotations

import os
import sys


def _build(cfg: dict, ref_dir: str):
    import torch

    torch.backends.cuda.preferred_blas_library("cublaslt")
    sys.path.insert(0, ref_dir)
    liger = "applied"
    try:
        from liger_kernel.transformers import apply_liger_kernel_to_qwen3_moe

        apply_liger_kernel_to_qwen3_moe()
    except Exception as e:  # recorded in the output line
        liger = f"not applied ({type(e).__name__})"
    from src.models import (GlobalMoEConfig, GlobalMoEForCausalLM, Qwen3MoeConfig, StandardMoEModel)
    from src.utils.training import TrainingConfig, build_lr_scheduler, build_optimizer, get_grad_norm

    m = cfg["model"]
    common = dict(
        vocab_size=m["vocab_size"], hidden_size=m["hidden_size"], num_hidden_layers=m["num_hidden_layers"],
        head_dim=m["head_dim"], num_attention_heads=m["num_attention_heads"],
        num_key_value_heads=m["num_key_value_heads"], moe_intermediate_size=m["moe_intermediate_size"],
        intermediate_size=m.get("intermediate_size", m["moe_intermediate_size"] * 4),
        max_position_embeddings=m.get("max_position_embeddings", 32768), rope_theta=m.get("rope_theta", 1e6),
        rms_norm_eps=m.get("rms_norm_eps", 1e-6), tie_word_embeddings=m.get("tie_word_embeddings", False),
        router_aux_loss_coef=m.get("router_aux_loss_coef", 0.001), norm_topk_prob=m.get("norm_topk_prob", True),
        num_experts_per_tok=m["num_experts_per_tok"], output_router_logits=True)
    if m["type"] == "standard_moe":
        config = Qwen3MoeConfig(num_experts=m["num_experts"], **common)
        model = StandardMoEModel(config)
    elif m["type"] == "global_moe":
        config = GlobalMoEConfig(num_experts=m["num_experts"], **common)
        model = GlobalMoEForCausalLM(config)
    else:
        raise ValueError(f"reference arm: model type {m['type']} not wired")
    # the reference's own selection (`train.py:241-245`): grouped_mm, and `eager` when that raises; what ran and
    # why is recorded, together with the class that actually computes the experts (Liger replaces HF's)
    impl = "grouped_mm"
    try:
        model.set_experts_implementation("grouped_mm")
    except Exception as e:
        impl = f"eager (grouped_mm raised {e!r})"
        try:
            model.set_experts_implementation("eager")
        except Exception as e2:
            impl += f"; eager raised {e2!r}"
    inner = getattr(model, "model", model)
    bank = getattr(inner, "global_experts", None)
    if bank is None:
        bank = inner.layers[0].mlp.experts
    impl += f", experts module {type(bank).__module__}.{type(bank).__name__}"
    t = cfg["training"]
    tcfg = TrainingConfig(
        learning_rate=t["learning_rate"], weight_decay=t["weight_decay"], beta1=t.get("beta1", 0.9),
        beta2=t.get("beta2", 0.95), max_grad_norm=t["max_grad_norm"], lr_scheduler=t["lr_scheduler"],
        warmup_steps=t["warmup_steps"], max_steps=t["max_steps"], min_lr_ratio=t["min_lr_ratio"],
        batch_size=t["batch_size"], gradient_accumulation=t["gradient_accumulation"],
        mixed_precision=t["mixed_precision"], log_every=t["log_every"], save_every=t["save_every"],
        output_dir=t["output_dir"], wandb_project=None)
    return model, config, tcfg, build_optimizer, build_lr_scheduler, get_grad_norm, liger, impl


def run(args, root, dist_setup, timed_region, make_batches, load_bench_config) -> dict:
    import torch

    rank, local, world = dist_setup(args.gpus)
    cfg = load_bench_config(args.config, args.batch, args.seq)
    torch.manual_seed(42 + rank)
    model, mcfg, tcfg, build_optimizer, build_lr_scheduler, get_grad_norm, liger, impl = _build(
        cfg, os.path.join(root, "baseline", "_ref"))
    model = model.to(f"cuda:{local}")
    model.train()
    raw = model
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])
    opt = build_optimizer(raw, tcfg)
    sched = build_lr_scheduler(opt, tcfg)
    B, S, V = tcfg.batch_size, cfg["data"]["seq_len"], cfg["model"]["vocab_size"]
    K, W = args.steps, args.warmup
    host = make_batches(W + 2 * K, B, S, V, rank, cfg["data"].get("seed", 0))

    def train_step(ids):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(input_ids=ids, labels=ids, output_router_logits=True)
        out.loss.backward()
        get_grad_norm(raw)
        torch.nn.utils.clip_grad_norm_(raw.parameters(), tcfg.max_grad_norm)
        opt.step()
        opt.zero_grad()
        sched.step()
        return out.loss

    for i in range(W):
        train_step(host[i].cuda(non_blocking=True))
    torch.cuda.synchronize()
    dev_batches = [b.cuda(non_blocking=True) for b in host[W:W + K]]
    last = {}

    def step_dev(i):
        last["loss"] = train_step(dev_batches[i])

    ms, clocks = timed_region(step_dev, K, world, local)
    losses = []

    def step_e2e(i):
        losses.append(float(train_step(host[W + K + i].cuda(non_blocking=True)).item()))

    ms_e2e, clocks_e2e = timed_region(step_e2e, K, world, local)
    tokens = B * S * world * K
    return {
        "metric": "train_tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": f"{args.config} ({cfg['model']['type']})", "global_batch": B * world,
                   "micro_batch_per_gpu": B, "seq_len": S, "parallelism": f"dp{world}",
                   "stack": f"HF transformers Qwen3-MoE + Liger ({liger}) + experts={impl} + torch DDP "
                            f"(accelerate is not in this image) + reference AdamW/LR/clip, bf16 autocast"},
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tok/s", "ms_per_step": ms_e2e / K,
                "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4, "clocks": clocks_e2e},
        "gpu_launches": None,  # kernels of this repository: none run in this arm (not counted, not zero by measurement)
        "clocks": clocks, "loss_last": float(last["loss"].item()), "loss_e2e_last": losses[-1],
        # rank 0's loss of every end-to-end step (same synthetic token stream in both arms)
        "losses_e2e": [round(x, 4) for x in losses[:256]],
    }
