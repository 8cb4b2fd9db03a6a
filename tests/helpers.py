import torch


def tiny_cfg(mtype="standard_moe", **kw):
    m = dict(type=mtype, vocab_size=256, hidden_size=64, num_hidden_layers=2, head_dim=16, num_attention_heads=4,
             num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    if mtype == "dense":
        m["intermediate_size"] = 128
    else:
        m.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, router_aux_loss_coef=0.01)
        if "global" in mtype:
            m["num_experts"] = 16
        if mtype.startswith("deepseek"):
            m.update(seq_aux_loss_coef=1e-3, bias_update_rate=1e-3, topk_scaling_factor=2.5, num_groups=4,
                     group_topk=2)
    m.update(kw)
    return {"model": m}


def batch(vocab=256, B=2, S=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (B, S), generator=g)
