"""Host-side rules that pick a kernel form (no GPU needed): pair tiles, weight folding, gathered operands, the fused
QKV epilogue and the contraction split of short, wide weight gradients."""
import torch

from moe_b200.ops import gemm as G


def test_pair_tiles_and_switch(monkeypatch):
    monkeypatch.delenv("MOE_B200_GEMM_PAIR", raising=False)
    assert G._use_pair(256, 128, None) and not G._use_pair(128, 1024, None) and not G._use_pair(4096, 64, None)
    monkeypatch.setenv("MOE_B200_GEMM_PAIR", "0")
    assert not G._use_pair(4096, 4096, None)


def test_expert_path_switches(monkeypatch):
    for v in ("MOE_B200_GEMM_PAIR", "MOE_B200_MOE_FOLD", "MOE_B200_MOE_GATHER"):
        monkeypatch.delenv(v, raising=False)
    # routing weight in the epilogues by default where the 256-wide SwiGLU tiles apply; gathered operand loads opt-in
    assert G.fold_supported(1024, 1536) and not G.gather_supported(1024, 1536)
    assert not G.fold_supported(1024, 256) and not G.fold_supported(128, 1536)
    monkeypatch.setenv("MOE_B200_MOE_GATHER", "1")
    assert G.gather_supported(1024, 1536)
    monkeypatch.setenv("MOE_B200_MOE_FOLD", "0")
    assert not G.fold_supported(1024, 1536) and not G.gather_supported(1024, 1536)


def test_fused_qkv_epilogue_rule(monkeypatch):
    monkeypatch.delenv("MOE_B200_QKV_FUSED", raising=False)
    monkeypatch.delenv("MOE_B200_GEMM_PAIR", raising=False)
    assert G.qkv_rope_supported(16384, 4096, 1024, 128)
    assert not G.qkv_rope_supported(16384, 2048, 1024, 64)   # head_dim 64: stand-alone kernel
    assert not G.qkv_rope_supported(128, 4096, 1024, 128)    # fewer rows than a pair tile
    monkeypatch.setenv("MOE_B200_QKV_FUSED", "0")
    assert not G.qkv_rope_supported(16384, 4096, 1024, 128)


def test_contraction_split_segments():
    G._SPLIT_SEG.clear()
    seg = G._split_k_segments(16384, torch.device("cpu"))
    assert seg.dtype == torch.int32 and seg.numel() == 65 and seg[0] == 0 and seg[-1] == 16384
    assert int((seg[1:] - seg[:-1]).unique().item()) == 256  # equal pieces of whole 64-row blocks
    seg = G._split_k_segments(64 * 9, torch.device("cpu"))     # 9 blocks: 9 pieces
    assert seg.numel() == 10 and seg[-1] == 576
    assert G._split_k_segments(64 * 7, torch.device("cpu")) is None   # fewer than 8 pieces: not worth a split
    assert G._split_k_segments(1000, torch.device("cpu")) is None     # not whole 64-row blocks
    G._SPLIT_SEG.clear()
