"""Synthetic token stream: uniform-random ids in `[0, vocab)`, reproducible and resumable.

Used by the benchmarks (no dataset or tokenizer is reachable offline) and by tests.  Sample `i` of
rank `r` depends only on `(seed, r, i)`, so a resumed run continues the exact stream, and the
stream of a rank does not change with the number of other ranks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch.utils.data import IterableDataset


@dataclass
class SyntheticConfig:
    vocab_size: int = 151936
    seq_len: int = 2048
    seed: int = 0


class SyntheticTokenDataset(IterableDataset):
    def __init__(self, config: SyntheticConfig, rank: int = 0, world_size: int = 1):
        self.config, self.rank, self.world_size = config, rank, world_size
        self._idx = 0

    def get_state(self) -> dict:
        return {"sample_idx": self._idx}

    def set_state(self, state: dict) -> None:
        self._idx = int(state.get("sample_idx", 0))

    def sample(self, i: int) -> torch.Tensor:
        g = torch.Generator().manual_seed((self.config.seed * 1_000_003 + self.rank) * 1_000_003 + i)
        return torch.randint(0, self.config.vocab_size, (self.config.seq_len,), generator=g, dtype=torch.int64)

    def __iter__(self):
        while True:
            ids = self.sample(self._idx)
            self._idx += 1
            yield {"input_ids": ids, "labels": ids.clone()}
