"""Stateful parquet text dataset (`src/data/parquet_dataset.py:24-150` of the reference).

Parquet files under `data_dir` are sorted, shuffled with a fixed seed and dealt to ranks
round-robin; each text row is tokenised, terminated with EOS and packed into a rolling token
buffer from which windows of `seq_len + 1` tokens sliding by `seq_len` are cut.

Differences from the reference, all on purpose:
  * the position is the absolute window index inside the current file, and the leftover token
    buffer is part of the state, so resuming is exact, also at file boundaries and more than once;
  * labels are the inputs (the model shifts once); `reference_double_shift=True` restores the
    reference's pre-shifted labels (`chunk[1:]`), which the model then shifts a second time;
  * `prefetch > 0` tokenises on a background thread and hands batches over together with the
    state that reproduces the stream after them.
"""
from __future__ import annotations

import glob
import json
import os
import queue
import random
import threading
from dataclasses import dataclass
from typing import Iterator

import torch
from torch.utils.data import IterableDataset


@dataclass
class DataConfig:
    data_dir: str = "./data/parquet"
    text_column: str = "text"
    seq_len: int = 2048
    tokenizer_name: str = "gpt2"
    num_workers: int = 4
    reference_double_shift: bool = False
    prefetch: int = 0


class StatefulParquetDataset(IterableDataset):
    def __init__(self, config: DataConfig, tokenizer, rank: int = 0, world_size: int = 1, seed: int = 42):
        self.config, self.tokenizer, self.rank, self.world_size = config, tokenizer, rank, world_size
        all_files = sorted(set(glob.glob(os.path.join(config.data_dir, "**/*.parquet"), recursive=True)
                               + glob.glob(os.path.join(config.data_dir, "*.parquet"))))
        if not all_files:
            raise FileNotFoundError(f"No parquet files found in {config.data_dir}")
        random.Random(seed).shuffle(all_files)  # own generator: the global RNG is left alone
        self.files = [f for i, f in enumerate(all_files) if i % world_size == rank]
        self._start = {"file_idx": 0, "seq_idx": 0, "buffer": []}
        self._cur = dict(self._start)

    # ------------------------------------------------------------------ state
    def get_state(self) -> dict:
        return {"file_idx": self._cur["file_idx"], "seq_idx": self._cur["seq_idx"],
                "buffer": list(self._cur["buffer"])}

    def set_state(self, state: dict) -> None:
        self._start = {"file_idx": int(state.get("file_idx", 0)), "seq_idx": int(state.get("seq_idx", 0)),
                       "buffer": list(state.get("buffer", []))}
        self._cur = dict(self._start)

    def save_state(self, path: str) -> None:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump(self.get_state(), f)

    def load_state(self, path: str) -> None:
        if os.path.exists(path):
            with open(path) as f:
                self.set_state(json.load(f))

    # -------------------------------------------------------------- iteration
    def _load_file(self, path: str):
        import pandas as pd

        return pd.read_parquet(path, columns=[self.config.text_column])

    def _windows(self) -> Iterator[tuple[dict, dict]]:
        """Yields (sample, state-after-sample); at the end of a file (None, state at the start of the next file).
        `_cur` is only ever assigned by the consumer, so a read-ahead worker cannot move it past what was
        handed out."""
        seq_len = self.config.seq_len
        eos = self.tokenizer.eos_token_id or 0
        start = self._start
        # `buffer` in the state is the carry-over at the START of file `file_idx`; windows already
        # consumed from that file are re-derived and skipped, so the same state resumes many times.
        carry = list(start["buffer"])
        for file_idx in range(start["file_idx"], len(self.files)):
            buf = list(carry)
            file_carry = list(carry)
            skip = start["seq_idx"] if file_idx == start["file_idx"] else 0
            produced = 0
            df = self._load_file(self.files[file_idx])
            for text in df[self.config.text_column]:
                if not isinstance(text, str) or not text.strip():
                    continue
                buf.extend(self.tokenizer.encode(text, add_special_tokens=False))
                buf.append(eos)
                pos = 0
                while len(buf) - pos >= seq_len + 1:
                    chunk = buf[pos:pos + seq_len + 1]
                    pos += seq_len
                    produced += 1
                    if produced <= skip:
                        continue
                    ids = torch.tensor(chunk[:-1], dtype=torch.long)
                    labels = torch.tensor(chunk[1:], dtype=torch.long) if self.config.reference_double_shift \
                        else ids.clone()
                    state = {"file_idx": file_idx, "seq_idx": produced, "buffer": file_carry}
                    yield {"input_ids": ids, "labels": labels}, state
                if pos:
                    del buf[:pos]
            carry = buf
            start = {"file_idx": file_idx + 1, "seq_idx": 0, "buffer": list(carry)}
            yield None, dict(start)

    def __iter__(self) -> Iterator[dict]:
        if self.config.prefetch <= 0:
            for sample, state in self._windows():
                self._cur = state
                if sample is not None:
                    yield sample
            return
        q: queue.Queue = queue.Queue(maxsize=self.config.prefetch)
        stop = threading.Event()

        def work():
            try:
                for item in self._windows():
                    while not stop.is_set():
                        try:
                            q.put(item, timeout=0.1)
                            break
                        except queue.Full:
                            continue
                    if stop.is_set():
                        return
                q.put(None)
            except BaseException as e:  # surfaced on the consumer side
                q.put(e)

        th = threading.Thread(target=work, daemon=True)
        th.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, BaseException):
                    raise item
                sample, state = item
                self._cur = state  # state of the sample handed out, not of what the worker has read ahead
                if sample is not None:
                    yield sample
        finally:
            stop.set()
