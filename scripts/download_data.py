#!/usr/bin/env python
"""Fetch the parquet shards of the training corpus into `data/parquet/`.

    python scripts/download_data.py                   # every shard of the default dataset repository
    python scripts/download_data.py --max_shards 64   # the first 64 shards (sorted by name)
    python scripts/download_data.py --workers 32      # download threads

Same job as the reference's `scripts/download_data.py:25-101` (and the copy inside its cluster launcher,
`modal_train.py:164-227`): list the `.parquet` files of the dataset repository, skip the ones already on disk,
download the rest in parallel, report failures and exit non-zero if any remain.  The hub is reached through a
small client object (`list_files()`, `download(name, out_dir)`), so the logic runs against a fake in tests and
against `huggingface_hub` in production; a shard is written under a temporary name and renamed when complete,
so an interrupted run never leaves a truncated file that a later run would skip.
"""
from __future__ import annotations

import argparse
import os
import sys
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

REPO_ID = "leonli66/latent-cot-finewebedu"
DEFAULT_OUT = Path("data/parquet")


class HubClient:
    """`huggingface_hub` behind the two calls the downloader needs."""

    def __init__(self, repo_id: str, token: str | None):
        from huggingface_hub import HfApi

        self.repo_id, self.token = repo_id, token
        self.api = HfApi(token=token)

    def list_files(self) -> list[str]:
        return list(self.api.list_repo_files(self.repo_id, repo_type="dataset"))

    def download(self, filename: str, out_dir: Path) -> Path:
        from huggingface_hub import hf_hub_download

        return Path(hf_hub_download(repo_id=self.repo_id, filename=filename, repo_type="dataset", token=self.token,
                                    cache_dir=None, local_dir=str(out_dir)))


def plan(client, out_dir: Path, max_shards: int | None = None) -> tuple[list[str], list[str]]:
    """(all selected shards, the ones still to fetch)."""
    files = sorted(f for f in client.list_files() if f.endswith(".parquet"))
    if max_shards is not None:
        files = files[:max_shards]
    return files, [f for f in files if not (out_dir / f).exists()]


def fetch_one(client, filename: str, out_dir: Path) -> Path:
    dest = out_dir / filename
    if dest.exists():
        return dest
    tmp_dir = out_dir / ".partial"
    tmp_dir.mkdir(parents=True, exist_ok=True)
    got = Path(client.download(filename, tmp_dir))
    dest.parent.mkdir(parents=True, exist_ok=True)
    os.replace(got, dest)  # complete files only under the final name
    return dest


def download_all(client, out_dir: Path, max_shards: int | None = None, workers: int = 16, log=print) -> list:
    """Returns the list of (shard, error text) that failed."""
    out_dir.mkdir(parents=True, exist_ok=True)
    files, todo = plan(client, out_dir, max_shards)
    log(f"Shards: {len(files)} total, {len(files) - len(todo)} already downloaded, {len(todo)} to fetch")
    log(f"Output: {out_dir.resolve()}")
    if not todo:
        log("All shards already present.")
        return []
    errors = []
    done = 0
    with ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
        futures = {pool.submit(fetch_one, client, f, out_dir): f for f in todo}
        for fut in as_completed(futures):
            name = futures[fut]
            try:
                fut.result()
                done += 1
            except Exception as e:  # keep going: one bad shard must not stop the others
                errors.append((name, str(e)))
                log(f"ERROR {name}: {e}")
            if (done + len(errors)) % 50 == 0:
                log(f"  {done + len(errors)} / {len(todo)}")
    log(f"\nDone. {done} downloaded, {len(errors)} failed.")
    for f, e in errors:
        log(f"  {f}: {e}")
    return errors


def parse_args(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--out_dir", default=str(DEFAULT_OUT))
    p.add_argument("--repo_id", default=REPO_ID)
    p.add_argument("--max_shards", type=int, default=None, help="Limit number of shards (default: all)")
    p.add_argument("--workers", type=int, default=16, help="Parallel download threads")
    return p.parse_args(argv)


def main(argv=None, client=None) -> int:
    args = parse_args(argv)
    if client is None:
        try:
            from dotenv import load_dotenv

            load_dotenv()
        except ImportError:
            pass
        token = os.environ.get("HF_TOKEN")
        if not token or token == "hf_...":
            print("ERROR: HF_TOKEN not set. Fill in .env first.", file=sys.stderr)
            return 2
        client = HubClient(args.repo_id, token)
    errors = download_all(client, Path(args.out_dir), args.max_shards, args.workers)
    return 1 if errors else 0


if __name__ == "__main__":
    sys.exit(main())
