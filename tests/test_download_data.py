"""The shard downloader against a fake hub (no network): listing, skipping, retry-ability, failures."""
import importlib.util
import os
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("download_data", ROOT / "scripts" / "download_data.py")
dd = importlib.util.module_from_spec(spec)
spec.loader.exec_module(dd)


class FakeHub:
    def __init__(self, names, fail=()):
        self.names, self.fail, self.calls = list(names), set(fail), []

    def list_files(self):
        return self.names + ["README.md", ".gitattributes"]

    def download(self, filename, out_dir):
        self.calls.append(filename)
        if filename in self.fail:
            raise OSError("connection reset")
        p = Path(out_dir) / filename
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_bytes(b"PAR1" + filename.encode())
        return p


def test_downloads_missing_shards_only_and_in_name_order(tmp_path):
    names = [f"data/shard-{i:04d}.parquet" for i in (3, 1, 2, 0)]
    hub = FakeHub(names)
    (tmp_path / "data").mkdir()
    (tmp_path / "data" / "shard-0001.parquet").write_bytes(b"old")
    assert dd.main(["--out_dir", str(tmp_path), "--max_shards", "3", "--workers", "2"], client=hub) == 0
    assert sorted(hub.calls) == ["data/shard-0000.parquet", "data/shard-0002.parquet"]  # first three, one present
    assert (tmp_path / "data" / "shard-0001.parquet").read_bytes() == b"old"
    assert not (tmp_path / "data" / "shard-0003.parquet").exists()
    assert dd.main(["--out_dir", str(tmp_path), "--max_shards", "3"], client=FakeHub(names)) == 0  # nothing left


def test_failures_are_reported_and_leave_no_partial_file(tmp_path):
    names = [f"s{i}.parquet" for i in range(4)]
    hub = FakeHub(names, fail={"s2.parquet"})
    logs = []
    errors = dd.download_all(hub, tmp_path, workers=3, log=logs.append)
    assert [e[0] for e in errors] == ["s2.parquet"] and "connection reset" in errors[0][1]
    assert not (tmp_path / "s2.parquet").exists() and (tmp_path / "s3.parquet").exists()
    assert dd.main(["--out_dir", str(tmp_path)], client=hub) == 1  # still failing: non-zero exit
    hub.fail.clear()
    assert dd.main(["--out_dir", str(tmp_path)], client=hub) == 0 and (tmp_path / "s2.parquet").exists()


def test_missing_token_is_refused(monkeypatch, tmp_path):
    monkeypatch.delenv("HF_TOKEN", raising=False)
    monkeypatch.chdir(tmp_path)
    assert dd.main(["--out_dir", str(tmp_path)]) == 2
