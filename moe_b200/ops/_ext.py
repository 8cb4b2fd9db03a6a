"""Build and load the sm_100a extension (`moe_b200/_C*.so`) in-tree.

`.cu` files are compiled by nvcc without any torch header (fast), the two
binding files by g++ against torch, and everything is linked into one shared
object next to the package.  A content hash of the sources decides whether a
rebuild is needed, so a tree copied to another machine (fresh mtimes) reuses
the shipped binary.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
_ROOT = _PKG.parent
_CSRC = _ROOT / "csrc"
_NAME = "_C"
_SO = _PKG / f"{_NAME}{sysconfig.get_config_var('EXT_SUFFIX')}"
_HASH = _PKG / f"{_NAME}.hash"
_OBJ = _ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

_module = None

# Kernels enqueued per binding call; `launch_count()` sums them (used by bench.py's gpu_launches).
KERNELS_PER_CALL = {"gemm": 1, "rmsnorm_fwd": 1, "rmsnorm_bwd": 2, "qknorm_rope_fwd": 1, "qknorm_rope_bwd": 2,
                    "router_fwd": 1, "router_bwd": 1, "moe_plan": 3, "moe_gather": 1, "moe_combine": 1,
                    "moe_combine_bwd": 1, "moe_slot_dot": 1, "moe_row_dot_reduce": 1, "lse_loss": 1, "lce_reduce": 1, "dlogits_": 1, "embed_fwd": 1, "embed_bwd": 1, "embed_sort": 1, "sumsq": 2,
                    "clip_coef": 1, "adamw": 1, "cast_bf16": 1, "sum_partials": 1, "allreduce": 1, "allgather_bf16": 1, "router_colsum": 1, "router_part_reduce": 1, "moe_aux": 1, "peer_barrier": 1, "clip_coef_multi": 1, "ep_exchange": 1, "ep_dispatch": 1}
_launches = 0


class _Counting:
    """Attribute proxy over the extension module that counts kernel launches."""

    def __init__(self, mod):
        self._mod = mod

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        n = KERNELS_PER_CALL.get(name, 0)
        if n == 0:
            return fn

        def call(*a, **k):
            global _launches
            _launches += n
            return fn(*a, **k)

        setattr(self, name, call)
        return call


def launch_count() -> int:
    return _launches


def add_launches(n: int) -> None:
    """Account for kernels that run without passing through the bindings (CUDA-graph replays)."""
    global _launches
    _launches += n


def sources() -> tuple[list[Path], list[Path], list[Path]]:
    cu = sorted(_CSRC.rglob("*.cu"))
    cpp = sorted(_CSRC.rglob("*.cpp"))
    hdr = sorted(list(_CSRC.rglob("*.cuh")) + list(_CSRC.rglob("*.h")))
    return cu, cpp, hdr


def _digest() -> str:
    h = hashlib.sha256()
    cu, cpp, hdr = sources()
    for p in cu + cpp + hdr:
        h.update(str(p.relative_to(_ROOT)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_built() -> bool:
    return _SO.exists() and _HASH.exists() and _HASH.read_text().strip() == _digest()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the extension."""
    if not force and is_built():
        return _SO
    import torch.utils.cpp_extension as ce

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    cu, cpp, _ = sources()
    _OBJ.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{_CSRC}"]
    jobs = []
    objs = []
    for s in cu:
        o = _OBJ / (str(s.relative_to(_CSRC)).replace("/", "_") + ".o")
        objs.append(o)
        jobs.append([nvcc, *NVCC_FLAGS, f"-I{_CSRC}", "-c", str(s), "-o", str(o)])
    for s in cpp:
        o = _OBJ / (str(s.relative_to(_CSRC)).replace("/", "_") + ".o")
        objs.append(o)
        jobs.append([
            "g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=" + _NAME,
            "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1", *inc, "-c", str(s), "-o", str(o),
        ])
    if verbose:
        print(f"[moe_b200] compiling {len(jobs)} translation units", file=sys.stderr)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        list(ex.map(_run, jobs))
    libs = [f"-L{p}" for p in ce.library_paths("cuda")]
    tlib = ce.library_paths("cuda")[0]
    link = [
        "g++", "-shared", "-o", str(_SO), *[str(o) for o in objs], *libs, f"-Wl,-rpath,{tlib}",
        "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
    ]
    _run(link)
    _HASH.write_text(_digest())
    return _SO


def load(build_if_missing: bool = True):
    """Import the extension module; build it first when allowed and needed."""
    global _module
    if _module is not None:
        return _module
    if not is_built():
        if not build_if_missing:
            raise RuntimeError("moe_b200._C is not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
        build()
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    spec = importlib.util.spec_from_file_location(f"moe_b200.{_NAME}", _SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[f"moe_b200.{_NAME}"] = mod
    _module = _Counting(mod)
    return _module


def available() -> bool:
    try:
        import torch

        return torch.cuda.is_available() and (is_built() or True)
    except Exception:
        return False
