"""Build the in-tree C-ABI shared library ``libb200lite.so`` with nvcc for sm_100a.

nvcc cross-compiles without a GPU, so this runs in the GPU-less build container; the ``.so``
then travels with the repo snapshot to the B200 box. No torch headers are involved: the
library only depends on the (statically linked) CUDA runtime.

Usage:
    python -m lite_llama_b200.build            # incremental
    python -m lite_llama_b200.build --force

``build(sources=...)`` compiles and links only the named sources (plus the library plumbing): a first run that
serves one model family does not wait for the kernels of the others.  A library that already holds the wanted
sources (a fuller build) is left alone; a later full build relinks.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
OUT = Path(__file__).resolve().parent / "libb200lite.so"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stamp(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(src: Path, force: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp_file = OBJ_DIR / (src.stem + ".stamp")
    stamp = _stamp(src)
    if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return obj


# plumbing every subset needs (error strings, launch counter, TMA descriptors)
BASE_SOURCES = ("core", "tma_desc")
# what the layer-list decoders launch between them: dense tcgen05 GEMM, fp32 / odd-shape / per-head / grouped GEMM,
# residual streams (sequential and parallel blocks), state-space and gated recurrences, attention, rotary and
# latent-attention kernels, expert routing, argmax and expert sum.  Each
# registered architecture names its own subset (executor.registry.Architecture.sources).
LAYERED_SOURCES = ("gemm_dense", "gemm_simt", "gemm_rows_mma", "residual_stream", "parallel_stream", "ssm_scan",
                   "decay_attention_mma", "gated_recurrence", "gated_linear_attention", "attention_sink", "rotary_heads", "latent_attention", "moe_routing", "elementwise")
LINK_STAMP = OBJ_DIR / "link.stamp"


def linked_sources() -> set[str]:
    """Source stems the current library was linked from (empty when there is none)."""
    if not OUT.exists() or not LINK_STAMP.exists():
        return set()
    return set(LINK_STAMP.read_text().split())


def build(force: bool = False, verbose: bool = True, sources: tuple[str, ...] | None = None) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    every = sorted(CSRC.glob("*.cu"))
    if not every:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    if sources is not None:
        wanted = set(BASE_SOURCES) | set(sources)
        have = linked_sources()
        if wanted <= have and not force:
            wanted = have                     # a fuller library is kept (and refreshed if its sources changed)
        every = [s for s in every if s.stem in wanted]
    with ThreadPoolExecutor(max_workers=min(8, len(every))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force), every))
    newest = max(o.stat().st_mtime for o in objs)
    stems = sorted(s.stem for s in every)
    if force or not OUT.exists() or OUT.stat().st_mtime < newest or linked_sources() != set(stems):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               "-o", str(OUT), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        LINK_STAMP.write_text(" ".join(stems))
        if verbose:
            print(f"[b200lite] linked {OUT} from {len(objs)} objects")
    elif verbose:
        print(f"[b200lite] {OUT.name} is up to date")
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv)
