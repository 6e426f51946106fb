"""Builds libb200_fattn.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200_fattn.so")
STAMP = LIB + ".srchash"   # hash of the sources and flags the library next to it was built from
SOURCES = ["fattn_api.cu", "fattn_mma.cu", "fattn_tc5.cu", "kv_slab.cu", "relpos_table.cu", "segment_sched.cpp", "slice_batch.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def source_hash() -> str:
    """SHA-256 over every file under csrc/, the public header and the compiler flags."""
    h = hashlib.sha256()
    files = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [os.path.join(HERE, "..", "include", "b200_fattn.h")]
    for path in files:
        h.update(os.path.basename(path).encode() + b"\0")
        h.update(open(path, "rb").read())
    h.update(" ".join(NVCC_FLAGS + SOURCES).encode())
    return h.hexdigest()


def built_hash() -> str | None:
    """The source hash recorded when the library in the tree was linked, or None."""
    try:
        return open(STAMP).read().strip() if os.path.exists(LIB) else None
    except OSError:
        return None


def needs_build() -> bool:
    return built_hash() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    if shutil.which(_nvcc()) is None and not os.path.exists(_nvcc()):
        raise RuntimeError(
            f"{LIB} is missing or was built from other sources (recorded {built_hash()}, tree {source_hash()}) "
            "and there is no nvcc to rebuild it with")
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in sources():
        obj = os.path.join(HERE, "build", os.path.basename(src) + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart", "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    with open(STAMP, "w") as f:
        f.write(source_hash() + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
