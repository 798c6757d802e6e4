"""Builds libfbgemm_b200.so in-tree with nvcc for sm_100a.

    python -m fbgemm_b200.build [--force] [--verbose]

The shared library holds the hand-written CUDA kernels, the C ABI
(include/fbgemm_b200/embedding_c_api.h) and the C++ generator templates
(include/fbgemm_b200/FbgemmEmbedding.h).  There is deliberately no arch list
and no CPU fallback: the one target is compute_100a / sm_100a.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG_DIR, "libfbgemm_b200.so")
STAMP_PATH = os.path.join(PKG_DIR, "csrc", ".build_stamp")

CUDA_SOURCES = ["spmdm_kernels.cu", "spmdm_direct_8.cu", "spmdm_direct_4.cu", "spmdm_direct_2.cu", "scan_kernels.cu", "quantize_kernels.cu", "remap_kernels.cu", "pruned_lookup_kernels.cu", "sequence_kernels.cu", "stage_kernels.cu", "plain_kernels.cu", "c_api.cu", "noalloc_entry.cu", "peer_sync_kernels.cu", "multi_host.cu"]
CXX_SOURCES = ["generators.cc"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    # IEEE arithmetic everywhere: results must be bit-equal to the CPU reference.
    "-ftz=false", "-prec-div=true", "-prec-sqrt=true", "-fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libfbgemm_b200.so cannot be built")


def _sources():
    out = [os.path.join(CSRC, s) for s in CUDA_SOURCES + CXX_SOURCES]
    return [s for s in out if os.path.exists(s)]


def _fingerprint() -> str:
    h = hashlib.sha256()
    paths = _sources()
    for d in (CSRC, os.path.join(INCLUDE, "fbgemm_b200")):
        for name in sorted(os.listdir(d)):
            if name.endswith((".h", ".cuh")):
                paths.append(os.path.join(d, name))
    for p in sorted(set(paths)):
        h.update(os.path.relpath(p, ROOT).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(f for f in NVCC_FLAGS if not f.startswith(ROOT)).encode())
    return h.hexdigest()


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(STAMP_PATH):
        return True
    with open(STAMP_PATH) as f:
        return f.read().strip() != _fingerprint()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if sources changed (or ``force``); return the library path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in _sources():
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("FBGEMM_B200_EXTRA_NVCC", "").split(), "-c", src, "-o", obj]
        if src.endswith(".cc"):
            cmd.insert(1, "-x")
            cmd.insert(2, "cu")
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src}\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    with open(STAMP_PATH, "w") as f:
        f.write(_fingerprint())
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
