"""Build libdm_b200.so (the C-ABI library with every CUDA kernel) in-tree with nvcc for sm_100a.

    python -m delta_matching_b200.build [--force] [--verbose]

One nvcc invocation per translation unit (objects cached under delta_matching_b200/build/ by source hash), then one
link into delta_matching_b200/libdm_b200.so.  No --use_fast_math anywhere: the quantizers need IEEE division and
explicitly rounded operations for bit-exact codes, and the attention kernels ask for approximate instructions by name.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdm_b200.so")
OBJ = os.path.join(HERE, "build")
SOURCES = ["dm_host.cu", "dm_quant.cu", "dm_probe.cu", "dm_fwd.cu", "dm_delta.cu", "dm_bwd1.cu", "dm_bwd2.cu", "dm_compose.cu", "dm_fwd256.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if c and os.path.isfile(c):
            return c
    raise RuntimeError("nvcc not found (set NVCC)")


def _digest(paths):
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        h.update(open(p, "rb").read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def source_files():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.isfile(os.path.join(CSRC, s))]


def code_sha():
    """12-hex content hash of the kernel sources and the public header (the numerics identity stamp)."""
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(os.path.dirname(HERE), "include", "dm_b200.h"))
    return _digest(files)[:12]


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "dm_b200.h"))
    srcs = source_files()
    objs, jobs = [], []
    for s in srcs:
        tag = _digest([s] + headers)
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + "." + tag + ".o")
        objs.append(o)
        if force or not os.path.isfile(o):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(o[:-2] + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + log)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{log}")
        if verbose:
            print(log)
        return o

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    stamp = os.path.join(OBJ, "link.stamp")
    want = " ".join(objs)
    if force or jobs or not os.path.isfile(OUT) or not os.path.isfile(stamp) or open(stamp).read() != want:
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        open(stamp, "w").write(want)
    keep = {os.path.basename(o) for o in objs} | {os.path.basename(o)[:-2] + ".log" for o in objs} | {"link.stamp"}
    for f in os.listdir(OBJ):          # objects of earlier source versions
        if f not in keep:
            os.remove(os.path.join(OBJ, f))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
