"""Ahead-of-time build of libictc_b200.so for sm_100a (nvcc cross-compiles without a GPU).

    python build.py [--force] [--verbose]

Objects go to csrc/build/, the library to ictc_o3/lib/libictc_b200.so (in-tree, git-ignored).
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT_DIR = os.path.join(PKG, "ictc_o3", "lib")
LIB = os.path.join(OUT_DIR, "libictc_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr"]


def units():
    sys.path.insert(0, HERE)
    import gen_tables
    gen_tables.main()
    res = [(f"tp_spec_{gen_tables.spec_name(s)}", "tp_spec.cu", [f"-DICTC_SPEC={gen_tables.spec_name(s)}"])
           for s in gen_tables.TP_SPECS]
    for name in sorted(os.listdir(HERE)):
        if name.endswith(".cu") and name != "tp_spec.cu":
            res.append((name[:-3], name, []))
    return res


def digest(src, extra):
    h = hashlib.sha256()
    h.update(" ".join(FLAGS + extra).encode())
    for root in (HERE, os.path.join(HERE, "generated"), os.path.join(PKG, "..", "include")):
        for name in sorted(os.listdir(root)):
            if name.endswith((".cuh", ".h")) or name == src:
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode())
                    h.update(f.read())
    return h.hexdigest()


def compile_one(job):
    name, src, extra, force, verbose = job
    obj = os.path.join(HERE, "build", name + ".o")
    stamp = obj + ".sha"
    dg = digest(src, extra)
    if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dg:
        return name, "cached", ""
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + extra + ["-c", os.path.join(HERE, src), "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{p.stdout}\n{p.stderr}")
    with open(stamp, "w") as f:
        f.write(dg)
    return name, "built", p.stderr


def build(force=False, verbose=False):
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    os.makedirs(OUT_DIR, exist_ok=True)
    jobs = [(n, s, e, force, verbose) for n, s, e in units()]
    rebuilt = False
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for name, state, log in ex.map(compile_one, jobs):
            rebuilt |= state == "built"
            if verbose:
                print(f"[{state}] {name}\n{log}")
    objs = [os.path.join(HERE, "build", n + ".o") for n, _s, _e, _f, _v in jobs]
    if rebuilt or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}\n{p.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
