"""Build step of the package: generate the tables, compile the CUDA library for sm_100a (in-tree) and the synthetic
corpus generator.  nvcc cross-compiles without a GPU.  (The test-side helpers, the CPU oracle and the host emulation
backend, are built by tests/build_helpers.py.)

    python -m zluda_b200.build            build everything that is out of date
    python -m zluda_b200.build --force
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libptxfe.so")
CORPUS_LIB = os.path.join(PKG, "libptxcorpus.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def _run(cmd, **kw):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))
    return r.stdout


def generate():
    g = os.path.join(PKG, "grammar")
    _run([sys.executable, os.path.join(g, "gen_tables.py"), "--out", os.path.join(CSRC, "gen")])
    _run([sys.executable, os.path.join(g, "gen_pow5.py"), "--out", os.path.join(CSRC, "gen")])
    _run([sys.executable, os.path.join(g, "gen_lex_tables.py"), "--out", os.path.join(CSRC, "gen")])


def build_library(force=False):
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".h", ".cpp"))]
    srcs += [os.path.join(CSRC, "gen", f) for f in os.listdir(os.path.join(CSRC, "gen"))]
    srcs.append(os.path.join(ROOT, "include", "ptxfe.h"))
    if not force and not _newer(LIB, srcs):
        return ""
    obj = os.path.join(CSRC, "ptxfe_dump.o")
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-c", os.path.join(CSRC, "ptxfe_dump.cpp"), "-o", obj])
    log = _run([NVCC] + NVCC_FLAGS + ["-shared", "-o", LIB, os.path.join(CSRC, "ptxfe.cu"), obj])
    with open(os.path.join(CSRC, "ptxas.log"), "w") as f:
        f.write(log)
    return log


def build_corpus_generator(force=False):
    """The synthetic-corpus generator (plain C, host only): used by the benchmark, the smoke run and the tests."""
    src = os.path.join(CSRC, "ptx_corpus.c")
    if force or _newer(CORPUS_LIB, [src]):
        _run(["gcc", "-O2", "-fPIC", "-shared", "-o", CORPUS_LIB, src, "-lm"])


def build(force=False):
    generate()
    log = build_library(force)
    build_corpus_generator(force)
    return log


if __name__ == "__main__":
    out = build("--force" in sys.argv)
    if "-v" in sys.argv:
        print(out)
    print("built", LIB)
