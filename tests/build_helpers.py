"""Builds the test-side helpers: the CPU oracle (oracle/, by its Makefile) and the host emulation backend of the
pipeline (tests/emu/).  Test infrastructure only; the package's own build is zluda_b200/build.py.

    python tests/build_helpers.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(ROOT, "zluda_b200", "csrc")


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build(force=False):
    _run(["make", "-C", os.path.join(ROOT, "oracle")] + (["-B"] if force else []))
    gen = os.path.join(CSRC, "gen")
    if not os.path.isdir(gen) or not os.listdir(gen):
        sys.path.insert(0, ROOT)
        from zluda_b200 import build as pkg_build
        pkg_build.generate()
    emu_src = os.path.join(HERE, "emu", "ptxfe_emu.cpp")
    emu = os.path.join(HERE, "emu", "libptxfe_emu.so")
    deps = [emu_src] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")] + [os.path.join(gen, f) for f in os.listdir(gen)]
    if force or _newer(emu, deps):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", emu, emu_src])


if __name__ == "__main__":
    build("--force" in sys.argv)
    print("built the oracle and the emulation backend")
