"""The batch driver (directory -> one parse batch): file discovery on the CPU, verdicts against the oracle on the GPU."""
import os

import pytest

import cases
from zluda_b200 import corpus, precompile


def _make_tree(root):
    mods = corpus.config1(n_modules=6, total_bytes=96 << 10, pool_lines=2000)
    files = {}
    for i, m in enumerate(mods):
        files["lib%d/k%d.ptx" % (i % 2, i)] = m
    files["lib0/broken.ptx"] = cases.body("bogus_op %r1;").encode()
    files["lib1/lexerr.ptx"] = cases.body("add.s32 %r1, %r2, #;").encode()
    files["lib1/notes.txt"] = b"not ptx"
    files["empty.ptx"] = b""
    for rel, data in files.items():
        p = os.path.join(root, rel)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        with open(p, "wb") as f:
            f.write(data)
    os.symlink(os.path.join(root, "lib0"), os.path.join(root, "link_to_lib0"))
    return files


def test_file_discovery(tmp_path):
    files = _make_tree(str(tmp_path))
    found = precompile.find_ptx_files(str(tmp_path))
    rel = [os.path.relpath(p, str(tmp_path)) for p in found]
    assert rel == sorted(r for r in files if r.endswith(".ptx"))
    with_links = precompile.find_ptx_files(str(tmp_path), follow_links=True)
    assert len(with_links) == len(found) + sum(1 for r in files if r.startswith("lib0/") and r.endswith(".ptx"))
    assert precompile.find_ptx_files(found[0]) == [found[0]]


@pytest.mark.gpu
def test_verdicts_match_the_oracle(tmp_path, oracle, capsys):
    import zluda_b200
    _make_tree(str(tmp_path))
    paths = precompile.find_ptx_files(str(tmp_path))
    ctx = zluda_b200.Context(0)
    for ignore in (False, True):
        results, seconds, nbytes = precompile.parse_files(ctx, paths, ignore_errors=ignore)
        for p, ok, nerr in results:
            st, dump = oracle.parse(open(p, "rb").read(), 1 if ignore else 0)
            assert ok == (st == 0), (p, ignore)
    ctx.close()
    assert precompile.main([str(tmp_path), "--quiet"]) == 1          # broken files fail a checked run
    assert precompile.main([str(tmp_path), "--ignore-errors"]) == 0
    out = capsys.readouterr().out
    assert "[1/2]" in out and "[2/2]" in out and "parse:" in out
