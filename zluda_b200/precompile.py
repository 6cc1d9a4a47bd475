"""Batch driver: every `.ptx` file under a directory through ONE ptxfe_parse_batch call.

The caller side of the parser in the reference is `zluda_precompile` (zluda_precompile/src/main.rs:29-125: walk a
directory, optionally following links, hand every module found to the compiler from a pool of worker threads) and
`compiler` (compiler/src/main.rs:103-108: `--ignore-errors` selects parse_module_unchecked, otherwise
parse_module_checked; main.rs:134-138 prints the time of every pass).  Here the files are collected first and parsed
as one batch on one GPU; the report has the same two steps and a "parse" pass time.

    python -m zluda_b200.precompile DIR [--follow-links] [--ignore-errors] [--device N] [--quiet] [--repeat N]
"""
import argparse
import os
import sys
import time


def find_ptx_files(root, follow_links=False):
    """All regular files ending in .ptx under `root` (or `root` itself), sorted by path."""
    if os.path.isfile(root):
        return [root]
    found = []
    for base, dirs, files in os.walk(root, followlinks=follow_links):
        dirs.sort()
        for f in sorted(files):
            p = os.path.join(base, f)
            if f.endswith(".ptx") and (follow_links or not os.path.islink(p)) and os.path.isfile(p):
                found.append(p)
    return found


def parse_files(ctx, paths, ignore_errors=False):
    """-> (results, seconds, bytes): results[i] = (path, ok, n_errors); one batch, mode as the reference's compiler picks it."""
    import zluda_b200
    texts = []
    for p in paths:
        with open(p, "rb") as f:
            texts.append(f.read())
    mode = zluda_b200.UNCHECKED if ignore_errors else zluda_b200.CHECKED
    t0 = time.perf_counter()
    batch = ctx.parse_batch(texts, mode)
    seconds = time.perf_counter() - t0
    results = [(p, batch.status(i) == 0, batch.error_count(i)) for i, p in enumerate(paths)]
    batch.free()
    return results, seconds, sum(len(t) for t in texts)


def main(argv=None):
    ap = argparse.ArgumentParser(description="parse every .ptx file under a directory in one GPU batch")
    ap.add_argument("input")
    ap.add_argument("--follow-links", action="store_true")
    ap.add_argument("--ignore-errors", action="store_true", help="parse_module_unchecked instead of parse_module_checked")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--quiet", action="store_true", help="no line per failing file")
    ap.add_argument("--repeat", type=int, default=1, help="parse the batch this many times (the first call on a context allocates)")
    a = ap.parse_args(argv)
    import zluda_b200
    paths = find_ptx_files(a.input, a.follow_links)
    print("[1/2] Building file list... %d file(s) scanned" % len(paths))
    if not paths:
        return 0
    ctx = zluda_b200.Context(a.device)
    times = []
    for _ in range(max(1, a.repeat)):
        results, seconds, nbytes = parse_files(ctx, paths, a.ignore_errors)
        times.append(seconds)
    failed = [r for r in results if not r[1]]
    if not a.quiet:
        for p, ok, nerr in failed:
            print("  %s: %d error(s)" % (p, nerr))
    print("[2/2] %d/%d file(s) parsed" % (len(results) - len(failed), len(results)))
    for i, seconds in enumerate(times):
        print("parse: %.3f ms (%.2f MB, %.2f GB/s%s)" % (seconds * 1e3, nbytes / 1e6, nbytes / seconds / 1e9,
                                                       ", first call on this context: includes its allocations" if i == 0 else ""))
    ctx.close()
    return 1 if failed and not a.ignore_errors else 0


if __name__ == "__main__":
    sys.exit(main())
