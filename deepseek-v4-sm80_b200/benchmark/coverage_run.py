"""Line coverage of the package under the CPU test tier, without external tools.

    python -m minisgl.benchmark.coverage_run [--tests tests/test_cache_cpu.py ...] [--min 0]

Runs pytest in-process under ``sys.settrace`` restricted to the package's files and prints, per module, executed /
executable lines (executable lines taken from the code objects' line tables), then the total.  The reference drives
``coverage.py`` from shell scripts for the same purpose (debug/dsv4/coverage/*.sh); this image has no coverage
package, hence the tracer.  Child processes (server and multi-rank tests) are not traced.
"""
from __future__ import annotations

import argparse
import os
import sys
import threading
from collections import defaultdict

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def executable_lines(path: str) -> set:
    try:
        code = compile(open(path, encoding="utf-8").read(), path, "exec")
    except SyntaxError:
        return set()
    lines, stack = set(), [code]
    while stack:
        c = stack.pop()
        lines.update(l for _, _, l in c.co_lines() if l)
        stack.extend(k for k in c.co_consts if hasattr(k, "co_lines"))
    return lines


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tests", nargs="*", default=[])
    ap.add_argument("--min", type=float, default=0.0, help="fail (exit 2) below this total percentage")
    a = ap.parse_args(argv)
    import pytest

    hits = defaultdict(set)
    real = os.path.realpath(PKG)

    def local(frame, event, arg):
        if event == "line":
            hits[frame.f_code.co_filename].add(frame.f_lineno)
        return local

    def tracer(frame, event, arg):
        fn = frame.f_code.co_filename
        if fn.startswith(PKG) or fn.startswith(real):
            return local(frame, event, arg) or local
        return None

    root = os.path.dirname(PKG)
    tests = a.tests or [os.path.join(root, "tests")]
    threading.settrace(tracer)
    sys.settrace(tracer)
    try:
        rc = pytest.main(["-q", "-x", "-m", "not gpu", "-p", "no:cacheprovider", *tests])
    finally:
        sys.settrace(None)
        threading.settrace(None)
    total_hit = total_exec = 0
    rows = []
    for dirpath, _, files in os.walk(PKG):
        if "__pycache__" in dirpath:
            continue
        for f in sorted(files):
            if not f.endswith(".py"):
                continue
            path = os.path.join(dirpath, f)
            ex = executable_lines(path)
            hit = (hits.get(path, set()) | hits.get(os.path.realpath(path), set())) & ex
            total_hit += len(hit)
            total_exec += len(ex)
            rows.append((os.path.relpath(path, PKG), len(hit), len(ex)))
    for name, h, e in rows:
        print(f"{name:45s} {h:5d} / {e:5d}  {100.0 * h / e if e else 100.0:5.1f}%")
    pct = 100.0 * total_hit / max(total_exec, 1)
    print(f"{'TOTAL':45s} {total_hit:5d} / {total_exec:5d}  {pct:5.1f}%   (pytest exit code {int(rc)})")
    if int(rc) != 0 or pct < a.min:
        sys.exit(2)
    return pct


if __name__ == "__main__":
    main()
