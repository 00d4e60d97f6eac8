"""Per-kernel summary of an Nsight Compute launch list.

    ncu --metrics gpu__time_duration.sum --clock-control none -c N --csv --log-file launches.csv <program>
    python -m minisgl.benchmark.ncu_summary launches.csv [first-kernel-substring]

Groups the launches of the last step (from the last launch whose name contains the given substring, default
``embed``: the first kernel of a forward) by kernel and grid, and prints count, total and mean device time and the
share of the step.  The committed summaries under ``profiles/`` are made with it.
"""
from __future__ import annotations

import csv
import re
import sys
from typing import Dict, List, Tuple


def read_launches(path: str) -> List[Tuple[str, str, float]]:
    """(kernel name, grid, nanoseconds) of every launch in an ``ncu --csv`` log, in launch order."""
    with open(path) as f:
        lines = [l for l in f if not l.startswith("==")]
    out = []
    for r in csv.DictReader(lines):
        if r.get("Metric Name") == "gpu__time_duration.sum":
            out.append((r["Kernel Name"], r.get("Grid Size", ""), float(r["Metric Value"].replace(",", ""))))
    return out


def short_name(kernel: str) -> str:
    n = re.sub(r"\(.*", "", kernel)
    return re.sub(r"void |<unnamed>::", "", n)[:44]


def last_step(launches, first: str = "embed"):
    """The launches from the last one whose name contains ``first`` (all of them when none does)."""
    idx = [i for i, (n, _, _) in enumerate(launches) if first in n]
    return launches[idx[-1]:] if idx else list(launches)


def aggregate(launches) -> Dict[Tuple[str, str], Tuple[int, float]]:
    """{(short kernel name, grid): (launch count, total nanoseconds)}, largest total first."""
    agg: Dict[Tuple[str, str], Tuple[int, float]] = {}
    for name, grid, ns in launches:
        key = (short_name(name), grid)
        c, t = agg.get(key, (0, 0.0))
        agg[key] = (c + 1, t + ns)
    return dict(sorted(agg.items(), key=lambda kv: -kv[1][1]))


def render(launches, top: int = 45) -> str:
    tot = sum(ns for _, _, ns in launches)
    lines = [f"kernels in last step {len(launches)} total us {tot / 1000}"]
    for (n, g), (c, t) in list(aggregate(launches).items())[:top]:
        lines.append(f"{n:44s} {g:>14s} x{c:3d} {t / 1000:8.1f} us {100 * t / tot:5.1f}%  avg {t / c / 1000:6.1f}")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        print(__doc__)
        return 2
    print(render(last_step(read_launches(argv[0]), argv[1] if len(argv) > 1 else "embed")))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
