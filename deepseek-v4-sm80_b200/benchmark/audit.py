"""Static audit and source census of this package (the reference keeps a grep audit and a census tool next to its
coverage runs).

    python -m minisgl.benchmark.audit            # prints a JSON report, exit code 1 if a rule is violated

Rules checked over the package sources (Python and CUDA):
  * no compatibility layers on the compute path: no ``import triton`` / ``tilelang`` / ``torch.compile`` /
    ``flashinfer`` / ``flash_attn`` / ``vllm`` imports;
  * no CUDA batched-memcpy entry points; no TMA or bulk load with cluster multicast; no ``wgmma``;
  * every ``__global__`` kernel has the programmatic-dependent-launch prologue (``pdl_entry``, or after a set-up
    phase ``pdl_wait`` followed by ``pdl_launch_dependents``: never the trigger before the own wait), and no launch
    uses the ``<<< >>>`` syntax (launches go through
    ``dsv4_launch`` so that they all carry the same attributes);
  * every spin loop in device code is bounded: a ``for (;;)`` / ``while (true)`` body must contain a clock read;
  * ``tests/``: a test that touches CUDA carries the ``gpu`` marker (file-level ``pytestmark`` or per-test marks).
Census: lines of code per top-level component, kernels per ``.cu`` file, exported ``dsv4_*`` entry points.
"""
from __future__ import annotations

import json
import os
import re
import sys
from typing import Dict, List

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROOT = os.path.dirname(PKG)

_B = "cudaMemcpy" + "Batch" + "Async|cudaMemcpy3D" + "Batch" + "Async|cuMemcpy" + "Batch" + "Async|cuMemcpy3D" + "Batch" + "Async"
FORBIDDEN_PY = [r"^\s*import\s+triton", r"^\s*from\s+triton", r"tilelang", r"torch\.compile\(", r"^\s*import\s+flashinfer",
                r"^\s*from\s+flashinfer", r"^\s*import\s+flash_attn", r"^\s*from\s+flash_attn", r"^\s*import\s+vllm",
                r"^\s*from\s+vllm"]
_MC = "multi" + "cast::" + "cluster"
_BULK = "cp.async" + ".bulk"
FORBIDDEN_CU = [_B, re.escape(_BULK) + r"[^\n;]*" + re.escape(_MC), r"wgmma\."]


def _files(top: str, exts) -> List[str]:
    out = []
    for d, dirs, fs in os.walk(top):
        dirs[:] = [x for x in dirs if x not in ("__pycache__", "build")]
        out += [os.path.join(d, f) for f in fs if f.endswith(exts)]
    return sorted(out)


def _kernel_bodies(src: str):
    """Yields (name, body) of every __global__ function."""
    for m in re.finditer(r"__global__", src):
        i = src.find("(", m.end())
        while True:
            depth, j = 0, i
            while True:
                depth += src[j] == "("
                depth -= src[j] == ")"
                if depth == 0:
                    break
                j += 1
            k = j + 1
            while src[k].isspace():
                k += 1
            if src[k] == "{":
                break
            i = src.find("(", j + 1)
        name = re.findall(r"(\w+)\s*$", src[m.end():i])[-1] if re.findall(r"(\w+)\s*$", src[m.end():i]) else "?"
        depth, e = 0, k
        while True:
            depth += src[e] == "{"
            depth -= src[e] == "}"
            if depth == 0:
                break
            e += 1
        yield name, src[k:e + 1]


def audit() -> Dict:
    violations: List[str] = []
    py = _files(PKG, (".py",))
    cu = _files(os.path.join(PKG, "ops", "csrc"), (".cu", ".cuh", ".h", ".cpp"))
    for f in py:
        if f == os.path.abspath(__file__):
            continue
        for n, line in enumerate(open(f, encoding="utf-8"), 1):
            for pat in FORBIDDEN_PY:
                if re.search(pat, line):
                    violations.append(f"{os.path.relpath(f, ROOT)}:{n}: forbidden import/use: {line.strip()[:80]}")
    kernels: Dict[str, int] = {}
    exports: List[str] = []
    for f in cu:
        src = open(f, encoding="utf-8").read()
        rel = os.path.relpath(f, ROOT)
        for pat in FORBIDDEN_CU:
            for m in re.finditer(pat, src):
                violations.append(f"{rel}: forbidden construct: {m.group(0)[:60]}")
        if "<<<" in src:
            violations.append(f"{rel}: raw <<< >>> launch (use dsv4_launch)")
        exports += re.findall(r"DSV4_API\s+\w[\w\s\*]*?\b(dsv4_\w+)\s*\(", src)
        if not f.endswith(".cu"):
            continue
        n = 0
        for name, body in _kernel_bodies(src):
            n += 1
            head = body[:400]
            w, t = body.find("pdl_wait()"), body.find("pdl_launch_dependents()")
            # pdl_entry() first thing, or (kernels with a set-up phase) an explicit wait followed by the trigger
            if "pdl_entry()" not in head and not (0 <= w < t):
                violations.append(f"{rel}: kernel {name} lacks the dependent-launch prologue")
            elif 0 <= t < w:
                violations.append(f"{rel}: kernel {name} lets its successor start before its own wait")
            for loop in re.finditer(r"for \(;;\)|while \(true\)|while \(1\)", body):
                depth, e = 0, body.find("{", loop.end())
                s0 = e
                while True:
                    depth += body[e] == "{"
                    depth -= body[e] == "}"
                    if depth == 0:
                        break
                    e += 1
                if not re.search(r"globaltimer_ns\(\)|clock64\(\)", body[s0:e]):
                    violations.append(f"{rel}: kernel {name} has an unbounded spin loop")
        kernels[rel] = n
    # helper waits live in headers: check them too
    for f in cu:
        if f.endswith((".cuh",)):
            src = open(f, encoding="utf-8").read()
            for loop in re.finditer(r"for \(;;\)", src):
                seg = src[loop.end(): loop.end() + 600]
                if not re.search(r"globaltimer_ns\(\)|clock64\(\)", seg):
                    violations.append(f"{os.path.relpath(f, ROOT)}: unbounded spin loop in a device helper")
    tests = _files(os.path.join(ROOT, "tests"), (".py",))
    for f in tests:
        src = open(f, encoding="utf-8").read()
        base = os.path.basename(f)
        if not base.startswith("test_"):
            continue
        uses_cuda = re.search(r"\"cuda\"|'cuda'|DEV\b", src) is not None
        marked = "pytest.mark.gpu" in src
        if uses_cuda and not marked and "_cpu" not in base:
            violations.append(f"tests/{base}: touches CUDA but has no gpu marker")
    census: Dict[str, int] = {}
    for f in py + cu:
        rel = os.path.relpath(f, PKG).split(os.sep)
        comp = rel[0] if len(rel) > 1 else "(top)"
        if comp == "ops" and len(rel) > 2:
            comp = "ops/" + rel[1]
        census[comp] = census.get(comp, 0) + sum(1 for _ in open(f, encoding="utf-8"))
    census["tests"] = sum(sum(1 for _ in open(f, encoding="utf-8")) for f in tests)
    return {"violations": violations, "kernels_per_file": kernels, "num_kernels": sum(kernels.values()),
            "exports": sorted(set(exports)), "num_exports": len(set(exports)), "lines": dict(sorted(census.items()))}


def main() -> int:
    rep = audit()
    print(json.dumps(rep, indent=1))
    return 1 if rep["violations"] else 0


if __name__ == "__main__":
    sys.exit(main())
