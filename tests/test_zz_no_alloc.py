"""The allocation-free indexer selection entry point (csrc/noalloc.h), called through its exported C symbol.

Some embedders cannot call cudaMalloc while serving (a latency-critical loop that must not take the allocator's locks,
a host framework that owns all device memory, a fixed start-up budget).  For them the library keeps the logits
workspace in a built-in device array.  This test checks that the entry point gives the same selection as the regular
path (dsv4_indexer_logits + dsv4_topk with a caller-allocated workspace), twice in a row on different inputs -- the
second call sees the first call's stale workspace -- and that an oversized request is refused with a clear message.
This file sorts last on purpose, so a run that stops at the first failure has already run every other test.
"""
import ctypes
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, positions):
    from minisgl.ops import quant

    ps = 256
    g = torch.Generator().manual_seed(seed)
    pages = torch.randperm(16, generator=g).tolist()
    pt = torch.zeros(2, 4096, dtype=torch.int32)
    for k in range(16):
        pt[1, k * ps:(k + 1) * ps] = torch.arange(pages[k] * ps, (pages[k] + 1) * ps, dtype=torch.int32)
    pos = torch.tensor(positions, dtype=torch.int32)
    t = pos.shape[0]
    qc = torch.randn(t, 64, 128, generator=g).to(quant.FP8).view(torch.uint8)
    wf = torch.randn(t, 64, generator=g)
    vals = torch.randn(16 * 64, 128, generator=g).to(quant.FP8).view(torch.uint8)
    scales = torch.rand(16 * 64, generator=g) + 0.5
    dev = lambda x: x.cuda()
    return dict(qc=dev(qc), wf=dev(wf), vals=dev(vals), scales=dev(scales), slots=dev(torch.ones(t, dtype=torch.int32)),
                pos=dev(pos), pt=dev(pt), ps=ps, t=t, max_context=int(pos.max()) + 1)


def _regular(x, k):
    from minisgl.ops import cuda

    fb = types.SimpleNamespace(positions=x["pos"], slots=x["slots"], page_table=x["pt"], max_context=x["max_context"])
    return cuda.indexer_select(x["qc"], x["wf"], x["vals"], x["scales"], fb, x["ps"], k)


def _noalloc(lib, x, k):
    width = (x["max_context"] // 4 + 63) // 64 * 64
    idx = torch.empty(x["t"], k, dtype=torch.int32, device="cuda")
    ln = torch.empty(x["t"], dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.dsv4_indexer_select_noalloc(p(x["qc"]), p(x["wf"]), p(x["vals"]), p(x["scales"]), p(x["slots"]), p(x["pos"]),
                                         p(x["pt"]), ctypes.c_int(x["pt"].stride(0)), ctypes.c_int(x["ps"]),
                                         ctypes.c_int(width), ctypes.c_int(x["t"]), ctypes.c_int(64), ctypes.c_int(128),
                                         p(idx), p(ln), ctypes.c_int(k),
                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, idx, ln


def test_noalloc_entry_point_matches_regular_path_twice():
    from minisgl.ops import native

    lib = native.cuda_lib()
    lib.dsv4_indexer_select_noalloc.restype = ctypes.c_int
    lib.dsv4_noalloc_last_error.restype = ctypes.c_char_p
    k = 512
    for seed, positions in ((1, [4000, 2100, 2047, 700, 3]), (2, [3000, 4095, 2600])):
        x = _inputs(seed, positions)
        rc, idx, ln = _noalloc(lib, x, k)
        assert rc == 0, lib.dsv4_noalloc_last_error()
        idx_r, ln_r = _regular(x, k)
        torch.cuda.synchronize()
        assert torch.equal(ln.cpu(), ln_r.cpu())
        assert torch.equal(idx.cpu(), idx_r.cpu())
    # a request larger than the built-in workspace is refused, nothing is launched
    x = _inputs(3, [4000] * 8)
    x["max_context"] = 4 * (1 << 20)
    rc, _, _ = _noalloc(lib, x, k)
    assert rc == 460
    assert b"exceeds the built-in workspace" in lib.dsv4_noalloc_last_error()
    native.assert_device_ok()
