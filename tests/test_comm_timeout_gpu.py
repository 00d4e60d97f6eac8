"""Failure detection on the device without a fault: a wait on a flag that nothing sets gives up after its limit,
records DSV4_ERR_PEER_TIMEOUT in the status word and returns; the context stays usable for the next kernel."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_survives():
    from minisgl.ops import api as O
    from minisgl.ops import native

    native.read_status(clear=True)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    # nobody ever writes 7 into the flag: the kernel must give up after 50 ms
    native.call("wait_flag", native.ptr(flag), ctypes.c_uint(7), ctypes.c_longlong(50_000_000), native.ptr(result))
    torch.cuda.synchronize()
    assert int(result.item()) == 0
    status = native.read_status(clear=True)
    assert status[0] == 3 and status[3] >= 1, status  # DSV4_ERR_PEER_TIMEOUT, counted once
    with pytest.raises(Exception):
        # a second timeout must surface through the checking helper
        native.call("wait_flag", native.ptr(flag), ctypes.c_uint(7), ctypes.c_longlong(1_000_000), native.ptr(result))
        native.assert_device_ok()
    native.read_status(clear=True)
    # a satisfied wait returns 1 and leaves the status clean
    flag.fill_(7)
    native.call("wait_flag", native.ptr(flag), ctypes.c_uint(7), ctypes.c_longlong(50_000_000), native.ptr(result))
    torch.cuda.synchronize()
    assert int(result.item()) == 1 and native.read_status()[0] == 0
    # and ordinary kernels still run on the same context
    x = torch.randn(4, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    y = O.rms_norm(x, w, 1e-6)
    ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    assert torch.allclose(y.float(), ref.float(), atol=2e-2, rtol=2e-2)
