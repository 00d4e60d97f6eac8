"""The hi / lo activation form of the block-scaled expert kernel, checked on the CPU restatement of its split
(``ops/quant.py: mx_split``; the device function is compared with the same property in tests/test_ops_gpu.py)."""
import torch

from minisgl.ops import quant


def _all_finite_bf16():
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.bfloat16)
    return x[torch.isfinite(x.float())]


def test_every_bf16_value_splits_exactly_next_to_any_larger_neighbour_within_2_to_14():
    """Every finite bf16 value, alone in its group (it is the group's largest magnitude) and next to a neighbour that is
    up to 2^14 times larger: hi + lo gives the value back bit for bit."""
    x = _all_finite_bf16()
    x = x[(x.float().abs() >= 2.0 ** -100) & (x.float().abs() <= 2.0 ** 100)]  # exponent bytes stay inside [5, 253]
    for shift in (0, 3, 7, 10, 13, 14):
        big = (x.float().abs() * 2.0 ** shift).to(torch.bfloat16)     # a power-of-two multiple: exact in bf16
        g = torch.zeros(x.numel(), 32, dtype=torch.bfloat16)
        g[:, 0], g[:, 1] = x, big
        hi, lo, eh, el = quant.mx_split(g)
        rec = quant.mx_join(hi, lo, eh, el)
        assert torch.equal(rec[:, 0], x.float()), shift
        assert torch.equal(rec[:, 1], big.float()), shift


def test_far_smaller_elements_keep_a_tiny_absolute_error():
    """Elements more than 2^14 below their group's largest magnitude are no longer exact, but their error stays below
    2^-21 of that magnitude (the fp32 accumulation of the dot product is coarser than that)."""
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(4096, 32, generator=g) * torch.exp(torch.randn(4096, 32, generator=g) * 6)).to(torch.bfloat16)
    hi, lo, eh, el = quant.mx_split(x)
    rec = quant.mx_join(hi, lo, eh, el)
    amax = x.float().abs().amax(-1, keepdim=True)
    near = x.float().abs() >= amax * 2.0 ** -13
    assert torch.equal(rec[near], x.float()[near])
    assert bool(((rec - x.float()).abs() <= amax * 2.0 ** -21).all())
    # hi alone carries 4 significant bits: relative error up to 2^-4 of the element, which is why lo exists
    err_hi = (hi.float() * torch.pow(2.0, eh.float() - 127).repeat_interleave(32, -1).reshape(x.shape) - x.float()).abs()
    assert float((err_hi / x.float().abs().clamp_min(1e-30))[near].max()) > 2.0 ** -6


def test_zero_groups_and_layout():
    x = torch.zeros(3, 64, dtype=torch.bfloat16)
    x[1, 40] = 3.0
    hi, lo, eh, el = quant.mx_split(x)
    assert hi.shape == x.shape and eh.shape == (3, 2) and torch.equal(el, eh - 5)
    assert torch.equal(quant.mx_join(hi, lo, eh, el), x.float())
