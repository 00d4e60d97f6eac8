"""Number-format codecs of the DeepSeek-V4 checkpoint, in plain PyTorch.

* FP8 e4m3 activations with one power-of-two scale per (row, 128 block)
  (reference semantics: debug/dsv4/kernel/deepseek_v4_reference.py:92-128).
* FP8 e4m3 weights with one e8m0 scale per 128 x 128 block
  (python/minisgl/kernel/deepseek_v4.py:350-374).
* Packed FP4 (E2M1, two nibbles per int8 byte, low nibble = even element) with one
  e8m0 scale per 32 elements along K (deepseek_v4_reference.py:44-89).

These functions are the CPU oracle for the CUDA kernels and are also used to
build synthetic checkpoints.
"""
from __future__ import annotations

import torch

FP8 = torch.float8_e4m3fn
E8M0 = getattr(torch, "float8_e8m0fnu", None)
FP8_MAX = 448.0

_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def e2m1_table(device=None) -> torch.Tensor:
    return torch.tensor(_E2M1 + [-v for v in _E2M1], dtype=torch.float32, device=device)


def pow2_scale(absmax: torch.Tensor, limit: float = FP8_MAX, floor: float = 1e-4) -> torch.Tensor:
    """2^ceil(log2(max(absmax, floor) / limit)) in fp32."""
    s = absmax.float().clamp_min(floor) / limit
    return torch.pow(2.0, torch.ceil(torch.log2(s)))


def fp8_act_quant(x: torch.Tensor, block: int = 128):
    """Returns (q e4m3 [..., K], scale fp32 [..., K/block]) with x ~= q * scale."""
    k = x.shape[-1]
    assert k % block == 0, (k, block)
    g = x.float().reshape(*x.shape[:-1], k // block, block)
    scale = pow2_scale(g.abs().amax(dim=-1, keepdim=True))
    q = (g / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.reshape(x.shape), scale.squeeze(-1)


def fp8_fake_quant(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Quantise-dequantise in the input dtype (what the reference feeds its bf16 GEMMs)."""
    q, s = fp8_act_quant(x, block)
    k = x.shape[-1]
    y = q.float().reshape(*x.shape[:-1], k // block, block) * s.unsqueeze(-1)
    return y.reshape(x.shape).to(x.dtype)


def e8m0_encode(scale: torch.Tensor) -> torch.Tensor:
    """fp32 power of two -> biased exponent byte (uint8)."""
    return (torch.log2(scale.float()).round().to(torch.int32) + 127).clamp(0, 254).to(torch.uint8)


def e8m0_decode(code: torch.Tensor) -> torch.Tensor:
    """e8m0 (uint8 view or float8_e8m0fnu) -> fp32."""
    if E8M0 is not None and code.dtype == E8M0:
        code = code.view(torch.uint8)
    if code.dtype != torch.uint8:
        return code.float()
    return torch.pow(2.0, code.to(torch.int32).float() - 127.0)


def fp8_weight_quant(w: torch.Tensor, block: int = 128):
    """[N,K] -> (e4m3 [N,K], e8m0 codes uint8 [ceil(N/b), ceil(K/b)])."""
    n, k = w.shape
    nb, kb = (n + block - 1) // block, (k + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:n, :k] = w.float()
    blocks = wp.view(nb, block, kb, block)
    scale = pow2_scale(blocks.abs().amax(dim=(1, 3)), floor=1e-12)
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(nb * block, kb * block)[:n, :k].contiguous(), e8m0_encode(scale)


def fp8_weight_dequant(q: torch.Tensor, scale_code: torch.Tensor, block: int = 128, dtype=torch.bfloat16):
    n, k = q.shape
    s = e8m0_decode(scale_code)
    s = s.repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return (q.float() * s).to(dtype)


def fp4_quant(w: torch.Tensor, group: int = 32):
    """[..., K] -> (int8 packed [..., K/2], e8m0 codes uint8 [..., K/group])."""
    k = w.shape[-1]
    assert k % group == 0 and group % 2 == 0
    g = w.float().reshape(*w.shape[:-1], k // group, group)
    scale = pow2_scale(g.abs().amax(dim=-1, keepdim=True), limit=6.0, floor=1e-12)
    v = (g / scale).clamp(-6.0, 6.0)
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=torch.float32, device=w.device)
    idx = torch.bucketize(v.abs(), bounds)
    code = (idx | ((v < 0) & (idx > 0)).to(idx.dtype) * 8).to(torch.uint8).reshape(*w.shape[:-1], k)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).view(torch.int8)
    return packed, e8m0_encode(scale.squeeze(-1))


def fp4_dequant(packed: torch.Tensor, scale_code: torch.Tensor, group: int = 32, dtype=torch.bfloat16):
    p = packed.contiguous().view(torch.uint8)
    table = e2m1_table(p.device)
    lo = table[(p & 0x0F).long()]
    hi = table[((p >> 4) & 0x0F).long()]
    v = torch.stack((lo, hi), dim=-1).flatten(-2)
    s = e8m0_decode(scale_code).repeat_interleave(group, dim=-1)[..., : v.shape[-1]]
    return (v * s).to(dtype)


# --------------------------------------------------------------------------- hi / lo split of bf16 activations
def mx_split(x: torch.Tensor, group: int = 32):
    """bf16 activations [..., K] -> (hi e4m3, lo e4m3, hi exponent bytes, lo exponent bytes) with one power-of-two
    scale per ``group`` K elements each, so that ``x == hi * 2^(eh - 127) + lo * 2^(el - 127)``.  This is the operand
    form of the block-scaled expert kernel (ops/csrc/moe_mx.cu: ``mx_block_exps`` / ``mx_split``), restated in torch:
    eh = biased exponent of the group's largest magnitude - 7 (clamped to [5, 253]), el = eh - 5; hi is x / 2^(eh-127)
    rounded to e4m3 (round to nearest even), lo is the remainder / 2^(el-127) rounded to e4m3.  A bf16 value has 8
    significant bits, hi keeps the upper 4, and the remainder is a multiple of the value's last place of at most half
    a place of hi, so lo is exact for every element within 2^14 of its group's largest magnitude."""
    xf = x.float()
    k = xf.shape[-1]
    assert k % group == 0
    g = xf.reshape(*xf.shape[:-1], k // group, group)
    amax = g.abs().amax(-1)
    ef = (amax.view(torch.int32) >> 23) & 0xFF
    eh = (ef - 7).clamp(5, 253)
    el = eh - 5
    sh = torch.pow(2.0, (eh - 127).float()).unsqueeze(-1)
    sl = torch.pow(2.0, (el - 127).float()).unsqueeze(-1)
    hi = (g / sh).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    lo = ((g - hi.float() * sh) / sl).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return hi.reshape(xf.shape), lo.reshape(xf.shape), eh.to(torch.uint8), el.to(torch.uint8)


def mx_join(hi: torch.Tensor, lo: torch.Tensor, eh: torch.Tensor, el: torch.Tensor, group: int = 32) -> torch.Tensor:
    """Inverse of :func:`mx_split` (fp32)."""
    k = hi.shape[-1]
    sh = torch.pow(2.0, eh.to(torch.int32).float() - 127.0).repeat_interleave(group, -1)
    sl = torch.pow(2.0, el.to(torch.int32).float() - 127.0).repeat_interleave(group, -1)
    return hi.float() * sh[..., :k] + lo.float() * sl[..., :k]

