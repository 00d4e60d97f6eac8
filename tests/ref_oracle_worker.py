"""Runs the reference's own pure-PyTorch operator oracle (debug/dsv4/kernel/deepseek_v4_reference.py of a reference
checkout) on seeded CPU inputs and saves inputs and outputs with torch.save.

It runs as a separate process because that file imports the reference's ``minisgl`` package, whose name collides with
this repository's import shim.  Usage: python ref_oracle_worker.py <reference checkout> <output file>
"""
import importlib.util
import os
import sys


def main(ref_root: str, out_path: str) -> None:
    sys.path = [p for p in sys.path if os.path.basename(p.rstrip("/")) != "tests" and "deepseek-v4-sm80_b200" not in p]
    sys.path.insert(0, os.path.join(ref_root, "python"))
    import torch

    spec = importlib.util.spec_from_file_location(
        "dsv4_reference_oracle", os.path.join(ref_root, "debug", "dsv4", "kernel", "deepseek_v4_reference.py"))
    R = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(R)
    assert not R.dsv4_triton_available(), "the oracle must take its torch paths"
    g = torch.Generator().manual_seed(20240607)
    rn = lambda *s, scale=1.0: torch.randn(*s, generator=g) * scale
    out = {}

    # FP8 activation fake-quant (1x128 blocks, power-of-two scales)
    x = torch.cat([rn(6, 512), rn(2, 512, scale=1e-6), rn(2, 512, scale=300.0)]).to(torch.bfloat16)
    out["fp8_act"] = {"x": x, "y": R.quantize_fp8_activation_ref(x.clone())}

    # FP4 (e2m1 nibbles, e8m0 scale per 32) dequantisation
    packed = torch.randint(0, 256, (24, 64), generator=g, dtype=torch.uint8).view(torch.int8)
    codes = torch.randint(110, 135, (24, 4), generator=g, dtype=torch.uint8)
    scale = torch.pow(2.0, codes.float() - 127.0)
    out["fp4"] = {"packed": packed, "codes": codes,
                  "w": R.dequant_fp4_weight(packed, scale, out_dtype=torch.float32)}

    # non-overlap (ratio 128) compressor on a prompt that starts at position 0
    d, t = 32, 300
    xs, w = rn(t, 48), rn(2 * d, 48, scale=0.2)
    ape = rn(128, d, scale=0.5)

    class Lin:
        def forward(self, v):
            return v @ w.t()

    class Ident:
        def forward(self, v):
            return v

    pooled = R.compress_forward_fallback(xs, torch.arange(t), ratio=128, head_dim=d, overlap=False, ape=ape,
                                         wkv_gate=Lin(), norm=Ident(), apply_norm=False)
    out["compress128"] = {"x": xs, "w": w, "ape": ape, "pooled": pooled}

    # rotary tail, plain and with YaRN-style frequency scaling, forward and inverse
    xr = rn(10, 3, 96)
    pos = torch.tensor([0, 1, 5, 17, 100, 1023, 4096, 65535, 300000, 1000000])
    rope = {}
    for name, kw in (("plain", dict(base=10000.0)),
                     ("yarn", dict(base=160000.0, original_seq_len=65536, factor=16.0, beta_fast=32, beta_slow=1))):
        for inv in (False, True):
            rope[(name, inv)] = R.apply_rotary_tail(xr.clone(), pos, rotary_dim=64, inverse=inv, **kw)
    out["rope"] = {"x": xr, "pos": pos, "y": rope}

    # paged FP8 indexer logits
    heads, dim, ps, rows = 4, 128, 16, 5
    kv = rn(6 * ps, dim)
    vals, sc = R.quantize_indexer_fp8_cache_ref(kv)
    cache = R.pack_indexer_fp8_paged_cache_ref(vals.view(-1, dim), sc.view(-1, 4), page_size=ps)
    q = (rn(rows, heads, dim) * 3).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    wts = rn(rows, heads).abs()
    lens = torch.tensor([1, 16, 17, 40, 96], dtype=torch.int32)
    table = torch.stack([torch.randperm(6, generator=g) for _ in range(rows)]).to(torch.int32)
    logits = R.indexer_fp8_paged_logits_fallback(q, cache, lens, table, page_size=ps, weights=wts)
    out["indexer"] = {"vals": vals, "scales": sc.contiguous().view(torch.float32).view(-1), "q": q, "w": wts,
                      "lens": lens, "table": table, "ps": ps, "logits": logits}

    # hyper-connection pre mix (Sinkhorn), post mix and head collapse
    m, h, tt = 4, 64, 7
    xh = rn(tt, m, h).to(torch.bfloat16)
    fn = rn((2 + m) * m, m * h, scale=0.05).to(torch.bfloat16).float()
    hs, hb = torch.tensor([0.7, 1.3, 0.9]), rn((2 + m) * m, scale=0.5)
    y, post, comb = R.hc_pre_fallback(xh, fn, hs, hb, hc_mult=m, sinkhorn_iters=20, eps=1e-6, norm_eps=1e-6)
    pre_s, post_s, comb_s = R.hc_split_sinkhorn_ref(rn(tt, (2 + m) * m), hs, hb, m, 20, 1e-6)
    blk = rn(tt, h).to(torch.bfloat16)
    mixed = R.hc_post_fallback(blk, xh, post, comb)
    fnh, hbh = rn(m, m * h, scale=0.05).to(torch.bfloat16).float(), rn(m, scale=0.5)
    head = R.hc_head_fallback(xh, fnh, torch.tensor([1.1]), hbh, eps=1e-6, norm_eps=1e-6)
    out["hc"] = {"x": xh, "fn": fn, "scale": hs, "base": hb, "y": y, "post": post, "comb": comb, "blk": blk,
                 "mixed": mixed, "fn_head": fnh, "base_head": hbh, "head": head}

    # RMSNorm and SwiGLU with clamp
    xn, wn = rn(5, 256).to(torch.bfloat16), (1 + rn(256, scale=0.1)).to(torch.bfloat16)
    out["rms"] = {"x": xn, "w": wn, "y": R.rms_norm_fallback(xn, wn, eps=1e-6)}

    # sparse attention over one shared cache (compressed rows followed by window rows), with sink
    hq, dd, toks = 3, 64, 6
    cache = rn(200, dd).to(torch.bfloat16)
    qa = rn(toks, hq, dd).to(torch.bfloat16)
    sink = rn(hq)
    ctx = [torch.randperm(200, generator=g)[: n] for n in (1, 5, 17, 40, 64, 130)]
    oa = R.paged_mqa_attention_fallback(qa, cache, ctx, softmax_scale=dd ** -0.5, attn_sink=sink)
    out["attention"] = {"q": qa, "cache": cache, "ctx": ctx, "sink": sink, "o": oa}

    gate, up = rn(9, 96, scale=4.0).to(torch.bfloat16), rn(9, 96, scale=4.0).to(torch.bfloat16)
    out["swiglu"] = {"gate": gate, "up": up, "y7": R.silu_and_mul_clamp_fallback(gate, up, swiglu_limit=7.0),
                     "y0": R.silu_and_mul_clamp_fallback(gate, up, swiglu_limit=0.0)}
    torch.save(out, out_path)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
