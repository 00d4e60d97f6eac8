"""The declarative tensor checks in front of the native launchers (minisgl.ops.tensorcheck): dtype, rank, literal and
symbolic dimensions that must agree across arguments, layout letters, optional arguments, device agreement -- and that
the wrappers in minisgl.ops.cuda carry a spec for every tensor they hand to a kernel by pointer."""
import pytest
import torch

from minisgl.ops.tensorcheck import TensorSpecError, tensors


@tensors(q="bf16[T,H,8]", idx="?i32[T,_]", sink="f32[H]", kv="bf16[T,8]s", w="i8|u8[_]*")
def op(q, idx, sink, kv, w, flag=True):
    return q.shape[0]


def _args():
    return dict(q=torch.zeros(3, 2, 8, dtype=torch.bfloat16), idx=torch.zeros(3, 5, dtype=torch.int32),
                sink=torch.zeros(2), kv=torch.zeros(3, 16, dtype=torch.bfloat16)[:, :8],
                w=torch.zeros(9, dtype=torch.uint8)[::2])


def test_matching_arguments_pass_and_none_is_allowed_where_optional():
    a = _args()
    assert op(**a) == 3
    a["idx"] = None
    assert op(**a) == 3
    assert op.tensor_specs["sink"] == "f32[H]"


@pytest.mark.parametrize("name,bad,msg", [
    ("q", torch.zeros(3, 2, 8), "dtype"),
    ("q", torch.zeros(3, 2, dtype=torch.bfloat16), "rank"),
    ("q", torch.zeros(3, 2, 7, dtype=torch.bfloat16), "wants 8"),
    ("sink", torch.zeros(3), "dimension H is 3 here but 2"),
    ("idx", torch.zeros(4, 5, dtype=torch.int32), "dimension T is 4 here but 3"),
    ("q", torch.zeros(3, 8, 2, dtype=torch.bfloat16).transpose(1, 2), "contiguous"),
    ("kv", torch.zeros(8, 3, dtype=torch.bfloat16).t(), "stride 1"),
    ("sink", None, "required"),
    ("w", [1, 2], "expected a tensor"),
])
def test_mismatches_are_refused_before_the_call(name, bad, msg):
    a = _args()
    a[name] = bad
    with pytest.raises(TensorSpecError, match=msg):
        op(**a)


def test_bad_specs_fail_at_decoration_time():
    with pytest.raises(ValueError):
        tensors(x="bf16(T)")(lambda x: x)
    with pytest.raises(ValueError, match="no parameter"):
        tensors(y="bf16[T]")(lambda x: x)
    with pytest.raises(KeyError):
        tensors(x="fp99[T]")(lambda x: x)


def test_kernel_wrappers_declare_their_tensor_arguments():
    from minisgl.ops import cuda

    declared = {n for n in dir(cuda) if hasattr(getattr(cuda, n), "tensor_specs")}
    assert {"embed", "greedy_tokens", "q_kv_norm_rope_store", "hc_pre", "hc_post", "indexer_q_encode", "indexer_logits",
            "attention", "moe_routed", "argmax", "sample", "add_cast"} <= declared
    # a wrong dtype is refused on the host, before any pointer reaches a launcher
    with pytest.raises(TensorSpecError, match="dtype"):
        cuda.hc_post(torch.zeros(2, 8), torch.zeros(2, 4, 8, dtype=torch.bfloat16), torch.zeros(2, 4),
                     torch.zeros(2, 4, 4))


def test_expert_tiling_keeps_every_byte_and_is_indexed_as_the_kernel_reads_it():
    """Load-time re-tiling for the block-scaled expert kernel: scale byte (tile row m, K block kb) of a 512-byte block
    sits at (m % 32) * 16 + (m // 32) * 4 + kb; a weight tile is 128 rows x 64 bytes; gate / up tiles interleave 64
    gate rows with the 64 matching up rows."""
    import torch

    from minisgl.ops.cuda import block_expert_scales, pack_expert_weights, prepare_experts, route_tile

    e, inter, k = 2, 128, 256
    s13 = torch.randint(0, 255, (e, 2 * inter, k // 32), dtype=torch.uint8)
    w13 = torch.randint(-128, 127, (e, 2 * inter, k // 2), dtype=torch.int8)
    s2 = torch.randint(0, 255, (e, 256, k // 32), dtype=torch.uint8)
    w2 = torch.randint(-128, 127, (e, 256, k // 2), dtype=torch.int8)
    b13, t13, b2, t2 = block_expert_scales(s13, True), pack_expert_weights(w13, True), block_expert_scales(s2, False), \
        pack_expert_weights(w2, False)
    assert b13.shape == (e, inter // 64, k // 128, 512) and t13.shape == (e, inter // 64, k // 128, 128, 64)
    assert b2.shape == (e, 2, k // 128, 512) and t2.shape == (e, 2, k // 128, 128, 64)
    for ee in range(e):
        for rt in range(inter // 64):
            for ch in range(k // 128):
                for m in (0, 31, 32, 63, 64, 100, 127):
                    row = rt * 64 + m if m < 64 else inter + rt * 64 + m - 64
                    assert torch.equal(t13[ee, rt, ch, m], w13[ee, row, ch * 64:(ch + 1) * 64])
                    for kb in range(4):
                        assert b13[ee, rt, ch, (m % 32) * 16 + (m // 32) * 4 + kb] == s13[ee, row, ch * 4 + kb]
        for rt in range(2):
            for ch in range(k // 128):
                for m in (0, 33, 127):
                    assert torch.equal(t2[ee, rt, ch, m], w2[ee, rt * 128 + m, ch * 64:(ch + 1) * 64])
                    for kb in range(4):
                        assert b2[ee, rt, ch, (m % 32) * 16 + (m // 32) * 4 + kb] == s2[ee, rt * 128 + m, ch * 4 + kb]
    w = {"L0.moe.w13": w13, "L0.moe.s13": s13, "L0.moe.w2": w2, "L0.moe.s2": s2}
    prepare_experts(w, "L0.moe.")
    assert torch.equal(w["L0.moe.w13"], t13) and torch.equal(w["L0.moe.s2"], b2)
    before = {k_: v.data_ptr() for k_, v in w.items()}
    prepare_experts(w, "L0.moe.")  # tiled tensors are left alone
    assert before == {k_: v.data_ptr() for k_, v in w.items()}
    assert [route_tile(r * 6, 256, "mx") for r in (64, 128, 256, 512, 1024)] == [8, 8, 16, 32, 64]
    assert route_tile(768, 256, "f16") == 32


def test_decode_tile_choice_is_launchable_and_prefers_fewer_bytes():
    """The FP8 decode tile model returns only configurations the kernel accepts (tile widths 32 / 64 / 128, splits
    1 / 2 / 4 with at least two k-tiles per split, at most 64 k-tiles per CTA) and moves to wide tiles with K splits
    where narrow tiles would re-read the activation tile most often."""
    from minisgl.ops.gemm import _pick_decode_fp8, pick_tiling

    for n in (256, 512, 1536, 2112, 4096, 8192, 32768, 129280):
        for k in (256, 1024, 1536, 2048, 4096, 8192):
            bn, splits = _pick_decode_fp8(n, k // 128)
            assert bn in (32, 64, 128) and splits in (1, 2, 4)
            assert splits == 1 or (k // 128) // splits >= 2
            assert -(-(k // 128) // splits) <= 64
            assert pick_tiling(128, n, k // 128, 1, True) == (bn, splits)
    assert _pick_decode_fp8(32768, 12) == (128, 1)          # enough column tiles: the widest tile, no split
    assert _pick_decode_fp8(4096, 64)[0] == 128 and _pick_decode_fp8(4096, 64)[1] > 1   # long K, few columns
    # explicit arguments are respected
    assert pick_tiling(128, 4096, 32, 1, True, bn=32, splits=1) == (32, 1)
