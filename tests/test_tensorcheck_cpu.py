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
