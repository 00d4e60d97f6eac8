"""Sampler and reasoning-sampler contract on CPU (the oracle sampling path): greedy short-cut, temperature / top-k /
top-p semantics of the inverse-CDF sampler, structural-token masks by reasoning state, and the strict resolution
of the structural token ids from a tokenizer."""
from types import SimpleNamespace

import pytest
import torch

from minisgl.core import SamplingParams
from minisgl.engine.sample import BatchSamplingArgs, ReasoningSampler, Sampler
from minisgl.ops import api as O
from minisgl.reasoning import ReasoningState, ReasoningTokenIds, resolve_reasoning_token_ids

V = 64
IDS = ReasoningTokenIds(bos=0, eos=1, think_start=2, think_end=3)


def _batch(params, padded=None):
    reqs = [SimpleNamespace(sampling_params=p, reasoning_state=ReasoningState.CHAT) for p in params]
    return SimpleNamespace(reqs=reqs, padded_size=padded or len(reqs))


def test_all_greedy_batches_need_no_tensors_and_take_the_argmax():
    s = Sampler("cpu", V, seed=0)
    args = s.prepare(_batch([SamplingParams(temperature=0.0), SamplingParams(top_k=1)]))
    assert args.all_greedy and args.mask_ids is None
    logits = torch.randn(2, V)
    assert torch.equal(s.sample(logits, args), logits.argmax(-1))


def test_mixed_batch_rows_keep_their_own_parameters_and_padding_is_greedy():
    s = Sampler("cpu", V, seed=0)
    args = s.prepare(_batch([SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, top_k=5, top_p=0.9)],
                            padded=4))
    assert args.temperature.tolist() == pytest.approx([0.0, 0.7, 0.0, 0.0])
    assert args.top_k.tolist()[1:] == [5, 1, 1] and args.top_p.tolist()[1] == pytest.approx(0.9)
    assert args.uniform.shape == (4,) and 0.0 <= float(args.uniform.min()) and float(args.uniform.max()) < 1.0
    logits = torch.randn(2, V)
    out = s.sample(logits, args)  # two live rows: the kernel is called with the first two rows of every tensor
    assert out.shape == (2,) and int(out[0]) == int(logits[0].argmax())


def test_top_k_and_top_p_restrict_the_support():
    torch.manual_seed(0)
    logits = torch.randn(1, V)
    order = logits[0].argsort(descending=True).tolist()
    probs = torch.softmax(logits[0], -1)
    seen_k, seen_p = set(), set()
    # smallest prefix of the sorted distribution whose mass reaches 0.5
    cum, nucleus = 0.0, []
    for i in order:
        nucleus.append(i)
        cum += float(probs[i])
        if cum >= 0.5:
            break
    for j in range(200):
        u = torch.tensor([(j + 0.5) / 200])
        one = torch.ones(1)
        seen_k.add(int(O.sample(logits, one, torch.tensor([3], dtype=torch.int32), one, u)[0]))
        seen_p.add(int(O.sample(logits, one, torch.tensor([-1], dtype=torch.int32), torch.tensor([0.5]), u)[0]))
    assert seen_k == set(order[:3])
    assert seen_p <= set(nucleus) and order[0] in seen_p
    # temperature -> 0 collapses onto the argmax whatever u is
    cold = O.sample(logits, torch.tensor([1e-4]), torch.tensor([-1], dtype=torch.int32), torch.ones(1),
                    torch.tensor([0.999]))
    assert int(cold[0]) == order[0]


def test_uniform_draw_maps_monotonically_onto_the_sorted_distribution():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.2] + [1e-9] * (V - 3)]))
    one, k = torch.ones(1), torch.tensor([-1], dtype=torch.int32)
    pick = lambda u: int(O.sample(logits, one, k, one, torch.tensor([u]))[0])
    assert [pick(0.1), pick(0.49), pick(0.55), pick(0.79), pick(0.85)] == [0, 0, 1, 1, 2]


@pytest.mark.parametrize("state,masked,free", [
    (ReasoningState.CHAT, (IDS.think_start, IDS.think_end), IDS.eos),
    (ReasoningState.THINKING, (IDS.think_start, IDS.eos), IDS.think_end),
    (ReasoningState.ANSWER, (IDS.think_start, IDS.think_end), IDS.eos),
])
def test_structural_tokens_are_masked_by_state(state, masked, free):
    s = ReasoningSampler("cpu", V, IDS, seed=0)
    assert s.mask_rows([int(state)]) == [list(masked)]
    logits = torch.zeros(1, V)
    logits[0, list(masked)] = 50.0  # the masked tokens would win by far
    logits[0, free] = 10.0
    args = s.prepare(_batch([SamplingParams(temperature=0.0)]), states=[int(state)])
    assert args.all_greedy and args.mask_ids.tolist() == [list(masked)]
    assert int(s.sample(logits, args)[0]) == free  # greedy rows go through the masking kernel too
    hot = s.prepare(_batch([SamplingParams(temperature=1.0)]), states=[int(state)])
    for _ in range(20):
        hot.uniform = torch.rand(1)
        assert int(s.sample(logits, hot)[0]) not in masked


def test_states_default_to_the_requests_and_padding_rows_are_chat():
    s = ReasoningSampler("cpu", V, IDS)
    b = _batch([SamplingParams(), SamplingParams()], padded=3)
    b.reqs[1].reasoning_state = ReasoningState.THINKING
    rows = s.prepare(b).mask_ids.tolist()
    assert rows == [[2, 3], [2, 1], [2, 3]]


class _Tok:
    """Smallest tokenizer surface the resolver reads."""

    def __init__(self, table, bos="<s>", eos="</s>"):
        self.table, self.bos_token, self.eos_token = table, bos, eos
        self.bos_token_id, self.eos_token_id = table.get(bos, [None])[0], table.get(eos, [None])[0]

    def encode(self, text, add_special_tokens=False):
        return list(self.table.get(text, [90, 91]))

    def convert_tokens_to_ids(self, text):
        ids = self.table.get(text)
        return ids[0] if ids and len(ids) == 1 else None


def test_structural_ids_resolve_strictly():
    good = {"<s>": [0], "</s>": [1], "<think>": [2], "</think>": [3]}
    assert resolve_reasoning_token_ids(_Tok(good)) == IDS
    with pytest.raises(RuntimeError, match="one token"):
        resolve_reasoning_token_ids(_Tok(dict(good, **{"</think>": [3, 4]})))
    with pytest.raises(RuntimeError, match="distinct"):
        resolve_reasoning_token_ids(_Tok(dict(good, **{"</think>": [2]})))
    no_bos = _Tok(good)
    no_bos.bos_token = None
    with pytest.raises(RuntimeError, match="BOS"):
        resolve_reasoning_token_ids(no_bos)
    wrong = _Tok(good)
    wrong.eos_token_id = 7
    with pytest.raises(RuntimeError, match="disagrees"):
        resolve_reasoning_token_ids(wrong)


def test_args_dataclass_defaults():
    a = BatchSamplingArgs()
    assert a.all_greedy and a.top_k is None and a.mask_ids is None
