"""The generation loop's decisions, with a scripted backend (no GPU)."""
import pytest

from lumenllm_b200.engine.generate import (GenerateRequest, GenerationError, generate,
                                           plan_batches, tokens_held)
from lumenllm_b200.sampling import SamplingConfig, uniform


class Scripted:
    """Every sequence produces script[slot-bound request][k] as its k-th token."""

    def __init__(self, scripts, n_slots=8):
        self.scripts = scripts
        self.free = list(range(n_slots - 1, -1, -1))
        self.held = {}
        self.calls = []          # per run: list of (slot, tokens fed)
        self.count = {}
        self.next_request = 0
        self.uniforms = []

    def alloc_slot(self):
        s = self.free.pop()
        self.held[s] = self.next_request
        self.count[s] = 0
        self.next_request += 1
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        del self.held[s]
        self.free.append(s)

    def run(self, entries, configs, uniforms):
        self.calls.append([(s, list(t)) for s, t in entries])
        self.uniforms.append(list(uniforms))
        out = []
        for s, _ in entries:
            assert s in self.held
            out.append(self.scripts[self.held[s]][self.count[s]])
            self.count[s] += 1
        return out


def test_eos_is_not_kept_stop_is_kept_length_ends_without_extra_forward():
    b = Scripted({0: [5, 6, 99], 1: [7, 42, 8], 2: [1, 2, 3, 4]})
    reqs = [GenerateRequest([10, 11, 12], max_tokens=8),
            GenerateRequest([13], max_tokens=8, stop_token_ids=[42]),
            GenerateRequest([14, 15], max_tokens=3)]
    outs = generate(b, reqs, eos_token_ids=[99])
    assert outs[0].tokens == [5, 6] and outs[0].finish_reason == "eos_token"
    assert outs[1].tokens == [7, 42] and outs[1].finish_reason == "stop"
    assert outs[2].tokens == [1, 2, 3] and outs[2].finish_reason == "length"
    assert [o.prompt_tokens for o in outs] == [3, 1, 2]
    assert [o.completion_tokens for o in outs] == [2, 2, 3]
    # step 0: the whole prompts together; then one token each; finished ones leave
    assert b.calls[0] == [(0, [10, 11, 12]), (1, [13]), (2, [14, 15])]
    assert b.calls[1] == [(0, [5]), (1, [7]), (2, [1])]
    assert b.calls[2] == [(0, [6]), (2, [2])]       # request 1 stopped; request 2 has one left
    assert len(b.calls) == 3                         # no forward after the last allowed token
    assert not b.held and sorted(b.free) == list(range(8))


def test_batches_follow_one_another_on_the_same_slots():
    scripts = {i: [i + 1] * 10 for i in range(5)}
    b = Scripted(scripts, n_slots=2)
    reqs = [GenerateRequest([1] * (i + 1), max_tokens=2 + i % 2) for i in range(5)]
    outs = generate(b, reqs, max_batch=2)
    assert [o.tokens for o in outs] == [[1, 1], [2, 2, 2], [3, 3], [4, 4, 4], [5, 5]]
    assert b.calls[0] == [(0, [1]), (1, [1, 1])]     # the first batch's prompts together
    used = {s for c in b.calls for s, _ in c}
    assert used == {0, 1}                            # slots were used again
    assert not b.held


def test_max_tokens_zero_and_empty_prompt():
    b = Scripted({0: [1]})
    outs = generate(b, [GenerateRequest([3], max_tokens=0)])
    assert outs[0].tokens == [] and outs[0].finish_reason == "length" and not b.calls
    with pytest.raises(GenerationError, match="no tokens"):
        generate(b, [GenerateRequest([], max_tokens=1)])


def test_first_token_can_end_a_request():
    b = Scripted({0: [99], 1: [42], 2: [3]})
    outs = generate(b, [GenerateRequest([1], 5), GenerateRequest([1], 5, stop_token_ids=[42]),
                        GenerateRequest([1], 1)], eos_token_ids=[99])
    assert [o.tokens for o in outs] == [[], [42], [3]]
    assert [o.finish_reason for o in outs] == ["eos_token", "stop", "length"]
    assert len(b.calls) == 1


def test_seeded_uniforms_do_not_depend_on_the_batch():
    s = SamplingConfig(temperature=0.8, seed=123)
    alone = Scripted({0: [1, 2, 3, 4]})
    generate(alone, [GenerateRequest([9], 4, s)])
    together = Scripted({0: [5] * 6, 1: [1, 2, 3, 4], 2: [6] * 2})
    generate(together, [GenerateRequest([9, 9], 6, SamplingConfig(temperature=1.0, seed=5)),
                        GenerateRequest([9], 4, s), GenerateRequest([8], 2, s)])
    a = [u[0] for u in alone.uniforms]
    t = [u[1] for u in together.uniforms[:4]]
    assert a == t == [uniform(123, 0, k) for k in range(4)]
    assert all(0.0 <= x < 1.0 for x in a) and len(set(a)) == 4


def test_plan_batches_respects_slots_and_cache():
    reqs = [GenerateRequest([0] * 60, 5), GenerateRequest([0] * 64, 2), GenerateRequest([0] * 10, 200),
            GenerateRequest([0] * 1, 1)]
    assert [tokens_held(r) for r in reqs] == [64, 128, 256, 64]
    assert plan_batches(reqs, 8, 1 << 20) == [[0, 1, 2, 3]]
    assert plan_batches(reqs, 2, 1 << 20) == [[0, 1], [2, 3]]
    assert plan_batches(reqs, 8, 256) == [[0, 1], [2], [3]]
    with pytest.raises(GenerationError, match="cache holds"):
        plan_batches(reqs, 8, 128)


def test_on_token_callback():
    seen = []
    b = Scripted({0: [4, 5, 99]})
    generate(b, [GenerateRequest([1], 9)], eos_token_ids=[99], on_token=lambda i, t: seen.append((i, t)))
    assert seen == [(0, 4), (0, 5)]
