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


class ScriptedAhead(Scripted):
    """The same scripted sequences behind launch / collect: a step's tokens become known
    only when it is collected, and a step may be fed from the step before it."""

    def __init__(self, scripts, n_slots=8):
        super().__init__(scripts, n_slots)
        self.in_flight = 0
        self.max_in_flight = 0
        self.freed_while_held = []

    def launch(self, entries, configs, uniforms, after=None, rows=None):
        fed = []
        for k, (s, t) in enumerate(entries):
            assert s in self.held, "a launched step names a slot that was given back"
            if after is None:
                fed.append((s, list(t)))
            else:
                assert t is None
                fed.append((s, [after["tokens"][rows[k]]]))
                assert after["slots"][rows[k]] == s
        self.calls.append(fed)
        self.uniforms.append(list(uniforms))
        toks = []
        for s, _ in entries:
            toks.append(self.scripts[self.held[s]][self.count[s]])
            self.count[s] += 1
        self.in_flight += 1
        self.max_in_flight = max(self.max_in_flight, self.in_flight)
        return {"tokens": toks, "slots": [s for s, _ in entries]}

    def collect(self, handle):
        self.in_flight -= 1
        return list(handle["tokens"])


def test_run_ahead_gives_the_same_tokens_and_reasons():
    scripts = {0: [5, 6, 99, 1, 1], 1: [7, 42, 8, 8], 2: [1, 2, 3, 4], 3: [9] * 12}
    reqs = [GenerateRequest([10, 11, 12], max_tokens=8),
            GenerateRequest([13], max_tokens=8, stop_token_ids=[42]),
            GenerateRequest([14, 15], max_tokens=3),
            GenerateRequest([16], max_tokens=6, sampling=SamplingConfig(temperature=0.5, seed=3))]
    plain_b, ahead_b = Scripted(scripts), ScriptedAhead(scripts)
    want = generate(plain_b, reqs, eos_token_ids=[99])
    got = generate(ahead_b, reqs, eos_token_ids=[99])
    assert [(o.tokens, o.finish_reason) for o in got] == [(o.tokens, o.finish_reason) for o in want]
    assert ahead_b.max_in_flight == 2                 # one step ahead, never more
    assert not ahead_b.held and sorted(ahead_b.free) == list(range(8))
    # request 2 ends by length: it is in no step after the one that gives its last token
    assert sum(1 for c in ahead_b.calls for s, _ in c if s == 2) == 3
    # request 0 ends by EOS at its third token: it was run ahead once more, and that is all
    assert sum(1 for c in ahead_b.calls for s, _ in c if s == 0) == 4
    # every sequence saw, step by step, the tokens it produced itself
    for c in ahead_b.calls[1:]:
        for s, t in c:
            assert len(t) == 1
    # uniforms are numbered by the request's own steps, as without the run-ahead
    u3 = [u for c, us in zip(ahead_b.calls, ahead_b.uniforms) for (s, _), u in zip(c, us) if s == 3]
    assert u3[:6] == [uniform(3, 0, k) for k in range(6)]


def test_run_ahead_batches_reuse_slots_only_after_their_last_step():
    scripts = {i: [i + 1, 77] + [i + 1] * 6 for i in range(6)}
    b = ScriptedAhead(scripts, n_slots=2)
    reqs = [GenerateRequest([1] * (i + 1), max_tokens=4) for i in range(6)]
    outs = generate(b, reqs, eos_token_ids=[77], max_batch=2)
    assert [o.tokens for o in outs] == [[i + 1] for i in range(6)]
    assert all(o.finish_reason == "eos_token" for o in outs)
    assert not b.held and b.in_flight == 0


@pytest.mark.parametrize("ahead", [False, True])
def test_a_refused_step_gives_the_slots_back(ahead):
    class Refusing(ScriptedAhead if ahead else Scripted):
        def _count(self):
            self.n = getattr(self, "n", 0) + 1
            if self.n == 3:
                raise RuntimeError("kv cache context exhausted")

        def run(self, entries, configs, uniforms):
            self._count()
            return Scripted.run(self, entries, configs, uniforms)

        def launch(self, entries, configs, uniforms, after=None, rows=None):
            self._count()
            return ScriptedAhead.launch(self, entries, configs, uniforms, after=after, rows=rows)

    b = Refusing({0: [1] * 9, 1: [2] * 9}, n_slots=4)
    with pytest.raises(RuntimeError, match="exhausted"):
        generate(b, [GenerateRequest([5, 6], max_tokens=8), GenerateRequest([7], max_tokens=8)])
    assert not b.held and sorted(b.free) == list(range(4))


def test_the_shape_of_a_captured_step_depends_on_counts_alone():
    """Which captured step serves a batch: tokens and sequences rounded up to buckets, the
    surplus tokens in the first padding sequence, the other padding sequences empty; a step of
    one token each has as many tokens as sequences."""
    from lumenllm_b200.engine.step_graph import StepGraphs
    assert StepGraphs.plan([1]) == (1, 1, [])
    assert StepGraphs.plan([1, 1, 1]) == (4, 4, [1])
    assert StepGraphs.plan([1] * 9) == (16, 16, [1] * 7)
    assert StepGraphs.plan([1] * 65) == (128, 128, [1] * 63)
    assert StepGraphs.plan([128]) == (128, 2, [0])                  # a full bucket needs no padding token
    assert StepGraphs.plan([33, 2, 65]) == (128, 4, [28])
    assert StepGraphs.plan([70, 20, 7]) == (128, 4, [31])           # another division, the same shape
    assert StepGraphs.plan([100, 1]) == (128, 4, [27, 0])
    assert StepGraphs.plan([513]) == (576, 2, [63])
    for lens in ([5], [1, 2], [600, 300], [31] * 7):
        n_tok, n_seq, pads = StepGraphs.plan(lens)
        assert n_tok == sum(lens) + sum(pads) and n_seq == len(lens) + len(pads) and n_tok > n_seq
