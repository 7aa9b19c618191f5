"""The engine against the plain implementation, in float32 and in bfloat16: each request
alone and whole; with the last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used
again; long decoding; the first tokens of a sequence; generation through the entry point;
the replay tool as a program."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from conftest import ROOT, TINY, Ref, check, plain_ref, seeded_tokens, tolerance

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D", "E"]


@pytest.fixture(scope="module")
def plain(tiny_models):
    return {n: P.load_model(tiny_models[n]) for n in NAMES}


@pytest.fixture(scope="module")
def engines(tiny_models):
    from lumenllm_b200 import Engine
    cache = {}

    def get(name, dtype, max_tokens=4096):
        key = (name, dtype, max_tokens)
        if key not in cache:
            cache[key] = Engine.from_folder(tiny_models[name], dtype=dtype, max_tokens=max_tokens)
        return cache[key]
    return get


def run_whole(eng, seq):
    from lumenllm_b200 import StepEntry
    s = eng.alloc_slot()
    lg = eng.step([StepEntry(s, seq, list(range(len(seq))))]).cpu()
    eng.free_slot(s)
    return lg


def eager_decode(eng, pairs):
    """One token each for [(slot, token)] through Engine.step (kernels launched one by one)."""
    from lumenllm_b200 import StepEntry
    return eng.step([StepEntry(s, [t], [0]) for s, t in pairs]).cpu()


def captured_decode(eng, pairs):
    """The same step the way generation and the benchmark run it: replayed from a CUDA graph
    captured for the batch's bucket (padding sequences fill it) and the page table's width
    bucket. The logits are the replayed step's own."""
    from lumenllm_b200.sampling import SamplingConfig
    n = len(pairs)
    before = eng.steps_run
    eng.run_device([(s, [t]) for s, t in pairs], [SamplingConfig()] * n, [0.0] * n)
    cap = eng.graphs.last
    assert eng.steps_run == before + 1 and cap.ctx.B >= n and cap.logits.shape[0] == cap.ctx.B
    return cap.logits[:n].float().cpu()


DECODERS = {"eager": eager_decode, "captured": captured_decode}


def run_tail(eng, seq, tail=32, decode=eager_decode):
    from lumenllm_b200 import StepEntry
    s = eng.alloc_slot()
    cut = max(1, len(seq) - tail)
    out = [eng.step([StepEntry(s, seq[:cut], list(range(cut)))]).cpu()]
    for t in seq[cut:]:
        out.append(decode(eng, [(s, t)]))
    eng.free_slot(s)
    return torch.cat(out)


def run_batch(eng, seqs, prompt_lens, decode=eager_decode):
    """All prompts in one step, then one token each; a finished request leaves at once."""
    from lumenllm_b200 import StepEntry
    slots = [eng.alloc_slot() for _ in seqs]
    lg = eng.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, prompt_lens)]).cpu()
    got, o = [], 0
    for c in prompt_lens:
        got.append([lg[o:o + c]])
        o += c
    pos = list(prompt_lens)
    live = list(range(len(seqs)))
    while True:
        for i in [i for i in live if pos[i] >= len(seqs[i])]:
            eng.free_slot(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
        if not live:
            break
        lg = decode(eng, [(slots[i], seqs[i][pos[i]]) for i in live])
        for k, i in enumerate(live):
            got[i].append(lg[k:k + 1])
            pos[i] += 1
    return [torch.cat(g) for g in got]


@pytest.fixture(scope="module")
def parity_refs(plain):
    """Sequences and their plain logits, shared by the eager and the captured run."""
    lens = [7, 1, 19, 150, 70, 33, 2, 64, 11, 129]
    out = {}
    for name in NAMES:
        cfg, w = plain[name]
        seqs = seeded_tokens(cfg["vocab_size"], lens, 100 + ord(name))
        out[name] = (seqs, [plain_ref(cfg, w, s) for s in seqs])
    return out


@pytest.mark.parametrize("how", ["eager", "captured"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_tail_and_batches(name, dtype, how, parity_refs, engines):
    """Each request whole; with its last 32 tokens one by one; in batches of unequal lengths
    one after another. Single tokens go through Engine.step ("eager") or through the replayed
    CUDA graph ("captured": batches of 1, 3, 4, 5 and 9 land in the buckets 1, 4, 8 and 16,
    the sequences of 129 and 150 tokens cross a page and a width bucket while decoding)."""
    decode = DECODERS[how]
    eng = engines(name, dtype)
    seqs, refs = parity_refs[name]
    if how == "eager":
        for s, r in zip(seqs, refs):
            check(run_whole(eng, s), r, dtype, f"{name} whole len {len(s)}")
    for s, r in zip(seqs, refs):
        check(run_tail(eng, s, decode=decode), r, dtype, f"{name} {how} tail32 len {len(s)}")
    # batches of unequal lengths, one after another on the same engine
    for batch in ([0, 1, 2], [3, 4, 5, 6], [7, 8, 9, 0, 3], [9, 8, 7, 6, 5, 4, 3, 2, 1]):
        bs = [seqs[i] for i in batch]
        cuts = [max(1, (len(s) * 2) // 3) for s in bs]
        for g, i in zip(run_batch(eng, bs, cuts, decode=decode), batch):
            check(g, refs[i], dtype, f"{name} {how} batch {batch} request {i}")
        eng.cache.check()
    assert not eng.cache.slots.held
    for g in eng.cache.groups:
        assert g.pool.free_count == g.pool.capacity


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again_hold_no_stale_keys(dtype, plain, tiny_models):
    """A cache just large enough: every page of the second batch was used by the first."""
    from lumenllm_b200 import Engine
    cfg, w = plain["B"]
    eng = Engine.from_folder(tiny_models["B"], dtype=dtype, max_tokens=4 * 64, max_slots=2)
    seqs = seeded_tokens(cfg["vocab_size"], [100, 120, 90, 128, 5, 70], 7)
    refs = [plain_ref(cfg, w, s) for s in seqs]
    for pair in ([0, 1], [2, 3], [4, 5], [1, 2]):
        bs = [seqs[i] for i in pair]
        for g, i in zip(run_batch(eng, bs, [len(s) // 2 for s in bs]), pair):
            check(g, refs[i], dtype, f"reuse pair {pair} request {i}")
        eng.cache.check()


@pytest.mark.parametrize("how", ["eager", "captured"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D", "E"])
def test_long_decoding(name, dtype, how, plain, engines):
    """3 prompt tokens, then 400 single tokens: page edges, the 128-key chunk edges of the
    attention kernels, for C and D the window sliding over page edges (pages given back
    while the captured step goes on), and for the captured step a new capture each time the
    page table's width bucket grows (1, 2, 4, 8 pages)."""
    cfg, w = plain[name]
    seq = seeded_tokens(cfg["vocab_size"], [403], 21)[0]
    ref = plain_ref(cfg, w, seq)
    eng = engines(name, dtype)
    check(run_tail(eng, seq, tail=400, decode=DECODERS[how]), ref, dtype, f"{name} long decode")
    if how == "captured":
        assert {k[2] for k in eng.graphs.captured if k[:2] == (1, 1)} >= {1, 2, 4, 8}


def captured_step(eng, pairs):
    """[(slot, tokens)] through the captured step (prompts or single tokens): the logits at
    each sequence's last token, and the captured step that was replayed."""
    from lumenllm_b200.sampling import SamplingConfig
    n = len(pairs)
    eng.run_device(pairs, [SamplingConfig()] * n, [0.0] * n)
    cap = eng.graphs.last
    return cap.logits[:n].float().cpu(), cap


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_captured_prompt_steps(name, dtype, plain, engines, tiny_models):
    """Prompts of unequal lengths through the captured prompt step, the way generation feeds
    them: a batch that captures a step for its buckets (128 tokens, 4 sequences, 2 pages); a
    second batch with another division of its tokens that replays the same captured step on
    the slots and pages the first gave back; a piece that continues cached prompts; then
    single tokens. Against the plain implementation, and bit for bit against the same steps
    launched kernel by kernel on a twin engine (padding tokens change nothing)."""
    from lumenllm_b200 import Engine, StepEntry
    cfg, w = plain[name]
    eng = engines(name, dtype)
    twin = Engine.from_folder(tiny_models[name], dtype=dtype, max_tokens=4096, use_graphs=False)
    first_cap = None
    for round_, lens in enumerate(([33, 2, 65], [70, 20, 7])):
        seqs = seeded_tokens(cfg["vocab_size"], [n + 12 for n in lens], 300 + round_)
        refs = [plain_ref(cfg, w, q) for q in seqs]
        slots = [eng.alloc_slot() for _ in seqs]
        tslots = [twin.alloc_slot() for _ in seqs]
        lg, cap = captured_step(eng, [(s, q[:n]) for s, q, n in zip(slots, seqs, lens)])
        assert (cap.ctx.N, cap.ctx.B) == (128, 4)
        check(lg, Ref.cat([r[n - 1:n] for r, n in zip(refs, lens)]), dtype, f"{name} captured prompts {lens}")
        eager = twin.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(tslots, seqs, lens)]).cpu()
        assert torch.equal(lg, eager), f"{name} {lens}: captured and eager prompt step differ"
        if first_cap is None:
            first_cap = cap
        else:
            assert cap is first_cap                  # replayed, not captured again
        # nine more tokens of each prompt on top of what is cached, then three single tokens
        lg, cap = captured_step(eng, [(s, q[n:n + 9]) for s, q, n in zip(slots, seqs, lens)])
        assert cap.ctx.N == 32
        check(lg, Ref.cat([r[n + 8:n + 9] for r, n in zip(refs, lens)]), dtype, f"{name} captured continuation {lens}")
        for t in range(9, 12):
            lg = captured_decode(eng, [(s, q[n + t]) for s, q, n in zip(slots, seqs, lens)])
            check(lg, Ref.cat([r[n + t:n + t + 1] for r, n in zip(refs, lens)]), dtype,
                  f"{name} token {t} after captured prompts {lens}")
        for s in slots:
            eng.free_slot(s)
        for s in tslots:
            twin.free_slot(s)
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E"])
def test_a_padded_captured_batch_equals_the_eager_step(name, dtype, plain, tiny_models):
    """Three sequences of unequal lengths in the bucket of four, 150 steps that cross 64 and
    128 keys and two width buckets: every replayed step against the plain implementation,
    and bit for bit against Engine.step on a twin engine (padding sequences, the padded page
    table and the replay itself change nothing)."""
    from lumenllm_b200 import Engine, StepEntry
    cfg, w = plain[name]
    seqs = seeded_tokens(cfg["vocab_size"], [40 + 150, 7 + 150, 100 + 150], 23)
    refs = [plain_ref(cfg, w, s) for s in seqs]
    cuts = [40, 7, 100]
    twins = [Engine.from_folder(tiny_models[name], dtype=dtype, max_tokens=2048) for _ in range(2)]
    slots = []
    for eng in twins:
        sl = [eng.alloc_slot() for _ in seqs]
        eng.step([StepEntry(s, q[:c], []) for s, q, c in zip(sl, seqs, cuts)])
        slots.append(sl)
    for t in range(150):
        toks = [q[c + t] for q, c in zip(seqs, cuts)]
        a = captured_decode(twins[0], list(zip(slots[0], toks)))
        b = eager_decode(twins[1], list(zip(slots[1], toks)))
        assert twins[0].graphs.last.ctx.B == 4
        assert torch.equal(a, b), f"{name} step {t}: replay and eager step differ"
        for k in range(3):
            check(a[k:k + 1], refs[k][cuts[k] + t:cuts[k] + t + 1], dtype, f"{name} step {t} request {k}")
    assert len({key[2] for key in twins[0].graphs.captured}) >= 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(name, dtype, plain, engines):
    from lumenllm_b200 import StepEntry
    cfg, w = plain[name]
    eng = engines(name, dtype)
    seqs = seeded_tokens(cfg["vocab_size"], [1, 2, 3, 1], 31)
    refs = [plain_ref(cfg, w, s) for s in seqs]
    slots = [eng.alloc_slot() for _ in seqs]
    # token by token from the very first one, all four together
    for t in range(3):
        live = [i for i in range(4) if t < len(seqs[i])]
        lg = eng.step([StepEntry(slots[i], [seqs[i][t]], [0]) for i in live]).cpu()
        for k, i in enumerate(live):
            check(lg[k:k + 1], refs[i][t:t + 1], dtype, f"{name} first tokens, request {i} place {t}")
    for s in slots:
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_want_selects_rows_and_may_be_empty(dtype, plain, engines):
    from lumenllm_b200 import StepEntry
    cfg, w = plain["B"]
    eng = engines("B", dtype)
    a, b = seeded_tokens(cfg["vocab_size"], [20, 9], 41)
    ra, rb = plain_ref(cfg, w, a), plain_ref(cfg, w, b)
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    lg = eng.step([StepEntry(sa, a[:10], []), StepEntry(sb, b, [8, 0])]).cpu()
    assert lg.shape[0] == 2
    check(lg, Ref.stack([rb[8], rb[0]]), dtype, "want order")
    assert eng.step([StepEntry(sa, a[10:15], [])]).shape[0] == 0
    lg = eng.step([StepEntry(sa, a[15:], [4])]).cpu()
    check(lg, ra[19:20], dtype, "after steps that wanted nothing")
    eng.free_slot(sa); eng.free_slot(sb)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_two_live_batches_take_turns(name, dtype, plain, engines):
    """Two batches hold the cache at the same time and are stepped in turn (prompts of the
    first, prompts of the second, then a token each, alternately): neither reads the other's
    keys, and the captured decode step serves whichever slots a step names."""
    from lumenllm_b200 import StepEntry
    cfg, w = plain[name]
    eng = engines(name, dtype)
    seqs = seeded_tokens(cfg["vocab_size"], [70, 9, 131, 40, 66], 61)
    refs = [plain_ref(cfg, w, s) for s in seqs]
    groups = ([0, 1], [2, 3, 4])
    cuts = [len(s) - 6 for s in seqs]
    slots = [eng.alloc_slot() for _ in seqs]
    for grp in groups:
        lg = eng.step([StepEntry(slots[i], seqs[i][:cuts[i]], [cuts[i] - 1]) for i in grp]).cpu()
        for k, i in enumerate(grp):
            check(lg[k:k + 1], refs[i][cuts[i] - 1:cuts[i]], dtype, f"{name} prompts of {grp}, request {i}")
    for t in range(6):
        for grp in groups:
            lg = captured_decode(eng, [(slots[i], seqs[i][cuts[i] + t]) for i in grp])
            for k, i in enumerate(grp):
                check(lg[k:k + 1], refs[i][cuts[i] + t:cuts[i] + t + 1], dtype,
                      f"{name} turn {t} of {grp}, request {i}")
    for s in slots:
        eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_nothing(dtype, plain, engines):
    from lumenllm_b200 import StepEntry
    cfg, w = plain["A"]
    eng = engines("A", dtype)
    a, b = seeded_tokens(cfg["vocab_size"], [30, 5], 51)
    outs = []
    for pad in (0, 8):
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        eng.step([StepEntry(sa, a[:-1], []), StepEntry(sb, b[:-1], [])])
        entries = [StepEntry(sa, a[-1:], [0]), StepEntry(sb, b[-1:], [0])]
        ctx = eng.build_context(entries, pad_to=pad)
        outs.append(eng.model.forward(ctx).cpu())
        eng.free_slot(sa); eng.free_slot(sb)
    assert torch.equal(outs[0], outs[1])
    ref = Ref.stack([plain_ref(cfg, w, a)[-1], plain_ref(cfg, w, b)[-1]])
    check(outs[1], ref, dtype, "padded step")


@pytest.mark.parametrize("dtype", DTYPES)
def test_large_step_is_cut_into_passes(dtype, plain, tiny_models):
    from lumenllm_b200 import Engine, StepEntry
    cfg, w = plain["A"]
    eng = Engine.from_folder(tiny_models["A"], dtype=dtype, max_tokens=1024, max_step_tokens=37)
    seqs = seeded_tokens(cfg["vocab_size"], [90, 10, 41], 61)
    slots = [eng.alloc_slot() for _ in seqs]
    wants = [[89, 0, 40], [9], [40, 36, 37]]
    lg = eng.step([StepEntry(s, q, wt) for s, q, wt in zip(slots, seqs, wants)]).cpu()
    ref = Ref.cat([plain_ref(cfg, w, q)[wt] for q, wt in zip(seqs, wants)])
    check(lg, ref, dtype, "cut step")


def test_refused_steps(engines):
    from lumenllm_b200 import StepEntry, StepError
    eng = engines("A", "float32")
    s = eng.alloc_slot()
    for bad, msg in (([], "at least one sequence"),
                     ([StepEntry(s, [], [])], "at least one token"),
                     ([StepEntry(s, [256], [])], "outside the vocabulary"),
                     ([StepEntry(s, [-1], [])], "outside the vocabulary"),
                     ([StepEntry(s, [1], [1])], "wanted place"),
                     ([StepEntry(s, [1], []), StepEntry(s, [2], [])], "twice"),
                     ([StepEntry(999, [1], [])], "not live"),
                     ([StepEntry(s, [1] * 1025, [])], "context")):
        with pytest.raises(StepError, match=msg):
            eng.step(bad)
    assert eng.length(s) == 0
    eng.free_slot(s)
    small = engines("A", "float32", 128)
    a, b = small.alloc_slot(), small.alloc_slot()
    small.step([StepEntry(a, [1] * 100, [])])
    with pytest.raises(StepError, match=f"slot {b}.*full"):
        small.step([StepEntry(b, [1] * 100, [])])
    small.free_slot(a); small.free_slot(b)


def _teacher_check(cfg, w, prompt, produced, dtype):
    """Every produced token is the plain implementation's choice given the same prefix,
    or ties with it within the tolerance."""
    lg = P.forward_logits(cfg, w, list(prompt) + list(produced))
    for k, tok in enumerate(produced):
        row = lg[len(prompt) - 1 + k]
        assert float(row.max() - row[tok]) <= 2 * tolerance(dtype, row), (k, tok)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name, dtype, plain, tiny_models):
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    cfg, w = plain[name]
    built = build(EngineConfig(model_path=str(tiny_models[name]), dtype=dtype, context_size=256,
                               max_batch=3))
    lens = [7, 1, 19] if name == "A" else [33, 2, 64, 11]
    steps = 8 if name == "A" else 12
    prompts = seeded_tokens(cfg["vocab_size"], lens, 71)
    outs = built.generate([GenerateRequest(p, steps) for p in prompts], eos_token_ids=[])
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and o.completion_tokens == steps
        _teacher_check(cfg, w, p, o.tokens, dtype)
        if dtype == "float32":
            assert o.tokens == P.generate_greedy(cfg, w, p, steps)[0]
    # stop and eos, decided from the tokens the first run produced
    first = outs[0].tokens
    o2 = built.generate(GenerateRequest(prompts[0], steps, stop_token_ids=[first[3]]), eos_token_ids=[])
    assert o2.tokens == first[:first.index(first[3]) + 1] and o2.finish_reason == "stop"
    o3 = built.generate(GenerateRequest(prompts[0], steps), eos_token_ids=[first[2]])
    assert o3.tokens == first[:first.index(first[2])] and o3.finish_reason == "eos_token"
    built.engine.cache.check()
    assert not built.engine.cache.slots.held


@pytest.mark.parametrize("dtype", DTYPES)
def test_seeded_sampling_alone_and_in_a_batch(dtype, plain, tiny_models):
    from lumenllm_b200 import EngineConfig, GenerateRequest, SamplingConfig, build
    cfg, w = plain["B"]
    built = build(EngineConfig(model_path=str(tiny_models["B"]), dtype=dtype, context_size=256,
                               max_batch=4))
    prompts = seeded_tokens(cfg["vocab_size"], [33, 2, 64, 11], 81)
    sc = [SamplingConfig(temperature=0.8, seed=1000 + i) for i in range(4)]
    together = built.generate([GenerateRequest(p, 12, s) for p, s in zip(prompts, sc)], eos_token_ids=[])
    again = built.generate([GenerateRequest(p, 12, s) for p, s in zip(prompts, sc)], eos_token_ids=[])
    assert [o.tokens for o in together] == [o.tokens for o in again]
    # a request's tokens do not depend on who else is in the batch, in either precision: every
    # cut of the keys and every split sum depends on the sequence and on the weights alone
    for p, s, o in zip(prompts, sc, together):
        alone = built.generate(GenerateRequest(p, 12, s), eos_token_ids=[])
        assert alone.tokens == o.tokens
    other = built.generate(GenerateRequest(prompts[0], 12, SamplingConfig(temperature=0.8, seed=5)),
                           eos_token_ids=[])
    assert other.tokens != together[0].tokens


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_decoded_logits_do_not_depend_on_the_batch(name, dtype, plain, engines):
    """One sequence decoded alone (bucket 1), among 5 (bucket 8) and among 40 (bucket 64),
    at 300 cached keys (five pages, two segments of the split attention): the same bits."""
    from lumenllm_b200 import StepEntry
    cfg, w = plain[name]
    eng = engines(name, dtype, 64 * 6 * 48)
    seqs = seeded_tokens(cfg["vocab_size"], [301] + [20] * 39, 95)
    outs = []
    for n in (1, 5, 40):
        slots = [eng.alloc_slot() for _ in range(n)]
        eng.step([StepEntry(s, q[:-1], []) for s, q in zip(slots, seqs)])
        outs.append(captured_decode(eng, [(s, q[-1]) for s, q in zip(slots, seqs)])[0])
        for sl in slots:
            eng.free_slot(sl)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    check(outs[0][None], plain_ref(cfg, w, seqs[0])[-1:], dtype, "alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "E"])
def test_a_prompt_joins_requests_that_decode(name, dtype, plain, engines):
    """A mixed step against the plain implementation: two requests bring one token each while
    a third brings its whole prompt; then all three decode; then the same on the slots and
    pages that these gave back."""
    from lumenllm_b200 import StepEntry
    cfg, w = plain[name]
    eng = engines(name, dtype)
    for round_ in range(2):
        seqs = seeded_tokens(cfg["vocab_size"], [90, 35, 70], 200 + round_)
        refs = [plain_ref(cfg, w, q) for q in seqs]
        a, b, c = (eng.alloc_slot() for _ in range(3))
        eng.step([StepEntry(a, seqs[0][:80], []), StepEntry(b, seqs[1][:30], [])])
        for t in range(2):
            eng.step([StepEntry(a, [seqs[0][80 + t]], []), StepEntry(b, [seqs[1][30 + t]], [])])
        lg = eng.step([StepEntry(a, [seqs[0][82]], [0]), StepEntry(c, seqs[2][:66], [0, 64, 65]),
                       StepEntry(b, [seqs[1][32]], [0])]).cpu()
        ref = Ref.cat([refs[0][82:83], refs[2][[0, 64, 65]], refs[1][32:33]])
        check(lg, ref, dtype, f"{name} mixed step, round {round_}")
        for t in range(2):
            lg = eng.step([StepEntry(a, [seqs[0][83 + t]], [0]), StepEntry(b, [seqs[1][33 + t]], [0]),
                           StepEntry(c, [seqs[2][66 + t]], [0])]).cpu()
            ref = Ref.cat([refs[0][83 + t:84 + t], refs[1][33 + t:34 + t], refs[2][66 + t:67 + t]])
            check(lg, ref, dtype, f"{name} after the mixed step, token {t}, round {round_}")
        for sl in (a, b, c):
            eng.free_slot(sl)
        eng.cache.check()


@pytest.mark.parametrize("how", ["eager", "captured"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_that_want_nothing_still_fill_the_cache(dtype, how, plain, engines):
    """Every entry of a step wants nothing (the last update of the stream is dropped, no head
    runs); the single tokens after it must find all keys of those steps."""
    from lumenllm_b200 import StepEntry
    cfg, w = plain["D"]
    eng = engines("D", dtype)
    a, b = seeded_tokens(cfg["vocab_size"], [75, 12], 43)
    ra, rb = plain_ref(cfg, w, a), plain_ref(cfg, w, b)
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    assert eng.step([StepEntry(sa, a[:70], []), StepEntry(sb, b[:9], [])]).shape[0] == 0
    assert eng.step([StepEntry(sa, a[70:71], []), StepEntry(sb, b[9:10], [])]).shape[0] == 0
    for t in range(2):
        lg = DECODERS[how](eng, [(sa, a[71 + t]), (sb, b[10 + t])])
        check(lg, Ref.stack([ra[71 + t], rb[10 + t]]), dtype, f"token {t} after steps that wanted nothing")
    eng.free_slot(sa); eng.free_slot(sb)


@pytest.mark.parametrize("dtype", DTYPES)
def test_positions_given_by_the_caller_reach_the_rotation(dtype, plain, engines):
    """`positions` of a StepEntry replace the cache index in the rotation only: a sequence
    whose tokens are rotated as if it began at position 1,000 gives the plain logits for
    positions 1,000.. (attention is a function of position differences, so they equal the
    unshifted ones within rounding), while keys still lie at the cache's own indices."""
    from lumenllm_b200 import StepEntry, StepError
    cfg, w = plain["B"]
    eng = engines("B", dtype)
    seq = seeded_tokens(cfg["vocab_size"], [50], 47)[0]
    ref = plain_ref(cfg, w, seq, positions=list(range(1000, 1050)))
    s = eng.alloc_slot()
    lg = [eng.step([StepEntry(s, seq[:40], list(range(40)), positions=list(range(1000, 1040)))]).cpu()]
    for t in range(40, 50):
        lg.append(eng.step([StepEntry(s, [seq[t]], [0], positions=[1000 + t])]).cpu())
    check(torch.cat(lg), ref, dtype, "shifted positions")
    assert eng.length(s) == 50
    with pytest.raises(StepError, match="positions"):
        eng.step([StepEntry(s, [1, 2], [], positions=[3])])
    eng.free_slot(s)
    # and positions that are no shift change the result
    s = eng.alloc_slot()
    odd = eng.step([StepEntry(s, seq[:40], [39], positions=list(range(0, 80, 2)))]).cpu()
    eng.free_slot(s)
    want = plain_ref(cfg, w, seq[:40], positions=list(range(0, 80, 2)))[-1:]
    check(odd, want, dtype, "stretched positions")
    assert float((odd - P.forward_logits(cfg, w, seq[:40])[-1:]).abs().max()) > 10 * tolerance(dtype, want.f32)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_kernel_that_gave_up_is_reported_and_the_engine_goes_on(dtype, plain, tiny_models):
    """The kernels' bounded waits set a flag on the device when they run out. Here the flag is
    set by hand (no kernel has to time out for this): generation raises instead of handing
    tokens back, gives its slots back, and the next call works; so does the step-by-step face
    and trace replay's check."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, KernelError, StepEntry, build
    from lumenllm_b200.ops import kernels as K
    cfg, w = plain["B"]
    built = build(EngineConfig(model_path=str(tiny_models["B"]), dtype=dtype, context_size=256, max_batch=4))
    eng = built.engine
    prompts = seeded_tokens(cfg["vocab_size"], [12, 5], 53)
    good = built.generate([GenerateRequest(p, 6) for p in prompts], eos_token_ids=[])
    K.error_flag(eng.device).fill_(1)
    K._decode_counters(eng.device)[:4].fill_(3)           # as blocks that gave up would leave them
    with pytest.raises(KernelError, match="gave up"):
        built.generate([GenerateRequest(p, 6) for p in prompts], eos_token_ids=[])
    assert not eng.cache.slots.held
    assert int(K.error_flag(eng.device).item()) == 0 and int(K._decode_counters(eng.device).abs().sum()) == 0
    again = built.generate([GenerateRequest(p, 6) for p in prompts], eos_token_ids=[])
    assert [o.tokens for o in again] == [o.tokens for o in good]
    # the face without run-ahead, and the check that trace replay makes before it writes
    s = eng.alloc_slot()
    K.error_flag(eng.device).fill_(1)
    with pytest.raises(KernelError):
        eng.run([(s, prompts[0])], [built.default_sampling()], [0.0])
    eng.free_slot(s)
    s = eng.alloc_slot()
    eng.step([StepEntry(s, prompts[0], [0])])
    K.error_flag(eng.device).fill_(1)
    with pytest.raises(KernelError):
        eng.check_kernels()
    eng.check_kernels()
    eng.free_slot(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_step_ahead_gives_what_step_by_step_gives(dtype, plain, tiny_models):
    """The engine offers launch / collect, so generation keeps one step in flight ahead of the
    host; behind a face that offers `run` alone it waits for every step. Same tokens and
    reasons either way: sampled requests of unequal lengths, one that meets a stop token, one
    that meets EOS (its token run ahead is dropped), one that uses its allowance up."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, SamplingConfig, build
    from lumenllm_b200.engine.generate import generate
    cfg, w = plain["B"]
    built = build(EngineConfig(model_path=str(tiny_models["B"]), dtype=dtype, context_size=256,
                               max_batch=4))
    eng = built.engine

    class StepByStep:
        alloc_slot, free_slot, run = eng.alloc_slot, eng.free_slot, eng.run

    prompts = seeded_tokens(cfg["vocab_size"], [21, 3, 40, 9, 5, 17], 83)
    probe = generate(StepByStep(), [GenerateRequest(p, 10, SamplingConfig(temperature=0.9, seed=50 + i))
                                    for i, p in enumerate(prompts)], max_batch=4)
    eos = [probe[1].tokens[3]]                       # request 1 would produce this as its 4th token
    stop = [probe[2].tokens[5]]
    reqs = [GenerateRequest(p, 10 if i != 4 else 2, SamplingConfig(temperature=0.9, seed=50 + i),
                            stop_token_ids=stop if i == 2 else ())
            for i, p in enumerate(prompts)]
    slow = generate(StepByStep(), reqs, eos_token_ids=eos, max_batch=4)
    fast = built.generate(reqs, eos_token_ids=eos)
    assert [(o.tokens, o.finish_reason) for o in fast] == [(o.tokens, o.finish_reason) for o in slow]
    assert slow[1].finish_reason == "eos_token" and slow[2].finish_reason == "stop"
    assert slow[4].finish_reason == "length" and len(slow[4].tokens) == 2
    eng.cache.check()
    assert not eng.cache.slots.held


def test_trace_run_program(tmp_path, plain, tiny_models):
    """bin/trace_run as a program: whole prompts of a batch, then single tokens, a request
    that ends earlier, then a second batch on the slots of the first."""
    cfg, w = plain["B"]
    a, b, c = seeded_tokens(cfg["vocab_size"], [40, 9, 70], 91)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]},
                                {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": [a[31]], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": [a[32]], "want": [0]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": c, "want": [69]}], "end": ["c"]},
    ]
    for dtype in DTYPES:
        out = tmp_path / dtype
        env = dict(os.environ)
        proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model",
                               str(tiny_models["B"]), "--dtype", dtype, "--out", str(out),
                               "--max-tokens", "128"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                              capture_output=True, env=env, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
        ra, rb, rc = (plain_ref(cfg, w, s) for s in (a, b, c))
        V = cfg["vocab_size"]
        rd = lambda k: torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(-1, V))
        check(rd(0), Ref.stack([ra[0], ra[29], rb[7]]), dtype, "trace step 0")
        check(rd(1), Ref.stack([ra[30], rb[8]]), dtype, "trace step 1")
        assert not (out / "2.f32").exists()
        check(rd(3), ra[32:33], dtype, "trace step 3")
        check(rd(4), rc[69:70], dtype, "trace step 4")


def _engines_on_the_same_random_weights(cfg, seed, max_tokens):
    """A float32 and a bfloat16 engine on the same random bfloat16 weights, and those weights
    as float32 on the CPU for the plain implementation."""
    from lumenllm_b200 import Engine
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.model import expected_tensors
    from lumenllm_b200.weights import random_weights
    spec = config_from_dict(cfg).model_spec()
    weights = random_weights(expected_tensors(spec), seed, 0.02, 0.1, torch.bfloat16, device="cuda")
    wf = {k: v.float().cpu() for k, v in weights.items()}

    def make(dtype):
        return Engine(spec, weights, dtype=dtype, max_tokens=max_tokens)
    return make, wf


@pytest.mark.parametrize("shape", ["14b", "32b"])
def test_serving_kernels_at_real_layer_sizes(shape):
    """One layer of the 14B / 32B shapes (width 5120, 40 or 64 heads in groups of 5 or 8, q width
    unequal to the width, the full vocabulary) with random bfloat16 weights: the bfloat16 path
    (tcgen05 products and attention, streaming products, split-KV decode) and the true 32-bit
    path of the same weights, for a prompt, a continuation and decoded tokens, against each
    other and, for the shorter request, against the plain implementation."""
    from lumenllm_b200 import StepEntry
    from lumenllm_b200.ops import kernels as K
    dims = {"14b": dict(hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
            "32b": dict(hidden_size=5120, num_attention_heads=64, intermediate_size=25600)}[shape]
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1,
               num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1000000.0,
               rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False, **dims)
    toks = seeded_tokens(151936, [300, 70, 1], 5)
    make, wf = _engines_on_the_same_random_weights(cfg, 3, 2048)
    outs = {}
    for dtype in ("float32", "bfloat16"):
        eng = make(dtype)
        slots = [eng.alloc_slot() for _ in toks]
        a = eng.step([StepEntry(s, t[:max(1, len(t) - 40)], [max(1, len(t) - 40) - 1])
                      for s, t in zip(slots, toks)])
        b = eng.step([StepEntry(slots[0], toks[0][260:290], [0, 29]), StepEntry(slots[1], toks[1][30:31], [0])])
        c = [eng.step([StepEntry(slots[0], [toks[0][290 + k]], [0]), StepEntry(slots[1], [toks[1][31 + k]], [0])])
             for k in range(3)]
        outs[dtype] = torch.cat([a, b] + c).float().cpu()
        eng.check_kernels()
        del eng
        torch.cuda.empty_cache()
    ref, got = outs["float32"], outs["bfloat16"]
    check(got, ref, "bfloat16", f"{shape} layer, serving path against the 32-bit path")
    # rows of the 70-token request: its prompt's last place, the continuation, three tokens
    plain = plain_ref(cfg, wf, toks[1][:34])
    rows, places = [1, 5, 7, 9, 11], [29, 30, 31, 32, 33]
    for dtype in ("float32", "bfloat16"):
        check(outs[dtype][rows], plain[places], dtype, f"{shape} layer against the plain implementation")


def test_a_long_prompt_at_real_layer_sizes():
    """1,200 prompt tokens through one layer of the 14B shape: the prompt-sized products run on
    pairs of SMs (the QKV product with norm, rotation and cache write in its epilogue), the
    output and down projections add to the residual stream in their epilogue, attention has
    many tiles per kv head; then a second piece of the prompt and decoded tokens over the
    cache that this left. Against the plain implementation, in both precisions."""
    from lumenllm_b200 import StepEntry
    from lumenllm_b200.ops import kernels as K
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=1,
               hidden_size=5120, num_attention_heads=40, intermediate_size=17408,
               num_key_value_heads=8, head_dim=128, vocab_size=32000, rope_theta=1000000.0,
               rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False)
    assert K.gemm_tc_adds(1200, 5120)              # the shapes this test is about
    assert K.gemm_tc_qkv_takes(1200, (40 + 16) * 128, 5120, 40, 8, 128, 128)
    toks = seeded_tokens(32000, [1493], 6)[0]
    make, wf = _engines_on_the_same_random_weights(cfg, 4, 4096)
    plain = plain_ref(cfg, wf, toks)[[0, 599, 1199, 1200, 1489, 1490, 1491, 1492]]
    for dtype in ("float32", "bfloat16"):
        eng = make(dtype)
        s = eng.alloc_slot()
        a = eng.step([StepEntry(s, toks[:1200], [0, 599, 1199])])
        b = eng.step([StepEntry(s, toks[1200:1490], [0, 289])])
        c = [eng.step([StepEntry(s, [toks[1490 + k]], [0])]) for k in range(3)]
        got = torch.cat([a, b] + c).float().cpu()
        eng.check_kernels()
        del eng
        torch.cuda.empty_cache()
        check(got, plain, dtype, "long prompt at the 14B layer sizes")
