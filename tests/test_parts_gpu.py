"""Each part of a layer alone against its plain formula, and the generality of the
composition: a layer named twice in the schedule, a layer that reads another layer's cache,
and toy parts (a mixer with per-sequence state of its own, a feed-forward with routing, a
position encoding with other frequencies and positions, another norm and another arrangement
of a block) that are registered here, in the test, and built and stepped without a change to
the library."""
from dataclasses import replace

import pytest
import torch

import plain_qwen3 as P
from conftest import TINY, seeded_tokens, tolerance

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16


def runtime(dtype):
    from lumenllm_b200.parts import Runtime
    return Runtime(torch.device("cuda", 0), dtype)


def make_ctx(rt, needs, seqs, starts=None, state_shapes=None, cache=None):
    """A cache and a step context for whole sequences (or continuations from `starts`)."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.engine.context import StepEntry, build_context
    if cache is None:
        cache = KVCache(needs, 4096, 8, 4096, dtype=rt.dtype, device=rt.device,
                        state_shapes=state_shapes)
        slots = [cache.alloc_slot() for _ in seqs]
    else:
        slots = sorted(cache.slots.held)
    ctx, _ = build_context(cache, rt, [StepEntry(s, q, list(range(len(q)))) for s, q in zip(slots, seqs)])
    return cache, slots, ctx


def commit(cache, slots, seqs):
    for s, q in zip(slots, seqs):
        cache.commit(s, len(q))


def spec_of(name):
    from lumenllm_b200.config import config_from_dict
    return config_from_dict(TINY[name]).model_spec()


def gpu_weights(folder, dtype=None):
    w = P.read_safetensors(folder / "model.safetensors")
    return {k: v.cuda() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_norm_part(dtype, tiny_models):
    from lumenllm_b200.parts import build_part
    spec = spec_of("B")
    w = gpu_weights(tiny_models["B"])
    part = build_part("norm", spec.layers[1].norms["ffn"], w, runtime(dtype))
    h = torch.randn(9, 96, generator=torch.Generator().manual_seed(0))
    ref = P.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"].float().cpu(), 1e-5)
    y = part.forward(h.cuda(), None, dtype).cpu().float()
    assert float((y - ref).abs().max()) < (1e-5 if dtype == F32 else 3e-2)
    off = replace(spec.layers[1].norms["ffn"], params=dict(spec.layers[1].norms["ffn"].params,
                                                           weight_offset=1.0))
    y1 = build_part("norm", off, w, runtime(F32)).forward(h.cuda(), None, F32).cpu()
    ref1 = P.rms_norm(h, 1 + w["model.layers.1.post_attention_layernorm.weight"].float().cpu(), 1e-5)
    assert float((y1 - ref1).abs().max()) < 1e-5


def test_position_part_table():
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import build_part
    p = build_part("position", PartSpec("rotary", {"head_dim": 48, "theta": 50000.0, "rotary_dim": 32}),
                   {}, runtime(F32))
    assert torch.equal(p.inv_freq.cpu(), P.rope_inv_freq(48, 50000.0, 32))
    assert build_part("position", PartSpec("none", {}), {}, runtime(F32)).rotary_dim == 0


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 2), ("C", 1)])
def test_attention_part(name, layer, dtype, tiny_models):
    """The mixer alone on two whole sequences, then continued by single tokens."""
    from lumenllm_b200.engine.context import EntryView
    from lumenllm_b200.parts import build_part
    cfg = TINY[name]
    spec = spec_of(name)
    rt = runtime(dtype)
    w = gpu_weights(tiny_models[name])
    mixer = build_part("mixer", spec.layers[layer].mixer, w, rt)
    wf = {k: v.float().cpu() for k, v in w.items()}
    g = torch.Generator().manual_seed(1)
    lens = [50, 7]
    ys = [torch.randn(n + 3, cfg["hidden_size"], generator=g).to(dtype).float() for n in lens]
    refs = [P.attention_block(y, wf, f"model.layers.{layer}.", cfg, torch.arange(y.shape[0]),
                              P.layer_window(cfg, layer)) for y in ys]
    cache, slots, ctx = make_ctx(rt, {0: mixer.cache_need()}, [[0] * n for n in lens])
    y = torch.cat([a[:n] for a, n in zip(ys, lens)]).to(dtype).cuda()
    out = mixer.forward(y, ctx, EntryView(ctx, 0, 0, True))
    out = out.sum(0).cpu() if out.dim() == 3 else out.cpu()
    commit(cache, slots, [[0] * n for n in lens])
    ref = torch.cat([r[:n] for r, n in zip(refs, lens)])
    tol = 2e-5 if dtype == F32 else 3e-2
    assert float((out - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    for t in range(3):
        _, _, ctx = make_ctx(rt, None, [[0], [0]], cache=cache)
        y = torch.stack([a[n + t] for a, n in zip(ys, lens)]).to(dtype).cuda()
        out = mixer.forward(y, ctx, EntryView(ctx, 0, 0, True))
        out = out.sum(0).cpu() if out.dim() == 3 else out.cpu()
        commit(cache, slots, [[0], [0]])
        ref = torch.stack([r[n + t] for r, n in zip(refs, lens)])
        assert float((out - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_ffn_embedding_and_head_parts(dtype, tiny_models):
    from lumenllm_b200.parts import build_part
    spec = spec_of("C")
    rt = runtime(dtype)
    w = gpu_weights(tiny_models["C"])
    wf = {k: v.float().cpu() for k, v in w.items()}
    g = torch.Generator().manual_seed(2)
    y = torch.randn(11, 80, generator=g).to(dtype)
    ffn = build_part("ffn", spec.layers[3].ffn, w, rt)
    out = ffn.forward(y.cuda(), None)
    out = out.sum(0).cpu() if out.dim() == 3 else out.cpu()
    ref = P.mlp_block(y.float(), wf, "model.layers.3.")
    tol = 2e-5 if dtype == F32 else 3e-2
    assert float((out - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    emb = build_part("embedding", spec.embedding, w, rt)
    tok = torch.tensor([0, 310, 17], dtype=torch.int32)
    assert torch.equal(emb.forward(tok.cuda()).cpu(), wf["model.embed_tokens.weight"][tok.long()])
    head = build_part("head", spec.head, w, rt)
    lg = head.forward(y.cuda()).cpu()
    ref = y.float() @ wf["lm_head.weight"].T
    assert lg.shape == (11, 311)
    assert float((lg - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    tied = build_part("head", spec_of("A").head, gpu_weights(tiny_models["A"]), rt)
    assert tied.proj.weight.shape == (256, 64)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_schedule_names_a_layer_twice_and_shares_a_cache(dtype, tiny_models):
    """Order of layers as data: layer 0, layer 1, layer 0 again (own cache), then layer 1
    reading the cache that its first run wrote."""
    from lumenllm_b200 import Engine, StepEntry
    from lumenllm_b200.config import ScheduleEntry
    cfg = TINY["A"]
    spec = replace(spec_of("A"), schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                           ScheduleEntry(1, cache_from=1)))
    w = gpu_weights(tiny_models["A"])
    wf = {k: v.float().cpu() for k, v in w.items()}
    eng = Engine(spec, w, dtype="float32" if dtype == F32 else "bfloat16", max_tokens=1024)
    assert sorted(eng.cache.group_of) == [0, 1, 2]            # three caches for four runs

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        kept = {}
        for run, layer in enumerate([0, 1, 0, 1]):
            p = f"model.layers.{layer}."
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-6)
            T = len(tokens)
            q = P.rms_norm((y @ wf[p + "self_attn.q_proj.weight"].T).view(T, 4, 16),
                           wf[p + "self_attn.q_norm.weight"], 1e-6)
            q = P.apply_rope(q, pos, 10000.0)
            if run == 3:
                k, v = kept[1]
            else:
                k = P.rms_norm((y @ wf[p + "self_attn.k_proj.weight"].T).view(T, 2, 16),
                               wf[p + "self_attn.k_norm.weight"], 1e-6)
                k = P.apply_rope(k, pos, 10000.0)
                v = (y @ wf[p + "self_attn.v_proj.weight"].T).view(T, 2, 16)
                kept[run] = (k, v)
            a = P.causal_attention(q, k, v).reshape(T, 64) @ wf[p + "self_attn.o_proj.weight"].T
            r = h + a
            h = r + P.mlp_block(P.rms_norm(r, wf[p + "post_attention_layernorm.weight"], 1e-6), wf, p)
        return P.rms_norm(h, wf["model.norm.weight"], 1e-6) @ wf["model.embed_tokens.weight"].T

    seqs = seeded_tokens(256, [40, 9], 3)
    slots = [eng.alloc_slot() for _ in seqs]
    lg = eng.step([StepEntry(s, q[:-2], list(range(len(q) - 2))) for s, q in zip(slots, seqs)]).cpu()
    more = [eng.step([StepEntry(s, [q[-2 + t]], [0]) for s, q in zip(slots, seqs)]).cpu() for t in range(2)]
    refs = [plain(q) for q in seqs]
    got0 = torch.cat([lg[:38], more[0][0:1], more[1][0:1]])
    got1 = torch.cat([lg[38:], more[0][1:2], more[1][1:2]])
    name = "float32" if dtype == F32 else "bfloat16"
    for got, ref in ((got0, refs[0]), (got1, refs[1])):
        assert float((got - ref).abs().max()) < tolerance(name, ref)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_toy_mixer_with_state_of_its_own(dtype, tiny_models):
    """A mixer that keeps, per sequence, a decaying sum of its inputs (fixed size, no keys):
    registered here, put into layer 1 of a model whose other layers use attention, and
    stepped whole, token by token and in a batch."""
    from lumenllm_b200 import Engine, StepEntry
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import Linear, register_part

    @register_part("mixer", "toy_decaying_sum")
    class DecayingSum:
        @classmethod
        def tensors(cls, spec):
            H = spec.params["hidden_size"]
            return {f"{spec.prefix}.mix.weight": ((H, H), "matrix")}

        def __init__(self, spec, weights, runtime):
            self.decay = float(spec.params["decay"])
            self.H = spec.params["hidden_size"]
            self.mix = Linear(weights[f"{spec.prefix}.mix.weight"], runtime)
            self.runtime = runtime

        def cache_need(self):
            return None

        def state_shape(self):
            return (self.H,), torch.float32

        def forward(self, y, ctx, entry):
            state = entry.state()                       # [max_slots, H], zero for a new sequence
            out = torch.empty(y.shape, dtype=torch.float32, device=y.device)
            n = 0
            for b in range(ctx.n_real):
                s = state[ctx.slots[b]]
                for t in range(ctx.q_lens[b]):
                    s.mul_(self.decay).add_(y[n].float())
                    out[n] = s
                    n += 1
            return self.mix(out.to(self.runtime.dtype))

    base = spec_of("B")
    toy = PartSpec("toy_decaying_sum", {"hidden_size": 96, "decay": 0.75}, prefix="model.layers.1.toy")
    layers = list(base.layers)
    layers[1] = replace(layers[1], mixer=toy)
    spec = replace(base, layers=tuple(layers))
    w = gpu_weights(tiny_models["B"])
    w["model.layers.1.toy.mix.weight"] = (0.05 * torch.randn(96, 96, generator=torch.Generator().manual_seed(4))
                                          ).to(torch.bfloat16).cuda()
    wf = {k: v.float().cpu() for k, v in w.items()}
    name = "float32" if dtype == F32 else "bfloat16"
    eng = Engine(spec, w, dtype=name, max_tokens=2048)
    assert sorted(eng.cache.group_of) == [0, 2] and list(eng.cache.state.tensors) == [1]
    cfg = TINY["B"]

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        for i in range(3):
            if i != 1:
                h = P.decoder_layer(h, wf, i, cfg, pos)
                continue
            p = "model.layers.1."
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
            s = torch.zeros(96)
            rows = []
            for t in range(len(tokens)):
                s = s * 0.75 + y[t]
                rows.append(s)
            r = h + torch.stack(rows) @ wf[p + "toy.mix.weight"].T
            h = r + P.mlp_block(P.rms_norm(r, wf[p + "post_attention_layernorm.weight"], 1e-5), wf, p)
        return P.rms_norm(h, wf["model.norm.weight"], 1e-5) @ wf["lm_head.weight"].T

    seqs = seeded_tokens(384, [30, 4, 17], 5)
    refs = [plain(q) for q in seqs]
    for round_ in range(2):                               # the second round meets used slots
        slots = [eng.alloc_slot() for _ in seqs]
        cuts = [20, 1, 17]
        lg = eng.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cuts)]).cpu()
        got = [[lg[0:20]], [lg[20:21]], [lg[21:38]]]
        pos = list(cuts)
        live = [0, 1]
        eng.free_slot(slots[2])
        while live:
            lg = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
            for k, i in enumerate(live):
                got[i].append(lg[k:k + 1]); pos[i] += 1
            for i in [i for i in live if pos[i] >= len(seqs[i])]:
                eng.free_slot(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
        for g, r in zip(got, refs):
            assert float((torch.cat(g) - r).abs().max()) < tolerance(name, r), round_
    eng.cache.check()


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_toy_mixer_with_state_in_a_captured_step(dtype, tiny_models):
    """The same decaying sum, written so that a decode step can be captured: single tokens
    index the state by `seq_slot` on the device. Three sequences in the bucket of four: the
    padding sequence reads and writes the state store's spare row, never a live sequence's,
    and the run that precedes a capture touches no state at all (it would count a token
    twice). Replayed steps against the plain sum."""
    from lumenllm_b200 import Engine, StepEntry
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import Linear, register_part
    from lumenllm_b200.sampling import SamplingConfig

    @register_part("mixer", "toy_decaying_sum_on_device")
    class DecayingSumOnDevice:
        graph_safe = True

        @classmethod
        def tensors(cls, spec):
            H = spec.params["hidden_size"]
            return {f"{spec.prefix}.mix.weight": ((H, H), "matrix")}

        def __init__(self, spec, weights, runtime):
            self.decay = float(spec.params["decay"])
            self.H = spec.params["hidden_size"]
            self.mix = Linear(weights[f"{spec.prefix}.mix.weight"], runtime)
            self.runtime = runtime

        def cache_need(self):
            return None

        def state_shape(self):
            return (self.H,), torch.float32

        def forward(self, y, ctx, entry):
            state = entry.state()                       # [max_slots + 1, H]
            if ctx.is_decode:                           # one token each: device indices only
                rows = ctx.seq_slot.long()
                s = state.index_select(0, rows) * self.decay + y.float()
                state.index_copy_(0, rows, s)
                return self.mix(s.to(self.runtime.dtype))
            out = torch.empty(y.shape, dtype=torch.float32, device=y.device)
            n = 0
            for b in range(ctx.n_real):
                s = state[ctx.slots[b]]
                for t in range(ctx.q_lens[b]):
                    s.mul_(self.decay).add_(y[n].float())
                    out[n] = s
                    n += 1
            return self.mix(out.to(self.runtime.dtype))

    base = spec_of("B")
    toy = PartSpec("toy_decaying_sum_on_device", {"hidden_size": 96, "decay": 0.75}, prefix="model.layers.1.toy")
    layers = list(base.layers)
    layers[1] = replace(layers[1], mixer=toy)
    spec = replace(base, layers=tuple(layers))
    w = gpu_weights(tiny_models["B"])
    w["model.layers.1.toy.mix.weight"] = (0.05 * torch.randn(96, 96, generator=torch.Generator().manual_seed(4))
                                          ).to(torch.bfloat16).cuda()
    wf = {k: v.float().cpu() for k, v in w.items()}
    name = "float32" if dtype == F32 else "bfloat16"
    eng = Engine(spec, w, dtype=name, max_tokens=2048, max_slots=6)
    assert eng.model.graph_safe
    cfg = TINY["B"]

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        for i in range(3):
            if i != 1:
                h = P.decoder_layer(h, wf, i, cfg, pos)
                continue
            p = "model.layers.1."
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
            s = torch.zeros(96)
            rows = []
            for t in range(len(tokens)):
                s = s * 0.75 + y[t]
                rows.append(s)
            r = h + torch.stack(rows) @ wf[p + "toy.mix.weight"].T
            h = r + P.mlp_block(P.rms_norm(r, wf[p + "post_attention_layernorm.weight"], 1e-5), wf, p)
        return P.rms_norm(h, wf["model.norm.weight"], 1e-5) @ wf["lm_head.weight"].T

    seqs = seeded_tokens(384, [30, 9, 17], 5)
    refs = [plain(q) for q in seqs]
    hold = [eng.alloc_slot() for _ in range(3)]        # the live sequences get the LAST slots,
    slots = [eng.alloc_slot() for _ in seqs]           # next to the spare row
    cuts = [20, 2, 10]
    eng.step([StepEntry(s, q[:c], []) for s, q, c in zip(slots, seqs, cuts)])
    state = eng.cache.state.of(1)
    for t in range(7):
        n = len(seqs)
        eng.run_device([(s, [q[c + t]]) for s, q, c in zip(slots, seqs, cuts)], [SamplingConfig()] * n, [0.0] * n)
        cap = eng.graphs.last
        assert cap.ctx.B == 4
        got = cap.logits[:n].float().cpu()
        for k in range(n):
            ref = refs[k][cuts[k] + t:cuts[k] + t + 1]
            assert float((got[k:k + 1] - ref).abs().max()) < tolerance(name, ref), (t, k)
    for s in hold:                                     # sequences that never ran: state untouched
        assert float(state[s].abs().max()) == 0.0
    for s in hold + slots:
        eng.free_slot(s)
    eng.cache.check()


def _step_whole_tail_and_batch(eng, seqs, cuts):
    """Logits of every position of each sequence: prompts of cuts[i] tokens in one batch, the
    rest token by token, shorter sequences ending earlier; slots are freed as they end."""
    from lumenllm_b200 import StepEntry
    slots = [eng.alloc_slot() for _ in seqs]
    lg = eng.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cuts)]).cpu()
    got, at = [], 0
    for c in cuts:
        got.append([lg[at:at + c]])
        at += c
    pos = list(cuts)
    live = [i for i in range(len(seqs)) if pos[i] < len(seqs[i])]
    for i in range(len(seqs)):
        if i not in live:
            eng.free_slot(slots[i])
    while live:
        lg = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
        for k, i in enumerate(live):
            got[i].append(lg[k:k + 1])
            pos[i] += 1
        for i in [i for i in live if pos[i] >= len(seqs[i])]:
            eng.free_slot(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    return [torch.cat(g) for g in got]


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_toy_feed_forward_with_routing(dtype, tiny_models):
    """A feed-forward that sends every token to ONE of three small experts, chosen by a
    router in float32, weighted by the margin between the best and the second-best router
    logit (so that the output is continuous where the choice flips, and a rounding
    difference cannot turn into a jump): registered here, put into layer 0 of a model whose
    other layers keep their dense feed-forward, stepped whole, by tokens and in a batch."""
    from lumenllm_b200 import Engine
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import Linear, register_part
    H, I, E = 96, 40, 3

    @register_part("ffn", "toy_routed")
    class Routed:
        @classmethod
        def tensors(cls, spec):
            t = {f"{spec.prefix}.router.weight": ((E, H), "matrix")}
            for e in range(E):
                t[f"{spec.prefix}.experts.{e}.up.weight"] = ((I, H), "matrix")
                t[f"{spec.prefix}.experts.{e}.down.weight"] = ((H, I), "matrix")
            return t

        def __init__(self, spec, weights, runtime):
            self.runtime = runtime
            self.router = weights[f"{spec.prefix}.router.weight"].float()
            self.up = [Linear(weights[f"{spec.prefix}.experts.{e}.up.weight"], runtime) for e in range(E)]
            self.down = [Linear(weights[f"{spec.prefix}.experts.{e}.down.weight"], runtime) for e in range(E)]

        def forward(self, y, ctx):
            logits = y.float() @ self.router.T                       # router in float32
            top = logits.topk(2, dim=-1)
            margin = top.values[:, 0] - top.values[:, 1]
            out = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
            for e in range(E):                                       # only the chosen expert's rows
                rows = (top.indices[:, 0] == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                z = torch.relu(self.up[e](y[rows].contiguous())).to(self.runtime.dtype)
                out[rows] = self.down[e](z) * margin[rows, None]
            return out

    base = spec_of("B")
    toy = PartSpec("toy_routed", {}, prefix="model.layers.0.moe")
    layers = list(base.layers)
    layers[0] = replace(layers[0], ffn=toy)
    spec = replace(base, layers=tuple(layers))
    w = gpu_weights(tiny_models["B"])
    g = torch.Generator().manual_seed(8)
    # margins of about one: the toy multiplies by them, and must not multiply the rounding of
    # its bfloat16 inputs beyond what the dense layers around it do
    w["model.layers.0.moe.router.weight"] = (0.1 * torch.randn(E, H, generator=g)).to(BF16).cuda()
    for e in range(E):
        w[f"model.layers.0.moe.experts.{e}.up.weight"] = (0.1 * torch.randn(I, H, generator=g)).to(BF16).cuda()
        w[f"model.layers.0.moe.experts.{e}.down.weight"] = (0.1 * torch.randn(H, I, generator=g)).to(BF16).cuda()
    for k in [k for k in w if k.startswith("model.layers.0.mlp.")]:
        del w[k]                                # the loader's rule: nothing unexpected
    wf = {k: v.float().cpu() for k, v in w.items()}
    name = "float32" if dtype == F32 else "bfloat16"
    eng = Engine(spec, w, dtype=name, max_tokens=2048)
    cfg = TINY["B"]
    seen = set()

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        for i in range(3):
            if i != 0:
                h = P.decoder_layer(h, wf, i, cfg, pos)
                continue
            p = "model.layers.0."
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
            r = h + P.attention_block(y, wf, p, cfg, pos, P.layer_window(cfg, 0))
            y2 = P.rms_norm(r, wf[p + "post_attention_layernorm.weight"], 1e-5)
            logits = y2 @ wf[p + "moe.router.weight"].T
            out = torch.zeros_like(y2)
            for t in range(len(tokens)):
                order = logits[t].argsort(descending=True)
                e = int(order[0])
                seen.add(e)
                z = torch.relu(wf[p + f"moe.experts.{e}.up.weight"] @ y2[t])
                out[t] = (wf[p + f"moe.experts.{e}.down.weight"] @ z) * (logits[t, order[0]] - logits[t, order[1]])
            h = r + out
        return P.rms_norm(h, wf["model.norm.weight"], 1e-5) @ wf["lm_head.weight"].T

    seqs = seeded_tokens(384, [33, 5, 18], 6)
    refs = [plain(q) for q in seqs]
    assert seen == {0, 1, 2}, "the test's tokens must reach every expert"
    for round_ in range(2):
        got = _step_whole_tail_and_batch(eng, seqs, [25, 1, 18])
        for a, r in zip(got, refs):
            assert float((a - r).abs().max()) < tolerance(name, r), round_
    eng.cache.check()


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_toy_position_encoding(dtype, tiny_models):
    """A rotation with other frequencies AND other positions than the library's (every
    position counts 2.5 steps, base 777): a position part is whatever fills the step's
    (cos, sin) table. Registered here and used by layer 1 only; layers 0 and 2 keep theirs."""
    from lumenllm_b200 import Engine
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.parts import register_part
    STRETCH, BASE = 2.5, 777.0

    @register_part("position", "toy_stretched")
    class Stretched:
        @classmethod
        def tensors(cls, spec):
            return {}

        def __init__(self, spec, weights, runtime):
            self.rotary_dim = int(spec.params["head_dim"])
            i2 = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
            self.inv_freq = (1.0 / (torch.tensor(BASE) ** (i2 / self.rotary_dim))).to(runtime.device)

        def angles(self, ctx):
            a = (ctx.rope_pos.float() * STRETCH)[:, None] * self.inv_freq[None, :]
            return torch.stack([torch.cos(a), torch.sin(a)], dim=-1).contiguous()

    cfg = TINY["B"]
    base = spec_of("B")
    layers = list(base.layers)
    d = layers[1].mixer.params["head_dim"]
    layers[1] = replace(layers[1], mixer=replace(layers[1].mixer, params=dict(
        layers[1].mixer.params, position=PartSpec("toy_stretched", {"head_dim": d}))))
    spec = replace(base, layers=tuple(layers))
    w = gpu_weights(tiny_models["B"])
    wf = {k: v.float().cpu() for k, v in w.items()}
    name = "float32" if dtype == F32 else "bfloat16"
    eng = Engine(spec, w, dtype=name, max_tokens=2048)

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        for i in range(3):
            if i != 1:
                h = P.decoder_layer(h, wf, i, cfg, pos)
                continue
            p = "model.layers.1."
            toy_cfg = dict(cfg, rope_theta=BASE)
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"], 1e-5)
            r = h + P.attention_block(y, wf, p, toy_cfg, pos.float() * STRETCH, P.layer_window(cfg, 1))
            h = r + P.mlp_block(P.rms_norm(r, wf[p + "post_attention_layernorm.weight"], 1e-5), wf, p)
        return P.rms_norm(h, wf["model.norm.weight"], 1e-5) @ wf["lm_head.weight"].T

    seqs = seeded_tokens(384, [41, 3, 20], 7)
    refs = [plain(q) for q in seqs]
    stock = P.forward_logits(cfg, wf, seqs[0])
    assert float((stock - refs[0]).abs().max()) > 5 * tolerance(name, refs[0]), "the toy must matter"
    got = _step_whole_tail_and_batch(eng, seqs, [30, 2, 20])
    for a, r in zip(got, refs):
        assert float((a - r).abs().max()) < tolerance(name, r)
    eng.cache.check()


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_toy_block_arrangement_and_a_toy_norm(dtype, tiny_models):
    """Another arrangement of a layer's parts, registered here: the mixer and the feed-forward
    both read ONE norm of the stream and their updates are added side by side
    (h' = h + mixer(n(h)) + ffn(n(h))), with a norm of its own kind (a root-mean-square norm
    whose weight is 1 + w, built on the library's norm kernel through its weight_offset). The
    block hands both updates on as one stack of partial sums for the next norm to add. Layer 1
    of model B is arranged this way, layers 0 and 2 keep the library's; stepped whole, token
    by token (through the captured step) and in a batch."""
    from lumenllm_b200 import Engine
    from lumenllm_b200.config import PartSpec
    from lumenllm_b200.ops import kernels as K
    from lumenllm_b200.parts import build_part, part_tensors, register_part

    @register_part("norm", "toy_one_plus_weight")
    class OnePlusWeight:
        @classmethod
        def tensors(cls, spec):
            return {f"{spec.prefix}.weight": ((spec.params["size"],), "norm")}

        def __init__(self, spec, weights, runtime):
            self.eps = float(spec.params["eps"])
            self.weight = (weights[f"{spec.prefix}.weight"].to(device=runtime.device, dtype=torch.float32) + 1.0).contiguous()

        def forward(self, h, delta, out_dtype, rows=None, write_h=True):
            return K.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows=rows, write_h=write_h)

    @register_part("block", "toy_parallel")
    class Parallel:
        @classmethod
        def tensors(cls, layer_spec):
            t = {}
            t.update(part_tensors("norm", layer_spec.norms["both"]))
            t.update(part_tensors("mixer", layer_spec.mixer))
            t.update(part_tensors("ffn", layer_spec.ffn))
            return t

        def __init__(self, layer_spec, weights, runtime):
            self.runtime = runtime
            self.norm = build_part("norm", layer_spec.norms["both"], weights, runtime)
            self.mixer = build_part("mixer", layer_spec.mixer, weights, runtime)
            self.ffn = build_part("ffn", layer_spec.ffn, weights, runtime)

        def forward(self, h, pending, ctx, entry):
            y = self.norm.forward(h, pending, self.runtime.dtype)
            a = self.mixer.forward(y, ctx, entry)
            m = self.ffn.forward(y, ctx)
            stack = lambda u: u if u.dim() == 3 else u.unsqueeze(0)
            return h, torch.cat([stack(a), stack(m)], dim=0).contiguous()

    cfg = TINY["B"]
    base = spec_of("B")
    layers = list(base.layers)
    toy_norm = PartSpec("toy_one_plus_weight", {"size": 96, "eps": 1e-5}, prefix="model.layers.1.input_layernorm")
    layers[1] = replace(layers[1], block="toy_parallel", norms={"both": toy_norm})
    spec = replace(base, layers=tuple(layers))
    w = gpu_weights(tiny_models["B"])
    del w["model.layers.1.post_attention_layernorm.weight"]          # the arrangement has one norm
    wf = {k: v.float().cpu() for k, v in w.items()}
    name = "float32" if dtype == F32 else "bfloat16"
    eng = Engine(spec, w, dtype=name, max_tokens=2048)
    assert eng.model.graph_safe

    def plain(tokens):
        tokens = torch.tensor(tokens)
        pos = torch.arange(len(tokens))
        h = P.embed(tokens, wf["model.embed_tokens.weight"])
        for i in range(3):
            if i != 1:
                h = P.decoder_layer(h, wf, i, cfg, pos)
                continue
            p = "model.layers.1."
            y = P.rms_norm(h, wf[p + "input_layernorm.weight"] + 1.0, 1e-5)
            h = h + P.attention_block(y, wf, p, cfg, pos, 0) + P.mlp_block(y, wf, p)
        return P.rms_norm(h, wf["model.norm.weight"], 1e-5) @ wf["lm_head.weight"].T

    seqs = seeded_tokens(384, [40, 3, 21], 9)
    refs = [plain(q) for q in seqs]
    got = _step_whole_tail_and_batch(eng, seqs, [30, 1, 21])
    for g, r in zip(got, refs):
        assert float((g - r).abs().max()) < tolerance(name, r)
    # and single tokens through the captured step
    from lumenllm_b200 import StepEntry
    from lumenllm_b200.sampling import SamplingConfig
    slots = [eng.alloc_slot() for _ in range(2)]
    eng.step([StepEntry(s, q[:10], []) for s, q in zip(slots, (seqs[0], seqs[2]))])
    for t in range(10, 14):
        eng.run_device([(slots[0], [seqs[0][t]]), (slots[1], [seqs[2][t]])], [SamplingConfig()] * 2, [0.0] * 2)
        lg = eng.graphs.last.logits[:2].float().cpu()
        for k, r in enumerate((refs[0], refs[2])):
            assert float((lg[k] - r[t]).abs().max()) < tolerance(name, r), (t, k)
    for s in slots:
        eng.free_slot(s)
    eng.cache.check()
