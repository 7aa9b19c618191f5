"""Configurations and batches drawn at random (from fixed seeds): sizes that no hand-written
case has, each compared with the plain implementation in both precisions. A seed draws the
head counts and groups, a head size in steps of 16, a width, a feed-forward width and a
vocabulary that are no powers of two, the norms' eps, the rotation base, a window or none and
where it starts, tied or untied head; then requests of unequal lengths that start together
(prompts of unequal lengths, some cut into two steps), go on token by token and end at
different times, twice over on the same slots."""
import random

import pytest
import torch

import plain_qwen3 as P
from conftest import seeded_tokens, tolerance

pytestmark = pytest.mark.gpu


def draw_config(rng):
    d = rng.choice([16, 32, 48, 64, 80, 128])
    nkv = rng.choice([1, 2, 3, 4])
    nq = nkv * rng.choice([1, 2, 3, 4, 8])
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3",
               hidden_size=4 * rng.randint(12, 80), num_hidden_layers=rng.randint(1, 3),
               num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
               intermediate_size=4 * rng.randint(10, 120), vocab_size=rng.randint(130, 1500),
               rope_theta=rng.choice([10000.0, 50000.0, 1000000.0]),
               rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]), max_position_embeddings=2048,
               tie_word_embeddings=rng.random() < 0.3)
    if rng.random() < 0.5:
        cfg.update(use_sliding_window=True, sliding_window=rng.randint(5, 150),
                   max_window_layers=rng.randint(0, cfg["num_hidden_layers"]))
    return cfg


@pytest.mark.parametrize("seed", range(16))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_drawn_configuration_and_batch(seed, dtype, tmp_path):
    from lumenllm_b200 import Engine, StepEntry
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.weights import write_random_model
    rng = random.Random(1000 + seed)
    cfg = draw_config(rng)
    folder = write_random_model(config_from_dict(cfg), tmp_path / "m", seed=seed, std=0.05, norm_jitter=0.1)
    cfg_read, w = P.load_model(folder)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=4096)
    n_req = rng.randint(2, 5)
    lens = [rng.choice([1, 2, rng.randint(3, 70), rng.randint(60, 260)]) for _ in range(n_req)]
    seqs = seeded_tokens(cfg["vocab_size"], lens, 2000 + seed)
    refs = [P.forward_logits(cfg_read, w, q) for q in seqs]
    for round_ in range(2):
        slots = [eng.alloc_slot() for _ in seqs]
        prompt = [rng.randint(1, len(q)) for q in seqs]
        got = [[] for _ in seqs]
        # prompts together; a long one may come in two steps while the short ones wait
        first = [min(p, rng.choice([p, max(1, p // 2)])) for p in prompt]
        lg = eng.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, first)]).cpu()
        o = 0
        for i, c in enumerate(first):
            got[i].append(lg[o:o + c]); o += c
        rest = [i for i in range(n_req) if first[i] < prompt[i]]
        if rest:
            lg = eng.step([StepEntry(slots[i], seqs[i][first[i]:prompt[i]], list(range(prompt[i] - first[i])))
                           for i in rest]).cpu()
            o = 0
            for i in rest:
                c = prompt[i] - first[i]
                got[i].append(lg[o:o + c]); o += c
        pos = list(prompt)
        live = list(range(n_req))
        while True:
            for i in [i for i in live if pos[i] >= len(seqs[i])]:
                eng.free_slot(slots[i])
            live = [i for i in live if pos[i] < len(seqs[i])]
            if not live:
                break
            lg = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
            for k, i in enumerate(live):
                got[i].append(lg[k:k + 1]); pos[i] += 1
        for i in range(n_req):
            g = torch.cat(got[i])
            err = float((g - refs[i]).abs().max())
            assert err <= tolerance(dtype, refs[i]), (seed, round_, i, cfg, lens, err)
    eng.cache.check()
    assert not eng.cache.slots.held


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,nq,nkv,hidden", [(96, 3, 1, 72), (112, 7, 7, 100), (160, 6, 2, 88), (192, 5, 5, 120),
                                            (256, 2, 1, 136), (240, 9, 3, 84)])
def test_head_sizes_up_to_256_and_odd_head_counts(d, nq, nkv, hidden, dtype, tmp_path):
    """Head sizes that the tensor-core attention kernels do not take (every multiple of 16 up to
    256 is allowed; 192 and 256 keep the swizzled cache layout, the others the plain one), with
    3, 5, 7 and 9 heads: the general kernels, whole prompts, a continuation and single tokens in
    a batch of two, through Engine.step and through the captured steps."""
    from lumenllm_b200 import Engine, StepEntry
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.sampling import SamplingConfig
    from lumenllm_b200.weights import write_random_model
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=hidden,
               num_hidden_layers=2, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
               intermediate_size=4 * (hidden // 3), vocab_size=257 + d, rope_theta=20000.0,
               rms_norm_eps=2e-6, max_position_embeddings=512, tie_word_embeddings=(d % 32 == 0))
    folder = write_random_model(config_from_dict(cfg), tmp_path / "m", seed=d, std=0.05, norm_jitter=0.1)
    cfg_read, w = P.load_model(folder)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    seqs = seeded_tokens(cfg["vocab_size"], [150, 70], 40 + d)
    refs = [P.forward_logits(cfg_read, w, q) for q in seqs]
    slots = [eng.alloc_slot() for _ in seqs]
    cuts = [100, 3]
    lg = eng.step([StepEntry(s, q[:c], list(range(c))) for s, q, c in zip(slots, seqs, cuts)]).cpu()
    got = [[lg[:100]], [lg[100:]]]
    lg = eng.step([StepEntry(slots[0], seqs[0][100:140], list(range(40))),
                   StepEntry(slots[1], seqs[1][3:60], list(range(57)))]).cpu()
    got[0].append(lg[:40]); got[1].append(lg[40:])
    for t in range(10):
        if t < 5:
            lg = eng.step([StepEntry(slots[0], [seqs[0][140 + t]], [0]), StepEntry(slots[1], [seqs[1][60 + t]], [0])]).cpu()
        else:                       # the same through the captured step
            eng.run_device([(slots[0], [seqs[0][140 + t]]), (slots[1], [seqs[1][60 + t]])], [SamplingConfig()] * 2, [0.0] * 2)
            lg = eng.graphs.last.logits[:2].float().cpu()
        got[0].append(lg[0:1]); got[1].append(lg[1:2])
    for i in range(2):
        g = torch.cat(got[i])
        err = float((g - refs[i]).abs().max())
        assert err <= tolerance(dtype, refs[i]), (d, nq, nkv, i, err)
    for s in slots:
        eng.free_slot(s)
    eng.cache.check()
