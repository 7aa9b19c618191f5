"""Each kernel alone against a plain float32 reference of the same operation, at sizes other
than the tiny models': widths and vocabularies that are no power of two, head sizes in steps
of 16, odd numbers of heads and groups, lengths that cross page and chunk edges, and inputs
made so that a single far key, a window's edge or a page of the cache decides the result."""
import math

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

F32, BF16, I32 = torch.float32, torch.bfloat16, torch.int32


def dev(t):
    return t.cuda()


def gen(seed):
    return torch.Generator().manual_seed(seed)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embed(dtype):
    from lumenllm_b200.ops import kernels as K
    V, H = 311, 1000
    table = torch.randn(V, H, generator=gen(0)).to(dtype)
    tok = torch.tensor([0, 310, 5, 5, 17], dtype=I32)
    out = K.embed(dev(tok), dev(table)).cpu()
    assert torch.equal(out, table[tok.long()].float())


@pytest.mark.parametrize("out_dtype", [F32, BF16])
@pytest.mark.parametrize("N", [1, 13, 301])   # one row, few rows and many: kernels of their own
@pytest.mark.parametrize("H,S", [(1000, 0), (80, 1), (4096 + 48, 3), (8192 + 8, 2)])
def test_add_rmsnorm(out_dtype, H, S, N):
    from lumenllm_b200.ops import kernels as K
    eps = 1e-5
    g = gen(1)
    h = torch.randn(N, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    delta = torch.randn(S, N, H, generator=g) if S else None
    x = h.clone()
    for s in range(S):
        x = x + delta[s]
    ref = P.rms_norm(x, w, eps)
    hd = dev(h.clone())
    y = K.add_rmsnorm(hd, dev(delta) if S else None, dev(w), eps, out_dtype).cpu().float()
    tol = 1e-5 if out_dtype == F32 else 2 ** -8
    assert float(((y - ref).abs() / (1 + ref.abs())).max()) < tol
    assert torch.allclose(hd.cpu(), x, atol=1e-6)             # the stream took the update
    # gathered rows, stream untouched
    rows = torch.tensor([12, 0, 7], dtype=I32) % N
    hd2 = dev(h.clone())
    y2 = K.add_rmsnorm(hd2, dev(delta) if S else None, dev(w), eps, out_dtype, rows=dev(rows),
                       write_h=False).cpu().float()
    assert float(((y2 - ref[rows.long()]).abs() / (1 + ref[rows.long()].abs())).max()) < tol
    assert torch.equal(hd2.cpu(), h)
    # one gathered row (the last row of a prompt before the head)
    y3 = K.add_rmsnorm(hd2, dev(delta) if S else None, dev(w), eps, out_dtype,
                       rows=dev(torch.tensor([N - 1], dtype=I32)), write_h=False).cpu().float()
    assert float(((y3 - ref[N - 1:]).abs() / (1 + ref[N - 1:].abs())).max()) < tol


@pytest.mark.parametrize("out_dtype", [F32, BF16])
def test_silu_mul(out_dtype):
    from lumenllm_b200.ops import kernels as K
    N, I = 7, 176
    gu = torch.randn(N, 2 * I, generator=gen(2)) * 3
    ref = P.swiglu(gu[:, :I], gu[:, I:])
    z = K.silu_mul(dev(gu), out_dtype).cpu().float()
    tol = 1e-6 if out_dtype == F32 else 2 ** -8
    assert float(((z - ref).abs() / (1 + ref.abs())).max()) < tol
    z2 = K.silu_mul(dev(torch.stack([0.5 * gu, 0.5 * gu])), out_dtype).cpu().float()
    assert torch.equal(z, z2)            # halves add up exactly
    odd = torch.randn(3, 2 * 7, generator=gen(22))           # a width that is no multiple of 4
    assert torch.allclose(K.silu_mul(dev(odd), F32).cpu(), P.swiglu(odd[:, :7], odd[:, 7:]), atol=1e-6)


def to_sw128(x):
    """[..., 64, d] tiles in key-major order -> the same tiles in the swizzled layout:
    [d/64][key][64] with the 16-byte chunk c of row `key` at chunk c ^ (key & 7)."""
    *lead, R, d = x.shape
    x = x.reshape(*lead, R, d // 64, 8, 8)
    r = torch.arange(R)
    phys = (torch.arange(8)[None, :] ^ (r[:, None] & 7))                 # [R, 8]
    idx = phys[:, None, :, None].expand(R, d // 64, 8, 8)
    idx = idx.expand(*lead, R, d // 64, 8, 8) if lead else idx
    out = torch.empty_like(x).scatter_(-2, idx.contiguous(), x)
    nd = out.dim()
    out = out.permute(*range(nd - 4), nd - 3, nd - 4, nd - 2, nd - 1)     # [..., cb, R, 8, 8]
    return out.reshape(*lead, R, d)                                       # same bytes, new order


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nq,nkv,d,rot", [(6, 3, 48, 48), (5, 5, 16, 8), (8, 2, 128, 128), (3, 1, 80, 80),
                                          (7, 3, 128, 128), (4, 4, 128, 128)])
@pytest.mark.parametrize("lens", [[70, 3], [250, 75]])   # few tokens and many: kernels of their own
def test_qk_norm_rope_store(dtype, nq, nkv, d, rot, lens):
    from lumenllm_b200.ops import kernels as K
    g = gen(3)
    starts = [60, 0]                       # two sequences; the first starts at position 60
    N = sum(lens)
    qkv = torch.randn(N, (nq + 2 * nkv) * d, generator=g)
    qw = 1 + 0.1 * torch.randn(d, generator=g)
    kw = 1 + 0.1 * torch.randn(d, generator=g)
    theta, eps = 50000.0, 1e-6
    inv = P.rope_inv_freq(d, theta, rot)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(I32)
    seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).to(I32)
    n_pages = 12
    table = torch.tensor([[9, 4, 7, 1, 10], [2, 6, 0, 0, 0]], dtype=I32)
    kc = torch.zeros(n_pages, nkv, 64, d, dtype=dtype)
    vc = torch.zeros_like(kc)
    kcd, vcd = dev(kc), dev(vc)
    cs = K.rope_table(dev(pos), dev(inv))
    assert torch.allclose(cs.cpu()[..., 0], torch.cos(pos.float()[:, None] * inv[None, :]), atol=2e-6)
    # the projection may arrive as partial sums: split it in three unequal parts
    parts = torch.stack([0.5 * qkv, 0.25 * qkv, 0.25 * qkv])
    q = K.qk_norm_rope_store(dev(parts), dev(qw), dev(kw), eps, cs, rot, dev(pos),
                             dev(seq), dev(table), kcd, vcd, nq, nkv, d, dtype).cpu().float()
    x = qkv.view(N, nq + 2 * nkv, d)
    qr = P.apply_rope(P.rms_norm(x[:, :nq], qw, eps), pos, theta, rot)
    kr = P.apply_rope(P.rms_norm(x[:, nq:nq + nkv], kw, eps), pos, theta, rot)
    vr = x[:, nq + nkv:]
    tol = 2e-6 if dtype == F32 else 2 ** -8
    rel = lambda a, b: float(((a - b).abs() / (1 + b.abs())).max())
    assert rel(q, qr) < tol
    kg, vg = kcd.cpu().float(), vcd.cpu().float()
    for n in range(N):
        pg = int(table[seq[n], pos[n] // 64])
        assert rel(kg[pg, :, pos[n] % 64], kr[n]) < tol
        assert rel(vg[pg, :, pos[n] % 64], vr[n]) < tol
    # nothing else was written: untouched pages stay zero
    used = {int(table[seq[n], pos[n] // 64]) for n in range(N)}
    for pg in range(n_pages):
        if pg not in used:
            assert float(kg[pg].abs().max()) == 0.0
    # without norm weights and without rotation the values pass through
    q2 = K.qk_norm_rope_store(dev(qkv), None, None, eps, None, 0, dev(pos), dev(seq),
                              dev(table), kcd, vcd, nq, nkv, d, dtype).cpu().float()
    assert rel(q2, x[:, :nq]) < tol


def _attn_case(lens, starts, nq, nkv, d, dtype, window, seed, n_pages=40):
    """Builds paged caches holding `starts[b] + lens[b]` positions for each sequence and
    queries for the last lens[b] positions; returns kernel inputs and the plain result."""
    g = gen(seed)
    B = len(lens)
    totals = [s + n for s, n in zip(starts, lens)]
    width = max((t + 63) // 64 for t in totals)
    table = torch.zeros(B, width, dtype=I32)
    free = list(range(n_pages - 1, 0, -1))
    ks, vs = [], []
    kc = torch.zeros(n_pages, nkv, 64, d)
    vc = torch.zeros_like(kc)
    for b, t in enumerate(totals):
        k = torch.randn(t, nkv, d, generator=g)
        v = torch.randn(t, nkv, d, generator=g)
        ks.append(k); vs.append(v)
        for p in range((t + 63) // 64):
            pg = free.pop(3 if len(free) > 3 else 0)     # not in order
            table[b, p] = pg
            n = min(64, t - 64 * p)
            kc[pg, :, :n] = k[64 * p:64 * p + n].transpose(0, 1)
            vc[pg, :, :n] = v[64 * p:64 * p + n].transpose(0, 1)
    qs = [torch.randn(n, nq, d, generator=g) for n in lens]
    return table, kc, vc, ks, vs, qs


def _attn_ref(qs, ks, vs, lens, starts, window, dtype):
    outs = []
    for q, k, v, n, s in zip(qs, ks, vs, lens, starts):
        k, v, q = (x.to(dtype).float() for x in (k, v, q))
        T = s + n
        qfull = torch.zeros(T, q.shape[1], q.shape[2])
        qfull[s:] = q
        outs.append(P.causal_attention(qfull, k, v, window=window)[s:])
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("nq,nkv,d,window", [(6, 3, 48, 0), (4, 4, 16, 0), (8, 2, 128, 0), (5, 1, 112, 0),
                                            (2, 1, 256, 0), (6, 2, 32, 24), (4, 2, 64, 130)])
def test_attention_generic(dtype, nq, nkv, d, window):
    from lumenllm_b200.ops import kernels as K
    lens, starts = [70, 1, 1, 130], [0, 299, 63, 5]
    table, kc, vc, ks, vs, qs = _attn_case(lens, starts, nq, nkv, d, dtype, window, 5)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(I32)
    seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).to(I32)
    out = K.attn_generic(dev(torch.cat(qs).to(dtype)), dev(kc.to(dtype)), dev(vc.to(dtype)), dev(table),
                         dev(seq), dev(pos), window, d ** -0.5).cpu().float()
    ref = _attn_ref(qs, ks, vs, lens, starts, window, dtype)
    tol = 1e-5 if dtype == F32 else 2 ** -7
    assert float((out - ref).abs().max()) < tol


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_one_far_key_and_the_windows_edge(dtype):
    """One key among 700 is made to dominate: the output must be its value. With a window,
    a dominating key one place outside the window must be invisible, one place inside must
    win."""
    from lumenllm_b200.ops import kernels as K
    nq, nkv, d, T = 2, 1, 32, 700
    for window, far, expect_far in ((0, 3, True), (100, T - 100, True), (100, T - 101, False)):
        g = gen(7)
        k = 0.1 * torch.randn(T, nkv, d, generator=g)
        v = torch.randn(T, nkv, d, generator=g)
        q = 0.1 * torch.randn(1, nq, d, generator=g)
        q[0, :, 0] = 12.0
        k[far, 0, 0] = 12.0                                  # score 144 / sqrt(32) = 25 above the rest
        pages = list(range(1, 12))
        table = torch.tensor([pages], dtype=I32)
        kc = torch.zeros(13, nkv, 64, d); vc = torch.zeros_like(kc)
        for p in range(11):
            n = min(64, T - 64 * p)
            kc[pages[p], :, :n] = k[64 * p:64 * p + n].transpose(0, 1)
            vc[pages[p], :, :n] = v[64 * p:64 * p + n].transpose(0, 1)
        out = K.attn_generic(dev(q.to(dtype)), dev(kc.to(dtype)), dev(vc.to(dtype)), dev(table),
                             dev(torch.zeros(1, dtype=I32)), dev(torch.tensor([T - 1], dtype=I32)),
                             window, d ** -0.5).cpu().float()
        target = v[far, 0].to(dtype).float()
        close = float((out[0, 0] - target).abs().max()) < 2e-2
        assert close == expect_far, (window, far)
        qf = torch.zeros(T, nq, d); qf[-1] = q[0].to(dtype).float()
        ref = P.causal_attention(qf, k.to(dtype).float(), v.to(dtype).float(), window=window)[-1:]
        assert float((out - ref).abs().max()) < (1e-5 if dtype == F32 else 2 ** -7)


def test_swizzled_writer_and_reader_agree():
    """The cache writer in the swizzled layout, read back by the general kernel and compared
    with the same data in the plain layout."""
    from lumenllm_b200.ops import kernels as K
    nq, nkv, d = 4, 2, 128
    g = gen(11)
    N = 150
    qkv = torch.randn(N, (nq + 2 * nkv) * d, generator=g)
    pos = torch.arange(N, dtype=I32)
    seq = torch.zeros(N, dtype=I32)
    table = torch.tensor([[5, 2, 7]], dtype=I32)
    outs, caches = [], []
    for layout in (K.LAYOUT_LINEAR, K.LAYOUT_SW128):
        kc = torch.zeros(9, nkv, 64, d, dtype=BF16).cuda()
        vc = torch.zeros_like(kc)
        q = K.qk_norm_rope_store(dev(qkv), None, None, 0.0, None, 0, dev(pos), dev(seq),
                                 dev(table), kc, vc, nq, nkv, d, BF16, layout=layout)
        outs.append(K.attn_generic(q, kc, vc, dev(table), dev(seq), dev(pos), 0, d ** -0.5,
                                   layout=layout).cpu())
        caches.append((kc.cpu(), vc.cpu()))
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(to_sw128(caches[0][0]), caches[1][0])
    assert torch.equal(to_sw128(caches[0][1]), caches[1][1])


@pytest.mark.parametrize("nq,nkv,d,window", [(8, 2, 128, 0), (4, 2, 64, 0), (32, 8, 128, 0), (3, 1, 64, 0),
                                            (16, 1, 128, 0), (4, 4, 64, 0), (8, 2, 128, 100), (4, 2, 64, 130)])
def test_attention_decode_kernel(nq, nkv, d, window):
    """Split-KV decode attention: lengths 1, 64, 128, 129, 300 and 1000 keys in one batch."""
    from lumenllm_b200.ops import kernels as K
    starts = [0, 63, 127, 128, 299, 999]
    lens = [1] * len(starts)
    table, kc, vc, ks, vs, qs = _attn_case(lens, starts, nq, nkv, d, BF16, window, 12, n_pages=60)
    pos = torch.tensor(starts, dtype=I32)
    out = K.attn_decode(dev(torch.cat(qs).to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))),
                        dev(table), dev(pos), window, d ** -0.5).cpu().float()
    K.check_error_flags()
    ref = _attn_ref(qs, ks, vs, lens, starts, window, BF16)
    assert float((out - ref).abs().max()) < 2 ** -6
    # a wider page table (as a captured step has) changes nothing
    wide = torch.zeros(table.shape[0], 32, dtype=I32); wide[:, :table.shape[1]] = table
    out2 = K.attn_decode(dev(torch.cat(qs).to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))),
                         dev(wide), dev(pos), window, d ** -0.5).cpu().float()
    assert torch.equal(out, out2)


def _last_query_attention(q, k, v, window):
    """The plain attention of the newest token alone (no other query exists in a decode
    step): weights softmax(q . k_j / sqrt(d)) over the keys j it sees, in float64.
    q [nq, d]; k, v [T, nkv, d]. Same formulas as plain_qwen3.causal_attention
    (crates/aegisllm-cpu/src/attention.rs:127-236; attention_decode_common.cuh:112-115)."""
    T, nkv, d = k.shape
    nq = q.shape[0]
    lo = max(0, T - window) if window > 0 else 0
    out = torch.empty(nq, d, dtype=torch.float64)
    for h in range(nq):
        kh = h // (nq // nkv)
        s = (k[lo:, kh].double() @ q[h].double()) / math.sqrt(d)
        out[h] = torch.softmax(s, dim=0) @ v[lo:, kh].double()
    return out.float()


@pytest.mark.parametrize("starts,window", [([4199], 0), ([8999], 0), ([8999], 3000),
                                           ([16999, 8191, 8192, 63, 12345, 4200, 100, 9000], 0),
                                           ([16999, 8191, 8192, 63, 12345, 4200, 100, 9000], 5000)])
def test_attention_decode_of_long_sequences(starts, window):
    """Sequences longer than 32 segments of the split attention (beyond 8,192 keys a block
    walks more pages than a segment usually has), at the cap and one page past it, with and
    without a window, alone and in a batch of 8 unequal ones. In every sequence one early
    key, which only the first segment holds, is made to matter."""
    from lumenllm_b200.ops import kernels as K
    nq, nkv, d = 4, 2, 128
    B = len(starts)
    g = gen(17)
    n_pages = sum((s + 64) // 64 for s in starts) + 2
    kc = torch.zeros(n_pages, nkv, 64, d, dtype=BF16)
    vc = torch.zeros_like(kc)
    width = max((s + 64) // 64 for s in starts)
    table = torch.zeros(B, width, dtype=I32)
    order = torch.randperm(n_pages - 1, generator=g) + 1
    at = 0
    qs, refs = [], []
    for b, s in enumerate(starts):
        T = s + 1
        k = torch.randn(T, nkv, d, generator=g)
        v = torch.randn(T, nkv, d, generator=g)
        q = torch.randn(nq, d, generator=g)
        far = max(0, T - window) + 5 if window else 5            # inside the first page seen
        if far < T:
            q[0, :8] = 4.0
            k[far, 0, :8] = 4.0                               # score +128/sqrt(128) = 11 above the rest
        k, v, q = k.to(BF16), v.to(BF16), q.to(BF16)
        np_ = (T + 63) // 64
        pages = order[at:at + np_]
        at += np_
        table[b, :np_] = pages.to(I32)
        pad = np_ * 64 - T
        kp = torch.cat([k, torch.zeros(pad, nkv, d, dtype=BF16)]).view(np_, 64, nkv, d).transpose(1, 2)
        vp = torch.cat([v, torch.zeros(pad, nkv, d, dtype=BF16)]).view(np_, 64, nkv, d).transpose(1, 2)
        kc[pages] = kp
        vc[pages] = vp
        qs.append(q)
        refs.append(_last_query_attention(q.float(), k.float(), v.float(), window))
    out = K.attn_decode(dev(torch.stack(qs)), dev(to_sw128(kc)), dev(to_sw128(vc)), dev(table),
                        dev(torch.tensor(starts, dtype=I32)), window, d ** -0.5).cpu().float()
    K.check_error_flags()
    err = (out - torch.stack(refs)).abs().amax(dim=(1, 2))
    assert float(err.max()) < 2 ** -6, (err.tolist(), starts, window)
    # the general kernel walks the same cache in its own chunks
    out_g = K.attn_generic(dev(torch.stack(qs)), dev(to_sw128(kc)), dev(to_sw128(vc)), dev(table),
                           dev(torch.arange(B, dtype=I32)), dev(torch.tensor(starts, dtype=I32)), window,
                           d ** -0.5, layout=K.LAYOUT_SW128).cpu().float()
    assert float((out_g - torch.stack(refs)).abs().max()) < 2 ** -6


@pytest.mark.parametrize("nq,nkv,S,rot,normed,window", [(8, 2, 3, 128, True, 0), (4, 4, 1, 128, False, 0),
                                                         (16, 1, 4, 0, True, 0), (6, 2, 2, 128, True, 90),
                                                         (32, 8, 3, 128, True, 0)])
def test_decode_attention_that_makes_its_own_queries(nq, nkv, S, rot, normed, window):
    """The decode attention given the QKV projection's partial sums instead of finished
    queries: the same bits, in its output and in the cache, as the rotary kernel followed by the
    attention kernel. Positions at a page's first and last row, in the first page, far in (so
    that several segments are merged), sequences of one token; page 0 stays empty. And both
    against the plain formulas."""
    from lumenllm_b200.ops import kernels as K
    d, eps, theta = 128, 1e-5, 30000.0
    g = gen(71 + nq)
    starts = [0, 63, 64, 127, 700, 1, 330, 1999][: 8 if nq < 32 else 5]
    B = len(starts)
    nh = nq + 2 * nkv
    parts = torch.randn(S, B, nh * d, generator=g) * (1.0 / math.sqrt(S))
    qw = dev(1 + 0.1 * torch.randn(d, generator=g)) if normed else None
    kw = dev(1 + 0.1 * torch.randn(d, generator=g)) if normed else None
    n_pages = 1 + sum(s // 64 + 1 for s in starts)
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    width = max(s // 64 + 1 for s in starts)
    table = torch.zeros(B, width, dtype=I32)
    kc = torch.zeros(n_pages, nkv, 64, d, dtype=BF16)
    vc = torch.zeros_like(kc)
    o = 0
    hist = []
    for b, s in enumerate(starts):
        np_ = s // 64 + 1
        pages = perm[o:o + np_]
        o += np_
        table[b, :np_] = pages.to(I32)
        k = torch.randn(np_ * 64, nkv, d, generator=g).to(BF16)
        v = torch.randn(np_ * 64, nkv, d, generator=g).to(BF16)
        k[s:] = 0
        v[s:] = 0                                     # what lies behind a sequence's end is nobody's
        kc[pages] = k.view(np_, 64, nkv, d).transpose(1, 2)
        vc[pages] = v.view(np_, 64, nkv, d).transpose(1, 2)
        hist.append((k[:s].float(), v[:s].float()))
    pos = dev(torch.tensor(starts, dtype=I32))
    seq = dev(torch.arange(B, dtype=I32))
    cs = K.rope_table(pos, dev(P.rope_inv_freq(d, theta, d))) if rot else None
    kc1, vc1, kc2, vc2 = dev(to_sw128(kc)), dev(to_sw128(vc)), dev(to_sw128(kc)), dev(to_sw128(vc))
    tab = dev(table)
    q = K.qk_norm_rope_store(dev(parts), qw, kw, eps, cs, rot, pos, seq, tab, kc1, vc1, nq, nkv, d, BF16,
                             layout=K.LAYOUT_SW128)
    out1 = K.attn_decode(q, kc1, vc1, tab, pos, window, d ** -0.5)
    out2 = K.attn_decode_qkv(dev(parts), qw, kw, eps, cs, rot, kc2, vc2, tab, pos, window, d ** -0.5, nq, nkv)
    K.check_error_flags()
    assert torch.equal(out1, out2)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert float(kc2[0].float().abs().max()) == 0.0 and float(vc2[0].float().abs().max()) == 0.0
    # the plain formulas: sum of the parts, head norm, rotation, attention over history + the new token
    x = parts.sum(0).view(B, nh, d)
    for b, s in enumerate(starts):
        qh, kh, vh = x[b, :nq], x[b, nq:nq + nkv], x[b, nq + nkv:]
        if normed:
            qh = P.rms_norm(qh, qw.cpu(), eps)
            kh = P.rms_norm(kh, kw.cpu(), eps)
        if rot:
            qh = P.apply_rope(qh[None], torch.tensor([s]), theta)[0]
            kh = P.apply_rope(kh[None], torch.tensor([s]), theta)[0]
        kh, vh, qh = kh.to(BF16).float(), vh.to(BF16).float(), qh.to(BF16).float()
        k_all = torch.cat([hist[b][0], kh[None]])
        v_all = torch.cat([hist[b][1], vh[None]])
        ref = _last_query_attention(qh, k_all, v_all, window)
        assert float((out2[b].cpu().float() - ref).abs().max()) < 2 ** -6, (b, s)


@pytest.mark.parametrize("tensor_memory", [True, False])
@pytest.mark.parametrize("nq,nkv,d,window", [(8, 2, 128, 0), (4, 2, 64, 0), (6, 2, 64, 0), (5, 1, 128, 0),
                                            (16, 1, 64, 0), (2, 2, 128, 0), (8, 2, 128, 70), (4, 2, 64, 24)])
def test_attention_prefill_kernel(nq, nkv, d, window, tensor_memory):
    """Flash attention for prompts: whole prompts, continuations from a cached prefix, and
    single tokens, of unequal lengths in one batch."""
    from lumenllm_b200.ops import kernels as K
    lens, starts = [70, 1, 1, 130, 17, 200], [0, 299, 63, 5, 64, 0]
    table, kc, vc, ks, vs, qs = _attn_case(lens, starts, nq, nkv, d, BF16, window, 13, n_pages=60)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=I32)
    out = K.attn_prefill(dev(torch.cat(qs).to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))),
                         dev(table), dev(cu), dev(torch.tensor(starts, dtype=I32)), lens, window,
                         d ** -0.5, tensor_memory=tensor_memory).cpu().float()
    K.check_error_flags()
    ref = _attn_ref(qs, ks, vs, lens, starts, window, BF16)
    err = (out - ref).abs().max(dim=-1).values.max(dim=-1).values
    assert float(err.max()) < 2 ** -6, (int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("kernel", ["decode", "prefill", "prefill_mma"])
def test_fast_attention_one_far_key_and_the_windows_edge(kernel):
    from lumenllm_b200.ops import kernels as K
    nq, nkv, d, T = 4, 1, 128, 700
    for window, far, expect_far in ((0, 3, True), (100, T - 100, True), (100, T - 101, False)):
        g = gen(7)
        k = 0.1 * torch.randn(T, nkv, d, generator=g)
        v = torch.randn(T, nkv, d, generator=g)
        q = 0.1 * torch.randn(1, nq, d, generator=g)
        q[0, :, 0] = 12.0
        k[far, 0, 0] = 12.0
        pages = list(range(11, 0, -1))
        table = torch.tensor([pages], dtype=I32)
        kc = torch.zeros(13, nkv, 64, d); vc = torch.zeros_like(kc)
        for p in range(11):
            n = min(64, T - 64 * p)
            kc[pages[p], :, :n] = k[64 * p:64 * p + n].transpose(0, 1)
            vc[pages[p], :, :n] = v[64 * p:64 * p + n].transpose(0, 1)
        args = (dev(q.to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))), dev(table))
        if kernel == "decode":
            out = K.attn_decode(*args, dev(torch.tensor([T - 1], dtype=I32)), window, d ** -0.5)
        else:
            out = K.attn_prefill(*args, dev(torch.tensor([0, 1], dtype=I32)),
                                 dev(torch.tensor([T - 1], dtype=I32)), [1], window, d ** -0.5,
                                 tensor_memory=(kernel == "prefill"))
        out = out.cpu().float()
        K.check_error_flags()
        target = v[far, 0].to(BF16).float()
        close = float((out[0, 0] - target).abs().max()) < 2e-2
        assert close == expect_far, (window, far)
        qf = torch.zeros(T, nq, d); qf[-1] = q[0].to(BF16).float()
        ref = P.causal_attention(qf, k.to(BF16).float(), v.to(BF16).float(), window=window)[-1:]
        assert float((out - ref).abs().max()) < 2 ** -6


@pytest.mark.parametrize("wdtype", [F32, BF16])
@pytest.mark.parametrize("M,N,K_", [(1, 311, 80), (7, 64, 176), (65, 130, 48), (130, 17, 1000)])
def test_gemm_f32_is_true_float32(wdtype, M, N, K_):
    from lumenllm_b200.ops import kernels as K
    g = gen(8)
    a = torch.randn(M, K_, generator=g)
    w = torch.randn(N, K_, generator=g).to(wdtype)
    out = K.gemm_f32(dev(a), dev(w)).cpu()
    ref = (a.double() @ w.double().T)
    # float32 products summed in float32: error grows like sqrt(K) * 2^-24, far below TF32's 2^-11
    assert float(((out.double() - ref).abs() / (1 + ref.abs())).max()) < 2e-6 * math.sqrt(K_)
    # a row's result does not depend on the other rows of the batch
    one = K.gemm_f32(dev(a[M // 2:M // 2 + 1].contiguous()), dev(w)).cpu()
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("M,N,K_", [(128, 256, 64), (200, 300, 320), (2048, 1024, 4096), (1, 256, 64),
                                    (8, 4096, 4096), (19, 311, 80), (33, 1000, 1000), (64, 6144, 1024),
                                    (65, 130, 72), (130, 17, 1000), (16, 151936 // 4 + 8, 256)])
def test_gemm_tc_tensor_memory_product(M, N, K_):
    """The tcgen05 / TMA product in both orientations: sizes that end inside a tile in every
    dimension, a k that is no multiple of the 64-wide block, one row, and the split of k."""
    from lumenllm_b200.ops import kernels as K
    g = gen(16)
    x = torch.randn(M, K_, generator=g).to(BF16)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(BF16)
    part = K.gemm_tc(dev(x), K.tile_weight(dev(w))).cpu()
    K.check_error_flags()
    assert part.shape == (K.gemm_tc_splits(M, N, K_), M, N)
    ref = x.double() @ w.double().T
    assert float((part.sum(0).double() - ref).abs().max()) < 1e-4
    if M <= 16:        # the same row alone: same tile shape, same order of sums
        one = K.gemm_tc(dev(x[M // 2:M // 2 + 1].contiguous()), K.tile_weight(dev(w))).cpu()
        assert torch.equal(one[:, 0], part[:, M // 2])


@pytest.mark.parametrize("M,N,K_", [(2048, 2560, 320), (1990, 2700, 136), (4100, 1300, 64), (2304, 2052, 72)])
def test_gemm_tc_two_sm_product(M, N, K_):
    """Prompt-sized products run on pairs of SMs (one 256 x 256 tile a pair, both halves of both
    operands read from the two shared memories): sizes that end inside a tile in every
    dimension, and rows that do not change when more rows follow them."""
    from lumenllm_b200.ops import kernels as K
    g = gen(26)
    x = torch.randn(M, K_, generator=g).to(BF16)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(BF16)
    w[7] *= 30.0                      # a row and a column that stand out show a misplaced tile
    x[M - 3] *= 20.0
    out = K.gemm_tc(dev(x), K.tile_weight(dev(w))).cpu()
    K.check_error_flags()
    assert out.shape == (1, M, N)
    ref = x.double() @ w.double().T
    assert float((out[0].double() - ref).abs().max()) < 1e-4 * max(1.0, float(ref.abs().max()))
    more = torch.cat([x, torch.randn(300, K_, generator=g).to(BF16)])
    out2 = K.gemm_tc(dev(more), K.tile_weight(dev(w))).cpu()
    assert torch.equal(out2[0, :M], out[0])
    # added in place to a float32 matrix (the residual stream): one add an element, exactly
    # what adding the product afterwards gives
    if K.gemm_tc_adds(M, N):
        h = torch.randn(M, N, generator=g)
        hd = dev(h.clone())
        assert K.gemm_tc(dev(x), K.tile_weight(dev(w)), add_to=hd) is None
        K.check_error_flags()
        assert torch.equal(hd.cpu(), h + out[0])


@pytest.mark.parametrize("N,K_", [(1, 8), (130, 72), (256, 64), (700, 200), (4100, 1032)])
def test_tiled_form_of_a_weight(N, K_):
    """The form the products read weights in, against its definition: k block after k block,
    rows padded to a multiple of 256, the 16-byte pieces of row r at the places (piece ^ (r & 7));
    zeros in the padding; back to rows; the first rows of a weight on the same memory; and an
    embedding table read from it."""
    from lumenllm_b200.ops import kernels as K
    g = gen(31)
    w = torch.randn(N, K_, generator=g).to(BF16)
    t = K.tile_weight(dev(w))
    KB, NP = (K_ + 63) // 64, (N + 255) // 256 * 256
    assert (t.rows, t.cols, t.padded_rows) == (N, K_, NP) and t.data.numel() == KB * NP * 64
    padded = torch.zeros(NP, KB * 64, dtype=BF16)
    padded[:N, :K_] = w
    want = torch.empty(KB, NP, 8, 8, dtype=BF16)
    for r8 in range(8):
        rows = padded[r8::8].view(-1, KB, 8, 8)                       # [row group, k block, piece, 8]
        for piece in range(8):
            want[:, r8::8, piece ^ r8] = rows[:, :, piece].permute(1, 0, 2)
    assert torch.equal(t.data.cpu().view(KB, NP, 8, 8), want)
    assert torch.equal(t.row_major().cpu(), w)
    n = max(1, N // 3)
    assert torch.equal(t.first_rows(n).row_major().cpu(), w[:n])
    tokens = torch.tensor([0, N - 1, N // 2, N, -1], dtype=I32)
    got = K.embed(dev(tokens), t).cpu()
    assert torch.equal(got[:3], w[[0, N - 1, N // 2]].float()) and float(got[3:].abs().max()) == 0.0
    x = torch.randn(5, K_, generator=g).to(BF16)
    part = K.gemm_tc(dev(x), t.first_rows(n)).cpu()
    K.check_error_flags()
    assert float((part.sum(0).double() - x.double() @ w[:n].double().T).abs().max()) < 1e-3


@pytest.mark.parametrize("M,I,H", [(300, 176, 80), (2048, 1536, 256), (40, 176, 80), (3, 12288, 128),
                                   (2048, 1300, 80), (100, 176, 80), (200, 520, 96)])
def test_gemm_tc_with_silu_epilogue_on_interleaved_rows(M, I, H):
    from lumenllm_b200.ops import kernels as K
    g = gen(17)
    x = torch.randn(M, H, generator=g).to(BF16)
    wg = (torch.randn(I, H, generator=g) / math.sqrt(H)).to(BF16)
    wu = (torch.randn(I, H, generator=g) / math.sqrt(H)).to(BF16)
    w = torch.stack([wg, wu], dim=1).reshape(2 * I, H)
    z = K.gemm_tc(dev(x), K.tile_weight(dev(w)), silu_interleaved=True).cpu().float()
    K.check_error_flags()
    ref = P.swiglu(x.float() @ wg.float().T, x.float() @ wu.float().T)
    assert z.shape == (M, I)
    assert float(((z - ref).abs() / (1 + ref.abs())).max()) < 2 ** -7
    # the same through the float32 product and the activation kernel
    gu = K.gemm_tc(dev(x), K.tile_weight(dev(w)))
    z2 = K.silu_mul(gu, BF16, interleaved=True).cpu().float()
    assert float(((z2 - ref).abs() / (1 + ref.abs())).max()) < 2 ** -7


def test_argmax_ties_and_odd_vocab():
    from lumenllm_b200.ops import kernels as K
    V = 151936 + 7
    lg = torch.randn(5, V, generator=gen(9))
    lg[0, 100] = lg[0, 77777] = 50.0            # equal maxima: lowest index
    lg[1, V - 1] = 60.0
    lg[2, 0] = 60.0
    lg[3] = -1.0
    lg[4, 5] = float("nan"); lg[4, 9] = 70.0
    out = K.argmax(dev(lg)).cpu().tolist()
    assert out == [100, V - 1, 0, 0, 9]
    view = dev(torch.cat([lg, lg], dim=1))[:, :V]            # rows with a stride
    assert K.argmax(view).cpu().tolist() == out


def _sample_rows(lg, opts, ks):
    from lumenllm_b200.ops import kernels as K
    o = torch.tensor(opts, dtype=F32)
    k = torch.tensor(ks, dtype=I32)
    return K.sample(dev(lg), dev(o), dev(k)).cpu().tolist()


def _acceptable(row, temperature, top_k, top_p, min_p, u, tol=3e-5):
    """Tokens the plain sampler gives for u and for u moved by a rounding's worth."""
    return {P.sample(row, temperature, top_k, top_p, min_p, min(max(x, 0.0), 0.9999999))[0]
            for x in (u, u - tol, u + tol)}


@pytest.mark.parametrize("V", [1000, 50257 + 3])
def test_sampler_against_the_plain_one(V):
    g = gen(10)
    settings = [(0.8, 0, 1.0, 0.0), (1.0, 50, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05),
                (1.0, 40, 0.95, 0.02), (0.0, 0, 1.0, 0.0), (0.9, 1, 0.5, 0.0), (2.0, 5, 0.5, 0.3)]
    us = [0.0, 0.013, 0.37, 0.5, 0.77, 0.93, 0.999]
    lg = torch.randn(len(settings) * len(us), V, generator=g) * 3
    lg[:, 11] = lg[:, 500]                                   # equal logits inside the row
    opts, ks = [], []
    for (t, k, p, m) in settings:
        for u in us:
            opts.append([t, p, m, u]); ks.append(k)
    got = _sample_rows(lg, opts, ks)
    for r, (tok, o, k) in enumerate(zip(got, opts, ks)):
        ok = _acceptable(lg[r], o[0], k, o[1], o[2], o[3])
        assert tok in ok, (r, o, k, tok, ok)
    # the same rows in another order and alone give the same tokens
    perm = torch.randperm(lg.shape[0], generator=g)
    again = _sample_rows(lg[perm], [opts[i] for i in perm], [ks[i] for i in perm])
    assert again == [got[i] for i in perm]
    assert _sample_rows(lg[3:4], opts[3:4], ks[3:4]) == got[3:4]


def test_sampler_edges():
    V = 777
    lg = torch.full((6, V), -5.0)
    lg[0, 3] = lg[0, 700] = 9.0                              # two equal candidates: u picks by index order
    lg[1, :] = float("-inf"); lg[1, 42] = 0.0                 # a single finite logit
    lg[2, :] = float("nan")                                   # nothing finite
    lg[3, 5] = float("inf"); lg[3, 6] = 1.0                   # +inf is left out of sampling
    lg[4, 10] = 100.0                                         # everything else underflows
    lg[5, 1] = 2.0; lg[5, 2] = 2.0; lg[5, 3] = 2.0            # top_k cuts among equal logits
    opts = [[1.0, 1.0, 0.0, 0.75], [1.0, 1.0, 0.0, 0.5], [1.0, 1.0, 0.0, 0.5], [1.0, 1.0, 0.0, 0.0],
            [0.01, 1.0, 0.0, 0.99], [1.0, 1.0, 0.0, 0.99]]
    got = _sample_rows(lg, opts, [2, 0, 0, 0, 0, 2])
    assert got[0] == 700 and got[1] == 42 and got[2] == 0 and got[4] == 10
    assert got[3] == 6
    assert got[5] == 2                                        # of 1,2,3 the first two are kept
    lo = _sample_rows(lg[:1], [[1.0, 1.0, 0.0, 0.25]], [2])
    assert lo == [3]


def test_sampler_runs_of_equal_logits_and_a_large_vocabulary():
    """Rows the sampler's quick route must hand to the exact radix route (thousands of equal
    logits fall into one bin), and the full-size vocabulary, against the plain sampler."""
    g = gen(31)
    V = 151936
    flat = torch.full((4, 6000), 1.0)
    flat[1, 17] = 3.0
    flat[2, ::2] = 1.0000001                                  # two keys one ulp apart, 3,000 each
    flat[3, 100:200] = 2.5
    opts = [[1.0, 1.0, 0.0, 0.61], [0.7, 0.9, 0.0, 0.95], [1.0, 1.0, 0.0, 0.25], [1.0, 0.5, 0.0, 0.5]]
    ks = [0, 0, 4000, 150]
    got = _sample_rows(flat, opts, ks)
    for r, (tok, o, k) in enumerate(zip(got, opts, ks)):
        assert tok in _acceptable(flat[r], o[0], k, o[1], o[2], o[3]), (r, tok)
    big = torch.randn(6, V, generator=g) * 2.5
    big[:, 7] = big[:, 150000]
    opts = [[0.8, 1.0, 0.0, 0.3], [1.0, 0.9, 0.0, 0.77], [0.6, 0.95, 0.0, 0.999], [1.0, 1.0, 0.0, 0.5],
            [1.5, 0.8, 0.0, 0.05], [1.0, 1.0, 0.02, 0.4]]
    ks = [0, 0, 50, 20, 1000, 0]
    got = _sample_rows(big, opts, ks)
    for r, (tok, o, k) in enumerate(zip(got, opts, ks)):
        assert tok in _acceptable(big[r], o[0], k, o[1], o[2], o[3]), (r, tok)
    assert _sample_rows(big[2:3], opts[2:3], ks[2:3]) == got[2:3]
    # the sampler spreads a row over 8, 4, 2 or 1 blocks by the size of the batch: same tokens
    for copies in (4, 7, 12):                                 # 24, 42 and 72 rows
        rep = _sample_rows(big.repeat(copies, 1), opts * copies, ks * copies)
        assert rep == got * copies, copies


@pytest.mark.parametrize("V,rows", [(777, 96), (5003, 64), (32000, 40)])
def test_sampler_with_drawn_settings(V, rows):
    """Rows, options and uniform numbers drawn from a fixed seed: spreads from flat to peaked,
    repeated values, some -inf entries, every combination of the filters."""
    import random
    rng = random.Random(V)
    g = gen(40 + V % 7)
    lg = torch.randn(rows, V, generator=g)
    opts, ks = [], []
    for r in range(rows):
        lg[r] *= rng.choice([0.3, 1.0, 3.0, 8.0])
        if rng.random() < 0.4:
            lg[r, torch.randint(0, V, (V // 10,), generator=g)] = float("-inf")
        if rng.random() < 0.4:
            src = torch.randint(0, V, (V // 20,), generator=g)
            lg[r, torch.randint(0, V, (V // 20,), generator=g)] = lg[r, src]      # repeated values
        t = rng.choice([0.3, 0.7, 1.0, 1.6])
        k = rng.choice([0, 0, 2, 7, 50, 300])
        p = rng.choice([1.0, 1.0, 0.99, 0.9, 0.5])
        m = rng.choice([0.0, 0.0, 0.0, 0.02, 0.2])
        opts.append([t, p, m, rng.random()])
        ks.append(k)
    got = _sample_rows(lg, opts, ks)
    for r, (tok, o, k) in enumerate(zip(got, opts, ks)):
        ok = _acceptable(lg[r], o[0], k, o[1], o[2], o[3])
        assert tok in ok, (r, o, k, tok, ok)


def test_products_of_drawn_shapes_through_the_router():
    """Shapes drawn from a fixed seed across every regime of the product's routing
    (weight-streaming tcgen05 orientation with k split, single-SM tiles with
    narrow widths or k split, two SMs a tile with staged stores, the library where a row is
    no multiple of 16 bytes): all against the double-precision product."""
    import random
    from lumenllm_b200.ops import gemm as G
    from lumenllm_b200.ops import kernels as K
    rng = random.Random(7)
    g = gen(51)
    shapes = []
    for lo, hi in [(1, 16), (17, 64), (65, 128), (129, 256), (257, 700), (701, 1400), (1401, 2600)]:
        for _ in range(4):
            M = rng.randint(lo, hi)
            N = rng.choice([rng.randint(8, 300), rng.randint(300, 3000), 4 * rng.randint(75, 1600)])
            Kd = rng.choice([8 * rng.randint(1, 40), 8 * rng.randint(40, 400), 4 * rng.randint(3, 200) + 2])
            shapes.append((M, N, Kd))
    shapes += [(2304, 5120, 264), (1536, 12288, 136)]          # two SMs a tile, ragged k
    for M, N, Kd in shapes:
        x = torch.randn(M, Kd, generator=g).to(BF16)
        w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(BF16)
        wd = dev(w)
        out = G.gemm_bf16(dev(x), K.tile_weight(wd) if K.can_tile(wd) else wd).cpu()   # as parts.Linear holds it
        ref = x.double() @ w.double().T
        err = float((out.double() - ref).abs().max())
        assert out.shape == (M, N) and err < 2e-4 * max(1.0, float(ref.abs().max())), (M, N, Kd, err)
    from lumenllm_b200.ops import kernels as K
    K.check_error_flags()


@pytest.mark.parametrize("seed", range(6))
def test_fast_attention_kernels_with_drawn_batches(seed):
    """Batches drawn from a fixed seed for the three fast attention kernels: group sizes 1 to
    8, head size 64 or 128, a window or none, decode batches of 1 to 40 sequences (which changes
    how a sequence is cut into segments) with up to 3,000 cached keys, prompts of 1 to 400
    tokens on cached prefixes of any length."""
    import random
    from lumenllm_b200.ops import kernels as K
    rng = random.Random(300 + seed)
    d = rng.choice([64, 128])
    nkv = rng.choice([1, 2, 4])
    nq = nkv * rng.choice([1, 2, 4, 5, 8])
    window = rng.choice([0, 0, rng.randint(3, 700)])
    # decode
    B = rng.choice([1, 2, 3, 9, 17, 40])
    starts = [rng.choice([0, rng.randint(1, 200), rng.randint(200, 3000)]) for _ in range(B)]
    lens = [1] * B
    n_pages = sum((s + 64) // 64 for s in starts) + 8
    table, kc, vc, ks, vs, qs = _attn_case(lens, starts, nq, nkv, d, BF16, window, 70 + seed, n_pages=n_pages)
    out = K.attn_decode(dev(torch.cat(qs).to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))),
                        dev(table), dev(torch.tensor(starts, dtype=I32)), window, d ** -0.5).cpu().float()
    K.check_error_flags()
    ref = _attn_ref(qs, ks, vs, lens, starts, window, BF16)
    assert float((out - ref).abs().max()) < 2 ** -6, ("decode", seed, B, nq, nkv, d, window)
    # prompts
    B = rng.randint(1, 5)
    lens = [rng.choice([1, rng.randint(2, 60), rng.randint(60, 400)]) for _ in range(B)]
    starts = [rng.choice([0, 0, rng.randint(1, 700)]) for _ in range(B)]
    n_pages = sum((s + n + 63) // 64 for s, n in zip(starts, lens)) + 8
    table, kc, vc, ks, vs, qs = _attn_case(lens, starts, nq, nkv, d, BF16, window, 90 + seed, n_pages=n_pages)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=I32)
    ref = _attn_ref(qs, ks, vs, lens, starts, window, BF16)
    for tensor_memory in (True, False):
        out = K.attn_prefill(dev(torch.cat(qs).to(BF16)), dev(to_sw128(kc.to(BF16))), dev(to_sw128(vc.to(BF16))),
                             dev(table), dev(cu), dev(torch.tensor(starts, dtype=I32)), lens, window,
                             d ** -0.5, tensor_memory=tensor_memory).cpu().float()
        K.check_error_flags()
        assert float((out - ref).abs().max()) < 2 ** -6, ("prefill", tensor_memory, seed, lens, starts, nq, nkv, d, window)


@pytest.mark.parametrize("args", [
    ["gemm_tc", "--m", "8", "--n", "512", "--k", "256"], ["gemm_tc", "--m", "300", "--n", "512", "--k", "256", "--silu"],
    ["attn_decode", "--batch", "2", "--len", "200"], ["attn_prefill", "--tokens", "256"],
    ["attn_prefill", "--tokens", "256", "--mma-sync"], ["add_rmsnorm", "--m", "64", "--splits", "2"],
    ["qk_rope", "--m", "64"], ["gemm_qkv", "--m", "2048", "--k", "256"], ["argmax", "--m", "2", "--n", "20000"],
    ["sample", "--m", "2", "--n", "20000", "--top-k", "50", "--top-p", "0.9"]])
def test_the_micro_benchmark_runs_every_kernel_it_names(args, capsys):
    from lumenllm_b200 import kbench
    kbench.main(args + ["--copies", "2", "--reps", "1"])
    line = capsys.readouterr().out.strip().splitlines()[-1]
    assert line.startswith(args[0] + ":") and "us per launch" in line


@pytest.mark.parametrize("nq,nkv,H,lens", [(8, 2, 512, [3100, 248]), (5, 1, 256, [2500, 2100, 501]),
                                           (32, 8, 256, [700, 333])])
@pytest.mark.parametrize("rot", [128, 0])
def test_qkv_product_with_norm_rotation_and_cache_write_in_its_epilogue(nq, nkv, H, lens, rot):
    """The fused kernel against the plain formulas, and the cache against what the separate
    kernels write: several sequences that start at different positions, a row count that is no
    multiple of the tile, an odd number of heads (a last tile of one head)."""
    from lumenllm_b200.ops import kernels as K
    g = gen(29)
    d = 128
    N = sum(lens)
    Wn = (nq + 2 * nkv) * d
    assert K.gemm_tc_qkv_takes(N, Wn, H, nq, nkv, d, rot)
    starts = [70, 0, 5][:len(lens)]
    x = torch.randn(N, H, generator=g).to(BF16)
    w = (torch.randn(Wn, H, generator=g) / math.sqrt(H)).to(BF16)
    qw = 1 + 0.1 * torch.randn(d, generator=g)
    kw = 1 + 0.1 * torch.randn(d, generator=g)
    theta, eps = 50000.0, 1e-6
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(I32)
    seq = torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).to(I32)
    width = max((s + n + 63) // 64 for s, n in zip(starts, lens))
    n_pages = 1 + sum((s + n + 63) // 64 for s, n in zip(starts, lens))
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    table = torch.zeros(len(lens), width, dtype=I32)
    o = 0
    for b, (s, n) in enumerate(zip(starts, lens)):
        k_ = (s + n + 63) // 64
        table[b, :k_] = perm[o:o + k_].to(I32)
        o += k_
    kc = torch.zeros(n_pages, nkv, 64, d, dtype=BF16)
    kcd, vcd = dev(kc), dev(kc.clone())
    kcd2, vcd2 = dev(kc.clone()), dev(kc.clone())
    cs = K.rope_table(dev(pos), dev(P.rope_inv_freq(d, theta, d))) if rot else None
    xd, wd = dev(x), K.tile_weight(dev(w))
    q = K.gemm_tc_qkv(xd, wd, dev(qw), dev(kw), eps, cs, rot, dev(pos), dev(seq), dev(table), kcd, vcd, nq, nkv)
    K.check_error_flags()
    # the separate kernels on the same product
    qkv = K.gemm_tc(xd, wd)
    q2 = K.qk_norm_rope_store(qkv, dev(qw), dev(kw), eps, cs, rot, dev(pos), dev(seq), dev(table), kcd2, vcd2,
                              nq, nkv, d, BF16, layout=K.LAYOUT_SW128)
    rel = lambda a, b: float(((a.float() - b.float()).abs() / (1 + b.float().abs())).max())
    assert rel(q.cpu(), q2.cpu()) < 2 ** -7          # a rounding step of bfloat16 at most
    assert rel(kcd.cpu(), kcd2.cpu()) < 2 ** -7
    assert torch.equal(vcd.cpu(), vcd2.cpu())        # values are only rounded
    assert float(kcd.cpu()[0].float().abs().max()) == 0.0      # page 0 is nobody's
    # and the plain formulas
    full = (x.float() @ w.float().T).view(N, nq + 2 * nkv, d)
    qr = P.rms_norm(full[:, :nq], qw, eps)
    if rot:
        qr = P.apply_rope(qr, pos, theta, rot)
    assert rel(q.cpu(), qr) < 2 ** -7


@pytest.mark.parametrize("seed", range(8))
def test_drawn_qkv_products_with_their_epilogue(seed):
    """Heads, groups, width, sequences, where they start, norm weights or none, rotation or none,
    drawn at random: the fused kernel against the product and the rotary kernel one after the
    other (queries and keys within a rounding step of bfloat16, values and untouched pages
    bit for bit)."""
    import random
    from lumenllm_b200.ops import kernels as K
    rng = random.Random(400 + seed)
    g = gen(400 + seed)
    d = 128
    while True:
        nkv = rng.choice([1, 2, 3, 4, 8])
        nq = nkv * rng.choice([1, 2, 3, 4, 8])
        H = 8 * rng.randint(4, 64)
        total = rng.randint(1200, 7000)
        rot = rng.choice([128, 128, 0])
        if K.gemm_tc_qkv_takes(total, (nq + 2 * nkv) * d, H, nq, nkv, d, rot):
            break
    nseq = rng.randint(1, 5)
    cuts = sorted(rng.sample(range(1, total), nseq - 1))
    lens = [b - a for a, b in zip([0] + cuts, cuts + [total])]
    starts = [rng.choice([0, 0, rng.randint(1, 300)]) for _ in lens]
    x = dev(torch.randn(total, H, generator=g).to(BF16))
    w = dev((torch.randn((nq + 2 * nkv) * d, H, generator=g) / math.sqrt(H)).to(BF16))
    normed = rng.random() < 0.8
    qw = dev(1 + 0.1 * torch.randn(d, generator=g)) if normed else None
    kw = dev(1 + 0.1 * torch.randn(d, generator=g)) if normed else None
    pos = dev(torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(I32))
    seq = dev(torch.cat([torch.full((n,), b) for b, n in enumerate(lens)]).to(I32))
    width = max((s + n + 63) // 64 for s, n in zip(starts, lens))
    n_pages = 1 + sum((s + n + 63) // 64 for s, n in zip(starts, lens))
    perm = torch.randperm(n_pages - 1, generator=g) + 1
    table = torch.zeros(len(lens), width, dtype=I32)
    o = 0
    for b, (s, n) in enumerate(zip(starts, lens)):
        k_ = (s + n + 63) // 64
        table[b, :k_] = perm[o:o + k_].to(I32)
        o += k_
    table = dev(table)
    kc, vc, kc2, vc2 = (dev(torch.zeros(n_pages, nkv, 64, d, dtype=BF16)) for _ in range(4))
    cs = K.rope_table(pos, dev(P.rope_inv_freq(d, 50000.0, d))) if rot else None
    wt = K.tile_weight(w)
    q = K.gemm_tc_qkv(x, wt, qw, kw, 1e-6, cs, rot, pos, seq, table, kc, vc, nq, nkv)
    K.check_error_flags()
    q2 = K.qk_norm_rope_store(K.gemm_tc(x, wt), qw, kw, 1e-6, cs, rot, pos, seq, table, kc2, vc2, nq, nkv, d,
                              BF16, layout=K.LAYOUT_SW128)
    rel = lambda a, b: float(((a.float() - b.float()).abs() / (1 + b.float().abs())).max())
    what = (seed, nq, nkv, H, lens, starts, rot, normed)
    assert rel(q, q2) < 2 ** -7, what
    assert rel(kc, kc2) < 2 ** -7, what
    assert torch.equal(vc, vc2), what
    assert float(kc[0].float().abs().max()) == 0.0, what
