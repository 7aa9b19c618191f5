"""The decode-attention entry point that allocates nothing, called the way a program without
PyTorch's allocator would call it: through its exported C symbol, with raw device pointers.

Such callers exist: code running inside another framework's allocator hooks, plug-ins with a
memory budget fixed at start-up, serving loops that forbid cudaMalloc on the hot path, C or Rust
programs that link the shared object directly. For them `lumen_attn_decode_noalloc` keeps the
partial results of a long sequence's segments in an array that is part of the library. This test checks, on two
calls in a row with different batches (the second meets what the first left in the array), that
it returns what the ordinary entry point returns, and that a batch too large for the array is
refused without a launch.

The file name sorts last so that a run that stops at the first failure has already run every
other test; it passes alone in a fresh process as well.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_SCRATCH_TOO_SMALL = 100004
MAX_FLOATS = 4 * 1024 * 1024


def _case(B, nq, nkv, d, lens, n_pages, width, seed):
    """Random swizzled caches are as good as any: both entry points read the same bytes."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, nq, d, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(n_pages, nkv, 64, d, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(n_pages, nkv, 64, d, generator=g).to(torch.bfloat16).cuda()
    table = torch.zeros(B, width, dtype=torch.int32)
    free = list(range(1, n_pages))
    for b, n in enumerate(lens):
        for p in range((n + 63) // 64):
            table[b, p] = free.pop()
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    return q, kc, vc, table.cuda(), pos


def _noalloc_fn():
    from lumenllm_b200.csrc import build
    lib = ctypes.CDLL(str(build.ensure_built(["attn_decode"])["attn_decode"]))
    f = lib.lumen_attn_decode_noalloc
    f.restype = ctypes.c_int
    P, I = ctypes.c_void_p, ctypes.c_int
    f.argtypes = [P, P, P, P, I, P, P, I, I, I, I, I, ctypes.c_float, I, P, P]
    return f


def _call(f, q, kc, vc, table, pos, window, err, out=None):
    B, nq, d = q.shape
    out = torch.empty_like(q) if out is None else out
    rc = f(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0),
           pos.data_ptr(), out.data_ptr(), B, nq, kc.shape[1], d, window, float(d) ** -0.5,
           (table.shape[1] + 7) // 8, err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def _plain(q, kc, vc, table, pos, window):
    """softmax(q . k / sqrt(d)) over the keys each query sees, straight from the pages
    (un-swizzled here), in float64: the same reference the other attention tests use."""
    B, nq, d = q.shape
    nkv = kc.shape[1]

    def linear(c):            # [pages, nkv, 64, d] swizzled -> key-major
        x = c.cpu().view(c.shape[0], nkv, d // 64, 64, 8, 8)
        r = torch.arange(64)
        src = (torch.arange(8)[None, :] ^ (r[:, None] & 7))
        x = torch.gather(x, 4, src[None, None, None, :, :, None].expand_as(x).contiguous())
        return x.permute(0, 1, 3, 2, 4, 5).reshape(c.shape[0], nkv, 64, d)
    kl, vl = linear(kc), linear(vc)
    out = torch.empty(B, nq, d, dtype=torch.float64)
    for b in range(B):
        T = int(pos[b]) + 1
        pages = table[b, :(T + 63) // 64].cpu().long()
        k = kl[pages].transpose(1, 2).reshape(-1, nkv, d)[:T].double()
        v = vl[pages].transpose(1, 2).reshape(-1, nkv, d)[:T].double()
        lo = max(0, T - window) if window else 0
        for h in range(nq):
            kh = h // (nq // nkv)
            w = torch.softmax((k[lo:, kh] @ q[b, h].cpu().double()) / d ** 0.5, dim=0)
            out[b, h] = w @ v[lo:, kh]
    return out.float()


def test_no_alloc_entry_point_matches_the_allocating_one_twice():
    from lumenllm_b200.ops import kernels as K
    f = _noalloc_fn()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    cases = [
        dict(B=5, nq=8, nkv=2, d=128, lens=[1, 64, 129, 700, 1000], n_pages=48, width=16, window=0),
        dict(B=3, nq=4, nkv=2, d=64, lens=[300, 17, 128], n_pages=20, width=8, window=100),
    ]
    for i, c in enumerate(cases):
        window = c.pop("window")
        q, kc, vc, table, pos = _case(seed=20 + i, **c)
        expected = K.attn_decode(q, kc, vc, table, pos, window, float(q.shape[2]) ** -0.5)
        got = None                                            # drop the last call's output first
        out = torch.empty_like(q)                             # the caller's output, made beforehand
        torch.cuda.synchronize()
        # nothing may be allocated by the call: neither through torch's allocator nor, as the
        # device's own count of free memory shows, behind its back (from the second call on;
        # the first use of a library on a device may still load its device image)
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc, got = _call(f, q, kc, vc, table, pos, window, err, out)
        assert got is out
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if i > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert rc == 0, f"call {i} returned {rc}"
        assert int(err.item()) == 0
        assert torch.isfinite(got.float()).all()
        # the tests of the allocating entry point allow 2^-6 against the plain implementation;
        # the two entry points run the same kernels (with segments of their own sizes) and
        # must agree with each other and with the plain attention at least that well
        assert float((got.float() - expected.float()).abs().max()) < 2 ** -6, f"call {i}"
        assert float((got.float().cpu() - _plain(q, kc, vc, table, pos, window)).abs().max()) < 2 ** -6, f"call {i}"
    K.check_error_flags()


def test_no_alloc_entry_point_refuses_what_does_not_fit(capfd):
    f = _noalloc_fn()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    B, nq, nkv, d, width = 64, 32, 8, 128, 256
    assert B * nq * ((width + 7) // 8) * (d + 2) > MAX_FLOATS
    q, kc, vc, table, pos = _case(B, nq, nkv, d, [10] * B, 80, width, 30)
    rc, out = _call(f, q, kc, vc, table, pos, 0, err)
    assert rc == ERR_SCRATCH_TOO_SMALL
    assert "floats of scratch" in capfd.readouterr().err
    torch.cuda.synchronize()
