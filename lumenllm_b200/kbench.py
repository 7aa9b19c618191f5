"""Micro-benchmarks of single kernels at chosen sizes:

    python -m lumenllm_b200.kbench gemm_tc --m 2048 --n 4096 --k 4096 [--silu] [--copies 8] [--reps 5]
    python -m lumenllm_b200.kbench attn_decode --batch 8 --len 1600 --heads 32 --kv-heads 8 --head-dim 128
    python -m lumenllm_b200.kbench attn_prefill --tokens 2048 --heads 32 --kv-heads 8 --head-dim 128
    python -m lumenllm_b200.kbench add_rmsnorm --m 2048 --n 4096 [--splits 9]
    python -m lumenllm_b200.kbench qk_rope --m 2048 --heads 32 --kv-heads 8 --head-dim 128
    python -m lumenllm_b200.kbench gemm_qkv --m 2048 --k 4096 --heads 32 --kv-heads 8
    python -m lumenllm_b200.kbench argmax --m 8 --n 151936
    python -m lumenllm_b200.kbench sample --m 8 --n 151936 [--top-k 50] [--top-p 0.9]
    python -m lumenllm_b200.kbench stream --blocks 148 --k 4096 --stages 6 [--tiled]   (no kernel of the
        model: blocks that only stream 16 KB stages into shared memory, csrc/stream_probe.cu)

Each run cycles through `--copies` distinct operand sets (more bytes than the L2 holds, so
that what is timed comes from HBM), times `--reps` passes with CUDA events after a warm-up and
prints one line: microseconds per launch, and GB/s of the bytes the kernel has to move or
TFLOP/s of its products. It is also the small workload that profiler captures are taken on.
"""
from __future__ import annotations

import argparse
import math
from ctypes import c_int, c_void_p

import torch

from .ops import kernels as K


def _time(fns, reps):
    """Microseconds per launch. The calls of one pass are captured in a CUDA graph and the
    graph is replayed, so that what is timed is the device's work and not the host's launch
    path (a Python launch costs more than a short kernel runs)."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / (reps * len(fns))


def _paged(B, length, nkv, d, dev):
    pages = (length + K.PAGE - 1) // K.PAGE
    n_pages = B * pages + 1
    kc = torch.randn(n_pages, nkv, K.PAGE, d, device=dev).to(torch.bfloat16)
    vc = torch.randn(n_pages, nkv, K.PAGE, d, device=dev).to(torch.bfloat16)
    table = (torch.arange(B * pages, device=dev, dtype=torch.int32) + 1).view(B, pages)
    return kc, vc, table


def main(argv=None):
    ap = argparse.ArgumentParser(prog="kbench")
    ap.add_argument("kernel", choices=["gemm_tc", "attn_decode", "attn_prefill",
                                       "add_rmsnorm", "qk_rope", "gemm_qkv", "argmax", "sample", "stream"])
    ap.add_argument("--splits", type=int, default=1, help="add_rmsnorm: partial sums to add")
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--silu", action="store_true")
    ap.add_argument("--mma-sync", action="store_true", help="attn_prefill: the mma.sync kernel")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--len", type=int, default=1600)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--no-pdl", action="store_true",
                    help="launch without programmatic dependent launch")
    ap.add_argument("--single-sm", action="store_true",
                    help="gemm_tc: keep prompt-sized products on the single-SM kernel")
    ap.add_argument("--bn", type=int, default=0, help="gemm_tc: fix the single-SM kernel's tile width")
    ap.add_argument("--blocks", type=int, default=148, help="stream: blocks, one an SM")
    ap.add_argument("--stages", type=int, default=6, help="stream: 16 KB stages of a block's ring")
    ap.add_argument("--tiled", action="store_true",
                    help="stream: the matrix in the tiled form of the products' weights (else row-major)")
    ap.add_argument("--rounds", type=int, default=0,
                    help="stream: tiles a block streams one after the other, all k blocks of each (tiled form)")
    ap.add_argument("--tile-major", action="store_true",
                    help="stream, with --rounds: the matrix stored tile after tile instead of k block after k block")
    ap.add_argument("--seg-pages", type=int, default=0,
                    help="attn_decode: pages a block walks (default: the product's rule)")
    a = ap.parse_args(argv)
    from .ops import native
    if a.no_pdl:
        native.preload(["core", "gemm_tc", "attn_decode", "attn_prefill_tc", "attn_prefill", "sample"])
        native.set_dependent_launch(False)
    if a.single_sm or a.bn:
        native.check(native.int_fn("gemm_tc", "lumen_gemm_tc_tune", [c_int, c_int])(0 if a.single_sm else 1, a.bn),
                     "gemm_tc_tune")
        native.launches -= 1
    if a.seg_pages:
        K.DECODE_SEG_PAGES = a.seg_pages
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    bf = torch.bfloat16
    note = ""
    if a.kernel == "gemm_tc":
        ws = [K.tile_weight((torch.randn(a.n, a.k, device=dev) / math.sqrt(a.k)).to(bf)) for _ in range(a.copies)]
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        fns = [lambda w=w: K.gemm_tc(x, w, silu_interleaved=a.silu) for w in ws]
        us = _time(fns, a.reps)
        nbytes = a.n * a.k * 2 + a.m * a.k * 2
        flops = 2.0 * a.m * a.n * a.k
        note = f"{nbytes / us / 1e3:.0f} GB/s  {flops / us / 1e6:.1f} TFLOP/s"
    elif a.kernel == "stream":
        # blocks x (k / 64) stages of 16 KB: what the SMs take in when nothing is done with it
        nkb = max(1, a.k // 64)
        rounds = max(1, a.rounds)
        mode = (3 if a.tile_major else 2) if a.rounds else (1 if a.tiled else 0)
        nbytes = a.blocks * rounds * nkb * 16384
        bufs = [torch.full((nbytes,), i + 1, dtype=torch.uint8, device=dev) for i in range(a.copies)]
        scratch = torch.zeros(2, dtype=torch.int32, device=dev)
        f = native.fn("stream_probe", "lumen_stream_probe", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
        fns = [lambda b=b: native.check(f(b.data_ptr(), a.blocks, nkb, a.stages, mode, rounds,
                                          scratch.data_ptr(), native.stream_ptr()), "stream_probe") for b in bufs]
        us = _time(fns, a.reps)
        if int(scratch[0]) != 0:
            raise native.KernelError("stream: a copy never arrived")
        note = (f"{nbytes / us / 1e3:.0f} GB/s  {nbytes / a.blocks / us / 1e3:.1f} GB/s a block  "
                f"{us * 1e3 / (nkb * rounds):.0f} ns a stage  ({['row-major', 'tiled', 'tiled, tile after tile of a tall matrix', 'tile-major'][mode]}, {a.stages} stages)")
    elif a.kernel == "attn_decode":
        sets = [_paged(a.batch, a.len, a.kv_heads, a.head_dim, dev) for _ in range(a.copies)]
        q = torch.randn(a.batch, a.heads, a.head_dim, device=dev).to(bf)
        pos = torch.full((a.batch,), a.len - 1, dtype=torch.int32, device=dev)
        fns = [lambda s=s: K.attn_decode(q, s[0], s[1], s[2], pos, 0, a.head_dim ** -0.5) for s in sets]
        us = _time(fns, a.reps)
        nbytes = 2 * a.batch * a.len * a.kv_heads * a.head_dim * 2
        note = f"{nbytes / us / 1e3:.0f} GB/s"
    elif a.kernel == "attn_prefill":
        kc, vc, table = _paged(1, a.tokens, a.kv_heads, a.head_dim, dev)
        q = torch.randn(a.tokens, a.heads, a.head_dim, device=dev).to(bf)
        cu = torch.tensor([0, a.tokens], dtype=torch.int32, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        fns = [lambda: K.attn_prefill(q, kc, vc, table, cu, st, [a.tokens], 0, a.head_dim ** -0.5,
                                      tensor_memory=not a.mma_sync)]
        us = _time(fns, a.reps)
        flops = 2.0 * a.tokens * a.tokens * a.head_dim * a.heads      # causal: half of 4 T^2 d
        note = f"{flops / us / 1e6:.1f} TFLOP/s"
    elif a.kernel == "add_rmsnorm":
        hs = [torch.randn(a.m, a.n, device=dev) for _ in range(a.copies)]
        ds = [torch.randn(a.splits, a.m, a.n, device=dev) for _ in range(a.copies)]
        w = torch.ones(a.n, device=dev)
        fns = [lambda h=h, d=d: K.add_rmsnorm(h, d, w, 1e-6, bf) for h, d in zip(hs, ds)]
        us = _time(fns, a.reps)
        # h read, y written; with partial sums those are read and h is written back
        note = f"{a.m * a.n * ((10 + 4 * a.splits) if a.splits else 6) / us / 1e3:.0f} GB/s"
    elif a.kernel in ("argmax", "sample"):
        lgs = [torch.randn(a.m, a.n, device=dev) * 3 for _ in range(a.copies)]
        if a.kernel == "argmax":
            fns = [lambda l=l: K.argmax(l) for l in lgs]
        else:
            opts = torch.tensor([[0.8, a.top_p, a.min_p, 0.37]] * a.m, dtype=torch.float32, device=dev)
            tk = torch.full((a.m,), a.top_k, dtype=torch.int32, device=dev)
            fns = [lambda l=l: K.sample(l, opts, tk) for l in lgs]
        us = _time(fns, a.reps)
        note = f"{a.m * a.n * 4 / us / 1e3:.0f} GB/s"
    elif a.kernel == "qk_rope":
        nh = a.heads + 2 * a.kv_heads
        xs = [torch.randn(a.m, nh * a.head_dim, device=dev) for _ in range(a.copies)]
        kc, vc, table = _paged(1, a.m, a.kv_heads, a.head_dim, dev)
        pos = torch.arange(a.m, dtype=torch.int32, device=dev)
        seq = torch.zeros(a.m, dtype=torch.int32, device=dev)
        inv = 1.0 / (1e6 ** (torch.arange(0, a.head_dim, 2, dtype=torch.float32) / a.head_dim))
        cs = K.rope_table(pos, inv.to(dev))
        wn = torch.ones(a.head_dim, device=dev)
        fns = [lambda x=x: K.qk_norm_rope_store(x, wn, wn, 1e-6, cs, a.head_dim, pos, seq, table, kc, vc,
                                                a.heads, a.kv_heads, a.head_dim, bf, layout=K.LAYOUT_SW128)
               for x in xs]
        us = _time(fns, a.reps)
        note = f"{a.m * nh * a.head_dim * 6 / us / 1e3:.0f} GB/s"
    else:
        # the QKV product of a prompt with norm, rotation and cache write in its epilogue
        nh = a.heads + 2 * a.kv_heads
        ws = [K.tile_weight((torch.randn(nh * 128, a.k, device=dev) / math.sqrt(a.k)).to(bf)) for _ in range(a.copies)]
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        kc, vc, table = _paged(1, a.m, a.kv_heads, 128, dev)
        pos = torch.arange(a.m, dtype=torch.int32, device=dev)
        seq = torch.zeros(a.m, dtype=torch.int32, device=dev)
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        cs = K.rope_table(pos, inv.to(dev))
        wn = torch.ones(128, device=dev)
        fns = [lambda w=w: K.gemm_tc_qkv(x, w, wn, wn, 1e-6, cs, 128, pos, seq, table, kc, vc, a.heads, a.kv_heads)
               for w in ws]
        us = _time(fns, a.reps)
        note = f"{2.0 * a.m * nh * 128 * a.k / us / 1e6:.1f} TFLOP/s"
    K.check_error_flags()
    print(f"{a.kernel}: {us:.1f} us per launch  {note}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
