"""Python faces of the hand-written kernels. Each function checks dtypes and
shapes, launches on the current CUDA stream and returns its output tensor.
Float32 tensors select the 32-bit variants, bfloat16 tensors the serving ones.

A tensor that a split matrix product made may come as S partial results stacked
in front, [S, rows, width]; the consumers below add the partials while reading.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc.build import page_size as _page_size
from .native import KernelError, check, fn, int_fn, library, ptr, require, stream_ptr

P = c_void_p
F32 = torch.float32
BF16 = torch.bfloat16
I32 = torch.int32

PAGE = _page_size()   # tokens per cache page: LUMEN_PAGE of csrc/common.cuh
LAYOUT_LINEAR, LAYOUT_SW128 = 0, 1   # tile layouts of the cache, as in csrc/common.cuh


def _is_bf16(t) -> int:
    if t.dtype == BF16:
        return 1
    if t.dtype == F32:
        return 0
    raise KernelError(f"expected float32 or bfloat16, got {t.dtype}")


def _partials(t, name):
    """[rows, width] or [S, rows, width] -> (tensor as [S, rows, width], S)."""
    require(t, F32, name)
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if t.dim() != 3:
        raise KernelError(f"{name}: expected [rows, width] or [S, rows, width]")
    return t, t.shape[0]


def embed(tokens, table, out=None):
    """h[t] = float32(table[tokens[t]]). tokens int32 [N]; table [V, H] float32|bfloat16, or
    a TiledWeight (the table an output head shares)."""
    require(tokens, I32, "embed.tokens")
    N = tokens.numel()
    V, H = table.shape
    if isinstance(table, TiledWeight):
        if out is None:
            out = torch.empty((N, H), dtype=F32, device=table.device)
        f = fn("core", "lumen_embed_tiled", [P, P, P, c_int, c_int, c_int, c_int, P])
        check(f(ptr(tokens), ptr(table.data), ptr(out), N, H, V, table.padded_rows, stream_ptr()), "embed")
        return out
    if not table.is_contiguous() or not table.is_cuda:
        raise KernelError("embed.table must be a contiguous CUDA tensor")
    if out is None:
        out = torch.empty((N, H), dtype=F32, device=table.device)
    f = fn("core", "lumen_embed", [P, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(tokens), ptr(table), _is_bf16(table), ptr(out), N, H, V, stream_ptr()), "embed")
    return out


def add_rmsnorm(h, delta, weight, eps, out_dtype, rows=None, write_h=True):
    """x = h + sum(delta[s]) ; y = rmsnorm(x) * weight. h float32 [N, H] (updated in
    place when write_h); delta None or float32 [S, N, H]; rows int32 [W] gathers."""
    require(h, F32, "add_rmsnorm.h")
    require(weight, F32, "add_rmsnorm.weight")
    N, H = h.shape
    if weight.numel() != H:
        raise KernelError(f"add_rmsnorm: weight has {weight.numel()} values, rows have {H}")
    S, stride = 0, 0
    if delta is not None:
        delta, S = _partials(delta, "add_rmsnorm.delta")
        if tuple(delta.shape[1:]) != (N, H):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match h {(N, H)}")
        stride = N * H
    n_rows = N
    if rows is not None:
        require(rows, I32, "add_rmsnorm.rows")
        n_rows = rows.numel()
    y = torch.empty((n_rows, H), dtype=out_dtype, device=h.device)
    f = fn("core", "lumen_add_rmsnorm",
           [P, P, c_int, c_longlong, P, c_float, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(h), ptr(delta), S, stride, ptr(weight), float(eps), ptr(y), _is_bf16(y), ptr(rows),
            n_rows, H, 1 if write_h else 0, stream_ptr()), "add_rmsnorm")
    return y


def silu_mul(gu, out_dtype, interleaved=False):
    """z = silu(gate) * up with gate = gu[..., :I], up = gu[..., I:] (or, interleaved,
    gate_i = gu[..., 2i], up_i = gu[..., 2i+1]); gu float32 [N, 2I] or [S, N, 2I] partials."""
    gu, S = _partials(gu, "silu_mul.gu")
    _, N, I2 = gu.shape
    if I2 % 2:
        raise KernelError("silu_mul: width must be even")
    z = torch.empty((N, I2 // 2), dtype=out_dtype, device=gu.device)
    f = fn("core", "lumen_silu_mul", [P, c_int, P, c_int, c_int, c_int, c_int, P])
    check(f(ptr(gu), S, ptr(z), _is_bf16(z), N, I2 // 2, 1 if interleaved else 0, stream_ptr()),
          "silu_mul")
    return z


def rope_table(positions, inv_freq):
    """(cos, sin) of float32(pos) * inv_freq: float32 [N, rot/2, 2]."""
    require(positions, I32, "rope_table.positions")
    require(inv_freq, F32, "rope_table.inv_freq")
    N, half = positions.numel(), inv_freq.numel()
    cs = torch.empty((N, half, 2), dtype=F32, device=positions.device)
    f = fn("core", "lumen_rope_table", [P, P, P, c_int, c_int, P])
    check(f(ptr(positions), ptr(inv_freq), ptr(cs), N, half, stream_ptr()), "rope_table")
    return cs


def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, eps, cs, rotary_dim, cache_pos, tok_seq,
                       block_table, kcache, vcache, nq, nkv, d, out_dtype, layout=LAYOUT_LINEAR):
    """Per-head RMSNorm of q and k, rotation by the angles of `cs` (from rope_table; None
    with rotary_dim 0), q out and k/v written to the paged cache.
    qkv float32 [N, (nq + 2 nkv) d] or [S, N, ...] partials; caches [pages, nkv, PAGE, d] of
    out_dtype (None with nkv == 0: a layer that reads another layer's cache)."""
    qkv, S = _partials(qkv, "qk_norm_rope_store.qkv")
    N = qkv.shape[1]
    if qkv.shape[2] != (nq + 2 * nkv) * d:
        raise KernelError(f"qk_norm_rope_store: row width {qkv.shape[2]} != (nq+2nkv)*d")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != d:
                raise KernelError(f"{nm} weight must have head_dim={d} values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"rope angles must be [N, rotary_dim/2, 2], got {tuple(cs.shape)}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < N:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    q_out = torch.empty((N, nq, d), dtype=out_dtype, device=qkv.device)
    if nkv:
        require(kcache, out_dtype, "kcache")
        require(vcache, out_dtype, "vcache")
    f = fn("core", "lumen_qk_norm_rope_store",
           [P, c_int, P, P, c_float, P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
            c_int, c_int, P])
    check(f(ptr(qkv), S, ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cs), int(rotary_dim),
            ptr(cache_pos), ptr(tok_seq), ptr(block_table), block_table.stride(0),
            ptr(q_out), ptr(kcache), ptr(vcache), _is_bf16(q_out), N, nq, nkv, d, int(layout),
            stream_ptr()),
          "qk_norm_rope_store")
    return q_out


def gemm_tc_qkv_takes(M, N, K, nq, nkv, d, rotary_dim) -> bool:
    """Whether gemm_tc_qkv takes this shape (a prompt-sized product, heads of 128, rotation
    over the whole head or none)."""
    return bool(int_fn("gemm_tc", "lumen_gemm_tc_qkv_ok", [c_int] * 7)(
        int(M), int(N), int(K), int(nq), int(nkv), int(d), int(rotary_dim)))


def gemm_tc_qkv(x, w, q_norm_w, k_norm_w, eps, cs, rotary_dim, cache_pos, tok_seq, block_table,
                kcache, vcache, nq, nkv):
    """The QKV product of a prompt with qk_norm_rope_store folded into its epilogue: x bfloat16
    [M, K], w a TiledWeight [(nq + 2 nkv) * 128, K] (q heads, k heads, v heads); returns q bfloat16
    [M, nq, 128], normed and rotated, and writes k and v to their places in the swizzled
    bfloat16 cache. Only where gemm_tc_qkv_takes says so."""
    require(x, BF16, "gemm_tc_qkv.x")
    if not isinstance(w, TiledWeight):
        raise KernelError("gemm_tc_qkv takes its weight in tiled form (tile_weight)")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not gemm_tc_qkv_takes(M, N, K, nq, nkv, 128, rotary_dim):
        raise KernelError(f"gemm_tc_qkv does not take [{M}, {K}] x [{N}, {w.shape[1]}] with {nq}+2x{nkv} heads")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != 128:
                raise KernelError(f"{nm} weight must have 128 values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if tuple(cs.shape) != (M, 64, 2):
            raise KernelError(f"rope angles must be [M, 64, 2], got {tuple(cs.shape)}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < M:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    require(kcache, BF16, "kcache")
    require(vcache, BF16, "vcache")
    if kcache.shape[1:] != (nkv, PAGE, 128) or vcache.shape != kcache.shape:
        raise KernelError(f"gemm_tc_qkv: caches must be [pages, nkv, {PAGE}, 128]")
    q_out = torch.empty((M, nq, 128), dtype=BF16, device=x.device)
    f = fn("gemm_tc", "lumen_gemm_tc_qkv",
           [P, P, c_int, c_int, c_int, c_int, P, P, P, P, P, c_float, P, c_int, P, P, P, c_int, c_int, c_int, P, P])
    check(f(ptr(x), ptr(w.data), M, N, K, w.padded_rows, ptr(q_out), ptr(kcache), ptr(vcache), ptr(q_norm_w), ptr(k_norm_w),
            float(eps), ptr(cs), int(rotary_dim), ptr(cache_pos), ptr(tok_seq), ptr(block_table),
            block_table.stride(0), nq, nkv, ptr(error_flag(x.device)), stream_ptr()), "gemm_tc_qkv")
    return q_out


def attn_generic(q, kcache, vcache, block_table, tok_seq, tok_pos, window, scale,
                 layout=LAYOUT_LINEAR):
    """Causal attention of N query tokens over the paged cache. q [N, nq, d]."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    require(q, q.dtype, "attn.q")
    require(kcache, q.dtype, "attn.kcache")
    require(vcache, q.dtype, "attn.vcache")
    require(block_table, I32, "attn.block_table")
    require(tok_seq, I32, "attn.tok_seq")
    require(tok_pos, I32, "attn.tok_pos")
    if d % 16 or d > 256:
        raise KernelError(f"attention takes head sizes in steps of 16 up to 256, not {d}")
    out = torch.empty_like(q)
    f = fn("attn_generic", "lumen_attn_generic",
           [P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(tok_seq),
            ptr(tok_pos), ptr(out), _is_bf16(q), N, nq, nkv, d, int(window), float(scale), int(layout),
            stream_ptr()), "attn_generic")
    return out


def gemm_f32(a, w, out=None):
    """C = a @ w.T in true float32 (FFMA). a float32 [M, K]; w [N, K] float32|bfloat16."""
    require(a, F32, "gemm_f32.a")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm_f32: inner sizes differ ({K} vs {K2})")
    if not (w.is_cuda and w.is_contiguous()):
        raise KernelError("gemm_f32.w must be a contiguous CUDA tensor")
    if out is None:
        out = torch.empty((M, N), dtype=F32, device=a.device)
    f = fn("gemm_f32", "lumen_gemm_f32", [P, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(a), ptr(w), _is_bf16(w), ptr(out), M, N, K, stream_ptr()), "gemm_f32")
    return out


class TiledWeight:
    """A bfloat16 weight [rows, cols] in the form the tensor-core products read: the image its
    tiles have in shared memory, k block after k block, rows padded to `padded_rows` (see the
    head of csrc/gemm_tc.cu). `first_rows(n)` is the weight's first n rows on the same memory."""
    __slots__ = ("data", "rows", "cols", "padded_rows")

    def __init__(self, data, rows, cols, padded_rows):
        self.data, self.rows, self.cols, self.padded_rows = data, int(rows), int(cols), int(padded_rows)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    def data_ptr(self):
        return self.data.data_ptr()

    def first_rows(self, n: int) -> "TiledWeight":
        if not 0 < n <= self.rows:
            raise KernelError(f"a tiled weight of {self.rows} rows has no first {n} rows")
        return TiledWeight(self.data, n, self.cols, self.padded_rows)

    def row_major(self) -> torch.Tensor:
        """The weight as an ordinary [rows, cols] tensor again (a copy; tests and debugging)."""
        kb = (self.cols + 63) // 64
        t = self.data.view(kb, self.padded_rows, 8, 8)                 # [k block, row, piece, 8 values]
        r = torch.arange(self.padded_rows, device=t.device) % 8
        j = torch.arange(8, device=t.device)
        src = (j[None, :] ^ r[:, None])                                # piece c of row r sits at place c ^ (r & 7)
        t = torch.gather(t, 2, src[None, :, :, None].expand(kb, -1, -1, 8))
        return t.permute(1, 0, 2, 3).reshape(self.padded_rows, kb * 64)[: self.rows, : self.cols].contiguous()


def can_tile(w) -> bool:
    return (isinstance(w, torch.Tensor) and w.dtype == BF16 and w.is_cuda and w.dim() == 2
            and w.shape[1] % 8 == 0 and w.shape[0] > 0)


def tile_weight(w) -> TiledWeight:
    """The tiled form of a bfloat16 weight [N, K], K a multiple of 8."""
    require(w, BF16, "tile_weight.w")
    if not can_tile(w):
        raise KernelError(f"tile_weight takes bfloat16 [N, K] with K a multiple of 8, not {tuple(w.shape)}")
    N, K = w.shape
    padded = int(int_fn("gemm_tc", "lumen_tiled_weight_rows", [c_int])(int(N)))
    out = torch.empty(((K + 63) // 64) * padded * 64, dtype=BF16, device=w.device)
    f = fn("gemm_tc", "lumen_tile_weight", [P, P, c_int, c_int, P])
    check(f(ptr(w), ptr(out), N, K, stream_ptr()), "tile_weight")
    return TiledWeight(out, N, K, padded)


def gemm_tc_splits(M, N, K, silu=False) -> int:
    return int(int_fn("gemm_tc", "lumen_gemm_tc_splits", [c_int, c_int, c_int, c_int])(
        int(M), int(N), int(K), 1 if silu else 0))


def gemm_tc_adds(M, N) -> bool:
    """Whether gemm_tc can add a product of this shape to a float32 matrix in place."""
    return bool(int_fn("gemm_tc", "lumen_gemm_tc_adds", [c_int, c_int])(int(M), int(N)))


def gemm_tc(x, w, silu_interleaved=False, add_to=None):
    """x @ w.T on the tcgen05 tensor cores. x bfloat16 [M, K], w a TiledWeight [N, K], K a
    multiple of 8. Returns float32 partials [S, M, N] (S = 1 unless M <= 256); or, with
    silu_interleaved (rows of w alternate gate_i, up_i), bfloat16 [M, N/2] = silu(gate)*up;
    or, with add_to (float32 [M, N], only where gemm_tc_adds(M, N)), adds the product to it
    in place (one float32 add an element, by the copy engine) and returns None."""
    require(x, BF16, "gemm_tc.x")
    if not isinstance(w, TiledWeight):
        raise KernelError("gemm_tc takes its weight in tiled form (tile_weight)")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or K % 8:
        raise KernelError(f"gemm_tc: inner sizes {K} and {K2} must agree and be a multiple of 8")
    epi = 0
    if add_to is not None:
        require(add_to, F32, "gemm_tc.add_to")
        if silu_interleaved or tuple(add_to.shape) != (M, N) or not gemm_tc_adds(M, N):
            raise KernelError(f"gemm_tc: a product [{M}, {N}] cannot be added in place")
        out, epi = add_to, 2
    elif silu_interleaved:
        if N % 2:
            raise KernelError("gemm_tc: gate/up rows must come in pairs")
        out, epi = torch.empty((M, N // 2), dtype=BF16, device=x.device), 1
    else:
        out = torch.empty((gemm_tc_splits(M, N, K), M, N), dtype=F32, device=x.device)
    f = fn("gemm_tc", "lumen_gemm_tc", [P, P, P, c_int, c_int, c_int, c_int, c_int, P, P])
    check(f(ptr(x), ptr(w.data), ptr(out), M, N, K, w.padded_rows, epi, ptr(error_flag(x.device)), stream_ptr()),
          "gemm_tc")
    return None if add_to is not None else out


def argmax(logits, out=None):
    """Row-wise argmax of float32 [B, V]; equal maxima give the lowest index."""
    require(logits, F32, "argmax.logits", contiguous=False)
    B, V = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("argmax: rows must be contiguous")
    if out is None:
        out = torch.empty((B,), dtype=I32, device=logits.device)
    scratch = torch.empty((2 * 64 * B,), dtype=I32, device=logits.device) if V >= 16384 else None
    f = fn("sample", "lumen_argmax", [P, c_longlong, c_int, c_int, P, P, P])
    check(f(ptr(logits), logits.stride(0), B, V, ptr(out), ptr(scratch), stream_ptr()), "argmax")
    return out


def sample(logits, opts, top_k, out=None):
    """Row-wise sampling. opts float32 [B, 4] = (temperature, top_p, min_p, u); top_k int32 [B]."""
    require(logits, F32, "sample.logits", contiguous=False)
    require(opts, F32, "sample.opts")
    require(top_k, I32, "sample.top_k")
    B, V = logits.shape
    if logits.stride(1) != 1 or opts.shape != (B, 4) or top_k.numel() != B:
        raise KernelError("sample: bad shapes")
    if out is None:
        out = torch.empty((B,), dtype=I32, device=logits.device)
    f = fn("sample", "lumen_sample", [P, c_longlong, c_int, c_int, P, P, P, P])
    check(f(ptr(logits), logits.stride(0), B, V, ptr(opts), ptr(top_k), ptr(out), stream_ptr()),
          "sample")
    return out


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """A device int that kernels with bounded waits set when a wait ran out."""
    key = torch.device(device).index
    t = _err_flags.get(key)
    if t is None:
        t = _err_flags[key] = torch.zeros((1,), dtype=I32, device=device)
    return t


def check_error_flags() -> None:
    """Raises if any kernel gave up on a wait since the last check (synchronises)."""
    for dev, t in _err_flags.items():
        if int(t.item()) != 0:
            recover(dev)
            raise KernelError(f"a kernel on cuda:{dev} gave up waiting for its own copies")


def recover(device) -> None:
    """After a kernel gave up: the flag back to zero, and the counters that the decode
    attention's blocks leave at zero only when all of them arrive."""
    key = torch.device("cuda", device).index if isinstance(device, int) else torch.device(device).index
    for table in (_err_flags, _counters):
        t = table.get(key)
        if t is not None:
            t.zero_()


_COUNTERS = 1 << 16
_counters = {}


def _decode_counters(device) -> torch.Tensor:
    """Zeroed ints that the decode-attention blocks count themselves in with; every call
    leaves them zero again, and calls on a device run in stream order."""
    key = torch.device(device).index
    t = _counters.get(key)
    if t is None:
        t = _counters[key] = torch.zeros((_COUNTERS,), dtype=I32, device=device)
    return t


DECODE_MAX_SEGS = 32
# Pages a decode-attention block walks (unless the sequence is longer than 32 segments of them).
# One number for every batch: how a sequence's keys are cut, and so the order in which its
# partial results are merged, depends on the sequence alone, never on who else is in the batch
# or on the page table's width.
DECODE_SEG_PAGES = 4


def attn_decode(q, kcache, vcache, block_table, seq_pos, window, scale):
    """Split-KV decode attention, bfloat16, swizzled cache, head size 64 or 128, at most
    16 query heads per kv head. q [B, nq, d]; seq_pos int32 [B]: each query's position."""
    B, nq, d = q.shape
    nkv = kcache.shape[1]
    require(q, BF16, "attn_decode.q")
    require(kcache, BF16, "attn_decode.kcache")
    require(vcache, BF16, "attn_decode.vcache")
    require(block_table, I32, "attn_decode.block_table")
    require(seq_pos, I32, "attn_decode.seq_pos")
    if seq_pos.numel() < B or block_table.shape[0] < B:
        raise KernelError("attn_decode: metadata shorter than the batch")
    width = block_table.shape[1]
    seg_pages = DECODE_SEG_PAGES
    max_segs = min(-(-width // seg_pages), DECODE_MAX_SEGS)
    out = torch.empty_like(q)
    part_o = torch.empty((B, nq, max_segs, d), dtype=F32, device=q.device)
    part_ml = torch.empty((B, nq, max_segs, 2), dtype=F32, device=q.device)
    counters = _decode_counters(q.device) if B * nkv <= _COUNTERS else None
    f = fn("attn_decode", "lumen_attn_decode",
           [P, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, P, P, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(seq_pos),
            ptr(out), ptr(part_o), ptr(part_ml), B, nq, nkv, d, int(window), float(scale), max_segs,
            seg_pages,
            ptr(error_flag(q.device)), ptr(counters), stream_ptr()), "attn_decode")
    return out


def attn_decode_qkv(qkv, q_norm_w, k_norm_w, eps, cs, rotary_dim, kcache, vcache, block_table, seq_pos,
                    window, scale, nq, nkv, store_kv=True):
    """Decode attention that does the rotary kernel's work itself: qkv is the projection as
    the product left it, float32 [B, (nq + 2 nkv) * 128] or [S, B, ...] partial sums; every
    block makes its query heads (sum of the parts, head norm with q_norm_w / k_norm_w [128] or
    None, rotation over the whole head when rotary_dim == 128, by cs [B, 64, 2]), and with
    store_kv the new token's key and value are made and written to the cache. The same bits as
    qk_norm_rope_store followed by attn_decode. Head size 128, swizzled bfloat16 cache."""
    qkv, S = _partials(qkv, "attn_decode_qkv.qkv")
    B = qkv.shape[1]
    d = 128
    if qkv.shape[2] != (nq + 2 * nkv) * d or kcache.shape[1:] != (nkv, PAGE, d) or rotary_dim not in (0, d):
        raise KernelError(f"attn_decode_qkv: projection {tuple(qkv.shape)} and cache {tuple(kcache.shape)} do not "
                          f"fit {nq}+2x{nkv} heads of {d} (rotation over {rotary_dim})")
    require(kcache, BF16, "attn_decode_qkv.kcache")
    require(vcache, BF16, "attn_decode_qkv.vcache")
    require(block_table, I32, "attn_decode_qkv.block_table")
    require(seq_pos, I32, "attn_decode_qkv.seq_pos")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != d:
                raise KernelError(f"{nm} weight must have {d} values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if cs.numel() < B * 64 * 2:
            raise KernelError("rope angles shorter than the batch")
    if seq_pos.numel() < B or block_table.shape[0] < B:
        raise KernelError("attn_decode_qkv: metadata shorter than the batch")
    width = block_table.shape[1]
    seg_pages = DECODE_SEG_PAGES
    max_segs = min(-(-width // seg_pages), DECODE_MAX_SEGS)
    out = torch.empty((B, nq, d), dtype=BF16, device=qkv.device)
    part_o = torch.empty((B, nq, max_segs, d), dtype=F32, device=qkv.device)
    part_ml = torch.empty((B, nq, max_segs, 2), dtype=F32, device=qkv.device)
    counters = _decode_counters(qkv.device) if B * nkv <= _COUNTERS else None
    f = fn("attn_decode", "lumen_attn_decode_qkv",
           [P, c_int, c_longlong, P, P, c_float, P, c_int, c_int, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int,
            c_int, c_int, c_float, c_int, c_int, P, P, P])
    check(f(ptr(qkv), S, qkv.stride(0) if S > 1 else 0, ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cs),
            1 if rotary_dim else 0, 1 if store_kv else 0, ptr(kcache), ptr(vcache), ptr(block_table),
            block_table.stride(0), ptr(seq_pos), ptr(out), ptr(part_o), ptr(part_ml), B, nq, nkv, d, int(window),
            float(scale), max_segs, seg_pages, ptr(error_flag(qkv.device)), ptr(counters), stream_ptr()),
          "attn_decode_qkv")
    return out


def attn_prefill(q, kcache, vcache, block_table, cu_q, seq_start, q_lens, window, scale,
                 tensor_memory=True, n_seqs=None):
    """Causal flash attention for sequences that bring q_lens[b] tokens each (host list),
    bfloat16, swizzled cache, head size 64 or 128, at most 16 query heads per kv head.
    q [N, nq, d]; cu_q int32 [B+1]; seq_start int32 [B]. With tensor_memory the tcgen05
    kernel (128 rows a block, S and O in tensor memory), else the mma.sync kernel (64 rows).
    With q_lens None and n_seqs = B the host need not know how the N tokens are divided (a
    captured step does not): enough blocks are launched for any division, every block finds
    its sequence and tile from cu_q on the device, and the blocks left over return at once."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    B = len(q_lens) if q_lens is not None else int(n_seqs)
    require(q, BF16, "attn_prefill.q")
    require(kcache, BF16, "attn_prefill.kcache")
    require(vcache, BF16, "attn_prefill.vcache")
    require(block_table, I32, "attn_prefill.block_table")
    require(cu_q, I32, "attn_prefill.cu_q")
    require(seq_start, I32, "attn_prefill.seq_start")
    if nq % nkv or nq // nkv > 16:
        raise KernelError("attn_prefill: at most 16 query heads per kv head")
    if cu_q.numel() < B + 1 or seq_start.numel() < B or block_table.shape[0] < B or \
            (q_lens is not None and sum(q_lens) != N):
        raise KernelError("attn_prefill: metadata does not match the batch")
    tq = (128 if tensor_memory else 64) // (nq // nkv)
    # sum of ceil(q_b / tq) over any division of N tokens into B sequences is at most N // tq + B
    n_tiles = sum((n + tq - 1) // tq for n in q_lens) if q_lens is not None else N // tq + B
    out = torch.empty_like(q)
    f = fn("attn_prefill_tc" if tensor_memory else "attn_prefill",
           "lumen_attn_prefill_tc" if tensor_memory else "lumen_attn_prefill",
           [P, P, P, P, c_int, P, P, c_int, c_int, P, c_int, c_int, c_int, c_int, c_float, P, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(cu_q),
            ptr(seq_start), B, n_tiles, ptr(out), nq, nkv, d, int(window), float(scale),
            ptr(error_flag(q.device)), stream_ptr()), "attn_prefill")
    return out
