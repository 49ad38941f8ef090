"""Typed Python faces of the CUDA entry points: tensors in, launch on the current
stream.  Nothing here computes; a missing or failing library raises NativeError.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .native import call, dtype_code, ptr, stream_ptr


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise native.NativeError("kernels take CUDA tensors only; there is no CPU path")


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t,:] = table[tokens[t],:] in float32."""
    _cuda(table, tokens, out)
    V, E = table.shape
    T = tokens.numel()
    assert out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous() and tokens.dtype == torch.int32
    call("gb_embed", ptr(table), dtype_code(table), ptr(tokens), T, E, V, ptr(out), stream_ptr())
    return out


def embed_shadow(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, xb: torch.Tensor, ssq: torch.Tensor) -> None:
    """embed plus what a deferred norm needs: xb = bfloat16(out), ssq[t] = sum(out[t,:]^2)."""
    _cuda(table, tokens, out, xb, ssq)
    V, E = table.shape
    T = tokens.numel()
    assert out.dtype == torch.float32 and out.shape == (T, E) and out.is_contiguous() and tokens.dtype == torch.int32
    assert xb.dtype == torch.bfloat16 and xb.shape == (T, E) and xb.is_contiguous() and ssq.dtype == torch.float32
    assert ssq.numel() >= T
    call("gb_embed_shadow", ptr(table), dtype_code(table), ptr(tokens), T, E, V, ptr(out), ptr(xb), ptr(ssq), stream_ptr())


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x: float32 [T,E] residual stream.  delta: None, [T,E] or [S,T,E] terms still to be
    added to x.  rows: int32 row numbers to gather (then out has len(rows) rows)."""
    _cuda(x, delta, weight, out, rows)
    T, E = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.numel() == E
    n_delta, stride = 0, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == (T, E)
        n_delta = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * E
    n_rows = T if rows is None else rows.numel()
    assert out.shape == (n_rows, E)
    call("gb_add_rmsnorm", ptr(x), ptr(delta), 0 if delta is None else dtype_code(delta), n_delta, stride, ptr(rows),
         n_rows, E, ptr(weight), dtype_code(weight), float(eps), ptr(out), dtype_code(out), int(write_x), stream_ptr())
    return out


def rope_kv_write(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], n_heads: int, n_kv_heads: int,
                  head_dim: int, inv_freq: Optional[torch.Tensor], rotary_dim: int, pairing: int,
                  seq_of: torch.Tensor, pos: torch.Tensor, table: Optional[torch.Tensor], ring_pages: int,
                  kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor]) -> None:
    """q, k, v: column slices [T, heads*head_dim] of one row-major buffer (equal row
    stride).  Rotates q in place; writes rotated k and v into the cache pages."""
    _cuda(q, k, v, inv_freq, seq_of, pos, table, kcache, vcache)
    T = q.shape[0]
    ld = q.stride(0)
    assert q.stride(1) == 1 and (k is None or (k.stride(0) == ld and v.stride(0) == ld and k.dtype == q.dtype))
    call("gb_rope_kv_write", ptr(q), ptr(k), ptr(v), dtype_code(q), ld, T, n_heads, n_kv_heads, head_dim,
         rotary_dim, pairing, ptr(inv_freq), ptr(seq_of), ptr(pos), ptr(table),
         0 if table is None else table.shape[1], ring_pages, ptr(kcache), ptr(vcache),
         0 if kcache is None else dtype_code(kcache), stream_ptr())


def attention_generic(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, ring_pages: int,
                      kcache: torch.Tensor, vcache: torch.Tensor, window: int, scale: float) -> torch.Tensor:
    _cuda(q, out, seq_of, pos, table, kcache, vcache)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * head_dim)
    call("gb_attention_generic", ptr(q), dtype_code(q), q.stride(0), ptr(out), dtype_code(out), out.stride(0), T,
         n_heads, n_kv_heads, head_dim, ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages, ptr(kcache),
         ptr(vcache), dtype_code(kcache), int(window or 0), float(scale), stream_ptr())
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gate_up: [T, 2F], gate in the first F columns; out[t,i] = silu(gate)*up."""
    _cuda(gate_up, out)
    T, F = out.shape
    assert gate_up.shape == (T, 2 * F) and gate_up.stride(1) == 1 and out.is_contiguous() and out.dtype == gate_up.dtype
    call("gb_swiglu", ptr(gate_up), gate_up.stride(0), ptr(out), T, F, dtype_code(out), stream_ptr())
    return out


def zero_rows(arena: torch.Tensor, table: torch.Tensor, slot: int) -> None:
    """Zeroes row `slot` of every region of a byte arena; table int64 [regions, 2] = (offset, bytes per row)."""
    _cuda(arena, table)
    assert arena.dtype == torch.uint8 and table.dtype == torch.int64 and table.is_contiguous()
    call("gb_zero_rows", ptr(arena), ptr(table), table.shape[0], int(slot), stream_ptr())


def gemm_generic(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[t,n] = sum_k x[t,k] w[n,k] + bias[n], 32-bit FMAs on the CUDA cores."""
    _cuda(x, w, bias, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    call("gb_gemm_generic", ptr(x), dtype_code(x), x.stride(0), ptr(w), dtype_code(w), w.stride(0), ptr(bias),
         0 if bias is None else dtype_code(bias), ptr(out), dtype_code(out), out.stride(0), T, N, K, stream_ptr())
    return out


def sample(logits: torch.Tensor, slots: torch.Tensor, seeds: torch.Tensor, temperature: float, top_k: int,
           top_p: float, rep_penalty: float, recent: torch.Tensor, count: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One token per row of float32 logits [n, V].  The logits are the kernel's scratch: the repetition
    penalty is applied to them in place, and with a temperature they are left divided by it.
    recent [slots, 64] and count [slots] are the sequences' own state."""
    _cuda(logits, slots, seeds, recent, count, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and seeds.dtype == torch.int64
    assert slots.dtype == torch.int32 and recent.dtype == torch.int32 and count.dtype == torch.int32
    assert recent.shape[1] == 64 and recent.is_contiguous() and out.dtype == torch.int32 and out.numel() >= n
    call("gb_sample", ptr(logits), logits.stride(0), n, V, ptr(slots), ptr(seeds), float(temperature), int(top_k),
         float(top_p), float(rep_penalty), ptr(recent), ptr(count), ptr(out), stream_ptr())
    return out


class _TcScratch:
    """Scratch of the kernels that split their work and merge it (the tensor-core product's K split,
    decode attention's page split), per device: partial results and arrival counters (zero between
    launches).  Launches on one stream follow one another, so they can share it.

    It is allocated once, at the most any launch can need, and never again: a captured CUDA graph
    holds its address, so a buffer that grew would leave every graph captured before pointing at
    freed memory.  The product needs at most one partial tile per resident CTA (two CTAs per SM with
    tiles of up to 64 tokens, one with wider tiles: 2 * sms * 64 * 128 floats), decode attention
    (head_dim + 2) floats per head and split with no more CTAs than two per SM.  A launch that would
    need more (only a tuning override can ask for it) runs without splitting instead."""
    COUNTERS = 4096

    def __init__(self, device):
        self.device = device
        self.sms = native.library().gb_sm_count()
        self.capacity = 2 * max(self.sms, 1) * 256 * 128
        self.floats = torch.empty(self.capacity, dtype=torch.float32, device=device)
        self.counters = torch.zeros(self.COUNTERS, dtype=torch.int32, device=device)

    def fits(self, n_floats: int) -> bool:
        return n_floats <= self.capacity


_tc_scratch = {}


def tc_scratch(device) -> _TcScratch:
    key = torch.device(device).index or 0
    if key not in _tc_scratch:
        _tc_scratch[key] = _TcScratch(device)
    return _tc_scratch[key]


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    return bool(native.library().gb_gemm_tc_supported(ptr(x), x.stride(0), ptr(w), w.stride(0), x.shape[1]))


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2*64*ceil(F/64), K]: row 2f is gate row f, row 2f+1 is up row f, zero rows padding F to
    a multiple of 64: the layout gemm_tc's gated epilogue reads."""
    F, K = gate.shape
    pad = (F + 63) // 64 * 64 - F
    if pad:
        zeros = torch.zeros(pad, K, dtype=gate.dtype, device=gate.device)
        gate, up = torch.cat([gate, zeros]), torch.cat([up, zeros])
    return torch.stack([gate, up], dim=1).reshape(2 * (F + pad), K).contiguous()


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor],
            split_k: bool = True, swiglu_features: int = 0, row_ssq: Optional[torch.Tensor] = None, ssq_parts: int = 0,
            norm_size: int = 0, eps: float = 0.0, resid_x: Optional[torch.Tensor] = None,
            resid_xb: Optional[torch.Tensor] = None, ssq_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """bf16 x bf16 -> f32 accumulate on tcgen05; out bf16 or f32.  Refuses what
    gemm_tc_supported refuses.  With swiglu_features = F, w is interleave_gate_up(gate, up)
    and out [T, F] = silu(x gate^T) * (x up^T).

    row_ssq [ssq_parts, T]: x holds rows whose RMS norm is deferred (its weight folded into w); each
    token's results are scaled by 1 / sqrt(sum_i row_ssq[i, t] / norm_size + eps).
    resid_x (f32 [T, N]): instead of writing `out`, resid_x += result in place, resid_xb gets the
    bfloat16 copy and ssq_out [ceil(N/128), T] the sums of squares per tile of 128 features."""
    _cuda(x, w, bias, out, row_ssq, resid_x, resid_xb, ssq_out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if resid_x is None:
        assert out.shape == (T, swiglu_features or N) and out.stride(1) == 1
    else:
        assert resid_x.shape == (T, N) and resid_x.dtype == torch.float32 and resid_x.stride(1) == 1
        assert resid_xb.shape == (T, N) and resid_xb.dtype == torch.bfloat16 and resid_xb.stride(0) == resid_x.stride(0)
        assert ssq_out.dtype == torch.float32 and ssq_out.numel() >= ((N + 127) // 128) * T
    if row_ssq is not None:
        assert row_ssq.dtype == torch.float32 and row_ssq.numel() >= ssq_parts * T and ssq_parts > 0
    sc = tc_scratch(x.device)
    scratch = counters = None
    if split_k:
        need = native.library().gb_gemm_tc_scratch_floats(T, N, K, sc.sms)
        if need and sc.fits(need):
            scratch, counters = sc.floats, sc.counters
    call("gb_gemm_tc_fused", ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias), 0 if bias is None else dtype_code(bias),
         ptr(out), 1 if out is None else dtype_code(out), 0 if out is None else out.stride(0), T, N, K, ptr(scratch),
         ptr(counters), 0 if counters is None else counters.numel(), sc.sms, int(swiglu_features), ptr(row_ssq),
         int(ssq_parts), int(norm_size), float(eps), ptr(resid_x), ptr(resid_xb), ptr(ssq_out),
         0 if resid_x is None else resid_x.stride(0), stream_ptr())
    return out


def attention_decode_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_decode_supported(head_dim, dtype_code(kcache), dtype_code(q)))


SPLIT_CLASSES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128)


def _split_class(n: int) -> int:
    return max(c for c in SPLIT_CLASSES if c <= max(n, 1))


def decode_split_class(max_kv: int) -> int:
    """The class of a step whose longest sequence has max_kv positions: a quarter of its pages, rounded down
    to one of a few values.  Steps of one class split their sequences' pages in the same way (decode_splits),
    and a captured graph is made per class."""
    return _split_class(((max_kv + 63) // 64) // 4)


def decode_splits(T: int, n_heads: int, n_kv_heads: int, max_kv: int, sms: int, mma: bool) -> int:
    """Splits of each sequence's pages for a decode step; a function of the step's class (decode_split_class)
    and its CTAs, so that all steps of a captured graph split alike.

    The tensor-core kernels split only while the step keeps to one CTA per SM, where the kernel of twelve warps
    runs (measured against the kernels of many CTAs with more splits at 8 to 16 sequences of 1,000 to 8,000
    positions: 17.5 instead of 21.1 us, 26.9 instead of 31.1, 14.8 instead of 20.5).  Few CTAs (a quarter of the
    SMs or fewer) are bound by what one SM can read and spread out: splits of at least 4 pages, at most 8 of them.
    More CTAs pay more for merging than they gain below about 12 pages per split.  Sequences of less than 16 pages
    are never split.  The CUDA-core kernel splits into 8 pages or more per split while all CTAs fit the device at
    once with two per SM."""
    group = n_heads // n_kv_heads
    tile = 16 if mma else (8 if group >= 8 else 4 if group > 2 else group)
    ctas = T * n_kv_heads * ((group + tile - 1) // tile)
    pages = (max_kv + 63) // 64
    if not mma:
        return max(1, min(_split_class(pages // 8), 32, (2 * sms) // ctas))
    cls = decode_split_class(max_kv)                       # a quarter of the pages, rounded down to a class
    if ctas > sms or cls < 4:
        return 1
    room = sms // ctas
    if 4 * ctas <= sms:
        return _split_class(min(room, 8, cls))
    return _split_class(min(room, cls // 3))


def attention_decode_mma_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_decode_mma_supported(head_dim, dtype_code(kcache), dtype_code(q)))


def attention_decode(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     seq_of: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, ring_pages: int,
                     kcache: torch.Tensor, vcache: torch.Tensor, window: int, scale: float,
                     splits: Optional[int] = None, mma: Optional[bool] = None, max_kv: Optional[int] = None,
                     rope: Optional[tuple] = None) -> torch.Tensor:
    """One token per sequence over the bf16 cache; all heads of a group share one pass over
    the keys and values.  mma: the tensor-core kernel (head sizes 64 and 128; the default
    where it fits) or the CUDA-core one (any head size that is a multiple of 16).
    rope = (k, v, inv_freq, rotary_dim, pairing), tensor-core kernel only: q, k and v are the
    unrotated projections; the kernel rotates q and k and writes k and v into the cache itself
    (k and v None: it reads another run's cache and only rotates q)."""
    _cuda(q, out, seq_of, pos, table, kcache, vcache)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * head_dim)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    lib = native.library()
    sc = tc_scratch(q.device)
    if mma is None:
        mma = attention_decode_mma_supported(q, kcache, head_dim)
    entry = "gb_attention_decode_mma" if mma else "gb_attention_decode"
    if splits is None:
        splits = decode_splits(T, n_heads, n_kv_heads, max_kv if max_kv else table.shape[1] * 64, sc.sms, mma)
    need = lib.gb_attention_decode_scratch_floats(T, n_heads, head_dim, splits)
    scratch = counters = None
    if need:
        scratch, counters = sc.floats, sc.counters
        if T * n_heads > sc.COUNTERS or not sc.fits(need):
            splits, scratch, counters = 1, None, None
    if rope is not None:
        k, v, inv_freq, rotary_dim, pairing = rope
        _cuda(k, v, inv_freq)
        assert mma and (k is None or (k.stride(0) == q.stride(0) and v.stride(0) == q.stride(0) and k.dtype == q.dtype))
        call("gb_attention_decode_mma_rope", ptr(q), ptr(k), ptr(v), q.stride(0), ptr(out), out.stride(0), T, n_heads,
             n_kv_heads, head_dim, rotary_dim, pairing, ptr(inv_freq), ptr(seq_of), ptr(pos), ptr(table), table.shape[1],
             ring_pages, ptr(kcache), ptr(vcache), int(window or 0), float(scale), splits, ptr(scratch), ptr(counters),
             0 if counters is None else counters.numel(), stream_ptr())
        return out
    call(entry, ptr(q), q.stride(0), ptr(out), out.stride(0), T, n_heads, n_kv_heads, head_dim,
         ptr(seq_of), ptr(pos), ptr(table), table.shape[1], ring_pages, ptr(kcache), ptr(vcache), int(window or 0),
         float(scale), splits, ptr(scratch), ptr(counters), 0 if counters is None else counters.numel(), stream_ptr())
    return out


def attention_prefill_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_prefill_supported(head_dim, dtype_code(kcache), dtype_code(q)))


def attention_prefill_tiles(qlens) -> list:
    """(sequence row, first query) of every tile of queries, flat, for the step's sequences."""
    bm = native.library().gb_attention_prefill_tile()
    tiles = [(b, q0) for b, n in enumerate(qlens) for q0 in range(0, n, bm)]
    # the later queries of a sequence see more keys: their tiles start first, so that the last CTAs to
    # start are the short ones (the order changes no result)
    tiles.sort(key=lambda t: -t[1])
    flat = []
    for b, q0 in tiles:
        flat += [b, q0]
    return flat


def attention_prefill_tc_supported(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    return bool(native.library().gb_attention_prefill_tc_supported(head_dim, dtype_code(kcache), dtype_code(q))) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0


def attention_prefill(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      tiles: torch.Tensor, cu: torch.Tensor, starts: torch.Tensor, qlens: torch.Tensor,
                      table: torch.Tensor, ring_pages: int, kcache: torch.Tensor, vcache: torch.Tensor, window: int,
                      scale: float, tc: Optional[bool] = None) -> torch.Tensor:
    """Many tokens per sequence over the bf16 cache (which already holds their keys and
    values), flash style.  tc: both products on tcgen05 with S and PV in TMEM (the default where it
    fits), else on mma.sync; both take head sizes 64 and 128."""
    _cuda(q, out, tiles, cu, starts, qlens, table, kcache, vcache)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (q.shape[0], n_heads * head_dim)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    if tc is None:
        tc = attention_prefill_tc_supported(q, kcache, head_dim)
    if tc:
        assert kcache.is_contiguous() and vcache.is_contiguous()
        call("gb_attention_prefill_tc", ptr(q), q.stride(0), ptr(out), out.stride(0), q.shape[0], n_heads, n_kv_heads,
             head_dim, ptr(tiles), tiles.numel() // 2, ptr(cu), ptr(starts), ptr(qlens), ptr(table), table.shape[1],
             ring_pages, ptr(kcache), ptr(vcache), kcache.shape[0], int(window or 0), float(scale), stream_ptr())
        return out
    call("gb_attention_prefill", ptr(q), q.stride(0), ptr(out), out.stride(0), n_heads, n_kv_heads, head_dim, ptr(tiles),
         tiles.numel() // 2, ptr(cu), ptr(starts), ptr(qlens), ptr(table), table.shape[1], ring_pages, ptr(kcache),
         ptr(vcache), int(window or 0), float(scale), stream_ptr())
    return out


def tc_status() -> int:
    """Non-zero when a bounded wait inside a tensor-core kernel gave up (read after a
    synchronise)."""
    return native.library().gb_tc_status()


def check_tc_status() -> None:
    lib = native.library()
    code = tc_status()
    if code:
        lib.gb_tc_status_clear()
        for sc in _tc_scratch.values():              # a kernel that gave up may have left a tile's counter half counted
            sc.counters.zero_()
        raise native.NativeError(f"a tensor-core product gave up waiting (code {code}: 1 a stage never came free, "
                                 f"2 a load never arrived, 3/4 an accumulator never completed, 5 a CTA that shares a tile never arrived); "
                                 f"its output is invalid")
    code = lib.gb_attention_tc_status()
    if code:
        lib.gb_attention_tc_status_clear()
        raise native.NativeError(f"the tensor-core attention kernel gave up waiting (code {code}); its output is invalid")


# ------------------------------------------------------------------ dispatch
def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """The product path of every projection: the tensor-core kernel when dtype and sizes
    fit it, else the CUDA-core kernel."""
    if gemm_tc_supported(x, w):
        return gemm_tc(x, w, bias, out)
    return gemm_generic(x, w, bias, out)


def decode_rotates(ctx, q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    """Whether this step's attention kernel rotates q and k and writes the cache itself (a step of single
    tokens on the tensor-core decode kernel), so that no separate rotation kernel runs before it."""
    return bool(ctx.decode) and attention_decode_supported(q, kcache, head_dim) and \
        attention_decode_mma_supported(q, kcache, head_dim)


def attention(q: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, ctx, table: torch.Tensor,
              ring_pages: int, kcache: torch.Tensor, vcache: torch.Tensor, window: int, scale: float,
              rope: Optional[tuple] = None, tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one step over the cache; picks the kernel for the step's shape.  rope: see
    attention_decode; allowed where decode_rotates() says so (q, k and v then come unrotated).
    tiles: attention_prefill_tiles() of the step's sequences on the device (prompts on the tiled kernels)."""
    if rope is not None:
        assert decode_rotates(ctx, q, kcache, head_dim)
    if ctx.decode and attention_decode_supported(q, kcache, head_dim):
        return attention_decode(q, out, n_heads, n_kv_heads, head_dim, ctx.seq_of, ctx.pos, table, ring_pages, kcache,
                                vcache, window, scale, max_kv=min(ctx.max_kv, window) if window else ctx.max_kv,
                                mma=True if rope is not None else None, rope=rope)
    if not ctx.decode and tiles is not None and attention_prefill_supported(q, kcache, head_dim):
        return attention_prefill(q, out, n_heads, n_kv_heads, head_dim, tiles, ctx.cu, ctx.starts, ctx.qlens, table,
                                 ring_pages, kcache, vcache, window, scale)
    return attention_generic(q, out, n_heads, n_kv_heads, head_dim, ctx.seq_of, ctx.pos, table, ring_pages, kcache,
                             vcache, window, scale)
