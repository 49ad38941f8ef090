"""Each kernel alone against its plain reference, at sizes other than the tiny models'."""
import math

import pytest
import torch

from tests import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF, F32 = torch.bfloat16, torch.float32


def K():
    from gguf_rs_cli_b200 import kernels
    return kernels


def rel_err(got, want):
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all()
    return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)


# ------------------------------------------------------------------ embedding
@pytest.mark.parametrize("dtype", [F32, BF])
def test_embed(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 200, generator=g).to(dtype)
    toks = torch.randint(0, 1000, (77,), generator=g)
    out = torch.empty(77, 200, dtype=F32, device=DEV)
    K().embed(table.to(DEV), toks.to(torch.int32).to(DEV), out)
    assert torch.equal(out.cpu(), P.embedding(table.float(), toks.tolist()))


# ----------------------------------------------------------------- norm + add
@pytest.mark.parametrize("E", [40, 320, 4096, 5000])
@pytest.mark.parametrize("dtype", [F32, BF])
def test_add_rmsnorm(E, dtype):
    g = torch.Generator().manual_seed(E)
    T, eps = 9, 3e-4
    x = torch.randn(T, E, generator=g) * 3
    w = (1 + 0.3 * torch.randn(E, generator=g)).to(dtype)
    d1 = torch.randn(T, E, generator=g).to(dtype)
    d3 = torch.randn(3, T, E, generator=g)
    tol = 1e-5 if dtype == F32 else 1e-2
    k = K()
    # no pending term
    xd, out = x.to(DEV).clone(), torch.empty(T, E, dtype=dtype, device=DEV)
    k.add_rmsnorm(xd, None, w.to(DEV), eps, out)
    assert rel_err(out, P.rmsnorm(x, w.float(), eps)) < tol and torch.equal(xd.cpu(), x)
    # one pending term of the working dtype: x is updated with the 32-bit sum
    k.add_rmsnorm(xd, d1.to(DEV), w.to(DEV), eps, out)
    assert rel_err(out, P.rmsnorm(x + d1.float(), w.float(), eps)) < tol
    assert torch.allclose(xd.cpu(), x + d1.float(), atol=1e-6)
    # several 32-bit partial sums, gathered rows, x untouched
    xd = x.to(DEV).clone()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, E, dtype=dtype, device=DEV)
    k.add_rmsnorm(xd, d3.to(DEV), w.to(DEV), eps, out3, rows=rows, write_x=False)
    want = P.rmsnorm((x + d3.sum(0))[[7, 0, 3]], w.float(), eps)
    assert rel_err(out3, want) < tol and torch.equal(xd.cpu(), x)


# --------------------------------------------------------------------- swiglu
@pytest.mark.parametrize("dtype", [F32, BF])
def test_swiglu(dtype):
    g = torch.Generator().manual_seed(1)
    gu = (torch.randn(13, 2 * 520, generator=g) * 4).to(dtype)
    out = torch.empty(13, 520, dtype=dtype, device=DEV)
    K().swiglu(gu.to(DEV), out)
    want = P.silu(gu.float()[:, :520]) * gu.float()[:, 520:]
    assert rel_err(out, want) < (1e-6 if dtype == F32 else 5e-3)


# ---------------------------------------------------------------------- gemms
SHAPES = [(1, 100, 72), (5, 257, 136), (70, 130, 1000), (129, 64, 24), (33, 300, 200)]


@pytest.mark.parametrize("T,N,Kd", SHAPES)
@pytest.mark.parametrize("xdt,wdt", [(F32, F32), (BF, BF), (BF, F32)])
def test_gemm_generic(T, N, Kd, xdt, wdt):
    g = torch.Generator().manual_seed(T * N)
    x, w = torch.randn(T, Kd, generator=g).to(xdt), (torch.randn(N, Kd, generator=g) * 0.1).to(wdt)
    b = torch.randn(N, generator=g)
    out = torch.empty(T, N, dtype=F32, device=DEV)
    K().gemm_generic(x.to(DEV), w.to(DEV), b.to(DEV), out)
    assert rel_err(out, P.linear(x.double(), w.double(), b.double())) < 2e-6
    outb = torch.empty(T, N + 3, dtype=xdt, device=DEV)[:, :N]               # a strided output
    K().gemm_generic(x.to(DEV), w.to(DEV), None, outb)
    assert rel_err(outb, P.linear(x.double(), w.double())) < (2e-6 if xdt == F32 else 5e-3)


def test_gemm_generic_rows_do_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(70, 200, generator=g).to(DEV), torch.randn(90, 200, generator=g).to(DEV)
    whole = torch.empty(70, 90, device=DEV)
    one = torch.empty(1, 90, device=DEV)
    K().gemm_generic(x, w, None, whole)
    K().gemm_generic(x[41:42], w, None, one)
    assert torch.equal(whole[41], one[0])


TC_SHAPES = [(1, 256, 512), (8, 128, 64), (16, 1000, 4096), (33, 300, 200), (64, 520, 320), (100, 136, 72),
             (129, 6144, 1024), (300, 520, 4096), (700, 257, 328)]


@pytest.mark.parametrize("T,N,Kd", TC_SHAPES + [(3, 40, 72), (9, 1000, 328), (16, 6144, 4096), (2, 130, 6144)])
@pytest.mark.parametrize("out_dtype", [F32, BF])
def test_gemm_tensor_core(T, N, Kd, out_dtype):
    k = K()
    g = torch.Generator().manual_seed(T + N + Kd)
    x = torch.randn(T, Kd, generator=g).to(BF).to(DEV)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(BF).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    assert k.gemm_tc_supported(x, w)
    want = P.linear(x.double().cpu(), w.double().cpu(), b.double().cpu())
    out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
    k.gemm_tc(x, w, b, out)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < (1e-5 if out_dtype == F32 else 5e-3)
    # the generic kernel is its twin
    twin = torch.empty(T, N, dtype=F32, device=DEV)
    k.gemm_generic(x, w, b, twin)
    assert rel_err(twin, want) < 1e-5
    # with whole tiles only (no scratch memory) the result is the same up to the order of the 32-bit sums
    nosplit = torch.empty(T, N, dtype=F32, device=DEV)
    k.gemm_tc(x, w, b, nosplit, split_k=False)
    assert rel_err(nosplit, want) < 1e-5
    # and twice in a row gives the same bits (the split's counters are left at zero)
    again = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
    k.gemm_tc(x, w, b, again)
    assert torch.equal(again, out)


def test_gemm_tensor_core_refuses_what_it_cannot_take():
    k = K()
    x = torch.zeros(4, 100, dtype=BF, device=DEV)
    w = torch.zeros(8, 100, dtype=BF, device=DEV)
    assert not k.gemm_tc_supported(x, w)                        # K = 100 is no multiple of 8
    assert not k.gemm_tc_supported(x.float(), w.float())
    from gguf_rs_cli_b200.native import NativeError
    with pytest.raises(NativeError, match="multiples of 8"):
        k.gemm_tc(x, w, None, torch.empty(4, 8, dtype=BF, device=DEV))
    out = torch.empty(4, 8, dtype=BF, device=DEV)
    k.gemm(x, w, None, out)                                     # the dispatcher takes the other kernel
    assert torch.equal(out.cpu(), torch.zeros(4, 8, dtype=BF))


# ------------------------------------------------- rotation, cache, attention
def make_cache(n_pages, nkv, hd, dtype):
    return (torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype, device=DEV),
            torch.full((n_pages, nkv, 64, hd), float("nan"), dtype=dtype, device=DEV))


def page_layout(lens, n_pages, seed=0):
    """A scattered page table for sequences of these lengths."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max((n + 63) // 64 for n in lens)
    rows, nxt = [], 0
    for n in lens:
        k = (n + 63) // 64
        rows.append(perm[nxt:nxt + k] + [0] * (width - k))
        nxt += k
    return torch.tensor(rows, dtype=torch.int32, device=DEV)


def read_cache(cache, table_row, n):
    out = []
    for p in range(n):
        out.append(cache[int(table_row[p // 64]), :, p % 64, :])
    return torch.stack(out).float().cpu()          # [n, nkv, hd]


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("nh,nkv,hd,rot,pairing", [(6, 3, 32, 32, 0), (4, 1, 48, 48, 0), (8, 8, 16, 8, 0), (2, 2, 64, 64, 1)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, rot, pairing):
    k = K()
    g = torch.Generator().manual_seed(nh * hd)
    lens, starts = [70, 5, 130], [3, 0, 64]                # new tokens and where each sequence stands
    T = sum(lens)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, generator=g).to(dtype)
    cfg = {"hidden_size": nh * rot, "num_attention_heads": nh, "head_dim": rot, "rope_theta": 50000.0}
    inv = P.inv_freq_table(cfg)
    seq_of = torch.tensor(sum(([b] * n for b, n in enumerate(lens)), []), dtype=torch.int32)
    pos = torch.tensor(sum((list(range(s, s + n)) for s, n in zip(starts, lens)), []), dtype=torch.int32)
    table = page_layout([s + n for s, n in zip(starts, lens)], 16)
    kc, vc = make_cache(16, nkv, hd, dtype)
    d = qkv.to(DEV).clone()
    q, kk, vv = d[:, :nh * hd], d[:, nh * hd:(nh + nkv) * hd], d[:, (nh + nkv) * hd:]
    k.rope_kv_write(q, kk, vv, nh, nkv, hd, inv.to(DEV), rot, pairing, seq_of.to(DEV), pos.to(DEV), table, 1 << 20, kc, vc)

    def plain_rot(x, heads):
        x = x.float().reshape(T, heads, hd)
        r = x[..., :rot]
        if pairing:
            r = torch.cat([r[..., 0::2], r[..., 1::2]], -1)
        r = P.rope(r, pos, inv)
        if pairing:
            out = torch.empty_like(r)
            out[..., 0::2], out[..., 1::2] = r[..., :rot // 2], r[..., rot // 2:]
            r = out
        return torch.cat([r, x[..., rot:]], -1)

    tol = 1e-5 if dtype == F32 else 1e-2
    assert rel_err(q.reshape(T, nh, hd), plain_rot(qkv[:, :nh * hd], nh)) < tol
    want_k, want_v = plain_rot(qkv[:, nh * hd:(nh + nkv) * hd], nkv), qkv[:, (nh + nkv) * hd:].float().reshape(T, nkv, hd)
    t0 = 0
    for b, (s, n) in enumerate(zip(starts, lens)):
        got_k, got_v = read_cache(kc, table[b].cpu(), s + n)[s:], read_cache(vc, table[b].cpu(), s + n)[s:]
        assert rel_err(got_k, want_k[t0:t0 + n]) < tol, f"keys of sequence {b}"
        assert torch.equal(got_v, want_v[t0:t0 + n].to(dtype).float()), f"values of sequence {b}"
        t0 += n
    # nothing else was written: pages not in the tables are still untouched
    used = set(table.cpu().flatten().tolist())
    for pg in range(16):
        if pg not in used:
            assert torch.isnan(kc[pg].float()).all()


def fill_cache(kseqs, vseqs, nkv, hd, dtype, n_pages=64, seed=0):
    lens = [k.shape[0] for k in kseqs]
    n_pages = max(n_pages, sum((n + 63) // 64 for n in lens) + 3)
    table = page_layout(lens, n_pages, seed)
    kc, vc = make_cache(n_pages, nkv, hd, dtype)
    rows = table.tolist()
    for b, (ks, vs) in enumerate(zip(kseqs, vseqs)):
        for first in range(0, ks.shape[0], 64):
            pg, cnt = rows[b][first // 64], min(64, ks.shape[0] - first)
            kc[pg, :, :cnt, :] = ks[first:first + cnt].transpose(0, 1).to(dtype).to(DEV)
            vc[pg, :, :cnt, :] = vs[first:first + cnt].transpose(0, 1).to(dtype).to(DEV)
    return table, kc, vc


def last_query_attention(q, k, v, window=None):
    """P.attention's last row alone (a decode step's query), for long sequences: q [n, nh, hd], k, v [n, nkv, hd]."""
    n, nh, hd = q.shape
    ratio = nh // k.shape[1]
    lo = max(0, n - window) if window else 0
    out = torch.zeros(nh, hd)
    for h in range(nh):
        s = (k[lo:, h // ratio, :] @ q[-1, h, :]) / math.sqrt(hd)
        out[h] = P.softmax(s[None, :])[0] @ v[lo:, h // ratio, :]
    return out.reshape(1, nh * hd)


def attention_case(nh, nkv, hd, lens, qlens, dtype, seed, window=None, boost=None):
    """Random q/k/v for sequences of `lens`, the last qlens[b] positions being this step's
    queries.  boost=(b, key position, head): that query/key pair gets a large score."""
    g = torch.Generator().manual_seed(seed)
    qs = [torch.randn(n, nh, hd, generator=g) for n in lens]
    ks = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    if boost:
        b, kp, h = boost
        ks[b][kp, h // (nh // nkv)] = qs[b][-1, h] * 3.0        # the last query finds this far key
    qs = [x.to(dtype).float() for x in qs]
    ks = [x.to(dtype).float() for x in ks]
    vs = [x.to(dtype).float() for x in vs]
    want = torch.cat([last_query_attention(q, k, v, window) if ql == 1 and n > 300 else P.attention(q, k, v, window=window)[n - ql:]
                      for q, k, v, n, ql in zip(qs, ks, vs, lens, qlens)])
    q = torch.cat([q[n - ql:] for q, n, ql in zip(qs, lens, qlens)]).reshape(-1, nh * hd).to(dtype).to(DEV)
    seq_of = torch.tensor(sum(([b] * ql for b, ql in enumerate(qlens)), []), dtype=torch.int32, device=DEV)
    pos = torch.tensor(sum((list(range(n - ql, n)) for n, ql in zip(lens, qlens)), []), dtype=torch.int32, device=DEV)
    table, kc, vc = fill_cache(ks, vs, nkv, hd, dtype, seed=seed)
    return q, seq_of, pos, table, kc, vc, want


ATT_SHAPES = [(6, 3, 32), (4, 1, 48), (8, 8, 16), (8, 2, 128), (5, 5, 80)]


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("nh,nkv,hd", ATT_SHAPES)
def test_attention_generic(dtype, nh, nkv, hd):
    k = K()
    lens, qlens = [200, 1, 65, 130], [200, 1, 1, 40]           # whole prompt, first token, decode, continuation
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, dtype, seed=hd)
    out = torch.empty(q.shape[0], nh * hd, dtype=dtype, device=DEV)
    k.attention_generic(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd))
    assert rel_err(out, want) < (2e-5 if dtype == F32 else 1e-2)


@pytest.mark.parametrize("dtype", [F32, BF])
def test_attention_generic_finds_a_far_key_and_respects_a_window(dtype):
    k = K()
    nh, nkv, hd = 4, 2, 32
    lens, qlens = [700, 300], [1, 1]
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, dtype, 5, boost=(0, 3, 2))
    out = torch.empty(2, nh * hd, dtype=dtype, device=DEV)
    k.attention_generic(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd))
    assert rel_err(out, want) < (2e-5 if dtype == F32 else 1e-2)
    # the boosted head's output is (nearly) the far key's value: a kernel that skipped position 3 fails
    q2, seq_of, pos, table, kc, vc, want_w = attention_case(nh, nkv, hd, lens, qlens, dtype, 5, window=100, boost=(0, 3, 2))
    k.attention_generic(q2, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 100, 1 / math.sqrt(hd))
    assert rel_err(out, want_w) < (2e-5 if dtype == F32 else 1e-2)
    assert rel_err(want_w, want) > 0.05                        # the window hides the far key
    # window edge: exactly W keys are seen
    for W in (1, 64, 65):
        _, _, _, _, _, _, ww = attention_case(nh, nkv, hd, lens, qlens, dtype, 5, window=W)
        k.attention_generic(q2, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, W, 1 / math.sqrt(hd))
        assert rel_err(out, ww) < (2e-5 if dtype == F32 else 1e-2), f"window {W}"


def test_attention_padding_tokens_give_zeros():
    k = K()
    nh, nkv, hd = 4, 2, 32
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, [70, 3], [1, 1], F32, 9)
    q = torch.cat([q, torch.randn(2, nh * hd, device=DEV)])
    seq_of = torch.cat([seq_of, torch.tensor([-1, -1], dtype=torch.int32, device=DEV)])
    pos = torch.cat([pos, torch.zeros(2, dtype=torch.int32, device=DEV)])
    out = torch.full((4, nh * hd), float("nan"), device=DEV)
    k.attention_generic(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd))
    assert rel_err(out[:2], want) < 2e-5 and torch.equal(out[2:].cpu(), torch.zeros(2, nh * hd))


# ------------------------------------------------------------------- sampling
def run_sample(logits, slots, keys, temperature, top_k, top_p, rep, recent, count):
    n = logits.shape[0]
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    K().sample(logits, slots, keys, temperature, top_k, top_p, rep, recent, count, out)
    return out.cpu().tolist()


@pytest.mark.parametrize("V", [384, 5003, 128256])
def test_sampling_matches_the_plain_sampler(V):
    from gguf_rs_cli_b200.sampling import stream_key
    g = torch.Generator().manual_seed(V)
    n_slots = 8
    slots = [6, 0, 3, 7, 2]
    settings = [(0.0, 0, 1.0, 1.0), (0.8, 0, 1.0, 1.0), (1.3, 40, 1.0, 1.0), (0.7, 0, 0.9, 1.0), (0.7, 40, 0.9, 1.1),
                (1.0, 3, 0.5, 1.3), (2.0, V + 5, 0.99, 1.0)]
    steps = 4
    if V > 100000:                                  # the plain sampler sorts in Python: keep the big case short
        slots, settings, steps = slots[:2], [settings[1], settings[4]], 2
    n = len(slots)
    for temperature, top_k, top_p, rep in settings:
        recent = torch.zeros(n_slots, 64, dtype=torch.int32, device=DEV)
        count = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
        hist = {s: [] for s in slots}
        keys = [stream_key(11, i) for i in range(n)]
        for step in range(steps):
            logits = (torch.randn(n, V, generator=g) * 3).to(DEV)
            logits[0, 5] = logits[0, 17] = logits[0].max() + 1           # equal maxima: the lower index wins
            ref = logits.cpu().clone()
            got = run_sample(logits, torch.tensor(slots, dtype=torch.int32, device=DEV),
                             torch.tensor(keys, dtype=torch.int64, device=DEV), temperature, top_k, top_p, rep, recent, count)
            for i, s in enumerate(slots):
                u = P.uniform(keys[i] & P.MASK64, len(hist[s]))
                want = P.sample(ref[i], temperature, top_k, top_p, rep, hist[s][-64:], u)
                assert got[i] == want, f"V={V} T={temperature} k={top_k} p={top_p} rep={rep} step {step} row {i}"
                hist[s].append(got[i])
        assert count.cpu().tolist() == [steps if s in slots else 0 for s in range(n_slots)]


@pytest.mark.parametrize("V", [50, 1000, 4099, 33001])
def test_sampling_with_many_equal_logits(V):
    """Logits that take few distinct values: the k-th largest and the edge of the nucleus fall among equal
    values, of which the lower indices are taken.  top_k from 1 to beyond the list the kernel keeps in shared
    memory, with and without top_p."""
    from gguf_rs_cli_b200.sampling import stream_key
    g = torch.Generator().manual_seed(V)
    n, n_slots = 4, 4
    slots = list(range(n))
    settings = [(1.0, 1, 1.0), (0.9, 7, 1.0), (1.1, 40, 0.8), (0.7, min(V - 1, 1024), 0.95), (1.0, min(V - 1, 1030), 0.9),
                (1.0, min(V - 1, 2000), 1.0), (1.5, 0, 1.0), (0.8, 0, 0.6), (1.0, 33, 0.05)]
    steps = 3
    all_levels = (2, 5, 64)
    if V > 30000:                                   # several CTAs share a row from here on; the plain sampler sorts in Python
        n, all_levels, steps = 2, (5,), 1
        slots = slots[:n]
    for levels in all_levels:
        for temperature, top_k, top_p in settings:
            recent = torch.zeros(n_slots, 64, dtype=torch.int32, device=DEV)
            count = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
            keys = [stream_key(5, i) for i in range(n)]
            for step in range(steps):
                logits = (torch.randint(0, levels, (n, V), generator=g).float() * (6.0 / levels) - 2.0).to(DEV)
                ref = logits.cpu()
                got = run_sample(logits, torch.tensor(slots, dtype=torch.int32, device=DEV),
                                 torch.tensor(keys, dtype=torch.int64, device=DEV), temperature, top_k, top_p, 1.0, recent, count)
                for r in range(n):
                    want = P.sample(ref[r], temperature, top_k, top_p, 1.0, [], P.uniform(keys[r] & P.MASK64, step))
                    assert got[r] == want, f"V {V} levels {levels} T {temperature} k {top_k} p {top_p} step {step} row {r}"


def test_sampling_ring_and_padding():
    V, n_slots = 50, 2
    recent = torch.zeros(n_slots, 64, dtype=torch.int32, device=DEV)
    count = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    slots = torch.tensor([1, -1], dtype=torch.int32, device=DEV)
    keys = torch.zeros(2, dtype=torch.int64, device=DEV)
    seen = []
    for step in range(70):
        logits = torch.zeros(2, V, device=DEV)
        logits[0, step % V] = 5.0
        seen.append(run_sample(logits, slots, keys, 0.0, 0, 1.0, 1.0, recent, count)[0])
    assert seen == [s % V for s in range(70)]
    assert count.cpu().tolist() == [0, 70]
    ring = recent[1].cpu().tolist()
    assert sorted(ring) == sorted(seen[-64:]) and recent[0].abs().sum() == 0
    # the penalty is applied once per occurrence and turns the choice
    logits = torch.zeros(1, V, device=DEV)
    logits[0, 19], logits[0, 40] = 5.0, 2.0                          # 19 is in the ring twice (5/2/2 < 2/2 fails: 1.25 > 1)
    logits[0, 45] = 1.2                                              # 45 is in the ring once: 0.6
    ref = logits.cpu()[0].clone()
    got = run_sample(logits, torch.tensor([1], dtype=torch.int32, device=DEV), keys[:1], 0.0, 0, 1.0, 2.0, recent, count)[0]
    want = P.sample(ref, 0.0, 0, 1.0, 2.0, seen[-64:], 0.0)
    assert got == want == 19 and seen[-64:].count(19) == 2 and seen[-64:].count(40) == 1


# ----------------------------------------------------------- decode attention
class TwoWarpShape:
    """mma == "two": the tensor-core decode kernel in its shape of two warps and half pages (heads of 128), which
    the library takes by itself only for steps of several hundred CTAs."""

    def __init__(self, mma, hd):
        self.on = mma == "two"
        if self.on and hd != 128:
            pytest.skip("CTAs of two warps are for heads of 128")

    def __enter__(self):
        from gguf_rs_cli_b200 import native
        if self.on:
            native.call("gb_attention_decode_set_two_warps", 2)

    def __exit__(self, *a):
        from gguf_rs_cli_b200 import native
        native.call("gb_attention_decode_set_two_warps", 1)


@pytest.mark.parametrize("nh,nkv,hd", [(6, 3, 32), (4, 1, 48), (8, 8, 16), (8, 2, 128), (5, 5, 80), (16, 1, 64),
                                       (12, 2, 256), (3, 1, 112), (40, 2, 64), (32, 8, 128), (7, 7, 128)])
@pytest.mark.parametrize("splits", [None, 1, 3, 7])
@pytest.mark.parametrize("mma", [False, True, "two"])
def test_attention_decode(nh, nkv, hd, splits, mma):
    if mma and hd not in (64, 128):
        pytest.skip("the tensor-core decode kernel takes head sizes 64 and 128")
    with TwoWarpShape(mma, hd):
        _attention_decode(nh, nkv, hd, splits, bool(mma))


def _attention_decode(nh, nkv, hd, splits, mma):
    k = K()
    lens = [200, 1, 65, 130, 64, 513]
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, [1] * len(lens), BF, seed=hd + nh)
    # two padding tokens in the middle of the batch
    T = len(lens) + 2
    order = [0, 1, -1, 2, 3, -1, 4, 5]
    qp = torch.randn(T, nh * hd, device=DEV).to(BF)
    sp = torch.full((T,), -1, dtype=torch.int32, device=DEV)
    pp = torch.zeros(T, dtype=torch.int32, device=DEV)
    rows = [i for i, o in enumerate(order) if o >= 0]
    qp[rows], sp[rows], pp[rows] = q, seq_of, pos
    out = torch.full((T, nh * hd), float("nan"), dtype=BF, device=DEV)
    assert k.attention_decode_supported(qp, kc, hd)
    k.attention_decode(qp, out, nh, nkv, hd, sp, pp, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), splits=splits, mma=mma)
    assert rel_err(out[rows], want) < 1e-2
    assert torch.equal(out[[2, 5]].float().cpu(), torch.zeros(2, nh * hd))
    twin = torch.empty(T, nh * hd, dtype=BF, device=DEV)
    k.attention_generic(qp, twin, nh, nkv, hd, sp, pp, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd))
    assert rel_err(out[rows], twin[rows]) < 1e-2
    again = torch.full((T, nh * hd), float("nan"), dtype=BF, device=DEV)
    k.attention_decode(qp, again, nh, nkv, hd, sp, pp, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), splits=splits, mma=mma)
    assert torch.equal(again, out)                 # counters were left at zero; the merge order is fixed


@pytest.mark.parametrize("window", [1, 31, 64, 65, 100, 300])
@pytest.mark.parametrize("mma,hd", [(False, 64), (True, 64), (True, 128), ("two", 128)])
def test_attention_decode_far_key_and_window(window, mma, hd):
    with TwoWarpShape(mma, hd):
        _far_key_and_window(window, bool(mma), hd)


def _far_key_and_window(window, mma, hd):
    k = K()
    nh, nkv = 8, 2
    lens = [700, 300, 50]
    scale = 1 / math.sqrt(hd)
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, [1, 1, 1], BF, 5, boost=(0, 3, 2))
    out = torch.empty(3, nh * hd, dtype=BF, device=DEV)
    k.attention_decode(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, scale, mma=mma)
    assert rel_err(out, want) < 1e-2               # the far key at position 3 dominates head 2 of sequence 0
    _, _, _, _, _, _, want_w = attention_case(nh, nkv, hd, lens, [1, 1, 1], BF, 5, window=window, boost=(0, 3, 2))
    for splits in (None, 1, 5):
        k.attention_decode(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, window, scale, splits=splits, mma=mma)
        assert rel_err(out, want_w) < 1e-2, f"window {window} splits {splits}"
    assert rel_err(want_w, want) > 0.05


@pytest.mark.parametrize("splits", [None, 16, 48])
@pytest.mark.parametrize("hd", [64, 128])
def test_attention_decode_few_long_sequences_in_many_splits(splits, hd):
    """Two sequences, one of them long: one CTA per SM takes a few pages each (more splits than the short
    sequence has pages: some CTAs get none), and a key far back in the long one carries a head."""
    k = K()
    nh, nkv = 8, 2
    lens = [2100, 130]
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, [1, 1], BF, 11, boost=(0, 77, 3))
    out = torch.full((2, nh * hd), float("nan"), dtype=BF, device=DEV)
    k.attention_decode(q, out, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), splits=splits, mma=True,
                       max_kv=max(lens))
    assert rel_err(out, want) < 1e-2
    v_key = read_cache(vc, table[0], lens[0])[77, 3 // (nh // nkv)]
    got = out[0, 3 * hd:4 * hd].float().cpu()
    assert float((got - v_key).abs().max()) < 0.05 * float(v_key.abs().max())
    assert k.decode_splits(2, nh, nkv, max(lens), 148, True) == 8 and k.decode_splits(64, nh, nkv, max(lens), 148, True) == 1


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (40, 2, 64), (7, 7, 128), (16, 1, 64)])
@pytest.mark.parametrize("pairing,rot", [(0, 1.0), (1, 1.0), (0, 0.5), (0, 0.0)])
@pytest.mark.parametrize("own_kv", [True, False])
@pytest.mark.parametrize("mma", [True, "two"])
def test_attention_decode_rotating(nh, nkv, hd, pairing, rot, own_kv, mma):
    with TwoWarpShape(mma, hd):
        _attention_decode_rotating(nh, nkv, hd, pairing, rot, own_kv)


def _attention_decode_rotating(nh, nkv, hd, pairing, rot, own_kv):
    """The decode kernel that rotates q and k and writes the cache itself gives, bit for bit, the output and
    the cache of the rotation kernel followed by the plain decode kernel: whole and split pages, a window,
    groups of more than 16 heads (two CTAs share the token's own key), padding tokens, positions that open
    a page (64) or half a page (32, 96) and positions that end one (191, 31)."""
    k = K()
    lens = [200, 1, 65, 130, 64, 513, 192, 33, 32, 97]
    _, seq_of, pos, table, kc, vc, _ = attention_case(nh, nkv, hd, lens, [1] * len(lens), BF, seed=3 * hd + nh)
    T = len(lens) + 1
    rows = [i for i in range(T) if i != 3]
    sp = torch.full((T,), -1, dtype=torch.int32, device=DEV)
    pp = torch.zeros(T, dtype=torch.int32, device=DEV)
    sp[rows], pp[rows] = seq_of, pos
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, generator=torch.Generator().manual_seed(nh + hd + pairing)).to(DEV).to(BF)
    rotary_dim = int(hd * rot)
    inv_freq = None
    if rotary_dim:
        inv_freq = (10000.0 ** (-torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim)).to(DEV)
    scale = 1 / math.sqrt(hd)
    for window, splits in ((0, None), (0, 1), (0, 3), (100, None), (70, 2)):
        got = []
        for fused in (False, True):
            x, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
            q, kn, vn = x[:, :nh * hd], x[:, nh * hd:(nh + nkv) * hd], x[:, (nh + nkv) * hd:]
            if not own_kv:
                kn = vn = None
            out = torch.full((T, nh * hd), float("nan"), dtype=BF, device=DEV)
            if fused:
                k.attention_decode(q, out, nh, nkv, hd, sp, pp, table, 1 << 20, kc2, vc2, window, scale, splits=splits,
                                   mma=True, rope=(kn, vn, inv_freq, rotary_dim, pairing))
                assert torch.equal(x, qkv)                       # the projections are left as they were
            else:
                k.rope_kv_write(q, kn, vn, nh, nkv, hd, inv_freq, rotary_dim, pairing, sp, pp, table if own_kv else None,
                                1 << 20, kc2 if own_kv else None, vc2 if own_kv else None)
                k.attention_decode(q, out, nh, nkv, hd, sp, pp, table, 1 << 20, kc2, vc2, window, scale, splits=splits, mma=True)
            got.append((out, kc2, vc2))
        (a, ka, va), (b, kb, vb) = got
        assert torch.equal(a, b), f"window {window} splits {splits}: outputs differ by {(a.float() - b.float()).abs().max()}"
        bits = lambda x: x.view(torch.int16)                     # unused rows of the cache hold NaNs
        for name, u, w in (("k", ka, kb), ("v", va, vb)):
            diff = (bits(u) != bits(w)).nonzero()
            assert diff.numel() == 0, f"window {window} splits {splits}: {name} caches differ at {diff[:8].tolist()} of {tuple(u.shape)}"
        assert own_kv == (not torch.equal(bits(ka), bits(kc)))


# ---------------------------------------------------------- prefill attention
def prefill_meta(lens, qlens):
    k = K()
    starts = [n - ql for n, ql in zip(lens, qlens)]
    cu = [0]
    for ql in qlens:
        cu.append(cu[-1] + ql)
    ti = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return ti(k.attention_prefill_tiles(qlens)), ti(cu), ti(starts), ti(qlens)


@pytest.mark.parametrize("nh,nkv,hd", [(6, 3, 64), (4, 1, 128), (8, 8, 64), (8, 2, 128), (5, 5, 128)])
@pytest.mark.parametrize("tc", [False, True])
def test_attention_prefill(nh, nkv, hd, tc):
    k = K()
    lens, qlens = [200, 1, 65, 130, 300, 513], [200, 1, 3, 40, 129, 513]   # whole prompts and further pieces
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, BF, seed=hd + nh)
    tiles, cu, starts, ql = prefill_meta(lens, qlens)
    out = torch.full((q.shape[0], nh * hd), float("nan"), dtype=BF, device=DEV)
    assert k.attention_prefill_supported(q, kc, hd)
    k.attention_prefill(q, out, nh, nkv, hd, tiles, cu, starts, ql, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), tc=tc)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < 1e-2
    twin = torch.empty_like(out)
    k.attention_generic(q, twin, nh, nkv, hd, seq_of, pos, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd))
    assert rel_err(out, twin) < 1e-2


@pytest.mark.parametrize("window", [1, 64, 65, 100, 300])
@pytest.mark.parametrize("hd,tc", [(64, False), (128, False), (64, True), (128, True)])
def test_attention_prefill_far_key_and_window(window, hd, tc):
    k = K()
    nh, nkv = 8, 2
    lens, qlens = [700, 300], [700, 150]
    scale = 1 / math.sqrt(hd)
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, BF, 5, boost=(0, 3, 2))
    tiles, cu, starts, ql = prefill_meta(lens, qlens)
    out = torch.empty(q.shape[0], nh * hd, dtype=BF, device=DEV)
    k.attention_prefill(q, out, nh, nkv, hd, tiles, cu, starts, ql, table, 1 << 20, kc, vc, 0, scale, tc=tc)
    assert rel_err(out, want) < 1e-2
    _, _, _, _, _, _, want_w = attention_case(nh, nkv, hd, lens, qlens, BF, 5, window=window, boost=(0, 3, 2))
    k.attention_prefill(q, out, nh, nkv, hd, tiles, cu, starts, ql, table, 1 << 20, kc, vc, window, scale, tc=tc)
    assert rel_err(out, want_w) < 1e-2, f"window {window}"
    assert rel_err(want_w, want) > 0.05


@pytest.mark.parametrize("key", [3, 70, 200, 449, 650])
@pytest.mark.parametrize("hd,tc", [(128, False), (64, True), (128, True)])
def test_attention_prefill_score_that_stands_out_anywhere_in_a_block(key, hd, tc):
    """One key whose score with the last query towers over the rest, placed in the first or second half of the
    first or a later block of 128 keys: the running maximum then jumps in the middle of a block, after sums,
    outputs and probabilities have been gathered relative to the old one."""
    k = K()
    nh, nkv = 8, 2
    lens, qlens = [700, 300], [700, 150]
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, BF, 9, boost=(0, key, 5))
    tiles, cu, starts, ql = prefill_meta(lens, qlens)
    out = torch.empty(q.shape[0], nh * hd, dtype=BF, device=DEV)
    k.attention_prefill(q, out, nh, nkv, hd, tiles, cu, starts, ql, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), tc=tc)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < 1e-2
    # the last query's head 5 is (nearly) that key's value
    v_key = read_cache(vc, table[0], 700)[key, 5 // (nh // nkv)]
    got = out[699, 5 * hd:6 * hd].float().cpu()
    assert float((got - v_key).abs().max()) < 0.05 * float(v_key.abs().max())


@pytest.mark.parametrize("hd,tc", [(128, False), (64, True), (128, True)])
def test_attention_prefill_ignores_unwritten_cache_rows(hd, tc):
    """Rows of a page beyond the sequence's end hold NaN here; they must not reach the output."""
    k = K()
    nh, nkv = 4, 2
    lens = qlens = [70]
    q, seq_of, pos, table, kc, vc, want = attention_case(nh, nkv, hd, lens, qlens, BF, 1)
    assert torch.isnan(kc[int(table[0, 1]), :, 10:, :].float()).all()
    tiles, cu, starts, ql = prefill_meta(lens, qlens)
    out = torch.empty(70, nh * hd, dtype=BF, device=DEV)
    k.attention_prefill(q, out, nh, nkv, hd, tiles, cu, starts, ql, table, 1 << 20, kc, vc, 0, 1 / math.sqrt(hd), tc=tc)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < 1e-2


# ------------------------------------------------- gated product (fused SwiGLU)
@pytest.mark.parametrize("T,F,Kd", [(1, 176, 64), (8, 520, 320), (16, 1024, 4096), (64, 200, 2048), (130, 520, 328),
                                    (300, 14336 // 8, 512)])
def test_gemm_tensor_core_gated(T, F, Kd):
    k = K()
    g = torch.Generator().manual_seed(T + F)
    x = torch.randn(T, Kd, generator=g).to(BF).to(DEV)
    wg = (torch.randn(F, Kd, generator=g) * 0.1).to(BF).to(DEV)
    wu = (torch.randn(F, Kd, generator=g) * 0.1).to(BF).to(DEV)
    w = k.interleave_gate_up(wg, wu)
    assert w.shape == (128 * ((F + 63) // 64), Kd)
    want = P.silu(P.linear(x.double().cpu(), wg.double().cpu())) * P.linear(x.double().cpu(), wu.double().cpu())
    for split in (True, False):
        out = torch.full((T, F), float("nan"), dtype=BF, device=DEV)
        k.gemm_tc(x, w, None, out, split_k=split, swiglu_features=F)
        torch.cuda.synchronize()
        k.check_tc_status()
        assert rel_err(out, want) < 5e-3, f"split_k={split}"
    out32 = torch.empty(T, F, dtype=F32, device=DEV)
    k.gemm_tc(x, w, None, out32, swiglu_features=F)
    assert rel_err(out32, want) < 1e-5


# ------------------------------------------ many tokens: two SMs per 256 x 256 tile
@pytest.mark.parametrize("T,N,Kd", [(1024, 2560, 512), (1000, 2500, 328), (257, 19000, 64), (3000, 1290, 1032)])
def test_gemm_tensor_core_two_sms_per_tile(T, N, Kd):
    """Steps of many tokens take the kernel whose tiles are worked by a pair of CTAs; it must agree with the plain
    product, and with the one-CTA kernel to the bit (same order of the sum over K), with ragged edges in
    tokens, features and K, with a bias, and twice in a row."""
    from gguf_rs_cli_b200 import native
    k = K()
    g = torch.Generator().manual_seed(T + N + Kd)
    x = torch.randn(T, Kd, generator=g).to(BF).to(DEV)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(BF).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    want = P.linear(x.double().cpu(), w.double().cpu(), b.double().cpu())
    outs = []
    try:
        native.call("gb_gemm_tc_set_mode", 1)              # whole tiles in the one-CTA kernel too: the same sums
        for pair in (1, 0):
            native.call("gb_gemm_tc_set_pair", pair)
            out = torch.full((T, N), float("nan"), dtype=F32, device=DEV)
            k.gemm_tc(x, w, b, out)
            again = torch.full((T, N), float("nan"), dtype=BF, device=DEV)
            k.gemm_tc(x, w, b, again)
            torch.cuda.synchronize()
            k.check_tc_status()
            assert rel_err(out, want) < 1e-5 and rel_err(again, want) < 5e-3
            outs.append(out)
    finally:
        native.call("gb_gemm_tc_set_pair", 1)
        native.call("gb_gemm_tc_set_mode", 0)
    assert torch.equal(outs[0], outs[1])


def test_gemm_tensor_core_two_sms_per_tile_gated():
    k = K()
    T, F, Kd = 1500, 2000, 264
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, Kd, generator=g).to(BF).to(DEV)
    wg = (torch.randn(F, Kd, generator=g) * 0.1).to(BF).to(DEV)
    wu = (torch.randn(F, Kd, generator=g) * 0.1).to(BF).to(DEV)
    w = k.interleave_gate_up(wg, wu)
    want = P.silu(P.linear(x.double().cpu(), wg.double().cpu())) * P.linear(x.double().cpu(), wu.double().cpu())
    out = torch.full((T, F), float("nan"), dtype=BF, device=DEV)
    k.gemm_tc(x, w, None, out, swiglu_features=F)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < 5e-3


# --------------------------- deferred norm and residual epilogue of the product
@pytest.mark.parametrize("T,N,Kd", [(1, 256, 512), (8, 520, 320), (16, 4096, 4096), (70, 384, 1024), (300, 640, 328),
                                    (2100, 512, 256)])
def test_gemm_tensor_core_deferred_norm_and_residual(T, N, Kd):
    k = K()
    g = torch.Generator().manual_seed(T * 7 + N)
    eps = 1e-5
    # a producer leaves x (f32), its bf16 copy and per-tile sums of squares; the consumer scales by them
    x = torch.randn(T, Kd, generator=g) * 3
    wn = 1 + 0.2 * torch.randn(Kd, generator=g)
    w = (torch.randn(N, Kd, generator=g) * 0.1)
    wf = (w * wn).to(BF)                                        # the norm's weight folded into the matrix
    b = torch.randn(N, generator=g)
    xb = x.to(BF)
    parts = (Kd + 127) // 128
    ssq = torch.zeros(parts, T)
    for i in range(parts):
        ssq[i] = (x[:, 128 * i:128 * (i + 1)] ** 2).sum(1)
    rstd = 1 / torch.sqrt((x.double() ** 2).sum(1, keepdim=True) / Kd + eps)
    want = (xb.double() * rstd) @ wf.double().t() + b.double()
    out = torch.full((T, N), float("nan"), dtype=F32, device=DEV)
    k.gemm_tc(xb.to(DEV), wf.to(DEV), b.to(DEV), out, row_ssq=ssq.to(DEV), ssq_parts=parts, norm_size=Kd, eps=eps)
    torch.cuda.synchronize()
    k.check_tc_status()
    assert rel_err(out, want) < 1e-5
    # residual epilogue: r += x W^T + b, its bf16 copy, and sums of squares per 128 features
    r0 = torch.randn(T, N, generator=g) * 2
    r = r0.to(DEV).clone()
    rb = torch.zeros(T, N, dtype=BF, device=DEV)
    tiles = (N + 127) // 128
    ssq_out = torch.full((tiles, T), float("nan"), device=DEV)
    k.gemm_tc(xb.to(DEV), wf.to(DEV), b.to(DEV), None, resid_x=r, resid_xb=rb, ssq_out=ssq_out)
    torch.cuda.synchronize()
    k.check_tc_status()
    want_r = r0.double() + xb.double() @ wf.double().t() + b.double()
    assert rel_err(r, want_r) < 1e-5
    assert torch.equal(rb.cpu(), r.cpu().to(BF))
    want_ssq = torch.stack([(r.cpu().double()[:, 128 * i:128 * (i + 1)] ** 2).sum(1) for i in range(tiles)])
    assert rel_err(ssq_out, want_ssq) < 1e-5


@pytest.mark.parametrize("T,N,Kd,tile", [(5, 384, 4096, 16), (16, 4096, 4096, 16), (40, 1000, 2048, 32), (64, 520, 1024, 64),
                                         (64, 4096, 4096, 64), (130, 300, 4096, 128), (300, 260, 2048, 256), (700, 264, 640, 64)])
@pytest.mark.parametrize("mode", [0, 2, 3])
def test_gemm_tensor_core_tiles_shared_between_ctas(T, N, Kd, tile, mode):
    """Tiles shared by CTAs in every way, at every tile width.  Mode 3: every CTA takes an equal share of all K
    blocks (a share that ends inside a tile, one that lies inside a tile, whole tiles between two partial ones);
    mode 2: where the sizes allow it, every tile has CTAs of its own instead (mode 0, the rule: only then are tiles
    shared).  With CTAs of its own, a tile of 32 tokens or more is finished by all of them, each a share of its
    tokens, after a bounded wait for one another; otherwise by the CTA that arrives last.  Plain,
    gated and residual epilogues against 64-bit products, twice in a row to the bit (the counters are left at
    zero), and the same values as with whole tiles only up to the order of the 32-bit sums."""
    from gguf_rs_cli_b200 import native
    k = K()
    g = torch.Generator().manual_seed(T + N + Kd)
    x = torch.randn(T, Kd, generator=g).to(BF).to(DEV)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(BF).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    want = P.linear(x.double().cpu(), w.double().cpu(), b.double().cpu())
    F_ = (N // 2 // 8) * 8
    wg, wu = w[:F_], w[F_:2 * F_]
    wgu = k.interleave_gate_up(wg, wu)
    want_g = P.silu(P.linear(x.double().cpu(), wg.double().cpu())) * P.linear(x.double().cpu(), wu.double().cpu())
    r0 = torch.randn(T, N, generator=g) * 2
    want_r = r0.double() + want
    parts = (Kd + 127) // 128
    ssq = torch.rand(parts, T, generator=g).to(DEV) * 50
    rstd = 1 / torch.sqrt(ssq.double().cpu().sum(0) / Kd + 1e-5)
    try:
        native.call("gb_gemm_tc_set_pair", 0)
        native.call("gb_gemm_tc_set_tile", tile)
        native.call("gb_gemm_tc_set_mode", mode)
        assert native.library().gb_gemm_tc_scratch_floats(T, N, Kd, native.library().gb_sm_count()) > 0
        outs = []
        for _ in range(2):
            out = torch.full((T, N), float("nan"), dtype=F32, device=DEV)
            k.gemm_tc(x, w, b, out)
            outb = torch.full((T, N), float("nan"), dtype=BF, device=DEV)
            k.gemm_tc(x, w, b, outb)
            gated = torch.full((T, F_), float("nan"), dtype=F32, device=DEV)
            k.gemm_tc(x, wgu, None, gated, swiglu_features=F_)
            normed = torch.full((T, N), float("nan"), dtype=F32, device=DEV)
            k.gemm_tc(x, w, b, normed, row_ssq=ssq, ssq_parts=parts, norm_size=Kd, eps=1e-5)
            r = r0.to(DEV).clone()
            rb = torch.zeros(T, N, dtype=BF, device=DEV)
            ssq_out = torch.full(((N + 127) // 128, T), float("nan"), device=DEV)
            k.gemm_tc(x, w, b, None, resid_x=r, resid_xb=rb, ssq_out=ssq_out)
            torch.cuda.synchronize()
            k.check_tc_status()
            outs.append((out, outb, gated, normed, r, rb, ssq_out))
        out, outb, gated, normed, r, rb, ssq_out = outs[0]
        assert rel_err(out, want) < 1e-5 and rel_err(outb, want) < 5e-3 and rel_err(gated, want_g) < 1e-5
        assert rel_err(normed, (want - b.double().cpu()) * rstd[:, None] + b.double().cpu()) < 1e-5
        assert rel_err(r, want_r) < 1e-5 and torch.equal(rb.cpu(), r.cpu().to(BF))
        want_ssq = torch.stack([(r.cpu().double()[:, 128 * i:128 * (i + 1)] ** 2).sum(1) for i in range((N + 127) // 128)])
        assert rel_err(ssq_out, want_ssq) < 1e-5
        for a, c in zip(outs[0], outs[1]):
            assert torch.equal(a, c)
        native.call("gb_gemm_tc_set_mode", 1)
        whole = torch.full((T, N), float("nan"), dtype=F32, device=DEV)
        k.gemm_tc(x, w, b, whole)
        assert rel_err(whole, want) < 1e-5 and rel_err(whole, out.double()) < 1e-5
    finally:
        native.call("gb_gemm_tc_set_pair", 1)
        native.call("gb_gemm_tc_set_tile", 0)
        native.call("gb_gemm_tc_set_mode", 0)


def test_embed_shadow():
    g = torch.Generator().manual_seed(0)
    table = torch.randn(300, 200, generator=g).to(BF)
    toks = torch.randint(0, 300, (33,), generator=g)
    out = torch.empty(33, 200, dtype=F32, device=DEV)
    xb = torch.empty(33, 200, dtype=BF, device=DEV)
    ssq = torch.empty(33, dtype=F32, device=DEV)
    K().embed_shadow(table.to(DEV), toks.to(torch.int32).to(DEV), out, xb, ssq)
    want = P.embedding(table.float(), toks.tolist())
    assert torch.equal(out.cpu(), want) and torch.equal(xb.cpu(), want.to(BF))
    assert rel_err(ssq, (want.double() ** 2).sum(1)) < 1e-6
