"""Each kernel alone against a plain float64 reference, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import plain_gptj as P
from qstream_b200.csrc import ops

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)


def dev(a, dtype=None):
    t = torch.as_tensor(a)
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def f64(t):
    return t.detach().cpu().to(torch.float64).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(37, 50, generator=g).to(DT[dtype])
    toks = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32)
    out = ops.embedding(table.cuda(), toks.cuda(), DT[dtype])
    assert torch.equal(out.cpu(), table[toks.long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,eps,wdtype", [(50, 1e-5, None), (4096, 1e-6, "float32"), (6000, 1e-3, None), (17, 1e-5, None)])
def test_layernorm(dtype, D, eps, wdtype):
    g = torch.Generator().manual_seed(D)
    x = (torch.randn(7, D, generator=g) * 3 + 1.5).to(DT[dtype])
    wd = DT[wdtype or dtype]
    w = (1 + 0.2 * torch.randn(D, generator=g)).to(wd)
    b = (0.1 * torch.randn(D, generator=g)).to(wd)
    ref = P.layer_norm(f64(x), f64(w), f64(b), eps)
    got = ops.layernorm(x.cuda(), w.cuda(), b.cuda(), eps)
    np.testing.assert_allclose(f64(got), ref, **tol(dtype))
    got = ops.layernorm(x.cuda(), w.cuda(), None, eps)
    np.testing.assert_allclose(f64(got), P.layer_norm(f64(x), f64(w), None, eps), **tol(dtype))
    # weights that are older than the stream's last kernel may be fetched before its end: the same bits
    xd, wdev, bdev = x.cuda(), w.cuda(), b.cuda()
    late = ops.layernorm(xd, wdev, bdev, eps)
    torch.cuda.synchronize()
    assert torch.equal(ops.layernorm(xd, wdev, bdev, eps, settled=True), late)


@pytest.mark.parametrize("adt,wdt,cdt", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                         ("bfloat16", "bfloat16", "float32"), ("bfloat16", "float32", "bfloat16"),
                                         ("float32", "bfloat16", "float32")])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 70, 33), (64, 64, 16), (65, 130, 100), (3, 200, 257)])
def test_linear_simt(adt, wdt, cdt, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    x = torch.randn(M, K, generator=g).to(DT[adt])
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(DT[wdt])
    bias = torch.randn(N, generator=g).to(DT[wdt])
    r1 = torch.randn(M, N, generator=g).to(DT[adt])
    r2 = torch.randn(M, N, generator=g).to(DT[adt])
    t = tol("float32" if cdt == "float32" and adt == "float32" else cdt)
    for act, fn in ((None, lambda u: u), ("gelu_new", P.gelu_new), ("gelu", P.gelu_erf)):
        ref = fn(f64(x) @ f64(w).T + f64(bias)) + f64(r1) + f64(r2)
        got = ops.linear_simt(x.cuda(), w.cuda(), bias.cuda(), act, (r1.cuda(), r2.cuda()), DT[cdt])
        assert got.dtype == DT[cdt]
        np.testing.assert_allclose(f64(got), ref, **t)
    got = ops.linear_simt(x.cuda(), w.cuda())
    np.testing.assert_allclose(f64(got), f64(x) @ f64(w).T, **tol(adt))


def test_linear_simt_row_does_not_depend_on_batch():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(70, 300, generator=g).cuda()
    w = torch.randn(90, 300, generator=g).cuda()
    whole = ops.linear_simt(x, w)
    for r in (0, 13, 69):
        assert torch.equal(ops.linear_simt(x[r:r + 1], w)[0], whole[r])


class PagedCase:
    """Sequences laid into a paged cache through shuffled pages."""

    def __init__(self, dtype, lens, H, Hkv, dh, page_tokens=64, seed=0, n_slots=6, fill=float("nan")):
        g = torch.Generator().manual_seed(seed)
        self.dtype, self.lens, self.H, self.Hkv, self.dh, self.pt = dtype, lens, H, Hkv, dh, page_tokens
        max_pages = max(-(-n // page_tokens) for n in lens) + 1
        n_pages = sum(-(-n // page_tokens) for n in lens) + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.table = torch.full((n_slots, max_pages), -1, dtype=torch.int32)
        self.slots = torch.randperm(n_slots, generator=g)[:len(lens)].tolist()
        for s, n in zip(self.slots, lens):
            for i in range(-(-n // page_tokens)):
                self.table[s, i] = perm.pop()
        self.k_cache = torch.full((n_pages, Hkv, page_tokens, dh), fill, dtype=DT[dtype]).cuda()
        self.v_cache = torch.full((n_pages, Hkv, page_tokens, dh), fill, dtype=DT[dtype]).cuda()
        self.q = [torch.randn(n, H, dh, generator=g).to(DT[dtype]) for n in lens]
        self.k = [torch.randn(n, Hkv, dh, generator=g).to(DT[dtype]) for n in lens]
        self.v = [torch.randn(n, Hkv, dh, generator=g).to(DT[dtype]) for n in lens]
        self.status = torch.zeros(1, dtype=torch.int32).cuda()

    def packed(self, ranges):
        """Rows of the given (sequence, start, stop) ranges as one packed batch."""
        qs, ks, vs, slot, pos = [], [], [], [], []
        for i, a, b in ranges:
            qs.append(self.q[i][a:b]); ks.append(self.k[i][a:b]); vs.append(self.v[i][a:b])
            slot += [self.slots[i]] * (b - a)
            pos += list(range(a, b))
        cat = lambda xs, h: torch.cat(xs).reshape(-1, h * self.dh).contiguous().cuda()
        return (cat(qs, self.H), cat(ks, self.Hkv), cat(vs, self.Hkv),
                torch.tensor(slot, dtype=torch.int32).cuda(), torch.tensor(pos, dtype=torch.int32).cuda())


def rope_table(max_pos, R, base=10000.0):
    i = torch.arange(0, R, 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(base, dtype=torch.float64), -i / R)[None]
    return torch.stack([ang.cos(), ang.sin()], -1).float().contiguous().cuda()


@pytest.mark.parametrize("settled", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,Hkv,dh,R,window", [(4, 4, 16, 8, 0), (6, 2, 48, 48, 0), (2, 1, 80, 64, 0),
                                                (3, 3, 256, 64, 0), (4, 2, 32, 16, 37), (2, 2, 16, 0, 64)])
def test_rope_store_and_attention(dtype, H, Hkv, dh, R, window, settled):
    """Prompts in one packed step, then some tokens one by one, through shuffled pages;
    compared with the plain rotary + causal attention on whole sequences.  `settled`: the kernel reads
    slots, positions and pages before the previous kernel has ended (they are older than it here: the
    test waits for the device before each call)."""
    lens = [1, 70, 130, 64]
    case = PagedCase(dtype, lens, H, Hkv, dh, seed=H * dh)
    table = rope_table(256, R) if R else None
    table_dev = case.table.cuda()
    outs = [[] for _ in lens]

    def run(ranges):
        q, k, v, slot, pos = case.packed(ranges)
        if settled:
            torch.cuda.synchronize()
        ops.rope_store(q, k, v, H, Hkv, dh, R, table, slot, pos, table_dev, case.pt, case.k_cache, case.v_cache, case.status,
                       settled=settled)
        o = ops.attention(q, H, Hkv, dh, dh ** -0.5, window, slot, pos, table_dev, case.pt, case.k_cache, case.v_cache, case.status)
        row = 0
        for i, a, b in ranges:
            outs[i].append(o[row:row + b - a].cpu())
            row += b - a

    heads = [max(1, n - 5) for n in lens]
    run([(i, 0, h) for i, h in enumerate(heads)])
    for step in range(5):
        rs = [(i, h + step, h + step + 1) for i, h in enumerate(heads) if h + step < lens[i]]
        if rs:
            run(rs)
    assert int(case.status.item()) == 0
    for i, n in enumerate(lens):
        pos = np.arange(n)
        q = P.rotary_interleaved(f64(case.q[i]), pos, R) if R else f64(case.q[i])
        k = P.rotary_interleaved(f64(case.k[i]), pos, R) if R else f64(case.k[i])
        if dtype == "bfloat16":     # the engine keeps rotated q and k in bfloat16
            q = f64(torch.from_numpy(q).to(torch.bfloat16))
            k = f64(torch.from_numpy(k).to(torch.bfloat16))
        ref = P.causal_attention(q, k, f64(case.v[i]), window)
        np.testing.assert_allclose(f64(torch.cat(outs[i])), ref, **tol(dtype), err_msg=f"sequence {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key(dtype):
    """One key among hundreds matches the query: the output must be that key's value,
    wherever it lies (first position, a page's edge, the window's edge)."""
    H, dh, n = 2, 32, 300
    for far, window in ((0, 0), (63, 0), (64, 0), (299, 0), (200, 100), (201, 100)):
        case = PagedCase(dtype, [n], H, H, dh, seed=far)
        case.q[0][:] = 0
        case.k[0][:] = 0
        case.q[0][n - 1, :, 0] = 12.0
        case.k[0][far, :, 0] = 12.0
        q, k, v, slot, pos = case.packed([(0, 0, n)])
        tdev = case.table.cuda()
        ops.rope_store(q, k, v, H, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        o = ops.attention(q, H, H, dh, dh ** -0.5, window, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        got = f64(o[n - 1]).reshape(H, dh)
        visible = window == 0 or far > n - 1 - window
        if visible:
            np.testing.assert_allclose(got, f64(case.v[0][far]), atol=5e-2 if dtype == "bfloat16" else 1e-4)
        else:
            lo = n - window
            np.testing.assert_allclose(got, f64(case.v[0][lo:n]).mean(0), atol=5e-2 if dtype == "bfloat16" else 1e-4)


def test_attention_skips_padding():
    case = PagedCase("float32", [10], 2, 2, 16)
    q, k, v, slot, pos = case.packed([(0, 0, 10)])
    slot[3] = -1
    tdev = case.table.cuda()
    ops.rope_store(q, k, v, 2, 2, 16, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    page = int(case.table[case.slots[0], 0])
    assert torch.isnan(case.k_cache[page, :, 3]).all() and not torch.isnan(case.k_cache[page, :, 2]).any()
    o = ops.attention(q, 2, 2, 16, 0.25, 0, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    assert torch.equal(o[3], torch.zeros_like(o[3]))
    # nothing but the nine written rows of the sequence's own page has changed (the cache started as NaN)
    others = [p for p in range(case.k_cache.shape[0]) if p != page]
    assert torch.isnan(case.k_cache[others]).all() and torch.isnan(case.v_cache[others]).all()
    assert torch.isnan(case.k_cache[page, :, 10:]).all() and torch.isnan(case.v_cache[page, :, 10:]).all()
    written = [r for r in range(10) if r != 3]
    assert torch.equal(case.k_cache[page][:, written].cpu(), case.k[0][written].transpose(0, 1))


def test_argmax_lowest_index_wins_ties():
    x = torch.full((4, 5000), -1.0)
    x[0, 4999] = 3.0
    x[1, 77] = 2.0; x[1, 4000] = 2.0
    x[2] = 0.5
    x[3, 1023] = 9.0; x[3, 1024] = 9.0
    assert ops.argmax(x.cuda()).tolist() == [4999, 77, 0, 1023]
    y = torch.randn(9, 321, generator=torch.Generator().manual_seed(1))
    assert ops.argmax(y.cuda()).tolist() == [P.argmax_lowest(r.numpy()) for r in y]
    # rows that start at every offset from a 16-byte boundary, widths with a ragged end
    for width in (50400, 4099, 7, 3, 1):
        z = torch.randn(5, width, generator=torch.Generator().manual_seed(width))
        assert ops.argmax(z.cuda()).tolist() == [P.argmax_lowest(r.numpy()) for r in z], width


def test_argmax_scans_like_a_strict_greater_than():
    """NaN is never greater, so it is skipped unless the row begins with it; -0 equals +0; -inf rows give 0."""
    nan, inf = float("nan"), float("inf")
    rows = [
        [1.0, nan, 5.0, nan, 5.0, 2.0, 0.0, 0.0],
        [nan, 9.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0],
        [-0.0, 0.0, -1.0, -1.0, -1.0, -1.0, -1.0, -1.0],
        [-inf] * 8,
        [-3.0, -inf, inf, inf, 1.0, 1.0, 1.0, 1.0],
    ]
    x = torch.tensor(rows)
    assert ops.argmax(x.cuda()).tolist() == [2, 0, 0, 0, 2]


def test_repeat_penalty():
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5], [4.0, 4.0, -1.0, 2.0]])
    recent = torch.zeros((2, 64), dtype=torch.int32)
    recent[0, :3] = torch.tensor([0, 1, 0])
    recent[1, :1] = torch.tensor([3])
    count = torch.tensor([3, 1], dtype=torch.int32)
    d = x.cuda()
    ops.repeat_penalty(d, recent.cuda(), count.cuda(), 2.0)
    ref0 = P.apply_repeat_penalty(x[0].double().numpy(), [0, 1, 0], 2.0)
    ref1 = P.apply_repeat_penalty(x[1].double().numpy(), [3], 2.0)
    np.testing.assert_allclose(d.cpu().numpy(), np.stack([ref0, ref1]), rtol=1e-6)


@pytest.mark.parametrize("V", [320, 50400])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 0, 1.0), (0.7, 40, 0.9), (1.3, 5, 1.0),
                                                     (0.9, 0, 0.5), (0.5, 1, 1.0), (1.0, 1000, 0.97), (0.9, 3000, 0.95),
                                                     (1.1, 300, 1.0), (3.0, 0, 0.9), (0.6, 0, 0.95)])
def test_sample_against_plain(V, temperature, top_k, top_p):
    """The chosen token's CDF interval in the plain pipeline must contain the draw (a
    little widened: 32-bit sums in another order)."""
    g = torch.Generator().manual_seed(V + top_k)
    rows = 24
    logits = (torch.randn(rows, V, generator=g) * 2.5).float()
    draws = torch.rand(rows, generator=g).float()
    draws[0], draws[1] = 0.0, 0.99999994
    got = ops.sample(logits.cuda(), temperature, top_k, top_p, draws.cuda()).tolist()
    for r in range(rows):
        y = logits[r].double().numpy()
        if temperature != 1.0:
            y = logits[r].numpy().astype(np.float32) * np.float32(1.0 / temperature)
            y = y.astype(np.float64)
        if 0 < top_k < V:
            y = P.top_k_filter(y, top_k)
        if 0 < top_p < 1:
            y = P.top_p_filter(y, top_p)
        probs = P.softmax(y)
        assert probs[got[r]] > 0, f"row {r}: token {got[r]} was filtered out"
        lo, hi = P.cdf_interval(probs, got[r])
        assert lo - 1e-4 <= float(draws[r]) <= hi + 1e-4, (r, got[r], lo, hi, float(draws[r]))


def test_repeat_penalty_of_a_full_window_with_repeats():
    g = torch.Generator().manual_seed(5)
    V = 1000
    x = torch.randn(3, V, generator=g) * 3
    recent = torch.randint(0, 40, (3, 64), generator=g).to(torch.int32)       # 64 entries over 40 tokens: many repeats
    recent[1, 5] = -1                                                          # entries outside the vocabulary are skipped
    recent[1, 6] = V
    count = torch.tensor([64, 64, 17], dtype=torch.int32)
    d = x.cuda()
    ops.repeat_penalty(d, recent.cuda(), count.cuda(), 1.3)
    for r in range(3):
        toks = [t for t in recent[r, :count[r]].tolist() if 0 <= t < V]
        ref = P.apply_repeat_penalty(x[r].double().numpy(), toks, 1.3)
        np.testing.assert_allclose(d[r].cpu().numpy(), ref, rtol=1e-5)


def test_sample_top_k_keeps_the_ties_at_the_kth_value():
    x = torch.full((1, 3000), -5.0)
    x[0, [7, 100, 2500, 2999]] = torch.tensor([3.0, 2.0, 2.0, 2.0])          # k = 2: the three equal seconds all stay
    got = set()
    for r in np.linspace(0.0, 0.9999, 60):
        got.add(ops.sample(x.cuda(), 1.0, 2, 1.0, torch.tensor([r], dtype=torch.float32).cuda()).item())
    assert got == {7, 100, 2500, 2999}
    # with top-p on top: 3.0 holds 0.475 of the four's mass, so p = 0.6 keeps it and the first of the equal ones
    got = set()
    for r in np.linspace(0.0, 0.9999, 60):
        got.add(ops.sample(x.cuda(), 1.0, 2, 0.6, torch.tensor([r], dtype=torch.float32).cuda()).item())
    assert got == {7, 100}
    # all equal: every element ties at the k-th value; p = 0.3 of eight keeps the first three by index
    z = torch.zeros(1, 8)
    got = set()
    for r in np.linspace(0.0, 0.999, 40):
        got.add(ops.sample(z.cuda(), 0.7, 5, 0.3, torch.tensor([r], dtype=torch.float32).cuda()).item())
    assert got == {0, 1, 2}


def test_sample_top_p_ties_keep_lower_indices():
    x = torch.zeros(1, 8)                       # eight equal tokens, p = 0.3 keeps the first three
    got = set()
    for r in np.linspace(0.0, 0.999, 40):
        got.add(ops.sample(x.cuda(), 1.0, 0, 0.3, torch.tensor([r], dtype=torch.float32).cuda()).item())
    assert got == {0, 1, 2}


@pytest.mark.parametrize("H,Hkv,dh,window", [(4, 4, 16, 0), (16, 16, 256, 0), (6, 2, 48, 0), (2, 1, 80, 0),
                                             (4, 4, 64, 300), (3, 3, 128, 0), (2, 2, 320, 0), (2, 2, 32, 1),
                                             # head sizes whose chunks do not fill a power of two of lanes, and a window
                                             (4, 2, 96, 0), (2, 2, 160, 0), (3, 1, 112, 0), (32, 32, 80, 100), (2, 2, 48, 1)])
def test_decode_attention_kernel(H, Hkv, dh, window):
    """The split decode kernel (bfloat16) against the plain attention at many lengths: page and
    split edges, one key, a window."""
    from qstream_b200.csrc import attention_bf16
    lens = [1, 64, 65, 256, 257, 700, 1024]
    case = PagedCase("bfloat16", lens, H, Hkv, dh, seed=dh + window, n_slots=9)
    tdev = case.table.cuda()
    q, k, v, slot, pos = case.packed([(i, 0, n) for i, n in enumerate(lens)])
    ops.rope_store(None, k, v, 0, Hkv, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    last_rows = np.cumsum(lens) - 1
    ql = q[torch.as_tensor(last_rows).cuda()].contiguous()
    slot_l = torch.tensor(case.slots[:len(lens)], dtype=torch.int32).cuda()
    pos_l = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    # a padding row in the middle
    slot_l = torch.cat([slot_l[:3], torch.tensor([-1], dtype=torch.int32).cuda(), slot_l[3:]])
    pos_l = torch.cat([pos_l[:3], torch.tensor([0], dtype=torch.int32).cuda(), pos_l[3:]])
    ql = torch.cat([ql[:3], ql[:1], ql[3:]])
    got = attention_bf16.decode(ql, H, Hkv, dh, dh ** -0.5, window, slot_l, pos_l, tdev, case.pt,
                                case.k_cache, case.v_cache, 1100, case.status)
    gen = ops.attention(ql, H, Hkv, dh, dh ** -0.5, window, slot_l, pos_l, tdev, case.pt, case.k_cache,
                        case.v_cache, case.status)
    assert int(case.status.item()) == 0
    assert torch.equal(got[3], torch.zeros_like(got[3]))
    keep = [0, 1, 2, 4, 5, 6, 7]
    for j, i in zip(keep, range(len(lens))):
        ref = P.causal_attention(f64(case.q[i]), f64(case.k[i]), f64(case.v[i]), window)[-1]
        np.testing.assert_allclose(f64(got[j]), ref, atol=2e-2, rtol=2e-2, err_msg=f"length {lens[i]}")
        np.testing.assert_allclose(f64(got[j]), f64(gen[j]), atol=2e-2, rtol=2e-2)


def test_decode_attention_finds_one_far_key():
    """One key among a thousand matches the query and its value is a marker: the split kernel's output is
    that marker when the key is visible (the first key, page and split edges, the window's first key) and
    free of it when the key lies just outside the window."""
    from qstream_b200.csrc import attention_bf16
    H, dh, n = 2, 64, 1000
    for far, window in ((0, 0), (63, 0), (64, 0), (255, 0), (256, 0), (999, 0), (700, 300), (699, 300), (744, 256)):
        case = PagedCase("bfloat16", [n], H, H, dh, seed=far + window, fill=0.0)
        case.q[0][:] = 0
        case.k[0][:] = 0
        case.q[0][n - 1, :, 0] = 12.0
        case.k[0][far, :, 0] = 12.0
        case.v[0][far] = 100.0
        q, k, v, slot, pos = case.packed([(0, 0, n)])
        tdev = case.table.cuda()
        ops.rope_store(None, k, v, 0, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        o = attention_bf16.decode(q[n - 1:n], H, H, dh, dh ** -0.5, window, slot[n - 1:n], pos[n - 1:n], tdev, case.pt,
                                  case.k_cache, case.v_cache, 1024, case.status)
        got = f64(o[0]).reshape(H, dh)
        if window == 0 or far > n - 1 - window:
            np.testing.assert_allclose(got, np.full((H, dh), 100.0), atol=0.5, err_msg=f"key {far} window {window}")
        else:                       # invisible: the mean of the window's values, none of them the marker
            np.testing.assert_allclose(got, f64(case.v[0][n - window:n]).mean(0), atol=5e-2,
                                       err_msg=f"key {far} window {window}")
    assert int(case.status.item()) == 0


def test_decode_attention_does_not_depend_on_the_batch():
    from qstream_b200.csrc import attention_bf16
    H, dh = 4, 64
    lens = [300, 900, 10]
    case = PagedCase("bfloat16", lens, H, H, dh, seed=3)
    tdev = case.table.cuda()
    q, k, v, slot, pos = case.packed([(i, 0, n) for i, n in enumerate(lens)])
    ops.rope_store(None, k, v, 0, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    rows = torch.as_tensor(np.cumsum(lens) - 1).cuda()
    ql = q[rows].contiguous()
    slot_l = torch.tensor(case.slots, dtype=torch.int32).cuda()
    pos_l = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    args = (H, H, dh, dh ** -0.5, 0)
    both = attention_bf16.decode(ql, *args, slot_l, pos_l, tdev, case.pt, case.k_cache, case.v_cache, 1024, case.status)
    for i in range(3):
        alone = attention_bf16.decode(ql[i:i + 1], *args, slot_l[i:i + 1], pos_l[i:i + 1], tdev, case.pt,
                                      case.k_cache, case.v_cache, 2048, case.status)
        assert torch.equal(alone[0], both[i])


def _tiles(ranges, slots):
    tiles, row = [], 0
    for i, a, b in ranges:
        for t in range(a, b, 128):
            tiles.append((row + t - a, min(128, b - t), t, slots[i]))
        row += b - a
    tiles.sort(key=lambda t: -(t[2] + t[1]))
    return torch.tensor(tiles, dtype=torch.int32).cuda()


@pytest.mark.parametrize("H,Hkv,dh,window", [(2, 2, 64, 0), (16, 16, 256, 0), (4, 4, 16, 0), (6, 2, 48, 0), (2, 1, 80, 0),
                                             (3, 3, 128, 0), (2, 2, 192, 0), (4, 4, 64, 100), (2, 2, 32, 1),
                                             (2, 2, 256, 200)])
def test_prefill_attention_kernel(H, Hkv, dh, window):
    """The tensor-core prefill kernel (bfloat16) against the plain attention: whole prompts of unequal
    lengths in one packed step (page and tile edges, a single token), then a second chunk of each
    sequence on top of the cached first one, with grouped heads, padded head sizes and windows."""
    from qstream_b200.csrc import attention_bf16
    lens = [1, 64, 129, 300, 700]
    case = PagedCase("bfloat16", lens, H, Hkv, dh, seed=dh + window, n_slots=7, fill=0.0)
    case.v_cache.fill_(1e30)                    # rows beyond a sequence's end: finite leftovers must not matter
    tdev = case.table.cuda()
    outs = [[] for _ in lens]
    cuts = [(0, max(1, n * 2 // 3)) for n in lens]
    for phase in range(2):
        ranges = [(i, a, b) for i, (a, b) in enumerate(cuts) if b > a]
        q, k, v, slot, pos = case.packed(ranges)
        ops.rope_store(None, k, v, 0, Hkv, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        o = attention_bf16.prefill(q, H, Hkv, dh, dh ** -0.5, window, _tiles(ranges, case.slots), tdev, case.pt,
                                   case.k_cache, case.v_cache, case.status)
        gen = ops.attention(q, H, Hkv, dh, dh ** -0.5, window, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        np.testing.assert_allclose(f64(o), f64(gen), atol=3e-2, rtol=3e-2)
        row = 0
        for i, a, b in ranges:
            outs[i].append(o[row:row + b - a].cpu())
            row += b - a
        cuts = [(b, n) for (a, b), n in zip(cuts, lens)]
    torch.cuda.synchronize()
    assert int(case.status.item()) == 0
    for i, n in enumerate(lens):
        ref = P.causal_attention(f64(case.q[i]), f64(case.k[i]), f64(case.v[i]), window)
        np.testing.assert_allclose(f64(torch.cat(outs[i])), ref, atol=3e-2, rtol=3e-2, err_msg=f"sequence {i} of {n}")


def test_prefill_attention_gives_the_same_bits_every_time():
    """Sixteen prompts of unequal lengths in one step, a thousand times over the same inputs, with what earlier
    sequences left in the pages still there: every launch must give the same bits.  (A softmax thread that
    had not rescaled in a tile's last blocks could pass the wait for the last P V while the one before it
    was still running, read O early and overwrite weights that the tensor core was still reading: two
    launches in three hundred gave other values, NaN among them, in the rows of one tile.)"""
    from qstream_b200.csrc import attention_bf16
    lens = [77, 427, 31, 472, 237, 413, 591, 579, 185, 586, 522, 116, 190, 250, 448, 217]
    H, dh = 16, 256
    case = PagedCase("bfloat16", lens, H, H, dh, seed=1, n_slots=16, fill=0.0)
    case.v_cache.normal_(0, 3.0)
    case.k_cache.normal_(0, 1.0)
    tdev = case.table.cuda()
    ranges = [(i, 0, n) for i, n in enumerate(lens)]
    q, k, v, slot, pos = case.packed(ranges)
    ops.rope_store(None, k, v, 0, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    tiles = _tiles(ranges, case.slots)
    first = attention_bf16.prefill(q, H, H, dh, dh ** -0.5, 0, tiles, tdev, case.pt, case.k_cache, case.v_cache, case.status).clone()
    different = 0
    for _ in range(1000):                           # each launch starts on an idle device: that is when it showed
        o = attention_bf16.prefill(q, H, H, dh, dh ** -0.5, 0, tiles, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        different += 0 if torch.equal(o, first) else 1
    assert different == 0
    assert int(case.status.item()) == 0
    assert torch.isfinite(first.float()).all()


def test_prefill_attention_finds_one_far_key_and_keeps_rows_apart():
    from qstream_b200.csrc import attention_bf16
    H, dh, n = 2, 64, 600
    for far, window in ((0, 0), (63, 0), (64, 0), (599, 0), (500, 100), (501, 100)):
        case = PagedCase("bfloat16", [n], H, H, dh, seed=far, fill=0.0)
        case.q[0][:] = 0
        case.k[0][:] = 0
        case.q[0][n - 1, :, 0] = 12.0
        case.k[0][far, :, 0] = 12.0
        q, k, v, slot, pos = case.packed([(0, 0, n)])
        tdev = case.table.cuda()
        ops.rope_store(None, k, v, 0, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
        o = attention_bf16.prefill(q, H, H, dh, dh ** -0.5, window, _tiles([(0, 0, n)], case.slots), tdev, case.pt,
                                   case.k_cache, case.v_cache, case.status)
        got = f64(o[n - 1]).reshape(H, dh)
        if window == 0 or far > n - 1 - window:
            np.testing.assert_allclose(got, f64(case.v[0][far]), atol=5e-2)
        else:
            np.testing.assert_allclose(got, f64(case.v[0][n - window:n]).mean(0), atol=5e-2)
        # every other row has all-zero scores: the mean of its visible values
        t = 300
        lo = 0 if window == 0 else t - window + 1
        np.testing.assert_allclose(f64(o[t]).reshape(H, dh), f64(case.v[0][lo:t + 1]).mean(0), atol=5e-2)


def test_kernels_give_the_same_bits_every_time():
    """Every kernel whose work is shared out between CTAs that meet again (partial tiles and arrival counters in the
    products, splits and their merge in the decode attention, counts and lists in the sampler), launched two
    hundred times on an idle device over the same inputs: the same bits each time."""
    import math
    from qstream_b200.csrc import attention_bf16, gemm_tc
    g = torch.Generator(device="cuda").manual_seed(0)

    def same(fn, reps=200):
        first = fn().clone()
        return all(torch.equal(fn(), first) for _ in range(reps))

    for M, N, K in [(8, 4096, 20480), (64, 4096, 20480), (1, 4096, 4096), (256, 4096, 20480), (300, 520, 16384), (2600, 1000, 4096)]:
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).bfloat16()
        b = torch.randn(N, device="cuda", generator=g).bfloat16()
        r = torch.randn(M, N, device="cuda", generator=g).bfloat16()
        assert same(lambda: gemm_tc.linear(x, w, b, "gelu_new", (r,))), (M, N, K)
    gemm_tc.check_status(torch.device("cuda"))
    lens = [2043, 1, 300, 1488, 64, 65, 700, 1025]
    H, dh = 16, 256
    case = PagedCase("bfloat16", lens, H, H, dh, seed=2, n_slots=10, fill=0.0)
    case.v_cache.normal_(0, 3.0)
    case.k_cache.normal_(0, 1.0)
    tdev = case.table.cuda()
    q, k, v, slot, pos = case.packed([(i, 0, n) for i, n in enumerate(lens)])
    ops.rope_store(None, k, v, 0, H, dh, 0, None, slot, pos, tdev, case.pt, case.k_cache, case.v_cache, case.status)
    ql = q[torch.as_tensor(np.cumsum(lens) - 1).cuda()].contiguous()
    slot_l = torch.tensor(case.slots, dtype=torch.int32).cuda()
    pos_l = torch.tensor([n - 1 for n in lens], dtype=torch.int32).cuda()
    assert same(lambda: attention_bf16.decode(ql, H, H, dh, dh ** -0.5, 0, slot_l, pos_l, tdev, case.pt, case.k_cache,
                                              case.v_cache, 2048, case.status))
    assert int(case.status.item()) == 0
    logits = torch.randn(16, 50400, device="cuda", generator=g)
    draws = torch.rand(16, device="cuda", generator=g)
    assert same(lambda: ops.sample(logits, 0.7, 40, 0.9, draws))
    assert same(lambda: ops.sample(logits, 0.7, 0, 0.9, draws))
