"""Each kernel alone against a plain float32 statement of the same operation, at sizes other than
the engine's own: odd widths, head sizes in steps of 16, many groups, page sizes that do not divide
the length, and inputs made so that a wrong key, page or window edge shows."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def dev(a, dtype=None):
    t = torch.as_tensor(a).cuda()
    return t.to(dtype) if dtype is not None else t


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1e-2


@pytest.fixture(scope="module")
def ops():
    from vitna_anchor_b200 import ops
    ops.lib()
    return ops


@pytest.mark.parametrize("dtype", DT)
def test_embed_rows(ops, dtype):
    table = torch.randn(77, 53).to(dtype).cuda()
    ids = dev(np.array([0, 76, 5, 5, 31], dtype=np.int32))
    out = torch.empty(5, 53, device="cuda")
    ops.embed_rows(table, ids, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("n", [37, 576, 1000])
def test_rmsnorm_rows(ops, dtype, n):
    x = (torch.randn(9, n) * 3).cuda()
    w = (1 + 0.1 * torch.randn(n)).cuda()
    want = torch.from_numpy(P.rms_norm(x.cpu().numpy(), w.cpu().numpy(), 1e-5))
    out = torch.empty(9, n, dtype=dtype, device="cuda")
    ops.rmsnorm_rows(x, w, 1e-5, out)
    assert (out.float().cpu() - want).abs().max() <= tol(dtype) * want.abs().max()
    rows = dev(np.array([8, 0, 3], dtype=np.int32))
    out2 = torch.empty(3, n, dtype=dtype, device="cuda")
    ops.rmsnorm_rows(x, w, 1e-5, out2, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("shape", [(3, 5, 7), (67, 131, 33), (64, 576, 576), (17, 1536, 100), (1, 960, 576), (8, 49, 128),
                                   (5, 200, 50), (130, 70, 300)])
def test_linear_simt(ops, dtype, shape):
    M, N, K = shape
    x = torch.randn(M, K).to(dtype).cuda()
    w = (torch.randn(N, K) / math.sqrt(K)).to(dtype).cuda()
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    same = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.linear_simt(x, w, same, ops.LINEAR_SAME)
    assert (same.double() - want).abs().max() <= tol(dtype) * scale
    f32 = torch.empty(M, N, device="cuda")
    ops.linear_simt(x, w, f32, ops.LINEAR_F32)
    assert (f32.double() - want).abs().max() <= 2e-5 * scale       # float32 sums of exact products in both dtypes
    acc = torch.ones(M, N, device="cuda")
    ops.linear_simt(x, w, acc, ops.LINEAR_ACC_F32)
    assert (acc.double() - 1 - want).abs().max() <= 2e-5 * scale
    if M <= 8:      # the same rows through the tile kernel agree to rounding
        tile = torch.empty(M, N, device="cuda")
        ops.linear_simt(x, w, tile, ops.LINEAR_F32, few_rows=0)
        assert (tile - f32).abs().max() <= 2e-5 * scale


@pytest.mark.parametrize("dtype", DT)
def test_linear_rows_do_not_depend_on_the_batch(ops, dtype):
    """A row's result is the same bits whatever else is in the batch (same kernel)."""
    x = torch.randn(40, 96).to(dtype).cuda()
    w = torch.randn(50, 96).to(dtype).cuda()
    a = torch.empty(40, 50, device="cuda")
    ops.linear_simt(x, w, a, ops.LINEAR_F32)
    b = torch.empty(13, 50, device="cuda")
    ops.linear_simt(x[20:33].contiguous(), w, b, ops.LINEAR_F32)
    assert torch.equal(a[20:33], b)
    xs = x[:, :64]                        # strided rows
    c = torch.empty(40, 50, device="cuda")
    ops.linear_simt(xs, w[:, :64].contiguous(), c, ops.LINEAR_F32)
    assert (c.double() - xs.double() @ w[:, :64].double().T).abs().max() < 1e-3


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,rot,ps", [(4, 2, 16, 16, 4), (3, 1, 32, 32, 8), (9, 3, 64, 64, 16), (5, 5, 48, 32, 16), (2, 1, 80, 80, 3)])
def test_rope_store(ops, dtype, nh, nkv, hd, rot, ps):
    T, pages = 11, 9
    qkv = torch.randn(T, (nh + 2 * nkv) * hd).to(dtype)
    positions = np.array([0, 1, 2, 77, 5, 300, 6, 7, 8, 9, 10], dtype=np.int32)
    cos, sin = P.rope_tables(np.arange(400), rot, 50000.0)
    slots = np.random.default_rng(0).permutation(pages * ps)[:T].astype(np.int32)
    slots[4] = -1
    cache = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
    q_out = torch.empty(T, nh * hd, dtype=dtype, device="cuda")
    ops.rope_store(qkv.cuda(), dev(positions), dev(cos), dev(sin), dev(slots), q_out, cache, nh, nkv, hd, rot, ps)
    f = qkv.float().numpy()
    q = f[:, :nh * hd].reshape(T, nh, hd)
    k = f[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    v = f[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    c, s = cos[positions], sin[positions]

    def rotate(a):
        out = a.copy()
        out[..., :rot] = P.rope_half(a[..., :rot], c, s)
        return out
    qr, kr = rotate(q), rotate(k)
    t = tol(dtype) * 4
    assert np.abs(q_out.float().cpu().numpy().reshape(T, nh, hd) - qr).max() <= t
    got = cache.float().cpu().numpy()
    touched = np.zeros((pages, ps), bool)
    for i in range(T):
        if slots[i] < 0:
            continue
        pg, off = slots[i] // ps, slots[i] % ps
        touched[pg, off] = True
        assert np.abs(got[pg, 0, :, off, :] - kr[i]).max() <= t
        assert np.abs(got[pg, 1, :, off, :] - v[i]).max() <= t
    untouched = got.transpose(0, 3, 1, 2, 4)[~touched]
    assert np.all(untouched == 7.0)           # no slot but the tokens' own was written


def _paged(k, v, ps, pages, rng, dtype):
    """Scatter k, v [n, nkv, hd] into a pool through a shuffled block table."""
    n, nkv, hd = k.shape
    nb = -(-n // ps)
    table = rng.permutation(pages)[:nb].astype(np.int32)
    cache = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype)
    cache += 1000.0      # a read outside the request's own slots shows
    for p in range(n):
        cache[table[p // ps], 0, :, p % ps] = torch.from_numpy(k[p]).to(dtype)
        cache[table[p // ps], 1, :, p % ps] = torch.from_numpy(v[p]).to(dtype)
    return cache.cuda(), table


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 4, 0), (3, 1, 32, 8, 0), (9, 3, 64, 16, 0), (6, 2, 48, 16, 0),
                                                 (2, 2, 80, 5, 0), (8, 1, 256, 16, 0), (4, 2, 16, 4, 5), (3, 3, 64, 16, 130)])
def test_attention_rows_mixed_batch(ops, dtype, nh, nkv, hd, ps, window):
    """Three requests in one batch: a decoded token far into a context, a prompt portion in mid-request,
    and a whole short prompt.  Scores are made sharp so that one wrong key changes the result."""
    rng = np.random.default_rng(3)
    lens = [301, 140, 9]                    # context after the step
    news = [1, 37, 9]                       # tokens of this step
    pages = sum(-(-n // ps) for n in lens) + 7
    pool = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype) + 1000.0
    free = list(rng.permutation(pages))
    maxb = max(-(-n // ps) for n in lens)
    bt = np.zeros((3, maxb), dtype=np.int32)
    q_all, seg, pos, want = [], [], [], []
    for s, (n, new) in enumerate(zip(lens, news)):
        k = (rng.standard_normal((n, nkv, hd)) * 2.0).astype(np.float32)
        v = rng.standard_normal((n, nkv, hd)).astype(np.float32)
        q = (rng.standard_normal((n, nh, hd)) * 2.0).astype(np.float32)
        if s == 0:      # one far key stands out for the decoded token
            k[3] = q[n - 1, 0::max(1, nh // nkv)][:nkv] * 3.0
        k = torch.from_numpy(k).to(dtype).float().numpy()
        v = torch.from_numpy(v).to(dtype).float().numpy()
        q = torch.from_numpy(q).to(dtype).float().numpy()
        for b in range(-(-n // ps)):
            bt[s, b] = free.pop()
        for p in range(n):
            pool[bt[s, p // ps], 0, :, p % ps] = torch.from_numpy(k[p]).to(dtype)
            pool[bt[s, p // ps], 1, :, p % ps] = torch.from_numpy(v[p]).to(dtype)
        ref = P.causal_attention(q, k, v, window=window or None).reshape(n, nh * hd)
        for p in range(n - new, n):
            q_all.append(q[p].reshape(-1)); seg.append(s); pos.append(p); want.append(ref[p])
    q_all = torch.from_numpy(np.stack(q_all)).to(dtype).cuda()
    out = torch.empty_like(q_all)
    ops.attention_rows(q_all, pool.cuda(), dev(bt), dev(np.array(seg, np.int32)), dev(np.array(pos, np.int32)), out, nh, nkv,
                       hd, 1.0 / math.sqrt(hd), window)
    want = np.stack(want)
    err = np.abs(out.float().cpu().numpy() - want).max()
    assert err <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, np.abs(want).max()), err


@pytest.mark.parametrize("dtype", DT)
def test_attention_window_edge(ops, dtype):
    """The key just inside the window is read, the key just outside is not."""
    nh = nkv = 1; hd = 16; ps = 4; n = 40; window = 8
    k = np.zeros((n, 1, hd), np.float32); v = np.zeros((n, 1, hd), np.float32)
    q = np.zeros((1, hd), np.float32); q[0, 0] = 8.0
    pos = n - 1
    k[pos - window + 1, 0, 0] = 8.0; v[pos - window + 1, 0, 1] = 1.0       # inside, strong
    k[pos - window, 0, 0] = 16.0; v[pos - window, 0, 2] = 1.0               # outside, stronger
    cache, table = _paged(k, v, ps, 20, np.random.default_rng(0), dtype)
    out = torch.empty(1, hd, dtype=dtype, device="cuda")
    ops.attention_rows(dev(q, dtype), cache, dev(table[None, :]), dev(np.array([0], np.int32)), dev(np.array([pos], np.int32)),
                       out, nh, nkv, hd, 0.25, window)
    o = out.float().cpu().numpy()[0]
    assert o[1] > 0.99 and abs(o[2]) < 1e-6


@pytest.mark.parametrize("dtype", DT)
def test_silu_mul(ops, dtype):
    gu = (torch.randn(7, 2 * 93) * 3).to(dtype).cuda()
    out = torch.empty(7, 93, dtype=dtype, device="cuda")
    ops.silu_mul(gu, out)
    g, u = gu.float()[:, :93], gu.float()[:, 93:]
    want = g / (1 + torch.exp(-g)) * u
    assert (out.float() - want).abs().max() <= tol(dtype) * want.abs().max()


def test_add_inplace(ops):
    y = torch.randn(1000, device="cuda"); x = torch.randn(1000, device="cuda"); y0 = y.clone()
    ops.add_inplace(y, x)
    assert torch.equal(y, y0 + x)
    xb = x.to(torch.bfloat16)
    ops.add_inplace(y, xb)
    assert torch.equal(y, y0 + x + xb.float())


def test_argmax_takes_the_lowest_id_of_equal_maxima(ops):
    l = torch.randn(5, 49155).cuda()
    l[0, 777] = 50.0; l[0, 40000] = 50.0; l[0, 12] = 50.0
    l[1, 49154] = 60.0
    l[2, 0] = 60.0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax_rows(l, out)
    assert out.tolist()[:3] == [12, 49154, 0]
    assert out.tolist()[3:] == l[3:].argmax(-1).tolist()


@pytest.mark.parametrize("vocab", [384, 49152, 1000])
def test_sample_rows_matches_the_plain_sampler(ops, vocab):
    rng = np.random.default_rng(9)
    settings = [(0.0, 0, 1.0), (0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.5), (0.8, 1, 1.0), (0.8, 0, 1e-6), (2.0, 0, 0.999)]
    rows = len(settings) * 4
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    logits[5, 100:110] = logits[5, 100]          # equal probabilities: the lower id comes first
    temp = np.array([settings[r % len(settings)][0] for r in range(rows)], np.float32)
    top_k = np.array([settings[r % len(settings)][1] for r in range(rows)], np.int32)
    top_p = np.array([settings[r % len(settings)][2] for r in range(rows)], np.float32)
    sampler = P.PlainSampler(1234)
    u = np.array([sampler.uniform() for _ in range(rows)], np.float64)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    scratch = torch.empty(rows * vocab, device="cuda")
    ops.sample_rows(dev(logits), dev(temp), dev(top_k), dev(top_p), dev(u), scratch, out)
    got = out.tolist()
    for r in range(rows):
        if temp[r] <= 0:
            assert got[r] == int(np.argmax(logits[r]))
            continue
        order, p, keep, mass = sampler.distribution(logits[r], float(temp[r]), int(top_k[r]), float(top_p[r]))
        cum = np.cumsum(p[:keep])
        target = u[r] * mass
        hit = np.nonzero(target < cum)[0]
        want = int(order[hit[0]] if len(hit) else order[keep - 1])
        if got[r] != want:
            # only when u falls within rounding of a boundary of the cumulative distribution
            i = list(order[:keep]).index(got[r]) if got[r] in order[:keep] else -1
            assert i >= 0 and min(abs(target - cum[i]), abs(target - (cum[i - 1] if i else 0.0))) < 1e-6, (r, got[r], want)


def test_sampling_proportions(ops):
    vocab, rows = 50, 4000
    logits = np.tile(np.linspace(-2, 2, vocab).astype(np.float32), (rows, 1))
    s = P.PlainSampler(5)
    u = np.array([s.uniform() for _ in range(rows)], np.float64)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample_rows(dev(logits), dev(np.full(rows, 1.0, np.float32)), dev(np.zeros(rows, np.int32)),
                    dev(np.ones(rows, np.float32)), dev(u), torch.empty(rows * vocab, device="cuda"), out)
    freq = np.bincount(out.cpu().numpy(), minlength=vocab) / rows
    p = np.exp(logits[0] - logits[0].max()); p /= p.sum()
    assert np.abs(freq - p).max() < 0.02


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 4, 0), (3, 1, 32, 8, 0), (9, 3, 64, 16, 0), (6, 2, 48, 16, 0),
                                                 (2, 2, 80, 5, 0), (18, 2, 128, 16, 0), (8, 1, 256, 16, 0), (4, 2, 16, 4, 5),
                                                 (3, 3, 64, 16, 300), (9, 3, 64, 16, 700),
                                                 # groups of 5, 7 and 8 heads: the routine with the keys as rows, its last
                                                 # pair of heads half used, and full; 12: the one with the heads as rows
                                                 (10, 2, 64, 16, 0), (7, 1, 32, 16, 0), (16, 2, 64, 8, 300), (12, 1, 64, 16, 0)])
def test_attention_decode_split_keys(ops, dtype, nh, nkv, hd, ps, window):
    """Single decoded tokens at contexts that end inside the first run of 256 keys, exactly on a run's edge,
    just past it, and far beyond; one key made to stand out in each; listed among tokens that are not run."""
    if not ops.attention_decode_takes(dtype, hd):
        pytest.skip("the split-key kernel does not take this head size in this dtype; attention_rows does")
    rng = np.random.default_rng(8)
    lens = [1, 7, 256, 257, 600, 1023]
    pages = sum(-(-n // ps) for n in lens) + 5
    pool = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype) + 1000.0
    free = list(rng.permutation(pages))
    maxb = max(-(-n // ps) for n in lens)
    bt = np.zeros((len(lens), maxb), dtype=np.int32)
    qs, want = [], []
    g = nh // nkv
    for s, n in enumerate(lens):
        k = (rng.standard_normal((n, nkv, hd)) * 1.5).astype(np.float32)
        v = rng.standard_normal((n, nkv, hd)).astype(np.float32)
        q = (rng.standard_normal((1, nh, hd)) * 1.5).astype(np.float32)
        far = min(n - 1, 3 if s % 2 else max(0, n - 260))
        k[far] = q[0, ::g][:nkv] * 2.0
        k, v, q = (torch.from_numpy(a).to(dtype).float().numpy() for a in (k, v, q))
        for b in range(-(-n // ps)):
            bt[s, b] = free.pop()
        kk = torch.from_numpy(k).to(dtype); vv = torch.from_numpy(v).to(dtype)
        for p in range(n):
            pool[bt[s, p // ps], 0, :, p % ps] = kk[p]
            pool[bt[s, p // ps], 1, :, p % ps] = vv[p]
        lo = max(0, n - window) if window else 0
        ref = P.causal_attention(np.concatenate([np.zeros((n - 1 - lo, nh, hd), np.float32), q]), k[lo:], v[lo:])[-1]
        qs.append(q.reshape(-1)); want.append(ref)
    # tokens 0, 2, 4, ... are the decoded ones; odd tokens are fillers that must be left alone
    T = 2 * len(lens)
    q_all = torch.zeros(T, nh * hd, dtype=dtype)
    q_all[0::2] = torch.from_numpy(np.stack(qs)).to(dtype)
    seg = np.repeat(np.arange(len(lens), dtype=np.int32), 2)
    pos = np.repeat(np.array(lens, np.int32) - 1, 2)
    out = torch.full((T, nh * hd), 5.0, dtype=dtype, device="cuda")
    cap, max_ctx = 8, 2048
    scratch = torch.zeros(ops.attention_decode_scratch_bytes(cap, nh, nkv, hd, max_ctx), dtype=torch.uint8, device="cuda")
    args = (q_all.cuda(), pool.cuda(), dev(bt), dev(seg), dev(pos))
    tok = dev(np.arange(0, T, 2, dtype=np.int32))
    for launch in range(2):          # twice: the scratch is left ready for the next launch
        out.fill_(5.0)
        ops.attention_decode(*args, out, scratch, cap, nh, nkv, hd, 1.0 / math.sqrt(hd), max_ctx, 1024 if launch else 2048,
                             window, tok)
        got = out.float().cpu().numpy()
        assert np.all(got[1::2] == 5.0)
        err = np.abs(got[0::2] - np.stack(want)).max()
        assert err <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, np.abs(np.stack(want)).max()), (launch, err)
    rows = torch.empty_like(out)
    ops.attention_rows(*args, rows, nh, nkv, hd, 1.0 / math.sqrt(hd), window, tok)
    assert (rows.float()[0::2] - out.float()[0::2]).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("simt", [False, True])
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,N,K", [(1, 50, 64), (3, 131, 576), (8, 960, 576), (9, 49, 128), (20, 200, 1536), (64, 96, 72),
                                   (5, 34, 8200), (33, 77, 960), (64, 130, 2048), (7, 40, 544), (2, 18, 12288)])
def test_linear_skinny_plain_epilogues(ops, dtype, M, N, K, simt):
    """Both few-rows kernels: CUDA cores (float32, and bfloat16 at sizes the other refuses) and tensor cores
    (bfloat16, K a multiple of 32)."""
    x = torch.randn(M, K).to(dtype).cuda()
    w = (torch.randn(N, K) / math.sqrt(K)).to(dtype).cuda()
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    same = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.linear_skinny(x, w, same, ops.EPI_SAME, force_simt=simt)
    assert (same.double() - want).abs().max() <= tol(dtype) * scale
    f32 = torch.empty(M, N, device="cuda")
    ops.linear_skinny(x, w, f32, ops.EPI_F32, force_simt=simt)
    assert (f32.double() - want).abs().max() <= 2e-5 * scale
    acc = torch.ones(M, N, device="cuda")
    ops.linear_skinny(x, w, acc, ops.EPI_ACC, force_simt=simt)
    assert (acc.double() - 1 - want).abs().max() <= 2e-5 * scale
    one = torch.empty(1, N, device="cuda")                 # a row alone gives the same bits as in the batch
    ops.linear_skinny(x[M - 1:M].contiguous(), w, one, ops.EPI_F32, force_simt=simt)
    assert torch.equal(one[0], f32[M - 1])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,K", [(1, 576), (8, 96), (13, 8200), (40, 1536), (3, 88)])
def test_linear_skinny_with_norm_and_rows(ops, dtype, M, K):
    N, rows_total = 70, 90
    x = (torch.randn(rows_total, K) * 2).cuda()
    nw = (1 + 0.1 * torch.randn(K)).cuda()
    w = (torch.randn(N, K) / math.sqrt(K)).to(dtype).cuda()
    rows = torch.randperm(rows_total)[:M].to(torch.int32).cuda()
    xn = torch.empty(M, K, dtype=dtype, device="cuda")
    ops.rmsnorm_rows(x, nw, 1e-5, xn, rows)                 # the unfused path rounds the same way
    want = xn.double() @ w.double().T
    got = torch.empty(M, N, device="cuda")
    ops.linear_skinny(x, w, got, ops.EPI_F32, norm_weight=nw, eps=1e-5, rows=rows)
    assert (got.double() - want).abs().max() <= (2e-5 if dtype == torch.float32 else 6e-3) * float(want.abs().max())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("K", [80, 576])
def test_linear_skinny_swiglu(ops, dtype, K):
    M, I = 7, 93
    x = (torch.randn(M, K) * 2).cuda()
    nw = torch.ones(K).cuda()
    w = (torch.randn(2 * I, K) / math.sqrt(K) * 2).to(dtype).cuda()
    xn = torch.empty(M, K, dtype=dtype, device="cuda")
    ops.rmsnorm_rows(x, nw, 1e-6, xn)
    gu = torch.empty(M, 2 * I, dtype=dtype, device="cuda")
    ops.linear_simt(xn, w, gu, ops.LINEAR_SAME)
    want = torch.empty(M, I, dtype=dtype, device="cuda")
    ops.silu_mul(gu, want)
    got = torch.empty(M, I, dtype=dtype, device="cuda")
    ops.linear_skinny(x, w, got, ops.EPI_SWIGLU, norm_weight=nw, eps=1e-6)
    assert (got.float() - want.float()).abs().max() <= tol(dtype) * float(want.float().abs().max())
    got2 = torch.empty(M, I, dtype=dtype, device="cuda")
    ops.linear_skinny(xn, w, got2, ops.EPI_SWIGLU)
    assert (got2.float() - want.float()).abs().max() <= tol(dtype) * float(want.float().abs().max())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 4), (3, 1, 32, 8), (9, 3, 64, 16), (2, 2, 80, 3)])
@pytest.mark.parametrize("K", [96, 72])
def test_linear_skinny_rope_store_matches_the_separate_kernels(ops, dtype, nh, nkv, hd, ps, K):
    M, pages = 6, 9
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(M, K) * 2).cuda()
    nw = (1 + 0.1 * torch.randn(K)).cuda()
    w = (torch.randn(N, K) / math.sqrt(K) * 2).to(dtype).cuda()
    positions = dev(np.array([0, 1, 77, 300, 5, 6], dtype=np.int32))
    cos, sin = P.rope_tables(np.arange(400), hd, 50000.0)
    slots = np.random.default_rng(1).permutation(pages * ps)[:M].astype(np.int32)
    slots[2] = -1
    xn = torch.empty(M, K, dtype=dtype, device="cuda")
    ops.rmsnorm_rows(x, nw, 1e-5, xn)
    qkv = torch.empty(M, N, dtype=dtype, device="cuda")
    ops.linear_simt(xn, w, qkv, ops.LINEAR_SAME)
    cache_a = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
    q_a = torch.empty(M, nh * hd, dtype=dtype, device="cuda")
    ops.rope_store(qkv, positions, dev(cos), dev(sin), dev(slots), q_a, cache_a, nh, nkv, hd, hd, ps)
    cache_b = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
    q_b = torch.empty(M, nh * hd, dtype=dtype, device="cuda")
    ops.linear_skinny(x, w, q_b, ops.EPI_ROPE, norm_weight=nw, eps=1e-5,
                      rope=(positions, dev(cos), dev(sin), dev(slots), cache_b, nh, nkv, hd))
    t = tol(dtype) * 4 * float(q_a.float().abs().max())
    assert (q_a.float() - q_b.float()).abs().max() <= t
    assert (cache_a.float() - cache_b.float()).abs().max() <= t
    assert torch.equal(cache_a == 7.0, cache_b == 7.0)        # the same slots were written, no others


@pytest.mark.parametrize("M,N,K", [(8, 5000, 2048), (3, 700, 8192), (16, 4100, 960), (40, 1200, 576), (5, 130, 8224), (7, 40, 544),
                                   (1, 18, 64), (64, 960, 1536), (11, 333, 12288)])
def test_the_streaming_few_rows_kernel_gives_the_bits_of_the_plain_one(ops, M, N, K):
    """The streaming kernel (weights kept on their way across tiles) against the tensor-core few-rows kernel that asks
    tile by tile, every epilogue, forced on at sizes its own rule would not take: the same bits, and both near float64."""
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=gen).to(dtype).cuda()
    xf = (torch.randn(M + 3, K, generator=gen) * 2).cuda()
    nw = (1 + 0.1 * torch.randn(K, generator=gen)).cuda()
    rows = torch.randperm(M + 3, generator=gen)[:M].to(torch.int32).cuda()
    N2 = N + (N % 2)
    w = (torch.randn(N2, K, generator=gen) / math.sqrt(K)).to(dtype).cuda()
    fused = ops.fused_norm_takes(dtype, M, K, N2)
    nh, nkv, hd, ps = 3, 1, 16, 4
    wq = (torch.randn((nh + 2 * nkv) * hd, K, generator=gen) / math.sqrt(K)).to(dtype).cuda()
    positions = dev(np.arange(M, dtype=np.int32) * 3)
    cos, sin = P.rope_tables(np.arange(3 * M + 1), hd, 10000.0)
    slots = dev(np.random.default_rng(M).permutation(M * 2)[:M].astype(np.int32))

    def run(mode):
        was = ops.set_skinny_stream(mode)
        try:
            outs = []
            f32 = torch.empty(M, N2, device="cuda")
            ops.linear_skinny(x, w, f32, ops.EPI_F32); outs.append(f32)
            acc = torch.ones(M, N2, device="cuda")
            ops.linear_skinny(x, w, acc, ops.EPI_ACC); outs.append(acc)
            same = torch.empty(M, N2, dtype=dtype, device="cuda")
            ops.linear_skinny(x, w, same, ops.EPI_SAME); outs.append(same)
            sw = torch.empty(M, N2 // 2, dtype=dtype, device="cuda")
            ops.linear_skinny(x, w, sw, ops.EPI_SWIGLU); outs.append(sw)
            cache = torch.full((M, 2, nkv, ps, hd), 7.0, dtype=dtype, device="cuda")
            q = torch.empty(M, nh * hd, dtype=dtype, device="cuda")
            ops.linear_skinny(x, wq, q, ops.EPI_ROPE, rope=(positions, dev(cos), dev(sin), slots, cache, nh, nkv, hd))
            outs += [q, cache]
            if fused:
                nf = torch.empty(M, N2, device="cuda")
                ops.linear_skinny(xf, w, nf, ops.EPI_F32, norm_weight=nw, eps=1e-5, rows=rows); outs.append(nf)
                ns = torch.empty(M, N2 // 2, dtype=dtype, device="cuda")
                ops.linear_skinny(xf, w, ns, ops.EPI_SWIGLU, norm_weight=nw, eps=1e-5, rows=rows); outs.append(ns)
            torch.cuda.synchronize()
            return outs
        finally:
            ops.set_skinny_stream(was)

    plain, stream = run(0), run(1)
    for i, (a, b) in enumerate(zip(plain, stream)):
        assert torch.equal(a, b), (i, float((a.float() - b.float()).abs().max()))
    want = x.double() @ w.double().T
    assert (stream[0].double() - want).abs().max() <= 2e-5 * float(want.abs().max())


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (128, 128, 576), (2048, 960, 576), (300, 576, 1536), (65, 200, 72), (1000, 3072, 576),
                                   (257, 49152, 576), (130, 72, 200), (700, 1100, 520), (1500, 2048, 2048)])   # the last three of the big ones: 128 x 256 tiles
def test_linear_tcgen05(ops, M, N, K):
    """The tcgen05 product against float64, and against the CUDA-core kernel (same exact products, float32 sums)."""
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K) / math.sqrt(K)).to(torch.bfloat16).cuda()
    want = x.double() @ w.double().T
    scale = float(want.abs().max())
    f32 = torch.full((M, N), 7.0, device="cuda")
    ops.linear_tcgen05(x, w, f32, ops.LINEAR_F32)
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert (f32.double() - want).abs().max() <= 2e-5 * scale
    same = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05(x, w, same, ops.LINEAR_SAME)
    assert (same.double() - want).abs().max() <= 1e-2 * scale
    acc = torch.ones(M, N, device="cuda")
    ops.linear_tcgen05(x, w, acc, ops.LINEAR_ACC_F32)
    assert (acc.double() - 1 - want).abs().max() <= 2e-5 * scale
    part = torch.empty(3, N, device="cuda")                  # rows alone (another tile position) give the same bits
    xs = torch.zeros(131, K, dtype=torch.bfloat16, device="cuda")
    xs[128:131] = x[M - 3:M]
    big = torch.empty(131, N, device="cuda")
    ops.linear_tcgen05(xs, w, big, ops.LINEAR_F32)
    assert torch.equal(big[128:131], f32[M - 3:M])
    torch.cuda.synchronize()
    ops.check_device_errors()


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 4, 0), (3, 1, 32, 8, 0), (9, 3, 64, 16, 0), (6, 2, 96, 16, 0), (4, 1, 128, 16, 0),
                                                 (4, 2, 16, 4, 5), (3, 3, 64, 16, 70), (2, 1, 64, 8, 200)])
def test_attention_prefill_tiles(ops, nh, nkv, hd, ps, window):
    """Prompt portions on the tensor cores: a whole prompt of 150 tokens, a portion of 37 tokens in mid-request
    (positions 103..139, across a boundary of 64), a portion of 2 tokens far into a context, and a portion that
    starts exactly at a multiple of 64.  Sharp scores; against the plain attention and against attention_rows."""
    _prefill_case(ops, ops.attention_prefill, 64, nh, nkv, hd, ps, window, [150, 140, 601, 128 + 70], [150, 37, 2, 70])


@pytest.fixture(params=[0, 1], ids=["two_threads_a_row", "two_streams"])
def prefill_kernel(ops, request):
    """Both tcgen05 prompt-attention kernels, whatever the launcher's size rule would take."""
    was = ops.set_prefill_streams(request.param)
    yield request.param
    ops.set_prefill_streams(was)


@pytest.mark.parametrize("nh,nkv,ps,window", [(9, 3, 16, 0), (4, 4, 8, 0), (2, 1, 32, 0), (6, 2, 64, 0), (3, 1, 128, 0),
                                              (3, 3, 16, 70), (2, 1, 8, 200)])
def test_attention_prefill_tcgen05(ops, prefill_kernel, nh, nkv, ps, window):
    """The same on the fifth-generation tensor cores (head size 64, tiles of up to 128 tokens), both kernels: a whole
    prompt of 300 tokens, portions in mid-request across boundaries of 64 and 128, two tokens far into a context, a
    portion that ends exactly at a multiple of 64, and pages of many sizes.  Unused slots of the pages hold 1000."""
    _prefill_case(ops, ops.attention_prefill_tcgen05, 128, nh, nkv, 64, ps, window, [300, 140, 601, 128 + 70, 448], [300, 37, 2, 70, 200])


@pytest.mark.parametrize("nh,nkv,ps,window", [(3, 1, 16, 0), (2, 2, 32, 0), (2, 1, 16, 1500)])
def test_attention_prefill_tcgen05_cuts_long_walks_into_parts(ops, prefill_kernel, nh, nkv, ps, window):
    """Tiles whose walk over the keys is longer than 16 steps of 64 are cut into parts that different blocks take and the
    last to arrive adds up: portions at the end of contexts of 2,300 and 4,000 positions (three and four parts), a whole
    prompt of 1,025 tokens (its last tile has one row, whose second part is a single key), a walk of exactly 16 steps, and
    a window that shortens the walk.  Run twice over the same scratch (the counters return to zero).  Both kernels."""
    for _ in range(2):
        _prefill_case(ops, ops.attention_prefill_tcgen05, 128, nh, nkv, 64, ps, window, [2300, 1100, 1025, 4000, 1024], [300, 70, 1025, 2, 128])


def test_attention_prefill_tcgen05_takes_the_kernel_by_the_size_of_the_launch(ops):
    """A launch of 32 heads and 13 tiles (416 blocks: the first kernel) and one of 8 heads (104 blocks: two streams) give
    the same result as each kernel forced on the same operands, to rounding: the size rule only chooses."""
    torch.manual_seed(5)
    hd, ps, T = 64, 16, 13 * 128
    pages = T // ps + 3
    for nh, nkv in ((32, 8), (8, 8)):
        pool = torch.randn(pages, 2, nkv, ps, hd, device="cuda").to(torch.bfloat16)
        bt = torch.randperm(pages, device="cuda")[: T // ps].to(torch.int32)[None, :].contiguous()
        q = torch.randn(T, nh * hd, device="cuda").to(torch.bfloat16)
        tiles = dev(np.asarray([(o, 128, o, 0) for o in range(0, T, 128)], np.int32))
        outs = []
        for mode in (2, 0, 1):
            was = ops.set_prefill_streams(mode)
            try:
                out = torch.empty_like(q)
                ops.attention_prefill_tcgen05(q, pool, bt, tiles, out, nh, nkv, hd, 0.125, 0)
                torch.cuda.synchronize()
                ops.check_device_errors()
                outs.append(out.float())
            finally:
                ops.set_prefill_streams(was)
        scale = float(outs[0].abs().max())
        assert (outs[0] - outs[1]).abs().max() <= 2e-2 * scale and (outs[0] - outs[2]).abs().max() <= 2e-2 * scale
        assert torch.equal(outs[0], outs[1] if nh == 32 else outs[2])        # the rule took the kernel this size stands for


def test_attention_prefill_tcgen05_refuses_what_it_does_not_take(ops):
    """Pages of 4 slots (a TMA box must be a multiple of eight 128-byte rows) and head sizes other than 64 are refused
    with a clear error; the dispatcher then takes the mma.sync kernel."""
    q = torch.zeros(8, 2 * 64, dtype=torch.bfloat16, device="cuda")
    tiles = dev(np.asarray([(0, 8, 0, 0)], np.int32))
    bt = dev(np.zeros((1, 4), np.int32))
    small_pages = torch.zeros(4, 2, 1, 4, 64, dtype=torch.bfloat16, device="cuda")
    assert not ops.attention_prefill_tcgen05_takes(q, small_pages, 64)
    with pytest.raises(ops.KernelError):
        ops.attention_prefill_tcgen05(q, small_pages, bt, tiles, torch.empty_like(q), 2, 1, 64, 0.125, 0)
    q32 = torch.zeros(8, 2 * 32, dtype=torch.bfloat16, device="cuda")
    pages32 = torch.zeros(4, 2, 1, 16, 32, dtype=torch.bfloat16, device="cuda")
    assert not ops.attention_prefill_tcgen05_takes(q32, pages32, 32)
    with pytest.raises(ops.KernelError):
        ops.attention_prefill_tcgen05(q32, pages32, bt, tiles, torch.empty_like(q32), 2, 1, 32, 0.125, 0)


def _prefill_case(ops, kernel, tile_rows, nh, nkv, hd, ps, window, lens, news):
    """lens: context after the step; news: tokens of this step."""
    rng = np.random.default_rng(6)
    dtype = torch.bfloat16
    pages = sum(-(-n // ps) for n in lens) + 7
    pool = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype) + 1000.0
    free = list(rng.permutation(pages))
    maxb = max(-(-n // ps) for n in lens)
    bt = np.zeros((len(lens), maxb), dtype=np.int32)
    q_all, seg, pos, want, tiles = [], [], [], [], []
    g = nh // nkv
    for s, (n, new) in enumerate(zip(lens, news)):
        k = (rng.standard_normal((n, nkv, hd)) * 1.5).astype(np.float32)
        v = rng.standard_normal((n, nkv, hd)).astype(np.float32)
        q = (rng.standard_normal((n, nh, hd)) * 1.5).astype(np.float32)
        k[3] = q[n - 1, ::g][:nkv] * 2.0               # a far key stands out for the last query
        k, v, q = (torch.from_numpy(a).to(dtype).float().numpy() for a in (k, v, q))
        for b in range(-(-n // ps)):
            bt[s, b] = free.pop()
        kk = torch.from_numpy(k).to(dtype); vv = torch.from_numpy(v).to(dtype)
        for p in range(n):
            pool[bt[s, p // ps], 0, :, p % ps] = kk[p]
            pool[bt[s, p // ps], 1, :, p % ps] = vv[p]
        ref = P.causal_attention(q, k, v, window=window or None).reshape(n, nh * hd)
        start = len(q_all)
        for o in range(0, new, tile_rows):
            tiles.append((start + o, min(tile_rows, new - o), n - new + o, s))
        for p in range(n - new, n):
            q_all.append(q[p].reshape(-1)); seg.append(s); pos.append(p); want.append(ref[p])
    q_dev = torch.from_numpy(np.stack(q_all)).to(dtype).cuda()
    out = torch.empty_like(q_dev)
    kernel(q_dev, pool.cuda(), dev(bt), dev(np.asarray(tiles, np.int32)), out, nh, nkv, hd, 1.0 / math.sqrt(hd), window)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want = np.stack(want)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 3e-2 * max(1.0, np.abs(want).max())
    rows = torch.empty_like(q_dev)
    ops.attention_rows(q_dev, pool.cuda(), dev(bt), dev(np.array(seg, np.int32)), dev(np.array(pos, np.int32)), rows, nh, nkv, hd,
                       1.0 / math.sqrt(hd), window)
    assert (rows.float() - out.float()).abs().max() <= 3e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("M,I,K", [(128, 64, 64), (2048, 1536, 576), (300, 200, 72), (70, 8192, 2048), (600, 1096, 520)])
def test_linear_tcgen05_swiglu_matches_the_separate_kernels(ops, M, I, K):
    torch.manual_seed(M + I)
    x = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * I, K) / math.sqrt(K) * 2).to(torch.bfloat16).cuda()
    gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05(x, w, gu, ops.LINEAR_SAME)
    want = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    ops.silu_mul(gu, want)
    got = torch.full((M, I), 9.0, dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05_swiglu(x, w, got)
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert torch.equal(got, want)              # the same sums and the same rounding points
    g = (x.double() @ w[:I].double().T); u = (x.double() @ w[I:].double().T)
    ref = g / (1 + torch.exp(-g)) * u
    assert (got.double() - ref).abs().max() <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("nh,nkv,hd,ps,M,K", [(9, 3, 64, 16, 200, 576), (2, 1, 128, 8, 130, 96), (32, 32, 64, 16, 70, 2048),
                                              (15, 5, 64, 16, 600, 960), (6, 3, 128, 32, 520, 512)])   # the last two: 128 x 256 tiles
def test_linear_tcgen05_rope_matches_the_separate_kernels(ops, nh, nkv, hd, ps, M, K):
    torch.manual_seed(nh + M)
    N = (nh + 2 * nkv) * hd
    pages = -(-M // ps) + 3
    x = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K) / math.sqrt(K) * 2).to(torch.bfloat16).cuda()
    positions = dev(np.random.default_rng(1).integers(0, 900, M).astype(np.int32))
    cos, sin = P.rope_tables(np.arange(1000), hd, 100000.0)
    slots = np.random.default_rng(2).permutation(pages * ps)[:M].astype(np.int32)
    slots[5] = -1
    qkv = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05(x, w, qkv, ops.LINEAR_SAME)
    cache_a = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    q_a = torch.empty(M, nh * hd, dtype=torch.bfloat16, device="cuda")
    ops.rope_store(qkv, positions, dev(cos), dev(sin), dev(slots), q_a, cache_a, nh, nkv, hd, hd, ps)
    cache_b = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    q_b = torch.empty(M, nh * hd, dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05_rope(x, w, q_b, positions, dev(cos), dev(sin), dev(slots), cache_b, nh, nkv, hd)
    torch.cuda.synchronize()
    ops.check_device_errors()
    t = 1e-2 * float(q_a.float().abs().max())      # the rotation's float32 arithmetic may contract differently: one bfloat16 step
    assert (q_a.float() - q_b.float()).abs().max() <= t
    assert (cache_a.float() - cache_b.float()).abs().max() <= t
    assert torch.equal(cache_a == 7.0, cache_b == 7.0)


@pytest.mark.parametrize("family,M,N,K,stage", [("linear_tcgen05", 300, 200, 576, 0), ("linear_tcgen05", 300, 200, 576, 5),
                                                ("linear_tcgen05_wide", 1024, 2048, 2048, 1), ("linear_tcgen05_wide", 2048, 4096, 2048, 40)])
def test_linear_tcgen05_gives_up_a_wait_and_says_so(ops, family, M, N, K, stage):
    """The producer leaves one stage unarmed (a hook for this test; nothing faults): the waits on it run out after the
    5 ms set here, every block returns by itself with its tensor memory freed, the error word is set, and the next
    launch of the same kernel is right."""
    torch.manual_seed(1)
    x = torch.randn(M, K).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K) / math.sqrt(K)).to(torch.bfloat16).cuda()
    want = x.double() @ w.double().T
    out = torch.zeros(M, N, device="cuda")
    ops.set_wait_limit_ms(5.0)
    try:
        ops.skip_stage_once(family, stage)
        ops.linear_tcgen05(x, w, out, ops.LINEAR_F32)
        torch.cuda.synchronize()
        with pytest.raises(ops.KernelGaveUp):
            ops.check_device_errors()
    finally:
        ops.set_wait_limit_ms(0)
    ops.linear_tcgen05(x, w, out, ops.LINEAR_F32)          # the hook was for one launch
    torch.cuda.synchronize()
    ops.check_device_errors()
    assert (out.double() - want).abs().max() <= 2e-5 * float(want.abs().max())


@pytest.mark.parametrize("stage", [0, 2])
def test_attention_prefill_tcgen05_gives_up_a_wait_and_says_so(ops, prefill_kernel, stage):
    """The same for the prompt attention, both kernels: one step's keys never arrive; the tensor-core lanes, the softmax
    warps and the copying warps each give up within the limit, keep their appointments, and the block returns."""
    ops.set_wait_limit_ms(5.0)
    try:
        ops.skip_stage_once("attention_prefill_tcgen05", stage)
        with pytest.raises(ops.KernelGaveUp):
            _prefill_case(ops, ops.attention_prefill_tcgen05, 128, 4, 2, 64, 16, 0, [300, 448], [300, 200])
    finally:
        ops.set_wait_limit_ms(0)
    _prefill_case(ops, ops.attention_prefill_tcgen05, 128, 4, 2, 64, 16, 0, [300, 448], [300, 200])


@pytest.mark.parametrize("nh,nkv,ps,window,lens", [
    (9, 3, 16, 0, [1, 7, 256, 257, 600, 1023]),
    (4, 4, 8, 0, [31, 32, 33, 290, 1500]),
    (32, 2, 32, 0, [5, 64, 300, 2047]),                       # a group of 16 heads: one full tile of rows
    (40, 2, 16, 0, [100, 700]),                               # a group of 20 heads: two tiles a key-value head
    (6, 2, 64, 0, [63, 64, 65, 1000]),
    (3, 1, 128, 0, [200, 129, 3000]),
    (3, 3, 16, 300, [10, 299, 300, 301, 900, 2000]),
    (9, 3, 16, 700, [2048, 1700, 701]),
    (9, 3, 16, 0, [int(n) for n in np.random.default_rng(3).integers(1, 2300, 200)]),     # many more units than warps: the ring runs across units
    (16, 2, 16, 0, [40, 513, 1100]),                          # groups of 8, 7 and 5 heads: the keys as rows, all eight columns
    (7, 1, 16, 200, [64, 450, 1800]),                         # in use, and the last pair of heads half used
    (10, 2, 32, 0, [33, 700, 2049]),
])
def test_attention_decode_tma_streams_the_pages(ops, nh, nkv, ps, window, lens):
    """The persistent decode kernel (TMA boxes from the pages, a warp a unit, online softmax over chunks of 32 keys),
    forced for every launch: contexts that end inside a chunk, on the edge of a chunk, a split and a page, windows that
    begin inside a chunk, groups of more than 16 heads, pages of many sizes, and a batch of 200 tokens whose units
    outnumber the grid's warps.  One key is made to stand out in each request; unused slots hold 1000.  Against the
    plain attention, against the separate kernel, and twice over the same scratch."""
    hd, dtype = 64, torch.bfloat16
    rng = np.random.default_rng(8)
    pages = sum(-(-n // ps) for n in lens) + 5
    pool = torch.zeros(pages, 2, nkv, ps, hd, dtype=dtype) + 1000.0
    free = list(rng.permutation(pages))
    maxb = max(-(-n // ps) for n in lens)
    bt = np.zeros((len(lens), maxb), dtype=np.int32)
    qs, want = [], []
    g = nh // nkv
    for s, n in enumerate(lens):
        k = (rng.standard_normal((n, nkv, hd)) * 1.5).astype(np.float32)
        v = rng.standard_normal((n, nkv, hd)).astype(np.float32)
        q = (rng.standard_normal((1, nh, hd)) * 1.5).astype(np.float32)
        lo = max(0, n - window) if window else 0
        far = min(n - 1, lo + 3 if s % 2 else max(lo, n - 260))
        k[far] = q[0, ::g][:nkv] * 2.0
        k, v, q = (torch.from_numpy(a).to(dtype).float().numpy() for a in (k, v, q))
        blocks = [free.pop() for _ in range(-(-n // ps))]
        bt[s, :len(blocks)] = blocks
        kk = torch.from_numpy(k).to(dtype).reshape(n, nkv, hd); vv = torch.from_numpy(v).to(dtype).reshape(n, nkv, hd)
        for b, page in enumerate(blocks):
            m = min(ps, n - b * ps)
            pool[page, 0, :, :m] = kk[b * ps:b * ps + m].transpose(0, 1)
            pool[page, 1, :, :m] = vv[b * ps:b * ps + m].transpose(0, 1)
        # the one query against its keys: scores, softmax, p * v (a query of the last position sees every key from lo on)
        kf, vf = k[lo:], v[lo:]
        ref = np.zeros((nh, hd), np.float32)
        for h in range(nh):
            sc = (kf[:, h // g] @ q[0, h]) / np.float32(math.sqrt(hd))
            e = np.exp(sc - sc.max()); e /= e.sum()
            ref[h] = e @ vf[:, h // g]
        qs.append(q.reshape(-1)); want.append(ref.reshape(-1))
    T = len(lens)
    q_all = torch.from_numpy(np.stack(qs)).to(dtype).cuda()
    seg = np.arange(T, dtype=np.int32)
    pos = np.array(lens, np.int32) - 1
    max_ctx = 4096
    scratch = torch.zeros(ops.attention_decode_scratch_bytes(T, nh, nkv, hd, max_ctx), dtype=torch.uint8, device="cuda")
    args = (q_all, pool.cuda(), dev(bt), dev(seg), dev(pos))
    want = np.stack(want)
    scale = max(1.0, float(np.abs(want).max()))
    outs = {}
    before = ops.set_decode_tma(1)
    few_before = ops.set_decode_tma_few(1)
    try:
        # the streaming kernel (keys as rows for groups of at most eight), the separate kernel, the streaming kernel again on
        # the same scratch, and the streaming kernel with the heads as rows for every group
        for mode in (1, 0, 1, 3):
            ops.set_decode_tma(min(mode, 1))
            ops.set_decode_tma_few(0 if mode == 3 else 1)
            out = torch.full((T, nh * hd), 5.0, dtype=dtype, device="cuda")
            reach = -(-max(lens) // 256) * 256
            ops.attention_decode(*args, out, scratch, T, nh, nkv, hd, 1.0 / math.sqrt(hd), max_ctx, reach if mode else max_ctx, window)
            torch.cuda.synchronize()
            ops.check_device_errors()
            got = out.float().cpu().numpy()
            assert np.isfinite(got).all()
            assert np.abs(got - want).max() <= 2e-2 * scale, (mode, float(np.abs(got - want).max()))
            outs.setdefault(mode, got)
    finally:
        ops.set_decode_tma(before)
        ops.set_decode_tma_few(few_before)
    assert np.abs(outs[1] - outs[0]).max() <= 1e-2 * scale
    assert np.abs(outs[3] - outs[0]).max() <= 1e-2 * scale


def _rope_oracle(x, w, positions, cos, sin, slots, nh, nkv, hd, ps, pages):
    """q rotated [M, nh*hd] and the cache [pages, 2, nkv, ps, hd] (7.0 where nothing is written), in float64 from bfloat16
    inputs, rounding where the kernels store: the products to bfloat16, then the rotated values to bfloat16."""
    M = x.shape[0]
    qkv = P.bf16_round((x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32))
    q = qkv[:, :nh * hd].reshape(M, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(M, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].reshape(M, nkv, hd)
    c, s = cos[positions], sin[positions]
    q_rot = P.bf16_round(P.rope_half(q, c, s)).reshape(M, nh * hd)
    k_rot = P.bf16_round(P.rope_half(k, c, s))
    cache = np.full((pages, 2, nkv, ps, hd), 7.0, np.float32)
    for m, sl in enumerate(slots):
        if sl >= 0:
            cache[sl // ps, 0, :, sl % ps] = k_rot[m]
            cache[sl // ps, 1, :, sl % ps] = v[m]
    return q_rot, cache


@pytest.mark.parametrize("kind,nh,nkv,hd,ps,M,K", [("skinny", 9, 3, 64, 16, 6, 576), ("skinny", 4, 1, 128, 8, 40, 256),
                                                   ("skinny_norm", 9, 3, 64, 16, 5, 576), ("tcgen05", 9, 3, 64, 16, 300, 576),
                                                   ("tcgen05", 4, 2, 128, 8, 130, 256), ("tcgen05", 32, 32, 64, 16, 1100, 2048)])
def test_fused_rotary_epilogues_against_a_plain_statement(ops, kind, nh, nkv, hd, ps, M, K):
    """The projections with the rotation and the cache write in their epilogue (few-rows kernel, with and without the
    fused norm; tcgen05 product, narrow and wide): q and every slot of the cache against float64 products rounded where
    the kernels round; slots that are not named stay as they were, a token with slot -1 writes nothing."""
    rng = np.random.default_rng(nh + M)
    N = (nh + 2 * nkv) * hd
    pages = -(-M // ps) + 3
    to_bf = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    w_t = to_bf(rng.standard_normal((N, K)) / math.sqrt(K) * 2)
    positions = rng.integers(0, 900, M).astype(np.int32)
    cos, sin = P.rope_tables(np.arange(1000), hd, 100000.0)
    slots = rng.permutation(pages * ps)[:M].astype(np.int32)
    slots[min(5, M - 1)] = -1
    cache = torch.full((pages, 2, nkv, ps, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    q_out = torch.empty(M, nh * hd, dtype=torch.bfloat16, device="cuda")
    if kind == "skinny_norm":
        xf = (rng.standard_normal((M, K)) * 2).astype(np.float32)
        nw = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
        x_np = P.bf16_round(P.rms_norm(xf, nw, 1e-5))
        ops.linear_skinny(dev(xf), w_t.cuda(), q_out, ops.EPI_ROPE, norm_weight=dev(nw), eps=1e-5,
                          rope=(dev(positions), dev(cos), dev(sin), dev(slots), cache, nh, nkv, hd))
    else:
        x_t = to_bf(rng.standard_normal((M, K)))
        x_np = x_t.float().numpy()
        if kind == "skinny":
            ops.linear_skinny(x_t.cuda(), w_t.cuda(), q_out, ops.EPI_ROPE,
                              rope=(dev(positions), dev(cos), dev(sin), dev(slots), cache, nh, nkv, hd))
        else:
            ops.linear_tcgen05_rope(x_t.cuda(), w_t.cuda(), q_out, dev(positions), dev(cos), dev(sin), dev(slots), cache, nh, nkv, hd)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want_q, want_cache = _rope_oracle(x_np, w_t.float().numpy(), positions, cos, sin, slots, nh, nkv, hd, ps, pages)
    got_q, got_cache = q_out.float().cpu().numpy(), cache.float().cpu().numpy()
    # one bfloat16 step of the largest value: a float32 sum that lands on the other side of a rounding point
    t = 2 ** -7 * max(1.0, float(np.abs(want_q).max()))
    assert np.abs(got_q - want_q).max() <= t
    assert np.array_equal(got_cache == 7.0, want_cache == 7.0)          # the same slots were written, no others
    assert np.abs(got_cache - want_cache).max() <= t
