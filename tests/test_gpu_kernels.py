"""Each kernel alone against a plain PyTorch restatement of the same op, at sizes other than
the tiny models' (odd widths, every head size in steps of 16, page edges, windows)."""
import math

import numpy as np
import pytest
import torch

from herbert_rs_b200 import ops
from herbert_rs_b200.errors import BackendError
from herbert_rs_b200.sampling import SamplingParams, host_sample, host_survivors
from plain_qwen3 import apply_rope, attention_scores, rms_norm, rope_tables, sample_distribution

pytestmark = pytest.mark.gpu
DT = [torch.float32, torch.bfloat16]


def dev(t):
    return t.cuda()


def close(got, ref, dtype, scale=1.0, rowwise=False):
    """|got - ref| <= tol * max(1, max|ref|); rowwise: <= tol * max|ref of that row| for every row, for
    outputs whose rows differ in size and are far below 1 (attention over many keys)."""
    got, ref = got.detach().double().cpu(), ref.double().cpu()
    rel = (2e-5 if dtype == torch.float32 else 1.2e-2) * scale
    if rowwise:
        err = (got - ref).abs().amax(dim=-1)
        lim = rel * ref.abs().amax(dim=-1)
        worst = int((err - lim).argmax())
        assert (err <= lim).all(), f"row {worst}: max error {err[worst]:.3e} > {lim[worst]:.3e}"
        return
    tol = rel * max(1.0, ref.abs().max().item())
    err = (got - ref).abs().max().item()
    assert err <= tol, f"max error {err:.3e} > {tol:.3e}"


def test_library_is_loaded_in_tree():
    from herbert_rs_b200.ops import lib
    lib.load()
    maps = open("/proc/self/maps").read()
    assert "libherbert_b200.so" in maps


@pytest.mark.parametrize("dtype", DT)
def test_embed(dtype):
    torch.manual_seed(0)
    table = torch.randn(301, 72).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 72, device="cuda")
    ops.embed(dev(table), dev(ids), out)
    assert torch.equal(out.cpu(), table[ids.long()].float())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("dim,eps", [(72, 1e-6), (1000, 1e-5), (4096, 1e-6), (33, 1e-3)])
def test_rmsnorm_and_gather(dtype, dim, eps):
    torch.manual_seed(1)
    x = torch.randn(9, dim) * 3
    w = 1 + 0.1 * torch.randn(dim)
    out = torch.empty(9, dim, device="cuda", dtype=dtype)
    ops.rmsnorm(dev(x), dev(w), out, eps)
    close(out, rms_norm(x.double(), w.double(), eps), dtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out2 = torch.empty(3, dim, device="cuda", dtype=dtype)
    ops.rmsnorm(dev(x), dev(w), out2, eps, dev(rows))
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("inter,interleave", [(24, 8), (172, 0), (1000, 8), (7, 0)])
def test_swiglu_layouts(dtype, inter, interleave):
    torch.manual_seed(2)
    g, u = (torch.randn(5, inter) * 2).to(dtype), torch.randn(5, inter).to(dtype)
    if interleave:
        gu = torch.cat([g.view(5, -1, 8), u.view(5, -1, 8)], dim=2).reshape(5, 2 * inter)
    else:
        gu = torch.cat([g, u], dim=1)
    out = torch.empty(5, inter, device="cuda", dtype=dtype)
    ops.swiglu(dev(gu.contiguous()), out, interleave)
    gd, ud = g.double(), u.double()
    close(out, gd / (1 + torch.exp(-gd)) * ud, dtype)
    with pytest.raises(BackendError, match="no multiple of the interleave"):
        ops.swiglu(dev(torch.zeros(1, 20, dtype=dtype)), torch.empty(1, 10, device="cuda", dtype=dtype), 8)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("M,N,K", [(1, 72, 96), (5, 100, 33), (70, 64, 64), (129, 301, 172), (64, 256, 1024)])
def test_gemm_simt_every_epilogue(dtype, M, N, K):
    torch.manual_seed(3)
    a, w = torch.randn(M, K).to(dtype), (torch.randn(N, K) * 0.1).to(dtype)
    ref = a.double() @ w.double().T
    c = torch.empty(M, N, device="cuda", dtype=dtype)
    ops.gemm_simt(dev(a), dev(w), c, ops.EPI_STORE)
    close(c, ref, dtype)
    c32 = torch.empty(M, N, device="cuda")
    ops.gemm_simt(dev(a), dev(w), c32, ops.EPI_STORE_F32)
    close(c32, ref, torch.float32, scale=1.0 if dtype == torch.float32 else 1.0)
    res = torch.randn(M, N)
    r = dev(res.clone())
    ops.gemm_simt(dev(a), dev(w), r, ops.EPI_RESIDUAL)
    close(r, res.double() + ref, torch.float32)
    # a padded leading dimension: only the first K columns of each row are read
    wide = torch.cat([a, torch.full((M, 5), 1e4).to(dtype)], dim=1)
    c2 = torch.empty(M, N, device="cuda", dtype=dtype)
    ops.gemm_simt(dev(wide)[:, :K], dev(w), c2, ops.EPI_STORE)
    assert torch.equal(c2, c)


def _paged(k, page, n_pages_total, perm_seed):
    """Scatter per-sequence [len, nkv, hd] tensors into a page pool in a shuffled page order.
    Returns (pool [pages, nkv, page, hd], table [B, P])."""
    B = len(k)
    nkv, hd = k[0].shape[1], k[0].shape[2]
    need = [-(-x.shape[0] // page) for x in k]
    P = max(need)
    order = torch.randperm(n_pages_total, generator=torch.Generator().manual_seed(perm_seed)).tolist()
    pool = torch.full((n_pages_total, nkv, page, hd), 777.0)        # poison: a stray read shows
    table = torch.zeros(B, P, dtype=torch.int32)
    for b, x in enumerate(k):
        for lp in range(need[b]):
            pg = order.pop()
            table[b, lp] = pg
            chunk = x[lp * page:(lp + 1) * page]
            pool[pg, :, :chunk.shape[0]] = chunk.transpose(0, 1)
    return pool, table


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,rot,norm", [(4, 2, 16, 16, True), (6, 3, 48, 24, True), (8, 1, 128, 128, False), (5, 5, 128, 128, True),
                                                (3, 3, 80, 80, True), (2, 1, 256, 64, True)])
def test_qk_norm_rope_cache_write(dtype, nh, nkv, hd, rot, norm):
    torch.manual_seed(4)
    page, eps = 16, 1e-5
    pos0, qlen = [0, 30, 15], [20, 3, 1]              # crosses page edges at 16 and 32
    B, T = 3, sum(qlen)
    tok_seq = torch.tensor(sum(([b] * n for b, n in enumerate(qlen)), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((list(range(p, p + n)) for p, n in zip(pos0, qlen)), []), dtype=torch.int32)
    qkv = (torch.randn(T, (nh + 2 * nkv) * hd + 8) * 2).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(hd), 1 + 0.1 * torch.randn(hd)
    cos, sin = rope_tables(rot, 10000.0, 64, torch.float32)
    table = torch.tensor([[5, 2, 0], [1, 7, 3], [4, 0, 0]], dtype=torch.int32)
    kc = torch.full((8, nkv, page, hd), 9.0).to(dtype).cuda()
    vc = torch.full((8, nkv, page, hd), 9.0).to(dtype).cuda()
    d_qkv = dev(qkv.clone())
    ops.qk_norm_rope_cache(d_qkv, dev(qw) if norm else None, dev(kw) if norm else None, eps, dev(cos), dev(sin), rot,
                           dev(tok_seq), dev(tok_pos), dev(table), kc, vc, nh, nkv, hd, page)
    x = qkv.double()[:, :(nh + 2 * nkv) * hd]
    q = x[:, :nh * hd].view(T, nh, hd)
    k = x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = x[:, (nh + nkv) * hd:].view(T, nkv, hd)
    if norm:
        q, k = rms_norm(q, qw.double(), eps), rms_norm(k, kw.double(), eps)
    c, s = cos.double()[tok_pos.long()], sin.double()[tok_pos.long()]
    q, k = apply_rope(q, c, s, rot), apply_rope(k, c, s, rot)
    close(d_qkv[:, :nh * hd], q.reshape(T, -1), dtype)
    assert torch.equal(d_qkv[:, nh * hd:].cpu(), qkv[:, nh * hd:])         # k, v columns and the padding stay
    written = torch.zeros(8, page, dtype=torch.bool)
    for t in range(T):
        b, p = tok_seq[t].item(), tok_pos[t].item()
        pg = table[b, p // page].item()
        close(kc[pg, :, p % page], k[t], dtype)
        assert torch.equal(vc[pg, :, p % page].cpu(), v[t].to(dtype))
        written[pg, p % page] = True
    untouched = lambda c: c.cpu().float().permute(0, 2, 1, 3)[~written]      # [pages, page, nkv, hd] rows never written
    assert (untouched(kc) == 9.0).all() and (untouched(vc) == 9.0).all()
    # a step that only reads another step's cache entry leaves it alone
    kc2, vc2 = kc.clone(), vc.clone()
    ops.qk_norm_rope_cache(dev(qkv.clone()), dev(qw) if norm else None, dev(kw) if norm else None, eps, dev(cos), dev(sin),
                           rot, dev(tok_seq), dev(tok_pos), dev(table), kc2.fill_(1.0), vc2.fill_(1.0), nh, nkv, hd, page,
                           write_cache=False)
    assert (kc2 == 1.0).all() and (vc2 == 1.0).all()


def _attention_case(dtype, nh, nkv, hd, lens, qlens, window, page=16, seed=5, sharp=None):
    """Random q/k/v for B sequences; the last qlen positions of each are this step's queries."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    ks = [torch.randn(n, nkv, hd, generator=g).to(dtype).float() for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g).to(dtype).float() for n in lens]
    qs = [torch.randn(n, nh, hd, generator=g).to(dtype).float() for n in lens]
    if sharp:
        for (b, qpos, h, kpos) in sharp:       # make key kpos stand out for query (b, qpos, h)
            kh = h // (nh // nkv)
            qs[b][qpos, h] = 0; qs[b][qpos, h, 3] = 12.0
            ks[b][:, kh, 3] = ks[b][:, kh, 3].clamp(-1, 1)
            ks[b][kpos, kh, 3] = 12.0
    scale = 1.0 / math.sqrt(hd)
    ref = [attention_scores(q.double(), k.double(), v.double(), scale, window)[n - ql:]
           for q, k, v, n, ql in zip(qs, ks, vs, lens, qlens)]
    kpool, table = _paged(ks, page, sum(-(-n // page) for n in lens) + 3, seed)
    vpool, _ = _paged(vs, page, sum(-(-n // page) for n in lens) + 3, seed)
    qrows = torch.cat([q[n - ql:] for q, n, ql in zip(qs, lens, qlens)]).reshape(-1, nh * hd)
    tok_seq = torch.tensor(sum(([b] * ql for b, ql in enumerate(qlens)), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((list(range(n - ql, n)) for n, ql in zip(lens, qlens)), []), dtype=torch.int32)
    return dict(q=qrows.to(dtype), k=kpool.to(dtype), v=vpool.to(dtype), table=table, tok_seq=tok_seq, tok_pos=tok_pos,
                ref=torch.cat(ref).reshape(-1, nh * hd), scale=scale, vs=vs)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 3, 48), (8, 1, 128), (5, 5, 80), (12, 4, 64), (2, 1, 256), (3, 1, 112)])
@pytest.mark.parametrize("window", [None, 21])
def test_attention_simt_prefill_and_decode_shapes(dtype, nh, nkv, hd, window):
    for lens, qlens in [([1, 70, 33], [1, 70, 33]), ([200, 17, 64, 65], [1, 1, 1, 1]), ([90, 50], [7, 50])]:
        c = _attention_case(dtype, nh, nkv, hd, lens, qlens, window)
        out = torch.empty(c["q"].shape, device="cuda", dtype=dtype)
        ops.attention_simt(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(c["tok_seq"]), dev(c["tok_pos"]),
                           dev(c["table"]), nh, nkv, hd, 16, c["scale"], window)
        close(out, c["ref"], dtype, rowwise=True)


@pytest.mark.parametrize("dtype", DT)
def test_attention_finds_a_far_key_and_respects_the_windows_edge(dtype):
    nh, nkv, hd = 4, 2, 64
    lens, qlens = [700, 300], [1, 1]
    # sequence 0: query head 3 looks at key 5 (far away, first page); sequence 1: head 0 at key 299-40+1
    W = 40
    for window, sharp, hit in [(None, [(0, 699, 3, 5)], True), (W, [(1, 299, 0, 299 - W + 1)], True),
                               (W, [(1, 299, 0, 299 - W)], False)]:
        c = _attention_case(dtype, nh, nkv, hd, lens, qlens, window, sharp=sharp)
        out = torch.empty(c["q"].shape, device="cuda", dtype=dtype)
        ops.attention_simt(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(c["tok_seq"]), dev(c["tok_pos"]),
                           dev(c["table"]), nh, nkv, hd, 16, c["scale"], window)
        close(out, c["ref"], dtype, rowwise=True)
        b, _, h, kpos = sharp[0]
        target = c["vs"][b][kpos, h // 2]
        got = out[b].view(nh, hd)[h].float().cpu()
        assert ((got - target).abs().max() < 0.05) == hit


def test_argmax_first_maximum_and_ties():
    torch.manual_seed(6)
    x = torch.randn(7, 5000)
    x[0, 4000] = x[0, 17] = 50.0
    x[1, :] = -float("inf")
    x[2, 4999] = 99.0
    x[3, 0] = 99.0
    out = torch.empty(7, dtype=torch.int32, device="cuda")
    ops.argmax(dev(x), out)
    want = [int(torch.argmax(r)) for r in x]
    want[0], want[1] = 17, 0
    assert out.cpu().tolist() == want
    padded = dev(torch.cat([x, torch.full((7, 9), 1e9)], dim=1))[:, :5000]       # a leading dimension beyond vocab
    ops.argmax(padded, out)
    assert out.cpu().tolist() == want


def test_argmax_two_stages_for_large_vocabularies():
    torch.manual_seed(13)
    x = torch.randn(9, 151936)
    x[0, 151935] = x[0, 2374] = 77.0          # equal maxima in different pieces: the lower index wins
    x[1, 0] = 50.0
    x[2, :] = -float("inf")
    x[3, 2373] = x[3, 2374] = 60.0            # on the edge between two pieces
    out = torch.empty(9, dtype=torch.int32, device="cuda")
    ops.argmax(dev(x), out)
    want = [int(torch.argmax(r)) for r in x]
    want[0], want[2], want[3] = 2374, 0, 2373
    assert out.cpu().tolist() == want


@pytest.mark.parametrize("t,k,p", [(0.8, 20, 0.9), (0.4, 40, 0.9), (1.0, 0, 1.0), (1.3, 0, 0.5), (0.7, 5, 1.0),
                                   (1.0, 1, 0.9), (1.0, 3000, 0.95), (2.0, 7, 0.01)])
def test_sample_kernel_against_its_host_twin_and_the_reference_distribution(t, k, p):
    rng = np.random.default_rng(7)
    V, R = 2500, 4096
    logits = (rng.standard_normal(V) * 2.0).astype(np.float32)
    us = ((np.arange(R) + 0.5) / R).astype(np.float32)
    rows = dev(torch.from_numpy(logits)).expand(R, V).contiguous()
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.sample(rows, t, k, p, dev(torch.from_numpy(us)), out)
    got = out.cpu().numpy()
    params = SamplingParams(t, k, p)
    keep, e = host_survivors(logits, params)
    assert keep[got].all()                                   # only survivors are ever drawn
    c = np.cumsum(e.astype(np.float64)); c /= c[-1]
    lo = np.concatenate([[0.0], c[:-1]])
    # the drawn token's cumulative interval contains r, up to float rounding of the running sums
    assert (us >= lo[got] - 1e-5).all() and (us <= c[got] + 1e-5).all()
    twin = np.array([host_sample(logits, params, float(u)) for u in us[::16]])
    assert (twin == got[::16]).mean() > 0.99
    want = sample_distribution(logits, t, k, p)
    assert np.abs(np.bincount(got, minlength=V) / R - want).max() < 3.0 / R + 1e-5


@pytest.mark.parametrize("t,k,p,listed", [(0.7, 40, 0.9, True), (1.0, 5, 1.0, True), (0.4, 1000, 0.95, None),
                                          (0.25, 0, 0.9, True), (0.3, 0, 0.999, True), (1.0, 0, 0.95, False)])
def test_sample_with_a_small_top_k_against_a_large_vocabulary(t, k, p, listed):
    """The two-pass kernel that works on a list of candidates: same survivors, intervals and
    distribution as the host twin; ties at the top_k-th value all survive; a row of flat logits (more
    candidates than the list holds) falls to the general kernel in the same call.  With top_p alone
    the list serves a peaked row and the general kernel a row whose nucleus is wider than the list;
    `listed` says which of the two is expected to have chosen (None: the general kernel alone)."""
    rng = np.random.default_rng(9)
    V, R = 40000, 2048
    logits = (rng.standard_normal(V) * 2.5).astype(np.float32)
    us = ((np.arange(R) + 0.5) / R).astype(np.float32)
    rows = dev(torch.from_numpy(logits)).expand(R, V).contiguous()
    out = torch.full((R,), -7, dtype=torch.int32, device="cuda")
    ops.sample(rows, t, k, p, dev(torch.from_numpy(us)), out)
    got = out.cpu().numpy()
    if listed is not None:
        assert (ops._sample_flags[ops.device_key(rows.device)][:R].cpu().numpy() == (0 if listed else 1)).all()
    params = SamplingParams(t, k, p)
    keep, e = host_survivors(logits, params)
    assert keep[got].all()
    c = np.cumsum(e.astype(np.float64)); c /= c[-1]
    lo = np.concatenate([[0.0], c[:-1]])
    assert (us >= lo[got] - 1e-5).all() and (us <= c[got] + 1e-5).all()
    twin = np.array([host_sample(logits, params, float(u)) for u in us[::64]])
    assert (twin == got[::64]).mean() > 0.99
    want = sample_distribution(logits, t, k, p)
    assert np.abs(np.bincount(got, minlength=V) / R - want).max() < 3.0 / R + 1e-5
    # mixed rows: row 0 flat (all values within an eighth of an octave: 40,000 candidates, more than
    # the list holds), row 1 as above, row 2 with four equal values across the top_k edge (all survive)
    flat = (1.0 + 0.1 * rng.random(V)).astype(np.float32)
    tied = logits.copy()
    order = np.argsort(-tied)
    if k > 0:
        tied[order[k - 1:k + 3]] = tied[order[k - 1]]
    three = dev(torch.from_numpy(np.stack([flat, logits, tied])))
    for u in (0.37, 0.999):
        out3 = torch.full((3,), -7, dtype=torch.int32, device="cuda")
        ops.sample(three, t, k, p, dev(torch.full((3,), u)), out3)
        g3 = out3.cpu().numpy()
        for row, g in zip((flat, logits, tied), g3):
            assert host_survivors(row, params)[0][g]
            assert g == host_sample(row, params, u)
    if p == 1.0:
        assert host_survivors(tied, params)[0].sum() == k + 3


@pytest.mark.parametrize("V,t,k,p", [(300001, 1.0, 0, 1.0), (300001, 0.5, 0, 0.8), (300001, 0.8, 600, 1.0),
                                     (4097, 1.0, 0, 1.0), (33, 1.3, 0, 0.7), (8192, 1.0, 0, 0.9)])
def test_sample_general_kernel_at_other_vocabulary_sizes(V, t, k, p):
    """The general kernel's draw in two levels: a vocabulary whose runs are too long for the
    registers (one warp walks the chosen run) and is no multiple of 4, one that leaves most warps
    an empty run, and a power of two; survivors and intervals as the host twin has them."""
    rng = np.random.default_rng(V + k)
    R = 256
    logits = (rng.standard_normal(V) * 2.0).astype(np.float32)
    us = ((np.arange(R) + 0.5) / R).astype(np.float32)
    rows = dev(torch.from_numpy(logits)).expand(R, V).contiguous()
    out = torch.full((R,), -7, dtype=torch.int32, device="cuda")
    ops.sample(rows, t, k, p, dev(torch.from_numpy(us)), out)
    got = out.cpu().numpy()
    params = SamplingParams(t, k, p)
    keep, e = host_survivors(logits, params)
    assert keep[got].all()
    c = np.cumsum(e.astype(np.float64)); c /= c[-1]
    lo = np.concatenate([[0.0], c[:-1]])
    assert (us >= lo[got] - 1e-4).all() and (us <= c[got] + 1e-4).all()
    assert (np.diff(got[np.argsort(us, kind="stable")]) >= 0).all()      # a larger uniform never draws an earlier token


def test_sample_refuses_bad_options():
    x = dev(torch.zeros(1, 8)); u = dev(torch.zeros(1)); o = torch.empty(1, dtype=torch.int32, device="cuda")
    with pytest.raises(BackendError, match="temperature must be > 0"):
        ops.sample(x, 0.0, 0, 1.0, u, o)
    with pytest.raises(BackendError, match="head size 272 exceeds"):
        ops.attention_simt(x, 8, x, x, x, o, o, o, 1, 1, 272, 16, 1.0, None)
    with pytest.raises(BackendError, match="CUDA tensor"):
        ops.argmax(torch.zeros(1, 8), o)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("N,K", [(96, 64), (304, 96), (1000, 1024), (48, 4104), (16, 8)])
def test_gemm_skinny_every_epilogue(M, N, K):
    torch.manual_seed(8)
    a, w = torch.randn(M, K).to(torch.bfloat16), (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_skinny(dev(a), dev(w), c, ops.EPI_STORE)
    close(c, ref, torch.bfloat16)
    c32 = torch.empty(M, N, device="cuda")
    ops.gemm_skinny(dev(a), dev(w), c32, ops.EPI_STORE_F32)
    close(c32, ref, torch.float32)
    res = torch.randn(M, N)
    r = dev(res.clone())
    ops.gemm_skinny(dev(a), dev(w), r, ops.EPI_RESIDUAL)
    close(r, res.double() + ref, torch.float32)
    if N % 16 == 0:
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        ops.gemm_skinny(dev(a), dev(w), out, ops.EPI_SWIGLU)
        blocks = ref.view(M, N // 16, 2, 8)
        gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
        close(out, gate / (1 + torch.exp(-gate)) * up, torch.bfloat16)


@pytest.mark.parametrize("M,H,N2,eps", [(M, H, N2, eps) for M in (1, 5, 8, 13, 16, 65, 200, 333)
                                        for H, N2, eps in ((96, 64, 1e-5), (304, 16 * 1024, 1e-6), (1000, 48, 3e-3))]
                         + [(17, 6144, 6144, 1e-6), (40, 6160, 6144, 1e-5), (64, 6144, 16 * 1024, 1e-6), (100, 4096, 4096, 1e-6),
                            (128, 4160, 6144, 1e-5), (200, 4096, 4096, 1e-6), (512, 4160, 4096, 1e-5), (300, 8192, 4096, 1e-6)])
def test_products_with_a_norm_shared_between_them(M, H, N2, eps):
    """First product: x += a w1^T, and it begins RMSNorm(x; nw, eps).  Second product: finishes the
    norm and multiplies with w2 (store, SwiGLU and residual epilogues).  Up to 16 rows the decode
    kernel does it, beyond 64 the tensor-memory kernel, and between them the tensor-memory kernel
    where it is the one that multiplies such a matrix (6,144 weight rows and more).  Reference: the norm as a
    step of its own in double precision, rounded to bfloat16 where the engine's plain path rounds."""
    torch.manual_seed(31)
    # between 17 and 64 rows only a large matrix goes through the tensor-memory kernel; up to 128 rows a
    # large one has its K cut over a cluster of CTAs, up to 512 over a cluster of pairs of CTAs
    K1 = 4096 if (16 < M <= 64 or (M <= 512 and H >= 4096)) else 72
    a = torch.randn(M, K1).to(torch.bfloat16)
    w1 = (torch.randn(H, K1) * 0.3 * (72 / K1) ** 0.5).to(torch.bfloat16)
    x0 = torch.randn(M, H) * 3.0
    x0[0] *= 40.0                                             # rows of very different size: one factor per row
    nw = 1.0 + 0.1 * torch.randn(H)
    w2 = (torch.randn(N2, H) * 0.1).to(torch.bfloat16)
    x_ref = x0.double() + a.double() @ w1.double().T
    y_ref = x_ref / torch.sqrt((x_ref ** 2).mean(dim=1, keepdim=True) + eps) * nw.double()
    out_ref = y_ref @ w2.double().T

    bufs = []
    def scratch(shape, dtype):
        bufs.append(torch.full(shape, float("nan"), device="cuda", dtype=dtype))
        return bufs[-1]
    x = dev(x0.clone())
    pend = ops.gemm(dev(a), dev(w1), x, ops.EPI_RESIDUAL, next_norm=(dev(nw), eps), scratch=scratch)
    assert isinstance(pend, ops.PendingNorm) and pend.parts == int(pend.sumsq.shape[0])
    close(x, x_ref, torch.float32)
    assert not torch.isnan(pend.xw).any() and not torch.isnan(pend.sumsq[:, :M]).any()
    torch.testing.assert_close(pend.sumsq[:, :M].sum(dim=0).double().cpu(), (x_ref ** 2).sum(dim=1), rtol=1e-5, atol=0)

    y = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    ops.finish_norm(pend, y)
    close(y, y_ref, torch.bfloat16)

    c = torch.empty(M, N2, device="cuda", dtype=torch.bfloat16)
    assert ops.gemm(pend, dev(w2), c, ops.EPI_STORE, scratch=scratch) is None
    close(c, out_ref, torch.bfloat16)
    res = torch.randn(M, N2)
    r = dev(res.clone())
    ops.gemm(pend, dev(w2), r, ops.EPI_RESIDUAL, scratch=scratch)
    close(r, res.double() + out_ref, torch.bfloat16)
    act = torch.empty(M, N2 // 2, device="cuda", dtype=torch.bfloat16)
    ops.gemm_swiglu(pend, dev(w2), act, 8, scratch)
    blocks = out_ref.view(M, N2 // 16, 2, 8)
    gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
    close(act, gate / (1 + torch.exp(-gate)) * up, torch.bfloat16)
    # twice in a row gives the same bits: the partial sums meet in a fixed order
    c2 = torch.empty_like(c)
    ops.gemm(pend, dev(w2), c2, ops.EPI_STORE, scratch=scratch)
    assert torch.equal(c, c2)


def test_a_pending_norm_is_finished_for_kernels_that_cannot_take_it():
    """More rows than the shared-norm kernel takes never get a PendingNorm; a product that cannot
    use the kernel for its sizes (K not a multiple of 8 is impossible here, so: float32) refuses."""
    torch.manual_seed(2)
    a, w1 = torch.randn(17, 64).to(torch.bfloat16), torch.randn(96, 64).to(torch.bfloat16)
    x = torch.zeros(17, 96, device="cuda")
    got = ops.gemm(dev(a), dev(w1), x, ops.EPI_RESIDUAL, next_norm=(torch.ones(96, device="cuda"), 1e-6),
                   scratch=lambda shape, dtype: torch.empty(shape, device="cuda", dtype=dtype))
    assert got is None
    close(x, a.double() @ w1.double().T, torch.float32)
    with pytest.raises(BackendError, match="residual epilogue"):
        ops.gemm_skinny_norm(dev(a[:4]), dev(w1), torch.zeros(4, 96, device="cuda", dtype=torch.bfloat16), ops.EPI_STORE,
                             next_norm=(torch.ones(96, device="cuda"), 1e-6), scratch=lambda s, d: torch.empty(s, device="cuda", dtype=d))


def test_gemm_skinny_refuses_what_it_cannot_do():
    a, w = dev(torch.zeros(65, 64, dtype=torch.bfloat16)), dev(torch.zeros(32, 64, dtype=torch.bfloat16))
    c = torch.empty(65, 32, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(BackendError, match="at most 64"):
        ops.gemm_skinny(a, w, c)
    with pytest.raises(BackendError, match="multiples of 8"):
        ops.gemm_skinny(a[:4, :60], w[:, :60], c[:4])
    ops.gemm(a, w, c)        # the dispatcher takes another kernel instead


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 3, 48), (32, 8, 128), (5, 5, 80), (16, 1, 64), (2, 1, 256), (12, 4, 112),
                                       (16, 1, 128), (8, 8, 128), (40, 8, 128), (24, 2, 128)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("nsplit", [1, 3, 8])
def test_attention_decode_kernel(nh, nkv, hd, window, nsplit):
    lens = [1, 64, 65, 300, 129, 17]
    c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, [1] * len(lens), window, page=64, seed=11)
    out = torch.empty(c["q"].shape, device="cuda", dtype=torch.bfloat16)
    scratch = torch.full((ops.attention_decode_scratch_floats(len(lens), nh, hd, nsplit),), float("nan"), device="cuda")
    ops.attention_decode(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(torch.tensor(lens, dtype=torch.int32)),
                         dev(c["table"]), scratch, nh, nkv, hd, 64, nsplit, c["scale"], window)
    close(out, c["ref"], torch.bfloat16, rowwise=True)


@pytest.mark.parametrize("nh,nkv,window,nsplit,norm", [(8, 2, 0, 1, True), (8, 2, 0, 3, True), (4, 4, 100, 2, False),
                                                       (12, 1, 0, 4, True), (16, 8, 70, 5, True), (10, 2, 0, 3, True),
                                                       (3, 1, 90, 2, True), (9, 1, 0, 2, False)])
def test_attention_decode_fused_equals_the_three_kernels_it_replaces(nh, nkv, window, nsplit, norm):
    """Norm + rotation + cache write, attention, combine in one launch (head size 128) against the
    same work as separate kernels: the bits of the output and of the cache must agree, the counters
    must be back at zero (second call), and a reader of another layer's cache writes nothing."""
    torch.manual_seed(21)
    hd, page, eps = 128, 64, 1e-6
    lens = [1, 64, 65, 300, 129, 17, 128]          # lengths after the step: new tokens at 0, 63, 64 (a new page), ...
    B = len(lens)
    n_pages = sum(-(-n // page) for n in lens) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).tolist()
    P = max(-(-n // page) for n in lens)
    table = torch.zeros(B, P, dtype=torch.int32)
    for b, n in enumerate(lens):
        for lp in range(-(-n // page)):
            table[b, lp] = order.pop()
    kc = torch.randn(n_pages, nkv, page, hd).to(torch.bfloat16).cuda()
    vc = torch.randn(n_pages, nkv, page, hd).to(torch.bfloat16).cuda()
    qkv = (torch.randn(B, (nh + 2 * nkv) * hd + 8) * 2).to(torch.bfloat16).cuda()
    qw, kw = (dev(1 + 0.1 * torch.randn(hd)), dev(1 + 0.1 * torch.randn(hd))) if norm else (None, None)
    cos, sin = (dev(t) for t in rope_tables(hd, 10000.0, 320, torch.float32))
    seq_len = dev(torch.tensor(lens, dtype=torch.int32))
    tok_seq = dev(torch.arange(B, dtype=torch.int32))
    tok_pos = dev(torch.tensor([n - 1 for n in lens], dtype=torch.int32))
    scale = hd ** -0.5
    n_scratch = ops.attention_decode_scratch_floats(B, nh, hd, nsplit)

    k1, v1, q1 = kc.clone(), vc.clone(), qkv.clone()
    ops.qk_norm_rope_cache(q1, qw, kw, eps, cos, sin, hd, tok_seq, tok_pos, dev(table), k1, v1, nh, nkv, hd, page)
    ref = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
    ops.attention_decode(q1, q1.stride(0), ref, k1, v1, seq_len, dev(table), torch.empty(n_scratch, device="cuda"),
                         nh, nkv, hd, page, nsplit, scale, window)
    for _ in range(2):
        k2, v2 = kc.clone(), vc.clone()
        out = torch.full((B, nh * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.attention_decode_fused(qkv, out, k2, v2, qw, kw, eps, cos, sin, True, seq_len, dev(table),
                                   torch.full((n_scratch,), float("nan"), device="cuda"), nh, nkv, page, nsplit, scale, window)
        assert torch.equal(out, ref)
        assert torch.equal(k2, k1) and torch.equal(v2, v1)
    # write_cache=False: the cache already holds the new position (written by the layer that owns it)
    k3, v3 = k1.clone(), v1.clone()
    out = torch.empty_like(ref)
    ops.attention_decode_fused(qkv, out, k3, v3, qw, kw, eps, cos, sin, False, seq_len, dev(table),
                               torch.empty(n_scratch, device="cuda"), nh, nkv, page, nsplit, scale, window)
    assert torch.equal(out, ref) and torch.equal(k3, k1) and torch.equal(v3, v1)


def test_attention_decode_finds_a_far_key_and_the_windows_edge():
    nh, nkv, hd = 8, 2, 128
    lens = [1500, 700]
    W = 200
    for window, sharp, hit in [(None, [(0, 1499, 5, 3)], True), (None, [(1, 699, 2, 64)], True),
                               (W, [(1, 699, 0, 699 - W + 1)], True), (W, [(1, 699, 0, 699 - W)], False)]:
        c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, [1, 1], window, page=64, sharp=sharp)
        out = torch.empty(c["q"].shape, device="cuda", dtype=torch.bfloat16)
        nsplit = 5
        scratch = torch.empty(ops.attention_decode_scratch_floats(2, nh, hd, nsplit), device="cuda")
        ops.attention_decode(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(torch.tensor(lens, dtype=torch.int32)),
                             dev(c["table"]), scratch, nh, nkv, hd, 64, nsplit, c["scale"], window)
        close(out, c["ref"], torch.bfloat16, rowwise=True)
        b, _, h, kpos = sharp[0]
        target = c["vs"][b][kpos, h // (nh // nkv)]
        assert (((out[b].view(nh, hd)[h].float().cpu() - target).abs().max()) < 0.05) == hit


def test_attention_decode_refuses_what_it_cannot_do():
    z = dev(torch.zeros(1, 4096, dtype=torch.bfloat16)); i = dev(torch.zeros(4, dtype=torch.int32).view(1, 4))
    sc = torch.empty(1 << 16, device="cuda")
    with pytest.raises(BackendError, match="at most 16 query heads"):
        ops.attention_decode(z, 4096, z, z, z, i, i, sc, 34, 2, 16, 64, 1, 1.0, None)
    with pytest.raises(BackendError, match="multiple of 16"):
        ops.attention_decode(z, 4096, z, z, z, i, i, sc, 4, 2, 24, 64, 1, 1.0, None)
    with pytest.raises(BackendError, match="page size"):
        ops.attention_decode(z, 4096, z, z, z, i, i, sc, 4, 2, 32, 16, 1, 1.0, None)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (1, 8, 8), (65, 96, 96), (200, 304, 224), (300, 1000, 1024),
                                   (257, 24, 4104), (2048, 512, 256), (130, 272, 72),
                                   # 512 rows and more, whole tiles of 256 columns: pairs of CTAs (cta_group::2); ragged edges in M, N and K
                                   (512, 256, 64), (700, 1000, 1024), (1061, 304, 4104), (513, 272, 72), (2048, 6144, 512)])
def test_gemm_tcgen05_every_epilogue(M, N, K):
    torch.manual_seed(9)
    a, w = torch.randn(M, K).to(torch.bfloat16), (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    c32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_tcgen05(dev(a), dev(w), c32, ops.EPI_STORE_F32)
    ops.check_kernel_errors()
    close(c32, ref, torch.float32)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_tcgen05(dev(a), dev(w), c, ops.EPI_STORE)
    close(c, ref, torch.bfloat16)
    res = torch.randn(M, N)
    r = dev(res.clone())
    ops.gemm_tcgen05(dev(a), dev(w), r, ops.EPI_RESIDUAL)
    close(r, res.double() + ref, torch.float32)
    if N % 16 == 0:
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        ops.gemm_tcgen05(dev(a), dev(w), out, ops.EPI_SWIGLU)
        blocks = ref.view(M, N // 16, 2, 8)
        gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
        close(out, gate / (1 + torch.exp(-gate)) * up, torch.bfloat16)
    # a tile of the output must not spill into its neighbours: guard columns stay as they were
    wide = torch.full((M, N + 8), 7.0, device="cuda")
    ops.gemm_tcgen05(dev(a), dev(w), wide[:, :N], ops.EPI_STORE_F32)
    assert (wide[:, N:] == 7.0).all()
    ops.check_kernel_errors()


@pytest.mark.parametrize("M,N,K", [(200, 4112, 2056), (700, 6512, 4800), (129, 4096, 4096),
                                   (64, 6144, 1024), (33, 4112, 4104), (17, 24592, 512), (50, 1000, 12288),
                                   (100, 4096, 4096), (128, 6144, 2048), (65, 4096, 12288), (1, 5120, 5120), (64, 10240, 5120),
                                   (256, 4096, 4096), (300, 4112, 12288), (512, 4096, 2048), (192, 6144, 4096), (257, 5120, 8192)])
def test_gemm_tcgen05_tiles_shared_between_ctas(M, N, K):
    """Sizes whose leftover tiles are cut into runs of k blocks (all 34 tiles; 8 of 156; 32 tiles;
    then decode batches, whose tiles are 128 weight rows wide and whose pieces hold only the rows
    there are: 48 tiles, 33 tiles, 45 of 193 tiles, 8 tiles of 192 k blocks; up to 128 rows a matrix
    with few tiles has its K cut over a cluster of CTAs instead, in tiles of 128 to 256 columns, and
    up to about 512 rows over a cluster of pairs of CTAs, in tiles of 256 x 256):
    every epilogue, the norm begun by the residual epilogue, twice the same bits, and the counters
    back at zero (the second and third call)."""
    torch.manual_seed(19)
    a, w = dev(torch.randn(M, K).to(torch.bfloat16)), dev((torch.randn(N, K) * 0.1).to(torch.bfloat16))
    ref = a.double() @ w.double().T
    c32 = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_tcgen05(a, w, c32, ops.EPI_STORE_F32)
    close(c32, ref, torch.float32, scale=4.0)          # float sums of up to 4,800 bfloat16 products
    again = torch.full((M, N), float("nan"), device="cuda")
    ops.gemm_tcgen05(a, w, again, ops.EPI_STORE_F32)
    assert torch.equal(c32, again)
    res = torch.randn(M, N, device="cuda")
    nw = dev(1.0 + 0.1 * torch.randn(N))
    r = res.clone()
    bufs = []
    def scratch(shape, dtype):
        bufs.append(torch.full(shape, float("nan"), device="cuda", dtype=dtype))
        return bufs[-1]
    x_ref = res.double() + ref
    if M > 64:
        pend = ops.gemm(a, w, r, ops.EPI_RESIDUAL, next_norm=(nw, 1e-6), scratch=scratch)
        close(r, x_ref, torch.float32, scale=4.0)
        assert isinstance(pend, ops.PendingNorm)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ops.finish_norm(pend, y)
        close(y, x_ref / torch.sqrt((x_ref ** 2).mean(dim=1, keepdim=True) + 1e-6) * nw.double(), torch.bfloat16)
    else:
        ops.gemm_tcgen05(a, w, r, ops.EPI_RESIDUAL)
        close(r, x_ref, torch.float32, scale=4.0)
        c16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ops.gemm_tcgen05(a, w, c16, ops.EPI_STORE)
        close(c16, ref, torch.bfloat16)
    if N % 16 == 0:
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        ops.gemm_tcgen05(a, w, out, ops.EPI_SWIGLU)
        blocks = ref.view(M, N // 16, 2, 8)
        gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
        close(out, gate / (1 + torch.exp(-gate)) * up, torch.bfloat16)
    ops.check_kernel_errors()


def test_gemm_tcgen05_refuses_rows_tma_cannot_address():
    a, w = dev(torch.zeros(16, 60, dtype=torch.bfloat16)), dev(torch.zeros(32, 60, dtype=torch.bfloat16))
    with pytest.raises(BackendError, match="multiples of 8"):
        ops.gemm_tcgen05(a, w, torch.empty(16, 32, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 3, 48), (8, 2, 128), (5, 5, 80), (2, 1, 256), (3, 1, 112)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_prefill_kernel(nh, nkv, hd, window):
    for lens, qlens in [([1, 70, 33, 200], [1, 70, 33, 200]), ([300, 130, 64], [100, 1, 64]), ([257], [129])]:
        c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, qlens, window, page=64, seed=12)
        out = torch.full(c["q"].shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        starts = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32)
        pos0 = torch.tensor([n - q for n, q in zip(lens, qlens)], dtype=torch.int32)
        ops.attention_prefill(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(starts), dev(pos0),
                              dev(c["table"]), len(lens), max(qlens), nh, nkv, hd, 64, c["scale"], window)
        close(out, c["ref"], torch.bfloat16, rowwise=True)


def test_attention_prefill_finds_a_far_key_and_the_windows_edge():
    nh, nkv, hd = 4, 2, 128
    lens, qlens = [900, 500], [300, 500]
    W = 150
    for window, sharp, hit in [(None, [(0, 870, 3, 2)], True), (None, [(1, 499, 1, 448)], True),
                               (W, [(1, 400, 0, 400 - W + 1)], True), (W, [(1, 400, 0, 400 - W)], False)]:
        c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, qlens, window, page=64, sharp=sharp)
        out = torch.empty(c["q"].shape, device="cuda", dtype=torch.bfloat16)
        starts = torch.tensor([0, 300, 800], dtype=torch.int32)
        pos0 = torch.tensor([600, 0], dtype=torch.int32)
        ops.attention_prefill(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(starts), dev(pos0),
                              dev(c["table"]), 2, 500, nh, nkv, hd, 64, c["scale"], window)
        close(out, c["ref"], torch.bfloat16, rowwise=True)
        b, qpos, h, kpos = sharp[0]
        row = (0 if b == 0 else 300) + qpos - int(pos0[b])
        target = c["vs"][b][kpos, h // (nh // nkv)]
        assert (((out[row].view(nh, hd)[h].float().cpu() - target).abs().max()) < 0.05) == hit


@pytest.mark.parametrize("M", [1, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(96, 64), (304, 96), (1000, 1024), (48, 4104), (16, 8), (4096, 4096), (640, 12288)])
def test_gemm_stream_every_epilogue(M, N, K):
    torch.manual_seed(10)
    a, w = torch.randn(M, K).to(torch.bfloat16), (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    da, dw = dev(a), dev(w)
    c32 = torch.full((M, N), float("nan"), device="cuda")
    for _ in range(2):                       # twice: the tiles' counters must be back at zero after a call
        ops.gemm_stream(da, dw, c32, ops.EPI_STORE_F32)
        ops.check_kernel_errors()
        close(c32, ref, torch.float32)
    again = torch.empty_like(c32)
    ops.gemm_stream(da, dw, again, ops.EPI_STORE_F32)
    assert torch.equal(again, c32)           # slices are summed in slice order, not in arrival order
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_stream(da, dw, c, ops.EPI_STORE)
    close(c, ref, torch.bfloat16)
    res = torch.randn(M, N)
    r = dev(res.clone())
    ops.gemm_stream(da, dw, r, ops.EPI_RESIDUAL)
    close(r, res.double() + ref, torch.float32)
    if N % 16 == 0:
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        ops.gemm_stream(da, dw, out, ops.EPI_SWIGLU)
        blocks = ref.view(M, N // 16, 2, 8)
        gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
        close(out, gate / (1 + torch.exp(-gate)) * up, torch.bfloat16)
    ops.check_kernel_errors()


def test_gemm_stream_refuses_what_it_cannot_do():
    a, w = dev(torch.zeros(65, 64, dtype=torch.bfloat16)), dev(torch.zeros(32, 64, dtype=torch.bfloat16))
    with pytest.raises(BackendError, match="at most 64"):
        ops.gemm_stream(a, w, torch.empty(65, 32, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(BackendError, match="multiples of 8"):
        ops.gemm_stream(a[:4, :60], w[:, :60], torch.empty(4, 32, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (4, 4, 64), (6, 3, 128), (2, 1, 64), (10, 2, 128), (3, 1, 128), (3, 3, 128)])
@pytest.mark.parametrize("window", [None, 70, 200])
def test_attention_prefill_tcgen05_kernel(nh, nkv, hd, window):
    for lens, qlens in [([1, 70, 33, 200], [1, 70, 33, 200]), ([300, 130, 64], [100, 1, 64]), ([257], [129]), ([700], [700])]:
        c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, qlens, window, page=64, seed=14)
        out = torch.full(c["q"].shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        starts = torch.tensor(np.concatenate([[0], np.cumsum(qlens)]), dtype=torch.int32)
        pos0 = torch.tensor([n - q for n, q in zip(lens, qlens)], dtype=torch.int32)
        ops.attention_prefill_tc(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(starts), dev(pos0),
                                 dev(c["table"]), len(lens), max(qlens), nh, nkv, hd, 64, c["scale"], window)
        ops.check_kernel_errors()
        close(out, c["ref"], torch.bfloat16, rowwise=True)
        # a longest prompt of 4,096 or more selects four threads per query row (head size 128); the
        # sequences here are shorter, so most query tiles are empty items that every warp must skip alike
        out.fill_(float("nan"))
        ops.attention_prefill_tc(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(starts), dev(pos0),
                                 dev(c["table"]), len(lens), 4096, nh, nkv, hd, 64, c["scale"], window)
        ops.check_kernel_errors()
        close(out, c["ref"], torch.bfloat16, rowwise=True)


def test_attention_prefill_tcgen05_finds_a_far_key_and_the_windows_edge():
    nh, nkv, hd = 4, 2, 128
    lens, qlens = [900, 500], [300, 500]
    W = 150
    for window, sharp, hit in [(None, [(0, 870, 3, 2)], True), (None, [(1, 499, 1, 448)], True),
                               (W, [(1, 400, 0, 400 - W + 1)], True), (W, [(1, 400, 0, 400 - W)], False)]:
        c = _attention_case(torch.bfloat16, nh, nkv, hd, lens, qlens, window, page=64, sharp=sharp)
        out = torch.empty(c["q"].shape, device="cuda", dtype=torch.bfloat16)
        starts = torch.tensor([0, 300, 800], dtype=torch.int32)
        pos0 = torch.tensor([600, 0], dtype=torch.int32)
        ops.attention_prefill_tc(dev(c["q"]), c["q"].shape[1], out, dev(c["k"]), dev(c["v"]), dev(starts), dev(pos0),
                                 dev(c["table"]), 2, 500, nh, nkv, hd, 64, c["scale"], window)
        ops.check_kernel_errors()
        close(out, c["ref"], torch.bfloat16, rowwise=True)
        b, qpos, h, kpos = sharp[0]
        row = (0 if b == 0 else 300) + qpos - int(pos0[b])
        target = c["vs"][b][kpos, h // (nh // nkv)]
        assert (((out[row].view(nh, hd)[h].float().cpu() - target).abs().max()) < 0.05) == hit


@pytest.mark.parametrize("heads", [(16, 4), (15, 1), (20, 4)])
@pytest.mark.parametrize("norm,shared_norm,write", [(True, False, True), (False, False, True), (True, True, True), (True, False, False)])
def test_qkv_product_with_head_norm_rotation_and_cache_write_in_its_epilogue(norm, shared_norm, write, heads):
    """Long prompts, heads of 128: q = rotate(norm(x Wq^T)) into the output, k likewise and v as
    projected into the paged cache, all in the product's epilogue (pairs of CTAs), against float64."""
    torch.manual_seed(41)
    (nh, nkv), hd, page, eps = heads, 128, 64, 1e-6
    lens, pos0 = [700, 401], [130, 0]                  # the first sequence continues at position 130
    M, K, N = sum(lens), 264, (nh + 2 * nkv) * hd
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    qw, kw = 1 + 0.1 * torch.randn(hd), 1 + 0.1 * torch.randn(hd)
    cos, sin = rope_tables(hd, 10000.0, 1024, torch.float32)
    tok_seq = torch.tensor(sum(([b] * n for b, n in enumerate(lens)), []), dtype=torch.int32)
    tok_pos = torch.tensor(sum((list(range(p, p + n)) for p, n in zip(pos0, lens)), []), dtype=torch.int32)
    n_pages = 32
    table = torch.randperm(n_pages)[:2 * 14].to(torch.int32).view(2, 14)
    kc = torch.full((n_pages, nkv, page, hd), 9.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full((n_pages, nkv, page, hd), 9.0, dtype=torch.bfloat16, device="cuda")
    out = torch.full((M, N + 8), 7.0, dtype=torch.bfloat16, device="cuda")[:, :N]
    a = dev(x)
    ref_in = x.double()
    if shared_norm:            # x = (residual * nw) with the row's 1/rms still to come
        sumsq = (torch.rand(3, (M + 3) // 4 * 4) * 40.0 + 1.0)
        a = ops.PendingNorm(dev(x), dev(sumsq), 3, 1e-5)
        ref_in = x.double() / torch.sqrt(sumsq[:, :M].double().sum(0) / K + 1e-5)[:, None]
    assert ops.gemm_qkv_fused_ok(a, dev(w), out, hd, hd, object())
    ops.gemm_qkv_fused(a, dev(w), out, dev(qw) if norm else None, dev(kw) if norm else None, eps, dev(cos), dev(sin), dev(tok_seq),
                       dev(tok_pos), dev(table), kc, vc, nh, nkv, page, write, None)
    ops.check_kernel_errors()
    y = ref_in @ w.double().T
    q = y[:, :nh * hd].view(M, nh, hd)
    k = y[:, nh * hd:(nh + nkv) * hd].view(M, nkv, hd)
    v = y[:, (nh + nkv) * hd:].view(M, nkv, hd)
    if norm:
        q, k = rms_norm(q, qw.double(), eps), rms_norm(k, kw.double(), eps)
    c, s = cos.double()[tok_pos.long()], sin.double()[tok_pos.long()]
    q, k = apply_rope(q, c, s, hd), apply_rope(k, c, s, hd)
    close(out[:, :nh * hd], q.reshape(M, -1), torch.bfloat16)
    assert (out[:, nh * hd:] == 7.0).all()                     # k and v are not written to the output
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    if write:
        rows = torch.stack([table[tok_seq.long(), (tok_pos // page).long()].long(), (tok_pos % page).long()], 1)
        got_k = kc[rows[:, 0], :, rows[:, 1]].double().cpu()     # [M, nkv, hd]
        got_v = vc[rows[:, 0], :, rows[:, 1]].double().cpu()
        close(got_k, k, torch.bfloat16)
        close(got_v, v, torch.bfloat16)
        written[rows[:, 0], rows[:, 1]] = True
    untouched = lambda cch: cch.cpu().float().permute(0, 2, 1, 3)[~written]
    assert (untouched(kc) == 9.0).all() and (untouched(vc) == 9.0).all()
