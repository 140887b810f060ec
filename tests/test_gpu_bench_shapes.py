"""The kernels at the shapes the benchmark times, each against a float64 restatement (torch on the
GPU, where the CPU would take minutes), and two layers at Qwen3-8B widths with the full vocabulary:
bfloat16 engine, float32 engine and plain implementation side by side.

Prefill attention: 32/8 heads of 128 with a 2,048-token prompt (512 items for 148 persistent CTAs,
each taking several items of up to 16 key tiles), 16 prompts of 512 tokens, a 4,096-token prompt
(four threads per query row), a prompt that continues a cached one.  Decode attention at context
2,048 and 4,096 with the split counts the engine picks for 1, 8 and 64 sequences.  The streaming
product at the output head's 151,936 rows.  Products at Qwen3-32B shapes.  Every attention case
plants far keys that single queries must find."""
import math

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
from herbert_rs_b200 import ops
from plain_qwen3 import PlainModel, bf16_storage, rope_tables

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _ref_attention(q, k, v, scale, window, qlen):
    """float64 attention of the last `qlen` positions of one sequence: q [qlen, nh, hd], k, v [n, nkv, hd]."""
    n, nkv, hd = k.shape
    nh = q.shape[1]
    qpos = torch.arange(n - qlen, n, device=q.device)[:, None]
    kpos = torch.arange(n, device=q.device)[None, :]
    mask = kpos <= qpos
    if window:
        mask = mask & (kpos > qpos - window)
    out = torch.empty(qlen, nh, hd, dtype=torch.float64, device=q.device)
    for h in range(nh):
        kh = h // (nh // nkv)
        s = (q[:, h].double() @ k[:, kh].double().T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ v[:, kh].double()
    return out


def _case(nh, nkv, hd, lens, qlens, window=None, sharp=(), seed=0, page=64, width=None):
    """Random bfloat16 q/k/v on the GPU, keys and values scattered into a shuffled page pool.
    sharp: (sequence, query position, head, key position): that query's score on that key stands out."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda").to(BF)
    ks, vs, qs = [rnd(n, nkv, hd) for n in lens], [rnd(n, nkv, hd) for n in lens], [rnd(q, nh, hd) for q in qlens]
    for b, qpos, h, kpos in sharp:
        kh, row = h // (nh // nkv), qpos - (lens[b] - qlens[b])
        qs[b][row, h] = 0
        qs[b][row, h, 3] = 16.0
        ks[b][:, kh, 3] = ks[b][:, kh, 3].clamp(-1, 1)
        ks[b][kpos, kh, 3] = 16.0
    scale = 1.0 / math.sqrt(hd)
    ref = torch.cat([_ref_attention(q, k, v, scale, window, ql) for q, k, v, ql in zip(qs, ks, vs, qlens)])
    need = [-(-n // page) for n in lens]
    total = sum(need) + 5
    order = torch.randperm(total, generator=torch.Generator().manual_seed(seed + 1)).tolist()
    P = max(max(need), width or 0)
    table = torch.zeros(len(lens), P, dtype=torch.int32)
    kpool = torch.full((total, nkv, page, hd), 777.0, dtype=BF, device="cuda")       # poison: a stray read shows
    vpool = torch.full((total, nkv, page, hd), 777.0, dtype=BF, device="cuda")
    for b, n in enumerate(lens):
        pg = [order.pop() for _ in range(need[b])]
        table[b, :need[b]] = torch.tensor(pg, dtype=torch.int32)
        pad = need[b] * page - n
        for pool, x in ((kpool, ks[b]), (vpool, vs[b])):
            xp = torch.cat([x, torch.full((pad, nkv, hd), 777.0, dtype=BF, device="cuda")]) if pad else x
            pool[torch.tensor(pg, device="cuda")] = xp.view(need[b], page, nkv, hd).permute(0, 2, 1, 3)
    return dict(q=torch.cat(qs).reshape(-1, nh * hd).contiguous(), k=kpool, v=vpool, table=table.cuda(), ref=ref, scale=scale,
                vs=vs, nh=nh, nkv=nkv, hd=hd, lens=lens, qlens=qlens)


def _check_attention(out, c, sharp, what):
    """Per query row and head: error at most 2^-6 of the row's largest reference value (bfloat16 output
    and bfloat16 softmax weights are 2^-9 relative each; the measured worst is below 2^-8), and every
    planted key is found: that head's output is the key's value row."""
    nh, hd = c["nh"], c["hd"]
    got = out.double().view(-1, nh, hd)
    ref = c["ref"]
    err = (got - ref).abs().amax(dim=-1)
    lim = ref.abs().amax(dim=-1) * 2.0 ** -6
    bad = err > lim
    assert not bad.any(), f"{what}: {int(bad.sum())} (row, head) pairs over the bound; worst ratio {(err / lim).max().item():.2f} " \
                          f"at {np.unravel_index(int((err / lim).argmax()), err.shape)}"
    starts = np.concatenate([[0], np.cumsum(c["qlens"])])
    for b, qpos, h, kpos in sharp:
        row = int(starts[b]) + qpos - (c["lens"][b] - c["qlens"][b])
        target = c["vs"][b][kpos, h // (nh // c["nkv"])].double()
        assert (got[row, h] - target).abs().max() < 0.05, f"{what}: query {qpos} of sequence {b}, head {h}, missed key {kpos}"
    return float((err / lim).max())


PREFILL_CASES = {
    "one prompt of 2048": dict(lens=[2048], qlens=[2048], max_q=2048,
                               sharp=[(0, 2047, 17, 3), (0, 1500, 5, 1499), (0, 130, 31, 64), (0, 1023, 0, 1)]),
    "sixteen prompts of 512": dict(lens=[512] * 16, qlens=[512] * 16, max_q=512,
                                   sharp=[(0, 511, 2, 0), (15, 400, 30, 129), (7, 64, 9, 63)]),
    "one prompt of 4096": dict(lens=[4096], qlens=[4096], max_q=4096,
                               sharp=[(0, 4095, 8, 2), (0, 2100, 21, 2049), (0, 3000, 13, 700)]),
    "1000 tokens after 2000 cached": dict(lens=[3000, 700], qlens=[1000, 700], max_q=1000,
                                          sharp=[(0, 2999, 1, 5), (0, 2001, 20, 1999), (1, 699, 11, 300)]),
    "a window of 1000": dict(lens=[2048], qlens=[2048], max_q=2048, window=1000,
                             sharp=[(0, 2047, 6, 1048), (0, 1500, 3, 501)]),
}


@pytest.mark.parametrize("name", list(PREFILL_CASES))
def test_prefill_attention_tcgen05_at_benchmark_shapes(name):
    p = PREFILL_CASES[name]
    c = _case(32, 8, 128, p["lens"], p["qlens"], p.get("window"), p["sharp"], seed=len(name))
    out = torch.full(c["q"].shape, float("nan"), device="cuda", dtype=BF)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(p["qlens"])]), dtype=torch.int32, device="cuda")
    pos0 = torch.tensor([n - q for n, q in zip(p["lens"], p["qlens"])], dtype=torch.int32, device="cuda")
    for _ in range(2):          # the second call finds the work counter and the barriers as the first left them
        out.fill_(float("nan"))
        ops.attention_prefill_tc(c["q"], c["q"].shape[1], out, c["k"], c["v"], starts, pos0, c["table"], len(p["lens"]),
                                 p["max_q"], 32, 8, 128, 64, c["scale"], p.get("window"))
        ops.check_kernel_errors()
        _check_attention(out, c, p["sharp"], name)


def test_prefill_attention_window_edge_at_2048():
    """One position outside the window: the planted key must not be found."""
    W = 1000
    sharp = [(0, 2047, 6, 2047 - W)]
    c = _case(32, 8, 128, [2048], [2048], W, sharp, seed=77)
    out = torch.empty(c["q"].shape, device="cuda", dtype=BF)
    ops.attention_prefill_tc(c["q"], c["q"].shape[1], out, c["k"], c["v"], torch.tensor([0, 2048], dtype=torch.int32, device="cuda"),
                             torch.zeros(1, dtype=torch.int32, device="cuda"), c["table"], 1, 2048, 32, 8, 128, 64, c["scale"], W)
    ops.check_kernel_errors()
    _check_attention(out, c, [], "window edge")
    target = c["vs"][0][2047 - W, 6 // 4].double()
    assert (out.double().view(-1, 32, 128)[2047, 6] - target).abs().max() > 0.5


@pytest.mark.parametrize("n_seqs,context", [(1, 2048), (8, 2048), (64, 2048), (1, 4096), (8, 4096), (64, 4095)])
def test_decode_attention_with_the_engines_splits(n_seqs, context):
    """Plain and fused decode attention (head size 128) at the benchmark's contexts, page table 64
    wide, with the split count the engine picks: 16 for one sequence, 4 for eight, 1 for sixty-four."""
    nh, nkv, hd, page = 32, 8, 128, 64
    rng = np.random.default_rng(context + n_seqs)
    lens = [context] + [int(x) for x in rng.integers(context // 2, context + 1, n_seqs - 1)]
    sharp = [(0, lens[0] - 1, 13, 2), (0, lens[0] - 1, 2, lens[0] - 1), (n_seqs - 1, lens[-1] - 1, 30, lens[-1] // 2)]
    if n_seqs > 1:
        sharp.append((1, lens[1] - 1, 7, 65))
    c = _case(nh, nkv, hd, lens, [1] * n_seqs, None, sharp, seed=context + n_seqs, width=64)
    nsplit = ops.decode_splits(n_seqs, nkv, c["table"].shape[1])
    assert nsplit == {1: 16, 8: 4, 64: 1}[n_seqs]
    seq_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scratch = torch.full((ops.attention_decode_scratch_floats(n_seqs, nh, hd, nsplit),), float("nan"), device="cuda")
    out = torch.full(c["q"].shape, float("nan"), device="cuda", dtype=BF)
    ops.attention_decode(c["q"], c["q"].shape[1], out, c["k"], c["v"], seq_len, c["table"], scratch, nh, nkv, hd, page,
                         nsplit, c["scale"], None)
    _check_attention(out, c, sharp, f"decode attention, {n_seqs} x {context}")

    # the fused form from raw projections: its reference is the three kernels it replaces (same bits),
    # which in turn are checked above and in the kernel tests
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = (torch.randn(n_seqs, (nh + 2 * nkv) * hd, generator=g, device="cuda") * 2).to(BF)
    qw, kw = (1 + 0.1 * torch.randn(hd, generator=g, device="cuda")), (1 + 0.1 * torch.randn(hd, generator=g, device="cuda"))
    cos, sin = (t.cuda() for t in rope_tables(hd, 1e6, 4096, torch.float32))
    tok_seq = torch.arange(n_seqs, dtype=torch.int32, device="cuda")
    k1, v1, q1 = c["k"].clone(), c["v"].clone(), qkv.clone()
    ops.qk_norm_rope_cache(q1, qw, kw, 1e-6, cos, sin, hd, tok_seq, seq_len - 1, c["table"], k1, v1, nh, nkv, hd, page)
    ref = torch.empty(n_seqs, nh * hd, device="cuda", dtype=BF)
    ops.attention_decode(q1, q1.stride(0), ref, k1, v1, seq_len, c["table"], scratch, nh, nkv, hd, page, nsplit, c["scale"], None)
    for _ in range(2):
        k2, v2 = c["k"].clone(), c["v"].clone()
        fused = torch.full((n_seqs, nh * hd), float("nan"), device="cuda", dtype=BF)
        ops.attention_decode_fused(qkv, fused, k2, v2, qw, kw, 1e-6, cos, sin, True, seq_len, c["table"],
                                   scratch.fill_(float("nan")), nh, nkv, page, nsplit, c["scale"], None)
        assert torch.equal(fused, ref) and torch.equal(k2, k1) and torch.equal(v2, v1)


def _check_product(got, ref, k_dim, what):
    """Float output of a bfloat16 product: float sums of k_dim exact products; bound 2e-6 * sqrt(k) of the scale."""
    err = (got.double() - ref).abs().max().item()
    lim = 4e-6 * math.sqrt(k_dim) * max(1.0, ref.abs().max().item())
    assert err <= lim, f"{what}: max error {err:.3e} > {lim:.3e}"


@pytest.mark.parametrize("M", [17, 40, 64])
def test_streaming_product_at_the_output_heads_size(M):
    """gemm_stream where production uses it: 151,936 weight rows, K = 4,096 in one slice, float out."""
    N, K = 151936, 4096
    g = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, K, generator=g, device="cuda").to(BF)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(BF)
    assert ops._decode_gemm(a, w) is ops.gemm_stream
    c = torch.full((M, N), float("nan"), device="cuda")
    for _ in range(2):
        ops.gemm_stream(a, w, c, ops.EPI_STORE_F32)
        ops.check_kernel_errors()
        ref = a.double() @ w.double().T
        _check_product(c, ref, K, f"head product, {M} rows")
    again = torch.empty_like(c)
    ops.gemm(a, w, again, ops.EPI_STORE_F32)
    assert torch.equal(again, c)


SHAPES_32B = {"q/k/v": (10240, 5120), "o": (5120, 8192), "gate/up": (51200, 5120), "down": (5120, 25600)}


@pytest.mark.parametrize("which", list(SHAPES_32B))
@pytest.mark.parametrize("M", [1, 8, 16, 32, 64, 1024])
def test_products_at_qwen3_32b_shapes(which, M):
    """Whatever kernel the dispatch picks for this many rows, in the epilogue production uses there."""
    N, K = SHAPES_32B[which]
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = torch.randn(M, K, generator=g, device="cuda").to(BF)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(BF)
    ref = a.double() @ w.double().T
    bf_lim = lambda r: 2.0 ** -7 * max(1e-3, r.abs().max().item())
    if which == "gate/up":
        out = torch.full((M, N // 2), float("nan"), device="cuda", dtype=BF)
        ops.gemm_swiglu(a, w, out, 8, lambda s, d: torch.empty(s, device="cuda", dtype=d))
        blocks = ref.view(M, N // 16, 2, 8)
        gate, up = blocks[:, :, 0].reshape(M, -1), blocks[:, :, 1].reshape(M, -1)
        want = gate / (1 + torch.exp(-gate)) * up
        assert (out.double() - want).abs().max().item() <= bf_lim(want)
    elif which == "q/k/v":
        out = torch.full((M, N), float("nan"), device="cuda", dtype=BF)
        ops.gemm(a, w, out)
        assert (out.double() - ref).abs().max().item() <= bf_lim(ref)
    else:
        res = torch.randn(M, N, generator=g, device="cuda")
        x = res.clone()
        ops.gemm(a, w, x, ops.EPI_RESIDUAL)
        _check_product(x, res.double() + ref, K, f"{which}, {M} rows")
    ops.check_kernel_errors()


# ---------------------------------------------------------------------------------------------
WIDE2 = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
             num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
             intermediate_size=12288, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096,
             tie_word_embeddings=False, eos_token_id=151645)


def test_two_layers_at_8b_widths_with_the_full_vocabulary(tmp_path):
    """A 2,048-token prompt and 32 decoded tokens: bfloat16 engine against float32 engine, float32
    engine against the plain implementation in float32 (sampled positions), and the bfloat16 error
    against what bfloat16 storage does to the plain implementation."""
    d = str(tmp_path / "wide2")
    hb.write_random_model(WIDE2, d, seed=71, device="cuda")
    rng = np.random.default_rng(71)
    ids = rng.integers(0, WIDE2["vocab_size"], 2048 + 32).tolist()
    want = [0, 1, 63, 64, 127, 128, 1000, 2046, 2047]
    rows = want + list(range(2048, 2080))
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = hb.Engine.from_folder(d, dtype=dtype, max_tokens=4096, max_slots=2)
        s = eng.alloc_slot()
        out = [eng.step([(s, ids[:2048])], [want]).double().cpu()]
        for t in ids[2048:]:
            out.append(eng.step([(s, [t])], "last").double().cpu())
        eng.free_slot(s)
        eng.check_kernels()
        got[dtype] = torch.cat(out).numpy()
        del eng
        torch.cuda.empty_cache()
    plain = PlainModel(d)
    ref = plain.logits(ids, torch.float32, rows=rows).double().numpy()
    scale = max(1.0, float(np.abs(ref).max()))
    e32 = np.abs(got["float32"] - ref).max()
    assert e32 <= 3e-5 * scale, f"float32 engine against the plain implementation: {e32:.3e}"
    own = np.abs(plain.logits(ids, torch.float32, bf16_storage, rows=rows).double().numpy() - ref).max()
    e16 = np.abs(got["bfloat16"] - got["float32"]).max()
    print(f"8B widths, 2 layers: float32 error {e32:.2e}, bfloat16 error {e16:.2e}, bfloat16 storage alone {own:.2e}")
    assert e16 <= 3.0 * own, f"bfloat16 engine against float32 engine: {e16:.3e} > 3 x {own:.3e}"
    # greedy tokens agree wherever the float32 margin exceeds the bound
    top2 = np.sort(got["float32"], axis=-1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 6.0 * own
    assert (got["bfloat16"].argmax(-1) == got["float32"].argmax(-1))[clear].all()


def test_prompts_and_decode_batches_of_17_to_700_rows_at_8b_widths(tmp_path):
    """The row counts between a decode batch of 16 and a long prompt go through kernels of their own
    (K cut over a cluster of CTAs up to 128 rows, over a cluster of pairs up to about 512): at 8B
    widths, prompts of such lengths and decode steps of such batches against the float32 engine,
    and no further from it than the same steps are with those kernels switched off."""
    cfg = dict(WIDE2, vocab_size=20040)
    d = str(tmp_path / "wide2s")
    hb.write_random_model(cfg, d, seed=73, device="cuda")
    rng = np.random.default_rng(73)
    prompts = {n: rng.integers(0, cfg["vocab_size"], n).tolist() for n in (17, 40, 64, 100, 128, 200, 300, 512, 700)}
    batches = {b: [rng.integers(0, cfg["vocab_size"], int(n)).tolist() for n in rng.integers(3, 90, b)] for b in (17, 40, 64)}

    def run(dtype, cluster):
        ops.set_gemm_ksplit(cluster)
        try:
            eng = hb.Engine.from_folder(d, dtype=dtype, max_tokens=64 * 64 * 4, max_slots=64)
            out = {}
            for n, ids in prompts.items():
                s = eng.alloc_slot()
                out["prompt", n] = eng.step([(s, ids)], [[0, n // 2, n - 1]]).double().cpu().numpy()
                eng.free_slot(s)
            for b, seqs in batches.items():
                slots = [eng.alloc_slot() for _ in seqs]
                eng.step([(s, ids[:-2]) for s, ids in zip(slots, seqs)], None)
                for t in (-2, -1):          # two decode steps: the second replays the recorded one
                    out["batch", b, t] = eng.step([(s, [ids[t]]) for s, ids in zip(slots, seqs)], "last").double().cpu().numpy()
                for s in slots:
                    eng.free_slot(s)
            eng.check_kernels()
            return out
        finally:
            ops.set_gemm_ksplit(True)

    ref, new, old = run("float32", True), run("bfloat16", True), run("bfloat16", False)
    worst = 0.0
    for key in ref:
        e_new, e_old = np.abs(new[key] - ref[key]).max(), np.abs(old[key] - ref[key]).max()
        worst = max(worst, e_new / max(e_old, 1e-9))
        assert e_new <= 1.5 * e_old + 1e-3, f"{key}: {e_new:.3e} with the cluster kernels, {e_old:.3e} without"
        top2 = np.sort(ref[key], axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4.0 * max(e_new, e_old)
        assert (new[key].argmax(-1) == ref[key].argmax(-1))[clear].all(), key
    print(f"17 to 700 rows at 8B widths: largest ratio of errors (cluster kernels / without) {worst:.2f}")
