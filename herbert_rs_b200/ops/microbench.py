"""Times single kernels with CUDA events, outside any profiler.

    python -m herbert_rs_b200.ops.microbench decode-gemm --rows 8 --layers 12
    python -m herbert_rs_b200.ops.microbench prefill-gemm --rows 2048
    python -m herbert_rs_b200.ops.microbench decode-attention --seqs 8 --context 2050 --splits 4
    python -m herbert_rs_b200.ops.microbench prefill-attention --seqs 1 --len 2048
    python -m herbert_rs_b200.ops.microbench sampling --seqs 8 --vocab 151936
    python -m herbert_rs_b200.ops.microbench step --len 2048 --seqs 8          # a whole model's steps, by launcher

Shapes default to the Qwen3-8B layer (hidden 4096, 32 query / 8 key-value heads of 128,
intermediate 12288).  Every launch of a timed loop reads other weights or another layer's cache
than the one before (several copies, more than L2 holds together), decode kernels are timed
inside a captured CUDA graph as the engine runs them, and the figure printed is the mean over the
launches between two events after three untimed repetitions.
"""

from __future__ import annotations

import argparse

import torch

from .. import ops


def _timed(fn, reps: int, per: int, graph: bool) -> float:
    """Mean microseconds per launch of fn() (which makes `per` launches)."""
    fn()
    torch.cuda.synchronize()
    run = fn
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        run = g.replay
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    return e0.elapsed_time(e1) * 1e3 / reps / per


def _shapes(a):
    q, kv = a.heads * a.head_dim, a.kv_heads * a.head_dim
    return [("q/k/v", q + 2 * kv, a.hidden, ops.EPI_STORE), ("o", a.hidden, q, ops.EPI_RESIDUAL),
            ("gate/up", 2 * a.intermediate, a.hidden, ops.EPI_SWIGLU), ("down", a.hidden, a.intermediate, ops.EPI_RESIDUAL)]


def _gemm(a, kernels, graph):
    M = a.rows
    shapes = _shapes(a) + ([("head", a.vocab, a.hidden, ops.EPI_STORE_F32)] if a.head else [])
    for name, N, K, epi in shapes:
        copies = 2 if name == "head" else a.layers          # two heads are already ten times L2
        ws = [torch.randn(N, K, device="cuda").bfloat16() for _ in range(copies)]
        x = torch.randn(M, K, device="cuda").bfloat16()
        c = (torch.zeros(M, N, device="cuda") if epi in (ops.EPI_RESIDUAL, ops.EPI_STORE_F32)
             else torch.empty(M, N // 2 if epi == ops.EPI_SWIGLU else N, device="cuda", dtype=torch.bfloat16))
        line = f"{name:8s} N={N:6d} K={K:6d} rows={M:5d}"
        for kname in kernels:
            fn = getattr(ops, kname)
            us = _timed(lambda: [fn(x, w, c, epi) for w in ws], a.reps, copies, graph)
            line += f"   {kname} {us:7.1f} us {N * K * 2 / us / 1e3:6.0f} GB/s {2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s"
        print(line, flush=True)
        del ws


def decode_gemm(a):
    _gemm(a, [k for k in ("gemm_skinny", "gemm_stream", "gemm_tcgen05") if k == "gemm_tcgen05" or a.rows <= 64], True)


def prefill_gemm(a):
    _gemm(a, ["gemm_tcgen05"], False)


def decode_attention(a):
    from ..parts.rope import rope_tables
    B, nh, nkv, hd, page = a.seqs, a.heads, a.kv_heads, a.head_dim, 64
    if hd != 128:
        raise SystemExit("decode-attention times the fused kernel: head size 128")
    P = -(-a.context // page)
    kc = [torch.randn(B * P, nkv, page, hd, device="cuda").bfloat16() for _ in range(a.layers)]
    vc = [torch.randn(B * P, nkv, page, hd, device="cuda").bfloat16() for _ in range(a.layers)]
    table = torch.arange(B * P, dtype=torch.int32, device="cuda").view(B, P).contiguous()
    seq_len = torch.full((B,), a.context, dtype=torch.int32, device="cuda")
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda").bfloat16()
    out = torch.empty(B, nh * hd, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(hd, device="cuda")
    cos, sin = (t.cuda() for t in rope_tables(hd, 1e6, max(4096, a.context + 1)))
    splits = a.splits or ops.decode_splits(B, nkv, P)
    scratch = torch.empty(ops.attention_decode_scratch_floats(B, nh, hd, splits), device="cuda")
    us = _timed(lambda: [ops.attention_decode_fused(qkv, out, kc[i], vc[i], w, w, 1e-6, cos, sin, True, seq_len, table, scratch,
                                                    nh, nkv, page, splits, hd ** -0.5, 0) for i in range(a.layers)],
                a.reps, a.layers, True)
    byts = B * a.context * nkv * hd * 2 * 2
    print(f"fused decode attention: {B} sequences of {a.context}, {splits} splits ({splits * B * nkv} CTAs): {us:7.2f} us  {byts / us / 1e3:6.0f} GB/s")


def prefill_attention(a):
    B, T, nh, nkv, hd = a.seqs, a.len, a.heads, a.kv_heads, a.head_dim
    P = -(-T // 64)
    q = torch.randn(B * T, (nh + 2 * nkv) * hd, device="cuda").bfloat16()
    k = torch.randn(B * P, nkv, 64, hd, device="cuda").bfloat16()
    v = torch.randn(B * P, nkv, 64, hd, device="cuda").bfloat16()
    table = torch.arange(B * P, dtype=torch.int32, device="cuda").view(B, P).contiguous()
    starts = torch.arange(0, B * T + 1, T, dtype=torch.int32, device="cuda")
    pos0 = torch.zeros(B, dtype=torch.int32, device="cuda")
    out = torch.empty(B * T, nh * hd, device="cuda", dtype=torch.bfloat16)
    us = _timed(lambda: ops.attention_prefill_tc(q, q.stride(0), out, k, v, starts, pos0, table, B, T, nh, nkv, hd, 64, hd ** -0.5, None),
                a.reps, 1, False)
    flops = 4.0 * B * nh * hd * T * (T + 1) / 2
    print(f"tcgen05 prefill attention: {B} prompts of {T}: {us:8.1f} us  {flops / us / 1e6:6.0f} TFLOP/s on the causal half")


def sampling(a):
    """argmax and the sampler's settings on rows of normal logits (standard deviation --spread)."""
    B, V = a.seqs, a.vocab
    logits = [torch.randn(B, V, device="cuda") * a.spread for _ in range(a.layers)]
    u = torch.rand(B, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    line = f"{B} rows of {V}: argmax {_timed(lambda: [ops.argmax(x, out) for x in logits], a.reps, a.layers, True):6.1f} us"
    for t, k, p in ((0.7, 40, 0.9), (1.0, 0, 0.95), (0.2, 0, 0.95), (1.0, 0, 1.0)):
        us = _timed(lambda: [ops.sample(x, t, k, p, u, out) for x in logits], a.reps, a.layers, True)
        line += f";  t {t} k {k} p {p} {us:7.1f} us"
    print(line)


def step(a):
    """A whole model's step by launcher (`ops.timed()`): a prompt of --len tokens, then one eager decode
    step of --seqs sequences of that length (decode steps normally replay a graph; eager, the gaps
    between launches are the host's)."""
    import numpy as np

    import herbert_rs_b200 as hb
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=a.vocab, hidden_size=a.hidden,
               num_hidden_layers=a.model_layers, num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, head_dim=a.head_dim,
               intermediate_size=a.intermediate, rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=32768,
               tie_word_embeddings=False)
    rt = hb.Runtime("cuda", torch.bfloat16)
    eng = hb.Engine(hb.random_model(cfg, 0, rt), max_tokens=hb.Engine.pages_for(a.len + 8, a.seqs) * rt.page_size,
                    max_slots=a.seqs, use_graphs=False)
    rng = np.random.default_rng(0)
    slots = [eng.alloc_slot() for _ in range(a.seqs)]

    def show(title, t):
        d = t.by_kernel()
        print(f"{title}: {sum(ms for _, ms in d.values()):.3f} ms")
        for k, (n, ms) in sorted(d.items(), key=lambda kv: -kv[1][1]):
            print(f"  {k:34s} {n:5d} launches {ms:9.3f} ms {ms / n * 1e3:9.1f} us each")

    for i, s in enumerate(slots):
        ids = rng.integers(0, a.vocab, a.len).tolist()
        if i == len(slots) - 1:
            with ops.timed() as t:
                eng.step([(s, ids)], "last")
            show(f"prefill of {a.len} tokens, {a.model_layers} layers", t)
        else:
            eng.step([(s, ids)], "last")
    toks = rng.integers(0, a.vocab, a.seqs).tolist()
    for _ in range(3):
        eng.step([(s, [x]) for s, x in zip(slots, toks)], "last")
    with ops.timed() as t:
        eng.step([(s, [x]) for s, x in zip(slots, toks)], "last")
    show(f"eager decode step of {a.seqs} sequences", t)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m herbert_rs_b200.ops.microbench", description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=["decode-gemm", "prefill-gemm", "decode-attention", "prefill-attention", "sampling", "step"])
    ap.add_argument("--model-layers", type=int, default=36, help="step: layers of the model")
    ap.add_argument("--rows", type=int, default=8, help="activation rows of the products")
    ap.add_argument("--layers", type=int, default=12, help="copies of the weights / caches cycled through")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--context", type=int, default=2050)
    ap.add_argument("--len", type=int, default=2048)
    ap.add_argument("--splits", type=int, default=0, help="key ranges per (sequence, kv head); 0: as the engine chooses")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--head", action="store_true", help="decode-gemm / prefill-gemm: also the output head (vocab x hidden)")
    ap.add_argument("--spread", type=float, default=3.0, help="standard deviation of the logits of `sampling`")
    ap.add_argument("--no-pairs", action="store_true", help="prefill-gemm: single CTAs instead of pairs (cta_group::2)")
    ap.add_argument("--no-ksplit", action="store_true", help="products of at most 128 rows: no K ranges over a cluster")
    ap.add_argument("--pdl", type=int, default=0, help="programmatic dependent launch: 0 off, 1 every kernel, 2 the launches that ask for it")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    if a.pdl:
        ops.set_pdl(a.pdl)
    if a.no_pairs:
        ops.set_gemm_pairs(False)
    if a.no_ksplit:
        ops.set_gemm_ksplit(False)
    {"decode-gemm": decode_gemm, "prefill-gemm": prefill_gemm, "decode-attention": decode_attention,
     "prefill-attention": prefill_attention, "sampling": sampling, "step": step}[a.what](a)


if __name__ == "__main__":
    main()
