"""The plain implementation checked against closed forms and a second, loop-by-loop
restatement of the reference's scalar code (no GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(P.rms_norm(x, w, 1e-6), torch.tensor([[3 * inv * 2, 4 * inv * 0.5]], dtype=torch.float64))


def test_rope_pairs_and_table():
    cos, sin = P.rope_tables(4, 10000.0, 3, torch.float64)
    assert cos.shape == (3, 2)
    assert abs(cos[2, 1].item() - math.cos(2 * 10000.0 ** (-2 / 4))) < 1e-12
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)  # hd 6, rot 4
    y = P.apply_rope(x, cos[1:2], sin[1:2], 4)[0, 0]
    c0, s0, c1, s1 = cos[1, 0], sin[1, 0], cos[1, 1], sin[1, 1]
    # pairs (0,2) and (1,3); elements 4,5 untouched (kernels.rs:739-759)
    want = [1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 1 * s0 + 3 * c0, 2 * s1 + 4 * c1, 5.0, 6.0]
    assert torch.allclose(y, torch.tensor([float(v) for v in want], dtype=torch.float64))
    assert abs(y[:4].norm().item() - x[0, 0, :4].norm().item()) < 1e-12


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nh, nkv, hd = 7, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=torch.float64) for n in (nh, nkv, nkv))
    o = P.attention_scores(q, k, v, 0.3, None)
    assert torch.allclose(o[0], v[0].repeat_interleave(2, 0))          # first token sees only itself
    k2, v2 = k.clone(), v.clone(); k2[5:] += 9; v2[5:] -= 3
    assert torch.allclose(P.attention_scores(q, k2, v2, 0.3, None)[:5], o[:5])   # later keys do not matter
    # a key that stands out: its value comes through, from the right kv head only
    qb, kb = q.clone(), k.clone()
    qb[6, 3] = 0; qb[6, 3, 0] = 50.0; kb[2, 1] = 0; kb[2, 1, 0] = 50.0
    ob = P.attention_scores(qb, kb, v, 1.0, None)
    assert torch.allclose(ob[6, 3], v[2, 1], atol=1e-9)
    assert torch.allclose(P.attention_scores(qb, kb, v, 1.0, 4)[6, 3], P.attention_scores(qb[3:], kb[3:], v[3:], 1.0, None)[3, 3])
    assert not torch.allclose(P.attention_scores(qb, kb, v, 1.0, 4)[6, 3], v[2, 1], atol=1e-3)  # key 2 is outside a window of 4


def _loop_model(w, cfg, ids):
    """The reference's scalar code restated loop by loop in float64: sequential sums, the online
    softmax of generic_attention/prefill/kernel_f32.rs:61-111, one token at a time."""
    f = lambda n: w[n].double().numpy()
    H, nh, nkv, hd, rot, eps = cfg["H"], cfg["nh"], cfg["nkv"], cfg["hd"], cfg["rot"], cfg["eps"]
    th = float(np.float32(cfg["theta"]))
    def norm(x, wt):
        s = 0.0
        for a in x:
            s += a * a
        inv = 1.0 / math.sqrt(s / len(x) + eps)
        return np.array([x[i] * inv * wt[i] for i in range(len(x))])
    def rope(x, pos):
        half = rot // 2
        y = x.copy()
        for j in range(half):
            ang = pos * (1.0 / th ** (2 * j / rot))
            c, s = math.cos(ang), math.sin(ang)
            y[j] = x[j] * c - x[j + half] * s
            y[j + half] = x[j] * s + x[j + half] * c
        return y
    xs = [f("model.embed_tokens.weight")[t].copy() for t in ids]
    for L in range(cfg["L"]):
        p = f"model.layers.{L}."
        ks, vs, outs = [], [], []
        for pos, x in enumerate(xs):
            n1 = norm(x, f(p + "input_layernorm.weight"))
            q = f(p + "self_attn.q_proj.weight") @ n1
            k = f(p + "self_attn.k_proj.weight") @ n1
            v = f(p + "self_attn.v_proj.weight") @ n1
            q = np.concatenate([rope(norm(q[h * hd:(h + 1) * hd], f(p + "self_attn.q_norm.weight")), pos) for h in range(nh)])
            k = np.concatenate([rope(norm(k[h * hd:(h + 1) * hd], f(p + "self_attn.k_norm.weight")), pos) for h in range(nkv)])
            ks.append(k); vs.append(v)
            att = np.zeros(nh * hd)
            win = cfg["windows"][L]
            lo = 0 if win is None else max(0, pos - win + 1)
            for h in range(nh):
                kh = h // (nh // nkv)
                m, l, o = -math.inf, 0.0, np.zeros(hd)
                for j in range(lo, pos + 1):
                    s = float(q[h * hd:(h + 1) * hd] @ ks[j][kh * hd:(kh + 1) * hd]) * cfg["scale"]
                    m_new = max(m, s)
                    corr, alpha = math.exp(m - m_new), math.exp(s - m_new)
                    l = corr * l + alpha
                    o = corr * o + alpha * vs[j][kh * hd:(kh + 1) * hd]
                    m = m_new
                att[h * hd:(h + 1) * hd] = o / l
            hres = x + f(p + "self_attn.o_proj.weight") @ att
            n2 = norm(hres, f(p + "post_attention_layernorm.weight"))
            g = f(p + "mlp.gate_proj.weight") @ n2
            u = f(p + "mlp.up_proj.weight") @ n2
            a = np.array([gi / (1.0 + math.exp(-gi)) for gi in g]) * u
            outs.append(hres + f(p + "mlp.down_proj.weight") @ a)
        xs = outs
    head = f("model.embed_tokens.weight") if cfg["tied"] else f("lm_head.weight")
    return np.stack([head @ norm(x, f("model.norm.weight")) for x in xs])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_two_restatements_agree(model_dirs, name):
    m = P.PlainModel(model_dirs[name])
    rng = np.random.default_rng(1)
    T = 50 if name == "C" else 12        # C: longer than its window of 40
    ids = rng.integers(0, m.cfg["V"], T).tolist()
    a = m.logits(ids, torch.float64).numpy()
    b = _loop_model(m.w, m.cfg, ids)
    assert np.abs(a - b).max() < 1e-10
    c = m.logits(ids, torch.float32).double().numpy()
    assert np.abs(a - c).max() < 2e-5 * max(1.0, np.abs(a).max())


def test_prefix_property(model_dirs):
    m = P.PlainModel(model_dirs["B"])
    ids = list(range(3, 40))
    full = m.logits(ids)
    assert torch.allclose(m.logits(ids[:20]), full[:20], atol=1e-12)
