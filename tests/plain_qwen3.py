"""A plain, slow implementation of the dense Qwen3 decoder: whole sequences, no cache, one
function per part, written from the reference's formulas.  It shares no code with the library:
it parses config.json and the safetensors file itself and computes with torch on the CPU.

The reference's own model code is Rust and cannot be compiled or imported here (there is no
Rust toolchain and no network), so this file rests on the formulas; every function cites the
place in the reference it restates (paths are relative to the reference's `crates/`).

`dtype` is the dtype of all arithmetic (float64 for a ground truth, float32 to mimic the
reference's f32 arithmetic).  Weights are used as stored (bfloat16 values widened exactly).
"""

from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ---- reading a model folder ---------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data (the container the reference
    reads in backends/backend_common/src/loader_common.rs:1182-1193)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            u = np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16  # core/src/tensor.rs:7-12
            t = torch.from_numpy(u.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f4").copy())
        elif info["dtype"] == "F16":
            t = torch.from_numpy(np.frombuffer(data[b:e], dtype="<f2").astype(np.float32))
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = t.reshape(info["shape"])
    return out


def read_config(path: str) -> dict:
    """Keys and defaults of core/src/config.rs:183-255, 490-694 (dense Qwen3 subset)."""
    with open(path) as f:
        c = json.load(f)
    cfg = {
        "V": c["vocab_size"], "H": c["hidden_size"], "L": c["num_hidden_layers"],
        "nh": c["num_attention_heads"], "nkv": c["num_key_value_heads"],
        "P": c["max_position_embeddings"], "I": c["intermediate_size"],
        "theta": c["rope_theta"] if "rope_theta" in c else c["rope_parameters"]["rope_theta"],
        "eps": c.get("rms_norm_eps", 1e-5),                       # config.rs:583-585
        "tied": c.get("tie_word_embeddings", True),               # config.rs:199-202
    }
    cfg["hd"] = c.get("head_dim") or cfg["H"] // cfg["nh"]         # config.rs:496-498
    cfg["rot"] = int(cfg["hd"] * c.get("partial_rotary_factor", 1.0))  # config.rs:516-525
    qpas = c.get("query_pre_attn_scalar")
    cfg["scale"] = 1.0 / math.sqrt(qpas) if qpas else 1.0 / math.sqrt(cfg["hd"])  # config.rs:645-646
    windows: List[Optional[int]] = [None] * cfg["L"]
    if c.get("use_sliding_window"):
        types = c.get("layer_types")
        for i in range(cfg["L"]):
            sliding = (types[i] == "sliding_attention") if types else i >= c.get("max_window_layers", cfg["L"])
            windows[i] = c["sliding_window"] if sliding else None
    cfg["windows"] = windows
    return cfg


# ---- the parts ------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: Sequence[int], dtype) -> torch.Tensor:
    """x[t,:] = float(E[id_t,:]), no scaling (backends/backend_common/src/generic_model.rs:104-111)."""
    return table[torch.tensor(list(ids), dtype=torch.long)].to(dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = 1/sqrt(sum(x^2)/dim + eps); y = x*inv*w (backends/backend_common/src/kernels.rs:54-64)."""
    dim = x.shape[-1]
    inv = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / dim + eps)
    return x * inv * w.to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """C[m,n] = sum_k A[m,k]*W[n,k]; weights are [out,in] (backends/backend_bf16/src/kernels.rs:95-143)."""
    return x @ w.to(x.dtype).T


def rope_tables(rot: int, theta: float, n_pos: int, dtype):
    """inv_freq_i = 1/theta^(2i/rot); angle = pos*inv_freq_i
    (backends/backend_common/src/loader_common.rs:179-202; float32 there)."""
    half = rot // 2
    if dtype == torch.float32:
        i = torch.arange(half, dtype=torch.float32)
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * i / float(rot))
        ang = torch.arange(n_pos, dtype=torch.float32)[:, None] * inv[None, :]
    else:
        i = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(float(np.float32(theta)), dtype=torch.float64), 2.0 * i / float(rot))
        ang = torch.arange(n_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int) -> torch.Tensor:
    """x: [T, heads, hd]; pairs (j, j+rot/2): x0*c - x1*s, x0*s + x1*c; the rest unchanged
    (backends/backend_common/src/kernels.rs:739-759)."""
    half = rot // 2
    x0, x1 = x[..., :half], x[..., half:rot]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, x[..., rot:]], dim=-1)


def attention_scores(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int]) -> torch.Tensor:
    """q: [T, nh, hd]; k, v: [T, nkv, hd].  Query head h uses kv head h // (nh/nkv)
    (loader_common.rs:1003-1005); s_j = (q.k_j)*scale for j <= i (causal;
    generic_attention/prefill/kernel_f32.rs:65, 81); softmax with the maximum subtracted
    (kernels.rs:716-731); o = sum_j p_j v_j (attention_common.rs:141-178)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask = mask & (idx[None, :] > idx[:, None] - window)
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def _same(x):
    return x


def bf16_storage(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 and back: what storing an activation in bfloat16 does to it."""
    return x.to(torch.bfloat16).to(x.dtype)


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, cos, sin,
                    window: Optional[int], store=_same) -> torch.Tensor:
    """Projections, per-head q/k norm before the rotation, rotation, attention, output projection
    (generic_attention/prefill/mod.rs:73-293; head norm generic_attention/mod.rs:62-76)."""
    T = h.shape[0]
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    q = store(linear(h, w[prefix + "q_proj.weight"])).view(T, nh, hd)
    k = store(linear(h, w[prefix + "k_proj.weight"])).view(T, nkv, hd)
    v = store(linear(h, w[prefix + "v_proj.weight"])).view(T, nkv, hd)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["eps"])
    q = store(apply_rope(q, cos[:T], sin[:T], cfg["rot"]))
    k = store(apply_rope(k, cos[:T], sin[:T], cfg["rot"]))
    o = store(attention_scores(q, k, v, cfg["scale"], window)).reshape(T, nh * hd)
    return linear(o, w[prefix + "o_proj.weight"])


def swiglu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, store=_same) -> torch.Tensor:
    """f = (silu(h Wg^T) * (h Wu^T)) Wd^T with silu(x) = x/(1+exp(-x))
    (generic_mlp.rs:83-96; kernels.rs:677-687)."""
    g = linear(h, w[prefix + "gate_proj.weight"])
    u = linear(h, w[prefix + "up_proj.weight"])
    return linear(store((g / (1.0 + torch.exp(-g))) * u), w[prefix + "down_proj.weight"])


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict, cos, sin, store=_same) -> torch.Tensor:
    """n1 = norm(x); h = x + attn(n1); n2 = norm(h); out = h + mlp(n2)
    (generic_layer.rs:1131-1328)."""
    p = f"model.layers.{i}."
    n1 = store(rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"]))
    h = x + attention_block(n1, w, p + "self_attn.", cfg, cos, sin, cfg["windows"][i], store)
    n2 = store(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]))
    return h + swiglu_mlp(n2, w, p + "mlp.", store)


def logits_all_positions(w: Dict[str, torch.Tensor], cfg: dict, ids: Sequence[int], dtype=torch.float64,
                         store=_same, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits at every position of one whole sequence: embed -> layers -> final norm -> head
    (generic_model.rs:131-319; the head is the embedding table when tied, loader_common.rs:1851-1860).
    `store` is applied wherever an engine would keep an activation between two kernels (norm
    outputs, projections, rotated q/k, attention output, the gated product); with `bf16_storage`
    the result shows how much of a bfloat16 engine's error is the storage format's own.
    `rows`: only these positions go through the final norm and the head (a large vocabulary)."""
    T = len(ids)
    cos, sin = rope_tables(cfg["rot"], cfg["theta"], T, dtype)
    x = embedding(w["model.embed_tokens.weight"], ids, dtype)
    for i in range(cfg["L"]):
        x = decoder_layer(x, w, i, cfg, cos, sin, store)
    if rows is not None:
        x = x[list(rows)]
    n = store(rms_norm(x, w["model.norm.weight"], cfg["eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return linear(n, head)


class PlainModel:
    def __init__(self, model_dir: str):
        self.cfg = read_config(f"{model_dir}/config.json")
        self.w = read_safetensors(f"{model_dir}/model.safetensors")

    def logits(self, ids: Sequence[int], dtype=torch.float64, store=_same, rows=None) -> torch.Tensor:
        return logits_all_positions(self.w, self.cfg, ids, dtype, store, rows)

    def greedy(self, prompt: Sequence[int], n: int, dtype=torch.float64) -> List[int]:
        """n greedy tokens, recomputing the whole sequence each time; first maximum wins
        (core/src/sampler.rs:244-254)."""
        ids, out = list(prompt), []
        for _ in range(n):
            tok = int(torch.argmax(self.logits(ids, dtype)[-1]))
            out.append(tok)
            ids.append(tok)
        return out


# ---- sampling, restated -------------------------------------------------------------------------
def sample_distribution(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """The probability of every token under the reference's sampler (core/src/sampler.rs:72-131):
    divide by temperature, keep the top_k, softmax, keep the shortest descending prefix whose
    cumulative probability reaches top_p, renormalise.  Computed in float64."""
    s = np.asarray(logits, dtype=np.float64) / temperature
    n = s.size
    keep = np.ones(n, dtype=bool)
    if 0 < top_k < n:
        keep[np.argsort(-s, kind="stable")[top_k:]] = False
    e = np.where(keep, np.exp(s - s.max()), 0.0)
    p = e / e.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        c = np.cumsum(p[order])
        cut = int(np.argmax(c >= top_p)) + 1 if (c >= top_p).any() else n
        p2 = np.zeros(n)
        p2[order[:cut]] = p[order[:cut]]
        p = p2 / p2.sum()
    return p
