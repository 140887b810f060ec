"""The attention mixer: q/k/v projections, per-head q/k norm, rotation, cache, GQA softmax
attention, output projection with the residual sum.

Order of operations (crates/backends/backend_common/src/generic_attention/prefill/mod.rs:73-293,
decode.rs:49-508): q,k,v = h W^T; RMSNorm over each head of q and of k with one weight vector
per projection (mod.rs:62-76), before the rotation; rotate q and k at the token's position;
store k (normed, rotated) and v; each query head attends the keys of kv head h / (nh/nkv) up to
its own position; result times o_proj, added to the residual stream.

The three projections are one matrix here (rows of q, then k, then v), joined at load time, so
one product yields the row layout the fused norm/rotation/cache kernel reads.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheNeed, KVNeed
from ..registry import build_part, register_part
from .base import Mixer, ParamSpec


class AttentionMixer(Mixer):
    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt
        self.nh, self.nkv, self.hd = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.qkv_dim = self.q_dim + 2 * self.kv_dim
        self.position = build_part("position", spec.position, rt=rt) if spec.position is not None else None
        self.wqkv = self.wo = self.q_norm = self.k_norm = None

    def param_specs(self):
        s = self.spec
        p = {
            "q_proj.weight": ParamSpec((self.q_dim, s.hidden_size)),
            "k_proj.weight": ParamSpec((self.kv_dim, s.hidden_size)),
            "v_proj.weight": ParamSpec((self.kv_dim, s.hidden_size)),
            "o_proj.weight": ParamSpec((s.hidden_size, self.q_dim)),
        }
        if s.qk_norm is not None:
            p["q_norm.weight"] = ParamSpec((self.hd,), role="vector", init="ones_noise")
            p["k_norm.weight"] = ParamSpec((self.hd,), role="vector", init="ones_noise")
        return p

    def load(self, tensors):
        self.wqkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0).contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        if self.spec.qk_norm is not None:
            self.q_norm = tensors["q_norm.weight"].contiguous()
            self.k_norm = tensors["k_norm.weight"].contiguous()

    def weight_bytes(self):
        return (self.wqkv.numel() + self.wo.numel()) * self.wqkv.element_size()

    def cache_need(self):
        return CacheNeed(kv=KVNeed(self.nkv, self.hd, self.spec.window))

    shares_norms = True

    def forward(self, h, residual, batch, cache, next_norm=None):
        ws, T = self.rt.workspace, h.shape[0]
        qkv = ws.take((T, self.qkv_dim), h.dtype)
        pages = batch.pages[cache.kv_group]
        pos = self.position
        att = ws.take((T, self.q_dim), h.dtype)
        norm_eps = self.spec.qk_norm.eps if self.spec.qk_norm is not None else 0.0
        if not batch.is_decode and pos is not None and cache.k is not None and \
                ops.gemm_qkv_fused_ok(h, self.wqkv, qkv, self.hd, pos.rotary_dim, pos):
            # long prompts: head norm, rotation and cache write happen in the product's epilogue
            ops.gemm_qkv_fused(h, self.wqkv, qkv, self.q_norm, self.k_norm, norm_eps, pos.cos, pos.sin, batch.tok_seq,
                               batch.tok_pos, pages, cache.k, cache.v, self.nh, self.nkv, cache.page_size, cache.writes_kv,
                               ws.take)
            ops.attention(qkv, qkv.stride(0), att, cache.k, cache.v, batch, self.nh, self.nkv, self.hd,
                          cache.page_size, self.spec.scale, self.spec.window, pages, scratch=ws.take)
            return ops.gemm(att, self.wo, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)
        ops.gemm(h, self.wqkv, qkv, scratch=ws.take)
        if batch.is_decode and pos is not None and ops.attention_decode_fused_ok(
                qkv, att, self.nh, self.nkv, self.hd, cache.page_size, pos.rotary_dim, batch.n_seqs):
            nsplit = ops.decode_splits(batch.n_seqs, self.nkv, pages.shape[1] * (cache.page_size // 64))
            buf = ws.take((ops.attention_decode_scratch_floats(batch.n_seqs, self.nh, self.hd, nsplit),), torch.float32)
            ops.attention_decode_fused(qkv, att, cache.k, cache.v, self.q_norm, self.k_norm, norm_eps, pos.cos, pos.sin,
                                       cache.writes_kv, batch.seq_len, pages, buf, self.nh, self.nkv, cache.page_size,
                                       nsplit, self.spec.scale, self.spec.window)
        else:
            ops.qk_norm_rope_cache(
                qkv, self.q_norm, self.k_norm, norm_eps,
                pos.cos if pos is not None else None, pos.sin if pos is not None else None,
                pos.rotary_dim if pos is not None else 0, batch.tok_seq, batch.tok_pos, pages,
                cache.k, cache.v, self.nh, self.nkv, self.hd, cache.page_size, write_cache=cache.writes_kv)
            ops.attention(qkv, qkv.stride(0), att, cache.k, cache.v, batch, self.nh, self.nkv, self.hd,
                          cache.page_size, self.spec.scale, self.spec.window, pages, scratch=ws.take)
        return ops.gemm(att, self.wo, residual, ops.EPI_RESIDUAL, next_norm=next_norm, scratch=ws.take)


register_part("mixer", "attention", AttentionMixer)
