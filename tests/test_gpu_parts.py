"""Each part alone, and the generality of the layer list: a toy mixer with state of its own
that is registered, built and stepped from here, a routed feed-forward, other position encodings,
another norm and another arrangement of a layer, an architecture with a model class of its own, a
layer that runs twice, and a layer that reads another layer's cache, none of which changes a file
of the library."""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import herbert_rs_b200 as hb
import plain_qwen3 as P
from gpu_util import DTYPES, assert_close, engine_for, random_ids, replay_batches, replay_tail_one_by_one, replay_whole, to_np
from herbert_rs_b200.cache import CacheNeed, SequenceCache, StateNeed
from herbert_rs_b200.config import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec, ScheduleStep,
                                    SwiGLUSpec)
from herbert_rs_b200.engine.batch import StepBatch
from herbert_rs_b200.parts import FeedForward, Mixer, ParamSpec, Part
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _bf(t):
    return t.to(torch.bfloat16)


def _batch(cache, rt, slots, lens):
    """A step batch over `cache` for sequences that bring `lens` new tokens each."""
    cache.reserve(list(zip(slots, lens)))
    b = StepBatch(slots, [[0] * n for n in lens], [cache.lengths[s] for s in slots], [[] for _ in slots],
                  cache.num_kv_groups, None, cache.page_size)
    host = np.zeros(b.layout.total, dtype=np.int32)
    b.fill_host(host, [cache.page_rows(g, slots, b.pages_width) for g in range(cache.num_kv_groups)])
    b.bind(torch.from_numpy(host).cuda())
    return b


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part_alone(dtype):
    rt = hb.Runtime("cuda", TD[dtype])
    part = hb.build_part("norm", NormSpec(200, 2e-5), rt=rt)
    assert list(part.param_specs()) == ["weight"]
    w = 1 + 0.1 * torch.randn(200)
    part.load({"weight": w.cuda()})
    x = torch.randn(6, 200) * 2
    out = torch.empty(6, 200, device="cuda", dtype=TD[dtype])
    part.forward(x.cuda(), out)
    assert_close(to_np(out), P.rms_norm(x.double(), w.double(), 2e-5).numpy(), dtype, "norm part")


@pytest.mark.parametrize("dtype", DTYPES)
def test_position_part_alone(dtype):
    rt = hb.Runtime("cuda", TD[dtype])
    part = hb.build_part("position", PositionSpec(48, 24, 500000.0, 300), rt=rt)
    cos, sin = P.rope_tables(24, 500000.0, 300, torch.float64)
    assert part.cos.dtype == torch.float32 and part.cos.shape == (300, 12)      # angles stay 32-bit on both paths
    assert (part.cos.cpu().double() - cos).abs().max() < 1e-5 and (part.sin.cpu().double() - sin).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 10])
def test_attention_mixer_alone(dtype, window):
    torch.manual_seed(0)
    rt = hb.Runtime("cuda", TD[dtype], page_size=16)
    H, nh, nkv, hd = 72, 6, 2, 32
    spec = AttentionSpec(H, nh, nkv, hd, scale=0.2, qk_norm=NormSpec(hd, 1e-5),
                         position=PositionSpec(hd, 16, 1e4, 128), window=window)
    mixer = hb.build_part("mixer", spec, rt=rt)
    w = {n: _bf(torch.randn(ps.shape) * (0.1 if ps.role == "matrix" else 0.0) + (1.0 if ps.role == "vector" else 0.0))
         for n, ps in mixer.param_specs().items()}
    w["q_norm.weight"] = _bf(1 + 0.2 * torch.randn(hd)); w["k_norm.weight"] = _bf(1 + 0.2 * torch.randn(hd))
    mixer.load({n: (t.float() if mixer.param_specs()[n].role == "vector" else t.to(TD[dtype])).cuda() for n, t in w.items()})
    need = mixer.cache_need()
    assert need.kv.num_kv_heads == nkv and need.kv.head_dim == hd and need.kv.window == window and need.state is None
    cache = SequenceCache([need], [None], 16, 4, page_size=16, dtype=TD[dtype], device="cuda")
    lens = [37, 5]
    hs = [_bf(torch.randn(n, H)) for n in lens]
    cfg = dict(nh=nh, nkv=nkv, hd=hd, eps=1e-5, rot=16, scale=0.2)
    cos, sin = P.rope_tables(16, 1e4, 64, torch.float64)
    wd = {"x." + k: v.float() for k, v in w.items()}
    ref = [P.attention_block(h.double(), wd, "x.", cfg, cos, sin, window) for h in hs]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    # prompts minus the last 4 tokens in one step, then 4 single-token steps
    outs = [[], []]
    fed = [n - 4 for n in lens]
    for step in range(5):
        ns = fed if step == 0 else [1, 1]
        off = [0, 0] if step == 0 else [fed[0] + step - 1, fed[1] + step - 1]
        rt.workspace.rewind()
        b = _batch(cache, rt, slots, ns)
        h = torch.cat([hs[i][off[i]:off[i] + ns[i]] for i in range(2)]).to(TD[dtype]).cuda()
        res = torch.zeros(sum(ns), H, device="cuda")
        mixer.forward(h, res, b, cache.view(0))
        for s, n in zip(slots, ns):
            cache.advance(s, n)
        outs[0].append(to_np(res[:ns[0]])); outs[1].append(to_np(res[ns[0]:]))
    for i in range(2):
        assert_close(np.concatenate(outs[i]), ref[i].numpy(), dtype, f"attention mixer seq {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [64, 52])
def test_feed_forward_part_alone(dtype, inter):
    torch.manual_seed(1)
    rt = hb.Runtime("cuda", TD[dtype])
    ffn = hb.build_part("ffn", SwiGLUSpec(40, inter), rt=rt)
    w = {n: _bf(torch.randn(ps.shape) * 0.2) for n, ps in ffn.param_specs().items()}
    ffn.load({n: t.to(TD[dtype]).cuda() for n, t in w.items()})
    h = _bf(torch.randn(9, 40))
    res0 = torch.randn(9, 40)
    res = res0.clone().cuda()
    rt.workspace.rewind()
    ffn.forward(h.to(TD[dtype]).cuda(), res, None)
    ref = res0.double() + P.swiglu_mlp(h.double(), {"m." + k: v.float() for k, v in w.items()}, "m.")
    assert_close(to_np(res), ref.numpy(), dtype, "feed-forward part")


# ---- a toy mixer with state of its own, defined here ---------------------------------------------
@dataclass(frozen=True)
class EmaSpec:
    hidden_size: int
    decay: float
    kind: str = "toy_ema"


class EmaMixer(Mixer):
    """s_t = decay * s_{t-1} + (1 - decay) * h_t per sequence; output s_t * w.  The state s is one
    vector per sequence, kept in the cache's fixed-size region between steps."""

    graph_safe = False      # it loops over the batch's host-side lists, so its steps cannot be replayed

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt

    def param_specs(self):
        return {"mix.weight": ParamSpec((self.spec.hidden_size,), role="vector", init="ones_noise")}

    def load(self, tensors):
        self.w = tensors["mix.weight"]

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.spec.hidden_size,)))

    def forward(self, h, residual, batch, cache):
        a = self.spec.decay
        for b, slot in enumerate(batch.slots):
            lo, hi = int(batch.seq_start_host[b]), int(batch.seq_start_host[b + 1])
            s = cache.state[slot]
            for t in range(lo, hi):
                s.mul_(a).add_(h[t].float(), alpha=1 - a)
                residual[t] += s * self.w


@dataclass(frozen=True)
class ToyConfig:
    """Layers alternate: EMA mixer, attention, EMA mixer ...; read from its own config.json keys."""
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    ema_decay: float
    intermediate_size: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["num_hidden_layers"], d["ema_decay"], d["intermediate_size"])

    def to_dict(self):
        return dict(architectures=["ToyEmaForCausalLM"], **self.__dict__)

    def model_spec(self):
        H = self.hidden_size
        norm = NormSpec(H, 1e-5)
        att = AttentionSpec(H, 4, 2, 16, scale=0.25, qk_norm=NormSpec(16, 1e-5), position=PositionSpec(16, 16, 1e4, 256))
        blocks = tuple(BlockSpec(mixer=EmaSpec(H, self.ema_decay) if i % 2 == 0 else att,
                                 ffn=SwiGLUSpec(H, self.intermediate_size), norm1=norm, norm2=norm,
                                 names=(("norm1", "input_layernorm"), ("mixer", "ema" if i % 2 == 0 else "self_attn"),
                                        ("norm2", "post_attention_layernorm"), ("ffn", "mlp")))
                       for i in range(self.num_hidden_layers))
        return ModelSpec("ToyEmaForCausalLM", self.vocab_size, H, blocks,
                         tuple(ScheduleStep(i) for i in range(self.num_hidden_layers)), norm, True, 256)


def _toy_plain(w, cfg, ids):
    x = P.embedding(w["model.embed_tokens.weight"], ids, torch.float64)
    T = len(ids)
    cos, sin = P.rope_tables(16, 1e4, T, torch.float64)
    acfg = dict(nh=4, nkv=2, hd=16, eps=1e-5, rot=16, scale=0.25)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5)
        if i % 2 == 0:
            s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
            out = []
            for t in range(T):
                s = cfg["ema_decay"] * s + (1 - cfg["ema_decay"]) * n1[t]
                out.append(s * w[p + "ema.mix.weight"].double())
            x = x + torch.stack(out)
        else:
            x = x + P.attention_block(n1, w, p + "self_attn.", acfg, cos, sin, None)
        n2 = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5)
        x = x + P.swiglu_mlp(n2, w, p + "mlp.")
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"]).numpy()


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    hb.register_part("mixer", "toy_ema", EmaMixer)
    hb.register_architecture("ToyEmaForCausalLM", ToyConfig)
    cfg = dict(architectures=["ToyEmaForCausalLM"], vocab_size=120, hidden_size=64, num_hidden_layers=3,
               ema_decay=0.8, intermediate_size=96)
    d = hb.write_random_model(cfg, str(tmp_path / "toy"), seed=4)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert "model.layers.0.ema.mix.weight" in w and "model.layers.1.self_attn.q_proj.weight" in w
    eng = engine_for(d, "float32", max_tokens=64 * 6, max_slots=3)
    assert len(eng.cache.state_needs) == 1 and eng.cache.state[0].shape == (2, 3, 64)   # 2 EMA layers, 3 slots
    assert eng.cache.num_kv_groups == 1 and eng.cache.kv[0].shape[0] == 1              # 1 attention layer
    rng = np.random.default_rng(1)
    reqs = [random_ids(rng, 120, n) for n in (30, 7, 45, 12, 20)]
    for r in reqs[:2]:
        ref = _toy_plain(w, cfg, r)
        assert_close(replay_whole(eng, r), ref, "float32", "toy whole")
        assert_close(replay_tail_one_by_one(eng, r, 5), ref, "float32", "toy one by one")     # state carried between steps
    got = replay_batches(eng, reqs, [20, 7, 1, 3, 9], [[0, 1, 2], [3, 4]])                    # slots reused: state starts at zero
    for g, r in zip(got, reqs):
        assert_close(g, _toy_plain(w, cfg, r), "float32", "toy batched")
    s = eng.alloc_slot()
    eng.step([(s, [1, 2, 3])], None)
    with pytest.raises(hb.CacheError, match="cannot be rolled back"):
        eng.truncate(s, 1)
    eng.free_slot(s)


# ---- a toy feed-forward with routing and a toy position encoding, defined here ---------------------
@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    num_experts: int
    expert_size: int
    kind: str = "toy_routed"


class RoutedFeedForward(FeedForward):
    """Each token goes to the one expert its router row scores highest (router logits in float);
    an expert is relu(h W1^T) W2^T.  Written with torch operations on device tensors only (every
    expert is evaluated and the choice is a mask), so its steps can be replayed from a CUDA graph;
    it neither takes nor begins a shared norm."""

    def __init__(self, spec, rt):
        self.spec, self.rt = spec, rt

    def param_specs(self):
        s = self.spec
        p = {"router.weight": ParamSpec((s.num_experts, s.hidden_size))}
        for e in range(s.num_experts):
            p[f"experts.{e}.w1.weight"] = ParamSpec((s.expert_size, s.hidden_size))
            p[f"experts.{e}.w2.weight"] = ParamSpec((s.hidden_size, s.expert_size))
        return p

    def load(self, tensors):
        E = self.spec.num_experts
        self.router = tensors["router.weight"].float()
        self.w1 = torch.stack([tensors[f"experts.{e}.w1.weight"].float() for e in range(E)])
        self.w2 = torch.stack([tensors[f"experts.{e}.w2.weight"].float() for e in range(E)])
        self.expert_ids = torch.arange(E, device=self.router.device)

    def forward(self, h, residual, batch):
        x = h.float()
        choice = torch.argmax(x @ self.router.T, dim=1)                            # [T]
        y = torch.stack([torch.relu(x @ self.w1[e].T) @ self.w2[e].T for e in range(self.spec.num_experts)])   # [E, T, H]
        mask = (choice[None, :] == self.expert_ids[:, None]).unsqueeze(-1).to(y.dtype)                             # [E, T, 1]
        residual += (y * mask).sum(dim=0)


@dataclass(frozen=True)
class SlowedRopeSpec:
    """Rotary tables whose positions are divided by `factor` (angles = pos / factor * inv_freq)."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_position: int
    factor: float
    kind: str = "toy_slowed_rope"


class SlowedRope(Part):
    """Another position encoding for the attention mixer: it only has to offer cos/sin tables
    [max_position, rotary_dim / 2] in float and `rotary_dim`; the mixer and its kernels take it as is."""

    def __init__(self, spec, rt):
        self.rotary_dim, self.max_position = spec.rotary_dim, spec.max_position
        cos, sin = _slowed_tables(spec.rotary_dim, spec.theta, spec.max_position, spec.factor, torch.float32)
        self.cos, self.sin = cos.to(rt.device), sin.to(rt.device)


def _slowed_tables(rot, theta, n_pos, factor, dtype):
    i = torch.arange(rot // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / float(rot))
    ang = (torch.arange(n_pos, dtype=torch.float64) / factor)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype).contiguous(), torch.sin(ang).to(dtype).contiguous()


@dataclass(frozen=True)
class RoutedConfig:
    """Every layer: attention with the slowed rotation; the feed-forward is routed in odd layers and
    the dense SwiGLU in even ones.  Head size 128 in order to meet the fused decode kernel too."""
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_experts: int
    expert_size: int
    intermediate_size: int
    rope_factor: float

    @classmethod
    def from_dict(cls, d):
        return cls(*(d[k] for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_experts", "expert_size",
                                    "intermediate_size", "rope_factor")))

    def to_dict(self):
        return dict(architectures=["ToyRoutedForCausalLM"], **self.__dict__)

    def model_spec(self):
        H = self.hidden_size
        norm = NormSpec(H, 1e-6)
        att = AttentionSpec(H, 2, 1, 128, scale=128 ** -0.5, qk_norm=NormSpec(128, 1e-6),
                            position=SlowedRopeSpec(128, 128, 1e4, 512, self.rope_factor))
        blocks = tuple(BlockSpec(mixer=att, ffn=RoutedSpec(H, self.num_experts, self.expert_size) if i % 2 else SwiGLUSpec(H, self.intermediate_size),
                                 norm1=norm, norm2=norm,
                                 names=(("norm1", "input_layernorm"), ("mixer", "self_attn"),
                                        ("norm2", "post_attention_layernorm"), ("ffn", "moe" if i % 2 else "mlp")))
                       for i in range(self.num_hidden_layers))
        return ModelSpec("ToyRoutedForCausalLM", self.vocab_size, H, blocks,
                         tuple(ScheduleStep(i) for i in range(self.num_hidden_layers)), norm, True, 512)


def _routed_plain(w, cfg, ids, store=None):
    st = store or (lambda t: t)
    x = P.embedding(w["model.embed_tokens.weight"], ids, torch.float64)
    T = len(ids)
    cos, sin = _slowed_tables(128, 1e4, T, cfg["rope_factor"], torch.float64)
    acfg = dict(nh=2, nkv=1, hd=128, eps=1e-6, rot=128, scale=128 ** -0.5)
    margins = []
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = x + P.attention_block(P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6), w, p + "self_attn.", acfg, cos, sin, None)
        n2 = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6)
        if i % 2:
            logits = n2 @ w[p + "moe.router.weight"].double().T
            top2 = torch.topk(logits, 2, dim=1).values
            margins.append((top2[:, 0] - top2[:, 1]).min().item())
            choice = torch.argmax(logits, dim=1)
            out = torch.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                out[t] = torch.relu(n2[t] @ w[p + f"moe.experts.{e}.w1.weight"].double().T) @ w[p + f"moe.experts.{e}.w2.weight"].double().T
            x = x + out
        else:
            x = x + P.swiglu_mlp(n2, w, p + "mlp.")
    logits = P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-6), w["model.embed_tokens.weight"]).numpy()
    return logits, min(margins)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path, dtype):
    """Both are defined and registered here; the framework's files do not know them.  The model mixes
    parts that share norms (attention, SwiGLU) with one that does not (the routed feed-forward), runs
    its decode steps from CUDA graphs, and meets the fused decode attention (head size 128) with the
    toy tables."""
    hb.register_part("ffn", "toy_routed", RoutedFeedForward)
    hb.register_part("position", "toy_slowed_rope", SlowedRope)
    hb.register_architecture("ToyRoutedForCausalLM", RoutedConfig)
    cfg = dict(architectures=["ToyRoutedForCausalLM"], vocab_size=150, hidden_size=64, num_hidden_layers=4,
               num_experts=3, expert_size=40, intermediate_size=96, rope_factor=3.0)
    d = hb.write_random_model(cfg, str(tmp_path / "routed"), seed=6)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert "model.layers.1.moe.experts.2.w2.weight" in w and "model.layers.0.mlp.gate_proj.weight" in w
    eng = engine_for(d, dtype, max_tokens=64 * 8, max_slots=3)
    assert eng.model.graph_safe
    rng = np.random.default_rng(3)
    reqs, refs = [], []
    while len(reqs) < 3:                         # keep prompts whose routing is not a near tie: a rounding must not flip an expert
        r = random_ids(rng, 150, int(rng.integers(20, 90)))
        ref, margin = _routed_plain(w, cfg, r)
        if margin > (1e-3 if dtype == "float32" else 2e-2):
            reqs.append(r); refs.append(ref)
    for r, ref in zip(reqs[:2], refs):
        assert_close(replay_whole(eng, r), ref, dtype, "routed whole")
        assert_close(replay_tail_one_by_one(eng, r, 12), ref, dtype, "routed one by one")
    got = replay_batches(eng, reqs, [len(r) - 6 for r in reqs], [[0, 1, 2]])
    for g, ref in zip(got, refs):
        assert_close(g, ref, dtype, "routed batched")
    assert eng.graph_replays > 0
    # a different factor gives different logits: the tables are really the toy's
    cfg2 = dict(cfg, rope_factor=1.0)
    assert np.abs(_routed_plain(w, cfg2, reqs[0])[0] - refs[0]).max() > 1e-3


# ---- an architecture with a model class of its own and two numbers per token position ---------------
@dataclass(frozen=True)
class GridMixerSpec:
    hidden_size: int
    rows: int
    cols: int
    kind: str = "toy_grid"


class GridMixer(Mixer):
    """out[t] = h[t] Wv^T + row_table[position component 0] + col_table[position component 1]: a mixer
    whose position encoding takes two numbers per token and that keeps nothing in the cache."""

    def __init__(self, spec, rt):
        self.spec = spec

    def param_specs(self):
        s = self.spec
        return {"v.weight": ParamSpec((s.hidden_size, s.hidden_size)), "row.weight": ParamSpec((s.rows, s.hidden_size)),
                "col.weight": ParamSpec((s.cols, s.hidden_size))}

    def load(self, tensors):
        self.wv, self.row, self.col = (tensors[n].float() for n in ("v.weight", "row.weight", "col.weight"))

    def forward(self, h, residual, batch, cache):
        pos = batch.positions.long()                       # [components, T], on the device
        residual += h.float() @ self.wv.T + self.row[pos[0]] + self.col[pos[1]]


class CappedLogitsModel(hb.DecoderModel):
    """A top level that differs from the generic decoder's: the embedding is scaled and the logits
    are squashed, both by constants of the spec's `extra`."""

    def load_embedding(self, t):
        super().load_embedding(t)
        self.embed = (self.embed.float() * self.spec.extra["embed_scale"]).to(self.embed.dtype)

    def forward(self, batch, cache):
        logits = super().forward(batch, cache)
        if logits is not None:
            cap = self.spec.extra["logit_cap"]
            logits.copy_(torch.tanh(logits / cap) * cap)
        return logits


@dataclass(frozen=True)
class GridConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    rows: int
    cols: int

    @classmethod
    def from_dict(cls, d):
        return cls(*(d[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "rows", "cols")))

    def to_dict(self):
        return dict(architectures=["ToyGridForCausalLM"], **self.__dict__)

    def model_spec(self):
        H = self.hidden_size
        norm = NormSpec(H, 1e-6)
        att = AttentionSpec(H, 4, 2, 32, scale=32 ** -0.5, qk_norm=NormSpec(32, 1e-6), position=PositionSpec(32, 32, 1e4, self.rows))
        names = (("norm1", "input_layernorm"), ("mixer", "grid"), ("norm2", "post_attention_layernorm"), ("ffn", "mlp"))
        blocks = (BlockSpec(mixer=att, ffn=SwiGLUSpec(H, self.intermediate_size), norm1=norm, norm2=norm),
                  BlockSpec(mixer=GridMixerSpec(H, self.rows, self.cols), ffn=SwiGLUSpec(H, self.intermediate_size),
                            norm1=norm, norm2=norm, names=names))
        return ModelSpec("ToyGridForCausalLM", self.vocab_size, H, blocks, (ScheduleStep(0), ScheduleStep(1)), norm, False,
                         self.rows, position_components=2, extra={"embed_scale": 2.0, "logit_cap": 0.5})


def _grid_plain(w, cfg, ids, cols):
    T = len(ids)
    acfg = dict(nh=4, nkv=2, hd=32, eps=1e-6, rot=32, scale=32 ** -0.5, windows=[None, None])
    cos, sin = P.rope_tables(32, 1e4, T, torch.float64)
    x = P.embedding(w["model.embed_tokens.weight"], ids, torch.float64)
    x = x * 2.0                                           # exact in bfloat16 too: a power of two
    x = P.decoder_layer(x, w, 0, acfg, cos, sin)
    p = "model.layers.1."
    n1 = P.rms_norm(x, w[p + "input_layernorm.weight"], 1e-6)
    x = x + n1 @ w[p + "grid.v.weight"].double().T + w[p + "grid.row.weight"].double()[torch.arange(T)] \
        + w[p + "grid.col.weight"].double()[torch.tensor(cols)]
    x = x + P.swiglu_mlp(P.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-6), w, p + "mlp.")
    logits = P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-6), w["lm_head.weight"])
    return (torch.tanh(logits / 0.5) * 0.5).numpy()


def test_an_architecture_with_its_own_model_class_and_two_position_components(tmp_path):
    """Registered from here: a configuration, a model class (scaled embedding, capped logits), and a
    mixer that reads two numbers per token position.  The second component is given by the caller,
    or defaults to the token's index; decode steps bump both and replay from a CUDA graph."""
    hb.register_part("mixer", "toy_grid", GridMixer)
    hb.register_architecture("ToyGridForCausalLM", GridConfig, model_cls=CappedLogitsModel)
    cfg = dict(architectures=["ToyGridForCausalLM"], vocab_size=120, hidden_size=64, intermediate_size=96, rows=200, cols=200)
    d = hb.write_random_model(cfg, str(tmp_path / "grid"), seed=12)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    eng = engine_for(d, "float32", max_tokens=64 * 6, max_slots=3)
    assert type(eng.model) is CappedLogitsModel and eng.model.spec.position_components == 2
    rng = np.random.default_rng(5)
    a, b = random_ids(rng, 120, 50), random_ids(rng, 120, 9)
    cols_a, cols_b = [int(c) for c in rng.integers(0, 200, 50)], [int(c) for c in rng.integers(0, 200, 9)]
    pos = lambda cols, lo, hi: np.stack([np.zeros(hi - lo, dtype=np.int64), np.asarray(cols[lo:hi])], axis=1)
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    got = to_np(eng.step([(sa, a[:40]), (sb, b[:5])], "all", positions=[pos(cols_a, 0, 40), pos(cols_b, 0, 5)]))
    ref_a, ref_b = _grid_plain(w, cfg, a, cols_a), _grid_plain(w, cfg, b, cols_b)
    assert_close(got[:40], ref_a[:40], "float32", "grid prompt a")
    assert_close(got[40:], ref_b[:5], "float32", "grid prompt b")
    for t in range(4):          # one token each, positions given
        got = to_np(eng.step([(sa, [a[40 + t]]), (sb, [b[5 + t]])], "all", positions=[pos(cols_a, 40 + t, 41 + t), pos(cols_b, 5 + t, 6 + t)]))
        assert_close(got, np.stack([ref_a[40 + t], ref_b[5 + t]]), "float32", f"grid decode {t}")
    eng.free_slot(sa); eng.free_slot(sb)
    with pytest.raises(hb.RequestError, match="positions of a sequence of 3 tokens"):
        s = eng.alloc_slot()
        eng.step([(s, [1, 2, 3])], "all", positions=[np.zeros((3, 3), dtype=np.int64)])
    eng.free_slot(s)
    # no positions given: the second component is the index too; generation's decode steps replay a graph
    ids = random_ids(rng, 120, 60)
    ref = _grid_plain(w, cfg, ids, list(range(60)))
    assert_close(replay_tail_one_by_one(eng, ids, 20), ref, "float32", "grid default positions")
    res = hb.generate(eng, [ids[:30], ids[:7]], hb.GenerationOptions(max_tokens=12, ignore_eos=True), hb.SamplingParams(temperature=0.0))
    for p0, toks in zip((ids[:30], ids[:7]), res.tokens):
        seq = list(p0)
        for tok in toks:
            r = _grid_plain(w, cfg, seq, list(range(len(seq))))[-1]
            assert r.max() - r[tok] <= 1e-5
            seq.append(tok)
    assert eng.graph_replays > 0 and eng.fast_decode_steps > 0


# ---- the order of layers is data -----------------------------------------------------------------
@dataclass(frozen=True)
class LoopedConfig(hb.Qwen3Config):
    """Tiny B's layers run in the order 0, 1, 0, 2r: layer 0 twice (each run with its own cache
    entry), and a last step that runs layer 2 but reads what step 1 (layer 1) stored."""

    def model_spec(self):
        s = super().model_spec()
        sched = (ScheduleStep(0), ScheduleStep(1), ScheduleStep(0), ScheduleStep(2, reads_cache_of=1))
        return ModelSpec("LoopedForCausalLM", s.vocab_size, s.hidden_size, s.blocks, sched, s.final_norm,
                         s.tie_word_embeddings, s.max_position, s.stop_token_ids)


def _looped_plain(w, cfg, ids):
    T = len(ids)
    cos, sin = P.rope_tables(cfg["rot"], cfg["theta"], T, torch.float64)
    x = P.embedding(w["model.embed_tokens.weight"], ids, torch.float64)
    x = P.decoder_layer(x, w, 0, cfg, cos, sin)
    x_in1 = x
    x = P.decoder_layer(x, w, 1, cfg, cos, sin)
    x = P.decoder_layer(x, w, 0, cfg, cos, sin)
    # step 3: layer 2's weights for q, o and the feed-forward; keys and values are those layer 1 stored
    p1, p2 = "model.layers.1.", "model.layers.2."
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    n_in1 = P.rms_norm(x_in1, w[p1 + "input_layernorm.weight"], cfg["eps"])
    k = P.apply_rope(P.rms_norm(P.linear(n_in1, w[p1 + "self_attn.k_proj.weight"]).view(T, nkv, hd),
                                w[p1 + "self_attn.k_norm.weight"], cfg["eps"]), cos, sin, cfg["rot"])
    v = P.linear(n_in1, w[p1 + "self_attn.v_proj.weight"]).view(T, nkv, hd)
    n1 = P.rms_norm(x, w[p2 + "input_layernorm.weight"], cfg["eps"])
    q = P.apply_rope(P.rms_norm(P.linear(n1, w[p2 + "self_attn.q_proj.weight"]).view(T, nh, hd),
                                w[p2 + "self_attn.q_norm.weight"], cfg["eps"]), cos, sin, cfg["rot"])
    o = P.attention_scores(q, k, v, cfg["scale"], None).reshape(T, nh * hd)
    h = x + P.linear(o, w[p2 + "self_attn.o_proj.weight"])
    x = h + P.swiglu_mlp(P.rms_norm(h, w[p2 + "post_attention_layernorm.weight"], cfg["eps"]), w, p2 + "mlp.")
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["lm_head.weight"]).numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_layer_named_twice_and_a_layer_reading_anothers_cache(tmp_path, dtype):
    hb.register_architecture("LoopedForCausalLM", LoopedConfig)
    cfg = dict(TINY["B"]); cfg["architectures"] = ["LoopedForCausalLM"]
    d = hb.write_random_model(cfg, str(tmp_path / "looped"), seed=8)
    with open(os.path.join(d, "config.json")) as f:
        c = json.load(f)
    c["architectures"] = ["LoopedForCausalLM"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c, f)
    eng = engine_for(d, dtype)
    assert eng.cache.kv[0].shape[0] == 3        # four steps, three cache entries: the reader has none
    pm = P.PlainModel(d)
    ids = random_ids(np.random.default_rng(2), 384, 80)
    ref = _looped_plain(pm.w, pm.cfg, ids)
    assert_close(replay_whole(eng, ids), ref, dtype, "looped whole")
    assert_close(replay_tail_one_by_one(eng, ids, 32), ref, dtype, "looped one by one")


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part_alone(dtype):
    """The pre-norm block built from a spec: x + attn(norm1 x), then + ffn(norm2 .), against the plain layer."""
    torch.manual_seed(3)
    rt = hb.Runtime("cuda", TD[dtype], page_size=16)
    H, nh, nkv, hd, inter = 48, 4, 2, 16, 88
    norm = NormSpec(H, 1e-5)
    spec = BlockSpec(mixer=AttentionSpec(H, nh, nkv, hd, scale=hd ** -0.5, qk_norm=NormSpec(hd, 1e-5),
                                         position=PositionSpec(hd, hd, 1e4, 64)),
                     ffn=SwiGLUSpec(H, inter), norm1=norm, norm2=norm)
    block = hb.build_part("block", spec, rt=rt)
    specs = block.param_specs()
    assert "self_attn.q_proj.weight" in specs and "mlp.down_proj.weight" in specs and "input_layernorm.weight" in specs
    w = {n: _bf(torch.randn(ps.shape) * 0.1 if ps.role == "matrix" else 1 + 0.1 * torch.randn(ps.shape)) for n, ps in specs.items()}
    block.load({n: (t.float() if specs[n].role == "vector" else t.to(TD[dtype])).cuda() for n, t in w.items()})
    cache = SequenceCache([block.cache_need()], [None], 8, 2, page_size=16, dtype=TD[dtype], device="cuda")
    x0 = torch.randn(21, H)
    slot = cache.alloc_slot()
    rt.workspace.rewind()
    b = _batch(cache, rt, [slot], [21])
    x = x0.clone().cuda()
    block.forward(x, b, cache.view(0))
    cfg = dict(nh=nh, nkv=nkv, hd=hd, eps=1e-5, rot=hd, scale=hd ** -0.5, windows=[None])
    cos, sin = P.rope_tables(hd, 1e4, 21, torch.float64)
    ref = P.decoder_layer(x0.double(), {"model.layers.0." + k: v.float() for k, v in w.items()}, 0, cfg, cos, sin)
    assert_close(to_np(x), ref.numpy(), dtype, "block part")


# ---- another norm and another arrangement of a layer -----------------------------------------------
@dataclass(frozen=True)
class OffsetNormSpec:
    """y = x / sqrt(mean(x^2) + eps) * (1 + w): the stored weight is an offset from one."""
    dim: int
    eps: float
    kind: str = "toy_offset_norm"


class OffsetNorm(hb.parts.Norm):
    """It has the form a product before it and a product after it can compute between them, with the
    weight 1 + w, and says so (`shareable`); alone it runs as torch operations on the device."""

    def __init__(self, spec, rt):
        self.dim, self.eps = spec.dim, spec.eps

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), role="vector", init="normal")}

    def load(self, tensors):
        self.scale = (1.0 + tensors["weight"].float()).contiguous()

    def forward(self, x, out, rows=None):
        src = x if rows is None else x[rows.long()]
        out.copy_((src * torch.rsqrt(src.pow(2).mean(dim=1, keepdim=True) + self.eps) * self.scale).to(out.dtype))

    def shareable(self):
        return (self.scale, self.eps)


@dataclass(frozen=True)
class SandwichSpec:
    """x += post(mixer(norm1(x))); x += ffn(norm2(x)): a third norm, on the mixer's result."""
    mixer: object
    ffn: object
    norm1: object
    norm2: object
    post: object
    kind: str = "toy_sandwich"
    names: tuple = (("norm1", "input_layernorm"), ("mixer", "self_attn"), ("post", "post_mixer_layernorm"),
                    ("norm2", "pre_feedforward_layernorm"), ("ffn", "mlp"))


class SandwichBlock(hb.parts.PreNormBlock):
    """Takes the library's block for the bookkeeping of its parts and replaces the arrangement; it
    neither takes a norm begun by the block before nor begins the next block's."""
    chains_norms = False

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.post = hb.build_part("norm", spec.post, rt=rt)

    def children(self):
        return super().children() + (("post", self.post),)

    def first_norm(self):
        return None

    def forward(self, x, batch, cache):
        ws = self.rt.workspace
        h = ws.take(x.shape, self.rt.dtype)
        self.norm1.forward(x, h)
        mixed = ws.take(x.shape, torch.float32)
        mixed.zero_()
        self.mixer.forward(h, mixed, batch, cache)          # adds into what it is given
        normed = ws.take(x.shape, self.rt.dtype)
        self.post.forward(mixed, normed)
        x += normed.float()
        h2 = ws.take(x.shape, self.rt.dtype)
        self.norm2.forward(x, h2)
        self.ffn.forward(h2, x, batch)


@dataclass(frozen=True)
class SandwichConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    eps: float

    @classmethod
    def from_dict(cls, d):
        return cls(*(d[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "eps")))

    def to_dict(self):
        return dict(architectures=["ToySandwichForCausalLM"], **self.__dict__)

    def model_spec(self):
        H = self.hidden_size
        off = OffsetNormSpec(H, self.eps)
        att = AttentionSpec(H, 4, 2, 32, scale=32 ** -0.5, qk_norm=NormSpec(32, 1e-6), position=PositionSpec(32, 32, 1e4, 256))
        ffn = SwiGLUSpec(H, self.intermediate_size)
        # even layers: the sandwich with offset norms; odd layers: the library's block, offset norms too (shared with its products)
        blocks = tuple(SandwichSpec(att, ffn, off, off, off) if i % 2 == 0 else BlockSpec(mixer=att, ffn=ffn, norm1=off, norm2=off)
                       for i in range(self.num_hidden_layers))
        return ModelSpec("ToySandwichForCausalLM", self.vocab_size, H, blocks,
                         tuple(ScheduleStep(i) for i in range(self.num_hidden_layers)), off, True, 256)


def _sandwich_plain(w, cfg, ids):
    T, eps = len(ids), cfg["eps"]
    acfg = dict(nh=4, nkv=2, hd=32, eps=1e-6, rot=32, scale=32 ** -0.5)
    cos, sin = P.rope_tables(32, 1e4, T, torch.float64)
    norm = lambda x, name: P.rms_norm(x, 1.0 + w[name].double(), eps)
    x = P.embedding(w["model.embed_tokens.weight"], ids, torch.float64)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        a = P.attention_block(norm(x, p + "input_layernorm.weight"), w, p + "self_attn.", acfg, cos, sin, None)
        if i % 2 == 0:
            x = x + norm(a, p + "post_mixer_layernorm.weight")
            x = x + P.swiglu_mlp(norm(x, p + "pre_feedforward_layernorm.weight"), w, p + "mlp.")
        else:
            x = x + a
            x = x + P.swiglu_mlp(norm(x, p + "post_attention_layernorm.weight"), w, p + "mlp.")
    return P.linear(norm(x, "model.norm.weight"), w["model.embed_tokens.weight"]).numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_norm_with_offset_weights_and_a_layer_with_a_third_norm(tmp_path, dtype):
    """A norm kind and a block kind defined and registered here.  The norm stands in the toy block, in
    the library's own block (where the products on either side of it share it) and as the final norm."""
    hb.register_part("norm", "toy_offset_norm", OffsetNorm)
    hb.register_part("block", "toy_sandwich", SandwichBlock)
    hb.register_architecture("ToySandwichForCausalLM", SandwichConfig)
    cfg = dict(architectures=["ToySandwichForCausalLM"], vocab_size=140, hidden_size=96, intermediate_size=160,
               num_hidden_layers=4, eps=3e-5)
    d = hb.write_random_model(cfg, str(tmp_path / "sandwich"), seed=8)
    w = P.read_safetensors(os.path.join(d, "model.safetensors"))
    assert "model.layers.0.post_mixer_layernorm.weight" in w and "model.layers.1.post_attention_layernorm.weight" in w
    assert "model.layers.1.post_mixer_layernorm.weight" not in w
    assert abs(float(w["model.layers.0.input_layernorm.weight"].float().mean())) < 0.02        # offsets, not weights near one
    eng = engine_for(d, dtype, max_tokens=64 * 8, max_slots=3)
    rng = np.random.default_rng(9)
    reqs = [random_ids(rng, 140, n) for n in (70, 9, 33)]
    refs = [_sandwich_plain(w, cfg, r) for r in reqs]
    for r, ref in zip(reqs[:2], refs):
        assert_close(replay_whole(eng, r), ref, dtype, "sandwich whole")
        assert_close(replay_tail_one_by_one(eng, r, 8), ref, dtype, "sandwich one by one")
    got = replay_batches(eng, reqs, [len(r) - 5 for r in reqs], [[0, 1, 2]])
    for g, ref in zip(got, refs):
        assert_close(g, ref, dtype, "sandwich batched")
    assert eng.graph_replays > 0
