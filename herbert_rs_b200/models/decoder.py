"""The generic decoder: embedding, a schedule of blocks, final norm, output head.

Structure of the reference's `GenericModel` (crates/backends/backend_common/src/generic_model.rs:27-46):
embedding table, decoder layers, final norm, lm_head (the embedding table again when tied).
Forward order (generic_model.rs:131-319): embed -> layers -> final norm -> head.  The
reference runs norm and head on the last position only (generic_model.rs:268-283); here they run
on exactly the rows whose logits are asked for, gathered before the norm.

The order in which blocks run is the spec's `schedule`, a list: a block may be named twice (its
weights run twice, each run with its own cache entry) and a step may read the cache entry of an
earlier step instead of storing its own.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..errors import ConfigError
from ..parts.base import ParamSpec
from ..registry import build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt):
        self.spec, self.rt = spec, rt
        self.blocks = [build_part("block", b, rt=rt) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, rt=rt)
        self.embed = None
        self.head = None
        for i, st in enumerate(spec.schedule):
            if not (0 <= st.layer < len(self.blocks)):
                raise ConfigError(f"schedule step {i} names layer {st.layer}, but there are {len(self.blocks)} layers")

    # -- tensors ---------------------------------------------------------------------------
    def block_prefix(self, i: int) -> str:
        return self.spec.layer_prefix.format(i=i)

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = self.spec
        out = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for i, b in enumerate(self.blocks):
            for name, ps in b.param_specs().items():
                out[self.block_prefix(i) + name] = ps
        for name, ps in self.final_norm.param_specs().items():
            out[self.final_norm_prefix() + name] = ps
        if not s.tie_word_embeddings:
            out[s.head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return out

    def final_norm_prefix(self) -> str:
        """'model.norm.' for the name 'model.norm.weight'."""
        return self.spec.final_norm_name.rsplit(".", 1)[0] + "."

    def ignored_names(self) -> set:
        """Tensors a file may hold without being used (a tied model's stored head)."""
        return {self.spec.head_name} if self.spec.tie_word_embeddings else set()

    def load_embedding(self, t: torch.Tensor) -> None:
        self.embed = t.contiguous()
        if self.spec.tie_word_embeddings:
            self.head = self.embed  # one buffer, two uses (loader_common.rs:1851-1860)

    def load_head(self, t: torch.Tensor) -> None:
        self.head = t.contiguous()

    def load_final_norm(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.final_norm.load(tensors)

    def weight_bytes(self, rows: int = 0) -> int:
        """Bytes of weights one step reads: every scheduled block, the final norm, the head;
        of the embedding only the gathered rows."""
        n = sum(self.blocks[st.layer].weight_bytes() for st in self.spec.schedule)
        n += self.final_norm.weight_bytes() + self.head.numel() * self.head.element_size()
        n += rows * self.spec.hidden_size * self.embed.element_size()
        return n

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    # -- cache -----------------------------------------------------------------------------
    def cache_needs(self) -> List:
        return [self.blocks[st.layer].cache_need() for st in self.spec.schedule]

    def reads_cache_of(self) -> List:
        return [st.reads_cache_of for st in self.spec.schedule]

    # -- running ---------------------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor | None:
        """Run the step's tokens; return float logits [n_want, vocab] (None if none are wanted).

        The result lives in the workspace and is valid until the next step."""
        ws = self.rt.workspace
        ws.rewind()
        x = ws.take((batch.n_tokens, self.spec.hidden_size), torch.float32)
        ops.embed(self.embed, batch.token_ids, x)
        # a block may begin the first norm of the block that runs after it (parts/base.py)
        sched, pending = self.spec.schedule, None
        for i, st in enumerate(sched):
            block = self.blocks[st.layer]
            ws.use(1 + i % 2)           # this layer's scratch; what the layer before handed over lies in the other lane
            if not block.chains_norms:
                block.forward(x, batch, cache.view(i))
                pending = None
                continue
            nxt = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
            nxt_norm = nxt.first_norm() if nxt is not None and nxt.chains_norms else None
            pending = block.forward(x, batch, cache.view(i), normed=pending,
                                    next_norm=nxt_norm.shareable() if nxt_norm is not None else None)
        ws.use(0)
        if batch.n_want == 0:
            return None
        hn = ws.take((batch.n_want, self.spec.hidden_size), self.rt.dtype)
        self.final_norm.forward(x, hn, rows=batch.want_rows)
        logits = ws.take((batch.n_want, self.spec.vocab_size), torch.float32)
        ops.gemm(hn, self.head, logits, ops.EPI_STORE_F32)
        return logits
