"""Builds part objects from a ModelDescription and runs them over one step's tokens.

Stands where the reference has ``QWen3Creator::build_graph``
(src/core/model/qwen3/QWen3Creator.cpp:15-166): embedding (:283-321), the layer
loop (:49-153), final norm and output projection (:156-165).  Unlike the reference,
logits are computed only for the rows that were asked for.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..registry import get_part
from .base import Part, Block, LayerContext, WeightSpec, MATRIX
from .description import ModelDescription, PartSpec


def build_part(family: str, spec: PartSpec) -> Part:
    cls = get_part(family, spec.kind)
    return cls(prefix=spec.prefix, **spec.params)


@dataclass
class CacheBinding:
    """Where one schedule entry keeps (or borrows) its cache."""
    group: Optional[int] = None       # index of the KV group, or None
    layer_in_group: int = 0
    write: bool = True
    state_index: Optional[int] = None  # index into the state tensors, or None


class Model:
    def __init__(self, desc: ModelDescription):
        self.desc = desc.validate()
        self.positions = {name: build_part("position", ps) for name, ps in desc.positions.items()}
        self.blocks: List[Block] = []
        for ls in desc.layers:
            block_cls = get_part("block", ls.block)
            self.blocks.append(block_cls(
                mixer=build_part("mixer", ls.mixer),
                feed_forward=build_part("feed_forward", ls.feed_forward),
                mixer_norm=build_part("norm", ls.mixer_norm) if ls.mixer_norm is not None else None,
                ffn_norm=build_part("norm", ls.ffn_norm) if ls.ffn_norm is not None else None,
                extra_norms={name: build_part("norm", ps) for name, ps in ls.extra_norms.items()}))
        self.layer_position = [self.positions[ls.position] if ls.position else None for ls in desc.layers]
        self.final_norm = build_part("norm", desc.final_norm)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # ---------------------------------------------------------------- weights
    def all_parts(self) -> List[Part]:
        parts: List[Part] = list(self.positions.values())
        for b in self.blocks:
            parts.extend(b.parts())
        parts.append(self.final_norm)
        return parts

    def expected_tensors(self) -> Dict[str, WeightSpec]:
        d = self.desc
        out = {d.embed_name: WeightSpec((d.vocab_size, d.hidden_size), MATRIX)}
        if d.lm_head_name is not None:
            out[d.lm_head_name] = WeightSpec((d.vocab_size, d.hidden_size), MATRIX)
        for p in self.all_parts():
            for rel, spec in p.weight_specs().items():
                name = p.full_name(rel)
                if name in out:
                    raise ValueError(f"two parts claim the tensor '{name}'")
                out[name] = spec
        return out

    def load(self, tensors: Dict[str, torch.Tensor], ops, act_dtype: torch.dtype, device) -> None:
        d = self.desc
        self.embed = tensors[d.embed_name]
        self.lm_head = tensors[d.lm_head_name] if d.lm_head_name is not None else self.embed
        for p in self.all_parts():
            p.load({rel: tensors[p.full_name(rel)] for rel in p.weight_specs()}, ops, act_dtype)
        for pos in self.positions.values():
            pos.prepare(ops, device, d.max_position)

    # ------------------------------------------------------------------ cache
    def cache_needs(self):
        """One entry per schedule entry: KVNeed | StateNeed | None (None also for
        entries that borrow another entry's cache)."""
        needs = []
        for e in self.desc.schedule:
            need = self.blocks[e.layer].mixer.cache_need()
            needs.append(None if e.cache_of is not None else need)
        return needs

    # ---------------------------------------------------------------- forward
    def forward(self, batch, ops, act_dtype, bindings: List[CacheBinding], kv_caches, block_tables,
                page_size: int, states) -> torch.Tensor:
        """batch: StepBatch.  kv_caches[g]: cache tensor of KV group g.  block_tables[g]:
        int32 [requests, max_blocks].  states[i]: state tensor i.  Returns float32
        logits [len(batch.logit_rows), vocab]."""
        d = self.desc
        T = batch.num_tokens
        x = torch.empty((T, d.hidden_size), dtype=torch.float32, device=self.embed.device)
        ops.embed(batch.token_ids, self.embed, x, d.embed_scale)
        for pos in self.positions.values():
            x = pos.embed(x, batch, ops)
        for e, entry in enumerate(d.schedule):
            b = bindings[e]
            ctx = LayerContext(
                batch=batch, ops=ops,
                kv_cache=kv_caches[b.group] if b.group is not None else None,
                kv_layer=b.layer_in_group,
                block_table=block_tables[b.group] if b.group is not None else None,
                page_size=page_size, write_cache=b.write,
                state=states[b.state_index] if b.state_index is not None else None,
                position=self.layer_position[entry.layer])
            x = self.blocks[entry.layer].forward(x, ctx, act_dtype)
        R = batch.num_logit_rows
        if R == 0:
            return torch.empty((0, d.vocab_size), dtype=torch.float32, device=x.device)
        hn = self.final_norm.forward(x, ops, act_dtype, row_index=batch.logit_rows)
        logits = torch.empty((R, d.vocab_size), dtype=torch.float32, device=x.device)
        ops.gemm(hn, self.lm_head, logits)
        if d.logit_scale != 1.0 or d.logit_softcap > 0.0:
            ops.logit_transform(logits, d.logit_scale, d.logit_softcap)
        return logits
