"""A model as data: which parts make each layer, and in which order layers run.

The reference builds its graph by calling reusable builders (``build_norm``,
``build_attn``, ``build_ffn`` ...; src/core/model/base/ModelCreatorBase.h:75-334) from
a per-architecture creator (src/core/model/qwen3/QWen3Creator.cpp:49-153).  Here the
creator returns a :class:`ModelDescription`; a generic builder (parts/model.py) turns
it into part objects by asking the registry for each ``PartSpec.kind``.  No part
knows which model it is in: it sees only its own parameters and its weight prefix.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    """One part: registry kind, constructor parameters, prefix of its tensor names."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass
class LayerSpec:
    """One layer's parts.  ``block`` names the arrangement (registry family "block") that decides how they
    are wired around the residual stream; ``mixer_norm`` and ``ffn_norm`` are the norms the pre-norm
    arrangement uses, ``extra_norms`` any further norms another arrangement names (after the mixer, after the
    feed-forward, ...), by a name of the arrangement's choosing.  ``position`` names an entry of
    ``ModelDescription.positions`` (or None)."""
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    block: str = "pre_norm"
    position: Optional[str] = None
    extra_norms: Dict[str, PartSpec] = field(default_factory=dict)


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelDescription.layers`` and may
    repeat (the same weights run twice, each run with a cache of its own).
    ``cache_of`` names an EARLIER schedule entry whose cache this run reads instead of
    keeping one (it then writes nothing)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelDescription:
    hidden_size: int
    vocab_size: int
    max_position: int
    embed_name: str                       # tensor name of the token embedding table [vocab, hidden]
    lm_head_name: Optional[str]           # None: logits use the embedding table (tied)
    final_norm: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    positions: Dict[str, PartSpec] = field(default_factory=dict)
    init_std: float = 0.02                # random-weights mode: std of matrices
    embed_scale: float = 1.0              # the embedding rows are multiplied by this (1: as they are)
    logit_scale: float = 1.0              # the logits are multiplied by this ...
    logit_softcap: float = 0.0            # ... and then, if > 0, squashed: softcap * tanh(logit / softcap)

    def validate(self) -> "ModelDescription":
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, model has {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"schedule[{i}].cache_of must name an earlier entry, got {e.cache_of}")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of names entry {e.cache_of}, which keeps no cache itself")
        for i, l in enumerate(self.layers):
            if l.position is not None and l.position not in self.positions:
                raise ValueError(f"layer {i} names position encoding '{l.position}', which is not defined")
        return self
