"""Interfaces of the parts a layer is put together from.

Each part is constructed with its sizes and constants as keyword parameters, says
which tensors it wants (:meth:`Part.weight_specs`), receives them
(:meth:`Part.load`) and runs on the flat token rows of one step.  The kernels come
in through ``ops`` (kernels/library.py): a part never touches a device API itself.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

# --- weights -----------------------------------------------------------------
MATRIX = "matrix"      # operand of a matrix product: held in the engine's compute dtype
VECTOR = "vector"      # small per-channel parameters (norm weights): always held in float32
INT_TABLE = "int"      # integer tables: held in int32


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    role: str = MATRIX
    init: str = "normal"          # random-weights mode: "normal" | "one_plus_normal" | "zeros"
    init_scale: Optional[float] = None   # std; None = the model's init_std (normal) or 0.1 (one_plus_normal)


# --- cache needs ---------------------------------------------------------------
@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every token (window == 0) or of the last ``window`` tokens."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A per-request state of fixed size (``shape`` elements of ``dtype`` per request)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


# --- run-time contexts ---------------------------------------------------------
@dataclass
class LayerContext:
    """What one run of one layer sees of the step.

    batch        the step's StepBatch (engine/batch.py): tokens, positions, per-request rows
    ops          the kernel library
    kv_cache     tensor [pages, layers_in_group, 2, kv_heads, page_size, head_dim] or None
    kv_layer     this run's index along the second axis of kv_cache
    block_table  int32 [requests_in_step, max_blocks] of the run's cache group, or None
    page_size    tokens per page
    write_cache  False when this run reads another run's cache
    state        tensor [slots, *StateNeed.shape] of this run, or None
    position     the layer's position-encoding part, or None
    """
    batch: Any
    ops: Any
    kv_cache: Optional[torch.Tensor] = None
    kv_layer: int = 0
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    write_cache: bool = True
    state: Optional[torch.Tensor] = None
    position: Any = None


class Part:
    """Base of every part.  ``prefix`` is prepended to the names in weight_specs()."""
    family = ""
    kind = ""

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Tensor names (relative to the prefix) -> what is expected in the file."""
        return {}

    def full_name(self, rel: str) -> str:
        return f"{self.prefix}.{rel}" if self.prefix else rel

    def load(self, tensors: Dict[str, torch.Tensor], ops, act_dtype: torch.dtype) -> None:
        """Receive the tensors named by weight_specs() (relative names), already on the
        device and in the dtype their role asks for.  Merging happens here."""


class Norm(Part):
    """x: float32 [rows, dim] -> activation dtype [rows or len(row_index), dim]."""
    def forward(self, x: torch.Tensor, ops, out_dtype: torch.dtype,
                row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into something a mixer applies.  ``prepare`` runs once after
    loading (tables); ``embed`` may change the residual stream after the embedding
    (absolute encodings); rotary encodings expose ``rotary()`` for mixers."""
    def prepare(self, ops, device, max_position: int) -> None:
        pass

    def embed(self, x: torch.Tensor, batch, ops) -> torch.Tensor:
        return x

    def rotary(self):
        """(cos_sin table float32 [max_position, rot_dim/2, 2], rot_dim) or None."""
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here).

    cache_need() -> KVNeed | StateNeed | None
    forward(h, ctx, residual) -> float32 [T, hidden]: residual + mixer(h)
    """
    def cache_need(self):
        return None

    def forward(self, h: torch.Tensor, ctx: LayerContext, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """forward(h, ctx, residual) -> float32 [T, hidden]: residual + f(h)."""
    def forward(self, h: torch.Tensor, ctx: LayerContext, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and norms around the residual stream.  Which norms there
    are is the arrangement's business: the two of the pre-norm arrangement have names of their own, any
    others come in ``extra_norms`` under the names the layer's description gave them."""
    family = "block"
    kind = ""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Optional[Norm] = None,
                 ffn_norm: Optional[Norm] = None, extra_norms: Optional[Dict[str, Norm]] = None):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        self.extra_norms = dict(extra_norms or {})

    def parts(self):
        named = [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward] + list(self.extra_norms.values())
        return [p for p in named if p is not None]

    def forward(self, x: torch.Tensor, ctx: LayerContext, act_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError
