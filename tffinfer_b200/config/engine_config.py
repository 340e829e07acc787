"""Run-time options of the engine (not properties of a checkpoint).

The reference hard-codes these as macros and struct literals: ``PAGE_SIZE 32``
(src/core/runtime/KVCache.h:16), ``MAX_SEQ_LENGTH 8192`` / ``MAX_BATCH_SIZE 512``
(GlobalDefine.h:39-40), the user flags of test/main.cu:21-30.  Here they are one
typed record filled from command-line flags or keyword arguments.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPE_NAMES = {
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float32": "float32", "fp32": "float32", "f32": "float32",
}


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16" (serving kernels) or "float32" (true 32-bit)
    page_size: int = 16                # tokens per cache page
    max_cache_tokens: Optional[int] = None   # pool size in tokens (per layer group); None = from free memory
    max_live_requests: int = 64        # rows of the block table / state slots
    max_tokens_per_step: int = 2048    # token budget of one step
    max_model_len: Optional[int] = None      # cap on a request's length; None = config.max_position
    use_cuda_graphs: bool = True       # capture decode-only steps per batch-size bucket
    async_steps: bool = True           # launch the next step before the drawn tokens of the last one are read
    seed: int = 0
    device: str = "cuda"
    memory_fraction: float = 0.85      # share of free device memory the cache may take when sized automatically

    def normalized(self) -> "EngineConfig":
        if self.dtype not in DTYPE_NAMES:
            raise ValueError(f"dtype must be one of {sorted(set(DTYPE_NAMES))}, got '{self.dtype}'")
        self.dtype = DTYPE_NAMES[self.dtype]
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.max_live_requests <= 0:
            raise ValueError("max_live_requests must be positive")
        if self.max_tokens_per_step <= 0:
            raise ValueError("max_tokens_per_step must be positive")
        return self
