"""Options of the engine itself (not of a model).

The names of the reference's command-line options are kept where it has them
(``litelang/apis/test_server.py:7-24``): ``max_output_length``,
``max_input_length``, ``max_batch_size``, ``mem_usage``, ``max_reqs``,
``busy_scale``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16" or "float32"
    page_size: int = 16                # tokens per cache page
    num_pages: Optional[int] = None    # pages per cache group; None: from mem_usage
    mem_usage: float = 0.5             # fraction of free device memory for the cache
    max_batch_size: int = 32           # live requests = request slots of the cache
    max_input_length: int = 4000       # most prompt tokens of a request
    max_output_length: int = 200       # most new tokens of a request
    max_model_len: Optional[int] = None  # most tokens a request may hold; None: input + output
    max_tokens_per_step: int = 2048    # token budget of one step
    max_reqs: int = 1000               # most waiting requests
    busy_scale: float = 0.6            # cache share above which the system counts as busy
    preempt_strategy: str = "LIFOStrategy"
    cuda_graphs: bool = True           # capture steps that hold decode tokens only
    seed: int = 0

    def __post_init__(self) -> None:
        if self.dtype in ("bf16", "bfloat16"):
            self.dtype = "bfloat16"
        elif self.dtype in ("fp32", "float32"):
            self.dtype = "float32"
        else:
            raise ValueError(f"dtype must be bfloat16 or float32, not {self.dtype!r}")
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.max_batch_size <= 0 or self.max_tokens_per_step <= 0:
            raise ValueError("max_batch_size and max_tokens_per_step must be positive")
        if not (0.0 < self.mem_usage <= 1.0):
            raise ValueError("mem_usage must lie in (0, 1]")

    @property
    def model_len(self) -> int:
        if self.max_model_len is not None:
            return self.max_model_len
        return self.max_input_length + self.max_output_length
