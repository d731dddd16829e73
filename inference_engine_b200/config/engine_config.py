"""Engine settings, named as the reference's ``LLMEngine`` arguments
(engine/runtime/engine.py:47-66) and ``engine serve`` options (engine/cli.py:160-193)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    dtype: str = "bfloat16"  # "bfloat16" (serving kernels) or "float32" (true 32-bit path)
    block_size: int = 16  # tokens per cache page
    num_blocks: int | None = None  # pages per cache group; None = fill free device memory
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 4096
    gpu_memory_utilization: float = 0.9
    enable_chunked_prefill: bool = True
    max_model_len: int | None = None
    enable_cuda_graphs: bool | None = None  # None: where they can be captured (a GPU, no state slots)
    enable_mixed_graphs: bool | None = None  # short steps with prompt portions captured too; None: with the above
    debug_checks: bool = False
    profile_kernels: bool = False  # time every eagerly launched step per kind of kernel (into step_log)

    def __post_init__(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', not {self.dtype!r}")
        if self.block_size < 1 or self.block_size & (self.block_size - 1):
            raise ValueError("block_size must be a power of two")
        if self.num_blocks is not None and self.num_blocks < 1:
            raise ValueError("num_blocks must be >= 1")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError("max_num_batched_tokens must be >= max_num_seqs (one per decode)")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ValueError("max_model_len must be >= 1")
