"""Engine-side settings: cache pool, step limits, scheduler policy, precision.

The scheduler's six limits carry the names and defaults of the reference's
``SchedulerConfig`` (crates/aien-scheduler/src/lib.rs:53-73); the page size defaults to the
reference's fixed block size of 16 (crates/aien-inference-abi/src/model_dir.rs:114).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16" (serving kernels) or "float32" (true 32-bit)
    page_size: int = 16                # tokens per cache page
    num_pages: int = 0                 # pages per cache group; 0 = derive from max_cache_tokens
    max_cache_tokens: int = 0          # tokens the pool must hold when num_pages is 0
    max_requests: int = 64             # live requests (rows of the block table, state slots)
    max_context: int = 0               # longest request; 0 = the model's max position
    # scheduler (reference names)
    max_batch_size: int = 64
    max_batch_tokens: int = 4096
    max_prefill_tokens: int = 2048
    prefill_chunk_size: int = 512
    chunk_prefill: bool = True
    watermark_blocks: int = 4
    align_step_tokens: int = 0         # own option: cut a portion so that a step's tokens fill whole tiles of this many rows (0: off)
    # execution
    use_cuda_graphs: bool = True       # replay captured graphs for decode-only steps
    async_scheduling: bool = True      # plan and launch step n+1 while step n runs; its tokens are fed on the device
    replay_steps: bool = True          # a step shaped like an earlier one re-issues that step's launches as recorded
    seed: int = 0

    def resolved_dtype(self) -> str:
        d = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32"}.get(self.dtype)
        if d is None:
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        return d
