"""Runtime knobs of the engine (not of the architecture).

Names and meanings follow ``emberserve/config.py:258-312`` where the reference has
them: ``block_size`` (tokens per cache page, 16), ``num_gpu_blocks`` (pages; None =
derive from free memory), ``gpu_memory_utilization`` (0.90), ``max_num_seqs`` (256),
``max_num_batched_tokens`` (token budget of a step, 8192), ``max_model_len`` (4096),
``enable_chunked_prefill``, ``seed``.  The device is always one CUDA GPU.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
}


def dtype_from_str(name: str) -> torch.dtype:
    """``float32`` (the true 32-bit path) or ``bfloat16`` (the serving path)."""
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"unsupported dtype {name!r}; choose float32 or bfloat16") from None


@dataclass
class EngineConfig:
    model_dir: str | None = None
    device: str = "cuda:0"
    dtype: torch.dtype = torch.bfloat16
    block_size: int = 16
    num_gpu_blocks: int | None = None
    gpu_memory_utilization: float = 0.90
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 4096
    enable_chunked_prefill: bool = True
    # Replay pure-decode steps from CUDA graphs (one per batch-size bucket).
    enable_cuda_graphs: bool = True
    # Capture the graphs of all batch-size buckets when the engine is built (as the reference
    # does at boot) instead of at the first step that needs each: a capture costs tens of
    # milliseconds, which a served request would otherwise wait for.
    eager_graph_capture: bool = True
    # Launch a step before the tokens of the step before it have been read on the host: the
    # sampled tokens stay on the device and feed the next step there, and step() returns the
    # outputs of the step before the one it launched.  Requests whose sampling needs their
    # token history on the host (a repetition penalty) switch the engine to plain stepping.
    async_scheduling: bool = True
    # Moves the seeds that requests without a seed of their own are given (sampling/sampler.py).
    seed: int = 0
    # Which attention kernels the bfloat16 path may use (the reference's `attn_backend` chooses
    # among its implementations in the same way, emberserve/config.py:258-312): "auto" the
    # fastest that takes the case, "mma" the mma.sync kernels only (no tcgen05 prompt kernel),
    # "generic" the 32-bit CUDA-core kernel everywhere (the one the float32 path always uses).
    attn_backend: str = "auto"
    # A debugging aid: scratch buffers of the steps get this many guard elements on either side
    # and the engine checks after every step that no kernel wrote there (it waits for the device
    # to do so, so steps no longer overlap).
    debug_scratch_guard: int = 0
    # A second, tiled copy of the projection weights for the kernels of decode steps (they read
    # whole DRAM pages from it: a decode step of a 7B model gets 3 % shorter, and the cache
    # gets smaller by the size of those weights).  None: where the copy takes at most a tenth
    # of the device's memory; True / False: always / never.
    tiled_weight_copies: bool | None = None

    def __post_init__(self) -> None:
        if isinstance(self.dtype, str):
            self.dtype = dtype_from_str(self.dtype)
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"unsupported dtype {self.dtype}; choose float32 or bfloat16")
        if self.attn_backend not in ("auto", "mma", "generic"):
            raise ValueError(f"attn_backend {self.attn_backend!r}: choose auto, mma or generic")
        if self.block_size <= 0:
            raise ValueError("block_size must be positive")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0 or self.max_model_len <= 1:
            raise ValueError("max_num_seqs, max_num_batched_tokens and max_model_len must be positive")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
