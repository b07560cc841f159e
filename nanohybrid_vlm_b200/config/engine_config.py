"""Engine options, with the reference's names and meanings where it has them.

The reference keeps them in one dataclass (nanovllm/config.py:9-152) that the entry
point fills from keyword arguments (nanovllm/engine/llm_engine.py:179-181).  The
options that belong to its hybrid (GDN, vision, joint prefix cache) path are absent.
Options that the reference does not have: ``dtype`` (run the checkpoint in another
precision; ``"float32"`` is the true 32-bit path), ``seed``, ``decode_weight_copy``,
``async_decode``, ``profile_ranges`` and ``poison_cache``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields

import torch

from .model_config import ConfigError, ModelConfig, parse_dtype
from .registry import ArchitectureEntry, load_model_config


@dataclass
class Config:
    model: str
    max_num_batched_tokens: int = 16384      # token budget of one step (nanovllm/config.py:12)
    scheduler_policy: str = "decode_first"   # or "prefill_first" (nanovllm/config.py:24)
    max_num_seqs: int = 512                  # live requests (nanovllm/config.py:25)
    max_model_len: int = 4096                # clamped to max_position_embeddings (nanovllm/config.py:420-423)
    gpu_memory_utilization: float = 0.9      # share of device memory the cache may grow into
    tensor_parallel_size: int = 1            # only 1: this engine runs on one GPU
    enforce_eager: bool = False              # True: no CUDA graphs for decode steps
    eos: int = -1                            # filled from config.json's eos_token_id
    kvcache_block_size: int = 256            # tokens per cache page (any positive number here)
    num_kvcache_blocks: int = -1             # pages per cache group; -1: sized from free memory
    num_state_slots: int = -1                # slots of fixed-size per-request state; -1: max_num_seqs if a layer needs them, else 0
    enable_prefix_cache: bool | None = None  # page reuse by content hash; None: on where the model allows it (nanovllm/config.py:393-399)
    decode_weight_copy: bool | None = None   # a second copy of the matrices a decode step streams, one share per SM (faster
                                             # small batches, twice the weight memory); None: when it fits in a
                                             # quarter of the free device memory
    async_decode: bool = True                # launch a decode step before the host has read the tokens of the one before
                                             # (they are passed on on the device); an end-of-sequence token is then seen
                                             # one step late and the extra token dropped.  Needs the CUDA graphs.
    profile_ranges: bool = False             # NVTX ranges around the step, every layer run, the final norm and the head,
                                             # for profilers that filter or group by range
    poison_cache: bool = False               # fill the cache pools with NaN at start: a read of a slot that no step
                                             # wrote shows in the logits (tests, replay)
    dtype: str | torch.dtype | None = None   # None: the checkpoint's own
    seed: int = 0
    # filled by __post_init__
    architecture: ArchitectureEntry | None = field(default=None, repr=False)
    model_config: ModelConfig | None = field(default=None, repr=False)

    def __post_init__(self):
        if not isinstance(self.model, (str, os.PathLike)) or not os.path.isdir(self.model):
            raise ConfigError(f"model must be a folder with config.json and safetensors, got {self.model!r}")
        if self.kvcache_block_size <= 0:
            raise ConfigError("kvcache_block_size must be positive")
        if self.tensor_parallel_size != 1:
            raise ConfigError("tensor_parallel_size must be 1: this engine runs on one GPU")
        if self.scheduler_policy not in ("decode_first", "prefill_first"):
            raise ConfigError("scheduler_policy must be 'decode_first' or 'prefill_first'")
        if self.max_num_batched_tokens <= 0 or self.max_num_seqs <= 0 or self.max_model_len <= 0:
            raise ConfigError("max_num_batched_tokens, max_num_seqs and max_model_len must be positive")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ConfigError("gpu_memory_utilization must be in (0, 1]")
        self.architecture, self.model_config = load_model_config(self.model)
        self.dtype = parse_dtype(self.dtype) if self.dtype is not None else self.model_config.dtype
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ConfigError(f"the engine runs in bfloat16 or float32, not {self.dtype}")
        self.max_model_len = min(self.max_model_len, self.model_config.max_position_embeddings)
        if self.eos == -1 and self.model_config.eos_token_id is not None:
            self.eos = self.model_config.eos_token_id

    @classmethod
    def option_names(cls) -> set[str]:
        return {f.name for f in fields(cls) if f.init and f.name not in ("architecture", "model_config")}
