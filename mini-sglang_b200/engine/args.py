"""Options of the engine, with the names and meanings of the reference's ServerArgs where it has
them (mini_sglang/managers/server_args.py:16-60) and its four environment tunables
(mini_sglang/utils/global_vars.py:11-27).  Options of things this engine does not have (HTTP
host/port, tensor parallel size, NCCL port, choice of attention backend, device) are left out;
`tp_size` and `device` are accepted only with their single legal value."""

from __future__ import annotations

import argparse
import dataclasses
import os
import random
from typing import List, Optional


def _env(name: str, default: float) -> float:
    return float(os.environ.get(name, default))


@dataclasses.dataclass
class EngineArgs:
    model: str
    page_size: int = 16                      # the reference's default is 1 (accepted here too); the kernels are tuned for 16
    max_num_reqs: int = 1024
    max_capture_bs: int = 128
    schedule_policy: str = "lpm"
    tp_size: int = 1
    device: str = "cuda"
    gpu_memory_utilization: float = 0.9
    log_level: str = "INFO"
    random_seed: Optional[int] = None
    profile: bool = False
    disable_radix_cache: bool = False
    disable_cuda_graph: bool = False
    schedule_conservativeness: float = 1.0
    max_prefill_tokens: int = 16384
    dummy_load: bool = False
    attention_backend: Optional[str] = None  # the reference chooses between library kernels here; this engine has its own kernels only
    # this engine's own
    dtype: str = "bfloat16"                  # "bfloat16" | "float32" (true 32-bit everywhere)
    num_pages: Optional[int] = None          # size of the cache in pages instead of a memory fraction
    chunk_size: int = 8192                   # longest portion of one prompt in one step
    max_context_len: Optional[int] = None    # default: the model's max_position_embeddings
    disable_overlap: bool = False            # read every step's tokens before the next step is launched
    profile_dir: str = "traces"              # where --profile saves its per-step records
    init_new_token_ratio: float = dataclasses.field(default_factory=lambda: _env("SGLANG_INIT_NEW_TOKEN_RATIO", 0.7))
    min_new_token_ratio_factor: float = dataclasses.field(default_factory=lambda: _env("SGLANG_MIN_NEW_TOKEN_RATIO_FACTOR", 0.14))
    new_token_ratio_decay_steps: int = dataclasses.field(default_factory=lambda: int(_env("SGLANG_NEW_TOKEN_RATIO_DECAY_STEPS", 600)))
    retract_decode_steps: int = dataclasses.field(default_factory=lambda: int(_env("SGLANG_RETRACT_DECODE_STEPS", 20)))

    def __post_init__(self):
        self.model = os.path.expanduser(self.model)
        if not os.path.isdir(self.model):
            raise ValueError(f"--model {self.model!r} is not a folder")
        if self.random_seed is None:
            self.random_seed = random.randint(0, 1 << 30)
        if self.tp_size != 1:
            raise ValueError("this engine runs on one GPU: tp_size must be 1")
        if not str(self.device).startswith("cuda"):
            raise ValueError("this engine runs on a CUDA device only")
        if self.dtype not in ("bfloat16", "float32", "bf16", "fp32"):
            raise ValueError("dtype must be bfloat16 or float32")
        if self.schedule_policy not in ("fcfs", "lof", "random", "lpm", "dfs-weight"):
            raise ValueError(f"unknown schedule policy {self.schedule_policy!r}")
        if self.disable_radix_cache and self.schedule_policy not in ("fcfs", "lof", "random"):
            raise ValueError(f"schedule policy {self.schedule_policy} needs the radix cache; with "
                             "--disable_radix_cache choose from fcfs, lof, random")
        if self.page_size < 1:
            raise ValueError("page_size must be at least 1")

    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> None:
        d = EngineArgs
        parser.add_argument("--model", type=str, required=True, help="Model folder: config.json and *.safetensors (and a tokenizer, for text prompts).")
        parser.add_argument("--page_size", type=int, default=d.page_size, help="Tokens per page of the key/value cache (a power of two from 8 on suits the TMA kernels; 1 is allowed).")
        parser.add_argument("--attention_backend", type=str, default=None,
                            help="Accepted so that the reference's command lines keep working; this engine has one attention backend, its own kernels.")
        parser.add_argument("--tp_size", type=int, default=1, help="Number of GPUs the model is split over; this engine takes 1 only.")
        parser.add_argument("--device", type=str, default="cuda", help="Where the model runs; a CUDA device, nothing else.")
        parser.add_argument("--gpu_memory_utilization", type=float, default=d.gpu_memory_utilization,
                            help="Share of the GPU's memory that weights and cache together may fill (0..1).")
        parser.add_argument("--max_num_reqs", type=int, default=d.max_num_reqs, help="Most requests that may hold a cache slot at one time.")
        parser.add_argument("--schedule_policy", type=str, default=d.schedule_policy,
                            choices=["fcfs", "lof", "random", "lpm", "dfs-weight"], help="Order in which waiting requests are admitted: lpm (longest cached prefix first), fcfs, lof (largest max_new_tokens first), random.")
        parser.add_argument("--log_level", type=str, default=d.log_level,
                            choices=["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"], help="Threshold of the engine's log output.")
        parser.add_argument("--random_seed", type=int, default=None, help="Seed of sampling and of --dummy_load weights; drawn at random when absent.")
        parser.add_argument("--profile", action="store_true", help="Time every step on host and device, mark steps and layers with NVTX ranges, and save one JSON record per step under --profile_dir.")
        parser.add_argument("--disable_radix_cache", action="store_true", help="Never share prompt prefixes between requests.")
        parser.add_argument("--disable_cuda_graph", action="store_true", help="Launch decode steps kernel by kernel instead of replaying a captured graph.")
        parser.add_argument("--max_capture_bs", type=int, default=d.max_capture_bs,
                            help="Largest decode batch that gets a captured graph; larger ones are launched kernel by kernel.")
        parser.add_argument("--schedule-conservativeness", type=float, default=d.schedule_conservativeness,
                            help="Scales the estimate of how many tokens a request will still generate when it is admitted: above 1 admits fewer at a time, below 1 more (and retracts when wrong).")
        parser.add_argument("--max_prefill_tokens", type=int, default=d.max_prefill_tokens,
                            help="Token budget of one step: decoded tokens plus prompt portions.")
        parser.add_argument("--dummy_load", action="store_true",
                            help="Random weights for the configuration in --model instead of its checkpoint.")
        parser.add_argument("--dtype", type=str, default=d.dtype, choices=["bfloat16", "float32"])
        parser.add_argument("--num_pages", type=int, default=None, help="Cache size in pages (default: from memory).")
        parser.add_argument("--chunk_size", type=int, default=d.chunk_size, help="Longest prompt portion per step.")
        parser.add_argument("--max_context_len", type=int, default=None)
        parser.add_argument("--profile_dir", type=str, default=d.profile_dir, help="Folder for the records of --profile.")
        parser.add_argument("--disable_overlap", action="store_true",
                            help="Read a step's tokens before launching the next step (no look-ahead decode).")

    @classmethod
    def from_cli_args(cls, ns: argparse.Namespace) -> "EngineArgs":
        names = [f.name for f in dataclasses.fields(cls)]
        return cls(**{n: getattr(ns, n) for n in names if hasattr(ns, n)})


ServerArgs = EngineArgs      # the reference's name for the same thing
