"""From a model folder (or a configuration and a seed) to an Engine."""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..config.registry import architecture_for, architecture_of, get_architecture
from ..kernels import build as kernel_build
from ..kernels import ops
from ..parts.base import Runtime
from ..parts.build import build_model
from ..weights.loader import load_weights
from ..weights.random_init import init_random
from .step import Engine

DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
DEFAULT_PAGE_SIZE = 16


def resolve_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype {name} is not float32 or bfloat16")
        return name
    if name not in DTYPES:
        raise ValueError(f"dtype {name!r} is not one of {', '.join(DTYPES)}")
    return DTYPES[name]


def require_gpu(device: Optional[str] = None) -> torch.device:
    """The engine runs on a GPU with its own compiled kernels, or not at all."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine has no CPU path")
    dev = torch.device(device or "cuda:0")
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"the kernels are built for sm_100a only; device {dev} is sm_{major}{minor}")
    return dev


def prepare_kernels(model=None) -> None:
    """Compile, at once and in parallel, every kernel object this model will ask for."""
    sources = ops.base_sources()
    if model is not None:
        for part in model.parts():
            for item in part.kernel_sources():
                if item not in sources:
                    sources.append(item)
    kernel_build.compile_many(sources)


def make_engine(model, page_size: int, num_pages: int, max_requests: int, max_step_tokens: Optional[int] = None,
                guard_pages: bool = False) -> Engine:
    cache = CacheManager(model.cache_entries, page_size, num_pages, max_requests, device=model.rt.device,
                         kv_dtype=model.rt.dtype, max_step_tokens=max_step_tokens, guard_pages=guard_pages)
    engine = Engine(model, cache)
    engine.max_step_tokens = max_step_tokens      # the promise the window groups' pools were sized on
    return engine


def pages_for_tokens(max_tokens: int, page_size: int) -> int:
    return max(1, (int(max_tokens) + page_size - 1) // page_size)


def load_engine(folder: str, dtype="bfloat16", page_size: int = DEFAULT_PAGE_SIZE, num_pages: Optional[int] = None,
                max_tokens: Optional[int] = None, max_requests: int = 64, device: Optional[str] = None,
                strict: bool = True, config_path: Optional[str] = None, weights_path: Optional[str] = None,
                max_step_tokens: Optional[int] = None, guard_pages: bool = False) -> Engine:
    """Read config.json, choose the architecture by its name, load model.safetensors, and set
    up a cache of `num_pages` pages per layer group (or enough for `max_tokens` tokens).  `max_step_tokens`:
    a promise that no request brings more tokens than this in one step, which lets groups of windowed layers
    have smaller pools (see CacheManager).  `guard_pages`: a page of a fixed pattern in front of and behind every
    pool, checked by `engine.cache.check_guards()` (debugging aid)."""
    dev = require_gpu(device)
    with open(config_path or os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    config = arch.config_class.from_dict(raw)
    rt = Runtime(dev, resolve_dtype(dtype))
    model = build_model(arch.build_spec(config), rt)
    prepare_kernels(model)
    report = load_weights(model, weights_path or folder, strict=strict)
    if num_pages is None:
        num_pages = pages_for_tokens(max_tokens if max_tokens is not None else config.max_position_embeddings, page_size)
    engine = make_engine(model, page_size, num_pages, max_requests, max_step_tokens, guard_pages)
    engine.config = config
    engine.load_report = report
    return engine


def random_engine(config, seed: int = 0, dtype="bfloat16", page_size: int = DEFAULT_PAGE_SIZE,
                  num_pages: Optional[int] = None, max_tokens: Optional[int] = None, max_requests: int = 64,
                  device: Optional[str] = None, architecture: Optional[str] = None,
                  storage_dtype: Optional[torch.dtype] = None, draw_on_device: bool = False) -> Engine:
    """An engine over random weights drawn from `seed`, without a model folder.  The architecture is the one
    the configuration's class belongs to, unless named."""
    dev = require_gpu(device)
    arch = get_architecture(architecture) if architecture else architecture_for(config)
    rt = Runtime(dev, resolve_dtype(dtype))
    model = build_model(arch.build_spec(config), rt)
    prepare_kernels(model)
    init_random(model, seed, storage_dtype=storage_dtype, draw_on_device=draw_on_device)
    if num_pages is None:
        num_pages = pages_for_tokens(max_tokens if max_tokens is not None else config.max_position_embeddings, page_size)
    engine = make_engine(model, page_size, num_pages, max_requests)
    engine.config = config
    return engine
