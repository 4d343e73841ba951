"""``Model``: a model folder (or a configuration and a seed) brought onto the device.

The Python surface follows the reference's binding (python/bindings.cpp:31-52):
``Model.load(path)``, ``.config``, ``.weight_bytes`` and ``.logits(tokens)`` -- the
logits at every position of one sequence, computed as a single prefill over a fresh
cache.  Added here: ``Model.random(config, seed)`` in the manner of the C++
``Model::random`` (src/model.cpp:176-218), a ``dtype`` that selects the serving
(bfloat16) or the exact (float32) kernels, and ``write_random_folder``.
"""
from __future__ import annotations

import os
import tempfile
from typing import Optional, Sequence

import numpy as np
import torch

from .cache.storage import build_cache
from .config.registry import architecture_of, config_from_folder, lookup_architecture
from .engine.step import StepEntry, Stepper
from .weights.loader import load_state, state_from_tensors
from .weights.random_init import random_tensors, write_model_folder

_TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_ALIASES = {"fp32": "float32", "f32": "float32", "float32": "float32", "bf16": "bfloat16", "bfloat16": "bfloat16"}


def normalize_dtype(dtype: str) -> str:
    try:
        return _ALIASES[str(dtype).replace("torch.", "")]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not one of float32, bfloat16") from None


def _default_ops(dtype: str):
    from .kernels.ops import get_ops
    return get_ops(dtype)


class Model:
    def __init__(self, decoder, dtype: str, device, ops):
        self.decoder = decoder
        self.dtype = dtype
        self.device = device
        self.ops = ops

    # -- construction ------------------------------------------------------------------
    @staticmethod
    def load(folder: str, dtype: str = "bfloat16", device="cuda:0", ops=None) -> "Model":
        """Read ``folder/config.json`` and its safetensors; the model class is chosen by
        config.json's ``architectures``."""
        dtype = normalize_dtype(dtype)
        arch, config = config_from_folder(folder)
        decoder = arch.build(config)
        ops = ops or _default_ops(dtype)
        state = load_state(folder, decoder.param_specs(), _TORCH_DTYPE[dtype], device,
                           ignorable=decoder.ignorable_tensor, aliases=decoder.tensor_aliases())
        decoder.load_params(state, dtype, device)
        decoder.prepare(ops)
        return Model(decoder, dtype, device, ops)

    @staticmethod
    def random(config, seed: int = 0, dtype: str = "bfloat16", device="cuda:0", ops=None, std: float = 0.02,
               norm_jitter: float = 0.0, fast: bool = False) -> "Model":
        """Random weights from a configuration and a seed.  By default the values are
        those that ``write_random_folder`` writes for the same seed; ``fast`` fills the
        tensors on the device with torch's generator instead (for timing runs of large
        shapes, not reproducible on the host)."""
        dtype = normalize_dtype(dtype)
        arch = lookup_architecture(config.architectures[0])
        decoder = arch.build(config)
        ops = ops or _default_ops(dtype)
        specs = decoder.param_specs()
        tdt = _TORCH_DTYPE[dtype]
        if fast:
            gen = torch.Generator(device=device)
            gen.manual_seed(seed)
            state = {}
            for s in specs:
                if s.init == "ones":
                    state[s.name] = torch.ones(s.shape, dtype=torch.float32, device=device)
                else:
                    t = torch.empty(s.shape, dtype=torch.float32, device=device)
                    t.normal_(0.0, std, generator=gen)
                    state[s.name] = t.to(tdt)
        else:
            tensors = random_tensors(specs, seed, torch.float32 if dtype == "float32" else torch.bfloat16,
                                     std, norm_jitter)
            state = state_from_tensors(tensors, specs, tdt, device)
        decoder.load_params(state, dtype, device)
        decoder.prepare(ops)
        return Model(decoder, dtype, device, ops)

    @staticmethod
    def write_random_folder(folder: str, config, seed: int = 0, dtype: str = "float32", std: float = 0.02,
                            norm_jitter: float = 0.0) -> str:
        """Write ``config.json`` and ``model.safetensors`` of a random model (no device needed)."""
        arch = lookup_architecture(config.architectures[0])
        decoder = arch.build(config)
        return write_model_folder(folder, config, decoder.param_specs(), seed,
                                  _TORCH_DTYPE[normalize_dtype(dtype)], std, norm_jitter)

    # -- the reference's read-only surface ----------------------------------------------
    @property
    def config(self):
        return self.decoder.config

    @property
    def weight_bytes(self) -> int:
        return self.decoder.param_bytes()

    def logits(self, tokens: Sequence[int], page_size: int = 16) -> np.ndarray:
        """Logits [len(tokens), vocab] of one sequence, as one prefill over a fresh cache
        (python/bindings.cpp:35-52)."""
        n = len(tokens)
        pages = (n + page_size - 1) // page_size
        manager, storage = build_cache(self.decoder, pages, page_size, 1, _TORCH_DTYPE[self.dtype], self.device)
        stepper = Stepper(self.decoder, manager, storage, self.ops, max_rows=n, max_seqs=1,
                          max_tokens_per_request=pages * page_size)
        out = stepper.run([StepEntry("logits", list(tokens), list(range(n)))])
        return out.float().cpu().numpy().copy()
