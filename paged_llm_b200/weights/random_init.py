"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode; its tests build the module under a fixed torch
seed (tests/test_engine_cpu.py:41-44).  Here one CPU generator draws every
tensor the model expects in float32, in the sorted order of tensor names:
matrices ~ N(0, std), norm weights 1 (or 1 + N(0, norm_std)); then they are cast
to the storage dtype.  float32 and bfloat16 folders of one seed hold the same
values up to that cast.
"""

from __future__ import annotations

import json
import os

import torch

from ..config.model import ModelConfig
from ..config.registry import ARCHITECTURES

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def random_tensors(config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                   dtype: str = "float32") -> dict[str, torch.Tensor]:
    from ..models.causal_lm import build_model

    arch = ARCHITECTURES[config.architecture]
    model = build_model(arch.build_spec(config))
    gen = torch.Generator().manual_seed(seed)
    out = {}
    specs = model.tensor_specs()
    for name in sorted(specs):
        spec = specs[name]
        if spec.optional and spec.alias_of is not None:
            continue                                    # tied: not written
        if spec.role == "table_int":
            raise NotImplementedError(f"{name}: random integer tables are not defined")
        if spec.init == "norm":
            t = torch.ones(spec.shape, dtype=torch.float32)
            if norm_std:
                t = t + norm_std * torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        else:
            t = std * torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        out[name] = t.to(_DTYPES[dtype]).contiguous()
    return out


def write_model_folder(path: str, config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                       dtype: str = "float32") -> str:
    """Writes `path`/config.json and `path`/model.safetensors; returns `path`."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    hf = config.to_hf_dict()
    hf["torch_dtype"] = dtype
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f, indent=1)
    save_file(random_tensors(config, seed, std, norm_std, dtype), os.path.join(path, "model.safetensors"))
    return path
