"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode; its tests build the module under a fixed torch
seed (tests/test_engine_cpu.py:41-44).  Here one CPU generator draws every
tensor the model expects in float32, in the sorted order of tensor names:
matrices ~ N(0, std), norm weights 1 (or 1 + N(0, norm_std)); then they are cast
to the storage dtype.  float32 and bfloat16 folders of one seed hold the same
values up to that cast.

For benchmark models that are too large to draw and store that way (8 billion
parameters), `write_random_stub` writes a folder with config.json and
`random_weights.json` (seed, std, norm_std) and no tensors; the loader then
draws every expected tensor on the device (`draw_on_device`) with a kernel of
this package, keyed by the seed and the tensor's name, so that the same stub
always gives the same model.
"""

from __future__ import annotations

import json
import os

import torch

import hashlib

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


STUB_FILE = "random_weights.json"


def write_random_stub(path: str, config: ModelConfig, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                      dtype: str = "bfloat16") -> str:
    """A model folder without tensors: config.json and `random_weights.json`.  Loading it draws
    the weights on the device (`draw_on_device`)."""
    os.makedirs(path, exist_ok=True)
    hf = config.to_hf_dict()
    hf["torch_dtype"] = dtype
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f, indent=1)
    with open(os.path.join(path, STUB_FILE), "w") as f:
        json.dump({"seed": int(seed), "std": float(std), "norm_std": float(norm_std)}, f)
    return path


def read_random_stub(path: str) -> dict | None:
    """The stub's parameters if `path` is a folder written by `write_random_stub`, else None."""
    file = os.path.join(path, STUB_FILE)
    if not os.path.isfile(file):
        return None
    with open(file) as f:
        stub = json.load(f)
    unknown = set(stub) - {"seed", "std", "norm_std"}
    if unknown or "seed" not in stub:
        raise ValueError(f"{file}: expected the keys seed, std, norm_std; got {sorted(stub)}")
    return {"seed": int(stub["seed"]), "std": float(stub.get("std", 0.02)), "norm_std": float(stub.get("norm_std", 0.0))}


def tensor_key(name: str) -> int:
    """The 64-bit stream key of a tensor name (so that a tensor's values do not depend on which
    other tensors the model has)."""
    return int.from_bytes(hashlib.blake2b(name.encode(), digest_size=8).digest(), "little")


def draw_on_device(expected: dict, stub: dict, compute: torch.dtype, device, ops) -> dict[str, torch.Tensor]:
    """Every expected tensor drawn on the device by `ops.fill_normal`: matrices ~ N(0, std) in the
    compute dtype, norm weights 1 + N(0, norm_std) in float32.  Tied tensors are left out."""
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.optional and spec.alias_of is not None:
            continue
        if spec.role == "table_int":
            raise NotImplementedError(f"{name}: random integer tables are not defined")
        if spec.init == "norm":
            t = torch.empty(spec.shape, dtype=torch.float32, device=device)
            if stub["norm_std"]:
                ops.fill_normal(t, stub["seed"], tensor_key(name), 1.0, stub["norm_std"])
            else:
                t.fill_(1.0)
        else:
            t = torch.empty(spec.shape, dtype=compute, device=device)
            ops.fill_normal(t, stub["seed"], tensor_key(name), 0.0, stub["std"])
        out[name] = t
    return out
