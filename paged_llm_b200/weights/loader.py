"""Weights from a model folder: config.json plus *.safetensors, by tensor name.

The reference copies every tensor of every `*.safetensors` file into the
parameter of the same name, ignores names ending in `rotary_emb.inv_freq`, and
raises on an unexpected name or on missing ones (pagedllm/model/loader.py:39-69).
Here the model says which tensors it expects (`tensor_specs`) and the loader
checks all of them at once: ONE error lists every missing tensor, every
unexpected tensor, every wrong shape and every tensor stored in a type that its
role cannot take (an integer or 8-bit tensor where a matrix is expected).

Storage: matrices are kept in the compute dtype (bfloat16 or float32); vectors
(norm weights) that the file stores in 32-bit stay 32-bit; integer tables become
int32.
"""

from __future__ import annotations

import glob
import json
import os

import torch

from ..config.registry import parse_model_config
from ..parts.base import TensorSpec

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class WeightError(KeyError):
    """The checkpoint does not match the model.  `missing`, `unexpected`,
    `wrong_shape`, `wrong_dtype` and `duplicates` hold the offending names."""

    def __init__(self, missing, unexpected, wrong_shape, duplicates=(), wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.duplicates = list(wrong_shape), list(duplicates)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file {tuple(got)} != expected {tuple(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n}: file stores {got}, a {role} needs {want}" for n, got, role, want in self.wrong_dtype))
        if self.duplicates:
            lines.append(f"  stored in more than one file ({len(self.duplicates)}): " + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))

    def __str__(self):
        return self.args[0]


def read_hf_config(path: str) -> dict:
    cfg_path = os.path.join(path, "config.json")
    if not os.path.isfile(cfg_path):
        raise FileNotFoundError(f"{path!r} has no config.json (a model folder holds config.json and *.safetensors)")
    with open(cfg_path) as f:
        return json.load(f)


def resolve_dtype(requested: str, hf_config: dict) -> torch.dtype:
    """'auto' follows the checkpoint's `torch_dtype` (or `dtype`) key, as the
    reference does (loader.py:33-36); half-precision checkpoints run in bfloat16."""
    if requested == "auto":
        requested = hf_config.get("torch_dtype") or hf_config.get("dtype") or "float16"
    if requested in ("float16", "half", "bf16"):
        requested = "bfloat16"
    if requested in ("fp32", "float"):
        requested = "float32"
    try:
        return _DTYPES[requested]
    except KeyError:
        raise ValueError(f"unknown dtype {requested!r}; use bfloat16 or float32") from None


def storage_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "table_int":
        return torch.int32
    if spec.role == "vector" and stored == torch.float32:
        return torch.float32
    return compute


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def stored_dtype_ok(spec: TensorSpec, stored: torch.dtype) -> bool:
    """Matrices and vectors must be stored as floating point of 16 bits or more (an 8-bit or
    integer tensor would be a quantized checkpoint, which this engine does not run, and casting
    it would give numbers that mean nothing); integer tables as integers."""
    return stored in (_INTS if spec.role == "table_int" else _FLOATS)


def read_safetensors(path: str) -> tuple[dict[str, torch.Tensor], list[str]]:
    """All tensors of all *.safetensors files of a folder, on the CPU, and the
    names that occur in more than one file."""
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"{path!r} holds no *.safetensors file")
    tensors: dict[str, torch.Tensor] = {}
    duplicates: list[str] = []
    for file in files:
        with safe_open(file, framework="pt", device="cpu") as f:
            for name in f.keys():
                if name in tensors:
                    duplicates.append(name)
                tensors[name] = f.get_tensor(name)
    return tensors, duplicates


def check_and_cast(expected: dict[str, TensorSpec], tensors: dict[str, torch.Tensor], compute: torch.dtype,
                   device, ignored_suffixes: tuple[str, ...] = (), duplicates=()) -> dict[str, torch.Tensor]:
    """Validate names and shapes against the model's expectations, then cast and
    move.  Raises one `WeightError` that lists everything that is wrong."""
    missing, unexpected, wrong_shape, wrong_dtype = [], [], [], []
    for name, spec in expected.items():
        if name not in tensors:
            if not spec.optional:
                missing.append(name)
            continue
        if tuple(tensors[name].shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(tensors[name].shape), tuple(spec.shape)))
        if not stored_dtype_ok(spec, tensors[name].dtype):
            wrong_dtype.append((name, str(tensors[name].dtype).replace("torch.", ""), spec.role,
                                "an integer type" if spec.role == "table_int" else "float32, bfloat16 or float16"))
    for name in tensors:
        if name not in expected and not any(name.endswith(s) for s in ignored_suffixes):
            unexpected.append(name)
    if missing or unexpected or wrong_shape or duplicates or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(duplicates), sorted(wrong_dtype))
    out = {}
    for name, spec in expected.items():
        if name not in tensors:
            continue
        if spec.optional and spec.alias_of is not None:
            continue        # a tied head: the tensor it is tied to is used
        t = tensors[name]
        out[name] = t.to(device=device, dtype=storage_dtype(spec, t.dtype, compute)).contiguous()
    return out


def load_model(path: str, dtype: str = "auto", device="cuda", ops=None):
    """Folder -> (model with weights on `device`, typed config, compute dtype).  A folder that
    holds `random_weights.json` instead of tensors (weights/random_init.py: `write_random_stub`)
    gets its weights drawn on the device by `ops`, the kernel library."""
    from ..models.causal_lm import build_model
    from .random_init import draw_on_device, read_random_stub

    hf_config = read_hf_config(path)
    arch, config = parse_model_config(hf_config)
    compute = resolve_dtype(dtype, hf_config)
    spec = arch.build_spec(config)
    model = build_model(spec)
    stub = read_random_stub(path)
    if stub is not None:
        if glob.glob(os.path.join(path, "*.safetensors")):
            raise ValueError(f"{path!r} holds both random_weights.json and *.safetensors files; remove one")
        if ops is None or not hasattr(ops, "fill_normal"):
            raise ValueError(f"{path!r} holds random_weights.json: its weights are drawn on the device, which needs "
                             "the kernel library (pass ops)")
        model.load(draw_on_device(model.tensor_specs(), stub, compute, device, ops))
        return model, config, compute
    tensors, duplicates = read_safetensors(path)
    cast = check_and_cast(model.tensor_specs(), tensors, compute, device, spec.ignored_tensors, duplicates)
    model.load(cast)
    return model, config, compute
