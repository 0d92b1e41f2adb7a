"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference's `Weights::random(cfg, seed)` fills matrices uniformly in
+-1/sqrt(d) with a splitmix-style generator and leaves biases empty
(crates/mach-model/src/weights.rs:230-245, :367-374, :665-690 of
gqf2008/machserve).  Here values are normal, biases are filled too, and the
generator is spelled out so that a folder is reproducible from (config, seed)
alone: value i of a tensor comes from two SplitMix64 outputs of a counter that
starts at a 64-bit hash of (seed, tensor name), turned into a normal deviate by
Box-Muller in float64.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable

import numpy as np
import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _name_key(seed: int, name: str) -> np.uint64:
    h = 0xCBF29CE484222325  # FNV-1a over the name's bytes
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    with np.errstate(over="ignore"):
        return _mix(np.array([(h ^ (seed & 0xFFFFFFFFFFFFFFFF)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0]


def normal_values(seed: int, name: str, count: int) -> np.ndarray:
    """`count` standard normal deviates (float64) that depend on (seed, name) only."""
    out = np.empty(count, dtype=np.float64)
    key = _name_key(seed, name)
    chunk = 1 << 22
    with np.errstate(over="ignore"):
        for start in range(0, count, chunk):
            n = min(chunk, count - start)
            idx = np.arange(start, start + n, dtype=np.uint64)
            a = _mix(key + (np.uint64(2) * idx + np.uint64(1)) * _GOLDEN)
            b = _mix(key + (np.uint64(2) * idx + np.uint64(2)) * _GOLDEN)
            u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740992.0  # (0, 1]
            u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0  # [0, 1)
            out[start : start + n] = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return out


def random_tensors(
    declared: Iterable[TensorDecl],
    seed: int,
    dtype: torch.dtype = torch.float32,
    weight_std: float = 0.02,
    bias_std: float = 0.02,
    norm_std: float = 0.05,
) -> Dict[str, torch.Tensor]:
    """CPU tensors for every declared tensor (optional ones too, unless declared with random=False)."""
    out: Dict[str, torch.Tensor] = {}
    for d in declared:
        if d.name in out or not d.random:
            continue
        count = int(np.prod(d.shape, dtype=np.int64)) if d.shape else 1
        if d.init == "table":
            out[d.name] = torch.zeros(d.shape, dtype=torch.int32)
            continue
        if d.init == "zeros":
            vals = np.zeros(count)
        else:
            vals = normal_values(seed, d.name, count)
            if d.init == "matrix":
                vals *= weight_std
            elif d.init == "bias":
                vals *= bias_std
            elif d.init == "scale":
                vals = 1.0 + norm_std * vals
            else:
                raise ValueError(f"tensor '{d.name}': unknown init '{d.init}'")
        out[d.name] = torch.from_numpy(vals.astype(np.float32).reshape(d.shape)).to(dtype)
    return out


def random_tensors_on_device(
    declared: Iterable[TensorDecl],
    seed: int,
    dtype: torch.dtype,
    device,
    weight_std: float = 0.02,
    bias_std: float = 0.02,
    norm_std: float = 0.05,
) -> Dict[str, torch.Tensor]:
    """The same kinds of values as `random_tensors`, drawn by the device's own generator: for models of
    billions of parameters whose values need not be reproducible elsewhere (a benchmark's weights).  A tensor's
    values depend on (seed, its name) and on the device's generator, not on the other tensors."""
    out: Dict[str, torch.Tensor] = {}
    gen = torch.Generator(device=device)
    for d in declared:
        if d.name in out or not d.random:
            continue
        if d.init == "table":
            out[d.name] = torch.zeros(d.shape, dtype=torch.int32, device=device)
            continue
        if d.init == "zeros":
            out[d.name] = torch.zeros(d.shape, dtype=dtype, device=device)
            continue
        gen.manual_seed(int(_name_key(seed, d.name)) & 0x7FFFFFFFFFFFFFFF)
        if d.init == "matrix":
            t = torch.randn(d.shape, dtype=dtype, device=device, generator=gen).mul_(weight_std)
        elif d.init == "bias":
            t = torch.randn(d.shape, dtype=torch.float32, device=device, generator=gen).mul_(bias_std).to(dtype)
        elif d.init == "scale":
            t = torch.randn(d.shape, dtype=torch.float32, device=device, generator=gen).mul_(norm_std).add_(1.0).to(dtype)
        else:
            raise ValueError(f"tensor '{d.name}': unknown init '{d.init}'")
        out[d.name] = t
    return out


def write_random_model(
    config,
    out_dir,
    seed: int,
    dtype: torch.dtype = torch.float32,
    weight_std: float = 0.02,
    bias_std: float = 0.02,
    norm_std: float = 0.05,
) -> Path:
    """Writes `out_dir/config.json` and `out_dir/model.safetensors` for `config` (a typed configuration)."""
    from ..parts.model import declared_tensors  # late: parts import this package

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    spec = config.model_spec()
    decls = declared_tensors(spec)
    tensors = random_tensors(decls, seed, dtype, weight_std, bias_std, norm_std)
    raw = config.to_json()
    raw["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float32"
    (out / "config.json").write_text(json.dumps(raw, indent=1))
    write_safetensors(out / "model.safetensors", tensors)
    return out
