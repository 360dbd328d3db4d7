"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed, or the same tensors made in memory.

Every tensor has its own generator seeded from ``(seed, index of its name in
sorted order)``, so a tensor's values do not depend on which other tensors exist
around it in the file.  Matrices are N(0, std), biases N(0, bias_std), norm
gains 1.  Values are made in float32 on the generator's device and rounded once
to the stored dtype.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch

from ..config.registry import parse_config
from ..parts.base import BuildContext, ParamSpec
from .safetensors_io import write_file

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def random_tensors(specs: Mapping[str, ParamSpec], seed: int, std: float = 0.02,
                   bias_std: Optional[float] = None, dtype: torch.dtype = torch.bfloat16,
                   device: str | torch.device = "cpu", skip_optional: bool = True) -> Dict[str, torch.Tensor]:
    bias_std = std if bias_std is None else bias_std
    out: Dict[str, torch.Tensor] = {}
    device = torch.device(device)
    for idx, name in enumerate(sorted(specs)):
        s = specs[name]
        if s.optional and skip_optional:
            continue
        g = torch.Generator(device=device)
        g.manual_seed((int(seed) * 1_000_003 + idx) & 0x7FFF_FFFF_FFFF_FFFF)
        if s.init == "ones":
            t = torch.ones(s.shape, dtype=torch.float32, device=device)
        elif s.init == "zeros":
            t = torch.zeros(s.shape, dtype=torch.float32, device=device)
        elif s.init in ("normal", "bias_normal"):
            sd = std if s.init == "normal" else bias_std
            t = torch.empty(s.shape, dtype=torch.float32, device=device).normal_(0.0, sd, generator=g)
        else:
            raise ValueError(f"tensor {name!r}: unknown init rule {s.init!r}")
        out[name] = t.to(torch.int32 if s.role == "int_table" else dtype)
    return out


def model_param_specs(raw_config: Mapping[str, object]) -> Dict[str, ParamSpec]:
    """The tensors a configuration's model wants; builds the parts without a device."""
    from ..models.decoder import DecoderModel  # local: models import parts import kernels
    cfg = parse_config(raw_config)
    model = DecoderModel(cfg, BuildContext(torch.device("cpu"), torch.float32))
    return model.param_specs()


def write_random_model(out_dir: str, raw_config: Mapping[str, object], seed: int, std: float = 0.02,
                       bias_std: Optional[float] = None, dtype: str = "bfloat16") -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``."""
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
    raw = dict(raw_config)
    raw["torch_dtype"] = dtype
    specs = model_param_specs(raw)
    tensors = random_tensors(specs, seed, std, bias_std, _DTYPES[dtype])
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    write_file(os.path.join(out_dir, "model.safetensors"), tensors,
               metadata={"format": "pt", "seed": str(seed), "std": repr(std)})
    return out_dir
