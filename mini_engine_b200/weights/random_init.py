"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (its parameters are ``torch.empty`` until loaded,
layers/linear.py:10,34).  The folder holds ``config.json`` and ``model.safetensors`` with
the architecture's own disk names (unpacked q/k/v and gate/up), so that the engine loads
it like any other model and the by-name loader is exercised.  Matrices are N(0, 0.02),
norm weights 1 + N(0, 0.1), drawn tensor by tensor in the model's declaration order from
one seeded CPU generator.
"""
from __future__ import annotations

import json
import os
from typing import Any

import torch
from safetensors.torch import save_file

from ..config.model_config import architecture_name
from ..config.registry import get_architecture
from ..parts.model import DecoderModel
from .loader import expected_disk_tensors, iter_param_decls


def build_model_from_config_dict(raw: dict[str, Any]) -> tuple[Any, DecoderModel]:
    arch = get_architecture(architecture_name(raw))
    cfg = arch.config_from_dict(raw)
    return cfg, DecoderModel(arch.plan(cfg))


def random_state_dict(model: DecoderModel, seed: int, dtype: torch.dtype = torch.bfloat16,
                      matrix_std: float = 0.02, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    init_of = {}
    for prefix, _, decl in iter_param_decls(model):
        if decl.tied_to is not None:
            continue
        names = [prefix + s.disk_name for s in decl.sources] or [prefix + decl.name]
        for n in names:
            init_of[n] = decl.init
    out: dict[str, torch.Tensor] = {}
    for name, e in expected_disk_tensors(model).items():
        x = torch.randn(e.shape, generator=gen, dtype=torch.float32)
        x = 1.0 + norm_std * x if init_of[name] == "norm" else matrix_std * x
        out[name] = x.to(dtype).contiguous()
    return out


def write_random_model(folder: str, config: dict[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, matrix_std: float = 0.02, norm_std: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``folder``; returns the folder.

    ``matrix_std``: with wider matrices (0.1, say) what the layers add to the residual stream outweighs the token's
    own embedding, so the next token depends on the cache far more than on the token itself."""
    folder = os.path.expanduser(folder)
    os.makedirs(folder, exist_ok=True)
    _, model = build_model_from_config_dict(config)
    tensors = random_state_dict(model, seed, dtype, matrix_std, norm_std)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder


def init_random_on_device(model: DecoderModel, seed: int, dtype: torch.dtype, device,
                          matrix_std: float = 0.02, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Fill every part's ``params`` with random numbers drawn on ``device``: no files, no host copy.

    For benchmarks at sizes whose files would take minutes to write and read (a 32B shape is 65 GB).  Same laws
    as ``write_random_model`` (matrices N(0, matrix_std) in ``dtype``, norm weights 1 + N(0, norm_std) in
    float32), drawn parameter by parameter in declaration order from one generator seeded on the device; the
    numbers are not those of ``write_random_model`` with the same seed."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    params: dict[str, torch.Tensor] = {}
    tied = []
    for prefix, part, decl in iter_param_decls(model):
        full = prefix + decl.name
        if decl.tied_to is not None:
            tied.append((full, part, decl))
            continue
        if decl.role == "vector":
            t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, 1.0, generator=gen)
            t = t.mul_(norm_std).add_(1.0) if decl.init == "norm" else t.mul_(matrix_std)
        else:
            t = torch.empty(decl.shape, dtype=dtype, device=device).normal_(0.0, matrix_std, generator=gen)
            if decl.init == "norm":
                t = t.mul_(norm_std / matrix_std).add_(1.0)
        params[full] = part.params[decl.name] = t
    for full, part, decl in tied:
        params[full] = part.params[decl.name] = params[decl.tied_to]
    return params
