"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration
and a seed, and the same weights made directly on the device for models too large to
write out.

Matrices and embeddings are N(0, 0.02); norm weights are 1 + N(0, 0.01) (or N(0, 0.01)
for norms stored as an offset from one).  Each checkpoint tensor has its own generator
seeded from (seed, tensor name), so a tensor's values do not depend on the others.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch
from safetensors.torch import save_file

from ..config.registry import ARCHITECTURES
from .loader import storage_dtype


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def _normal(std: float, mean: float = 0.0):
    def draw(shape, gen, device):
        t = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
        return t + mean if mean else t
    return draw


# init kind (``ParamDecl.init``) -> function (shape, generator, device) -> float32 tensor
INITS = {
    "normal": _normal(0.02),
    "norm": _normal(0.01, 1.0),
    "zeros_noise": _normal(0.01),
    "zeros": lambda shape, gen, device: torch.zeros(shape, dtype=torch.float32, device=device),
}


def register_init(kind: str, draw) -> None:
    """Another way of filling a tensor in the random-weights mode: ``draw(shape, generator, device)`` returns
    a float32 tensor; parts name it in ``ParamDecl.init``."""
    INITS[kind] = draw


def _draw(shape, init: str, gen: torch.Generator, device) -> torch.Tensor:
    if init not in INITS:
        raise ValueError(f"unknown init kind {init!r}; known: {sorted(INITS)}")
    return INITS[init](tuple(shape), gen, device)


def random_checkpoint(model, seed: int, dtype: torch.dtype) -> dict[str, torch.Tensor]:
    """CPU tensors under the checkpoint's own names (separate q/k/v, gate/up)."""
    out = {}
    for bp in model.param_table():
        for src in bp.decl.sources:
            gen = torch.Generator(device="cpu").manual_seed(tensor_seed(seed, src.name))
            t = _draw(src.checkpoint_shape(bp.decl.shape), bp.decl.init, gen, "cpu")     # in the file's own layout
            out[src.name] = t.to(storage_dtype(bp.decl.storage, dtype)).contiguous()
    return out


def write_random_model(model_dir: str, config: dict, seed: int) -> str:
    """Write ``config.json`` and ``model.safetensors`` for the architecture that ``config`` names.

    ``config`` is a config.json dictionary (it must carry ``architectures`` and a dtype).  The
    tensors are stored in that dtype."""
    from ..engine.model import CausalLM
    from .. import models  # noqa: F401
    entry = ARCHITECTURES.resolve(config)
    cfg = entry.parse_config(config)
    model = CausalLM(entry.build_spec(cfg), cfg.dtype, "cpu")
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_checkpoint(model, seed, cfg.dtype)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    return model_dir


def materialize_random(model, seed: int) -> dict[str, torch.Tensor]:
    """Fill the model with random weights made on its own device (no file).  Used where writing the
    checkpoint out would cost more than the run (benchmarks and replay at full size).

    The rule, so that another program can make the same tensors: every checkpoint tensor is ONE draw of its
    whole shape in float32 from ``torch.Generator(device).manual_seed(tensor_seed(seed, name))``, then cast.
    (The device's generator is not the CPU's: a folder written by ``write_random_model`` from the same seed
    holds other numbers.)"""
    tensors = {}
    for bp in model.param_table():
        dst = torch.empty(bp.decl.shape, dtype=storage_dtype(bp.decl.storage, model.dtype), device=model.device)
        for src in bp.decl.sources:
            gen = torch.Generator(device=model.device).manual_seed(tensor_seed(seed, src.name))
            t = _draw(src.checkpoint_shape(bp.decl.shape), bp.decl.init, gen, model.device)
            dst.narrow(src.dim, src.row, src.rows).copy_(src.to_slice(t, bp.decl.shape))
        tensors[bp.name] = dst
    model.bind(tensors)
    return tensors
