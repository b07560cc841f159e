"""Weights from safetensors, by tensor name.

Every ``*.safetensors`` file of the folder is read (sorted, as nanovllm/utils/loader.py:33-46
does).  The model's tensor table says which checkpoint tensors fill which slice of which
parameter (q/k/v packed into one matrix, gate/up into one; nanovllm/layers/linear.py:102-108,
153-167; a slice may also run along another dimension, be stored transposed, or be one
entry of a stack).  Tensors are kept in the engine's dtype; a parameter declared "float32" stays
32-bit and an "int32" table stays integer.  All problems are collected and raised as ONE
error that lists missing tensors, unexpected tensors and wrong shapes
(nanovllm/utils/loader.py:231-278 reports the same categories).
"""
from __future__ import annotations

import glob
import os

import torch
from safetensors import safe_open


class WeightError(RuntimeError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and ``wrong_shape`` list the tensors."""

    def __init__(self, missing, unexpected, wrong_shape, where: str):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"the checkpoint in {where} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: checkpoint {tuple(got)} but the model wants {tuple(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def storage_dtype(storage: str, model_dtype: torch.dtype) -> torch.dtype:
    if storage == "model":
        return model_dtype
    if storage == "float32":
        return torch.float32
    if storage == "int32":
        return torch.int32
    raise ValueError(f"unknown storage kind {storage!r}")


def checkpoint_files(model_dir: str) -> list[str]:
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {model_dir!r}")
    return files


def load_weights(model, model_dir: str) -> dict[str, torch.Tensor]:
    """Read the checkpoint into device tensors keyed by the model's full parameter names and bind them."""
    table = model.param_table()
    wanted: dict[str, tuple] = {}          # checkpoint name -> (param, source)
    for bp in table:
        for src in bp.decl.sources:
            wanted[src.name] = (bp, src)
    ignored = set(model.spec.ignored_checkpoint_tensors)

    tensors = {bp.name: torch.empty(bp.decl.shape, dtype=storage_dtype(bp.decl.storage, model.dtype),
                                    device=model.device) for bp in table}
    seen, unexpected, wrong = set(), [], []
    for path in checkpoint_files(model_dir):
        with safe_open(path, framework="pt", device="cpu") as f:
            for name in f.keys():
                if name in ignored and name not in wanted:
                    continue
                if name not in wanted:
                    unexpected.append(name)
                    continue
                bp, src = wanted[name]
                got_shape = tuple(f.get_slice(name).get_shape())
                part = src.to_slice(torch.empty(got_shape, device="meta"), bp.decl.shape)
                if part is None:
                    wrong.append((name, got_shape, src.checkpoint_shape(bp.decl.shape)))
                    seen.add(name)
                    continue
                t = src.to_slice(f.get_tensor(name), bp.decl.shape)
                dst = tensors[bp.name]
                dst.narrow(src.dim, src.row, src.rows).copy_(t.to(dst.dtype) if t.dtype != dst.dtype else t)
                seen.add(name)
    missing = [n for n in wanted if n not in seen]
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong), model_dir)
    model.bind(tensors)
    return tensors
