"""Loading a model's weights by tensor name, and writing a random model folder.

The loader compares what the model declares with what the folder holds BEFORE anything is copied,
and raises one :class:`WeightError` that lists every missing tensor, every unexpected tensor and
every wrong shape.  Tensors that parts declare ignorable (a tied model's redundant ``lm_head.weight``,
stored ``rotary_emb.inv_freq``) are passed over as the reference passes them over
(src/model/mod.rs:725).  The reference reports a missing tensor by name (src/weights.rs:501-505) and
lets shape mismatches surface later as matmul errors; here nothing loads unless all of it fits.

Matrices are held in the compute dtype (bfloat16, or float32 on the 32-bit path); norm weights are
held in float32 whatever they were stored in, so a tensor stored in 32-bit stays so.
"""
from __future__ import annotations

import fnmatch
import json
import os
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import TensorSpec
from .random_init import RandomWeights
from .safetensors_io import TensorDirectory, write_safetensors


class WeightError(ValueError):
    def __init__(self, missing: Sequence[str], unexpected: Sequence[str], wrong_shape: Sequence[str],
                 wrong_dtype: Sequence[str] = ()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unsupported dtypes ({len(self.wrong_dtype)}): " + "; ".join(self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def check_tensors(specs: Sequence[TensorSpec], directory: TensorDirectory, ignorable: Sequence[str] = ()) -> None:
    """``ignorable``: names or shell patterns of tensors the folder may hold without the model using them
    (a copy of a tied head, stored rotary frequencies); every other undeclared tensor is an error."""
    expected: Dict[str, TensorSpec] = {s.name: s for s in specs}
    have = set(directory.names())
    missing = [n for n in expected if n not in have]
    unexpected = sorted(n for n in have if n not in expected and not any(fnmatch.fnmatchcase(n, pat) for pat in ignorable))
    wrong_shape: List[str] = []
    wrong_dtype: List[str] = []
    for n, s in expected.items():
        if n in have:
            if tuple(directory.shape(n)) != tuple(s.shape):
                wrong_shape.append(f"{n}: stored {list(directory.shape(n))}, model wants {list(s.shape)}")
            if directory.dtype(n) not in _FLOATS:
                wrong_dtype.append(f"{n}: {directory.dtype(n)}")
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)


def load_from_folder(model, model_dir: str, device: torch.device, dtype: torch.dtype) -> None:
    directory = TensorDirectory(model_dir)
    check_tensors(model.all_tensor_specs(), directory, model.all_ignorable_tensors())
    model.load_weights(directory.get, device, dtype)


def load_random(model, seed: int, device: torch.device, dtype: torch.dtype) -> None:
    """Weights equal to those :func:`write_random_model` stores for the same seed."""
    model.load_weights(RandomWeights(model.all_tensor_specs(), seed, device), device, dtype)


def write_random_model(config, out_dir: str, seed: int = 0, store_dtype: torch.dtype = torch.bfloat16,
                       architecture=None) -> str:
    """Write ``config.json`` and ``model.safetensors`` of a random model and return the folder.

    Matrices are stored in ``store_dtype``; norm weights are stored in float32.
    """
    from ..config.registry import resolve_architecture
    raw = config.to_json_dict()
    arch = architecture or resolve_architecture(raw)
    model = arch.build_model(config, config.max_position_embeddings)
    os.makedirs(out_dir, exist_ok=True)
    gen = RandomWeights(model.all_tensor_specs(), seed, torch.device("cpu"), store_dtype)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      ((s.name, gen(s.name)) for s in model.all_tensor_specs()))
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(raw, fh, indent=2)
    return out_dir
