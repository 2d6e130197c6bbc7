"""Weights from safetensors by tensor name.

The model description says which tensors it reads (name, shape, precision); the loader finds them
in the folder's *.safetensors files, checks all of them, and only then copies them to the device.
A checkpoint that does not fit raises ONE `WeightError` that lists every missing tensor, every
unexpected tensor and every wrong shape, instead of stopping at the first (the reference stops at
the first: "missing weight: <name>", "shape mismatch for <name>", src/model.cpp:107-142).

Precision on the device: matrices that feed matrix products take the engine's dtype (bfloat16, or
float32 on the 32-bit path: a bf16/f16 file is widened exactly, src/model.cpp:14-40); vectors such
as norm weights are always float32; tensors asked for as "stored" keep the file's type, so a
32-bit tensor stays 32-bit and integer tables stay int32.
"""
from __future__ import annotations

from fnmatch import fnmatchcase
from typing import Dict, Iterable, List, Mapping, Sequence

import torch

from ..parts.spec import TensorNeed
from .safetensors_io import SafetensorsFile, list_safetensors

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


class WeightError(RuntimeError):
    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"checkpoint in {model_dir} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def merge_needs(needs: Iterable[TensorNeed]) -> Dict[str, TensorNeed]:
    """One need per name; two parts may read the same tensor (tied embeddings) if they agree."""
    out: Dict[str, TensorNeed] = {}
    for n in needs:
        prev = out.get(n.name)
        if prev is None:
            out[n.name] = n
        elif tuple(prev.shape) != tuple(n.shape) or prev.precision != n.precision:
            raise ValueError(f"two parts read '{n.name}' with different shape or precision: {prev} vs {n}")
    return out


class Checkpoint:
    """The *.safetensors files of a model folder as one name -> tensor map (memory-mapped)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files = [SafetensorsFile(p) for p in list_safetensors(model_dir)]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.names():
                self.where[name] = f

    def names(self) -> List[str]:
        return sorted(self.where)

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def shape(self, name: str):
        return self.where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self.where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)


def load_tensors(ckpt: Checkpoint, needs: Mapping[str, TensorNeed], duplicates: Mapping[str, str],
                 device: torch.device, compute_dtype: torch.dtype, ignore: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """ignore: shell-style patterns of names the checkpoint may carry unread (ModelSpec.ignore)."""
    missing, unexpected, wrong = [], [], []
    for name, need in sorted(needs.items()):
        if name not in ckpt:
            missing.append(name)
            continue
        if tuple(ckpt.shape(name)) != tuple(need.shape):
            wrong.append(f"{name}: expected {list(need.shape)}, got {list(ckpt.shape(name))}")
        elif need.precision in ("compute", "float32") and ckpt.dtype(name) not in _FLOATS:
            wrong.append(f"{name}: expected a floating-point tensor, got {ckpt.dtype(name)}")
    for name in ckpt.names():
        if name in needs:
            continue
        twin = duplicates.get(name)
        if twin is None:
            if not any(fnmatchcase(name, pat) for pat in ignore):
                unexpected.append(name)
        elif twin in ckpt and (tuple(ckpt.shape(name)) != tuple(ckpt.shape(twin)) or ckpt.dtype(name) != ckpt.dtype(twin)):
            # a tied output embedding saved beside the input embedding must agree with it
            # (src/weights.cpp:259-264)
            wrong.append(f"{name}: tied to {twin} but shape/dtype disagree "
                         f"({list(ckpt.shape(name))} {ckpt.dtype(name)} vs {list(ckpt.shape(twin))} {ckpt.dtype(twin)})")
    if missing or unexpected or wrong:
        raise WeightError(ckpt.model_dir, missing, unexpected, wrong)

    out: Dict[str, torch.Tensor] = {}
    for name, need in needs.items():
        t = ckpt.tensor(name)
        if need.precision == "compute":
            target = compute_dtype
        elif need.precision == "float32":
            target = torch.float32
        elif need.precision == "stored":
            target = t.dtype
        else:
            raise ValueError(f"tensor need '{name}': unknown precision '{need.precision}'")
        out[name] = t.to(device=device, dtype=target, copy=True).contiguous()
    return out
