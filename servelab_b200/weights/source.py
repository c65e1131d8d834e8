"""Where tensors come from: a model folder of safetensors, or a seeded generator.

A model states the tensors it needs as ``TensorDecl`` records (full checkpoint
name, shape, role).  A ``WeightSource`` answers for names, shapes, stored dtypes
and data.  ``check_source`` compares the two and raises ONE ``WeightsError``
that lists every missing tensor, every unexpected tensor and every wrong shape.

Parity: the reference loads safetensors / .bin by the checkpoint's own names
(docs/architecture.md:70), skips ``rotary_emb.inv_freq`` (servelab/parallel/
tp_model.py:104), raises on missing tensors (tp_model.py:108-110) and only
prints unexpected ones (servelab/engine/engine.py:88-90); here unexpected
tensors are part of the error, because a silently ignored tensor is usually a
misnamed one.
"""

from __future__ import annotations

import json
import os
import zlib
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile

# roles decide the random distribution and the precision kept on the device
MATRIX = "matrix"     # GEMM operand or embedding table: N(0, std)
BIAS = "bias"         # additive vector: N(0, std); kept in float32
NORM = "norm"         # multiplicative norm weight: 1 + N(0, norm_std); kept in float32
TABLE = "table"       # integer table: kept as int32


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX


class WeightsError(RuntimeError):
    """The checkpoint does not match the model; lists all differences at once."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, tuple, tuple]]):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file {list(got)} != model {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


class WeightSource:
    where = "<source>"

    def names(self) -> List[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def stored_dtype(self, name: str) -> torch.dtype:
        raise NotImplementedError

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored, on the CPU (or already on a device)."""
        raise NotImplementedError


class _StateDictFile:
    """A ``pytorch_model.bin``: a state dict written by ``torch.save`` (the reference's tests
    write their tiny checkpoints so, tests/helpers_tiny_model.py:55).  Read with
    ``weights_only=True`` (tensors only, nothing is unpickled into code) and memory-mapped."""

    def __init__(self, path: str):
        try:
            self._tensors = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
        except (RuntimeError, ValueError):                 # (an archive written without mmap support)
            self._tensors = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(self._tensors, dict) or not all(
                isinstance(v, torch.Tensor) for v in self._tensors.values()):
            raise ValueError(f"{path}: not a state dict of tensors")

    def names(self):
        return list(self._tensors)

    def shape(self, name):
        return tuple(self._tensors[name].shape)

    def dtype(self, name):
        return self._tensors[name].dtype

    def read(self, name):
        return self._tensors[name]


class FolderSource(WeightSource):
    """``model.safetensors``, the shards named by ``model.safetensors.index.json``, or a
    ``pytorch_model.bin`` state dict (in that order)."""

    def __init__(self, folder: str):
        self.where = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._file_of: Dict[str, object] = {}
        if os.path.isfile(single):
            files = [SafetensorsFile(single)]
        elif os.path.isfile(index):
            with open(index) as f:
                shard_names = sorted(set(json.load(f)["weight_map"].values()))
            files = [SafetensorsFile(os.path.join(folder, s)) for s in shard_names]
        elif os.path.isfile(os.path.join(folder, "pytorch_model.bin")):
            files = [_StateDictFile(os.path.join(folder, "pytorch_model.bin"))]
        else:
            raise FileNotFoundError(
                f"model folder {folder!r} has neither model.safetensors, "
                f"model.safetensors.index.json nor pytorch_model.bin")
        for sf in files:
            for n in sf.names():
                self._file_of[n] = sf

    def names(self):
        return list(self._file_of)

    def shape(self, name):
        return self._file_of[name].shape(name)

    def stored_dtype(self, name):
        return self._file_of[name].dtype(name)

    def read(self, name):
        return self._file_of[name].read(name)


class RandomSource(WeightSource):
    """Seeded random tensors for a list of declarations.

    Each tensor has its own generator seeded by (seed, crc32(name)), so a tensor
    does not depend on which others are drawn or in what order.  Matrices and
    biases are N(0, std^2); norm weights 1 + N(0, norm_std^2).  On a CUDA
    device the draw uses the device generator (fast for billions of values; the
    values then differ from the CPU's for the same seed).
    """

    def __init__(self, decls: Iterable[TensorDecl], seed: int, std: float = 0.02,
                 norm_std: float = 0.1, device: str = "cpu",
                 dtype: torch.dtype = torch.float32, std_of: Optional[Dict[str, float]] = None):
        """``std_of``: standard deviations for tensors whose name contains a key (the first
        key that matches), e.g. {"q_proj.weight": 0.25} for queries large enough that the
        softmax of a tiny model is peaked."""
        self.decls = {d.name: d for d in decls}
        self.seed, self.std, self.norm_std = int(seed), std, norm_std
        self.std_of = dict(std_of or {})
        self.device, self.dtype = device, dtype
        self.where = f"<random weights, seed {seed}>"

    def names(self):
        return list(self.decls)

    def shape(self, name):
        return tuple(self.decls[name].shape)

    def stored_dtype(self, name):
        return torch.int32 if self.decls[name].role == TABLE else self.dtype

    def read(self, name):
        d = self.decls[name]
        gen = torch.Generator(device=self.device)
        gen.manual_seed((self.seed * 0x9E3779B1 + zlib.crc32(name.encode())) % (2 ** 63))
        if d.role == TABLE:
            return torch.zeros(d.shape, dtype=torch.int32, device=self.device)
        t = torch.randn(d.shape, generator=gen, device=self.device, dtype=torch.float32)
        if d.role == NORM:
            t.mul_(self.norm_std).add_(1.0)
        else:
            t.mul_(next((v for k, v in self.std_of.items() if k in name), self.std))
        return t.to(self.dtype)


def check_source(source: WeightSource, decls: Iterable[TensorDecl],
                 ignored_suffixes: Sequence[str] = (),
                 optional: Sequence[str] = ()) -> None:
    """Raise WeightsError unless the source holds exactly the declared tensors
    (plus ignorable ones) with the declared shapes."""
    want = {d.name: tuple(d.shape) for d in decls}
    have = set(source.names())
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(
        n for n in have
        if n not in want and n not in optional
        and not any(n.endswith(s) for s in ignored_suffixes))
    wrong = sorted((n, source.shape(n), want[n]) for n in want
                   if n in have and tuple(source.shape(n)) != want[n])
    if missing or unexpected or wrong:
        raise WeightsError(source.where, missing, unexpected, wrong)
