"""Structured rotations.

The operator API takes a dense fp16 `[heads, D, D]` rotation (reference:
plugins/residual_quantization/csrc/common/api.h:42-55).  When that matrix is `diag(+-1) @ H_D * c` -- the
shape every Hadamard-initialised rotation of the benchmark configurations has
(scripts/calibration/rotation_math.py:6-32) -- the kernels never need the matrix: they take the sign of every
channel as a bit mask and run a fast Walsh-Hadamard transform in registers.  `register_rotation` inspects a
matrix ONCE (at model-install time, on the host) and remembers the masks under the tensor's data pointer, so
the per-call path is a dictionary lookup.
"""

from __future__ import annotations

import weakref
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch


def paley12() -> np.ndarray:
    residues = {i * i % 11 for i in range(1, 11)}
    m = np.ones((12, 12), dtype=np.float32)
    for i in range(11):
        for j in range(11):
            m[i + 1, j + 1] = -1 if i == j else (1 if (i - j) % 11 in residues else -1)
    return m


def hadamard_unnormalized(dim: int) -> np.ndarray:
    """+-1 matrix H_D: Sylvester for powers of two, Paley-12 (x) Sylvester-8 for 96."""
    def sylvester(n):
        m = np.ones((1, 1), dtype=np.float32)
        while m.shape[0] < n:
            m = np.block([[m, m], [m, -m]])
        return m
    if dim == 96:
        return np.kron(paley12(), sylvester(8)).astype(np.float32)
    if dim <= 0 or dim & (dim - 1):
        raise ValueError("Hadamard dimension must be a power of two or 96")
    return sylvester(dim)


@dataclass
class SignedHadamardRotation:
    """Device-side description of R[h] = diag(sign[h]) @ H_D * scale."""

    sign_masks: torch.Tensor  # int32 [heads, D/32] on the rotation's device; bit set = -1
    scale: float
    heads: int
    head_dim: int

    def dense(self, dtype=torch.float16) -> torch.Tensor:
        h = torch.from_numpy(hadamard_unnormalized(self.head_dim))
        bits = self.sign_masks.cpu().numpy().view(np.uint32)
        signs = np.ones((self.heads, self.head_dim), dtype=np.float32)
        for c in range(self.head_dim):
            signs[:, c] = 1.0 - 2.0 * ((bits[:, c // 32] >> (c % 32)) & 1)
        return (torch.from_numpy(signs)[:, :, None] * h[None] * self.scale).to(dtype).to(self.sign_masks.device)


def pack_signs(signs: np.ndarray) -> np.ndarray:
    """[heads, D] of +-1 -> uint32 [heads, D/32], bit c%32 of word c//32 set when sign is -1."""
    heads, dim = signs.shape
    bits = (np.asarray(signs) < 0).astype(np.uint64).reshape(heads, dim // 32, 32)
    words = (bits << np.arange(32, dtype=np.uint64)[None, None]).sum(-1)
    return words.astype(np.uint32)


def signed_hadamard(signs: np.ndarray, scale: float, device) -> SignedHadamardRotation:
    masks = torch.from_numpy(pack_signs(signs).view(np.int32)).to(device)
    return SignedHadamardRotation(masks, float(scale), signs.shape[0], signs.shape[1])


def analyze(rotation: torch.Tensor) -> Optional[Tuple[np.ndarray, float]]:
    """(signs [heads, D], scale) if `rotation` is exactly diag(+-1) @ H_D * scale, else None."""
    if rotation.dim() != 3 or rotation.shape[1] != rotation.shape[2]:
        return None
    dim = rotation.shape[1]
    if dim != 96 and (dim & (dim - 1)):
        return None
    dense = rotation.detach().float().cpu().numpy()
    scale = float(np.abs(dense[0, 0, 0]))
    if scale <= 0 or not np.all(np.abs(dense) == np.float32(scale)):
        return None
    h = hadamard_unnormalized(dim)
    signs = np.sign(dense[:, :, 0] * h[None, :, 0])           # row sign = entry of column 0 (H[:, 0] == +1)
    if not np.array_equal(np.sign(dense), signs[:, :, None] * h[None]):
        return None
    return signs.astype(np.int8), scale


# key -> (structure, weak reference to the registered tensor, its version counter at registration)
_registry: Dict[Tuple[int, int, Tuple[int, ...]], Tuple[SignedHadamardRotation, "weakref.ref", int]] = {}


def _key(rotation: torch.Tensor):
    return (rotation.data_ptr(), rotation.device.index or 0, tuple(rotation.shape))


def register_rotation(rotation: torch.Tensor) -> Optional[SignedHadamardRotation]:
    """Inspect a dense fp16 rotation once; remember its structure when it is a signed Hadamard matrix.
    The entry is tied to this very tensor object: it is dropped when the tensor dies or is modified in place, so a
    different matrix that later lands at the same address is never mistaken for it."""
    found = analyze(rotation)
    if found is None:
        return None
    signs, scale = found
    structured = signed_hadamard(signs, scale, rotation.device)
    key = _key(rotation)
    _registry[key] = (structured, weakref.ref(rotation), rotation._version)
    weakref.finalize(rotation, _drop_if_dead, key)
    return structured


def _drop_if_dead(key) -> None:
    entry = _registry.get(key)
    if entry is not None and entry[1]() is None:
        del _registry[key]


def lookup(rotation: torch.Tensor) -> Optional[SignedHadamardRotation]:
    key = _key(rotation)
    entry = _registry.get(key)
    if entry is None:
        return None
    structured, owner, version = entry
    alive = owner()
    # While the registered tensor lives, nothing else can be allocated at its address: any tensor that matches the key
    # is that tensor or a view of it.  Its version counter moves with every in-place write.
    if alive is None or alive._version != version:
        del _registry[key]
        return None
    return structured


def forget(rotation: torch.Tensor) -> None:
    _registry.pop(_key(rotation), None)
