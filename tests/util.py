"""Helpers shared by the tests: fixture loading and bf16 <-> bit-pattern conversion."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16)


def bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().cpu().view(torch.int16)


def same_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.equal(bits(a), bits(b)))
