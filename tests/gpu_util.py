"""Helpers for the GPU parity tests: host numpy storage <-> device tensors."""
from __future__ import annotations

import numpy as np
import torch

from rocwmma_b200.synth import BF16, E4M3


def to_device(arr: np.ndarray, dtype_code: int) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dtype_code == BF16:
        t = t.view(torch.int16)
    t = t.cuda()
    if dtype_code == BF16:
        t = t.view(torch.bfloat16)
    return t


def to_host(t: torch.Tensor, dtype_code: int) -> np.ndarray:
    if dtype_code == BF16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).cpu().numpy()
    return t.cpu().numpy()
