"""Helpers for the GPU parity tests: device buffers are plain byte tensors whose
addresses go through the C ABI; torch is only the allocator."""
from __future__ import annotations

import numpy as np
import torch


def to_device(array: np.ndarray) -> torch.Tensor:
    flat = np.ascontiguousarray(array).reshape(-1).view(np.uint8)
    return torch.from_numpy(flat.copy()).cuda()


def device_zeros(nbytes: int, fill: int = 0) -> torch.Tensor:
    return torch.full((max(nbytes, 1),), fill, dtype=torch.uint8, device="cuda")


def to_host(buffer: torch.Tensor, dtype, shape=None) -> np.ndarray:
    torch.cuda.synchronize()
    out = buffer.cpu().numpy().view(dtype)
    return out.reshape(shape) if shape is not None else out


def ptr(buffer) -> int:
    return 0 if buffer is None else buffer.data_ptr()
