"""Error metrics used by every parity test (test infrastructure only)."""
from __future__ import annotations

import torch


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    if a.numel() == 0:
        return 0.0
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_2 / ||b||_2 with b the trusted value."""
    if a.numel() == 0:
        return 0.0
    a = a.double().cpu()
    b = b.double().cpu()
    den = b.norm().item()
    return (a - b).norm().item() / max(den, 1e-30)


def bf16_floor(ref: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> float:
    """rel-L2 error that pure output rounding to `dtype` introduces on `ref`.

    A 16-bit kernel cannot beat this number; tests compare against a small
    multiple of it next to the absolute tolerance.
    """
    return rel_l2(ref.to(dtype).float(), ref)
