"""Zero-copy torch views of device buffers owned by the C library (torch is plumbing: memory and streams)."""
from __future__ import annotations

import numpy as np
import torch

from . import capi

_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.bfloat16: "<u2", torch.int32: "<i4"}


class _Span:
    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"data": (int(ptr), False), "shape": tuple(shape), "typestr": typestr,
                                         "version": 3, "strides": None}


def view(ptr: int, shape, dtype: torch.dtype, device: int = 0) -> torch.Tensor:
    """Tensor aliasing `ptr` (no ownership: the handle must outlive the view)."""
    t = torch.as_tensor(_Span(ptr, shape, _TYPESTR[dtype]), device=f"cuda:{device}")
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


def state_view(h: "capi.Handle") -> torch.Tensor:
    """[B][rows incl. halo][W][64] view of the stored (un-normalised) state."""
    ptr, _ = h.buffer(capi.BUF_STATE)
    rows = h.cfg.height + (6 if h.cfg.stripe else 0)
    dt = torch.bfloat16 if h.cfg.dtype == capi.BF16 else torch.float32
    return view(ptr, (h.cfg.batch, rows, h.cfg.width, 64), dt, h.cfg.device)


def sums_view(h: "capi.Handle") -> torch.Tensor:
    ptr, _ = h.buffer(capi.BUF_SUMS)
    return view(ptr, (h.cfg.batch, 64), torch.float64, h.cfg.device)


def vprime(h: "capi.Handle", which: int) -> np.ndarray:
    """V' of the last (capi.BUF_VPRIME_LAST) or previous step as host fp32 [B][H][W][512] (index h*64+d)."""
    ptr, n = h.buffer(which)
    if not ptr or not n:
        raise RuntimeError("handle keeps no V' (create it with keep_vprime=True)")
    dt = torch.bfloat16 if h.cfg.dtype == capi.BF16 else torch.float32
    B, H, W = h.cfg.batch, h.cfg.height, h.cfg.width
    t = view(ptr, (B, 8, H, W, 64), dt, h.cfg.device)
    return t.float().permute(0, 2, 3, 1, 4).reshape(B, H, W, 512).cpu().numpy()
