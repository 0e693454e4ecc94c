"""Helpers of the GPU parity tests: numpy bit patterns <-> device buffers."""
import numpy as np
import torch

from oracle import oracle as orc  # the checker


def dev(a):
    """numpy array -> CUDA tensor with the same bytes (unsigned types travel as signed views)."""
    a = np.ascontiguousarray(a)
    view = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32, np.dtype(np.uint64): np.int64}.get(a.dtype)
    return torch.from_numpy(a.view(view) if view else a).cuda()


def host(t, dtype):
    """CUDA tensor -> numpy array reinterpreted as dtype."""
    return t.detach().cpu().contiguous().numpy().view(dtype).reshape(-1)


def u16(t):
    return host(t, np.uint16)


def rand_bf16(rs, n, scale=1.0):
    return orc.f32_to_bf16((rs.standard_normal(n) * scale).astype(np.float32))


def norm_err(x, y):
    x, y = np.asarray(x, np.float64), np.asarray(y, np.float64)
    return float(np.sqrt(((x - y) ** 2).sum() / max((y ** 2).sum(), 1e-300))), float(np.abs(x - y).max() / max(np.abs(y).max(), 1e-300))
