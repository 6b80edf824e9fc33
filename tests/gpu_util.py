"""Helpers shared by the GPU tests: one context per process, weights from numpy bytes."""
import numpy as np
import torch

_ctx = None


def ctx():
    global _ctx
    if _ctx is None:
        from zllm_b200.backend import B200Context

        _ctx = B200Context(0)
    return _ctx


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    ctx().sync()
    return t.float().cpu().numpy() if t.dtype != torch.float32 else t.cpu().numpy()
