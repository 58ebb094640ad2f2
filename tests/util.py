"""Shared helpers of the GPU parity tests: seeded inputs, bf16 bit patterns, the normalised error metric."""
import numpy as np
import torch

import oracle as mo


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 CUDA tensor -> uint16 bit patterns on the host (what the oracle's bf16 entry points take)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f64(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float64).cpu().numpy()


def randn(shape, seed, std=1.0, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype).cuda()


def uniform(shape, seed, lo=-1.0, hi=1.0, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.rand(shape, generator=g, dtype=torch.float32) * (hi - lo) + lo).to(dtype).cuda()


def nerr(got, want) -> float:
    """max|got - want| / max|want| -- the metric the tolerances (1e-5 f32, 2e-2 bf16) are stated in."""
    return mo.normalised_error(got, want)


TOL_F32 = 1e-5
TOL_BF16 = 2e-2
