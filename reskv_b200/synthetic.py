"""Seeded synthetic K/V with the statistics the compression is designed for.

Stand-in for activations of a real model (no checkpoints or datasets are needed):
per (sequence, KV head) a mixture of ``clusters`` Gaussian clusters -- centres
~ N(0,1), within-cluster sigma 0.3 -- multiplied by per-channel scales drawn
log-normal(0, 1), which creates the outlier channels real keys show.
"""

from __future__ import annotations

import torch


def mixture(batch: int, heads: int, tokens: int, *, seed: int, device="cpu", clusters: int = 32, sigma: float = 0.3,
            dtype=torch.float16, chunk: int = 8192) -> torch.Tensor:
    """``[batch, heads, tokens, 128]`` tensor of the cluster mixture.

    The generator lives on ``device``; CPU-generated tensors are what the parity
    tests use (device generators differ between GPUs), the benchmark generates
    on the GPU.  Tokens are produced in chunks to bound temporary memory.
    """
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    centres = torch.randn(batch, heads, clusters, 128, generator=gen, device=device)
    scales = torch.randn(batch, heads, 1, 128, generator=gen, device=device).exp()
    out = torch.empty(batch, heads, tokens, 128, dtype=dtype, device=device)
    for t0 in range(0, tokens, chunk):
        n = min(chunk, tokens - t0)
        which = torch.randint(clusters, (batch, heads, n), generator=gen, device=device)
        x = torch.gather(centres, 2, which.unsqueeze(-1).expand(-1, -1, -1, 128))
        x = x + sigma * torch.randn(batch, heads, n, 128, generator=gen, device=device)
        out[:, :, t0:t0 + n] = (x * scales).to(dtype)
    return out


def gaussian(*shape, seed: int, device="cpu", dtype=torch.float16, std: float = 1.0) -> torch.Tensor:
    """N(0, std^2) tensor from a seeded generator on ``device``."""
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(*shape, generator=gen, device=device) * std).to(dtype)
