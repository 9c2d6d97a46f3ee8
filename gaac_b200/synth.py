"""Seeded synthetic KV with the shapes and value distribution of the benchmark configurations, generated on the GPU.

x[h, t, d] = N(0,1) * s[h, d], s = exp(N(0, 1.0)) for K and exp(N(0, 0.5)) for V, rounded to BF16.  Per (head, token, stored
group of 8 positions): with probability 0.2 % one element is multiplied by 2^7 (forces the raw tier), with probability 10 %
one element by 2^4 (forces the 4-bit window).  Real-model KV is not available offline; this stands in for it.
"""
from __future__ import annotations
import torch
from .codec import perm, D


def synth_kv(kind: str, H: int, S: int, seed: int, device="cuda", raw_frac: float = 0.002, four_frac: float = 0.10, chunk: int = 16384) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed * 2 + (0 if kind == "k" else 1))
    sd = 1.0 if kind == "k" else 0.5
    s = torch.exp(torch.randn(H, 1, D, generator=g, device=device) * sd)
    p = perm(kind).to(device)
    inv = torch.empty_like(p); inv[p] = torch.arange(D, device=device)
    out = torch.empty(H, S, D, dtype=torch.bfloat16, device=device)
    for t0 in range(0, S, chunk):
        n = min(chunk, S - t0)
        x = torch.randn(H, n, D, generator=g, device=device) * s
        xs = x[..., p].view(H, n, 16, 8)
        u = torch.rand(H, n, 16, generator=g, device=device)
        pos = torch.randint(0, 8, (H, n, 16), generator=g, device=device)
        mult = torch.where(u < raw_frac, 128.0, torch.where(u < raw_frac + four_frac, 16.0, 1.0))
        onehot = pos.unsqueeze(-1) == torch.arange(8, device=device)
        xs = torch.where(onehot, xs * mult.unsqueeze(-1), xs)
        out[:, t0:t0 + n] = xs.reshape(H, n, D)[..., inv].to(torch.bfloat16)
    return out
