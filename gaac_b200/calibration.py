"""Offline calibration of the exponent bases (drop-in for gaac/calibration.py).

Run a model over representative prompts, hand every layer's prefill K and V to `BaseCollector.observe`, and `bases()` returns
per layer the start of the densest 8-wide and 16-wide exponent window of every (kv head, channel): the tables the encoder
codes exponents against.  `save` writes them as {layer: {'k3', 'k4', 'v3', 'v4'}} of uint8 [n_kv, 128] CPU tensors with
torch.save, the file the reference's engine loads (nanovllm/engine/model_runner.py:135).  The histograms are built on the GPU
(gaac_exponent_hist) and only summed here.
"""
from __future__ import annotations
import torch
from .codec import bases_from_hist, exponent_hist


class _LayerCounts:
    """Running exponent histograms of one layer: int64 [n_kv*128, 256] for K and for V."""
    __slots__ = ("n_kv", "k", "v")

    def __init__(self, n_kv: int):
        self.n_kv, self.k, self.v = n_kv, None, None

    def add(self, k: torch.Tensor, v: torch.Tensor):
        hk, hv = exponent_hist(k, self.n_kv), exponent_hist(v, self.n_kv)
        self.k = hk if self.k is None else self.k + hk
        self.v = hv if self.v is None else self.v + hv


class BaseCollector:
    """Accumulates exponent statistics layer by layer (gaac/calibration.py:13-32)."""

    def __init__(self):
        self.hist: dict[int, _LayerCounts] = {}

    def observe(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        """k, v: [N, n_kv, 128] bf16, the keys and values of N prompt tokens of `layer`."""
        if layer not in self.hist:
            self.hist[layer] = _LayerCounts(k.shape[1])
        self.hist[layer].add(k, v)

    def bases(self) -> dict:
        tables = {}
        for layer in sorted(self.hist):
            c = self.hist[layer]
            (k3, k4), (v3, v4) = bases_from_hist(c.k, c.n_kv), bases_from_hist(c.v, c.n_kv)
            tables[layer] = {"k3": k3.cpu(), "k4": k4.cpu(), "v3": v3.cpu(), "v4": v4.cpu()}
        return tables

    def save(self, path: str) -> int:
        """Write the tables with torch.save; returns the number of layers written."""
        tables = self.bases()
        torch.save(tables, path)
        return len(tables)
