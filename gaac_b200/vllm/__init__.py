"""Paged layout used by the vLLM backend: LayerState (store side) and paged_attention (decode side)."""
