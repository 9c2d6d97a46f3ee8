"""gaac_b200: B200 (sm_100a) implementation of the GAAC lossless compressed BF16 KV cache and its fused decode attention.

Same public names as the reference package `gaac` (gaac/__init__.py:2-8).
"""
from .codec import Codec, Page
from .encoder import TileEncoder
from .kernel import attention, choose_nsplit, choose_nsplit_sm100
from .kv_cache import CompressedKVCache
from .calibration import BaseCollector

__all__ = ["Codec", "Page", "TileEncoder", "attention", "choose_nsplit", "choose_nsplit_sm100", "CompressedKVCache", "BaseCollector"]
