"""Drop-in name of the reference package (flashbev/flashbevpool/__init__.py:3-6): the same three
exports, served by the B200 implementation in ``flashbev_b200``."""
from flashbev_b200 import FlashBEVPool, SamplingVT, flash_bevpool

__all__ = ["FlashBEVPool", "flash_bevpool", "SamplingVT"]
