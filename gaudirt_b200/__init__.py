"""B200-native paged KV-store / paged-attention path behind the GaudiRT operator surface."""
from . import abi  # noqa: F401

__all__ = ["abi"]
