"""The cache manager: pages and block tables per group, state slots per request."""

from .manager import CacheManager, NoFreeSlot, OutOfPages, Reservation
from .spec import CacheBinding, CacheGroupSpec

__all__ = ["CacheManager", "OutOfPages", "NoFreeSlot", "Reservation", "CacheBinding", "CacheGroupSpec"]
