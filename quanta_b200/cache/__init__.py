"""Paged cache bookkeeping: pages, block tables, state slots."""
from .manager import CacheManager, OutOfPages, OutOfSlots, PagePool, SlotPool  # noqa: F401
