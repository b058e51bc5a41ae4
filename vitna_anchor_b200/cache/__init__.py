from .manager import CacheManager, KVSpec, LayerCacheView, StateSpec  # noqa: F401
from .pages import CacheError, OutOfPages, PageGroup, PagePool, PageTables, SlotPool, UNMAPPED  # noqa: F401
