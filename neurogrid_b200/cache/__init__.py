from .manager import CacheManager, PagedNeed, SlotNeed
from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool
