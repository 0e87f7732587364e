from .pages import PagePool, SlotPool, PageError
from .manager import CacheManager, CacheGroup, RELEASED, group_key
