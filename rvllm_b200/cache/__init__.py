from .manager import CacheManager, CacheView, Group, PageTable, RequestCache
from .pages import PagePool
