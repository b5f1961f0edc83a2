from .manager import CacheManager, CacheView, Group, RequestCache
from .pages import PagePool
