from .pages import IdPool, OutOfPages
from .manager import NULL_PAGE, NULL_SLOT, CacheGroup, CacheManager, CacheView, RequestCache
