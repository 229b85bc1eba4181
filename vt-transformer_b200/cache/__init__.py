from .manager import CacheManager, OutOfPages, OutOfRows, PagePool
