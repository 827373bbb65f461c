from .manager import NULL_PAGE, CacheError, CacheManager, GroupSpec, PagePool

__all__ = ["NULL_PAGE", "CacheError", "CacheManager", "GroupSpec", "PagePool"]
