from .manager import (CacheError, CacheLayout, CacheManager, OutOfPages, OutOfSlots, PageGroup,  # noqa: F401
                      cache_key, layout_of)
