from .manager import (
    CacheError,
    CacheGroup,
    CacheManager,
    LayerMemory,
    OutOfPages,
    PagePool,
    RequestCache,
    StepMemories,
)

__all__ = [
    "CacheError",
    "CacheGroup",
    "CacheManager",
    "LayerMemory",
    "OutOfPages",
    "PagePool",
    "RequestCache",
    "StepMemories",
]
