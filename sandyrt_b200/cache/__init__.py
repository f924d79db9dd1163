from .pages import (FREED, BlockAllocator, CacheError, CacheLayout, NoFreeSlot, OutOfPages,  # noqa: F401
                    PagePool)
