from .need import CacheNeed
from .pages import CacheFull, FreeList, PageBook
from .kv import TOKENS_PER_PAGE, EntryView, LayerKV, SequenceCache

__all__ = ["CacheNeed", "CacheFull", "FreeList", "PageBook", "TOKENS_PER_PAGE", "EntryView", "LayerKV",
           "SequenceCache"]
