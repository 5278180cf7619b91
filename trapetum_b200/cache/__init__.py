from .slots import CacheError, CacheFull, Pool
from .kv import Cache, KVGroup, KVLineView, StateView, pages_for

__all__ = ["Cache", "CacheError", "CacheFull", "KVGroup", "KVLineView", "Pool", "StateView", "pages_for"]
