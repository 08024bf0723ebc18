from .pages import CacheError, FreeList
from .requests import KVRequest, StateRequest
from .sequence_cache import SequenceCache, KVGroup, KVView, StateView, PAGE, pages_for
