from .page_pool import PagePool, PagePoolError
from .state_slots import StateSlotPool
from .manager import CacheHolder, CacheManager, GroupSpec, compute_hash
