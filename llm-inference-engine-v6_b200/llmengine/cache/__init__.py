"""Cache manager: pages with a block table per request, groups of layers with different needs,
slots for per-request state of fixed size."""
from .host import host_module
from .storage import CacheGroup, allocate_run_caches, bytes_per_token, plan_groups

__all__ = ["host_module", "CacheGroup", "allocate_run_caches", "bytes_per_token", "plan_groups"]
