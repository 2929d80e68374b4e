"""DLSlimeCache: a slab directory plus registered memory that peers fill and read with one-sided I/O."""

from .._slime_c import Assignment
from .._slime_c import cache as ccache
from .._slime_c.cache import AssignmentManifest, CacheStats
from .._slime_c.cache import CacheServer as CacheDirectory
from .client import CacheClient, discover_cache_url, get_json, post_json
from .service import CacheHttpServer, CacheServer, CacheService, NanoCtrlRegistration, resolve_host_for_registration
from .types import (DEFAULT_AGENT_ALIAS, DEFAULT_CACHE_MR_NAME, DEFAULT_MEMORY_SIZE, DEFAULT_SERVICE_ID, DEFAULT_SLAB_SIZE,
                    assignment_from_json, assignment_to_json, assignment_to_tuple, manifest_to_json, stats_to_json)

__all__ = ["Assignment", "AssignmentManifest", "CacheStats", "CacheDirectory", "CacheClient", "CacheService", "CacheHttpServer",
           "CacheServer", "NanoCtrlRegistration", "discover_cache_url", "post_json", "get_json", "assignment_to_json",
           "assignment_from_json", "manifest_to_json", "stats_to_json", "DEFAULT_SLAB_SIZE", "DEFAULT_MEMORY_SIZE",
           "DEFAULT_CACHE_MR_NAME", "DEFAULT_SERVICE_ID", "DEFAULT_AGENT_ALIAS", "assignment_to_tuple", "ccache",
           "resolve_host_for_registration"]
