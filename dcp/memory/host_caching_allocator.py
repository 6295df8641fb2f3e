from dcp_b200.memory.host_caching_allocator import HostCachingAllocator, apply_monkey_patch  # noqa: F401
