from dcp_b200.memory.allocation_simulator import AllocationSimulator, TorchCachingAllocatorSimulator  # noqa: F401
