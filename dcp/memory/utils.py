from dcp_b200.memory.utils import reserve_full_memory  # noqa: F401
