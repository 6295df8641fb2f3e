from dcp_b200.runtime.interface import AttentionExecutor, DCPAttention, get_executor  # noqa: F401
