from dcp_b200.core.executor import DCPExecutor  # noqa: F401
