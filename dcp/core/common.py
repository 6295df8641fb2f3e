from dcp_b200.core.common import ExecutionContext, ModelSpec, get_default_execution_context  # noqa: F401
