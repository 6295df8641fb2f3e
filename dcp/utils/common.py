from dcp_b200.utils.common import read_env_int, trepr  # noqa: F401
