from dcp_b200.utils.logger import create_logger, logger, read_env_bool  # noqa: F401
