from dcp_b200.ops.block_ops import *  # noqa: F401,F403
