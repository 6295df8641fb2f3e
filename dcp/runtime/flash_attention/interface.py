from dcp_b200.runtime.interface import *  # noqa: F401,F403
