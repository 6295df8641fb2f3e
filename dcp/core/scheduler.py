from dcp_b200.planner.scheduler import convert_forward_to_backward, schedule  # noqa: F401
