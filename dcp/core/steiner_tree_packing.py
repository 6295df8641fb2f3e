from dcp_b200.planner.steiner import pack_multicast_trees  # noqa: F401
