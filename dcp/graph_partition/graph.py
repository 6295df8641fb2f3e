from dcp_b200.planner.partition import (HGPSolver, PlacementGraph, assign_device_by_heuristic, assign_input_outputs, construct_and_partition_graph_multiconstraint)  # noqa: F401
