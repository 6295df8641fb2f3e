from dcp_b200.data.dataloader import (DCPDataLoader, ExecutionPlanner, KVStoreMetaKeys, TrainingSpec, generate_workload)  # noqa: F401
from dcp_b200.planner.workload import block_size_heuristic as _block_size_heuristic  # noqa: F401
from dcp_b200.planner.workload import generate_workload as _generate_workload  # noqa: F401
