from dcp_b200.core.blocks import *  # noqa: F401,F403
from dcp_b200.core.blocks import (BlockManager, BlockMappings, BlockMeta, BlockType, ComputationBlockMeta, DataBlockMeta, WorkloadSpec, deserialize_list_of_workloads, serialize_list_of_workloads)  # noqa: F401
