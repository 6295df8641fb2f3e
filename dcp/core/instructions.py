from dcp_b200.core.instructions import *  # noqa: F401,F403
from dcp_b200.core.instructions import (BlockInstrBase, deserialize_list_of_execution_plans, serialize_list_of_execution_plans)  # noqa: F401
