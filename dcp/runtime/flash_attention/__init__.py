from dcp_b200.runtime.interface import (AttentionExecutor, DCPAttention, FusedPlanExecutor, get_executor, get_local_q_kv, prepare_dcp_distributed_attn_for_test)  # noqa: F401
