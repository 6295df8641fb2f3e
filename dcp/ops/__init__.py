from dcp_b200.ops.block_ops import (flash_attn_update_out_lse, fused_blockwise_sum, fused_copy_bf16, fused_copy_fp16, fused_copy_fp32, warmup_triton_ops)  # noqa: F401
