"""Worker of test_gloo_world2_reference_config (launched by torch.distributed.run, backend gloo)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.core.common import get_default_execution_context  # noqa: E402
from dcp_b200.core.instructions import BufferType  # noqa: E402
from dcp_b200.planner.compiler import InstrCompiler  # noqa: E402
from dcp_b200.planner.workload import generate_workload, pad_seqlens  # noqa: E402
from dcp_b200.runtime.comm import TorchDistComm  # noqa: E402
from dcp_b200.runtime.executor_ref import ReferenceAttentionExecutor  # noqa: E402
from dcp_b200.runtime.layout import gather_local, scatter_to_global  # noqa: E402
from dcp_b200.runtime.simulate import dense_reference  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    torch.set_num_threads(2)
    raw, bs, H, Hkv, d = [512, 1024, 2048, 4096], 256, 8, 2, 64
    ctx = get_default_execution_context(world, 1)
    pad = pad_seqlens(raw, bs)
    wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, 4, ctx.comp_cost_model, None,
                           torch.float32)
    fw_wl, bw_wl, fw, bw = InstrCompiler(ctx).compile(wl)      # deterministic: both ranks get the same plans
    T = sum(raw)
    q, kv, dout = torch.randn(T, H, d), torch.randn(T, 2, Hkv, d), torch.randn(T, H, d)
    dev = (0, rank)
    ex = ReferenceAttentionExecutor(TorchDistComm(), fw_wl, dev, world, 1)
    lay = ex.layout
    lo, ll = ex.forward(fw[dev], gather_local(q, lay, BufferType.LOCAL_Q, raw, 1),
                        gather_local(kv, lay, BufferType.LOCAL_KV, raw, 2))
    ldq, ldkv = ex.backward(bw[dev], bw_wl, gather_local(dout, lay, BufferType.LOCAL_OUT, raw, 1))
    out_g, lse_g = torch.zeros_like(q), torch.zeros(H, T)
    dq_g, dkv_g = torch.zeros_like(q), torch.zeros_like(kv)
    scatter_to_global(lo, out_g, lay, BufferType.LOCAL_OUT, raw, 1)
    scatter_to_global(ll, lse_g, lay, BufferType.LOCAL_LSE, raw, 0, token_axis_local=1)
    scatter_to_global(ldq, dq_g, ex.layout, BufferType.LOCAL_dQ, raw, 1)
    scatter_to_global(ldkv, dkv_g, ex.layout, BufferType.LOCAL_dKV, raw, 2)
    for t in (out_g, lse_g, dq_g, dkv_g):
        dist.all_reduce(t)
    if rank == 0:
        ro, rl, rdq, rdkv = dense_reference(q, kv, raw, pad, None, d ** -0.5, dout)
        errs = [(out_g - ro).abs().max().item(), (lse_g - rl).abs().max().item(), (dq_g - rdq).abs().max().item(),
                (dkv_g - rdkv).abs().max().item()]
        print("errors out/lse/dq/dkv", errs)
        assert max(errs) < 1e-5, errs
        print("GLOO_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
