"""Worker of test_interpreter_tensor_times_context_parallel (torch.distributed.run, 4 gloo ranks):
tensor parallelism 2 (heads and FFN channels split, adjacent ranks) x context parallelism 2 on the plan
interpreter against the unsplit fp32 model: loss, the gradients of every shard (= the matching slices
of the unsplit gradients) and identical replicated parameters after an optimizer step."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.data import synth  # noqa: E402
from dcp_b200.models.llama import LlamaConfig  # noqa: E402
from dcp_b200.models.reference import reference_loss  # noqa: E402
from dcp_b200.train_interp import InterpreterEngine, init_params, shard_params  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.set_num_threads(1)
    tp, n_cp = 2, world // 2
    t, c = rank % tp, rank // tp
    tp_groups = [dist.new_group([k * tp + j for j in range(tp)]) for k in range(n_cp)]
    cp_groups = [dist.new_group([k * tp + j for k in range(n_cp)]) for j in range(tp)]
    cfg = LlamaConfig(2, 64, 4, 2, 16, 96, 101)
    eng = InterpreterEngine(cfg, 1500, block_size=128, group=cp_groups[t], seed=7, lr=1e-2, tp_group=tp_groups[c])
    assert eng.cfg.n_heads == 2 and eng.cfg.n_kv_heads == 1 and eng.cfg.ffn == 48 and eng.spec.n_heads == 2
    plan = eng.plan()
    loss = eng.loss_and_grads(plan)
    ref_p = init_params(cfg, 7)
    seed = eng.spec.seed * 1000003
    seqlens = synth.sample_seqlens(eng.spec.tokens_per_step, eng.spec.length_dist, seed)
    batch = synth.make_token_batch(seqlens, cfg.vocab, seed)
    ref = reference_loss(cfg, ref_p, torch.from_numpy(batch["tokens"]), torch.from_numpy(batch["labels"]),
                         torch.from_numpy(batch["positions"]), seqlens, 1.0 / sum(seqlens))
    ref.backward()
    ok = abs(loss - ref.item()) < 1e-5 * abs(ref.item())
    ref_shard = shard_params(cfg, {k: v.grad for k, v in ref_p.items()}, tp, t)
    for name, r in ref_shard.items():
        g = eng.p[name].grad
        err = (g - r).abs().max().item() / (r.abs().max().item() + 1e-12)
        if g.shape != r.shape or err > 2e-4:
            print(f"rank {rank} {name}: relative gradient error {err}", flush=True)
            ok = False
    torch.nn.utils.clip_grad_norm_(list(eng.p.values()), 1e9)
    eng.opt.step()
    both = [torch.empty_like(eng.p["norm_f"]) for _ in range(tp)]
    dist.all_gather(both, eng.p["norm_f"].detach(), group=tp_groups[c])
    ok &= torch.allclose(both[0], both[1], atol=1e-7)          # replicated parameters stay together
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("INTERP_TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
