"""Worker of test_interpreter_training_matches_unsplit_model (torch.distributed.run, backend gloo):
a DCP training step on the plan interpreter over N ranks against the unsplit fp32 model on the whole
batch: same loss, same summed gradients, and after three optimizer steps the same parameters."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.data import synth  # noqa: E402
from dcp_b200.models.llama import LlamaConfig  # noqa: E402
from dcp_b200.models.reference import reference_loss, sequence_masks  # noqa: E402
from dcp_b200.planner import masks  # noqa: E402
from dcp_b200.planner.workload import pad_seqlens  # noqa: E402
from dcp_b200.train_interp import InterpreterEngine, init_params  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.set_num_threads(2)
    mask = sys.argv[1] if len(sys.argv) > 1 else "causal"
    dcp_size = int(sys.argv[2]) if len(sys.argv) > 2 else world          # < world: CP x DP
    cfg = LlamaConfig(2, 64, 4, 2, 16, 96, 101)
    group = dist.group.WORLD
    if dcp_size < world:
        groups = [dist.new_group(list(range(g * dcp_size, (g + 1) * dcp_size))) for g in range(world // dcp_size)]
        group = groups[rank // dcp_size]
    eng = InterpreterEngine(cfg, 1500, block_size=128, mask=mask, group=group, seed=3, lr=1e-2,
                            replica_group=dist.group.WORLD)
    ref_p = init_params(cfg, 3)
    ref_opt = torch.optim.AdamW(list(ref_p.values()), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    ok = True
    for it in range(3):
        plan = eng.plan()
        assert plan.tokens.numel() > 0 and plan.n_global_tokens > plan.tokens.numel()   # the batch really is split
        loss = eng.loss_and_grads(plan)
        # the unsplit model on the whole batch (every rank computes it: same seeds)
        seed = eng.spec.seed * 1000003 + it
        n_groups = world // dcp_size
        if n_groups > 1:        # every context-parallel group draws its own sub-batch; the job's batch is their union
            seqlens = [n for g in range(n_groups)
                       for n in synth.sample_seqlens(eng.spec.tokens_per_step // n_groups, eng.spec.length_dist, seed * 64 + g + 1)]
        else:
            seqlens = synth.sample_seqlens(eng.spec.tokens_per_step, eng.spec.length_dist, seed)
        batch = synth.make_token_batch(seqlens, cfg.vocab, seed)
        for t in ref_p.values():
            t.grad = None
        allow = None
        if mask != "causal":
            pad = pad_seqlens(seqlens, eng.spec.block_size)
            allow = sequence_masks(seqlens, masks.get_mask_fn(mask)(seqlens, pad, torch.int32), pad)
        ref = reference_loss(cfg, ref_p, torch.from_numpy(batch["tokens"]), torch.from_numpy(batch["labels"]),
                             torch.from_numpy(batch["positions"]), seqlens, 1.0 / sum(seqlens), allow)
        ref.backward()
        ok &= abs(loss - ref.item()) < 1e-5 * abs(ref.item())
        for name in ref_p:
            g, r = eng.p[name].grad, ref_p[name].grad
            err = (g - r).abs().max().item() / (r.abs().max().item() + 1e-12)
            if err > 2e-4:
                print(f"rank {rank} iteration {it} {name}: relative gradient error {err}", flush=True)
                ok = False
        torch.nn.utils.clip_grad_norm_(list(eng.p.values()), 1.0)
        torch.nn.utils.clip_grad_norm_(list(ref_p.values()), 1.0)
        eng.opt.step()
        ref_opt.step()
        eng.iteration += 1
    ok &= all((eng.p[n] - ref_p[n]).abs().max().item() < 1e-4 for n in ref_p)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("INTERP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
