"""Worker of test_pipeline_stage_boundary (torch.distributed.run, backend gloo): a small MLP cut into
pipeline stages, variable-length micro-batches in one-forward-one-backward order; every stage's
parameter gradients and the losses must equal those of the unsplit model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.parallel.pipeline import PipelineComm, run_stage_1f1b  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(3)
    hidden, n_layers, tokens = 32, 2 * world, [40, 17, 64, 5, 33]
    layers = [torch.nn.Linear(hidden, hidden, dtype=torch.float64) for _ in range(n_layers)]
    xs = [torch.randn(n, hidden, dtype=torch.float64) for n in tokens]
    ys = [torch.randn(n, hidden, dtype=torch.float64) for n in tokens]
    run = lambda ls, x: [x := torch.tanh(l(x)) for l in ls][-1]
    # unsplit reference (every rank computes it: same seed)
    ref_losses = []
    for x, y in zip(xs, ys):
        loss = ((run(layers, x) - y) ** 2).mean()
        loss.backward()
        ref_losses.append(loss.item())
    ref_grads = [l.weight.grad.clone() for l in layers]
    for l in layers:
        l.weight.grad = None
        l.bias.grad = None
    mine = layers[rank * 2:(rank + 1) * 2]
    comm = PipelineComm(dist.group.WORLD, lambda mb: (tokens[mb], hidden), torch.float64, torch.device("cpu"))
    losses = run_stage_1f1b(comm, len(tokens), lambda mb, x: run(mine, xs[mb] if x is None else x),
                            lambda mb, y: ((y - ys[mb]) ** 2).mean())
    ok = all((l.weight.grad - g).abs().max().item() < 1e-10 for l, g in zip(mine, ref_grads[rank * 2:(rank + 1) * 2]))
    if comm.is_last:
        ok = ok and len(losses) == len(tokens) and all(abs(a.item() - b) < 1e-12 for a, b in zip(losses, ref_losses))
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("PP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
