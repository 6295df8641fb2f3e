"""Two-rank worker: trains two steps and writes a checkpoint into the directory given as argv[1]
(launched with torch.distributed.run by tests/test_gpu_engine.py, which then resumes it on one GPU)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.data import synth  # noqa: E402
from dcp_b200.models.llama import tiny_config  # noqa: E402
from dcp_b200.train import EngineConfig, TrainEngine, init_distributed  # noqa: E402


def engine_config():
    return EngineConfig(tiny_config(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, ffn=2048, vocab=2048),
                        tokens_per_step=1536, block_size=256,
                        length_dist=synth.LengthDist("lognormal", 400.0, 0.6, 64, 1536), planner_workers=0, lr=1e-3)


def main():
    rank, world, local, group = init_distributed()
    dev = torch.device("cuda", local)
    eng = TrainEngine(engine_config(), dev, group)
    eng.train_step()
    eng.train_step()
    eng.save_checkpoint(sys.argv[1])
    torch.cuda.synchronize()
    eng.close()
    if rank == 0:
        print("CKPT_OK", flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
