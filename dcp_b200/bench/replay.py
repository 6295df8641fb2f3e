"""Offline replay of saved planner artefacts (the reference's debug scripts:
scripts/testing/debug_compiler.py, tests/core/debug_compiler.py, tests/runtime/debug_attn.py).

    DCP_DEBUG_SAVE_PARTITION_RESULTS=1 DCP_DEBUG_SAVE_PARTITION_RESULTS_FILE=part.pkl  (during a run)
    python -m dcp_b200.bench.replay plans dcp_exec_plans.pkl     # validate + summarise saved plans
    python -m dcp_b200.bench.replay plan-bytes plan.bin          # decode a serialized ExecutionPlan
"""
from __future__ import annotations

import pickle
import sys

from ..core.common import get_default_execution_context
from ..core.instructions import ExecutionPlan
from ..planner.validate import validate_plans


def replay_plans(path: str) -> dict:
    fw_wl, bw_wl, fw, bw = pickle.load(open(path, "rb"))
    any_plan = next(iter(fw.values()))
    ctx = get_default_execution_context(any_plan.n_nodes * any_plan.n_devices_per_node, any_plan.n_nodes)
    out = {"forward": validate_plans(ctx, fw_wl, fw, True)}
    if bw:
        out["backward"] = validate_plans(ctx, bw_wl, bw, False)
    out["instructions_per_device"] = {str(d): len(p.instructions) for d, p in fw.items()}
    return out


def main(argv=None):
    argv = argv or sys.argv[1:]
    if len(argv) != 2 or argv[0] not in ("plans", "plan-bytes"):
        print(__doc__)
        return 2
    if argv[0] == "plans":
        print(replay_plans(argv[1]))
    else:
        plan, rest = ExecutionPlan.deserialize(open(argv[1], "rb").read())
        print(plan)
        print(f"{len(rest)} trailing bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
