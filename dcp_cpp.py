"""``dcp_cpp`` compatibility module: the native greedy stage selector under the reference's name
and signature (csrc/pipeline_generator/pipeline_generator.hpp:37-50)."""
from dcp_b200._planner import greedy_selection_per_device  # noqa: F401
