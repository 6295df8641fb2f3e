from dcp_b200.planner.stages import generate_pipelines_n_stages, pipeline_chrome_trace, summarize_pipeline  # noqa: F401
from dcp_b200.planner.steiner import generate_pipelines_n_stages_with_tree_packing  # noqa: F401
