from dcp_b200.utils.visualization import visualize_workload_spec_figure, visualize_workload_spec_tty  # noqa: F401
