from dcp_b200.planner.compiler import CompilerConfig, InstrCompiler  # noqa: F401
