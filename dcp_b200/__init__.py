"""dcp_b200: dynamic context parallelism for variable-length, structured-mask LLM training on B200.

Layers (CPU planner -> per-device execution plans -> GPU executors) mirror the capabilities of the
DCP reference (dcp/__init__.py and the packages below it); the GPU side is written for sm_100a.
"""
__version__ = "0.1.0"
