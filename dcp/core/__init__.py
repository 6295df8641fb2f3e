"""Core IR (re-exports of dcp_b200.core and dcp_b200.planner)."""
