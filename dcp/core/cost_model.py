from dcp_b200.core.cost_model import AttnRooflineCostModel, CommunicationCostModel, CostModel  # noqa: F401
