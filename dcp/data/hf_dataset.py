from dcp_b200.data.datasets import (DummyMultiModelDataset, HuggingFaceDataset, HuggingFaceDatasetConfig, MockGPTLowLevelDataset, OrderedBatchSampler)  # noqa: F401
