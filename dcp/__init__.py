"""Import-path compatibility: ``dcp.*`` resolves to the B200-native implementation in ``dcp_b200``.

Users of the reference import ``dcp.core.instructions``, ``dcp.data.dataloader``,
``dcp.runtime.flash_attention`` and friends; each of those module paths is a thin re-export here.
"""
from dcp_b200 import __version__  # noqa: F401
