from dcp_b200.core.serialization import *  # noqa: F401,F403
from dcp_b200.core.serialization import ByteReader, ByteWriter  # noqa: F401
