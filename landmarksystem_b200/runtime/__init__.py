"""Runtime services around the trainers: failure detection (heartbeats between ranks) and checkpoint I/O."""
from .checkpoint import AsyncCheckpointer, load_sharded, save_sharded  # noqa: F401
from .health import HeartbeatMonitor, PeerFailure, StatusWords  # noqa: F401
