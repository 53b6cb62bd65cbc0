"""Platform surfaces: REST API (FastAPI), MCP tool server, shared in-memory state."""
from .store import LiveStateStore

__all__ = ["LiveStateStore"]
