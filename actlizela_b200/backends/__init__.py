"""Backend catalog of the B200 build (one target, one algorithm)."""
from .registry import backend_inventory, require_backend, require_implementation

__all__ = ["backend_inventory", "require_backend", "require_implementation"]
