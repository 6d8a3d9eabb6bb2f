from molt_b200.core.errors import CapabilityError, IntegrityError, MoltError, MoltStreamError

__all__ = ["CapabilityError", "IntegrityError", "MoltError", "MoltStreamError"]
