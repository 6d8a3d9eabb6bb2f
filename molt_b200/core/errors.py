"""Error types of the hot path; same names and hierarchy as the reference's ``core/errors.py:1-13``."""


class MoltStreamError(RuntimeError):
    """Explicit failure; nothing falls back silently."""


class CapabilityError(MoltStreamError):
    """The requested mechanism cannot run on this runtime, device, dtype or shape."""


class IntegrityError(MoltStreamError):
    """Persistent state failed an integrity check."""


MoltError = MoltStreamError
