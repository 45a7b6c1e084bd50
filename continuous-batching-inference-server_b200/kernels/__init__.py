from . import library, ops  # noqa: F401
