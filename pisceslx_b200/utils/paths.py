"""Directory layout helper (see ``utils.dc.PiscesLxPaths``)."""
from .dc import PiscesLxPaths  # noqa: F401
