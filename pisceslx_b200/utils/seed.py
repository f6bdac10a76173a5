"""Seeding helper (see ``utils.dc.PiscesLxDeterminism``)."""
from .dc import PiscesLxDeterminism  # noqa: F401
