"""Platform utilities."""
from .dc import (PiscesLxDeterminism, PiscesLxDeviceResolver, PiscesLxHostMemoryBudget, PiscesLxLogger, PiscesLxMetrics,
                 PiscesLxPaths, PiscesLxTracing, PiscesLxVramController)
