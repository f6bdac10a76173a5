"""Parallel runtime: process-group mesh, tensor / expert / data / pipeline / context parallel layers and the
symmetric-memory fused collectives."""
from .state import YvParallelState, destroy_parallel, get_state, init_parallel
