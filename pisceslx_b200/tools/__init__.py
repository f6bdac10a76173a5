"""User-facing tools beside the engine: benchmark harness, export / packaging."""
