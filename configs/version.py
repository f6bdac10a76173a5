"""Version substituted for the ``{{VERSION}}`` placeholder of the YAML presets."""
VERSION = "0.1.0"
