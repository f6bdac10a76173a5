"""Configuration presets (model and training YAML files) and the version constant."""
