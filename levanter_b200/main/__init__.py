"""Entry points: ``python -m levanter_b200.main.<name> --config_path cfg.yaml --key.subkey value``."""
