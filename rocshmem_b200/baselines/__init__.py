"""baselines."""
