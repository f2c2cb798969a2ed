"""Presets, tuner and benchmark drivers (counterparts of the reference's tools/ and tests/ scripts)."""
