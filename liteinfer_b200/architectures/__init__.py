"""Architectures: functions from a typed configuration to a `ModelSpec`."""
