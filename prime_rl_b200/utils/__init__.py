"""Logging, paths, process supervision and small helpers."""
