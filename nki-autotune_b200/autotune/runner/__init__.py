"""Compile-check -> time-on-GPU -> tabulate pipeline (mirrors ``autotune.runner`` upstream)."""
