"""Baselines: the unmodified reference library (built with dependency shims) and NCCL."""
