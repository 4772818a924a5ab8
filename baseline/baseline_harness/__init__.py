"""Comparison harness: one launcher for this framework, the reference engine and third-party trainers."""
