"""Harness that runs the unmodified reference engine (installed under ``baseline/_ref``)."""
