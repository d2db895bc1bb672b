"""Timing, clock sampling, checkpointing and profiling helpers."""
