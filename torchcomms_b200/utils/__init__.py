"""Timing, clock sampling and small helpers shared by benchmarks."""
