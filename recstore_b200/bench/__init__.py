"""Micro-benchmarks of the native kernels and subsystems (roofline fractions against measured peaks)."""
