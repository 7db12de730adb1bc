"""Kernel-level entry points with the reference's eDSL kernel signatures (output passed in)."""
