"""Tensor / expert / context parallelism over NVLink 5 + NVSwitch (one process per GPU)."""
