"""B200-native PULP-NN 8-bit kernels: Python-side mirror of the C kernel API."""
from . import workloads  # noqa: F401
