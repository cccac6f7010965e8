"""Counterpart of the reference's lib/cuda directory."""
from .cudacaller import CudaCaller  # noqa: F401
