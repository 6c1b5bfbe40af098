"""Library kernels: ``reduction`` (cuda.reduce) and ``transpose``."""
