"""stratum_b200: a small model library with generation of its own for one B200 GPU."""
__version__ = "0.1.0"
