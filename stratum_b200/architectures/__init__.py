from . import llama  # noqa: F401  (registers the architecture)
