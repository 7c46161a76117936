"""stratum_b200: a small model library with generation of its own for one B200 GPU."""
__version__ = "0.1.0"


def __getattr__(name):
    # the entry point imports torch and the kernels; keep `import stratum_b200` itself light
    if name in ("Stratum", "SamplingParams", "StepEntry", "GenerationResult"):
        from .engine.api import Stratum
        from .engine.generate import GenerationResult
        from .engine.step import StepEntry
        from .sampling import SamplingParams
        return {"Stratum": Stratum, "SamplingParams": SamplingParams, "StepEntry": StepEntry,
                "GenerationResult": GenerationResult}[name]
    raise AttributeError(name)
