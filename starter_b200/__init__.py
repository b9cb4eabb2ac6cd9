"""starter_b200: a small model library with generation of its own for the Qwen3 dense decoder on
one B200 (sm_100a): typed config and registry, safetensors weights, layer parts, a paged cache with
per-sequence slots, one step function, a generation loop, sampling, and hand-written CUDA kernels."""

__version__ = "0.1.0"


def __getattr__(name):
    # the entry point needs torch and the kernels; import it on first use
    if name in ("Engine", "Completion", "Request", "SamplingParams"):
        from .engine import entry
        return getattr(entry, name)
    raise AttributeError(f"module 'starter_b200' has no attribute {name!r}")
