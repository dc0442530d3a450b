"""reinfer_b200: a single-GPU inference engine for B200 (sm_100a), with hand-written
CUDA kernels, a paged cache, one step function for mixed batches, a scheduler and
samplers.  Public entry points: `LLM` / `SamplingParams` (generation), `Engine` /
`StepEntry` (the step function), `bin/trace_run` (replay), `python -m reinfer_b200`
(command line)."""

__version__ = "0.1.0"

from .engine import Engine, StepEntry  # noqa: E402,F401


def __getattr__(name):
    if name in ("LLM", "SamplingParams", "RequestOutput"):
        from .engine import llm as _llm
        return getattr(_llm, name)
    raise AttributeError(name)
