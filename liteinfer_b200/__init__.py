"""liteinfer_b200: a small, whole inference engine for the dense Llama decoder on one B200."""

__version__ = "0.1.0"

from liteinfer_b200.config.engine_config import EngineConfig  # noqa: F401
from liteinfer_b200.sampling.params import SamplingParams  # noqa: F401


def __getattr__(name: str):
    # The entry points pull in the whole engine; import them on first use.
    if name == "LLM":
        from liteinfer_b200.engine.llm import LLM
        return LLM
    if name == "AsyncLLM":
        from liteinfer_b200.engine.async_llm import AsyncLLM
        return AsyncLLM
    if name in ("RequestOutput", "StreamEvent"):
        from liteinfer_b200.engine import outputs
        return getattr(outputs, name)
    raise AttributeError(name)
