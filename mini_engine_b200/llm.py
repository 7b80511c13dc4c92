"""``LLM`` is the engine under the name users know (reference: llm.py:1-4)."""
from .engine.llm_engine import LLMEngine


class LLM(LLMEngine):
    pass
