"""``LLM``: the engine under the name that users of the reference know (``from llm import LLM`` there).

    llm = LLM(model_folder, dtype="bfloat16", max_num_seqs=256, max_num_batched_tokens=16384)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.6, max_tokens=128))
"""
from .engine.llm_engine import LLMEngine

LLM = LLMEngine

__all__ = ["LLM"]
