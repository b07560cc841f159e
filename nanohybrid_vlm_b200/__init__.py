"""A single-GPU inference engine for Qwen3 dense on NVIDIA B200 (sm_100a).

    from nanohybrid_vlm_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model_folder")
    out = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=8))
"""
from .sampling.params import SamplingParams


def __getattr__(name):
    # the engine pulls in torch and the kernels; keep `import nanohybrid_vlm_b200` light
    if name in ("LLM", "LLMEngine"):
        from .engine.llm_engine import LLM, LLMEngine
        return {"LLM": LLM, "LLMEngine": LLMEngine}[name]
    raise AttributeError(name)


__all__ = ["LLM", "LLMEngine", "SamplingParams"]
