"""spark_engine_b200: a B200-native (sm_100a) MoE inference engine.

Hybrid linear-attention / sparse-attention Mixture-of-Experts language models served from EXL3,
MXFP4 and FP8 block-scaled weights, with speculative decoding, a KV pool, prefix caches and an
OpenAI-compatible server; hand-written tcgen05/TMA kernels and fused compute+collective kernels
over NVLink peer memory.
"""
__version__ = "0.1.0"

from .config import EngineConfig, ModelConfig, get_model_config  # noqa: F401
