from .engine import InferenceEngine
from .types import InferenceRequest, InferenceResult, ModelConfig, SamplingParams, ServerConfig
