from .engine import BLOCK_SIZE, InferenceEngine, SamplingParams, TokenOutput  # noqa: F401
