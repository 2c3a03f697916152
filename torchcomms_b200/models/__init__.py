"""Model definitions used by the benchmarks and tests."""
from .llama import LlamaConfig, build_stages  # noqa: F401
