"""ferrite_b200: a Blackwell-native (sm_100a) LLM inference framework."""
__version__ = "0.1.0"
from .config import GlmConfig, EngineConfig, SchedConfig  # noqa: F401
