"""mintext_b200: a Blackwell-native (sm_100a) LLM pre-training framework with the public surface of MinText."""

from mintext_b200.config import MinTextConfig, load_config

__version__ = "0.1.0"
__all__ = ["MinTextConfig", "load_config", "__version__"]
