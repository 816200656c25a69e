"""litellmengine_b200: a small, whole inference engine for Qwen3 dense on one B200."""
__version__ = "0.1.0"
