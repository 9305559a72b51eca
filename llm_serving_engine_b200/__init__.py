"""B200-native inference engine for the Qwen2.5 dense decoder."""
__version__ = "0.1.0"
