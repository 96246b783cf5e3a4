"""kareus_b200: a Blackwell-native, energy-aware Megatron-style LLM training runtime."""
__version__ = "0.1.0"
