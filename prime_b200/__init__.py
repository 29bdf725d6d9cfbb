"""prime_b200: Blackwell-native decentralized LLM pre-training (DiLoCo + ZeRO-3 + elastic mesh)."""
__version__ = "0.1.0"
