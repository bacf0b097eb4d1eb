"""sparkflash_b200: a B200-native (sm_100a) inference framework for the DeepSeek-V4.1-Flash family."""
__version__ = "0.1.0"
