"""stkernel_b200: a Blackwell-native (sm_100a) DeepSeek-V4-Flash serving engine."""
__version__ = "0.1.0"
