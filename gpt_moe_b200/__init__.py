"""gpt_moe_b200: a Blackwell-native GPT-MoE training framework (PyTorch + hand-written sm_100a kernels)."""
__version__ = "0.1.0"
