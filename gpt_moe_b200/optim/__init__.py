from .adamw import AdamW, configure_adamw_moments
from .muon import Muon

__all__ = ["AdamW", "Muon", "configure_adamw_moments"]
