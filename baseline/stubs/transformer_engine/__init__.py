"""Offline stand-in for Transformer Engine (not installed in this image).  The reference derives its `Linear`
from `te.Linear`; with every role at default precision only plain `nn.Linear` behaviour is exercised."""
