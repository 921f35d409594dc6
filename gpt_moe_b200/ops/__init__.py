"""Ops: `api` (entry points), `reference` (plain PyTorch definitions / oracle), `cuda_ops` (sm_100a kernels)."""
