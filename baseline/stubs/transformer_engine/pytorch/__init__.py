import contextlib

import torch.nn as nn


class Linear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, params_dtype=None, device=None, init_method=None, **kwargs):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=params_dtype)


@contextlib.contextmanager
def autocast(enabled=True, recipe=None):
    raise RuntimeError("Transformer Engine FP8 is not available in this image")
    yield
