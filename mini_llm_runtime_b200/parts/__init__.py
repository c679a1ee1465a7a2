"""Importing this package registers the built-in parts."""
from . import attention, block, embedding, masked_attention, mlp, norm, parallel, recurrent, rotary  # noqa: F401
