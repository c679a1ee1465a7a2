"""Importing this package registers the built-in parts."""
from . import (attention, block, embedding, experts, latent_attention, masked_attention, mlp, norm, parallel, recurrent, rotary,
               streams)  # noqa: F401
