"""Built-in parts.  Importing this package registers them by kind."""

from . import base  # noqa: F401
from . import norm, position, attention, attention_mix, attention_latent, recurrent, feed_forward, block  # noqa: F401
from .base import (Block, BuiltLayer, CacheBinding, Deferred, Embedding, FeedForward, KVGroupView, KVNeed, LMHead, Mixer, Norm,
                   PagedCacheNeed, Part, PositionEncoding, Precision, Runtime, StateNeed, StepContext, TensorDecl, TensorSum, WeightedRowSum,
                   apply_norm, linear, precision_from_name, resolve, split_sum)

__all__ = ["Block", "BuiltLayer", "CacheBinding", "Deferred", "Embedding", "FeedForward", "KVGroupView", "KVNeed", "PagedCacheNeed", "LMHead", "Mixer",
           "Norm", "Part", "PositionEncoding", "Precision", "Runtime", "StateNeed", "StepContext", "TensorDecl",
           "TensorSum", "WeightedRowSum", "apply_norm", "linear", "precision_from_name", "resolve", "split_sum"]
