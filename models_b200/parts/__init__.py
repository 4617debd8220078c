from . import (attention, block, capped_attention, dense_feed_forward, embedding, feed_forward, gated_block, head,  # noqa: F401
               hyper_block, latent_attention, layer_norm, min_gru, norm, parallel_block, retention, rope,
               routed_feed_forward, side_by_side, sigmoid_attention, talking_attention)  # registers the built-in parts
from .base import MODES, Mixer, Part, Prenormed, RunContext, Runtime, StreamsRead, as_delta
from .linear import add_linear, linear
from .registry import build_part, known_parts, register_part, unregister_part
