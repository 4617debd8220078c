from . import (attention, block, capped_attention, chunked_attention, dense_feed_forward, embedding, feed_forward, gated_block,  # noqa: F401
               gated_delta, head, hyper_block, latent_attention, layer_norm, min_gru, norm, normed_pair, output_norm_block,
               parallel_block, retention, rglru, rope, routed_feed_forward, side_by_side, sigmoid_attention,
               talking_attention)  # registers the built-in parts
from .base import MODES, Mixer, Part, Prenormed, RunContext, Runtime, StreamRows, StreamsRead, as_delta
from .linear import add_linear, linear
from .registry import build_part, known_parts, register_part, unregister_part
