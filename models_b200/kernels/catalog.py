"""Every kernel library of the package, for building them all ahead of time."""

from __future__ import annotations

from .build import build_library

# (name, sources, definitions)
LIBRARIES = [
    ("mb_elementwise", ["elementwise.cu"], {}),
    ("mb_attention_rows", ["attention_rows.cu"], {}),
    ("mb_gemm_f32", ["gemm_f32.cu"], {}),
    ("mb_sampling", ["sampling.cu"], {}),
    ("mb_talking_attention", ["talking_attention.cu"], {}),
    ("mb_gated_recurrence", ["gated_recurrence.cu"], {}),
    ("mb_gated_delta", ["gated_delta.cu"], {}),
    ("mb_gated_attention", ["gated_attention.cu"], {}),
    ("mb_retention", ["retention.cu"], {}),
    ("mb_hyper_streams", ["hyper_streams.cu"], {}),
    ("mb_routed_experts", ["routed_experts.cu"], {}),
    # the tensor-core form is compiled per (key size, value size, values read from the key rows) at first use; these
    # are the sizes of the benchmark's models of the design that uses it
    ("mb_gated_attention_tc", ["gated_attention_tc.cu"], {"MB_KEY_DIM": 64, "MB_VALUE_DIM": 128, "MB_SHARED_ROWS": 0}),
    ("mb_gated_attention_tc", ["gated_attention_tc.cu"], {"MB_KEY_DIM": 256, "MB_VALUE_DIM": 256, "MB_SHARED_ROWS": 1}),
    ("mb_random_init", ["random_init.cu"], {}),
    ("mb_skinny_gemm", ["skinny_gemm.cu"], {}),
    ("mb_gemm_tcgen05", ["gemm_tcgen05.cu"], {}),
    ("mb_wide_gemm_tcgen05", ["wide_gemm_tcgen05.cu"], {}),
    # the tensor-core attention is compiled per head size when a model first needs it; these are
    # the sizes of the benchmark models and of the tests
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 16}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 32}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 48}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_attention_tc", ["attention_tc.cu"], {"MB_HEAD_DIM": 128}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 16}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 32}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 48}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_decode_step", ["decode_step.cu"], {"MB_HEAD_DIM": 128}),
    ("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": 64}),
    ("mb_prefill_attention_tcgen05", ["prefill_attention_tcgen05.cu"], {"MB_HEAD_DIM": 128}),
    # the tensor-core attention with weights mixed across heads is compiled per (heads, key size, value size);
    # these are the sizes of the benchmark's models of that design
    ("mb_talking_attention_tc", ["talking_attention_tc.cu"], {"MB_HEADS": 8, "MB_KEY_DIM": 64, "MB_VALUE_DIM": 128}),
    ("mb_talking_attention_tc", ["talking_attention_tc.cu"], {"MB_HEADS": 16, "MB_KEY_DIM": 64, "MB_VALUE_DIM": 128}),
]


def build_all(quiet: bool = False):
    return [build_library(name, sources, defines, quiet=quiet) for name, sources, defines in LIBRARIES]
