"""B200 (sm_100a) implementation of the TensorRT-OSS BERT encoder plugin hot path.

The native library is mandatory: importing the package loads tensorrt_b200/libbert_b200.so and raises if
it is missing (build it with `python tensorrt_b200/csrc/build.py`). There is no CPU or PyTorch fallback.
"""
from . import _lib  # noqa: F401  (loads the shared library, fails loudly when absent)
from .ops import (ACT_GELU_ERF, ACT_NONE, FP16, FP32, INT8, attention_bnsd, compute_mask_idx, convert_mask, emb_layer_norm,
                  emb_layer_norm_var_seqlen, fc, lengths_to_cu_seqlens, mha, packed_mask_to_lengths, skip_layer_norm, skip_layer_norm_dqq,
                  skip_layer_norm_interleaved)
from .encoder import BertEncoder
from .sharding import shard_even, shard_by_tokens

__all__ = [
    "ACT_GELU_ERF", "ACT_NONE", "FP16", "FP32", "INT8", "BertEncoder", "compute_mask_idx", "convert_mask",
    "emb_layer_norm", "emb_layer_norm_var_seqlen", "fc", "lengths_to_cu_seqlens", "mha", "packed_mask_to_lengths", "skip_layer_norm",
    "skip_layer_norm_dqq", "skip_layer_norm_interleaved", "shard_even", "shard_by_tokens",
]
