"""ctypes binding of libbert_b200.so (declarations mirror include/bert_b200.h).

There is no CPU fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libbert_b200.so"

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python tensorrt_b200/csrc/build.py` (needs nvcc). "
        "tensorrt_b200 has no CPU or PyTorch fallback.")

lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)

vp = C.c_void_p
i32 = C.c_int32
i64 = C.c_int64
u32 = C.c_uint32
f32 = C.c_float


class FcParams(C.Structure):
    _fields_ = [("type_id", i32), ("out_type_id", i32), ("m", i64), ("n", i64), ("k", i64), ("a", vp), ("lda", i64),
                ("wt", vp), ("c", vp), ("ldc", i64), ("bias", vp), ("activation", i32), ("alpha", f32),
                ("out_scale", f32), ("status_word", vp)]


class MhaParams(C.Structure):
    _fields_ = [("type_id", i32), ("B", i32), ("S", i32), ("num_heads", i32), ("head_size", i32), ("total", i32),
                ("qkv", vp), ("out", vp), ("cu_seqlens", vp), ("mask_idx", vp), ("interleaved", i32),
                ("scale_bmm1", f32), ("scale_softmax", f32), ("scale_bmm2", f32), ("status_word", vp), ("workspace", vp),
                ("workspace_bytes", i64)]


class AttentionBnsdParams(C.Structure):
    _fields_ = [("type_id", i32), ("B", i32), ("S", i32), ("num_heads", i32), ("head_size", i32), ("q", vp), ("k", vp),
                ("v", vp), ("out", vp), ("kv_lengths", vp), ("scale_bmm1", f32), ("scale_softmax", f32),
                ("scale_bmm2", f32), ("status_word", vp)]


class LayerWeights(C.Structure):
    _fields_ = [("wt_qkv", vp), ("b_qkv", vp), ("wt_out", vp), ("b_out", vp), ("ln1_gamma", vp), ("ln1_beta", vp),
                ("wt_ffn1", vp), ("b_ffn1", vp), ("wt_ffn2", vp), ("b_ffn2", vp), ("ln2_gamma", vp), ("ln2_beta", vp),
                ("s_in", f32), ("s_wqkv", f32), ("s_qkv", f32), ("s_ctx", f32), ("s_wout", f32), ("s_attn_out", f32),
                ("s_ln1", f32), ("s_wffn1", f32), ("s_ffn1", f32), ("s_wffn2", f32), ("s_ffn2", f32), ("s_out", f32)]


class EncoderConfig(C.Structure):
    _fields_ = [("type_id", i32), ("num_layers", i32), ("hidden_size", i32), ("num_heads", i32), ("ffn_size", i32),
                ("vocab_size", i32), ("max_positions", i32), ("type_vocab_size", i32), ("dq_probs", f32),
                ("word_emb", vp), ("pos_emb", vp), ("tok_emb", vp), ("emb_gamma", vp), ("emb_beta", vp),
                ("layers_host", C.POINTER(LayerWeights))]


# name -> (restype, argtypes); must list every BERT_B200_API symbol of include/bert_b200.h
SIGNATURES = {
    "bert_b200_version": (i32, []),
    "bert_b200_last_error": (C.c_char_p, []),
    "bert_b200_read_status_word": (i32, [vp, vp, C.POINTER(u32)]),
    "bert_b200_skip_layer_norm": (i32, [vp, i32, i32, i64, vp, vp, vp, vp, vp, vp]),
    "bert_b200_skip_layer_norm_dqq": (i32, [vp, i32, i64, vp, vp, vp, vp, vp, vp, f32, f32, f32]),
    "bert_b200_skip_layer_norm_interleaved_hface": (i32, [vp, i32, i32, vp, vp, vp, vp, vp, f32, f32, f32]),
    "bert_b200_skip_layer_norm_interleaved_mtron": (i32, [vp, i32, i32, vp, vp, vp, vp, vp, vp, f32, f32, f32, f32]),
    "bert_b200_emb_layer_norm": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32]),
    "bert_b200_emb_layer_norm_mask_idx": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, vp, vp]),
    "bert_b200_emb_layer_norm_var_seqlen": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, f32]),
    "bert_b200_compute_mask_idx": (i32, [vp, i32, i32, vp, vp]),
    "bert_b200_convert_mask": (i32, [u32, u32, u32, u32, u32, vp, vp, vp]),
    "bert_b200_packed_mask_to_lengths": (i32, [vp, i32, i32, u32, u32, u32, vp, vp]),
    "bert_b200_lengths_to_cu_seqlens": (i32, [vp, i32, vp, vp]),
    "bert_b200_fc": (i32, [C.POINTER(FcParams), vp]),
    "bert_b200_attention_bnsd": (i32, [C.POINTER(AttentionBnsdParams), vp]),
    "bert_b200_mha_workspace_size": (i64, [C.POINTER(MhaParams)]),
    "bert_b200_mha": (i32, [C.POINTER(MhaParams), vp]),
    "bert_b200_selftest_wait_expiry": (i32, [vp, i64, vp, vp]),
    "bert_b200_probe_mma_rate": (i32, [vp, i32, i32, vp, C.POINTER(f32)]),
    "bert_b200_encoder_workspace_size": (i64, [C.POINTER(EncoderConfig), i32, i32]),
    "bert_b200_encoder_create": (i32, [C.POINTER(EncoderConfig), C.POINTER(vp)]),
    "bert_b200_encoder_destroy": (i32, [vp]),
    "bert_b200_encoder_last_launch_count": (i32, [vp]),
    "bert_b200_encoder_enable_timing": (i32, [vp, i32]),
    "bert_b200_encoder_read_timing": (i32, [vp, C.POINTER(f32), C.POINTER(i32)]),
    "bert_b200_encoder_calibrate": (i32, [vp, vp, i32, i32, i32, vp, vp, vp, vp, i64, vp, vp, C.POINTER(f32)]),
    "bert_b200_encoder_forward": (i32, [vp, vp, i32, i32, i32, vp, vp, vp, vp, i64, vp]),
    "bert_b200_encoder_static_workspace_limit": (i64, []),
    "bert_b200_encoder_forward_static": (i32, [vp, vp, i32, i32, i32, vp, vp, vp, vp]),
    "bert_b200_encoder_forward_host": (i32, [vp, vp, i32, i32, i32, vp, vp, vp, vp, i64, vp, vp]),
    "bert_b200_encoder_forward_host_async": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, i64, vp, vp]),
    "bert_b200_encoder_wait_host": (i32, [vp, i32]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library and the header disagree
    _fn.restype = _res
    _fn.argtypes = _args


class BertB200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        msg = lib.bert_b200_last_error().decode(errors="replace")
        super().__init__(f"{where} failed with status {status}: {msg}")
        self.status = status


def check(status: int, where: str) -> None:
    if status != 0:
        raise BertB200Error(status, where)
