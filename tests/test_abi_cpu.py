"""The C-ABI library loads without a GPU and exports every symbol include/bert_b200.h declares; argument
validation (host code) returns error statuses instead of touching the device."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "bert_b200.h").read_text()
    return sorted(set(re.findall(r"BERT_B200_API\s+[\w\s\*]+?\b(bert_b200_\w+)\s*\(", text)))


def test_header_symbols_exported():
    from tensorrt_b200 import _lib

    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in bert_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_version_and_error_text():
    from tensorrt_b200 import _lib

    assert _lib.lib.bert_b200_version() >= 100
    st = _lib.lib.bert_b200_skip_layer_norm(None, 1, 768, 100, None, None, None, None, None, None)
    assert st == 2  # BERT_B200_BAD_PARAM: n is not a multiple of ld
    assert b"multiple" in _lib.lib.bert_b200_last_error()
    st = _lib.lib.bert_b200_skip_layer_norm(None, 1, 768, 768, None, None, None, None, None, None)
    assert st == 2 and b"null" in _lib.lib.bert_b200_last_error()


def test_fc_and_mha_validation():
    from tensorrt_b200 import _lib

    p = _lib.FcParams()
    p.type_id, p.out_type_id, p.m, p.n, p.k = 1, 1, 8, 16, 0
    assert _lib.lib.bert_b200_fc(C.byref(p), None) == 2
    assert _lib.lib.bert_b200_fc(None, None) == 2
    m = _lib.MhaParams()
    # INT8 outside the tensor-core kernel's shapes (FP16 would take the SIMT kernel there)
    m.type_id, m.B, m.S, m.num_heads, m.head_size = 2, 1, 1024, 2, 64
    m.qkv = m.out = C.c_void_p(0x1000)
    assert _lib.lib.bert_b200_mha(C.byref(m), None) == 3  # BERT_B200_NOT_SUPPORTED: S > 512
    m.S, m.head_size = 128, 80
    assert _lib.lib.bert_b200_mha(C.byref(m), None) == 3
    m.head_size = 24
    assert _lib.lib.bert_b200_mha(C.byref(m), None) == 3


def test_attention_workspace_and_separate_tensor_entry_validation():
    from tensorrt_b200 import _lib

    m = _lib.MhaParams()
    m.type_id, m.B, m.S, m.num_heads, m.head_size = 1, 4, 1024, 16, 64
    # no attention kernel needs scratch memory: FP16 streams the key blocks of long sequences through tensor memory
    assert _lib.lib.bert_b200_mha_workspace_size(C.byref(m)) == 0
    m.S, m.type_id = 1024, 2
    assert _lib.lib.bert_b200_mha_workspace_size(C.byref(m)) == 0
    assert _lib.lib.bert_b200_mha_workspace_size(None) == 0

    a = _lib.AttentionBnsdParams()
    assert _lib.lib.bert_b200_attention_bnsd(None, None) == 2
    a.type_id, a.B, a.S, a.num_heads, a.head_size = 1, 1, 128, 2, 64
    assert _lib.lib.bert_b200_attention_bnsd(C.byref(a), None) == 2 and b"null" in _lib.lib.bert_b200_last_error()
    a.q = a.k = a.v = a.out = C.c_void_p(0x1000)
    a.S, a.type_id = 600, 2
    assert _lib.lib.bert_b200_attention_bnsd(C.byref(a), None) == 3      # BERT_B200_NOT_SUPPORTED: INT8 beyond 512 keys
    a.type_id = 1
    assert _lib.lib.bert_b200_attention_bnsd(C.byref(a), None) == 2 and b"scale_bmm1" in _lib.lib.bert_b200_last_error()
    a.S, a.head_size = 128, 40
    assert _lib.lib.bert_b200_attention_bnsd(C.byref(a), None) == 3
    a.head_size, a.type_id = 64, 0
    assert _lib.lib.bert_b200_attention_bnsd(C.byref(a), None) == 2      # FP32 is not offered here


def test_encoder_config_validation():
    from tensorrt_b200 import _lib

    cfg = _lib.EncoderConfig()
    assert _lib.lib.bert_b200_encoder_workspace_size(C.byref(cfg), 128, 1) == -1
    h = C.c_void_p()
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 2


def test_encoder_create_checks_int8_scales():
    """INT8: every dequantisation step must be finite and positive, and a layer must read its input with the step the
    previous layer wrote it with - otherwise the quantising epilogues produce inf / NaN or silently wrong values."""
    from tensorrt_b200 import _lib

    fake = C.c_void_p(0x1000)   # never dereferenced by create
    layers = (_lib.LayerWeights * 2)()
    names = [n for n, _ in _lib.LayerWeights._fields_]
    for lw in layers:
        for n in names:
            setattr(lw, n, fake if not n.startswith("s_") else 0.05)
    cfg = _lib.EncoderConfig(2, 2, 128, 2, 512, 100, 64, 2, 1.0 / 127, fake, fake, fake, fake, fake, layers)
    h = C.c_void_p()
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 0
    _lib.lib.bert_b200_encoder_destroy(h)
    layers[1].s_ffn1 = 0.0
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 2
    assert b"layer 1" in _lib.lib.bert_b200_last_error()
    layers[1].s_ffn1 = float("nan")
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 2
    layers[1].s_ffn1 = 0.05
    layers[1].s_in = 0.06                                  # layer 0 wrote its output with step 0.05
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 2
    assert b"s_in != s_out" in _lib.lib.bert_b200_last_error()
    cfg.type_id = 1                                        # FP16 ignores the scales
    assert _lib.lib.bert_b200_encoder_create(C.byref(cfg), C.byref(h)) == 0
    _lib.lib.bert_b200_encoder_destroy(h)


def test_no_cpu_fallback():
    import torch

    import tensorrt_b200 as T

    with pytest.raises(ValueError):
        T.skip_layer_norm(torch.zeros(2, 8), torch.zeros(2, 8), torch.ones(8), torch.zeros(8))
