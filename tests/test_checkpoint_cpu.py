"""Checkpoint packing (tensorrt_b200/checkpoint.py) and the whole-encoder wiring of the oracle against an independent
implementation: a randomly initialised Hugging Face BertModel (FP32, CPU). The weights are first rounded to FP16 values
so that both sides see the same numbers."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O
from tensorrt_b200.checkpoint import pack_padded_batch, params_from_bert_state_dict

transformers = pytest.importorskip("transformers")


def make_hf(layers=2, hidden=128, heads=2, ffn=512, vocab=500, max_pos=64, seed=0, pooler=False):
    torch.manual_seed(seed)
    cfg = transformers.BertConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                                  intermediate_size=ffn, max_position_embeddings=max_pos, type_vocab_size=2,
                                  hidden_act="gelu", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = transformers.BertModel(cfg, add_pooling_layer=pooler).eval()
    with torch.no_grad():
        for p in model.parameters():
            p.copy_((p + 0.05 * torch.randn_like(p)).half().float())  # biases / LayerNorm off their trivial init
    return model


def padded_batch(rng, B, S, vocab):
    lengths = rng.integers(3, S + 1, size=B)
    lengths[0] = S
    ids = rng.integers(0, vocab, size=(B, S))
    seg = (np.arange(S)[None] >= rng.integers(1, S, size=(B, 1))).astype(np.int64)
    mask = (np.arange(S)[None] < lengths[:, None]).astype(np.int64)
    return ids, seg, mask, lengths


def test_oracle_encoder_matches_huggingface_bert():
    model = make_hf()
    rng = np.random.default_rng(0)
    B, S = 5, 48
    ids, seg, mask, lengths = padded_batch(rng, B, S, 500)
    with torch.no_grad():
        want = model(input_ids=torch.from_numpy(ids), token_type_ids=torch.from_numpy(seg),
                     attention_mask=torch.from_numpy(mask)).last_hidden_state.numpy()
    p = params_from_bert_state_dict(model.state_dict(), num_heads=2)
    pid, pseg, cu = pack_padded_batch(ids, seg, mask)
    got = O.encoder_fp(p, pid, pseg, cu, S, round_fp16=False)
    want_packed = np.concatenate([want[b, :lengths[b]] for b in range(B)])
    # same weights, FP32 vs float64 arithmetic, LayerNorm epsilon 1e-12 vs none
    assert np.abs(got - want_packed).max() < 2e-4


def test_qkv_packing_order():
    model = make_hf(layers=1, hidden=64, heads=4, ffn=128)
    sd = model.state_dict()
    p = params_from_bert_state_dict({"bert." + k: v for k, v in sd.items()}, num_heads=4)  # prefix is stripped
    d = 16
    wq = sd["encoder.layer.0.attention.self.query.weight"].numpy()
    wv = sd["encoder.layer.0.attention.self.value.weight"].numpy()
    w = p.layers[0].w_qkv.astype(np.float32)
    for h in range(4):
        assert np.array_equal(w[:, (h * 3 + 0) * d:(h * 3 + 1) * d], wq[h * d:(h + 1) * d].T)
        assert np.array_equal(w[:, (h * 3 + 2) * d:(h * 3 + 3) * d], wv[h * d:(h + 1) * d].T)
    assert p.ffn == 128 and p.hidden == 64 and len(p.layers) == 1
    with pytest.raises(ValueError):
        params_from_bert_state_dict(sd, num_heads=5)


def test_empty_sequences_are_rejected_before_packing():
    """An all-zero mask row would make the next sequence's first token look like this one's [CLS] row."""
    import pytest

    from tensorrt_b200.checkpoint import pack_padded_batch

    ids = np.ones((3, 4), dtype=np.int64)
    mask = np.array([[1, 1, 0, 0], [0, 0, 0, 0], [1, 0, 0, 0]])
    with pytest.raises(ValueError, match="no valid token"):
        pack_padded_batch(ids, ids * 0, mask)
