"""End to end against an independent implementation: a randomly initialised Hugging Face BertModel (FP32, CPU) and
this library's encoder built from its state dict (tensorrt_b200/checkpoint.py), FP16 and INT8."""
import numpy as np
import pytest
import torch

from tests.test_checkpoint_cpu import make_hf, padded_batch

pytestmark = pytest.mark.gpu


# head sizes 64, 32 and 48 (the tiles are 64 channels wide; smaller heads are zero-filled by the TMA unit)
@pytest.mark.parametrize("hidden,heads", [(256, 4), (256, 8), (192, 4)])
def test_encoder_from_checkpoint_matches_huggingface(cuda, hidden, heads):
    import tensorrt_b200 as T
    from tensorrt_b200 import synthetic
    from tensorrt_b200.checkpoint import pack_padded_batch, params_from_bert_state_dict

    model = make_hf(layers=3, hidden=hidden, heads=heads, ffn=1024, vocab=800, max_pos=128)
    rng = np.random.default_rng(1)
    B, S = 6, 128
    ids, seg, mask, lengths = padded_batch(rng, B, S, 800)
    with torch.no_grad():
        want = model(input_ids=torch.from_numpy(ids), token_type_ids=torch.from_numpy(seg),
                     attention_mask=torch.from_numpy(mask)).last_hidden_state.numpy()
    want = np.concatenate([want[b, :lengths[b]] for b in range(B)])
    p = params_from_bert_state_dict(model.state_dict(), num_heads=heads)
    pid, pseg, cu = pack_padded_batch(ids, seg, mask)
    dev = lambda a: torch.from_numpy(a).to(cuda)
    enc = T.BertEncoder(p, T.FP16, cuda)
    got = enc.forward(dev(pid), dev(pseg), dev(cu), S).float().cpu().numpy()
    err = np.abs(got - want)
    # FP16 storage of every activation through three layers; outputs are O(1) after the final LayerNorm
    assert err.max() < 5e-2 and err.mean() < 4e-3, (err.max(), err.mean())
    # INT8 with max calibration on the same batch: statistical agreement (per-tensor 8-bit activations)
    amax = enc.calibrate(dev(pid), dev(pseg), dev(cu), S)
    for lp in p.layers:  # the scale assignment works on torch tensors
        for name in ("w_qkv", "w_out", "w_ffn1", "w_ffn2"):
            setattr(lp, name, torch.from_numpy(getattr(lp, name)))
    synthetic.assign_int8_scales(p, amax)
    enc8 = T.BertEncoder(p, T.INT8, cuda)
    got8 = enc8.forward(dev(pid), dev(pseg), dev(cu), S).float().cpu().numpy()
    cos = float((got8 * want).sum() / np.sqrt((got8 ** 2).sum() * (want ** 2).sum()))
    assert cos > 0.98, cos
    enc.close()
    enc8.close()


def test_question_answering_head_matches_huggingface(cuda):
    """BertForQuestionAnswering end to end: encoder + span head against Hugging Face on the valid tokens."""
    import transformers

    import tensorrt_b200 as T
    from tensorrt_b200.checkpoint import QaHead, pack_padded_batch, params_from_bert_state_dict

    torch.manual_seed(3)
    cfg = transformers.BertConfig(vocab_size=600, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                                  intermediate_size=1024, max_position_embeddings=128, hidden_act="gelu",
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = transformers.BertForQuestionAnswering(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():
            p.copy_((p + 0.05 * torch.randn_like(p)).half().float())
    rng = np.random.default_rng(4)
    B, S = 4, 96
    ids, seg, mask, lengths = padded_batch(rng, B, S, 600)
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(ids), token_type_ids=torch.from_numpy(seg), attention_mask=torch.from_numpy(mask))
    want = torch.stack([out.start_logits, out.end_logits], dim=-1).numpy()
    want = np.concatenate([want[b, :lengths[b]] for b in range(B)])
    sd = model.state_dict()
    p = params_from_bert_state_dict(sd, num_heads=4)
    pid, pseg, cu = pack_padded_batch(ids, seg, mask)
    dev = lambda a: torch.from_numpy(a).to(cuda)
    enc = T.BertEncoder(p, T.FP16, cuda)
    hidden = enc.forward(dev(pid), dev(pseg), dev(cu), S)
    got = QaHead(sd, cuda)(hidden).float().cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 5e-2, np.abs(got - want).max()
    enc.close()


def test_pooler_head_matches_huggingface(cuda):
    """BertModel.pooler_output: encoder + pooler (first token of every packed sequence) against Hugging Face."""
    import tensorrt_b200 as T
    from tensorrt_b200.checkpoint import PoolerHead, pack_padded_batch, params_from_bert_state_dict

    model = make_hf(layers=2, hidden=256, heads=4, ffn=1024, vocab=700, max_pos=128, pooler=True)
    rng = np.random.default_rng(9)
    B, S = 5, 64
    ids, seg, mask, lengths = padded_batch(rng, B, S, 700)
    with torch.no_grad():
        want = model(input_ids=torch.from_numpy(ids), token_type_ids=torch.from_numpy(seg),
                     attention_mask=torch.from_numpy(mask)).pooler_output.numpy()
    sd = model.state_dict()
    p = params_from_bert_state_dict(sd, num_heads=4)
    pid, pseg, cu = pack_padded_batch(ids, seg, mask)
    dev = lambda a: torch.from_numpy(a).to(cuda)
    enc = T.BertEncoder(p, T.FP16, cuda)
    cu_dev = dev(cu)
    hidden = enc.forward(dev(pid), dev(pseg), cu_dev, S)
    got = PoolerHead(sd, cuda)(hidden, cu_dev).float().cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 3e-2, np.abs(got - want).max()
    enc.close()
