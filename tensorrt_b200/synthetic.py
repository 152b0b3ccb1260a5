"""Seeded synthetic BERT weights / inputs on the device and INT8 scale assignment from calibration maxima.

Distributions follow the benchmark configurations: weights and biases ~N(0, 0.02), LayerNorm gamma 1 + N(0, 0.02),
beta ~N(0, 0.02); token ids uniform over the vocabulary; segment id 0 before a random split point, 1 after.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

AMAX_SLOTS = ("s_in", "s_qkv", "s_ctx", "s_attn_out", "s_ln1", "s_ffn1", "s_ffn2", "s_out")


def make_params(layers, hidden, heads, ffn, vocab=30522, max_pos=512, type_vocab=2, seed=0, device="cuda:0"):
    g = torch.Generator(device=device).manual_seed(seed)

    def n(*shape):
        return torch.randn(shape, device=device, generator=g) * 0.02

    ls = []
    for _ in range(layers):
        ls.append(SimpleNamespace(
            w_qkv=n(hidden, 3 * hidden).half(), b_qkv=n(3 * hidden), w_out=n(hidden, hidden).half(), b_out=n(hidden).half(),
            ln1_gamma=(1 + n(hidden)).half(), ln1_beta=n(hidden).half(), w_ffn1=n(hidden, ffn).half(), b_ffn1=n(ffn),
            w_ffn2=n(ffn, hidden).half(), b_ffn2=n(hidden).half(), ln2_gamma=(1 + n(hidden)).half(),
            ln2_beta=n(hidden).half(), scales={}))
    return SimpleNamespace(hidden=hidden, heads=heads, ffn=ffn, word_emb=n(vocab, hidden).half(),
                           pos_emb=n(max_pos, hidden).half(), tok_emb=n(type_vocab, hidden).half(),
                           emb_gamma=1 + n(hidden), emb_beta=n(hidden), layers=ls, dq_probs=1.0 / 127.0)


def make_inputs(batch, seqlen, vocab=30522, seed=0, min_len=None, device="cuda:0"):
    """Packed (ids, segment ids, cu_seqlens, lengths); lengths uniform in [min_len, seqlen] (all seqlen if None)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    if min_len is None:
        lengths = torch.full((batch,), seqlen, dtype=torch.int32)
    else:
        lengths = torch.randint(min_len, seqlen + 1, (batch,), generator=g, dtype=torch.int32)
    cu = torch.zeros(batch + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lengths, 0)
    total = int(cu[-1])
    ids = torch.randint(0, vocab, (total,), generator=g, dtype=torch.int32)
    seg = torch.zeros(total, dtype=torch.int32)
    for b in range(batch):
        ln = int(lengths[b])
        split = int(torch.randint(1, max(2, ln), (1,), generator=g))
        seg[int(cu[b]) + split:int(cu[b + 1])] = 1
    return ids.to(device), seg.to(device), cu.to(device), lengths


def assign_int8_scales(params, amax):
    """Per-tensor symmetric scales: activations amax/127 from `amax` [layers, 8] (BertEncoder.calibrate), weights
    amax/127 of each matrix; adds the INT8 weights q_w_* = clamp(rni(w / s), -127, 127)."""
    for li, lp in enumerate(params.layers):
        for si, name in enumerate(AMAX_SLOTS):
            a = float(amax[li][si])
            lp.scales[name] = (a if a > 0 else 1.0) / 127.0
        for name in ("w_qkv", "w_out", "w_ffn1", "w_ffn2"):
            w = getattr(lp, name).float()
            s = float(w.abs().max()) / 127.0 or 1.0 / 127.0
            lp.scales["s_" + name] = s
            lp.scales["q_" + name] = torch.clamp(torch.round(w / s), -127, 127).to(torch.int8)
    # a layer consumes exactly what the previous one produced
    for li in range(1, len(params.layers)):
        params.layers[li].scales["s_in"] = params.layers[li - 1].scales["s_out"]
    return params
