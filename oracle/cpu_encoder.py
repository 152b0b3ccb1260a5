"""FP32 PyTorch-CPU restatement of the BERT encoder forward (TEST / CPU-BASELINE INFRASTRUCTURE, not product).

Same operator order and math as oracle/bert_oracle.py (which cites the reference files), written with torch
CPU tensor ops so that it can use every host core; bench.py times it as the CPU baseline ("port": the reference
itself has no CPU implementation of this path, and ONNX-Runtime / Polygraphy are not installed).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def random_params(layers, hidden, heads, ffn, vocab=30522, max_pos=512, type_vocab=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(s, generator=g) * 0.02
    ls = [dict(w_qkv=n(hidden, 3 * hidden), b_qkv=n(3 * hidden), w_out=n(hidden, hidden), b_out=n(hidden),
               ln1_gamma=1 + n(hidden), ln1_beta=n(hidden), w_ffn1=n(hidden, ffn), b_ffn1=n(ffn), w_ffn2=n(ffn, hidden),
               b_ffn2=n(hidden), ln2_gamma=1 + n(hidden), ln2_beta=n(hidden)) for _ in range(layers)]
    return dict(hidden=hidden, heads=heads, word_emb=n(vocab, hidden), pos_emb=n(max_pos, hidden),
                tok_emb=n(type_vocab, hidden), emb_gamma=1 + n(hidden), emb_beta=n(hidden), layers=ls)


@torch.no_grad()
def forward(p, ids, seg, batch, seqlen):
    """ids/seg int64 [batch, seqlen] (all sequences full length). Returns FP32 [batch, seqlen, E]."""
    E, N = p["hidden"], p["heads"]
    d = E // N
    x = p["word_emb"][ids] + p["tok_emb"][seg] + p["pos_emb"][:seqlen][None]
    x = F.layer_norm(x, (E,), p["emb_gamma"], p["emb_beta"], eps=0.0)
    for l in p["layers"]:
        qkv = x @ l["w_qkv"] + l["b_qkv"]                       # columns ordered [N][3][d]
        qkv = qkv.view(batch, seqlen, N, 3, d)
        q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
        att = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(d), dim=-1)
        ctx = (att @ v).transpose(1, 2).reshape(batch, seqlen, E)
        h1 = F.layer_norm(ctx @ l["w_out"] + l["b_out"] + x, (E,), l["ln1_gamma"], l["ln1_beta"], eps=0.0)
        f1 = F.gelu(h1 @ l["w_ffn1"] + l["b_ffn1"])             # erf form
        x = F.layer_norm(f1 @ l["w_ffn2"] + l["b_ffn2"] + h1, (E,), l["ln2_gamma"], l["ln2_beta"], eps=0.0)
    return x
