"""BERT checkpoint -> encoder parameters.

Takes a state dict in the Hugging Face `BertModel` naming (`embeddings.word_embeddings.weight`,
`encoder.layer.{i}.attention.self.query.weight`, ...; an optional leading `bert.` is stripped) and packs it the way
the plugins expect it: FC weights as [in, out] (the checkpoint stores [out, in]), and the three attention projections
of a layer fused into one [E, 3E] matrix whose output channels are ordered [head][q | k | v][d]
(ref: plugin/bertQKVToContextPlugin/README.md:26-30). The result has the attributes `BertEncoder` reads
(`synthetic.make_params` builds the same object from random numbers).

This is the step the removed `demo/BERT` builder performed before it wired the plugins into a network; the wiring
itself is `BertEncoder` / `bert_b200_encoder_forward`.
"""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np


def _np(a) -> np.ndarray:
    if hasattr(a, "detach"):
        a = a.detach().cpu().float().numpy()
    return np.asarray(a, dtype=np.float32)


def params_from_bert_state_dict(state_dict, num_heads: int) -> SimpleNamespace:
    sd = {}
    for k, v in state_dict.items():
        k = k[5:] if k.startswith("bert.") else k
        sd[k] = v
    get = lambda name: _np(sd[name])
    word = get("embeddings.word_embeddings.weight")
    hidden = word.shape[1]
    if hidden % num_heads:
        raise ValueError(f"hidden size {hidden} is not a multiple of num_heads {num_heads}")
    d = hidden // num_heads
    layers = []
    i = 0
    while f"encoder.layer.{i}.attention.self.query.weight" in sd:
        p = f"encoder.layer.{i}."
        # checkpoint [out, in] -> [in, out]; output channels regrouped per head as (q, k, v)
        q, k, v = (get(p + f"attention.self.{n}.weight").T.reshape(hidden, num_heads, d) for n in ("query", "key", "value"))
        bq, bk, bv = (get(p + f"attention.self.{n}.bias").reshape(num_heads, d) for n in ("query", "key", "value"))
        w_qkv = np.stack([q, k, v], axis=2).reshape(hidden, 3 * hidden)
        b_qkv = np.stack([bq, bk, bv], axis=1).reshape(3 * hidden)
        h16 = lambda a: np.ascontiguousarray(a).astype(np.float16)
        layers.append(SimpleNamespace(
            w_qkv=h16(w_qkv), b_qkv=b_qkv.astype(np.float32),
            w_out=h16(get(p + "attention.output.dense.weight").T), b_out=h16(get(p + "attention.output.dense.bias")),
            ln1_gamma=h16(get(p + "attention.output.LayerNorm.weight")), ln1_beta=h16(get(p + "attention.output.LayerNorm.bias")),
            w_ffn1=h16(get(p + "intermediate.dense.weight").T), b_ffn1=get(p + "intermediate.dense.bias"),
            w_ffn2=h16(get(p + "output.dense.weight").T), b_ffn2=h16(get(p + "output.dense.bias")),
            ln2_gamma=h16(get(p + "output.LayerNorm.weight")), ln2_beta=h16(get(p + "output.LayerNorm.bias")), scales={}))
        i += 1
    if not layers:
        raise ValueError("no encoder.layer.* entries in the state dict")
    ffn = layers[0].w_ffn1.shape[1]
    return SimpleNamespace(
        hidden=hidden, heads=num_heads, ffn=ffn, word_emb=word.astype(np.float16),
        pos_emb=get("embeddings.position_embeddings.weight").astype(np.float16),
        tok_emb=get("embeddings.token_type_embeddings.weight").astype(np.float16),
        emb_gamma=get("embeddings.LayerNorm.weight"), emb_beta=get("embeddings.LayerNorm.bias"), layers=layers,
        dq_probs=1.0 / 127.0)


def pack_padded_batch(input_ids, token_type_ids, attention_mask):
    """[B, S] padded arrays (mask 1 = valid, valid tokens first) -> packed (ids, segment ids, cu_seqlens) int32."""
    ids, seg, mask = (np.asarray(a) for a in (input_ids, token_type_ids, attention_mask))
    lengths = mask.astype(np.int64).sum(axis=1)
    if (lengths == 0).any():
        raise ValueError("pack_padded_batch: sequence(s) %s have no valid token; drop them before packing (an empty "
                         "sequence has no [CLS] row for the heads to read)" % np.nonzero(lengths == 0)[0].tolist())
    cu = np.zeros(len(lengths) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(lengths)
    pid = np.concatenate([ids[b, :lengths[b]] for b in range(len(lengths))]).astype(np.int32)
    pseg = np.concatenate([seg[b, :lengths[b]] for b in range(len(lengths))]).astype(np.int32)
    return pid, pseg, cu


class QaHead:
    """The span-prediction head of `BertForQuestionAnswering` (`qa_outputs`: hidden -> start / end logits) on top of
    the encoder output, run through the FC kernel. The two output channels are padded to 16 (the kernel's granularity);
    the padding rows are zero and dropped from the result."""

    def __init__(self, state_dict, device="cuda:0"):
        import torch

        w = _np(state_dict["qa_outputs.weight"])  # [2, hidden]
        b = _np(state_dict["qa_outputs.bias"])
        wt = np.zeros((16, w.shape[1]), dtype=np.float16)
        wt[:2] = w.astype(np.float16)
        bias = np.zeros(16, dtype=np.float32)
        bias[:2] = b
        self.wt = torch.from_numpy(wt).to(device)      # already [out, in], the layout the FC kernel reads
        self.bias = torch.from_numpy(bias).to(device)

    def __call__(self, hidden):
        """hidden: FP16 [total, hidden] (packed tokens) -> FP16 [total, 2] (start logit, end logit)."""
        from . import ops

        return ops.fc(hidden, self.wt, bias=self.bias)[:, :2]


class PoolerHead:
    """The pooler of `BertModel` (`pooler.dense` + tanh on the first token of every sequence) on top of the packed
    encoder output: the [CLS] rows are gathered with `cu_seqlens`, the dense layer runs through the FC kernel; the tanh
    of the B x hidden result is left to torch (the FC plugin has no tanh epilogue, neither has the reference's)."""

    def __init__(self, state_dict, device="cuda:0", prefix=""):
        import torch

        w = _np(state_dict[prefix + "pooler.dense.weight"])  # [hidden, hidden] = [out, in]
        b = _np(state_dict[prefix + "pooler.dense.bias"])
        self.wt = torch.from_numpy(np.ascontiguousarray(w.astype(np.float16))).to(device)
        self.bias = torch.from_numpy(b.astype(np.float32)).to(device)

    def __call__(self, hidden, cu_seqlens):
        """hidden: FP16 [total, hidden]; cu_seqlens: int32 [B + 1] -> FP16 [B, hidden]."""
        import torch

        from . import ops

        starts = cu_seqlens[:-1].long()
        if bool((cu_seqlens[1:].long() <= starts).any()):
            raise ValueError("PoolerHead: every sequence needs at least one token (its first row is the [CLS] row)")
        first = hidden.index_select(0, starts).contiguous()
        return torch.tanh(ops.fc(first, self.wt, bias=self.bias).float()).half()
