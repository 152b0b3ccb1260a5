"""torch-tensor front end of the C ABI (include/bert_b200.h).

torch is used only to own device memory and streams; every function forwards raw pointers to
libbert_b200.so. Names follow the reference free functions they replace
(embSkipLayerNorm, computeSkipLayerNorm, computeMaskIdx, convertMask, MHARunner::run, FC enqueue).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, lib

FP32, FP16, INT8 = 0, 1, 2
ACT_NONE, ACT_GELU_ERF = 0, 1

_TYPE_ID = {torch.float32: FP32, torch.float16: FP16, torch.int8: INT8}


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("tensorrt_b200 kernels need CUDA tensors; there is no CPU path")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return C.c_void_p(t.data_ptr())


def _stream():
    if not torch.cuda.is_available():
        raise ValueError("tensorrt_b200 kernels need a CUDA device; there is no CPU path")
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def skip_layer_norm(x, skip, gamma, beta, bias=None, out=None):
    """FP32/FP16 residual + bias + LayerNorm over the last dimension."""
    ld = x.shape[-1]
    out = torch.empty_like(x) if out is None else out
    check(lib.bert_b200_skip_layer_norm(_stream(), _TYPE_ID[x.dtype], ld, x.numel(), _ptr(x), _ptr(skip), _ptr(beta),
                                        _ptr(gamma), _ptr(out), _ptr(bias)), "skip_layer_norm")
    return out


def skip_layer_norm_dqq(x, skip, gamma, beta, bias, dq_in, dq_skip, q_scale, out=None):
    """INT8 in/out residual + bias + LayerNorm (linear layout); gamma/beta/bias FP16."""
    ld = x.shape[-1]
    out = torch.empty_like(x) if out is None else out
    check(lib.bert_b200_skip_layer_norm_dqq(_stream(), ld, x.numel(), _ptr(x), _ptr(skip), _ptr(beta), _ptr(gamma),
                                            _ptr(out), _ptr(bias), dq_in, dq_skip, q_scale), "skip_layer_norm_dqq")
    return out


def skip_layer_norm_interleaved(x, skip, gamma, beta, dq_in, dq_skip, q_scale, q_skip_scale=None):
    """INT8 CHW32 [ld/32, total, 32]; returns out, or (out, preln) when q_skip_scale is given (MTron)."""
    g, total, _ = x.shape
    ld = g * 32
    out = torch.empty_like(x)
    if q_skip_scale is None:
        check(lib.bert_b200_skip_layer_norm_interleaved_hface(_stream(), ld, total, _ptr(x), _ptr(skip), _ptr(beta),
                                                              _ptr(gamma), _ptr(out), dq_in, dq_skip, q_scale),
              "skip_layer_norm_interleaved_hface")
        return out
    preln = torch.empty_like(x)
    check(lib.bert_b200_skip_layer_norm_interleaved_mtron(_stream(), ld, total, _ptr(x), _ptr(skip), _ptr(beta),
                                                          _ptr(gamma), _ptr(out), _ptr(preln), dq_in, dq_skip, q_scale,
                                                          q_skip_scale), "skip_layer_norm_interleaved_mtron")
    return out, preln


def emb_layer_norm(input_ids, token_ids, word_emb, pos_emb, tok_emb, gamma, beta, q_scale=None, mask=None):
    """Fixed layout: ids [S, B] int32 -> [S, B, E]; optional fused INT8 copy when q_scale is given; with the [S, B] int32
    `mask` the same launch also returns the mask index [B] (last element of the result)."""
    S, B = input_ids.shape
    ld = word_emb.shape[1]
    out = torch.empty((S, B, ld), dtype=word_emb.dtype, device=word_emb.device)
    out_i8 = torch.empty((S, B, ld), dtype=torch.int8, device=word_emb.device) if q_scale is not None else None
    mask_idx = torch.empty((B,), dtype=torch.int32, device=word_emb.device) if mask is not None else None
    if mask is not None and (tuple(mask.shape) != (S, B) or mask.dtype != torch.int32 or not mask.is_contiguous()):
        raise ValueError("mask must be a contiguous int32 [S, B] tensor")
    check(lib.bert_b200_emb_layer_norm_mask_idx(_stream(), _TYPE_ID[word_emb.dtype], ld, B, S, _ptr(input_ids),
                                                _ptr(token_ids), _ptr(beta), _ptr(gamma), _ptr(word_emb), _ptr(pos_emb),
                                                _ptr(tok_emb), word_emb.shape[0], tok_emb.shape[0], pos_emb.shape[0],
                                                _ptr(out), _ptr(out_i8), q_scale or 0.0, _ptr(mask), _ptr(mask_idx)),
          "emb_layer_norm")
    res = [out]
    if q_scale is not None:
        res.append(out_i8)
    if mask is not None:
        res.append(mask_idx)
    return res[0] if len(res) == 1 else tuple(res)


def emb_layer_norm_var_seqlen(input_ids, token_ids, cu_seqlens, max_seqlen, word_emb, pos_emb, tok_emb, gamma, beta,
                              with_skip=False, q_scale=None):
    """Packed layout: ids [total] -> [total, E] (+ pre-LN sum when with_skip, + INT8 copy when q_scale)."""
    total = input_ids.shape[0]
    B = cu_seqlens.shape[0] - 1
    ld = word_emb.shape[1]
    out = torch.empty((total, ld), dtype=word_emb.dtype, device=word_emb.device)
    skip = torch.empty_like(out) if with_skip else None
    out_i8 = torch.empty((total, ld), dtype=torch.int8, device=word_emb.device) if q_scale is not None else None
    check(lib.bert_b200_emb_layer_norm_var_seqlen(_stream(), _TYPE_ID[word_emb.dtype], ld, B, max_seqlen, total,
                                                  _ptr(input_ids), _ptr(token_ids), _ptr(cu_seqlens), _ptr(beta),
                                                  _ptr(gamma), _ptr(word_emb), _ptr(pos_emb), _ptr(tok_emb),
                                                  word_emb.shape[0], tok_emb.shape[0], pos_emb.shape[0], _ptr(out), _ptr(skip),
                                                  _ptr(out_i8), q_scale or 0.0), "emb_layer_norm_var_seqlen")
    res = [out]
    if with_skip:
        res.append(skip)
    if q_scale is not None:
        res.append(out_i8)
    return res[0] if len(res) == 1 else tuple(res)


def compute_mask_idx(mask_sb):
    S, B = mask_sb.shape
    out = torch.empty((B,), dtype=torch.int32, device=mask_sb.device)
    check(lib.bert_b200_compute_mask_idx(_stream(), S, B, _ptr(mask_sb), _ptr(out)), "compute_mask_idx")
    return out


def convert_mask(mask_sb, warps_m, warps_n, warps_k=1):
    S, B = mask_sb.shape
    xm = (S + 16 * warps_m - 1) // (16 * warps_m)
    out = torch.empty((B, xm, warps_m * warps_n * warps_k * 32), dtype=torch.int32, device=mask_sb.device)
    check(lib.bert_b200_convert_mask(S, B, warps_m, warps_n, warps_k, _ptr(mask_sb), _ptr(out), _stream()),
          "convert_mask")
    return out


def packed_mask_to_lengths(packed, S, warps_m, warps_n):
    """packed: [B, words] int32/uint32 as written by convert_mask -> lengths [B] int32."""
    B = packed.shape[0]
    row_words = packed[0].numel()
    out = torch.empty((B,), dtype=torch.int32, device=packed.device)
    check(lib.bert_b200_packed_mask_to_lengths(_stream(), S, B, warps_m, warps_n, row_words, _ptr(packed), _ptr(out)),
          "packed_mask_to_lengths")
    return out


def lengths_to_cu_seqlens(lengths):
    B = lengths.shape[0]
    out = torch.empty((B + 1,), dtype=torch.int32, device=lengths.device)
    check(lib.bert_b200_lengths_to_cu_seqlens(_stream(), B, _ptr(lengths), _ptr(out)), "lengths_to_cu_seqlens")
    return out


def fc(a, wt, bias=None, activation=ACT_NONE, alpha=1.0, out_dtype=None, out_scale=1.0, status=None, out=None):
    """C[m, n] = epilogue(A[m, k] . Wt[n, k]); Wt is the [n, k] (transposed) weight."""
    m, k = a.shape
    n = wt.shape[0]
    out_dtype = a.dtype if out_dtype is None else out_dtype
    out = torch.empty((m, n), dtype=out_dtype, device=a.device) if out is None else out
    p = _lib.FcParams(_TYPE_ID[a.dtype], _TYPE_ID[out_dtype], m, n, k, _ptr(a), a.stride(0), _ptr(wt), _ptr(out),
                      out.stride(0), _ptr(bias), activation, alpha, out_scale, _ptr(status))
    check(lib.bert_b200_fc(C.byref(p), _stream()), "fc")
    return out


def attention_bnsd(q, k, v, kv_lengths=None, scale_bmm1=None, scale_softmax=1.0, scale_bmm2=1.0, status=None):
    """Fused attention on separate q, k, v of shape [B, N, S, d]; returns [B, N, S, d]."""
    B, N, S, d = q.shape
    out = torch.empty_like(q)
    if scale_bmm1 is None:
        scale_bmm1 = d ** -0.5
    p = _lib.AttentionBnsdParams(_TYPE_ID[q.dtype], B, S, N, d, _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(kv_lengths),
                                 scale_bmm1, scale_softmax, scale_bmm2, _ptr(status))
    check(lib.bert_b200_attention_bnsd(C.byref(p), _stream()), "attention_bnsd")
    return out


def mha(qkv, B, S, num_heads, head_size=64, cu_seqlens=None, mask_idx=None, scale_bmm1=None, scale_softmax=1.0,
        scale_bmm2=1.0, status=None, interleaved=False, workspace=None, use_workspace=True, out=None):
    """Fused attention. qkv: fixed [S, B, 3*N*d] (cu_seqlens None), packed [total, 3*N*d], or with
    interleaved=True the INT8 CHW32 form [3*N*d/32, total, 32] (output [N*d/32, total, 32]). `out`: a tensor of the
    output's shape and type to write into instead of a new one."""
    E = num_heads * head_size
    if interleaved:
        total = qkv.shape[1]
        shape = (E // 32, total, 32)
    elif cu_seqlens is None:
        shape = (S, B, E)
        total = 0
    else:
        total = qkv.shape[0]
        shape = (total, E)
    if out is None:
        out = torch.empty(shape, dtype=qkv.dtype, device=qkv.device)
    elif tuple(out.shape) != shape or out.dtype != qkv.dtype or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {qkv.dtype} tensor of shape {shape}")
    if scale_bmm1 is None:
        scale_bmm1 = head_size ** -0.5
    p = _lib.MhaParams(_TYPE_ID[qkv.dtype], B, S, num_heads, head_size, total, _ptr(qkv), _ptr(out), _ptr(cu_seqlens),
                       _ptr(mask_idx), 1 if interleaved else 0, scale_bmm1, scale_softmax, scale_bmm2, _ptr(status))
    if workspace is None and use_workspace:
        need = int(lib.bert_b200_mha_workspace_size(C.byref(p)))
        workspace = torch.empty(need, dtype=torch.uint8, device=qkv.device) if need > 0 else None
    if workspace is not None:
        p.workspace, p.workspace_bytes = _ptr(workspace), workspace.numel() * workspace.element_size()
    check(lib.bert_b200_mha(C.byref(p), _stream()), "mha")
    return out
