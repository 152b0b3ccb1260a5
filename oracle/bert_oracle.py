"""CPU restatement of the TensorRT-OSS BERT encoder plugin math (TEST INFRASTRUCTURE, not product).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this
module; the product path (tensorrt_b200/) never does and has no CPU fallback.

PARITY PINNED against outputs of the reference itself: the reference tree ships no golden I/O for these plugins
(the `*_PluginGoldenIO.json` / `*_PluginReference.py` files named by the plugin YAMLs are absent), so the reference's
own kernels - its SIMT LayerNorm / embedding / mask kernels compiled from source and the precompiled sm100 attention
kernels it ships - were run on a B200 (oracle/build_ref.py -> oracle/_ref/libref_bert.so, tests/golden/make_golden.py)
and their outputs are committed as tests/golden/reference_kernels.npz. tests/test_golden_cpu.py checks every function
below against them (index outputs and the INT8 attention output bit-exact, FP32 1e-5, FP16 1e-2, INT8 LayerNorm
+-1 LSB); tests/test_reference_pin_gpu.py repeats the comparison live on larger inputs. Each function restates the
reference's source-visible algorithm in NumPy (float64 statistics, exact integer accumulation) and cites the
file:line it follows. The FC plugin's cuBLASLt GEMM and the whole-encoder wiring have no reference output here.

Paths are relative to the TensorRT-OSS tree.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

# ------------------------------------------------------------------------------------------------
# quantisation helpers
# ------------------------------------------------------------------------------------------------


def quantize(x: np.ndarray, inv_scale: float) -> np.ndarray:
    """sat8(rni(x * inv_scale)): round-half-even, saturate to [-128, 127].

    ref: plugin/common/common.cuh:482-504 (float4_to_char4: cvt.rni.sat.s32.f32 + cvt.pack.sat.s8).
    The multiplication is done in float32 like the kernels do.
    """
    y = np.asarray(x, dtype=np.float32) * np.float32(inv_scale)
    return np.clip(np.rint(y), -128, 127).astype(np.int8)


def amax_scale(x: np.ndarray) -> float:
    """Per-tensor symmetric dequantisation step amax/127.

    ref: tools/pytorch-quantization/pytorch_quantization/tensor_quant.py:511-556 (scale = 127/amax).
    """
    a = float(np.max(np.abs(x)))
    return (a if a > 0 else 1.0) / 127.0


# ------------------------------------------------------------------------------------------------
# embedding + LayerNorm, mask helpers
# ------------------------------------------------------------------------------------------------


def _layer_norm_rows(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float) -> np.ndarray:
    x = x.astype(np.float64)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return gamma.astype(np.float64) * (x - mu) / np.sqrt(var + eps) + beta.astype(np.float64)


def emb_layer_norm(input_ids, token_ids, word_emb, pos_emb, tok_emb, gamma, beta):
    """Fixed-length embedding + LayerNorm. ids are [S, B]; returns float64 [S, B, E].

    x = word[id] + tok[seg] + pos[s]; y = gamma * (x - mean) * rsqrt(var) + beta  (no epsilon).
    ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:185-235, plugin/common/common.cuh:253-281.
    Ids outside a table: the reference leaves the row undefined; the product defines it as `beta`.
    """
    S, B = input_ids.shape
    ok = (input_ids >= 0) & (input_ids < word_emb.shape[0]) & (token_ids >= 0) & (token_ids < tok_emb.shape[0])
    wi = np.where(ok, input_ids, 0)
    ti = np.where(ok, token_ids, 0)
    x = word_emb[wi].astype(np.float64) + tok_emb[ti].astype(np.float64) + pos_emb[:S].astype(np.float64)[:, None, :]
    with np.errstate(invalid="ignore", divide="ignore"):
        y = _layer_norm_rows(x, gamma, beta, 0.0)
    y[~ok] = beta.astype(np.float64)
    return y


def emb_layer_norm_var_seqlen(input_ids, token_ids, cu_seqlens, word_emb, pos_emb, tok_emb, gamma, beta):
    """Packed embedding + LayerNorm: position = index inside the sequence. Returns (y, pre_ln) float64 [total, E].

    ref: plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernelHFace.cu:38-103 and ...KernelMTron.cu:38-104
    (the MTron variant also returns the un-normalised sum).
    """
    total = int(cu_seqlens[-1])
    pos = np.zeros(total, dtype=np.int64)
    for b in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        pos[lo:hi] = np.arange(hi - lo)
    ids = np.asarray(input_ids[:total])
    seg = np.asarray(token_ids[:total])
    ok = (ids >= 0) & (ids < word_emb.shape[0]) & (seg >= 0) & (seg < tok_emb.shape[0])
    x = (word_emb[np.where(ok, ids, 0)].astype(np.float64) + tok_emb[np.where(ok, seg, 0)].astype(np.float64)
         + pos_emb[pos].astype(np.float64))
    x[~ok] = 0.0
    with np.errstate(invalid="ignore", divide="ignore"):
        y = _layer_norm_rows(x, gamma, beta, 0.0)
    y[~ok] = beta.astype(np.float64)
    return y, x


def mask_idx(mask_sb: np.ndarray) -> np.ndarray:
    """Index of the first 0 in each column of the [S, B] mask, S if none.

    ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:98-183 (maskIdxKernel*, computeMaskIdx).
    """
    S, B = mask_sb.shape
    out = np.full(B, S, dtype=np.int32)
    for b in range(B):
        z = np.nonzero(mask_sb[:, b] == 0)[0]
        if z.size:
            out[b] = z[0]
    return out


def packed_mask(mask_sb: np.ndarray, warps_m: int, warps_n: int, warps_k: int = 1) -> np.ndarray:
    """Fragment-ownership bit mask of the reference fused attention kernels.

    Returns uint32 [B, xmmas_m, threads_per_cta]. Positions beyond S count as masked.
    ref: plugin/embLayerNormPlugin/embLayerNormKernel.cu:41-96 (fillSBSMaskKernel, convertMask).
    """
    S, B = mask_sb.shape
    xmmas_m = (S + 16 * warps_m - 1) // (16 * warps_m)
    xmmas_n = (S + 16 * warps_n - 1) // (16 * warps_n)
    threads = warps_m * warps_n * warps_k * 32
    out = np.zeros((B, xmmas_m, threads), dtype=np.uint32)
    padded = np.zeros((xmmas_n * 16 * warps_n + 16, B), dtype=np.int64)
    padded[:S] = mask_sb
    for b in range(B):
        m = (padded[:, b] == 1).astype(np.uint32)
        for t in range(threads):
            warp = t // 32
            warp_n = warp // warps_m
            col = warp_n * 16 + (t % 4) * 2
            bits = 0
            for ni in range(xmmas_n):
                off = ni * 16 * warps_n + col
                sel = (m[off], m[off + 1], m[off], m[off + 1], m[off + 8], m[off + 9], m[off + 8], m[off + 9])
                for k, v in enumerate(sel):
                    bits |= int(v) << (8 * ni + k)
            out[b, :, t] = bits
    return out


def cu_seqlens(lengths: np.ndarray) -> np.ndarray:
    """Exclusive prefix sum of the sequence lengths, int32 [B+1] (what the var-seqlen plugins take as input,
    plugin/embLayerNormPlugin/embLayerNormVarSeqlenPlugin.cpp:370-396)."""
    out = np.zeros(len(lengths) + 1, dtype=np.int64)
    np.cumsum(lengths, out=out[1:])
    return out.astype(np.int32)


# ------------------------------------------------------------------------------------------------
# skip + bias + LayerNorm
# ------------------------------------------------------------------------------------------------

EPS_F32 = float(np.finfo(np.float32).eps)


def skip_layer_norm(x, skip, gamma, beta, bias=None, eps=0.0):
    """y = gamma * (v - mean) * rsqrt(var + eps) + beta, v = x + skip (+ bias), rows along the last axis.

    ref: plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:108-161 (skipln_vec) and :163-217.
    eps: FP32 -> numeric_limits<float>::epsilon() (:149); FP16 -> 0 (numeric_limits<__half> is unspecialised).
    """
    v = x.astype(np.float64) + skip.astype(np.float64)
    if bias is not None:
        v = v + bias.astype(np.float64)
    return _layer_norm_rows(v, gamma, beta, eps)


def skip_layer_norm_dqq(x_i8, skip_i8, gamma, beta, bias, dq_in, dq_skip, q_scale, eps=0.0):
    """INT8 in / INT8 out: v = dq_in*x + dq_skip*skip (+bias); out = sat8(rni(LN(v) * q_scale)).

    ref: plugin/skipLayerNormPlugin/skipLayerNormKernel.cu:43-106 (skiplnDQQ). Returns (int8 out, float64 v).
    """
    v = np.float32(dq_in) * x_i8.astype(np.float32) + np.float32(dq_skip) * skip_i8.astype(np.float32)
    v = v.astype(np.float64)
    if bias is not None:
        v = v + bias.astype(np.float64)
    y = _layer_norm_rows(v, gamma, beta, eps)
    return quantize(y, q_scale), v


def to_chw32(x_tc: np.ndarray) -> np.ndarray:
    """[total, C] -> CHW32-interleaved [C/32, total, 32] (ref: include/NvInferRuntime.h:1464-1471;
    addressing in plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelHFace.cu:262-271)."""
    total, c = x_tc.shape
    assert c % 32 == 0
    return np.ascontiguousarray(x_tc.reshape(total, c // 32, 32).transpose(1, 0, 2))


def from_chw32(x: np.ndarray) -> np.ndarray:
    g, total, _ = x.shape
    return np.ascontiguousarray(x.transpose(1, 0, 2).reshape(total, g * 32))


def skip_layer_norm_interleaved(x_il, skip_il, gamma, beta, dq_in, dq_skip, q_scale, q_skip_scale=None):
    """CHW32 variants (HFace; MTron when q_skip_scale is given: also returns preln = sat8(rni(v*q_skip_scale))).

    ref: plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelHFace.cu:47-221, 261-332 and
    ...KernelMTron.cu:282-337. The large kernels add FP32 epsilon to the variance (HFace.cu:178).
    """
    out, v = skip_layer_norm_dqq(from_chw32(x_il), from_chw32(skip_il), gamma, beta, None, dq_in, dq_skip, q_scale, EPS_F32)
    if q_skip_scale is None:
        return to_chw32(out)
    return to_chw32(out), to_chw32(quantize(v, q_skip_scale))


# ------------------------------------------------------------------------------------------------
# fully connected
# ------------------------------------------------------------------------------------------------


def gelu_erf(x: np.ndarray) -> np.ndarray:
    """0.5 x (1 + erf(x / sqrt(2))) (the benchmark configurations' 'FFN 3072 with erf-GELU')."""
    from scipy.special import erf

    x = x.astype(np.float64)
    return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))


def fc(a: np.ndarray, w_kn: np.ndarray, bias=None, activation: str | None = None) -> np.ndarray:
    """out[m, o] = sum_k a[m, k] * W[k, o] (W not transposed, plugin/fcPlugin/README.md:16,45;
    plugin/fcPlugin/fcPlugin.cpp:551-610); optional bias / erf-GELU of the layers that follow it."""
    y = a.astype(np.float64) @ w_kn.astype(np.float64)
    if bias is not None:
        y = y + bias.astype(np.float64)
    if activation == "gelu":
        y = gelu_erf(y)
    return y


def fc_int8(a_i8, w_kn_i8, alpha, bias=None, activation=None, out_inv_scale=None):
    """INT8 x INT8 -> INT32 (exact), then float: acc*alpha + bias, activation, optional requantisation
    (benchmark configuration 3: 'int8 x int8 -> int32 with the fp32 scale epilogue')."""
    acc = a_i8.astype(np.float64) @ w_kn_i8.astype(np.float64)  # exact: |acc| < 2^53
    y = acc.astype(np.float32) * np.float32(alpha)
    y = y.astype(np.float64)
    if bias is not None:
        y = y + bias.astype(np.float64)
    if activation == "gelu":
        y = gelu_erf(y)
    if out_inv_scale is None:
        return y
    return quantize(y, out_inv_scale)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------


def _seq_views(qkv, B, S, N, d, cu=None):
    """Yields (b, rows, view[len_or_S, N, 3, d]) for the fixed [S,B,N,3,d] or packed [total,N,3,d] layout
    (ref: plugin/bertQKVToContextPlugin/README.md:26-30; mhaRunner.cu:550-552, 1006)."""
    if cu is None:
        q = qkv.reshape(S, B, N, 3, d)
        for b in range(B):
            yield b, q[:, b]
    else:
        q = qkv.reshape(-1, N, 3, d)
        for b in range(B):
            yield b, q[int(cu[b]):int(cu[b + 1])]


def mha(qkv, B, S, N, d, cu=None, lengths=None, scale=None):
    """O = softmax(Q K^T * scale over keys < len) V; float64.

    Fixed layout: every one of the S query rows attends to keys [0, len_b) and is written (like the
    unfused reference path, mhaRunner.cu:533-601 with the masked softmax of common.cuh:386-419);
    len 0 gives zero rows (common.cuh:343-363). Packed layout: sequence b has cu[b+1]-cu[b] rows.
    Returns [S,B,N*d] or [total,N*d].
    """
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = np.zeros((S, B, N * d) if cu is None else (qkv.reshape(-1, N, 3, d).shape[0], N * d), dtype=np.float64)
    for b, v in _seq_views(qkv.astype(np.float64), B, S, N, d, cu):
        rows = v.shape[0]
        ln = rows if cu is not None else (S if lengths is None else int(min(max(lengths[b], 0), S)))
        if rows == 0:
            continue
        if ln == 0:
            o = np.zeros((rows, N, d))
        else:
            q, k, val = v[:, :, 0], v[:ln, :, 1], v[:ln, :, 2]
            logits = np.einsum("qnd,knd->nqk", q, k) * scale
            logits -= logits.max(axis=-1, keepdims=True)
            p = np.exp(logits)
            p /= p.sum(axis=-1, keepdims=True)
            o = np.einsum("nqk,knd->qnd", p, val)
        if cu is None:
            out[:, b] = o.reshape(rows, N * d)
        else:
            out[int(cu[b]):int(cu[b + 1])] = o.reshape(rows, N * d)
    return out


def mha_int8(qkv_i8, B, S, N, d, scale_bmm1, scale_softmax, scale_bmm2, cu=None, lengths=None):
    """INT8 attention: logit = (q.k)_i32 * scale_bmm1; P_q = sat8(rni(softmax * scale_softmax));
    out = sat8(rni((P_q.v)_i32 * scale_bmm2)).

    ref: plugin/bertQKVToContextPlugin/mhaRunner.cu:1178-1190 and
    plugin/bertQKVToContextPlugin/qkvToContextInt8InterleavedPlugin.cpp:269-285 (scale algebra);
    the kernels themselves are precompiled, so the order of roundings inside them is not visible.
    """
    tot_rows = S * B if cu is None else qkv_i8.reshape(-1, N, 3, d).shape[0]
    out = np.zeros((S, B, N * d) if cu is None else (tot_rows, N * d), dtype=np.int8)
    for b, v in _seq_views(qkv_i8.astype(np.float64), B, S, N, d, cu):
        rows = v.shape[0]
        ln = rows if cu is not None else (S if lengths is None else int(min(max(lengths[b], 0), S)))
        if rows == 0:
            continue
        if ln == 0:
            o = np.zeros((rows, N, d), dtype=np.int8)
        else:
            q, k, val = v[:, :, 0], v[:ln, :, 1], v[:ln, :, 2]
            acc = np.einsum("qnd,knd->nqk", q, k)
            logits = acc.astype(np.float32).astype(np.float64) * np.float64(np.float32(scale_bmm1))
            logits -= logits.max(axis=-1, keepdims=True)
            p = np.exp(logits)
            p /= p.sum(axis=-1, keepdims=True)
            pq = quantize(p, scale_softmax).astype(np.float64)
            acc2 = np.einsum("nqk,knd->qnd", pq, val)
            o = quantize(acc2, scale_bmm2)
        if cu is None:
            out[:, b] = o.reshape(rows, N * d)
        else:
            out[int(cu[b]):int(cu[b + 1])] = o.reshape(rows, N * d)
    return out


# ------------------------------------------------------------------------------------------------
# whole encoder (packed layout), synthetic configurations
# ------------------------------------------------------------------------------------------------


@dataclass
class LayerParams:
    w_qkv: np.ndarray   # [E, 3E]  columns ordered [N][3][d]
    b_qkv: np.ndarray
    w_out: np.ndarray   # [E, E]
    b_out: np.ndarray
    ln1_gamma: np.ndarray
    ln1_beta: np.ndarray
    w_ffn1: np.ndarray  # [E, F]
    b_ffn1: np.ndarray
    w_ffn2: np.ndarray  # [F, E]
    b_ffn2: np.ndarray
    ln2_gamma: np.ndarray
    ln2_beta: np.ndarray
    scales: dict = field(default_factory=dict)  # INT8: dequantisation steps, filled by calibrate_int8


@dataclass
class BertParams:
    hidden: int
    heads: int
    ffn: int
    word_emb: np.ndarray
    pos_emb: np.ndarray
    tok_emb: np.ndarray
    emb_gamma: np.ndarray
    emb_beta: np.ndarray
    layers: list
    dq_probs: float = 1.0 / 127.0


def make_bert_params(rng, layers, hidden, heads, ffn, vocab=30522, max_pos=512, type_vocab=2) -> BertParams:
    """Weights ~N(0, 0.02), LN gamma 1+N(0,0.02), beta ~N(0,0.02); tables rounded to FP16 (the plugin stores
    the tables in the output type, plugin/embLayerNormPlugin/embLayerNormPlugin.cpp:63-67)."""
    def n(*shape):
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)

    def h(x):
        return x.astype(np.float16)

    ls = []
    for _ in range(layers):
        ls.append(LayerParams(
            w_qkv=h(n(hidden, 3 * hidden)), b_qkv=n(3 * hidden), w_out=h(n(hidden, hidden)), b_out=h(n(hidden)),
            ln1_gamma=h(1 + n(hidden)), ln1_beta=h(n(hidden)), w_ffn1=h(n(hidden, ffn)), b_ffn1=n(ffn),
            w_ffn2=h(n(ffn, hidden)), b_ffn2=h(n(hidden)), ln2_gamma=h(1 + n(hidden)), ln2_beta=h(n(hidden))))
    return BertParams(hidden, heads, ffn, h(n(vocab, hidden)), h(n(max_pos, hidden)), h(n(type_vocab, hidden)),
                      1 + n(hidden), n(hidden), ls)


def make_inputs(rng, B, S, vocab=30522, min_len=None, max_len=None):
    """Token ids uniform in [0, vocab); segment 0 before a random split, 1 after; lengths uniform in
    [min_len, max_len] (defaults: all S). Returns packed (ids, seg, lengths, cu)."""
    min_len = S if min_len is None else min_len
    max_len = S if max_len is None else max_len
    lengths = rng.integers(min_len, max_len + 1, size=B).astype(np.int32)
    cu = cu_seqlens(lengths)
    total = int(cu[-1])
    ids = rng.integers(0, vocab, size=total).astype(np.int32)
    seg = np.zeros(total, dtype=np.int32)
    for b in range(B):
        ln = int(lengths[b])
        split = int(rng.integers(1, max(2, ln)))
        seg[int(cu[b]) + split:int(cu[b + 1])] = 1
    return ids, seg, lengths, cu


def encoder_layer_fp(x, lp: LayerParams, B, S, N, cu, round_fp16=True):
    """One post-LN encoder layer on packed rows [total, E] in float64, rounding every stored tensor to FP16
    when round_fp16 (what an FP16 engine materialises between plugins)."""
    r = (lambda t: t.astype(np.float16).astype(np.float64)) if round_fp16 else (lambda t: t)
    E = x.shape[1]
    d = E // N
    qkv = r(fc(x, lp.w_qkv, lp.b_qkv))
    ctx = r(mha(qkv, B, S, N, d, cu=cu))
    ao = r(fc(ctx, lp.w_out))
    h1 = r(skip_layer_norm(ao, x, lp.ln1_gamma, lp.ln1_beta, lp.b_out))
    f1 = r(fc(h1, lp.w_ffn1, lp.b_ffn1, "gelu"))
    f2 = r(fc(f1, lp.w_ffn2))
    out = r(skip_layer_norm(f2, h1, lp.ln2_gamma, lp.ln2_beta, lp.b_ffn2))
    return out, dict(qkv=qkv, ctx=ctx, ao=ao, h1=h1, f1=f1, f2=f2)


def encoder_fp(p: BertParams, ids, seg, cu, S, round_fp16=True, return_all=False):
    B = len(cu) - 1
    x, _ = emb_layer_norm_var_seqlen(ids, seg, cu, p.word_emb, p.pos_emb, p.tok_emb, p.emb_gamma, p.emb_beta)
    if round_fp16:
        x = x.astype(np.float16).astype(np.float64)
    inter = []
    for lp in p.layers:
        x, t = encoder_layer_fp(x, lp, B, S, p.heads, cu, round_fp16)
        inter.append(t)
    return (x, inter) if return_all else x


def quantize_weights(p: BertParams):
    """Per-tensor symmetric INT8 weights (scale amax/127)."""
    for lp in p.layers:
        for name in ("w_qkv", "w_out", "w_ffn1", "w_ffn2"):
            w = getattr(lp, name).astype(np.float32)
            s = amax_scale(w)
            lp.scales["s_" + name] = s
            lp.scales["q_" + name] = quantize(w, 1.0 / s)


def calibrate_int8(p: BertParams, ids, seg, cu, S):
    """Sets every activation scale to amax/127 of the FP32 forward on one calibration batch
    (benchmark configuration 3). Layer l's input scale equals layer l-1's output scale."""
    quantize_weights(p)
    B = len(cu) - 1
    x, _ = emb_layer_norm_var_seqlen(ids, seg, cu, p.word_emb, p.pos_emb, p.tok_emb, p.emb_gamma, p.emb_beta)
    for lp in p.layers:
        lp.scales["s_in"] = amax_scale(x)
        x, t = encoder_layer_fp(x, lp, B, S, p.heads, cu, round_fp16=False)
        lp.scales.update(s_qkv=amax_scale(t["qkv"]), s_ctx=amax_scale(t["ctx"]), s_attn_out=amax_scale(t["ao"]),
                         s_ln1=amax_scale(t["h1"]), s_ffn1=amax_scale(t["f1"]), s_ffn2=amax_scale(t["f2"]),
                         s_out=amax_scale(x))


def encoder_layer_int8(x_i8, lp: LayerParams, B, S, N, cu, dq_probs):
    """Explicit-INT8 layer: INT8 tensors between all ops, exact integer contractions."""
    s = lp.scales
    E = x_i8.shape[1]
    d = E // N
    qkv = fc_int8(x_i8, s["q_w_qkv"], s["s_in"] * s["s_w_qkv"], lp.b_qkv, None, 1.0 / s["s_qkv"])
    ctx = mha_int8(qkv, B, S, N, d, np.float32(s["s_qkv"]) * np.float32(s["s_qkv"]) * np.float32(1.0 / math.sqrt(d)),
                   1.0 / dq_probs, dq_probs * s["s_qkv"] / s["s_ctx"], cu=cu)
    ao = fc_int8(ctx, s["q_w_out"], s["s_ctx"] * s["s_w_out"], None, None, 1.0 / s["s_attn_out"])
    h1, _ = skip_layer_norm_dqq(ao, x_i8, lp.ln1_gamma, lp.ln1_beta, lp.b_out, s["s_attn_out"], s["s_in"], 1.0 / s["s_ln1"])
    f1 = fc_int8(h1, s["q_w_ffn1"], s["s_ln1"] * s["s_w_ffn1"], lp.b_ffn1, "gelu", 1.0 / s["s_ffn1"])
    f2 = fc_int8(f1, s["q_w_ffn2"], s["s_ffn1"] * s["s_w_ffn2"], None, None, 1.0 / s["s_ffn2"])
    out, _ = skip_layer_norm_dqq(f2, h1, lp.ln2_gamma, lp.ln2_beta, lp.b_ffn2, s["s_ffn2"], s["s_ln1"], 1.0 / s["s_out"])
    return out, dict(qkv=qkv, ctx=ctx, ao=ao, h1=h1, f1=f1, f2=f2)


def encoder_int8(p: BertParams, ids, seg, cu, S, return_all=False):
    B = len(cu) - 1
    x, _ = emb_layer_norm_var_seqlen(ids, seg, cu, p.word_emb, p.pos_emb, p.tok_emb, p.emb_gamma, p.emb_beta)
    x_i8 = quantize(x, 1.0 / p.layers[0].scales["s_in"])
    inter = []
    for lp in p.layers:
        x_i8, t = encoder_layer_int8(x_i8, lp, B, S, p.heads, cu, p.dq_probs)
        inter.append(t)
    out = x_i8.astype(np.float64) * p.layers[-1].scales["s_out"]
    return (out, x_i8, inter) if return_all else out


# ------------------------------------------------------------------------------------------------
# tolerance checks (Polygraphy semantics)
# ------------------------------------------------------------------------------------------------


def close_abs_or_rel(out, ref, atol, rtol):
    """Element passes if |out-ref| <= atol OR |out-ref|/|ref| <= rtol
    (ref: tools/Polygraphy/polygraphy/comparator/compare.py:477-509). Returns (ok, worst_abs, n_bad)."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = np.abs(out - ref)
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = diff / np.abs(ref)
    bad = ~((diff <= atol) | (rel <= rtol))
    bad |= ~np.isfinite(out)
    return (not bad.any()), float(diff.max() if diff.size else 0.0), int(bad.sum())


def int8_within_lsb(out_i8, ref_i8, lsb=1):
    d = np.abs(out_i8.astype(np.int32) - ref_i8.astype(np.int32))
    return bool((d <= lsb).all()), int(d.max() if d.size else 0), int((d > lsb).sum())
