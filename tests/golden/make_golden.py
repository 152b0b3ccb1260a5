"""Generates tests/golden/reference_kernels.npz: small known-answer vectors produced by the REFERENCE's own kernels
(oracle/_ref/libref_bert.so, built by oracle/build_ref.py from the TensorRT-OSS sources) on a B200.

    python tests/golden/make_golden.py [output.npz]

Needs a GPU and the built reference library. The committed .npz is what tests/test_golden_cpu.py checks the CPU
oracle against on every run; tests/test_reference_pin_gpu.py repeats the comparison live on larger random inputs.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import bert_oracle as O  # noqa: E402
from oracle.ref_lib import RefLib  # noqa: E402


def main(out_path):
    ref = RefLib()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(2026)
    g = {}
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    # SkipLayerNorm FP16 (ld 768, bias) and FP32 (ld 128): shapes of the reference's own plugin configuration
    for name, dt, ld, rows in (("skipln_f16", np.float16, 768, 4), ("skipln_f32", np.float32, 128, 3)):
        x, s = rng.standard_normal((rows, ld)).astype(dt), rng.standard_normal((rows, ld)).astype(dt)
        gam, bet, bia = (1 + 0.1 * rng.standard_normal(ld)).astype(dt), (0.1 * rng.standard_normal(ld)).astype(dt), (0.1 * rng.standard_normal(ld)).astype(dt)
        y = ref.skip_layer_norm(t(x), t(s), t(gam), t(bet), t(bia)).cpu().numpy()
        g.update({f"{name}_x": x, f"{name}_skip": s, f"{name}_gamma": gam, f"{name}_beta": bet, f"{name}_bias": bia, f"{name}_out": y})

    # INT8 SkipLayerNorm, linear (bias) and CHW32-interleaved (small / large kernels, HFace / MTron)
    ld, rows = 768, 6
    x = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
    s = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
    gam, bet, bia = (1 + 0.1 * rng.standard_normal(ld)).astype(np.float16), (0.1 * rng.standard_normal(ld)).astype(np.float16), (0.1 * rng.standard_normal(ld)).astype(np.float16)
    scales = np.array([0.021, 0.017, 1 / 0.03, 1 / 0.04], dtype=np.float32)
    g.update(dqq_x=x, dqq_skip=s, dqq_gamma=gam, dqq_beta=bet, dqq_bias=bia, dqq_scales=scales)
    g["dqq_out"] = ref.skip_layer_norm_dqq(t(x), t(s), t(gam), t(bet), t(bia), *map(float, scales[:3])).cpu().numpy()
    xi, si = O.to_chw32(x), O.to_chw32(s)
    for variant, nm in ((0, "small_hface"), (1, "large_hface"), (2, "small_mtron"), (3, "large_mtron")):
        out, pre = ref.skip_layer_norm_interleaved(variant, t(xi), t(si), t(gam), t(bet), *map(float, scales))
        g[f"il_{nm}_out"] = out.cpu().numpy()
        if variant >= 2:
            g[f"il_{nm}_preln"] = pre.cpu().numpy()

    # Embedding + LayerNorm: FP32 100 x 128 vocabulary, 20 positions (the reference configuration), and FP16 packed
    E, vocab, S, B = 128, 100, 6, 2
    word, pos, tok = (rng.standard_normal((n, E)).astype(np.float32) for n in (vocab, 20, 2))
    gam, bet = (1 + 0.1 * rng.standard_normal(E)).astype(np.float32), (0.1 * rng.standard_normal(E)).astype(np.float32)
    ids, seg = rng.integers(0, vocab, size=(S, B)).astype(np.int32), rng.integers(0, 2, size=(S, B)).astype(np.int32)
    g.update(emb_word=word, emb_pos=pos, emb_tok=tok, emb_gamma=gam, emb_beta=bet, emb_ids=ids, emb_seg=seg)
    g["emb_f32_out"] = ref.emb_layer_norm(t(ids), t(seg), t(word), t(pos), t(tok), t(gam), t(bet)).cpu().numpy()
    lengths = np.array([5, 1, 9], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    pids = rng.integers(0, vocab, size=int(cu[-1])).astype(np.int32)
    pseg = rng.integers(0, 2, size=int(cu[-1])).astype(np.int32)
    h = lambda a: a.astype(np.float16)
    out, skip = ref.emb_layer_norm_var_seqlen(t(pids), t(pseg), t(cu), 16, t(h(word)), t(h(pos)), t(h(tok)), t(gam), t(bet), mtron=True)
    out_h, _ = ref.emb_layer_norm_var_seqlen(t(pids), t(pseg), t(cu), 16, t(h(word)), t(h(pos)), t(h(tok)), t(gam), t(bet), mtron=False)
    g.update(embv_ids=pids, embv_seg=pseg, embv_cu=cu, embv_mtron_out=out.cpu().numpy(), embv_mtron_skip=skip.cpu().numpy(),
             embv_hface_out=out_h.cpu().numpy())

    # mask index and packed mask
    for S_, wm, wn in ((128, 2, 2), (384, 1, 8)):
        ln = np.array([S_, 37, 1], dtype=np.int32)
        mask = (np.arange(S_)[:, None] < ln[None, :]).astype(np.int32)
        g[f"mask{S_}"] = mask
        g[f"mask{S_}_idx"] = ref.compute_mask_idx(t(mask)).cpu().numpy()
        g[f"mask{S_}_packed"] = ref.convert_mask(t(mask), wm, wn).cpu().numpy()

    # attention: the reference's precompiled sm100 kernels, S bucket 64, one head of 64
    N, d, S_ = 1, 64, 64
    lengths = np.array([64, 17], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    xq = rng.standard_normal((total, 3 * N * d))
    q16 = xq.astype(np.float16)
    g.update(mha_cu=cu, mha_qkv_f16=q16)
    g["mha_f16_out"] = ref.fmha_v2(t(q16), t(cu), len(lengths), S_, N, d).cpu().numpy()
    s_qkv = O.amax_scale(xq)
    q8 = O.quantize(xq, 1.0 / s_qkv)
    s1 = float(np.float32(s_qkv) * np.float32(s_qkv) * np.float32(0.125))
    s2 = float((1.0 / 127.0) * s_qkv / (0.5 * s_qkv))
    g.update(mha_qkv_i8=q8, mha_i8_scales=np.array([s1, 127.0, s2], dtype=np.float32))
    g["mha_i8_out"] = ref.fmha_v2(t(q8), t(cu), len(lengths), S_, N, d, scales=(s1, 127.0, s2)).cpu().numpy()
    il = np.ascontiguousarray(q8.reshape(total, N, 3, 2, 32).transpose(2, 1, 3, 0, 4)).reshape(3 * N * 2, total, 32)
    oil = ref.fmha_v2(t(il), t(cu), len(lengths), S_, N, d, scales=(s1, 127.0, s2), interleaved=True).cpu().numpy()
    g["mha_il_i8_out"] = oil.reshape(N, 2, total, 32).transpose(2, 0, 1, 3).reshape(total, N * d)

    np.savez_compressed(out_path, **g)
    print("wrote", out_path, os.path.getsize(out_path), "bytes,", len(g), "arrays")

    # a file of its own (the arrays above stay byte-identical): the fixed-length kernels of plugin versions 1-3, S = 128,
    # one head of 64, input mask packed by the reference's convertMask
    rng = np.random.default_rng(20250101)
    f = {}
    N, d, S_ = 1, 64, 128
    lengths = np.array([128, 45], dtype=np.int32)
    B = len(lengths)
    mask = (np.arange(S_)[:, None] < lengths[None, :]).astype(np.int32)
    xq = rng.standard_normal((S_, B, 3 * N * d))
    q16 = xq.astype(np.float16)
    s_qkv = O.amax_scale(xq)
    q8 = O.quantize(xq, 1.0 / s_qkv)
    s1 = float(np.float32(s_qkv) * np.float32(s_qkv) * np.float32(0.125))
    s2 = float((1.0 / 127.0) * s_qkv / (0.5 * s_qkv))
    f.update(lengths=lengths, qkv_f16=q16, qkv_i8=q8, i8_scales=np.array([s1, 127.0, s2], dtype=np.float32))
    f["f16_out"] = ref.fmha_v1(t(q16), t(mask), N, d).cpu().numpy()
    f["i8_out"] = ref.fmha_v1(t(q8), t(mask), N, d, scales=(s1, 127.0, s2)).cpu().numpy()
    fixed_path = os.path.join(os.path.dirname(out_path), "reference_kernels_fixed_length.npz")
    np.savez_compressed(fixed_path, **f)
    print("wrote", fixed_path, os.path.getsize(fixed_path), "bytes,", len(f), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz"))
