"""Live three-way comparison on a B200: the reference's own kernels (oracle/_ref/libref_bert.so, compiled from the
TensorRT-OSS sources by oracle/build_ref.py; its attention kernels are the precompiled sm100 binaries the reference
ships) vs the CPU oracle vs the product kernels, on random inputs larger than the committed golden vectors."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O
from oracle import ref_lib

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref/libref_bert.so not built "
                                                  "(needs the reference tree: python oracle/build_ref.py)")]


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.fixture(scope="module")
def ref():
    return ref_lib.RefLib()


@pytest.mark.parametrize("ld", [768, 1024, 4096, 128])
def test_skip_ln_fp16_three_way(cuda, ref, ld):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld)
    rows = 500
    x, s = (rng.standard_normal((rows, ld)).astype(np.float16) for _ in range(2))
    g, b, bi = ((1 + 0.02 * rng.standard_normal(ld)).astype(np.float16), (0.02 * rng.standard_normal(ld)).astype(np.float16),
                (0.02 * rng.standard_normal(ld)).astype(np.float16))
    y_ref = ref.skip_layer_norm(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), _t(bi, cuda)).cpu().numpy()
    y_new = T.skip_layer_norm(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), _t(bi, cuda)).cpu().numpy()
    y_orc = O.skip_layer_norm(x, s, g, b, bi)
    assert O.close_abs_or_rel(y_ref, y_orc, 1e-2, 1e-2)[0]       # oracle pinned by the reference
    assert O.close_abs_or_rel(y_new, y_orc, 1e-2, 1e-2)[0]       # product vs oracle
    assert O.close_abs_or_rel(y_new, y_ref, 1e-2, 1e-2)[0]       # product vs reference
    # the FP32-statistics product kernel is the closer of the two to the float64 oracle
    assert np.abs(y_new - y_orc).max() <= np.abs(y_ref - y_orc).max() + 1e-3


@pytest.mark.parametrize("ld", [768, 1024])
def test_skip_ln_int8_three_way(cuda, ref, ld):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld + 1)
    rows = 500
    x, s = (rng.integers(-127, 128, size=(rows, ld)).astype(np.int8) for _ in range(2))
    g, b, bi = ((1 + 0.02 * rng.standard_normal(ld)).astype(np.float16), (0.02 * rng.standard_normal(ld)).astype(np.float16),
                (0.02 * rng.standard_normal(ld)).astype(np.float16))
    args = (0.021, 0.017, 1 / 0.03)
    y_ref = ref.skip_layer_norm_dqq(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), _t(bi, cuda), *args).cpu().numpy()
    y_new = T.skip_layer_norm_dqq(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), _t(bi, cuda), *args).cpu().numpy()
    y_orc, _ = O.skip_layer_norm_dqq(x, s, g, b, bi, *args)
    assert O.int8_within_lsb(y_ref, y_orc)[0]
    assert O.int8_within_lsb(y_new, y_orc)[0]
    assert O.int8_within_lsb(y_new, y_ref, lsb=2)[0]            # each is within 1 LSB of the oracle
    xi, si = O.to_chw32(x), O.to_chw32(s)
    for variant, mtron in ((0, False), (1, False), (2, True), (3, True)):
        o_ref, p_ref = ref.skip_layer_norm_interleaved(variant, _t(xi, cuda), _t(si, cuda), _t(g, cuda), _t(b, cuda), *args, 1 / 0.04)
        res = T.skip_layer_norm_interleaved(_t(xi, cuda), _t(si, cuda), _t(g, cuda), _t(b, cuda), *args, 1 / 0.04 if mtron else None)
        o_new = (res[0] if mtron else res).cpu().numpy()
        o_orc = O.skip_layer_norm_interleaved(xi, si, g, b, *args)
        assert O.int8_within_lsb(o_ref.cpu().numpy(), o_orc)[0]
        assert O.int8_within_lsb(o_new, o_orc)[0]
        if mtron:
            _, p_orc = O.skip_layer_norm_interleaved(xi, si, g, b, *args, 1 / 0.04)
            assert O.int8_within_lsb(p_ref.cpu().numpy(), p_orc)[0]
            assert O.int8_within_lsb(res[1].cpu().numpy(), p_orc)[0]


def test_emb_and_masks_three_way(cuda, ref):
    import tensorrt_b200 as T

    rng = np.random.default_rng(3)
    S, B, E, vocab = 128, 8, 768, 2000
    word, pos, tok = ((0.02 * rng.standard_normal((n, E))).astype(np.float16) for n in (vocab, 512, 2))
    gam, bet = (1 + 0.02 * rng.standard_normal(E)).astype(np.float32), (0.02 * rng.standard_normal(E)).astype(np.float32)
    ids = rng.integers(0, vocab, size=(S, B)).astype(np.int32)
    seg = rng.integers(0, 2, size=(S, B)).astype(np.int32)
    args = (_t(ids, cuda), _t(seg, cuda), _t(word, cuda), _t(pos, cuda), _t(tok, cuda), _t(gam, cuda), _t(bet, cuda))
    y_ref = ref.emb_layer_norm(*args).cpu().numpy()
    y_new = T.emb_layer_norm(*args).cpu().numpy()
    y_orc = O.emb_layer_norm(ids, seg, word, pos, tok, gam, bet)
    assert O.close_abs_or_rel(y_ref, y_orc, 1e-2, 1e-2)[0] and O.close_abs_or_rel(y_new, y_orc, 1e-2, 1e-2)[0]
    lengths = rng.integers(0, S + 1, size=B)
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    assert np.array_equal(ref.compute_mask_idx(_t(mask, cuda)).cpu().numpy(), T.compute_mask_idx(_t(mask, cuda)).cpu().numpy())
    assert np.array_equal(ref.convert_mask(_t(mask, cuda), 2, 2).cpu().numpy(), T.convert_mask(_t(mask, cuda), 2, 2).cpu().numpy())
    lens = rng.integers(1, 129, size=6).astype(np.int32)
    cu = O.cu_seqlens(lens)
    pids = rng.integers(0, vocab, size=int(cu[-1])).astype(np.int32)
    pseg = rng.integers(0, 2, size=int(cu[-1])).astype(np.int32)
    o_ref, s_ref = ref.emb_layer_norm_var_seqlen(_t(pids, cuda), _t(pseg, cuda), _t(cu, cuda), 128, *args[2:], mtron=True)
    o_new, s_new = T.emb_layer_norm_var_seqlen(_t(pids, cuda), _t(pseg, cuda), _t(cu, cuda), 128, *args[2:], with_skip=True)
    o_orc, s_orc = O.emb_layer_norm_var_seqlen(pids, pseg, cu, word, pos, tok, gam, bet)
    assert O.close_abs_or_rel(o_ref.cpu().numpy(), o_orc, 1e-2, 1e-2)[0] and O.close_abs_or_rel(o_new.cpu().numpy(), o_orc, 1e-2, 1e-2)[0]
    assert O.close_abs_or_rel(s_ref.cpu().numpy(), s_orc, 1e-2, 1e-2)[0] and O.close_abs_or_rel(s_new.cpu().numpy(), s_orc, 1e-2, 1e-2)[0]


@pytest.mark.parametrize("S,lengths", [(128, [128, 77, 5]), (384, [384, 200, 1, 129]), (512, [512, 300])])
def test_attention_fp16_three_way(cuda, ref, S, lengths):
    import tensorrt_b200 as T

    rng = np.random.default_rng(S)
    N, d = 4, 64
    lengths = np.array(lengths, dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    qkv = rng.standard_normal((int(cu[-1]), 3 * N * d)).astype(np.float16)
    y_ref = ref.fmha_v2(_t(qkv, cuda), _t(cu, cuda), len(lengths), S, N, d).cpu().numpy()
    y_new = T.mha(_t(qkv, cuda), len(lengths), S, N, cu_seqlens=_t(cu, cuda)).cpu().numpy()
    y_orc = O.mha(qkv, len(lengths), S, N, d, cu=cu)
    assert O.close_abs_or_rel(y_ref, y_orc, 1e-2, 1e-2)[0]
    assert O.close_abs_or_rel(y_new, y_orc, 1e-2, 1e-2)[0]
    assert O.close_abs_or_rel(y_new, y_ref, 1e-2, 1e-2)[0]


@pytest.mark.parametrize("S,lengths,interleaved", [(128, [128, 77, 5], False), (384, [384, 200, 1, 129], False),
                                                   (384, [384, 200, 1, 129], True), (128, [100], True)])
def test_attention_int8_three_way(cuda, ref, S, lengths, interleaved):
    import tensorrt_b200 as T

    rng = np.random.default_rng(S + interleaved)
    N, d = 4, 64
    lengths = np.array(lengths, dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, B = int(cu[-1]), len(lengths)
    x = rng.standard_normal((total, 3 * N * d))
    s_qkv = O.amax_scale(x)
    q8 = O.quantize(x, 1.0 / s_qkv)
    s1 = float(np.float32(s_qkv) * np.float32(s_qkv) * np.float32(0.125))
    s2 = float((1.0 / 127.0) * s_qkv / (0.5 * s_qkv))
    y_orc = O.mha_int8(q8, B, S, N, d, s1, 127.0, s2, cu=cu)
    if interleaved:
        il = np.ascontiguousarray(q8.reshape(total, N, 3, 2, 32).transpose(2, 1, 3, 0, 4)).reshape(3 * N * 2, total, 32)
        unil = lambda o: o.reshape(N, 2, total, 32).transpose(2, 0, 1, 3).reshape(total, N * d)
        y_ref = unil(ref.fmha_v2(_t(il, cuda), _t(cu, cuda), B, S, N, d, scales=(s1, 127.0, s2), interleaved=True).cpu().numpy())
        y_new = unil(T.mha(_t(il, cuda), B, S, N, cu_seqlens=_t(cu, cuda), scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=s2,
                           interleaved=True).cpu().numpy())
    else:
        y_ref = ref.fmha_v2(_t(q8, cuda), _t(cu, cuda), B, S, N, d, scales=(s1, 127.0, s2)).cpu().numpy()
        y_new = T.mha(_t(q8, cuda), B, S, N, cu_seqlens=_t(cu, cuda), scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=s2).cpu().numpy()

    def close(a, b):
        dd = np.abs(a.astype(np.int32) - b.astype(np.int32))
        return dd.max() <= 2 and (dd > 1).sum() <= max(1, int(1e-5 * dd.size)) and (dd == 0).mean() > 0.98

    assert close(y_ref, y_orc), "reference kernels vs oracle"
    assert close(y_new, y_orc), "product vs oracle"
    assert close(y_new, y_ref), "product vs reference kernels"


@pytest.mark.parametrize("S,lengths,int8", [(128, [128, 77, 5, 128], False), (384, [384, 200, 1], False), (64, [64, 33], False),
                                            (96, [96, 50], False), (128, [128, 77, 5, 128], True), (384, [384, 200, 1], True)])
def test_attention_fixed_length_kernels_three_way(cuda, ref, S, lengths, int8):
    """The fixed-length path of plugin versions 1-3 ([S, B, N, 3, d] input, input mask packed by convertMask): the
    reference's precompiled fixed-length sm100 kernels, the oracle and the product."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(S + 100 * int8)
    N, d = 4, 64
    lengths = np.array(lengths, dtype=np.int32)
    B = len(lengths)
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    x = rng.standard_normal((S, B, 3 * N * d))
    if int8:
        s_qkv = O.amax_scale(x)
        q8 = O.quantize(x, 1.0 / s_qkv)
        s1 = float(np.float32(s_qkv) * np.float32(s_qkv) * np.float32(0.125))
        s2 = float((1.0 / 127.0) * s_qkv / (0.5 * s_qkv))
        y_orc = O.mha_int8(q8, B, S, N, d, s1, 127.0, s2, lengths=lengths)
        y_ref = ref.fmha_v1(_t(q8, cuda), _t(mask, cuda), N, d, scales=(s1, 127.0, s2)).cpu().numpy()
        y_new = T.mha(_t(q8, cuda), B, S, N, mask_idx=_t(lengths, cuda), scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=s2).cpu().numpy()

        def close(a, b):
            dd = np.abs(a.astype(np.int32) - b.astype(np.int32))
            return dd.max() <= 2 and (dd > 1).sum() <= max(1, int(1e-5 * dd.size)) and (dd == 0).mean() > 0.98

        assert close(y_ref, y_orc), "reference kernels vs oracle"
        assert close(y_new, y_orc), "product vs oracle"
        assert close(y_new, y_ref), "product vs reference kernels"
    else:
        qkv = x.astype(np.float16)
        y_orc = O.mha(qkv, B, S, N, d, lengths=lengths)
        y_ref = ref.fmha_v1(_t(qkv, cuda), _t(mask, cuda), N, d).cpu().numpy()
        y_new = T.mha(_t(qkv, cuda), B, S, N, mask_idx=_t(lengths, cuda)).cpu().numpy()
        assert O.close_abs_or_rel(y_ref, y_orc, 1e-2, 1e-2)[0]
        assert O.close_abs_or_rel(y_new, y_orc, 1e-2, 1e-2)[0]
        assert O.close_abs_or_rel(y_new, y_ref, 1e-2, 1e-2)[0]


@pytest.mark.parametrize("int8", [False, True])
def test_attention_benchmark_size_three_way(cuda, ref, int8):
    """BERT-large S = 384, 64 sequences x 16 heads, ragged packed lengths: the product against the reference's own
    sm100 kernel over the WHOLE output (every work item of every persistent CTA), and both against the oracle on a
    sample of sequences."""
    import tensorrt_b200 as T

    S, B, N, d = 384, 64, 16, 64
    rng = np.random.default_rng(7 + int8)
    lengths = rng.integers(1, S + 1, size=B).astype(np.int32)
    lengths[[0, 31, 63]] = S
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    x = rng.standard_normal((total, 3 * N * d)).astype(np.float32)
    if int8:
        s_qkv = O.amax_scale(x)
        data = O.quantize(x, 1.0 / s_qkv)
        s1 = float(np.float32(s_qkv) * np.float32(s_qkv) * np.float32(0.125))
        s2 = float((1.0 / 127.0) * s_qkv / (0.5 * s_qkv))
        y_ref = ref.fmha_v2(_t(data, cuda), _t(cu, cuda), B, S, N, d, scales=(s1, 127.0, s2)).cpu().numpy()
        y_new = T.mha(_t(data, cuda), B, S, N, cu_seqlens=_t(cu, cuda), scale_bmm1=s1, scale_softmax=127.0, scale_bmm2=s2).cpu().numpy()
        dd = np.abs(y_new.astype(np.int32) - y_ref.astype(np.int32))
        assert dd.max() <= 2 and (dd > 1).sum() <= max(1, int(1e-5 * dd.size)) and (dd == 0).mean() > 0.98
    else:
        data = x.astype(np.float16)
        y_ref = ref.fmha_v2(_t(data, cuda), _t(cu, cuda), B, S, N, d).cpu().numpy()
        y_new = T.mha(_t(data, cuda), B, S, N, cu_seqlens=_t(cu, cuda)).cpu().numpy()
        assert O.close_abs_or_rel(y_new, y_ref, 1e-2, 1e-2)[0]
    for b in (0, 20, 41, 63):
        seq = data[int(cu[b]):int(cu[b + 1])]
        one = np.array([0, seq.shape[0]], dtype=np.int32)
        for y in (y_ref, y_new):
            got = y[int(cu[b]):int(cu[b + 1])]
            if int8:
                orc = O.mha_int8(seq, 1, S, N, d, s1, 127.0, s2, cu=one)
                dd = np.abs(got.astype(np.int32) - orc.astype(np.int32))
                assert dd.max() <= 2 and (dd > 1).sum() <= max(1, int(1e-5 * dd.size))
            else:
                assert O.close_abs_or_rel(got, O.mha(seq, 1, S, N, d, cu=one), 1e-2, 1e-2)[0]
