"""Whole-encoder parity (C++ layer loop over the kernels) with the CPU oracle on small configurations.

Per-operator parity at the stated tolerances lives in the op tests; through several layers rounding differences
compound, so the whole-model checks are: FP16 - at least 99.9 % of the values inside rtol/atol 1e-2 and none off
by more than 5e-2; INT8 - cosine similarity with the INT8 oracle above 0.999 and 99 % of the final INT8 values
within 2 LSB.
"""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _small(rng, layers=2, hidden=128, heads=2, ffn=512):
    return O.make_bert_params(rng, layers, hidden, heads, ffn, vocab=1000, max_pos=512)


@pytest.mark.parametrize("lengths", [[128, 128], [384, 17, 200, 1], [96]])
def test_encoder_fp16(cuda, lengths):
    import tensorrt_b200 as T

    rng = np.random.default_rng(len(lengths))
    p = _small(rng)
    lengths = np.array(lengths, dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, S = int(cu[-1]), int(lengths.max())
    ids = rng.integers(0, 1000, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    ref = O.encoder_fp(p, ids, seg, cu, S)
    enc = T.BertEncoder(p, T.FP16, cuda)
    out = enc.forward(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), S).cpu().numpy()
    assert enc.status_word() == 0
    assert enc.launches_per_forward == 1 + 7 * len(p.layers)
    ok, worst, bad = O.close_abs_or_rel(out, ref, 1e-2, 1e-2)
    assert bad <= out.size * 1e-3 and worst < 5e-2, (worst, bad)
    # host-buffer entry point gives the same bytes
    out_dev = torch.empty((total, p.hidden), dtype=torch.float16, device=cuda)
    out_h = torch.empty((total, p.hidden), dtype=torch.float16).pin_memory()
    enc.forward_host(torch.from_numpy(ids).pin_memory(), torch.from_numpy(seg).pin_memory(),
                     torch.from_numpy(cu).pin_memory(), S, out_dev, out_h)
    assert np.array_equal(out_h.numpy(), out)
    enc.close()


@pytest.mark.parametrize("lengths", [[128, 128], [384, 17, 200, 1]])
def test_encoder_int8(cuda, lengths):
    import tensorrt_b200 as T

    rng = np.random.default_rng(10 + len(lengths))
    p = _small(rng)
    lengths = np.array(lengths, dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, S = int(cu[-1]), int(lengths.max())
    ids = rng.integers(0, 1000, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    O.calibrate_int8(p, ids, seg, cu, S)
    ref, ref_i8, _ = O.encoder_int8(p, ids, seg, cu, S, return_all=True)
    enc = T.BertEncoder(p, T.INT8, cuda)
    out = enc.forward(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), S).cpu().numpy().astype(np.float64)
    assert enc.status_word() == 0
    assert enc.launches_per_forward == 2 + 7 * len(p.layers)
    cos = float((out * ref).sum() / np.sqrt((out * out).sum() * (ref * ref).sum()))
    assert cos > 0.999, cos
    s_out = p.layers[-1].scales["s_out"]
    lsb = np.abs(np.rint(out / s_out) - ref_i8.astype(np.float64))
    assert (lsb <= 2).mean() > 0.99, float((lsb <= 2).mean())
    # the INT8 path also tracks the unquantised FP32 oracle
    ref_fp = O.encoder_fp(p, ids, seg, cu, S, round_fp16=False)
    cos_fp = float((out * ref_fp).sum() / np.sqrt((out * out).sum() * (ref_fp * ref_fp).sum()))
    assert cos_fp > 0.99, cos_fp
    enc.close()


def test_forward_host_async_matches_forward_host(cuda):
    """The pipelined host interface (two alternating output slots, copy on a second stream) returns what the
    synchronous one returns, for several steps in flight and different inputs per step."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(11)
    p = O.make_bert_params(rng, 2, 256, 4, 1024, vocab=1000)
    enc = T.BertEncoder(p, T.FP16, cuda)
    B, S = 6, 96
    lengths = rng.integers(10, S + 1, size=B).astype(np.int32)
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    steps = 5
    ids = [torch.from_numpy(rng.integers(0, 1000, size=total).astype(np.int32)).pin_memory() for _ in range(steps)]
    seg = torch.from_numpy(rng.integers(0, 2, size=total).astype(np.int32)).pin_memory()
    cu_h = torch.from_numpy(cu).pin_memory()
    out_dev = [torch.empty((total, 256), dtype=torch.float16, device=cuda) for _ in range(2)]
    want = []
    for i in range(steps):
        out_h = torch.empty((total, 256), dtype=torch.float16).pin_memory()
        enc.forward_host(ids[i], seg, cu_h, S, out_dev[0], out_h)
        want.append(out_h.clone())
    copy_stream = torch.cuda.Stream()
    outs_h = [torch.empty((total, 256), dtype=torch.float16).pin_memory() for _ in range(2)]
    got = []
    for i in range(steps):
        if i >= 2:  # the slot is about to be reused: collect its previous result first
            enc.wait_host(i & 1)
            got.append(outs_h[i & 1].clone())
        enc.forward_host_async(ids[i], seg, cu_h, S, out_dev[i & 1], outs_h[i & 1], copy_stream, i & 1)
    for i in range(steps - 2, steps):
        enc.wait_host(i & 1)
        got.append(outs_h[i & 1].clone())
    for i in range(steps):
        assert torch.equal(got[i], want[i]), i
    enc.close()


@pytest.mark.parametrize("int8", [False, True])
def test_forward_is_graph_capturable(cuda, int8):
    """TensorRT replays engines as CUDA graphs: a forward captured into a graph (kernels launched with programmatic
    stream serialisation included) must replay to the same bits as the eager call."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(31)
    p = _small(rng)
    lengths = np.array([200, 64, 384, 3], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, S = int(cu[-1]), int(lengths.max())
    ids = _t(rng.integers(0, 1000, size=total).astype(np.int32), cuda)
    seg = _t(rng.integers(0, 2, size=total).astype(np.int32), cuda)
    cu_d = _t(cu, cuda)
    if int8:
        O.calibrate_int8(p, ids.cpu().numpy(), seg.cpu().numpy(), cu, S)
    enc = T.BertEncoder(p, T.INT8 if int8 else T.FP16, cuda)
    out = torch.empty((total, 128), dtype=torch.float16, device=cuda)
    eager = enc.forward(ids, seg, cu_d, S, out=out).clone()
    stream = torch.cuda.Stream(device=cuda)
    with torch.cuda.stream(stream):
        enc.forward(ids, seg, cu_d, S, out=out)       # warm-up on the capturing stream
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            enc.forward(ids, seg, cu_d, S, out=out)
    out.zero_()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    assert enc.status_word() == 0
    enc.close()


def test_calibration_maxima_match_oracle(cuda):
    """bert_b200_encoder_calibrate: the |tensor| maxima taken on the device during an FP16 forward equal the oracle's
    (float64 forward with FP16-rounded tensors) up to FP16 rounding of the tensors they are taken from, and the
    scales derived from them equal amax / 127."""
    import tensorrt_b200 as T
    from tensorrt_b200 import synthetic

    rng = np.random.default_rng(41)
    p = _small(rng, layers=3)
    lengths = np.array([384, 17, 200, 1, 128], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, S = int(cu[-1]), int(lengths.max())
    ids = rng.integers(0, 1000, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    enc = T.BertEncoder(p, T.FP16, cuda)
    amax = enc.calibrate(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), S)
    enc.close()
    # oracle: the same forward with every stored tensor rounded to FP16, maxima in the device's slot order
    x, _ = O.emb_layer_norm_var_seqlen(ids, seg, cu, p.word_emb, p.pos_emb, p.tok_emb, p.emb_gamma, p.emb_beta)
    x = x.astype(np.float16).astype(np.float64)
    want = np.zeros_like(amax)
    for li, lp in enumerate(p.layers):
        want[li, 0] = np.abs(x).max()
        x, t = O.encoder_layer_fp(x, lp, len(lengths), S, p.heads, cu, round_fp16=True)
        want[li, 1:7] = [np.abs(t[k]).max() for k in ("qkv", "ctx", "ao", "h1", "f1", "f2")]
        want[li, 7] = np.abs(x).max()
    # the maxima are FP16 values; kernels and oracle may round an extreme element to neighbouring FP16 numbers, and
    # through three layers inputs differ by a few FP16 ulps
    assert np.all(np.abs(amax - want) <= 1e-2 * want + 1e-3), (amax, want)
    # the scales the INT8 encoder is given are exactly amax / 127 (weights: amax of the matrix / 127)
    import types
    layers = [types.SimpleNamespace(scales={}, **{n: torch.from_numpy(getattr(lp, n).astype(np.float32)) for n in
                                                 ("w_qkv", "w_out", "w_ffn1", "w_ffn2")}) for lp in p.layers]
    synthetic.assign_int8_scales(types.SimpleNamespace(layers=layers), amax)
    for li, lp in enumerate(p.layers):
        assert layers[li].scales["s_qkv"] == pytest.approx(float(amax[li, 1]) / 127.0, rel=1e-6)
        assert layers[li].scales["s_w_qkv"] == pytest.approx(O.amax_scale(lp.w_qkv.astype(np.float32)), rel=1e-6)
        if li > 0:
            assert layers[li].scales["s_in"] == layers[li - 1].scales["s_out"]
