"""Parity of the fully connected kernels (tcgen05 FP16 / INT8, SIMT FP32) with the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _status(cuda):
    return torch.zeros(4, dtype=torch.int32, device=cuda)


# (m, k, n): BERT-base / BERT-large projections, ragged m, k not a multiple of the 64-wide k block
SHAPES = [(1024, 768, 2304), (1024, 768, 768), (300, 768, 3072), (129, 3072, 768), (1, 64, 16), (257, 1024, 1024),
          (130, 80, 48), (640, 4096, 1024)]


@pytest.mark.parametrize("m,k,n", SHAPES)
@pytest.mark.parametrize("epi", ["none", "bias", "bias_gelu"])
def test_fc_fp16(cuda, m, k, n, epi):
    import tensorrt_b200 as T

    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal((m, k)).astype(np.float16)
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float16)   # reference layout [K, out]
    bias = (0.02 * rng.standard_normal(n)).astype(np.float32) if epi != "none" else None
    ref = O.fc(a, w, bias, "gelu" if epi == "bias_gelu" else None)
    st = _status(cuda)
    out = T.fc(_t(a, cuda), _t(np.ascontiguousarray(w.T), cuda), None if bias is None else _t(bias, cuda),
               T.ACT_GELU_ERF if epi == "bias_gelu" else T.ACT_NONE, status=st)
    assert int(st[0]) == 0
    # the reference plugin states 1e-3 for its FP16 GEMM (CustomFCPluginDynamic_PluginConfig.yaml:72-77);
    # outputs here are O(0.5), FP16 rounding alone is 2.4e-4 relative
    ok, worst, bad = O.close_abs_or_rel(out.cpu().numpy(), ref, 2e-3, 2e-3)
    assert ok, (worst, bad)


@pytest.mark.parametrize("m,k,n", SHAPES)
@pytest.mark.parametrize("epi", ["none", "bias_gelu"])
@pytest.mark.parametrize("out_i8", [True, False])
def test_fc_int8(cuda, m, k, n, epi, out_i8):
    import tensorrt_b200 as T

    rng = np.random.default_rng(m + k + n + 1)
    a = rng.integers(-127, 128, size=(m, k)).astype(np.int8)
    w = rng.integers(-127, 128, size=(k, n)).astype(np.int8)
    bias = (0.5 * rng.standard_normal(n)).astype(np.float32) if epi != "none" else None
    alpha = 2.0 / (127 * 127 * np.sqrt(k))
    inv = 1.0 / 0.02
    ref = O.fc_int8(a, w, alpha, bias, "gelu" if epi == "bias_gelu" else None, inv if out_i8 else None)
    st = _status(cuda)
    out = T.fc(_t(a, cuda), _t(np.ascontiguousarray(w.T), cuda), None if bias is None else _t(bias, cuda),
               T.ACT_GELU_ERF if epi == "bias_gelu" else T.ACT_NONE, alpha=alpha,
               out_dtype=torch.int8 if out_i8 else torch.float16, out_scale=inv, status=st)
    assert int(st[0]) == 0
    if out_i8:
        ok, worst, bad = O.int8_within_lsb(out.cpu().numpy(), ref)
        assert ok, (worst, bad)
        # Without activation only rounding ties can differ. With GELU the kernel evaluates a fitted tanh form with
        # the hardware's packed FP16 tanh (absolute error up to ~1e-3 * |x| / 2, a few percent of one INT8 step here),
        # so a few percent of the values land on the neighbouring step - never further.
        assert (out.cpu().numpy() == ref).mean() > (0.93 if epi == "bias_gelu" else 0.99)
    else:
        ok, worst, bad = O.close_abs_or_rel(out.cpu().numpy(), ref, 2e-3, 2e-3)
        assert ok, (worst, bad)


def test_fc_int8_exact_accumulation(cuda):
    """alpha = 1, no rounding anywhere: the INT32 accumulators themselves must be exact (FP16 output of small sums)."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(5)
    m, k, n = 256, 128, 256
    a = rng.integers(-3, 4, size=(m, k)).astype(np.int8)
    w = rng.integers(-3, 4, size=(k, n)).astype(np.int8)
    out = T.fc(_t(a, cuda), _t(np.ascontiguousarray(w.T), cuda), out_dtype=torch.float16)
    ref = a.astype(np.int32) @ w.astype(np.int32)
    assert np.abs(ref).max() < 2048  # exactly representable in FP16
    assert np.array_equal(out.cpu().numpy().astype(np.int32), ref)


@pytest.mark.parametrize("m,k,n", [(100, 96, 72), (64, 768, 768)])
def test_fc_fp32(cuda, m, k, n):
    import tensorrt_b200 as T

    rng = np.random.default_rng(m)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (0.02 * rng.standard_normal((k, n))).astype(np.float32)
    bias = (0.02 * rng.standard_normal(n)).astype(np.float32)
    ref = O.fc(a, w, bias, "gelu")
    out = T.fc(_t(a, cuda), _t(np.ascontiguousarray(w.T), cuda), _t(bias, cuda), T.ACT_GELU_ERF)
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-5, 1e-5)[0]


def test_fc_linearity_full_size(cuda):
    """BERT-large sizes (24576 x 1024 -> 4096): fc(a1 + a2) == fc(a1) + fc(a2) within FP16 rounding, and a
    checksum of the INT8 product equals the checksum computed from row/column sums."""
    import tensorrt_b200 as T

    gen = torch.Generator(device=cuda).manual_seed(0)
    m, k, n = 24576, 1024, 4096
    a8 = torch.randint(-127, 128, (m, k), device=cuda, generator=gen, dtype=torch.int32).to(torch.int8)
    w8 = torch.randint(-127, 128, (n, k), device=cuda, generator=gen, dtype=torch.int32).to(torch.int8)
    out = T.fc(a8, w8, alpha=1.0 / 65536, out_dtype=torch.float16).double() * 65536
    # sum over all outputs = sum_k (sum_m a[m,k]) * (sum_n w[n,k])
    expect = (a8.double().sum(0) * w8.double().sum(0)).sum().item()
    got = out.sum().item()
    scale = (a8.double().abs().sum(0) * w8.double().abs().sum(0)).sum().item()
    assert abs(got - expect) / scale < 1e-4
    a1 = torch.randn((2048, k), device=cuda, generator=gen).half()
    a2 = torch.randn((2048, k), device=cuda, generator=gen).half()
    wt = (0.02 * torch.randn((n, k), device=cuda, generator=gen)).half()
    lhs = T.fc((a1.float() + a2.float()).half(), wt).float()
    rhs = T.fc(a1, wt).float() + T.fc(a2, wt).float()
    assert (lhs - rhs).abs().max().item() < 2e-2


def _sampled_rows(m, rng):
    """Rows spread over the whole range: two of every 256-row block (the unit a pair of CTAs owns), the last 32 rows
    and some at random - so that every tile a persistent cluster takes, not only its first, is compared."""
    rows = [blk * 256 + int(o) for blk in range(m // 256) for o in rng.integers(0, 256, size=2)]
    rows += list(range(m - 32, m)) + list(rng.integers(0, m, size=128))
    return np.unique(np.array(rows, dtype=np.int64))


# the four projections of a BERT-large layer at the benchmark's row count (64 sequences x 384 tokens)
LARGE = [(24576, 1024, 3072, "bias"), (24576, 1024, 1024, "none"), (24576, 1024, 4096, "bias_gelu"), (24576, 4096, 1024, "none")]


@pytest.mark.parametrize("m,k,n,epi", LARGE)
def test_fc_fp16_benchmark_shapes(cuda, m, k, n, epi):
    """Element-wise against the oracle at the benchmarked size: 312-1248 tiles on 74 CTA pairs, i.e. the second and
    later tiles of every persistent cluster (accumulator double-buffering, stage parities) are checked too."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(m + k + n)
    gen = torch.Generator(device=cuda).manual_seed(k + n)
    a = torch.randn((m, k), device=cuda, generator=gen).half()
    wt = (0.02 * torch.randn((n, k), device=cuda, generator=gen)).half()
    bias = (0.02 * torch.randn((n,), device=cuda, generator=gen)).float() if epi != "none" else None
    st = _status(cuda)
    out = T.fc(a, wt, bias, T.ACT_GELU_ERF if epi == "bias_gelu" else T.ACT_NONE, status=st)
    assert int(st[0]) == 0
    rows = _sampled_rows(m, rng)
    idx = torch.from_numpy(rows).to(cuda)
    ref = O.fc(a[idx].cpu().numpy(), wt.cpu().numpy().T, None if bias is None else bias.cpu().numpy(),
               "gelu" if epi == "bias_gelu" else None)
    ok, worst, bad = O.close_abs_or_rel(out[idx].cpu().numpy(), ref, 2e-3, 2e-3)
    assert ok, (worst, bad)


@pytest.mark.parametrize("m,k,n,epi", LARGE)
def test_fc_int8_benchmark_shapes(cuda, m, k, n, epi):
    import tensorrt_b200 as T

    rng = np.random.default_rng(m + k + n + 1)
    gen = torch.Generator(device=cuda).manual_seed(k + n + 1)
    a = torch.randint(-127, 128, (m, k), device=cuda, generator=gen, dtype=torch.int32).to(torch.int8)
    wt = torch.randint(-127, 128, (n, k), device=cuda, generator=gen, dtype=torch.int32).to(torch.int8)
    bias = (0.5 * torch.randn((n,), device=cuda, generator=gen)).float() if epi != "none" else None
    alpha = 2.0 / (127 * 127 * np.sqrt(k))
    inv = 1.0 / 0.02
    st = _status(cuda)
    out = T.fc(a, wt, bias, T.ACT_GELU_ERF if epi == "bias_gelu" else T.ACT_NONE, alpha=alpha, out_dtype=torch.int8,
               out_scale=inv, status=st)
    assert int(st[0]) == 0
    rows = _sampled_rows(m, rng)
    idx = torch.from_numpy(rows).to(cuda)
    ref = O.fc_int8(a[idx].cpu().numpy(), wt.cpu().numpy().T, alpha, None if bias is None else bias.cpu().numpy(),
                    "gelu" if epi == "bias_gelu" else None, inv)
    got = out[idx].cpu().numpy()
    ok, worst, bad = O.int8_within_lsb(got, ref)
    assert ok, (worst, bad)
    assert (got == ref).mean() > (0.93 if epi == "bias_gelu" else 0.99)
