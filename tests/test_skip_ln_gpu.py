"""Parity of the SkipLayerNorm kernels (through the C ABI) with the CPU oracle.

Tolerances: FP16 rtol 1e-2 / atol 1e-2 (abs OR rel) vs the float64 oracle, FP32 1e-5, INT8 +-1 LSB
(plugin/skipLayerNormPlugin/CustomSkipLayerNormPluginDynamic_PluginConfig.yaml:111-141 and the stated targets).
"""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def _t(a, cuda, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("ld", [8, 24, 128, 768, 1024, 1536, 4096, 8192, 100])
@pytest.mark.parametrize("bias", [False, True])
def test_skip_ln_fp16(cuda, ld, bias):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld + bias)
    rows = 77
    x = rng.standard_normal((rows, ld)).astype(np.float16)
    s = rng.standard_normal((rows, ld)).astype(np.float16)
    g = (1 + 0.02 * rng.standard_normal(ld)).astype(np.float16)
    b = (0.02 * rng.standard_normal(ld)).astype(np.float16)
    bi = (0.02 * rng.standard_normal(ld)).astype(np.float16) if bias else None
    ref = O.skip_layer_norm(x, s, g, b, bi, eps=0.0)
    out = T.skip_layer_norm(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), None if bi is None else _t(bi, cuda))
    ok, worst, bad = O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)
    assert ok, (worst, bad)


@pytest.mark.parametrize("ld", [4, 128, 768, 1024, 4096, 30])
def test_skip_ln_fp32(cuda, ld):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld)
    rows = 33
    x = rng.standard_normal((rows, ld)).astype(np.float32)
    s = rng.standard_normal((rows, ld)).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(ld)).astype(np.float32)
    b = (0.02 * rng.standard_normal(ld)).astype(np.float32)
    bi = (0.02 * rng.standard_normal(ld)).astype(np.float32)
    ref = O.skip_layer_norm(x, s, g, b, bi, eps=O.EPS_F32)
    out = T.skip_layer_norm(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), _t(bi, cuda))
    ok, worst, bad = O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-5, 1e-5)
    assert ok, (worst, bad)


def test_skip_ln_empty_and_3d(cuda):
    import tensorrt_b200 as T

    g = torch.ones(768, dtype=torch.float16, device=cuda)
    e = torch.empty((0, 768), dtype=torch.float16, device=cuda)
    assert T.skip_layer_norm(e, e, g, g).shape == (0, 768)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 3, 768)).astype(np.float16)  # [S, B, E] like plugin version 5
    out = T.skip_layer_norm(_t(x, cuda), _t(x, cuda), g, torch.zeros_like(g))
    ref = O.skip_layer_norm(x, x, np.ones(768), np.zeros(768))
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]


def _int8_case(rng, rows, ld):
    x = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
    s = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
    g = (1 + 0.02 * rng.standard_normal(ld)).astype(np.float16)
    b = (0.02 * rng.standard_normal(ld)).astype(np.float16)
    bi = (0.02 * rng.standard_normal(ld)).astype(np.float16)
    return x, s, g, b, bi


@pytest.mark.parametrize("ld", [16, 256, 768, 1024, 4096, 6144, 8192, 12288, 16384])
@pytest.mark.parametrize("bias", [False, True])
def test_skip_ln_dqq(cuda, ld, bias):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld)
    x, s, g, b, bi = _int8_case(rng, 50, ld)
    if not bias:
        bi = None
    dq_in, dq_skip, q = 0.021, 0.017, 1.0 / 0.03
    ref, _ = O.skip_layer_norm_dqq(x, s, g, b, bi, dq_in, dq_skip, q)
    out = T.skip_layer_norm_dqq(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), None if bi is None else _t(bi, cuda),
                                dq_in, dq_skip, q)
    ok, worst, bad = O.int8_within_lsb(out.cpu().numpy(), ref)
    assert ok, (worst, bad)
    # rows up to 8192 wide take the packed-FP16 kernel (like the reference's kernel it normalises in half2): its steps
    # add a few tenths of an LSB, so some values land on the neighbouring step - never further
    exact = float((out.cpu().numpy() == ref).mean())
    print("skip_ln_dqq ld", ld, "bias", bias, "exact", exact)
    assert exact > (0.85 if ld <= 8192 else 0.99), exact


@pytest.mark.parametrize("ld", [32, 768, 1024, 1536, 2048, 3072, 4096])
@pytest.mark.parametrize("total", [1, 7, 8, 1000])
def test_skip_ln_interleaved(cuda, ld, total):
    import tensorrt_b200 as T

    rng = np.random.default_rng(ld + total)
    x, s, g, b, _ = _int8_case(rng, total, ld)
    dq_in, dq_skip, q, qs = 0.021, 0.017, 1.0 / 0.03, 1.0 / 0.04
    xi, si = O.to_chw32(x), O.to_chw32(s)
    ref = O.skip_layer_norm_interleaved(xi, si, g, b, dq_in, dq_skip, q)
    out = T.skip_layer_norm_interleaved(_t(xi, cuda), _t(si, cuda), _t(g, cuda), _t(b, cuda), dq_in, dq_skip, q)
    assert O.int8_within_lsb(out.cpu().numpy(), ref)[0]
    ref2, refp = O.skip_layer_norm_interleaved(xi, si, g, b, dq_in, dq_skip, q, qs)
    out2, outp = T.skip_layer_norm_interleaved(_t(xi, cuda), _t(si, cuda), _t(g, cuda), _t(b, cuda), dq_in, dq_skip, q, qs)
    assert O.int8_within_lsb(out2.cpu().numpy(), ref2)[0]
    assert O.int8_within_lsb(outp.cpu().numpy(), refp)[0]
    # linear and interleaved kernels agree with each other on the same values
    lin = T.skip_layer_norm_dqq(_t(x, cuda), _t(s, cuda), _t(g, cuda), _t(b, cuda), None, dq_in, dq_skip, q)
    assert O.int8_within_lsb(O.from_chw32(out.cpu().numpy()), lin.cpu().numpy())[0]


def test_skip_ln_full_size_properties(cuda):
    """BERT-large S=384 B=64 sizes: LayerNorm output rows have mean beta-mean and unit variance when gamma=1, beta=0."""
    import tensorrt_b200 as T

    tokens, ld = 384 * 64, 1024
    gen = torch.Generator(device=cuda).manual_seed(0)
    x = torch.randn((tokens, ld), device=cuda, generator=gen).half()
    s = torch.randn((tokens, ld), device=cuda, generator=gen).half()
    g = torch.ones(ld, dtype=torch.float16, device=cuda)
    b = torch.zeros(ld, dtype=torch.float16, device=cuda)
    out = T.skip_layer_norm(x, s, g, b).float()
    assert out.mean(dim=1).abs().max().item() < 2e-3
    assert (out.var(dim=1, unbiased=False) - 1).abs().max().item() < 5e-3
    # scaling the input by a power of two leaves the normalised output bit-identical
    out2 = T.skip_layer_norm((x * 2), (s * 2), g, b).float()
    assert torch.equal(out, out2)


def test_bad_params_report_errors(cuda):
    import tensorrt_b200 as T
    from tensorrt_b200._lib import BertB200Error

    g = torch.ones(768, dtype=torch.float16, device=cuda)
    x = torch.zeros((3, 768), dtype=torch.int8, device=cuda)
    with pytest.raises(BertB200Error):  # ld not a multiple of 16
        T.skip_layer_norm_dqq(x[:, :760].contiguous(), x[:, :760].contiguous(), g, g, None, 1.0, 1.0, 1.0)
    with pytest.raises(ValueError):  # CPU tensors are rejected, there is no CPU path
        T.skip_layer_norm(torch.zeros(2, 8), torch.zeros(2, 8), torch.ones(8), torch.zeros(8))
