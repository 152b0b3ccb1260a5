"""Parity of embedding + LayerNorm and the mask helpers with the CPU oracle. Index outputs bit-exact."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _tables(rng, vocab, maxpos, E, dtype):
    n = lambda *s: (0.02 * rng.standard_normal(s)).astype(dtype)
    return n(vocab, E), n(maxpos, E), n(2, E), (1 + 0.02 * rng.standard_normal(E)).astype(np.float32), (
        0.02 * rng.standard_normal(E)).astype(np.float32)


@pytest.mark.parametrize("E,dtype,tol", [(128, np.float32, 1e-5), (768, np.float16, 1e-2), (1024, np.float16, 1e-2),
                                         (4096, np.float16, 1e-2), (100, np.float32, 1e-5)])
def test_emb_fixed(cuda, E, dtype, tol):
    import tensorrt_b200 as T

    rng = np.random.default_rng(E)
    S, B, vocab = 20, 5, 100  # the reference configuration uses vocab 100 x 128, 20 positions
    word, pos, tok, gamma, beta = _tables(rng, vocab, S, E, dtype)
    ids = rng.integers(0, vocab, size=(S, B)).astype(np.int32)
    seg = rng.integers(0, 2, size=(S, B)).astype(np.int32)
    ids[3, 1] = vocab + 5   # out-of-table ids give the row `beta`
    seg[4, 2] = -1
    ref = O.emb_layer_norm(ids, seg, word, pos, tok, gamma, beta)
    out = T.emb_layer_norm(_t(ids, cuda), _t(seg, cuda), _t(word, cuda), _t(pos, cuda), _t(tok, cuda), _t(gamma, cuda),
                           _t(beta, cuda))
    ok, worst, bad = O.close_abs_or_rel(out.cpu().numpy(), ref, tol, tol)
    assert ok, (worst, bad)


def test_emb_fixed_config2_shapes_and_int8(cuda):
    import tensorrt_b200 as T

    rng = np.random.default_rng(2)
    S, B, E = 128, 32, 768
    word, pos, tok, gamma, beta = _tables(rng, 30522, 512, E, np.float16)
    ids = rng.integers(0, 30522, size=(S, B)).astype(np.int32)
    seg = (np.arange(S)[:, None] >= rng.integers(1, 128, size=B)[None, :]).astype(np.int32)
    ref = O.emb_layer_norm(ids, seg, word, pos, tok, gamma, beta)
    q = 1.0 / O.amax_scale(ref)
    out, out8 = T.emb_layer_norm(_t(ids, cuda), _t(seg, cuda), _t(word, cuda), _t(pos, cuda), _t(tok, cuda),
                                 _t(gamma, cuda), _t(beta, cuda), q_scale=q)
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]
    assert O.int8_within_lsb(out8.cpu().numpy(), O.quantize(ref, q))[0]


@pytest.mark.parametrize("E", [768, 1024])
def test_emb_var_seqlen(cuda, E):
    import tensorrt_b200 as T

    rng = np.random.default_rng(E)
    lengths = np.array([1, 17, 0, 128, 64, 3], dtype=np.int32)  # includes an empty sequence
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    word, pos, tok, gamma, beta = _tables(rng, 1000, 128, E, np.float16)
    ids = rng.integers(0, 1000, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    ref, ref_skip = O.emb_layer_norm_var_seqlen(ids, seg, cu, word, pos, tok, gamma, beta)
    out, skip = T.emb_layer_norm_var_seqlen(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), 128, _t(word, cuda), _t(pos, cuda),
                                            _t(tok, cuda), _t(gamma, cuda), _t(beta, cuda), with_skip=True)
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]
    assert O.close_abs_or_rel(skip.cpu().numpy(), ref_skip, 1e-2, 1e-2)[0]


def test_emb_gather_identity_bit_exact(cuda):
    """With zero position/segment rows the pre-LN output is exactly the gathered word row."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(9)
    E, vocab = 1024, 30522
    word = rng.standard_normal((vocab, E)).astype(np.float16)
    zeros = np.zeros((512, E), dtype=np.float16)
    lengths = rng.integers(32, 385, size=16).astype(np.int32)
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    ids = rng.integers(0, vocab, size=total).astype(np.int32)
    seg = np.zeros(total, dtype=np.int32)
    _, skip = T.emb_layer_norm_var_seqlen(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), 384, _t(word, cuda), _t(zeros, cuda),
                                          _t(zeros[:2], cuda), _t(np.ones(E, np.float32), cuda),
                                          _t(np.zeros(E, np.float32), cuda), with_skip=True)
    assert np.array_equal(skip.cpu().numpy(), word[ids])


@pytest.mark.parametrize("S,B", [(1, 1), (32, 3), (128, 32), (384, 64), (200, 7), (512, 2)])
def test_mask_idx_bit_exact(cuda, S, B):
    import tensorrt_b200 as T

    rng = np.random.default_rng(S * B)
    lengths = rng.integers(0, S + 1, size=B)
    lengths[0] = S  # a full row: no zero anywhere
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    out = T.compute_mask_idx(_t(mask, cuda)).cpu().numpy()
    assert np.array_equal(out, O.mask_idx(mask))
    assert np.array_equal(out, lengths.astype(np.int32))


@pytest.mark.parametrize("S,B,E,dtype", [(1, 1, 128, np.float32), (20, 5, 100, np.float32), (128, 32, 768, np.float16),
                                         (384, 64, 1024, np.float16), (3, 700, 1024, np.float16)])
def test_mask_idx_from_the_embedding_launch(cuda, S, B, E, dtype):
    """The fixed-length embedding launch also emits the mask index (more sequences than warps in the grid included);
    the hidden states are bit-identical to the launch without a mask."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(S * B + E)
    word, pos, tok, gamma, beta = _tables(rng, 1000, 512, E, dtype)
    ids = rng.integers(0, 1000, size=(S, B)).astype(np.int32)
    seg = rng.integers(0, 2, size=(S, B)).astype(np.int32)
    lengths = rng.integers(0, S + 1, size=B)
    lengths[0] = S
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    args = [_t(a, cuda) for a in (ids, seg, word, pos, tok, gamma, beta)]
    out, idx = T.emb_layer_norm(*args, mask=_t(mask, cuda))
    assert np.array_equal(idx.cpu().numpy(), O.mask_idx(mask))
    assert torch.equal(out, T.emb_layer_norm(*args))


@pytest.mark.parametrize("S,wm,wn", [(64, 2, 2), (96, 2, 2), (128, 2, 2), (384, 1, 8)])
def test_packed_mask_bit_exact(cuda, S, wm, wn):
    import tensorrt_b200 as T

    rng = np.random.default_rng(S)
    B = 4
    lengths = rng.integers(1, S + 1, size=B)
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    packed = T.convert_mask(_t(mask, cuda), wm, wn)
    out = packed.cpu().numpy().view(np.uint32)
    assert np.array_equal(out, O.packed_mask(mask, wm, wn))
    # and back: the attention plugin recovers the lengths from the packed form
    back = T.packed_mask_to_lengths(packed, S, wm, wn).cpu().numpy()
    assert np.array_equal(back, lengths.astype(np.int32))


@pytest.mark.parametrize("B", [0, 1, 31, 256, 1024, 5000])
def test_cu_seqlens_bit_exact(cuda, B):
    import tensorrt_b200 as T

    rng = np.random.default_rng(B)
    lengths = rng.integers(0, 385, size=B).astype(np.int32)
    out = T.lengths_to_cu_seqlens(_t(lengths, cuda)).cpu().numpy()
    assert out.dtype == np.int32
    assert np.array_equal(out, O.cu_seqlens(lengths))


def test_positions_outside_the_table_are_guarded(cuda):
    """A packed sequence longer than the position table, and a cu_seqlens that does not start at 0, would index the
    position table out of range: such tokens read nothing and produce the row `beta` (like ids outside their
    tables); every other token is unaffected. The fixed-length entry refuses S beyond the table on the host."""
    import tensorrt_b200 as T

    rng = np.random.default_rng(9)
    E, vocab, npos = 256, 100, 40
    word, pos, tok = ((0.02 * rng.standard_normal((n, E))).astype(np.float16) for n in (vocab, npos, 2))
    gam = (1 + 0.02 * rng.standard_normal(E)).astype(np.float32)
    bet = (0.02 * rng.standard_normal(E)).astype(np.float32)
    dev = [_t(a, cuda) for a in (word, pos, tok, gam, bet)]
    lengths = np.array([30, 55, 40], dtype=np.int32)           # the second sequence overruns the 40-row table
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    ids = rng.integers(0, vocab, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    out = T.emb_layer_norm_var_seqlen(_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), 64, *dev).float().cpu().numpy()
    posn = np.concatenate([np.arange(n) for n in lengths])
    ok_rows = posn < npos
    sub_cu = O.cu_seqlens(np.minimum(lengths, npos))
    ref, _ = O.emb_layer_norm_var_seqlen(ids[ok_rows], seg[ok_rows], sub_cu, word, pos, tok, gam, bet)
    assert O.close_abs_or_rel(out[ok_rows], ref, 1e-2, 1e-2)[0]
    assert np.allclose(out[~ok_rows], bet.astype(np.float16).astype(np.float32)[None], atol=1e-3)
    # cu_seqlens starting at 5: tokens 0..4 lie before every sequence start (negative position)
    cu2 = (cu + 5).astype(np.int32)
    cu2[-1] = total
    out2 = T.emb_layer_norm_var_seqlen(_t(ids, cuda), _t(seg, cuda), _t(cu2, cuda), 64, *dev).float().cpu().numpy()
    assert np.isfinite(out2).all()
    assert np.allclose(out2[:5], bet.astype(np.float16).astype(np.float32)[None], atol=1e-3)
    with pytest.raises(RuntimeError, match="position table"):
        T.emb_layer_norm(_t(np.zeros((npos + 1, 2), np.int32), cuda), _t(np.zeros((npos + 1, 2), np.int32), cuda), *dev)
