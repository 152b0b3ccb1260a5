"""enqueue() of every plugin object (driven through IPluginV3OneRuntime by the C harness) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu

EMB, QKV, SKIP, FC = ("CustomEmbLayerNormPluginDynamic", "CustomQKVToContextPluginDynamic",
                      "CustomSkipLayerNormPluginDynamic", "CustomFCPluginDynamic")


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _int8_attention_ok(out, ref):
    """+-1 LSB except for rare rounding ties of the quantised probabilities (see tests/test_mha_gpu.py)."""
    d = np.abs(out.astype(np.int32) - ref.astype(np.int32))
    return d.max() <= 2 and (d > 1).sum() <= max(1, int(1e-5 * d.size))


def _run(p, H, ins, outs, in_descs, out_descs, workspace=None):
    st = p.enqueue(in_descs, out_descs, [t.data_ptr() for t in ins], [t.data_ptr() for t in outs],
                   workspace.data_ptr() if workspace is not None else None, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == 0, st


@pytest.mark.parametrize("S", [128, 384, 200])
def test_emb_v6_then_qkv_v4(cuda, S):
    """Embedding plugin emits the packed mask (S = 128 / 384) or the mask index (other S); the attention plugin
    consumes exactly that tensor."""
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(S)
    B, E, N, vocab = 3, 128, 2, 100
    word = (0.02 * rng.standard_normal((vocab, E))).astype(np.float16)
    pos = (0.02 * rng.standard_normal((512, E))).astype(np.float16)
    tok = (0.02 * rng.standard_normal((2, E))).astype(np.float16)
    gamma = (1 + 0.02 * rng.standard_normal(E)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(E)).astype(np.float32)
    emb = H.Plugin(EMB, "6", [("bert_embeddings_layernorm_beta", beta), ("bert_embeddings_layernorm_gamma", gamma),
                              ("bert_embeddings_word_embeddings", word.ravel()), ("bert_embeddings_token_type_embeddings", tok.ravel()),
                              ("bert_embeddings_position_embeddings", pos.ravel()), ("output_fp16", 1), ("mha_type_id", 1)]).attach()
    assert emb.ok
    ids = rng.integers(0, vocab, size=(S, B)).astype(np.int32)
    seg = rng.integers(0, 2, size=(S, B)).astype(np.int32)
    lengths = np.array([S, S // 3, 1], dtype=np.int32)
    mask = (np.arange(S)[:, None] < lengths[None, :]).astype(np.int32)
    (_, mask_shape) = emb.output_shapes([(S, B)] * 3, 2)
    out = torch.empty((S, B, E), dtype=torch.float16, device=cuda)
    mask_out = torch.zeros(mask_shape, dtype=torch.int32, device=cuda)
    ind = [H.make_desc((S, B), H.INT32)] * 3
    outd = [H.make_desc((S, B, E, 1, 1), H.HALF), H.make_desc(mask_shape, H.INT32)]
    _run(emb, H, [_t(ids, cuda), _t(seg, cuda), _t(mask, cuda)], [out, mask_out], ind, outd)
    ref = O.emb_layer_norm(ids, seg, word, pos[:S], tok, gamma, beta)
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]
    if mask_shape[1] == 1:
        assert np.array_equal(mask_out.cpu().numpy().ravel(), lengths)
    else:
        wm, wn = (2, 2) if S == 128 else (1, 8)
        packed = O.packed_mask(mask, wm, wn).reshape(B, -1)
        assert np.array_equal(mask_out.cpu().numpy().view(np.uint32)[:, :packed.shape[1]], packed)

    qkv_p = H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", E), ("num_heads", N), ("has_mask", 1)]).attach()
    qkv = rng.standard_normal((S, B, 3 * E)).astype(np.float16)
    ctx = torch.empty((S, B, E), dtype=torch.float16, device=cuda)
    ind = [H.make_dyn((S, B, 3 * E, 1, 1), H.HALF), H.make_dyn(mask_shape, H.INT32)]
    outd = [H.make_dyn((S, B, E, 1, 1), H.HALF)]
    assert qkv_p.configure(ind, outd) == 0
    ws = torch.empty(max(256, qkv_p.workspace_size(ind, outd)), dtype=torch.uint8, device=cuda)
    assert qkv_p.on_shape_change([d.desc for d in ind], [d.desc for d in outd]) == 0
    _run(qkv_p, H, [_t(qkv, cuda), mask_out], [ctx], [d.desc for d in ind], [d.desc for d in outd], ws)
    ref = O.mha(qkv, B, S, N, 64, lengths=lengths)
    ok, worst, bad = O.close_abs_or_rel(ctx.cpu().numpy(), ref, 1e-2, 1e-2)
    assert ok, (worst, bad)
    emb.close()
    qkv_p.close()


def test_qkv_plugin_fp16_beyond_512_tokens(cuda):
    """Version 4, FP16, S = 640 (the reference sends this to its unfused runner and asks for a score matrix in the
    workspace): the tensor-core kernel streams the five key blocks, needs nothing beyond the room for the lengths, and
    the result is one softmax over all 640 keys."""
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(12)
    S, B, N, E = 640, 3, 2, 128
    lengths = np.array([640, 200, 513], dtype=np.int32)
    qkv_p = H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", E), ("num_heads", N), ("has_mask", 1)]).attach()
    qkv = rng.standard_normal((S, B, 3 * E)).astype(np.float16)
    ctx = torch.empty((S, B, E), dtype=torch.float16, device=cuda)
    ind = [H.make_dyn((S, B, 3 * E, 1, 1), H.HALF), H.make_dyn((B,), H.INT32)]
    outd = [H.make_dyn((S, B, E, 1, 1), H.HALF)]
    assert qkv_p.configure(ind, outd) == 0
    need = qkv_p.workspace_size(ind, outd)
    assert need <= 256                            # the recovered lengths only
    ws = torch.full((max(need, 256),), 0xFF, dtype=torch.uint8, device=cuda)
    assert qkv_p.on_shape_change([d.desc for d in ind], [d.desc for d in outd]) == 0
    _run(qkv_p, H, [_t(qkv, cuda), _t(lengths, cuda)], [ctx], [d.desc for d in ind], [d.desc for d in outd], ws)
    ref = O.mha(qkv, B, S, N, 64, lengths=lengths)
    ok, worst, bad = O.close_abs_or_rel(ctx.cpu().numpy(), ref, 1e-2, 1e-2)
    assert ok, (worst, bad)
    qkv_p.close()


@pytest.mark.parametrize("ver", ["4", "5"])
def test_emb_var_seqlen_plugin(cuda, ver):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(4)
    E, vocab = 256, 300
    word = (0.02 * rng.standard_normal((vocab, E))).astype(np.float16)
    pos = (0.02 * rng.standard_normal((512, E))).astype(np.float16)
    tok = (0.02 * rng.standard_normal((2, E))).astype(np.float16)
    gamma = (1 + 0.02 * rng.standard_normal(E)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(E)).astype(np.float32)
    p = H.Plugin(EMB, ver, [("bert_embeddings_layernorm_beta", beta), ("bert_embeddings_layernorm_gamma", gamma),
                            ("bert_embeddings_word_embeddings", word.ravel()), ("bert_embeddings_token_type_embeddings", tok.ravel()),
                            ("bert_embeddings_position_embeddings", pos.ravel()), ("output_fp16", 1)])
    lengths = np.array([40, 1, 384, 77], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    ids = rng.integers(0, vocab, size=total).astype(np.int32)
    seg = rng.integers(0, 2, size=total).astype(np.int32)
    out = torch.empty((total, E), dtype=torch.float16, device=cuda)
    second = torch.zeros((total, E), dtype=torch.float16, device=cuda)
    dummy = torch.zeros(384, dtype=torch.int32, device=cuda)
    ind = [H.make_desc((total,), H.INT32), H.make_desc((total,), H.INT32), H.make_desc((len(cu),), H.INT32), H.make_desc((384,), H.INT32)]
    outd = [H.make_desc((total, E, 1, 1), H.HALF), H.make_desc((total, E, 1, 1), H.HALF) if ver == "5" else H.make_desc((), H.INT32)]
    _run(p, H, [_t(ids, cuda), _t(seg, cuda), _t(cu, cuda), dummy], [out, second], ind, outd)
    ref, ref_skip = O.emb_layer_norm_var_seqlen(ids, seg, cu, word, pos, tok, gamma, beta)
    assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]
    if ver == "5":
        assert O.close_abs_or_rel(second.cpu().numpy(), ref_skip, 1e-2, 1e-2)[0]
    else:
        assert float(second.abs().max()) == 0.0  # untouched
    p.close()


@pytest.mark.parametrize("type_id", [1, 2])
def test_qkv_v5_var_seqlen(cuda, type_id):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(type_id)
    N, d = 4, 64
    E = N * d
    lengths = np.array([384, 33, 128, 1], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, B, S = int(cu[-1]), len(lengths), 384
    p = H.Plugin(QKV, "5", [("type_id", type_id), ("hidden_size", E), ("num_heads", N), ("has_mask", 1), ("var_seqlen", 1)])
    assert p.ok
    x = rng.standard_normal((total, 3 * E))
    dummy_mask = torch.zeros(1, dtype=torch.int32, device=cuda)
    dummy = torch.zeros(S, dtype=torch.int32, device=cuda)
    if type_id == 1:
        qkv = x.astype(np.float16)
        ref = O.mha(qkv, B, S, N, d, cu=cu)
        dt, fmt, s_in, s_out = H.HALF, H.LINEAR, 1.0, 1.0
        out = torch.empty((total, E), dtype=torch.float16, device=cuda)
    else:
        s_in = O.amax_scale(x)
        s_out = s_in * 0.5
        qkv = O.quantize(x, 1.0 / s_in)
        ref = O.mha_int8(qkv, B, S, N, d, float(np.float32(s_in) * np.float32(s_in) * np.float32(0.125)), 127.0,
                         (1.0 / 127.0) * s_in / s_out, cu=cu)
        dt, fmt = H.INT8, H.CHW32
        out = torch.empty((total, E), dtype=torch.int8, device=cuda)
    ind = [H.make_desc((total, 3 * E, 1, 1), dt, fmt, s_in), H.make_desc((1,), H.INT32), H.make_desc((B + 1,), H.INT32), H.make_desc((S,), H.INT32)]
    outd = [H.make_desc((total, E, 1, 1), dt, fmt, s_out)]
    _run(p, H, [_t(qkv, cuda), dummy_mask, _t(cu, cuda), dummy], [out], ind, outd)
    if type_id == 1:
        assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-2, 1e-2)[0]
    else:
        assert _int8_attention_ok(out.cpu().numpy(), ref)
    p.close()


def test_qkv_v6_interleaved(cuda):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(6)
    N, d = 4, 64
    E = N * d
    lengths = np.array([200, 33, 128], dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total, B, S = int(cu[-1]), len(lengths), 256
    x = rng.standard_normal((total, 3 * E))
    s_in = O.amax_scale(x)
    s_out = s_in * 0.5
    q8 = O.quantize(x, 1.0 / s_in)
    ref = O.mha_int8(q8, B, S, N, d, float(np.float32(s_in) * np.float32(s_in) * np.float32(0.125)), 127.0,
                     (1.0 / 127.0) * s_in / s_out, cu=cu)
    il = np.ascontiguousarray(q8.reshape(total, N, 3, 2, 32).transpose(2, 1, 3, 0, 4))
    p = H.Plugin(QKV, "6", [("hidden_size", E), ("num_heads", N), ("use_explicit_int8", 1), ("input_qkv_scale", float(s_in)),
                            ("output_ctx_scale", float(s_out))])
    out = torch.empty((N * 2, total, 32), dtype=torch.int8, device=cuda)
    ind = [H.make_desc((1, 3 * E, total, 1), H.INT8, H.CHW32, 123.0), H.make_desc((B + 1,), H.INT32), H.make_desc((S,), H.INT32)]
    outd = [H.make_desc((1, E, total, 1), H.INT8, H.CHW32, 456.0)]  # descriptor scales are ignored with use_explicit_int8
    _run(p, H, [_t(il, cuda), _t(cu, cuda), torch.zeros(S, dtype=torch.int32, device=cuda)], [out], ind, outd)
    lin = out.cpu().numpy().reshape(N, 2, total, 32).transpose(2, 0, 1, 3).reshape(total, E)
    assert _int8_attention_ok(lin, ref)
    p.close()


@pytest.mark.parametrize("type_id,ver", [(0, "5"), (1, "5"), (1, "6"), (2, "6")])
def test_skip_ln_plugins(cuda, type_id, ver):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(type_id)
    ld, rows = 768, 300
    g = (1 + 0.02 * rng.standard_normal(ld)).astype(np.float32)
    b = (0.02 * rng.standard_normal(ld)).astype(np.float32)
    bias = (0.02 * rng.standard_normal(ld)).astype(np.float32)
    items = [("type_id", type_id), ("beta", b), ("gamma", g), ("bias", bias)] + ([("ld", ld)] if ver == "5" else [])
    p = H.Plugin(SKIP, ver, items).clone()
    shape = (100, 3, ld, 1, 1) if ver == "5" else (rows, ld, 1, 1)
    if type_id == 2:
        x = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
        s = rng.integers(-127, 128, size=(rows, ld)).astype(np.int8)
        h = lambda a: a.astype(np.float16)
        ref, _ = O.skip_layer_norm_dqq(x, s, h(g), h(b), h(bias), 0.02, 0.03, 1 / 0.025)
        out = torch.empty((rows, ld), dtype=torch.int8, device=cuda)
        ind = [H.make_desc(shape, H.INT8, H.CHW32, 0.02), H.make_desc(shape, H.INT8, H.CHW32, 0.03)]
        outd = [H.make_desc(shape, H.INT8, H.CHW32, 0.025)]
        _run(p, H, [_t(x, cuda), _t(s, cuda)], [out], ind, outd)
        assert O.int8_within_lsb(out.cpu().numpy(), ref)[0]
    else:
        dt = np.float32 if type_id == 0 else np.float16
        x = rng.standard_normal((rows, ld)).astype(dt)
        s = rng.standard_normal((rows, ld)).astype(dt)
        ref = O.skip_layer_norm(x, s, g.astype(dt), b.astype(dt), bias.astype(dt), eps=O.EPS_F32 if type_id == 0 else 0.0)
        out = torch.empty((rows, ld), dtype=torch.float32 if type_id == 0 else torch.float16, device=cuda)
        ind = [H.make_desc(shape, type_id)] * 2
        _run(p, H, [_t(x, cuda), _t(s, cuda)], [out], ind, [H.make_desc(shape, type_id)])
        tol = 1e-5 if type_id == 0 else 1e-2
        assert O.close_abs_or_rel(out.cpu().numpy(), ref, tol, tol)[0]
    p.close()


@pytest.mark.parametrize("ver", ["7", "8"])
def test_skip_ln_interleaved_plugins(cuda, ver):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(7)
    ld, total = 1024, 777
    g = (1 + 0.02 * rng.standard_normal(ld)).astype(np.float16)
    b = (0.02 * rng.standard_normal(ld)).astype(np.float16)
    x = rng.integers(-127, 128, size=(total, ld)).astype(np.int8)
    s = rng.integers(-127, 128, size=(total, ld)).astype(np.int8)
    p = H.Plugin(SKIP, ver, [("beta", b), ("gamma", g)])
    xi, si = O.to_chw32(x), O.to_chw32(s)
    out = torch.empty((ld // 32, total, 32), dtype=torch.int8, device=cuda)
    pre = torch.empty_like(out)
    shape = (1, ld, total, 1)
    ind = [H.make_desc(shape, H.INT8, H.CHW32, 0.02), H.make_desc(shape, H.INT8, H.CHW32, 0.03)]
    outd = [H.make_desc(shape, H.INT8, H.CHW32, 0.025), H.make_desc(shape, H.INT8, H.CHW32, 0.04)]
    _run(p, H, [_t(xi, cuda), _t(si, cuda)], [out, pre][: 1 if ver == "7" else 2], ind, outd[: 1 if ver == "7" else 2])
    if ver == "7":
        ref = O.skip_layer_norm_interleaved(xi, si, g, b, 0.02, 0.03, 1 / 0.025)
    else:
        ref, refp = O.skip_layer_norm_interleaved(xi, si, g, b, 0.02, 0.03, 1 / 0.025, 1 / 0.04)
        assert O.int8_within_lsb(pre.cpu().numpy(), refp)[0]
    assert O.int8_within_lsb(out.cpu().numpy(), ref)[0]
    p.close()


@pytest.mark.parametrize("mode", ["fp16", "fp16_bias_gelu", "fp32", "int8"])
def test_fc_plugin(cuda, mode):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(11)
    S, B, K, out_dim = 128, 3, 768, 2304
    W = (0.02 * rng.standard_normal((K, out_dim))).astype(np.float32)   # [K, out], not transposed
    bias = (0.02 * rng.standard_normal(out_dim)).astype(np.float32)
    x = rng.standard_normal((S * B, K))
    if mode == "fp32":
        p = H.Plugin(FC, "2", [("out_dims", out_dim), ("type_id", 0), ("W", W.ravel())])
        a = x.astype(np.float32)
        ref = O.fc(a, W)
        out = torch.empty((S * B, out_dim), dtype=torch.float32, device=cuda)
        ind, outd = [H.make_desc((S, B, K, 1, 1), H.FLOAT)], [H.make_desc((S, B, out_dim, 1, 1), H.FLOAT)]
        _run(p, H, [_t(a, cuda)], [out], ind, outd)
        assert O.close_abs_or_rel(out.cpu().numpy(), ref, 1e-5, 1e-5)[0]
    elif mode.startswith("fp16"):
        items = [("out_dims", out_dim), ("type_id", 1), ("W", W.ravel())]
        if mode.endswith("gelu"):
            items += [("bias", bias), ("activation", 1)]
        p = H.Plugin(FC, "2", items).attach()
        a = x.astype(np.float16)
        ref = O.fc(a, W.astype(np.float16), bias if mode.endswith("gelu") else None, "gelu" if mode.endswith("gelu") else None)
        out = torch.empty((S * B, out_dim), dtype=torch.float16, device=cuda)
        ind, outd = [H.make_desc((S, B, K, 1, 1), H.HALF)], [H.make_desc((S, B, out_dim, 1, 1), H.HALF)]
        _run(p, H, [_t(a, cuda)], [out], ind, outd)
        assert O.close_abs_or_rel(out.cpu().numpy(), ref, 2e-3, 2e-3)[0]
    else:
        p = H.Plugin(FC, "2", [("out_dims", out_dim), ("type_id", 2), ("W", W.ravel()), ("bias", bias)])
        s_in, s_out = O.amax_scale(x), 0.05
        a = O.quantize(x, 1.0 / s_in)
        s_w = O.amax_scale(W)
        wq = np.clip(np.rint(W / np.float32(s_w)), -127, 127).astype(np.int8)
        ref = O.fc_int8(a, wq, np.float32(s_in) * np.float32(s_w), bias, None, 1.0 / s_out)
        out = torch.empty((S * B, out_dim), dtype=torch.int8, device=cuda)
        ind = [H.make_desc((S, B, K, 1, 1), H.INT8, H.CHW32, s_in)]
        outd = [H.make_desc((S, B, out_dim, 1, 1), H.INT8, H.CHW32, s_out)]
        _run(p, H, [_t(a, cuda)], [out], ind, outd)
        assert O.int8_within_lsb(out.cpu().numpy(), ref)[0]
    p.close()
