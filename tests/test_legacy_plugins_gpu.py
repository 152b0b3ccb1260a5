"""Legacy IPluginV2DynamicExt versions enqueue the same kernels as the IPluginV3 versions they correspond to: outputs
must be bit-identical, also after a serialise -> deserialise round trip through the flat buffer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

EMB, QKV, SKIP = ("CustomEmbLayerNormPluginDynamic", "CustomQKVToContextPluginDynamic", "CustomSkipLayerNormPluginDynamic")


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _enqueue(p, ins, outs, in_descs, out_descs, ws=None):
    st = p.enqueue(in_descs, out_descs, [t.data_ptr() for t in ins], [t.data_ptr() for t in outs],
                   ws.data_ptr() if ws is not None else None, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == 0, st


def test_skip_ln_legacy_matches_v5(cuda):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(0)
    S, B, E = 64, 3, 256
    beta, gamma, bias = (rng.standard_normal(E).astype(np.float32) for _ in range(3))
    items = [("ld", E), ("type_id", 1), ("beta", beta), ("gamma", gamma), ("bias", bias)]
    x = _t(rng.standard_normal((S, B, E)).astype(np.float16), cuda)
    skip = _t(rng.standard_normal((S, B, E)).astype(np.float16), cuda)
    d = H.make_desc((S, B, E, 1, 1), H.HALF)
    v5 = H.Plugin(SKIP, "5", items).attach()
    want = torch.empty_like(x)
    _enqueue(v5, [x, skip], [want], [d, d], [d])
    v1 = H.LegacyPlugin(SKIP, "1", items)
    again = H.LegacyPlugin(SKIP, "1", serialized=v1.serialize())
    for p in (v1, again, again.clone()):
        got = torch.zeros_like(x)
        _enqueue(p, [x, skip], [got], [d, d], [d])
        assert torch.equal(got, want)
        p.close()
    v5.close()


def test_qkv_var_seqlen_legacy_matches_v5(cuda):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(1)
    N, dh, S = 4, 64, 160
    E = N * dh
    lengths = np.array([160, 37, 128, 5], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    total, B = int(cu[-1]), len(lengths)
    qkv = _t(rng.standard_normal((total, 3 * E, 1, 1)).astype(np.float16), cuda)
    items = [("type_id", 1), ("hidden_size", E), ("num_heads", N), ("has_mask", 1), ("var_seqlen", 1)]
    ind = [H.make_desc((total, 3 * E, 1, 1), H.HALF), H.make_desc((1,), H.INT32), H.make_desc((B + 1,), H.INT32),
           H.make_desc((S,), H.INT32)]
    outd = [H.make_desc((total, E, 1, 1), H.HALF)]
    dummy = torch.zeros(1, dtype=torch.int32, device=cuda)
    maxlen = torch.zeros(S, dtype=torch.int32, device=cuda)
    cu_d = _t(cu, cuda)
    v5 = H.Plugin(QKV, "5", items).attach()
    want = torch.empty((total, E, 1, 1), dtype=torch.float16, device=cuda)
    _enqueue(v5, [qkv, dummy, cu_d, maxlen], [want], ind, outd)
    v2 = H.LegacyPlugin(QKV, "2", items)
    again = H.LegacyPlugin(QKV, "2", serialized=v2.serialize())
    for p in (v2, again):
        got = torch.zeros_like(want)
        _enqueue(p, [qkv, dummy, cu_d, maxlen], [got], ind, outd)
        assert torch.equal(got, want)
        p.close()
    v5.close()


def test_emb_var_seqlen_legacy_matches_v4(cuda):
    from tensorrt_b200 import plugin_harness as H

    rng = np.random.default_rng(2)
    E, vocab, S = 128, 300, 64
    lengths = np.array([64, 10, 33], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    total, B = int(cu[-1]), len(lengths)
    weights = [("bert_embeddings_layernorm_beta", (0.1 * rng.standard_normal(E)).astype(np.float32)),
               ("bert_embeddings_layernorm_gamma", (1 + 0.1 * rng.standard_normal(E)).astype(np.float32)),
               ("bert_embeddings_word_embeddings", (0.05 * rng.standard_normal(vocab * E)).astype(np.float16)),
               ("bert_embeddings_token_type_embeddings", (0.05 * rng.standard_normal(2 * E)).astype(np.float16)),
               ("bert_embeddings_position_embeddings", (0.05 * rng.standard_normal(512 * E)).astype(np.float16)),
               ("output_fp16", 1)]
    ids = _t(rng.integers(0, vocab, size=total).astype(np.int32), cuda)
    seg = _t(rng.integers(0, 2, size=total).astype(np.int32), cuda)
    cu_d = _t(cu, cuda)
    maxlen = torch.zeros(S, dtype=torch.int32, device=cuda)
    ind = [H.make_desc((total,), H.INT32), H.make_desc((total,), H.INT32), H.make_desc((B + 1,), H.INT32),
           H.make_desc((S,), H.INT32)]
    v4 = H.Plugin(EMB, "4", weights).attach()
    shapes = v4.output_shapes([(total,), (total,), (B + 1,), (S,)], 2)
    outd = [H.make_desc(shapes[0], H.HALF), H.make_desc(shapes[1], H.HALF)]
    want = [torch.empty(shapes[0], dtype=torch.float16, device=cuda), torch.empty(shapes[1], dtype=torch.float16, device=cuda)]
    _enqueue(v4, [ids, seg, cu_d, maxlen], want, ind, outd)
    v2 = H.LegacyPlugin(EMB, "2", weights)
    assert v2.output_dims(0, [(total,), (total,), (B + 1,), (S,)]) == tuple(shapes[0])
    again = H.LegacyPlugin(EMB, "2", serialized=v2.serialize())
    for p in (v2, again):
        got = [torch.zeros_like(want[0]), torch.zeros_like(want[1])]
        _enqueue(p, [ids, seg, cu_d, maxlen], got, ind, outd)
        assert torch.equal(got[0], want[0])
        p.close()
    v4.close()


def test_fc_v1_matches_v2(cuda):
    from tensorrt_b200 import plugin_harness as H

    FC = "CustomFCPluginDynamic"
    rng = np.random.default_rng(3)
    S, B, K, out = 40, 8, 256, 384
    W = (0.05 * rng.standard_normal(K * out)).astype(np.float32)
    bias = rng.standard_normal(out).astype(np.float32)
    items = [("out_dims", out), ("type_id", 1), ("W", W), ("bias", bias), ("activation", 1)]
    x = _t(rng.standard_normal((S, B, K, 1, 1)).astype(np.float16), cuda)
    ind, outd = [H.make_desc((S, B, K, 1, 1), H.HALF)], [H.make_desc((S, B, out, 1, 1), H.HALF)]
    v2 = H.Plugin(FC, "2", items).attach()
    want = torch.empty((S, B, out, 1, 1), dtype=torch.float16, device=cuda)
    _enqueue(v2, [x], [want], ind, outd)
    v1 = H.LegacyPlugin(FC, "1", items)
    again = H.LegacyPlugin(FC, "1", serialized=v1.serialize())
    for p in (v1, again):
        got = torch.zeros_like(want)
        _enqueue(p, [x], [got], ind, outd)
        assert torch.equal(got, want)
        p.close()
    v2.close()
