"""Host-side behaviour of the IPluginV3 adapters, driven through their real interfaces by the C harness:
creator names / versions / fields, field validation, shape and format rules, serialise -> runtime-create round
trip. No kernel is launched (creating a plugin without a GPU just leaves its device copies empty)."""
import numpy as np
import pytest

from tensorrt_b200 import plugin_harness as H

EMB, QKV, SKIP, FC = ("CustomEmbLayerNormPluginDynamic", "CustomQKVToContextPluginDynamic",
                      "CustomSkipLayerNormPluginDynamic", "CustomFCPluginDynamic")


def _emb_fields(E=64, vocab=50, fp16=1, extra=()):
    rng = np.random.default_rng(0)
    dt = np.float16 if fp16 else np.float32
    return [("bert_embeddings_layernorm_beta", rng.standard_normal(E).astype(np.float32)),
            ("bert_embeddings_layernorm_gamma", rng.standard_normal(E).astype(np.float32)),
            ("bert_embeddings_word_embeddings", rng.standard_normal(vocab * E).astype(dt)),
            ("bert_embeddings_token_type_embeddings", rng.standard_normal(2 * E).astype(dt)),
            ("bert_embeddings_position_embeddings", rng.standard_normal(20 * E).astype(dt)),
            ("output_fp16", fp16)] + list(extra)


def test_creator_inventory():
    got = {(n, v) for n, v, ns, _ in H.creators()}
    want = {(EMB, "4"), (EMB, "5"), (EMB, "6"), (QKV, "4"), (QKV, "5"), (QKV, "6"), (SKIP, "5"), (SKIP, "6"),
            (SKIP, "7"), (SKIP, "8"), (FC, "2")}
    legacy = {(QKV, "1"), (QKV, "2"), (QKV, "3"), (EMB, "1"), (EMB, "2"), (EMB, "3"), (SKIP, "1"), (SKIP, "2"),
              (SKIP, "3"), (SKIP, "4"), (FC, "1")}
    assert got == want | legacy
    assert set(H.legacy_creators()) == legacy
    assert all(ns == "" for _, _, ns, _ in H.creators())
    fields = {(n, v): f for n, v, _, f in H.creators()}
    assert set(fields[(QKV, "4")]) == {"type_id", "hidden_size", "num_heads", "has_mask", "dq_probs"}
    assert {"var_seqlen", "use_int8_scale_max"} <= set(fields[(QKV, "5")])
    assert {"use_explicit_int8", "input_qkv_scale", "output_ctx_scale"} <= set(fields[(QKV, "6")])
    assert {"ld", "type_id", "beta", "gamma", "bias"} == set(fields[(SKIP, "5")])
    assert "ld" not in fields[(SKIP, "6")]
    assert set(fields[(SKIP, "7")]) == {"beta", "gamma"}
    assert {"out_dims", "type_id", "W"} <= set(fields[(FC, "2")])
    assert {"full_mask", "mha_type_id", "output_fp16"} <= set(fields[(EMB, "6")])


def test_missing_required_fields_return_null():
    assert not H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", 768)]).ok
    assert not H.Plugin(SKIP, "5", [("type_id", 1), ("ld", 8)]).ok
    assert not H.Plugin(FC, "2", [("out_dims", 8), ("type_id", 1)]).ok
    assert not H.Plugin(EMB, "6", [("output_fp16", 1)]).ok
    assert not H.Plugin(QKV, "4", [("type_id", 7), ("hidden_size", 768), ("num_heads", 12), ("has_mask", 1)]).ok
    assert not H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", 770), ("num_heads", 12), ("has_mask", 1)]).ok


def test_qkv_v4_shapes_formats_serialisation():
    p = H.Plugin(QKV, "4", [("type_id", 1), ("hidden_size", 768), ("num_heads", 12), ("has_mask", 1)])
    assert p.ok and p.core_info() == (QKV, "4", "") and p.nb_outputs() == 1
    S, B = 128, 8
    assert p.output_shapes([(S, B, 2304, 1, 1), (B, 512)], 1) == [(S, B, 768, 1, 1)]
    assert p.output_types([H.HALF, H.INT32], 1) == [H.HALF]
    descs = [H.make_dyn((S, B, 2304, 1, 1), H.HALF), H.make_dyn((B, 512), H.INT32), H.make_dyn((S, B, 768, 1, 1), H.HALF)]
    assert all(p.supports(i, descs, 2, 1) for i in range(3))
    bad = list(descs)
    bad[0] = H.make_dyn((S, B, 2304, 1, 1), H.FLOAT)
    assert not p.supports(0, bad, 2, 1)
    bad = list(descs)
    bad[2] = H.make_dyn((S, B, 770, 1, 1), H.HALF)
    assert not p.supports(2, bad, 2, 1)
    assert p.configure(descs[:2], descs[2:]) == 0
    assert p.workspace_size(descs[:2], descs[2:]) >= B * 4
    ser = p.serialize()
    assert {"type_id", "hidden_size", "num_heads", "has_mask", "S", "B", "SM", "hasUnfusedDispatcher"} <= set(ser)
    assert int(ser["S"][0]) == S and int(ser["B"][0]) == B
    # an engine written by the reference library also carries runnerStateBuffer: accepted and ignored
    items = [(k, v if v.size > 1 else (int(v[0]) if v.dtype == np.int32 else float(v[0]))) for k, v in ser.items()]
    q = H.Plugin(QKV, "4", items + [("runnerStateBuffer", np.zeros(16, np.int32))], phase=H.RUNTIME)
    assert q.ok and q.serialize().keys() == ser.keys()
    c = q.clone()
    a = c.attach()
    assert c.ok and a.ok and a.core_info() == (QKV, "4", "")
    for x in (a, c, q, p):
        x.close()


def test_qkv_int8_defaults_and_v5_v6():
    p = H.Plugin(QKV, "4", [("type_id", 2), ("hidden_size", 1024), ("num_heads", 16), ("has_mask", 1)])
    assert abs(float(p.serialize()["dq_probs"][0]) - 1 / 127) < 1e-9
    d = [H.make_dyn((384, 4, 3072, 1, 1), H.INT8, H.CHW32), H.make_dyn((4, 6144), H.INT32), H.make_dyn((384, 4, 1024, 1, 1), H.INT8, H.CHW32)]
    assert all(p.supports(i, d, 2, 1) for i in range(3))
    d[0] = H.make_dyn((384, 4, 3072, 1, 1), H.INT8, H.LINEAR)
    assert not p.supports(0, d, 2, 1)
    p.close()
    v5 = H.Plugin(QKV, "5", [("type_id", 1), ("hidden_size", 1024), ("num_heads", 16), ("has_mask", 1), ("var_seqlen", 1)])
    assert v5.ok
    total = 1000
    d = [H.make_dyn((total, 3072, 1, 1), H.HALF), H.make_dyn((1,), H.INT32), H.make_dyn((9,), H.INT32), H.make_dyn((384,), H.INT32),
         H.make_dyn((total, 1024, 1, 1), H.HALF)]
    assert all(v5.supports(i, d, 4, 1) for i in range(5))
    assert v5.output_shapes([(total, 3072, 1, 1), (1,), (9,), (384,)], 1) == [(total, 1024, 1, 1)]
    assert {"var_seqlen", "use_int8_scale_max", "S", "B"} <= set(v5.serialize())
    v5.close()
    # FP32 cannot use var_seqlen (as in the reference)
    assert not H.Plugin(QKV, "5", [("type_id", 0), ("hidden_size", 64), ("num_heads", 1), ("has_mask", 1), ("var_seqlen", 1)]).ok
    v6 = H.Plugin(QKV, "6", [("hidden_size", 1024), ("num_heads", 16), ("use_explicit_int8", 1), ("input_qkv_scale", 0.05),
                             ("output_ctx_scale", 0.02)])
    assert v6.ok
    d = [H.make_dyn((1, 3072, total, 1), H.INT8, H.CHW32), H.make_dyn((9,), H.INT32), H.make_dyn((384,), H.INT32),
         H.make_dyn((1, 1024, total, 1), H.INT8, H.CHW32)]
    assert all(v6.supports(i, d, 3, 1) for i in range(4))
    assert v6.output_shapes([(1, 3072, total, 1), (9,), (384,)], 1) == [(1, 1024, total, 1)]
    ser = v6.serialize()
    assert abs(float(ser["input_qkv_scale"][0]) - 0.05) < 1e-7 and int(ser["use_explicit_int8"][0]) == 1
    v6.close()


@pytest.mark.parametrize("S,expect", [(128, 512), (64, 512), (96, 512), (384, 6144), (200, 1), (512, 1)])
def test_emb_v6_mask_shape_rule(S, expect):
    p = H.Plugin(EMB, "6", _emb_fields(extra=[("mha_type_id", 1)]))
    assert p.ok and p.nb_outputs() == 2
    B = 3
    assert p.output_shapes([(S, B)] * 3, 2) == [(S, B, 64, 1, 1), (B, expect)]
    assert p.output_types([H.INT32] * 3, 2) == [H.HALF, H.INT32]
    p.close()
    # FP32 attention downstream: always the 1-wide mask index
    q = H.Plugin(EMB, "6", _emb_fields(fp16=0, extra=[("mha_type_id", 0)]))
    assert q.output_shapes([(S, B)] * 3, 2)[1] == (B, 1)
    assert q.output_types([H.INT32] * 3, 2) == [H.FLOAT, H.INT32]
    q.close()


def test_emb_var_seqlen_and_serialisation_round_trip():
    for ver, second in (("4", ()), ("5", (77, 64, 1, 1))):
        p = H.Plugin(EMB, ver, _emb_fields())
        assert p.ok
        shapes = p.output_shapes([(77,), (77,), (5,), (128,)], 2)
        assert shapes == [(77, 64, 1, 1), second]
        assert p.output_types([H.INT32] * 4, 2) == [H.HALF, H.HALF if ver == "5" else H.INT32]
        ser = p.serialize()
        assert ser["bert_embeddings_word_embeddings"].dtype == np.float16 and ser["bert_embeddings_layernorm_beta"].dtype == np.float32
        items = [(k, v if v.size > 1 else int(v[0])) for k, v in ser.items()]
        q = H.Plugin(EMB, ver, items, phase=H.RUNTIME)
        ser2 = q.serialize()
        assert ser.keys() == ser2.keys() and all(np.array_equal(ser[k], ser2[k]) for k in ser)
        q.close()
        p.close()
    # FP32 field data is converted to the FP16 table type
    p = H.Plugin(EMB, "4", [(k, v.astype(np.float32) if isinstance(v, np.ndarray) else v) for k, v in _emb_fields()])
    assert p.serialize()["bert_embeddings_word_embeddings"].dtype == np.float16
    p.close()


def test_skip_ln_variants():
    ld = 768
    g, b, bias = (np.ones(ld, np.float32), np.zeros(ld, np.float32), np.full(ld, 0.5, np.float32))
    p5 = H.Plugin(SKIP, "5", [("type_id", 1), ("ld", ld), ("beta", b), ("gamma", g), ("bias", bias)])
    assert p5.ok
    ser = p5.serialize()
    assert ser["beta"].dtype == np.float16 and "bias" in ser and int(ser["ld"][0]) == ld
    d = [H.make_dyn((128, 2, ld, 1, 1), H.HALF)] * 3
    assert all(p5.supports(i, d, 2, 1) for i in range(3))
    assert p5.output_shapes([(128, 2, ld, 1, 1)] * 2, 1) == [(128, 2, ld, 1, 1)]
    p5.close()
    p6 = H.Plugin(SKIP, "6", [("type_id", 2), ("beta", b), ("gamma", g)])  # INT8 I/O: FP16 parameters, CHW32
    assert p6.ok and "ld" not in p6.serialize() and p6.serialize()["gamma"].dtype == np.float16
    d8 = [H.make_dyn((500, ld, 1, 1), H.INT8, H.CHW32)] * 3
    assert all(p6.supports(i, d8, 2, 1) for i in range(3))
    assert not p6.supports(0, [H.make_dyn((500, ld, 1, 1), H.INT8, H.LINEAR)] * 3, 2, 1)
    p6.close()
    assert not H.Plugin(SKIP, "5", [("type_id", 1), ("ld", 100), ("beta", b), ("gamma", g)]).ok  # ld != len(beta)
    for ver, n_out in (("7", 1), ("8", 2)):
        p = H.Plugin(SKIP, ver, [("beta", b), ("gamma", g)])
        assert p.ok and p.nb_outputs() == n_out
        di = [H.make_dyn((1, ld, 999, 1), H.INT8, H.CHW32)] * (2 + n_out)
        assert all(p.supports(i, di, 2, n_out) for i in range(2 + n_out))
        assert p.output_shapes([(1, ld, 999, 1)] * 2, n_out) == [(1, ld, 999, 1)] * n_out
        assert set(p.serialize()) == {"beta", "gamma"} and p.serialize()["beta"].dtype == np.float16
        p.close()


def test_fc_plugin_host_side():
    K, out = 96, 48
    W = np.random.default_rng(0).standard_normal(K * out).astype(np.float32)
    p = H.Plugin(FC, "2", [("out_dims", out), ("type_id", 1), ("W", W)])
    assert p.ok
    assert p.output_shapes([(128, 2, K, 1, 1)], 1) == [(128, 2, out, 1, 1)]
    d = [H.make_dyn((128, 2, K, 1, 1), H.HALF), H.make_dyn((128, 2, out, 1, 1), H.HALF)]
    assert p.supports(0, d, 1, 1) and p.supports(1, d, 1, 1)
    assert p.configure(d[:1], d[1:]) == 0
    assert p.configure([H.make_dyn((128, 2, K + 16, 1, 1), H.HALF)], d[1:]) != 0  # K does not match W
    ser = p.serialize()
    assert ser["W"].dtype == np.float16 and ser["W"].size == K * out and int(ser["out_dims"][0]) == out
    assert np.array_equal(ser["W"], W.astype(np.float16))
    p.close()
    assert not H.Plugin(FC, "2", [("out_dims", 50), ("type_id", 1), ("W", W)]).ok  # W.count % out_dims != 0
