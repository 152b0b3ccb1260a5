"""Legacy IPluginV2DynamicExt versions (QKV 1-3, Emb 1-3, SkipLN 1-4): interface behaviour and the flat serialisation
buffers, byte for byte in the reference's field order and widths
(plugin/bertQKVToContextPlugin/qkvToContextPluginLegacy.cpp:399-422, 909-925,
 plugin/bertQKVToContextPlugin/qkvToContextInt8InterleavedPluginLegacy.cpp:203-216,
 plugin/embLayerNormPlugin/embLayerNormPluginLegacy.cpp:451-470, embLayerNormVarSeqlenPluginLegacy.cpp:545-562,
 plugin/skipLayerNormPlugin/skipLayerNormPluginLegacy.cpp:381-397, skipLayerNormInt8InterleavedPluginLegacy.cpp:426-435).
No GPU needed: nothing is enqueued."""
import struct

import numpy as np

from tensorrt_b200 import plugin_harness as H

EMB, QKV, SKIP = ("CustomEmbLayerNormPluginDynamic", "CustomQKVToContextPluginDynamic", "CustomSkipLayerNormPluginDynamic")


def test_skip_ln_legacy_flat_buffer_and_round_trip():
    rng = np.random.default_rng(0)
    ld = 64
    beta, gamma, bias = (rng.standard_normal(ld).astype(np.float32) for _ in range(3))
    for version, items in (("1", [("ld", ld), ("type_id", 1)]), ("2", [("type_id", 1)])):
        p = H.LegacyPlugin(SKIP, version, items + [("beta", beta), ("gamma", gamma), ("bias", bias)])
        assert p.ok and p.info() == (SKIP, version, "")
        assert p.nb_outputs() == 1
        assert p.output_dims(0, [(128, 4, ld, 1, 1), (128, 4, ld, 1, 1)]) == (128, 4, ld, 1, 1)
        assert p.output_type(0, [H.HALF, H.HALF]) == H.HALF
        d = H.make_desc((128, 4, ld, 1, 1), H.HALF)
        assert p.supports(2, [d, d, d], 2, 1)
        assert not p.supports(1, [d, H.make_desc((128, 4, ld, 1, 1), H.FLOAT), d], 2, 1)
        blob = p.serialize()
        h16 = lambda a: a.astype(np.float16).tobytes()
        want = struct.pack("<iiQB", H.HALF, H.HALF, ld, 1) + h16(beta) + h16(gamma) + h16(bias)
        assert blob == want
        q = H.LegacyPlugin(SKIP, version, serialized=blob)
        assert q.ok and q.serialize() == blob
        c = q.clone()
        assert c.ok and c.serialize() == blob
        for o in (p, q, c):
            o.close()
    # INT8 I/O keeps FP16 parameters; no bias; FP32 type keeps FP32 parameters
    p = H.LegacyPlugin(SKIP, "2", [("type_id", 2), ("beta", beta), ("gamma", gamma)])
    assert p.serialize() == struct.pack("<iiQB", H.INT8, H.HALF, ld, 0) + beta.astype(np.float16).tobytes() + gamma.astype(np.float16).tobytes()
    p.close()
    p = H.LegacyPlugin(SKIP, "1", [("ld", ld), ("type_id", 0), ("beta", beta), ("gamma", gamma)])
    assert p.serialize() == struct.pack("<iiQB", H.FLOAT, H.FLOAT, ld, 0) + beta.tobytes() + gamma.tobytes()
    p.close()


def test_skip_ln_interleaved_legacy():
    rng = np.random.default_rng(1)
    ld = 96
    beta, gamma = (rng.standard_normal(ld).astype(np.float16) for _ in range(2))
    for version in ("3", "4"):
        p = H.LegacyPlugin(SKIP, version, [("beta", beta), ("gamma", gamma)])
        assert p.ok and p.nb_outputs() == (1 if version == "3" else 2)
        blob = p.serialize()
        assert blob == struct.pack("<Q", ld) + beta.tobytes() + gamma.tobytes()
        q = H.LegacyPlugin(SKIP, version, serialized=blob)
        assert q.ok and q.serialize() == blob
        d = H.make_desc((1, ld, 200, 1), H.INT8, H.CHW32)
        assert q.supports(0, [d, d] + [d] * q.nb_outputs(), 2, q.nb_outputs())
        p.close()
        q.close()


def test_qkv_legacy_flat_buffers():
    # version 1: fixed length
    p = H.LegacyPlugin(QKV, "1", [("type_id", 1), ("hidden_size", 768), ("num_heads", 12), ("has_mask", 1)])
    assert p.ok and p.nb_outputs() == 1
    assert p.output_dims(0, [(128, 8, 2304, 1, 1), (8, 1)]) == (128, 8, 768, 1, 1)
    qkv = H.make_dyn((128, 8, 2304, 1, 1), H.HALF)
    p.configure([qkv, H.make_dyn((8, 1), H.INT32)], [H.make_dyn((128, 8, 768, 1, 1), H.HALF)])
    blob = p.serialize()
    # type, heads, head size, has_mask (1 byte), hidden, SM, S, B, dq_probs, "no unfused runner"
    t, heads, d, mask, hidden, sm, S, B, dq, has_unfused = struct.unpack("<iiiBiiiifi", blob)
    assert (t, heads, d, mask, hidden, S, B, has_unfused) == (1, 12, 64, 1, 768, 128, 8, 0) and sm >= 75
    q = H.LegacyPlugin(QKV, "1", serialized=blob)
    assert q.ok and q.serialize() == blob
    # a buffer written by the reference carries its unfused runner state at the end: accepted and ignored
    ref_blob = blob[:-4] + struct.pack("<i", 1) + struct.pack("<iiiii", 99, 99, 128, 8, 64)
    r = H.LegacyPlugin(QKV, "1", serialized=ref_blob)
    assert r.ok and r.serialize() == blob
    assert not H.LegacyPlugin(QKV, "1", serialized=blob[:10]).ok  # truncated
    for o in (p, q, r):
        o.close()

    # version 2: variable sequence length (INT8 with dq_probs)
    p = H.LegacyPlugin(QKV, "2", [("type_id", 2), ("hidden_size", 1024), ("num_heads", 16), ("has_mask", 1),
                                   ("dq_probs", 1.0 / 127), ("var_seqlen", 1), ("use_int8_scale_max", 1)])
    assert p.ok
    assert p.output_dims(0, [(5000, 3072, 1, 1), (1,), (65,), (384,)]) == (5000, 1024, 1, 1)
    blob = p.serialize()
    vals = struct.unpack("<iiiBiiiifBiBiii", blob)
    assert vals[:5] == (2, 16, 64, 1, 1024) and abs(vals[8] - 1.0 / 127) < 1e-9 and vals[9:12] == (1, 64, 1)
    q = H.LegacyPlugin(QKV, "2", serialized=blob)
    assert q.ok and q.serialize() == blob
    p.close()
    q.close()

    # version 3: INT8 interleaved
    p = H.LegacyPlugin(QKV, "3", [("hidden_size", 1024), ("num_heads", 16), ("dq_probs", 1.0 / 127),
                                   ("use_int8_scale_max", 1), ("use_explicit_int8", 1), ("input_qkv_scale", 0.05),
                                   ("output_ctx_scale", 0.02)])
    assert p.ok
    blob = p.serialize()
    heads, d, hidden, sm, S, B, dq, smax, explicit, sq, sc = struct.unpack("<iiiiiifBBff", blob)
    assert (heads, d, hidden, smax, explicit) == (16, 64, 1024, 1, 1) and abs(sq - 0.05) < 1e-7 and abs(sc - 0.02) < 1e-7
    q = H.LegacyPlugin(QKV, "3", serialized=blob)
    assert q.ok and q.serialize() == blob
    p.close()
    q.close()


def test_emb_legacy_flat_buffers():
    rng = np.random.default_rng(2)
    E, vocab = 32, 50
    beta, gamma = (rng.standard_normal(E).astype(np.float32) for _ in range(2))
    word = rng.standard_normal(vocab * E).astype(np.float16)
    tok = rng.standard_normal(2 * E).astype(np.float16)
    pos = rng.standard_normal(20 * E).astype(np.float16)
    weights = [("bert_embeddings_layernorm_beta", beta), ("bert_embeddings_layernorm_gamma", gamma),
               ("bert_embeddings_word_embeddings", word), ("bert_embeddings_token_type_embeddings", tok),
               ("bert_embeddings_position_embeddings", pos)]
    # version 1: fixed length with mask index output
    p = H.LegacyPlugin(EMB, "1", weights + [("output_fp16", 1), ("full_mask", 0), ("mha_type_id", 1)])
    assert p.ok and p.nb_outputs() == 2
    assert p.output_dims(0, [(16, 4), (16, 4), (16, 4)]) == (16, 4, E, 1, 1)
    blob = p.serialize()
    head = struct.calcsize("<iiQQQQQBi")
    t, mha, ld, S, wv, pv, tv, full, sm = struct.unpack("<iiQQQQQBi", blob[:head])
    assert (t, mha, ld, wv, pv, tv, full) == (1, 1, E, vocab, 20, 2, 0)
    # parameters: beta, gamma (FP32), then word, position, token-type tables in the output type
    assert blob[head:] == beta.tobytes() + gamma.tobytes() + word.tobytes() + pos.tobytes() + tok.tobytes()
    q = H.LegacyPlugin(EMB, "1", serialized=blob)
    assert q.ok and q.serialize() == blob
    p.close()
    q.close()
    # versions 2 / 3: variable sequence length
    for version, nb_out in (("2", 2), ("3", 2)):
        p = H.LegacyPlugin(EMB, version, weights + [("output_fp16", 1)])
        assert p.ok and p.nb_outputs() == nb_out
        blob = p.serialize()
        head = struct.calcsize("<iQQQQi")
        t, ld, wv, pv, tv, mask_t = struct.unpack("<iQQQQi", blob[:head])
        assert (t, ld, wv, pv, tv) == (1, E, vocab, 20, 2)
        assert blob[head:] == beta.tobytes() + gamma.tobytes() + word.tobytes() + pos.tobytes() + tok.tobytes()
        q = H.LegacyPlugin(EMB, version, serialized=blob)
        assert q.ok and q.serialize() == blob
        p.close()
        q.close()


def test_fc_v1_flat_buffer():
    """CustomFCPluginDynamic version 1 is an IPluginV2DynamicExt as in the reference, serialised as
    type, out_dims (8 bytes), number of weights (8 bytes), Nmax, K, the 64-byte cuBLASLt algorithm blob, then W
    (plugin/fcPlugin/fcPlugin.cpp:661-673); bias / activation of this library follow in a tagged block."""
    FC = "CustomFCPluginDynamic"
    rng = np.random.default_rng(3)
    K, out = 48, 32
    W = rng.standard_normal(K * out).astype(np.float32)
    p = H.LegacyPlugin(FC, "1", [("out_dims", out), ("type_id", 1), ("W", W)])
    assert p.ok and p.info() == (FC, "1", "") and p.nb_outputs() == 1
    assert p.output_dims(0, [(7, 3, K, 1, 1)]) == (7, 3, out, 1, 1)
    blob = p.serialize()
    head = struct.calcsize("<iQQii")
    assert struct.unpack("<iQQii", blob[:head]) == (1, out, K * out, 0, K)
    assert blob[head:head + 64] == bytes(64)
    assert blob[head + 64:] == W.astype(np.float16).tobytes()
    q = H.LegacyPlugin(FC, "1", serialized=blob)
    assert q.ok and q.serialize() == blob
    # a buffer written by the reference carries a non-zero algorithm blob: accepted
    ref_blob = blob[:head] + bytes(range(64)) + blob[head + 64:]
    r = H.LegacyPlugin(FC, "1", serialized=ref_blob)
    assert r.ok and r.serialize() == blob
    for o in (p, q, r):
        o.close()
    bias = rng.standard_normal(out).astype(np.float32)
    p = H.LegacyPlugin(FC, "1", [("out_dims", out), ("type_id", 0), ("W", W), ("bias", bias), ("activation", 1)])
    blob = p.serialize()
    assert blob[head + 64:head + 64 + W.nbytes] == W.tobytes()
    assert blob[head + 64 + W.nbytes:] == struct.pack("<IiB", 0x30303242, 1, 1) + bias.tobytes()
    q = H.LegacyPlugin(FC, "1", serialized=blob)
    assert q.ok and q.serialize() == blob
    p.close()
    q.close()
