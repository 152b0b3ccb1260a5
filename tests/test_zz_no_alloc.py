"""The workspace-free encoder entry point (bert_b200_encoder_forward_static) against the ordinary one.

This file sorts last on purpose: a run that stops at the first failure has then already exercised everything else.
The entry point is for callers that cannot allocate device memory (see include/bert_b200.h); its scratch is a fixed
buffer inside the library that all calls share, so the test calls it twice in a row, with different inputs, and
checks both results against bert_b200_encoder_forward through the C ABI.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def _t(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _inputs(rng, lengths):
    lengths = np.array(lengths, dtype=np.int32)
    cu = O.cu_seqlens(lengths)
    total = int(cu[-1])
    return (rng.integers(0, 1000, size=total).astype(np.int32), rng.integers(0, 2, size=total).astype(np.int32), cu,
            total, int(lengths.max()))


@pytest.mark.parametrize("mode", ["fp16", "int8"])
def test_forward_static_matches_forward_twice(cuda, mode):
    import tensorrt_b200 as T
    from tensorrt_b200._lib import lib

    rng = np.random.default_rng(5)
    p = O.make_bert_params(rng, 2, 128, 2, 512, vocab=1000)
    first = _inputs(rng, [128, 40, 7])
    second = _inputs(rng, [200, 1])          # other sizes: the shared buffer is carved differently the second time
    if mode == "int8":
        O.calibrate_int8(p, first[0], first[1], first[2], first[4])
    enc = T.BertEncoder(p, T.INT8 if mode == "int8" else T.FP16, cuda)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for ids, seg, cu, total, S in (first, second):
        d_ids, d_seg, d_cu = _t(ids, cuda), _t(seg, cuda), _t(cu, cuda)
        ref = enc.forward(d_ids, d_seg, d_cu, S)                       # existing entry point, caller's workspace
        out = torch.zeros((total, p.hidden), dtype=torch.float16, device=cuda)
        st = lib.bert_b200_encoder_forward_static(enc._h, stream, len(cu) - 1, total, S, C.c_void_p(d_ids.data_ptr()),
                                                  C.c_void_p(d_seg.data_ptr()), C.c_void_p(d_cu.data_ptr()),
                                                  C.c_void_p(out.data_ptr()))
        assert st == 0, lib.bert_b200_last_error()
        torch.cuda.synchronize()
        # the same kernels over the same carve of a different buffer: identical bits, not merely close
        assert torch.equal(out, ref)
        # "allocates nothing": a repeat of the call leaves the device's free memory where it was
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        st = lib.bert_b200_encoder_forward_static(enc._h, stream, len(cu) - 1, total, S, C.c_void_p(d_ids.data_ptr()),
                                                  C.c_void_p(d_seg.data_ptr()), C.c_void_p(d_cu.data_ptr()),
                                                  C.c_void_p(out.data_ptr()))
        assert st == 0, lib.bert_b200_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before
        assert torch.equal(out, ref)
    # per-kernel timing brackets launches with events the entry point would have to create: it refuses instead
    enc.enable_timing(True)
    ids, seg, cu, total, S = first
    d_ids, d_seg, d_cu = _t(ids, cuda), _t(seg, cuda), _t(cu, cuda)
    out = torch.zeros((total, p.hidden), dtype=torch.float16, device=cuda)
    st = lib.bert_b200_encoder_forward_static(enc._h, stream, len(cu) - 1, total, S, C.c_void_p(d_ids.data_ptr()),
                                              C.c_void_p(d_seg.data_ptr()), C.c_void_p(d_cu.data_ptr()),
                                              C.c_void_p(out.data_ptr()))
    assert st == 2, st                                                   # BERT_B200_BAD_PARAM
    assert "timing" in lib.bert_b200_last_error().decode()
    enc.enable_timing(False)
    enc.close()


def test_forward_static_rejects_sizes_beyond_its_buffer(cuda):
    import tensorrt_b200 as T
    from tensorrt_b200._lib import lib

    rng = np.random.default_rng(6)
    p = O.make_bert_params(rng, 1, 128, 2, 512, vocab=1000)
    enc = T.BertEncoder(p, T.FP16, cuda)
    limit = lib.bert_b200_encoder_static_workspace_limit()
    assert limit == 16 * 1024 * 1024
    total = 40000                                                        # needs far more than 16 MiB of scratch
    assert lib.bert_b200_encoder_workspace_size(C.byref(enc.cfg), total, 128) > limit
    ids = torch.zeros(total, dtype=torch.int32, device=cuda)
    cu = torch.arange(0, total + 1, total // 128, dtype=torch.int32, device=cuda)
    out = torch.empty((total, p.hidden), dtype=torch.float16, device=cuda)
    st = lib.bert_b200_encoder_forward_static(enc._h, None, 128, total, 384, C.c_void_p(ids.data_ptr()),
                                              C.c_void_p(ids.data_ptr()), C.c_void_p(cu.data_ptr()),
                                              C.c_void_p(out.data_ptr()))
    assert st == 3                                                       # BERT_B200_NOT_SUPPORTED
    msg = lib.bert_b200_last_error().decode()
    assert "16777216" in msg and "scratch" in msg
    enc.close()
