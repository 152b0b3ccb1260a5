"""The bounded device wait runs out, safely: the library's wait routine waits (1 ms instead of the kernels' 2 s) on an
mbarrier that nothing arrives at. The kernel must return by itself, the status word must carry the wait's code through
bert_b200_read_status_word, and the next ordinary kernel on the same stream must run and be right. No GPU fault is
involved: the wait is the product's own polling loop with its own time limit."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from oracle import bert_oracle as O

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_and_context_stays_usable(cuda):
    import tensorrt_b200 as T
    from tensorrt_b200._lib import lib

    status = torch.zeros(4, dtype=torch.int32, device=cuda)
    done = torch.full((1,), 7, dtype=torch.int32, device=cuda)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    st = lib.bert_b200_selftest_wait_expiry(stream, 1_000_000, C.c_void_p(status.data_ptr()), C.c_void_p(done.data_ptr()))
    assert st == 0, lib.bert_b200_last_error()
    # an ordinary kernel right behind it on the same stream
    rng = np.random.default_rng(0)
    x, s = (rng.standard_normal((64, 256)).astype(np.float16) for _ in range(2))
    g, b = np.ones(256, np.float16), np.zeros(256, np.float16)
    dev = lambda a: torch.from_numpy(a).to(cuda)
    y = T.skip_layer_norm(dev(x), dev(s), dev(g), dev(b))
    v = C.c_uint32(0)
    assert lib.bert_b200_read_status_word(C.c_void_p(status.data_ptr()), stream, C.byref(v)) == 0
    elapsed = time.perf_counter() - t0
    assert v.value == 1                      # kWaitTmaFull: the first waiter's code; the second saw the flag and left
    assert int(done[0]) == 0                 # the wait reported failure, it did not pretend to have completed
    assert elapsed < 1.0                     # 1 ms limit + 0.1 ms drain, not the kernels' 2 s
    assert O.close_abs_or_rel(y.cpu().numpy(), O.skip_layer_norm(x, s, g, b), 1e-2, 1e-2)[0]
    # limits beyond 100 ms are refused on the host
    assert lib.bert_b200_selftest_wait_expiry(stream, 10_000_000_000, C.c_void_p(status.data_ptr()), None) == 2
