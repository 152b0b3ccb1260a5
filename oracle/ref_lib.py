"""ctypes front end of oracle/_ref/libref_bert.so (the reference's own kernels, see oracle/build_ref.py).
TEST INFRASTRUCTURE: imported only by tests and by tests/golden/make_golden.py."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libref_bert.so"


def available() -> bool:
    return LIB_PATH.exists()


class RefLib:
    def __init__(self):
        self.lib = C.CDLL(str(LIB_PATH))
        for n in ("ref_skip_layer_norm", "ref_skip_layer_norm_dqq", "ref_skip_layer_norm_interleaved", "ref_emb_layer_norm",
                  "ref_emb_layer_norm_var_seqlen", "ref_compute_mask_idx", "ref_convert_mask", "ref_fmha_v2", "ref_fmha_v1"):
            getattr(self.lib, n).restype = C.c_int32

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr()) if t is not None else None

    @staticmethod
    def _s():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _check(self, st, what):
        torch.cuda.synchronize()
        if st != 0:
            raise RuntimeError(f"reference {what} returned {st}")

    def skip_layer_norm(self, x, skip, gamma, beta, bias=None):
        out = torch.empty_like(x)
        tid = 1 if x.dtype == torch.float16 else 0
        self._check(self.lib.ref_skip_layer_norm(self._s(), tid, x.shape[-1], x.numel(), self._p(x), self._p(skip), self._p(beta),
                                                 self._p(gamma), self._p(out), self._p(bias)), "computeSkipLayerNorm")
        return out

    def skip_layer_norm_dqq(self, x, skip, gamma, beta, bias, dq_in, dq_skip, q):
        out = torch.empty_like(x)
        self._check(self.lib.ref_skip_layer_norm_dqq(self._s(), x.shape[-1], x.numel(), self._p(x), self._p(skip), self._p(beta),
                                                     self._p(gamma), self._p(out), self._p(bias), C.c_float(dq_in),
                                                     C.c_float(dq_skip), C.c_float(q)), "computeSkipLayerNormDQQ")
        return out

    def skip_layer_norm_interleaved(self, variant, x, skip, gamma, beta, dq_in, dq_skip, q, q_skip):
        g, total, _ = x.shape
        out, pre = torch.empty_like(x), torch.empty_like(x)
        self._check(self.lib.ref_skip_layer_norm_interleaved(self._s(), variant, g * 32, total, self._p(x), self._p(skip),
                                                             self._p(beta), self._p(gamma), self._p(out), self._p(pre),
                                                             C.c_float(dq_in), C.c_float(dq_skip), C.c_float(q),
                                                             C.c_float(q_skip)), "launch_*_hface/mtron")
        return out, pre

    def emb_layer_norm(self, ids, seg, word, pos, tok, gamma, beta):
        S, B = ids.shape
        ld = word.shape[1]
        out = torch.empty((S, B, ld), dtype=word.dtype, device=word.device)
        tid = 1 if word.dtype == torch.float16 else 0
        self._check(self.lib.ref_emb_layer_norm(self._s(), tid, ld, B, S, self._p(ids), self._p(seg), self._p(beta), self._p(gamma),
                                                self._p(word), self._p(pos), self._p(tok), word.shape[0], tok.shape[0],
                                                self._p(out)), "embSkipLayerNorm")
        return out

    def emb_layer_norm_var_seqlen(self, ids, seg, cu, S, word, pos, tok, gamma, beta, mtron):
        total, ld, B = ids.shape[0], word.shape[1], cu.shape[0] - 1
        out = torch.empty((total, ld), dtype=torch.float16, device=word.device)
        skip = torch.empty_like(out) if mtron else None
        self._check(self.lib.ref_emb_layer_norm_var_seqlen(self._s(), ld, B, S, self._p(ids), self._p(seg), self._p(cu),
                                                           self._p(beta), self._p(gamma), self._p(word), self._p(pos),
                                                           self._p(tok), word.shape[0], tok.shape[0], self._p(out),
                                                           self._p(skip)), "embSkipLayerNormHFace/MTron")
        return out, skip

    def compute_mask_idx(self, mask):
        S, B = mask.shape
        out = torch.empty(B, dtype=torch.int32, device=mask.device)
        self._check(self.lib.ref_compute_mask_idx(self._s(), S, B, self._p(mask), self._p(out)), "computeMaskIdx")
        return out

    def convert_mask(self, mask, wm, wn):
        S, B = mask.shape
        xm = (S + 16 * wm - 1) // (16 * wm)
        out = torch.zeros((B, xm, wm * wn * 32), dtype=torch.int32, device=mask.device)
        self._check(self.lib.ref_convert_mask(S, B, wm, wn, 1, self._p(mask), self._p(out), self._s()), "convertMask")
        return out

    def fmha_v2(self, qkv, cu, B, S, N, d, scales=None, interleaved=False):
        """qkv FP16/INT8 [total, 3*N*d] (or CHW32 [3*N*d/32, total, 32]); returns the same form with N*d channels."""
        if interleaved:
            total = qkv.shape[1]
            out = torch.zeros((N * d // 32, total, 32), dtype=qkv.dtype, device=qkv.device)
        else:
            total = qkv.shape[0]
            out = torch.zeros((total, N * d), dtype=qkv.dtype, device=qkv.device)
        tid = 2 if qkv.dtype == torch.int8 else 1
        s1, ssm, s2 = scales if scales is not None else (d ** -0.5, 1.0, 1.0)
        st = self.lib.ref_fmha_v2(self._s(), tid, B, S, N, d, total, self._p(qkv), self._p(out), self._p(cu),
                                  1 if interleaved else 0, C.c_float(s1), C.c_float(ssm), C.c_float(s2))
        self._check(st, "fmha_v2 (precompiled sm100 kernel)")
        return out

    def fmha_v1(self, qkv, mask, N, d, scales=None):
        """Fixed-length kernels of plugin versions 1-3: qkv FP16/INT8 [S, B, 3*N*d], mask int32 [S, B] (1 = key
        present); returns [S, B, N*d]. S in {64, 96, 128, 384} (FP16) or {128, 384} (INT8)."""
        S, B = mask.shape
        wm, wn = (1, 8) if S == 384 else (2, 2)
        packed = self.convert_mask(mask, wm, wn)
        out = torch.zeros((S, B, N * d), dtype=qkv.dtype, device=qkv.device)
        tid = 2 if qkv.dtype == torch.int8 else 1
        s1, ssm, s2 = scales if scales is not None else (d ** -0.5, 1.0, 1.0)
        st = self.lib.ref_fmha_v1(self._s(), tid, B, S, N, d, self._p(qkv), self._p(out), self._p(packed), C.c_float(s1),
                                  C.c_float(ssm), C.c_float(s2))
        self._check(st, "fmha_v1 (precompiled sm100 kernel)")
        return out
