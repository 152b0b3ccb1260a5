"""BERT encoder object on top of the C++ driver (bert_b200_encoder_* in include/bert_b200.h).

Owns the device copies of the weights (made once, like the reference plugins do in their constructors,
plugin/common/bertCommon.h:447-457) and the workspace; the layer loop itself runs in C++.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .ops import FP16, INT8


def _dev(a, dtype, device, transpose=False):
    """numpy array or torch tensor -> contiguous device tensor of `dtype` (optionally transposed)."""
    t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))
    t = t.to(device=device)
    if transpose:
        t = t.t()
    return t.to(dtype).contiguous()


class BertEncoder:
    """`params` is any object with the attributes hidden, heads, ffn, word_emb, pos_emb, tok_emb, emb_gamma,
    emb_beta, dq_probs and layers[i].{w_qkv [E,3E], b_qkv, w_out, b_out, ln1_gamma, ln1_beta, w_ffn1, b_ffn1,
    w_ffn2, b_ffn2, ln2_gamma, ln2_beta, scales}. FC weights arrive as [in, out] (the reference FC plugin's `W`
    field, plugin/fcPlugin/README.md:45) and are stored transposed [out, in] for the K-major tensor-core tiles.
    For type_id INT8, layers[i].scales holds q_w_* (INT8 weights) and the s_* dequantisation steps."""

    def __init__(self, params, type_id=FP16, device="cuda:0"):
        self.device = torch.device(device)
        self.type_id = type_id
        self.hidden = params.hidden
        self.heads = params.heads
        self.ffn = params.ffn
        self._keep = []  # device tensors referenced by raw pointer from C++
        d = self.device

        def keep(t):
            self._keep.append(t)
            return C.c_void_p(t.data_ptr())

        self.word_emb = _dev(params.word_emb, torch.float16, d)
        self.pos_emb = _dev(params.pos_emb, torch.float16, d)
        self.tok_emb = _dev(params.tok_emb, torch.float16, d)
        self.emb_gamma = _dev(params.emb_gamma, torch.float32, d)
        self.emb_beta = _dev(params.emb_beta, torch.float32, d)
        n_layers = len(params.layers)
        self._layers = (_lib.LayerWeights * n_layers)()
        for i, lp in enumerate(params.layers):
            lw = self._layers[i]
            if type_id == INT8:
                s = lp.scales
                wq = lambda name: keep(_dev(s["q_" + name], torch.int8, d, transpose=True))
                lw.wt_qkv, lw.wt_out, lw.wt_ffn1, lw.wt_ffn2 = wq("w_qkv"), wq("w_out"), wq("w_ffn1"), wq("w_ffn2")
                lw.s_in, lw.s_wqkv, lw.s_qkv, lw.s_ctx = s["s_in"], s["s_w_qkv"], s["s_qkv"], s["s_ctx"]
                lw.s_wout, lw.s_attn_out, lw.s_ln1 = s["s_w_out"], s["s_attn_out"], s["s_ln1"]
                lw.s_wffn1, lw.s_ffn1, lw.s_wffn2, lw.s_ffn2, lw.s_out = (s["s_w_ffn1"], s["s_ffn1"], s["s_w_ffn2"],
                                                                          s["s_ffn2"], s["s_out"])
            else:
                wt = lambda a: keep(_dev(a, torch.float16, d, transpose=True))
                lw.wt_qkv, lw.wt_out, lw.wt_ffn1, lw.wt_ffn2 = wt(lp.w_qkv), wt(lp.w_out), wt(lp.w_ffn1), wt(lp.w_ffn2)
            lw.b_qkv = keep(_dev(lp.b_qkv, torch.float32, d))
            lw.b_ffn1 = keep(_dev(lp.b_ffn1, torch.float32, d))
            for name in ("b_out", "ln1_gamma", "ln1_beta", "b_ffn2", "ln2_gamma", "ln2_beta"):
                setattr(lw, name, keep(_dev(getattr(lp, name), torch.float16, d)))
        self.cfg = _lib.EncoderConfig(
            type_id, n_layers, params.hidden, params.heads, params.ffn, self.word_emb.shape[0], self.pos_emb.shape[0],
            self.tok_emb.shape[0], float(params.dq_probs), C.c_void_p(self.word_emb.data_ptr()),
            C.c_void_p(self.pos_emb.data_ptr()), C.c_void_p(self.tok_emb.data_ptr()),
            C.c_void_p(self.emb_gamma.data_ptr()), C.c_void_p(self.emb_beta.data_ptr()), self._layers)
        handle = C.c_void_p()
        check(lib.bert_b200_encoder_create(C.byref(self.cfg), C.byref(handle)), "encoder_create")
        self._h = handle
        self._ws = None
        self._ws_key = (0, 0)

    def close(self):
        if getattr(self, "_h", None):
            lib.bert_b200_encoder_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def _workspace(self, total, B):
        if self._ws is None or total > self._ws_key[0] or B > self._ws_key[1]:
            t, b = max(total, self._ws_key[0]), max(B, self._ws_key[1])
            n = lib.bert_b200_encoder_workspace_size(C.byref(self.cfg), t, b)
            if n < 0:
                raise RuntimeError("encoder_workspace_size failed")
            # torch's caching allocator returns 512-byte aligned blocks; over-allocate and align to 1024
            self._ws_raw = torch.empty(n + 1024, dtype=torch.uint8, device=self.device)
            off = (-self._ws_raw.data_ptr()) % 1024
            self._ws = self._ws_raw[off:off + n]
            self._ws_key = (t, b)
            self._ws_bytes = n
        return self._ws

    @property
    def launches_per_forward(self):
        return lib.bert_b200_encoder_last_launch_count(self._h)

    def forward(self, ids, seg, cu, max_seqlen, out=None):
        """ids/seg [total] int32, cu [B+1] int32, all on the device. Returns FP16 [total, E]."""
        total, B = ids.shape[0], cu.shape[0] - 1
        ws = self._workspace(total, B)
        self._last = (total, B)
        out = torch.empty((total, self.hidden), dtype=torch.float16, device=self.device) if out is None else out
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.bert_b200_encoder_forward(self._h, s, B, total, max_seqlen, C.c_void_p(ids.data_ptr()),
                                            C.c_void_p(seg.data_ptr()), C.c_void_p(cu.data_ptr()),
                                            C.c_void_p(ws.data_ptr()), self._ws_bytes, C.c_void_p(out.data_ptr())),
              "encoder_forward")
        return out

    def forward_host(self, ids_h, seg_h, cu_h, max_seqlen, out_dev, out_h):
        """Same through host (pinned) int32 tensors; the FP16 result lands in the host tensor out_h.
        Copies in, runs, copies out and synchronises the current stream."""
        total, B = ids_h.shape[0], cu_h.shape[0] - 1
        ws = self._workspace(total, B)
        self._last = (total, B)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.bert_b200_encoder_forward_host(self._h, s, B, total, max_seqlen, C.c_void_p(ids_h.data_ptr()),
                                                 C.c_void_p(seg_h.data_ptr()), C.c_void_p(cu_h.data_ptr()),
                                                 C.c_void_p(ws.data_ptr()), self._ws_bytes,
                                                 C.c_void_p(out_dev.data_ptr()), C.c_void_p(out_h.data_ptr())),
              "encoder_forward_host")
        return out_h

    def forward_host_async(self, ids_h, seg_h, cu_h, max_seqlen, out_dev, out_h, copy_stream, slot):
        """Pipelined form of forward_host: nothing is synchronised. The encoder runs on the current stream, the copy
        of the result into the pinned host tensor out_h on `copy_stream` (a torch.cuda.Stream), overlapping the next
        call. `slot` (0 / 1) names one of two (out_dev, out_h) pairs used alternately; wait_host(slot) blocks until
        that slot's out_h is complete."""
        total, B = ids_h.shape[0], cu_h.shape[0] - 1
        ws = self._workspace(total, B)
        self._last = (total, B)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.bert_b200_encoder_forward_host_async(self._h, s, C.c_void_p(copy_stream.cuda_stream), slot, B, total,
                                                       max_seqlen, C.c_void_p(ids_h.data_ptr()),
                                                       C.c_void_p(seg_h.data_ptr()), C.c_void_p(cu_h.data_ptr()),
                                                       C.c_void_p(ws.data_ptr()), self._ws_bytes,
                                                       C.c_void_p(out_dev.data_ptr()), C.c_void_p(out_h.data_ptr())),
              "encoder_forward_host_async")
        return out_h

    def wait_host(self, slot):
        check(lib.bert_b200_encoder_wait_host(self._h, slot), "encoder_wait_host")

    def enable_timing(self, on=True):
        """Bracket every kernel of forward() with CUDA events (see read_timing)."""
        check(lib.bert_b200_encoder_enable_timing(self._h, 1 if on else 0), "encoder_enable_timing")

    def read_timing(self, ms=None, launches=None):
        """Adds the last forward's per-kind milliseconds / launch counts to the given ctypes arrays
        (kinds: 0 emb, 1 fc, 2 mha, 3 skipln, 4 other) and returns them."""
        ms = (C.c_float * 5)() if ms is None else ms
        launches = (C.c_int32 * 5)() if launches is None else launches
        check(lib.bert_b200_encoder_read_timing(self._h, ms, launches), "encoder_read_timing")
        return ms, launches

    def calibrate(self, ids, seg, cu, max_seqlen):
        """Max calibration (FP16 encoder only): returns a float32 array [layers, 8] of |tensor| maxima in the order
        layer input, qkv, ctx, attention-out projection, ln1 output, ffn1 output, ffn2 output, layer output."""
        total, B = ids.shape[0], cu.shape[0] - 1
        ws = self._workspace(total, B)
        self._last = (total, B)
        n_layers = self.cfg.num_layers
        out = torch.empty((total, self.hidden), dtype=torch.float16, device=self.device)
        amax_dev = torch.zeros((n_layers, 8), dtype=torch.float32, device=self.device)
        amax_host = np.zeros((n_layers, 8), dtype=np.float32)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.bert_b200_encoder_calibrate(self._h, s, B, total, max_seqlen, C.c_void_p(ids.data_ptr()),
                                              C.c_void_p(seg.data_ptr()), C.c_void_p(cu.data_ptr()),
                                              C.c_void_p(ws.data_ptr()), self._ws_bytes, C.c_void_p(out.data_ptr()),
                                              C.c_void_p(amax_dev.data_ptr()),
                                              amax_host.ctypes.data_as(C.POINTER(C.c_float))), "encoder_calibrate")
        return amax_host

    def status_word(self):
        """Non-zero if a bounded device wait expired in the last forward (see bert_b200.h)."""
        if self._ws is None:
            return 0
        # the status word sits after ids, seg and cu in the workspace; read it through the C helper
        t, b = self._last
        off = 0
        for nbytes in (t * 4, t * 4, (b + 1) * 4):
            off = (off + nbytes + 1023) // 1024 * 1024
        v = C.c_uint32(0)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        check(lib.bert_b200_read_status_word(C.c_void_p(self._ws.data_ptr() + off), s, C.byref(v)), "read_status_word")
        return v.value
