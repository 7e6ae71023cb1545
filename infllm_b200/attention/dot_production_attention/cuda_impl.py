"""Multi-stage attention on the CUDA kernels of libinfllm_b200, with the interface of the
reference's MultiStageDotProductionAttention (dot_production_attention/base.py:3-30)."""
import torch

from ... import _lib


class CudaMultiStageDotProductionAttention:
    """append() any number of (q, k, v, mask) stages; the softmax is normalised jointly over all of
    them; get_result() returns (out (B, H, Lq, D) in q's dtype, [per-key score (B, H, Lk) or None]).

    Mirrors torch_impl.py:6-96 / triton_impl.py:488-556: `sliding_window` is None, an int w (meaning
    (Lk - Lq, w)) or (offset, size); with `complement_sliding_window` the kept pairs are
    dist >= size instead of 0 <= dist < size, dist = i - j + offset."""

    def __init__(self, q_shape, dtype, device):
        if len(q_shape) != 4:
            raise ValueError("q_shape must be (batch, heads, len_q, dim_head)")
        self.q_shape = tuple(q_shape)
        self.dtype = dtype
        self.device = torch.device(device)
        self._code = _lib.dtype_code(dtype)
        b, h, lq, d = self.q_shape
        self._acc = torch.empty((b, h, lq, d), dtype=torch.float32, device=self.device)
        self._m = torch.empty((b, h, lq), dtype=torch.float32, device=self.device)
        self._l = torch.empty((b, h, lq), dtype=torch.float32, device=self.device)
        self._stages = []
        self._first = True
        self.end = False
        self.ret = None
        self.score_list = []
        self.score_list_fp32 = []  # the same scores before rounding to the activation dtype

    def append(self, q, k, v, sliding_window=None, complement_sliding_window=False, end=False, get_score=False,
               *args, **kwargs):
        if self.end:
            raise RuntimeError("append after end=True")
        if tuple(q.shape) != self.q_shape:
            raise ValueError(f"q shape {tuple(q.shape)} != {self.q_shape}")
        for t, n in ((q, "q"), (k, "k"), (v, "v")):
            _lib.require_cuda(t, n)
            if t.dtype != self.dtype:
                raise TypeError(f"{n} dtype {t.dtype} != {self.dtype}")
        b, h, lq, d = self.q_shape
        hkv, lk = k.size(1), k.size(2)
        if sliding_window is None:
            mode, off, size = _lib.MASK_NONE, 0, 0
        else:
            if isinstance(sliding_window, int):
                sliding_window = (lk - lq, sliding_window)  # torch_impl.py:67-68
            off, size = int(sliding_window[0]), int(sliding_window[1])
            mode = _lib.MASK_COMPLEMENT if complement_sliding_window else _lib.MASK_WINDOW
        if q.stride(-1) != 1:
            q = q.contiguous()
        if k.stride(-1) != 1 or k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
        stream = _lib.stream_ptr(self.device)
        for bi in range(b):
            _lib.check(_lib.lib.infllm_attn_stage(
                q[bi].data_ptr(), q.stride(1), q.stride(2), k[bi].data_ptr() if lk else None, k.stride(1), k.stride(2),
                v[bi].data_ptr() if lk else None, v.stride(1), v.stride(2), h, hkv, lq, lk, d, mode, off, size,
                self._acc[bi].data_ptr(), self._m[bi].data_ptr(), self._l[bi].data_ptr(), int(self._first),
                self._code, stream))
        self._first = False
        self._stages.append((q, k, mode, off, size) if get_score else None)
        if end:
            self._finalize()

    def _finalize(self):
        self.end = True
        b, h, lq, d = self.q_shape
        self.ret = torch.empty(self.q_shape, dtype=self.dtype, device=self.device)
        lse = torch.empty((b, h, lq), dtype=torch.float32, device=self.device)
        stream = _lib.stream_ptr(self.device)
        for bi in range(b):
            _lib.check(_lib.lib.infllm_attn_finalize(
                self._acc[bi].data_ptr(), self._m[bi].data_ptr(), self._l[bi].data_ptr(), self.ret[bi].data_ptr(),
                self.ret.stride(1), self.ret.stride(2), lse[bi].data_ptr(), h, lq, d, self._code, stream))
        for st in self._stages:
            if st is None:
                self.score_list.append(None)
                self.score_list_fp32.append(None)
                continue
            q, k, mode, off, size = st
            lk, hkv = k.size(2), k.size(1)
            score = torch.zeros((b, h, lk), dtype=torch.float32, device=self.device)
            for bi in range(b):
                _lib.check(_lib.lib.infllm_attn_colsum(
                    q[bi].data_ptr(), q.stride(1), q.stride(2), k[bi].data_ptr() if lk else None, k.stride(1),
                    k.stride(2), h, hkv, lq, lk, d, mode, off, size, lse[bi].data_ptr(), score[bi].data_ptr(),
                    score.stride(1), 0, self._code, stream))
            self.score_list_fp32.append(score)
            self.score_list.append(score.to(self.dtype))
        self._stages = []

    def get_result(self):
        return self.ret, self.score_list
