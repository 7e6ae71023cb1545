"""RotaryEmbeddingESM with the interface of the reference (inf_llm/attention/rope.py:4-112),
computed by the CUDA kernels of libinfllm_b200 (infllm_rope_table / infllm_rope_apply)."""
import ctypes

import torch

from .. import _lib


class RotaryEmbeddingESM(torch.nn.Module):
    """Half-rotation RoPE; fp32 math, result cast back to the input dtype.

    Same constructor and methods as the reference class: `forward(q, k)` rotates keys to
    positions 0..Lk-1 and queries to Lk-Lq..Lk-1 (rope.py:107-112);
    `apply_rotary_pos_emb_one_angle(x, index)` rotates every row to position index-1
    (rope.py:89-104).  The context memory reads `dim`, `base` and `distance_scale` from it."""

    def __init__(self, dim, base=10000, distance_scale=1):
        super().__init__()
        self.dim = dim
        self.base = base
        self.distance_scale = distance_scale
        # rope.py:22-24, computed on the host so that construction needs no device
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._seq_len_cached = -1
        self._cos = None
        self._sin = None

    def _tables(self, length, device):
        if self._cos is None or length > self._seq_len_cached or self._cos.device != device:
            n = max(length, 2 * max(self._seq_len_cached, 0), 64)
            self._cos = torch.empty((n, self.dim // 2), dtype=torch.float32, device=device)
            self._sin = torch.empty_like(self._cos)
            inv = self.inv_freq.detach().to("cpu", torch.float32).contiguous()
            _lib.check(_lib.lib.infllm_rope_table(
                ctypes.cast(inv.data_ptr(), ctypes.POINTER(ctypes.c_float)), float(self.distance_scale), self.dim, n,
                self._cos.data_ptr(), self._sin.data_ptr(), _lib.stream_ptr(device)))
            self._seq_len_cached = n
        return self._cos, self._sin

    def _update_cos_sin_tables_len(self, seq_len, device, dim=None):
        """Kept for callers of the reference interface (context_manager.py:345-347)."""
        return self._tables(seq_len, torch.device(device))

    def _rotate(self, x, pos0, step):
        _lib.require_cuda(x, "RoPE input")
        if x.size(-1) != self.dim:
            raise ValueError(f"last dimension {x.size(-1)} != rotary dim {self.dim}")
        shape = x.shape
        length = shape[-2]
        x3 = x.reshape(-1, length, self.dim)
        if x3.stride(-1) != 1:
            x3 = x3.contiguous()
        out = torch.empty(x3.shape, dtype=x.dtype, device=x.device)
        need = pos0 + (length - 1) * step + 1 if length else 1
        cos, sin = self._tables(need, x.device)
        _lib.check(_lib.lib.infllm_rope_apply(
            x3.data_ptr(), x3.stride(0), x3.stride(1), out.data_ptr(), out.stride(0), out.stride(1), x3.size(0),
            length, self.dim, cos.data_ptr(), sin.data_ptr(), cos.size(0), pos0, step, _lib.dtype_code(x.dtype),
            _lib.stream_ptr(x.device)))
        return out.view(shape)

    def apply_rotary_pos_emb_one_angle(self, x, index):
        return self._rotate(x, index - 1, 0)

    def apply_rotary_pos_emb(self, x, length, right, cos=None, sin=None):
        """Rows 0..length-1 of x rotated to positions right-length..right-1 (rope.py:35-47).  The reference takes
        its cached tables as arguments; this class keeps its own, so `cos` and `sin` are ignored."""
        if x.size(-2) != length:
            raise ValueError(f"x has {x.size(-2)} rows, length says {length}")
        return self._rotate(x, right - length, 1)

    # the reference exposes its cached tables under these names (stream_llm.py:74 passes them back in)
    _cos_cached = None
    _sin_cached = None

    def forward(self, q, k, seq_dim=-2):
        if seq_dim not in (-2, q.dim() - 2):
            raise ValueError("the sequence dimension must be the second to last")
        lq, lk = q.size(-2), k.size(-2)
        return self._rotate(q, lk - lq, 1), self._rotate(k, 0, 1)
