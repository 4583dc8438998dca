"""The kernel library as Python calls: one method per entry point of ``csrc``.

Arguments are torch tensors on the GPU; the methods check dtypes, shapes and contiguity, pass raw
pointers and the current CUDA stream to the C entry points, and turn a refusal into an exception
with the library's own sentence.  There is no CPU path and no substitute: if the library cannot be
built or loaded, ``Kernels()`` raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import BuildError, library_path

F32, BF16 = 0, 1
ABI_VERSION = 30
SPLIT_BLOCKS = 296          # blocks of the decode attention that one wave holds (two per SM, 148 SMs)
TC_ATTENTION_MIN_LEN = 256  # prompts from this length on take the tcgen05 attention (head_dim 64 or 128)
SPLIT_FEW_BLOCKS = 148      # below this many blocks at 8 splits, more splits are taken
SHORT_CONTEXT_BYTES = 96 * 1024   # up to this many bytes of keys and values (one kv head) a sequence's context is one block's
                                  # work in the decode attention: no split, no merge kernel.  Measured at the 7B shape
                                  # (head_dim 128: 192 positions), batch 1 and 8: up to ~190 positions 4.4 to 6.1 us against
                                  # 6.1 to 6.6 with splits, from ~280 on 7.7 to 10 against 5.7 to 7.4; at head_dim 64 the
                                  # same bytes are 384 positions (Qwen2.5-0.5B, batch 1, contexts 137 to 265: 0.526 ms a
                                  # step without splits, 0.567 with)


def short_context(head_dim: int) -> int:
    """Positions (whole pages of 64) up to which the decode attention of this head size runs without splits."""
    return SHORT_CONTEXT_BYTES // (4 * head_dim) // 64 * 64


# epilogues of the skinny product
SK_STORE, SK_ACCUM, SK_SWIGLU, SK_STORE_F32 = 0, 1, 2, 3
# activations of a gated feed-forward's gate (CIMA_ACT_* of csrc/common.cuh), by the names config files use
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu_new": 1, "gelu": 2, "relu": 3,
               # min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1): the kernels that take it take the limit L beside the code
               "swish_clamped": 4}
GATED_ONLY = 4              # codes from here on are forms of the whole gated middle, not activations of the gate alone
# activations of an ungated feed-forward's middle (``activate``): the gate activations and the square of ReLU
UNGATED_ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu_new": 1, "gelu": 2, "relu": 3, "relu2": 5}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt is torch.float32:
        return F32
    if dt is torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is neither float32 nor bfloat16")


_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "cima_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp, _vp, _vp, _vp],
    "cima_rmsnorm": [_vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "cima_swiglu": [_vp, _vp, _i, _i, _i, _i, _f, _vp],
    "cima_add_residual": [_vp, _vp, _i, _sz, _vp],
    "cima_gather_rows": [_vp, _vp, _vp, _i, _i, _vp],
    "cima_add_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "cima_decode_advance": [_vp, _vp, _vp, _vp, _i, _vp],
    "cima_linear_plain": [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_linear_skinny": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _f, _vp],
    "cima_linear_skinny_norm": [_vp, _vp, _i, _f, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_qkv_rope_skinny": [_vp, _vp, _i, _f, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                             _i, _i, _i, _i, _vp],
    "cima_rope_append": [_vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _f, _vp],
    "cima_attention_plain": [_vp, _i, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                             _f, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "cima_attention_decode": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _f, _i, _i, _vp, _vp],
    "cima_attention_prefill": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _f, _i, _i, _vp, _vp],
    "cima_attention_extend": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _i, _f, _i, _i, _vp, _vp],
    "cima_attention_extend_tc": [_vp, _i, _vp, _vp, _vp, _vp, ctypes.c_longlong, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                 _f, _i, _vp, _i, _f, _vp, _vp],
    "cima_short_conv": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_dyt": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "cima_dyt_add": [_vp, _vp, _vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "cima_embed_bigram": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _f, _i, ctypes.c_longlong, ctypes.c_longlong, _vp, _vp, _vp, _vp, _vp,
                          _i, _vp],
    "cima_recurrence": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_delta_prepare": [_vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "cima_group_rmsnorm_gate": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _vp],
    "cima_rms_mean": [_vp, _vp, _i, _vp, _i, _i, _f, _i, _vp],
    "cima_moe_route": [_vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cima_moe_sort": [_vp, _i, _i, _vp, _vp, _vp, _vp],
    "cima_moe_gemm": [_vp, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
    "cima_moe_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp],
    "cima_moe_sort_tiles": [_vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "cima_moe_gather_rows": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "cima_moe_few": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
    "cima_gemm_tcgen05_pair_grouped": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp],
    "cima_depth_average": [_vp, ctypes.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _i, _vp, _vp, _vp, _vp],
    "cima_latent_append": [_vp, _i, _i, _vp, _f, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp],
    "cima_head_linear": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "cima_latent_prepare": [_vp, _i, _i, _i, _vp, _vp, _i, _vp, _f, _i, _i, _vp, _f, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp,
                            _vp, _i, _i, _i, _vp],
    "cima_rope_rows": [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _vp, _f, _i, _vp, _i, _vp],
    "cima_hyper_connect": [_vp, _vp, _vp, _vp, _f, _i, _vp, _vp, _f, _vp, _i, _i, _i, _i, _vp],
    "cima_activate": [_vp, _i, _sz, _i, _vp],

    "cima_head_linear_append": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _vp, _vp, _vp,
                                _i, _vp],
    "cima_attention_prefill_tc": [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp, _f, _vp, _vp],
    "cima_gemm_tcgen05_pair": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "cima_diff_combine": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _f, _vp],
    "cima_scale_add_group_rmsnorm": [_vp, _vp, _f, _vp, _vp, _i, _i, _i, _i, _f, _vp],
    "cima_cast_rows": [_vp, _vp, _i, _sz, _vp],
    "cima_softcap": [_vp, _sz, _f, _vp],
    "cima_argmax": [_vp, _i, _i, _i, _vp, _vp],
    "cima_sample": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cima_sample_general": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda dev: torch.cuda.current_stream(dev).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Kernels:
    """Loads (building first if needed) the CUDA library; fails loudly when it cannot."""

    def __init__(self, verbose: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this library runs on the GPU only")
        try:
            path = library_path(build=True, verbose=verbose)
        except BuildError as e:
            raise KernelError(f"the CUDA kernel library is missing and could not be built: {e}") from e
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from e
        self.path = path
        self.lib.cima_last_error.restype = ctypes.c_char_p
        self.lib.cima_abi_version.restype = ctypes.c_int
        if self.lib.cima_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} has ABI {self.lib.cima_abi_version()}, this package wants {ABI_VERSION}")
        for name, sig in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = sig
            fn.restype = ctypes.c_int
        self.launches = 0
        self.library_launches = 0   # matrix products handed to the library (not counted in ``launches``)
        self._scratch_bufs = {}
        self._retired = []          # replaced scratch buffers, kept alive for the graphs recorded with them
        self._error_flag = None
        self.profile = None         # a StepProfile while a step's launches are being counted and timed

    # ------------------------------------------------------------------ plumbing
    def _admit(self, name: str, nbytes: float = 0, flops: float = 0) -> bool:
        """Asked before every launch.  Without a profile it says yes.  With one (``self.profile``, see
        ``cima_b200.engine.profile``) the launch is noted with the bytes it has to move and the operations it has
        to do, and launches beyond the profile's limit are left out: a step cut after its n-th launch, timed
        against the step cut after launch n - 1, gives launch n's time inside the step."""
        p = self.profile
        return True if p is None else p.admit(name, nbytes, flops)

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            raise KernelError(f"{what}: {self.lib.cima_last_error().decode()} (code {code})")

    @staticmethod
    def _stream() -> int:
        """The current stream's handle (the capture stream while a graph is recorded).  Asked of torch's C layer
        directly: the Python wrapper costs 15 us a call, and a prompt's step makes some 150 of them."""
        return _raw_stream(torch.cuda.current_device())

    @staticmethod
    def _need(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
        if not t.is_cuda:
            raise KernelError(f"{name} is on {t.device}; the kernels take GPU tensors only")
        if dtype is not None and t.dtype is not dtype:
            raise KernelError(f"{name} is {t.dtype}, expected {dtype}")
        if dims is not None and t.dim() != dims:
            raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")
        if not t.is_contiguous():
            raise KernelError(f"{name} is not contiguous")

    # ------------------------------------------------------------------ elementwise
    def embed(self, ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0,
              ssq: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
              xw: Optional[torch.Tensor] = None) -> None:
        """x[t] = scale * table[ids[t]]; ``ssq`` [T, 1] (optional) receives each row's sum of squares, ``xw``
        [T, H] bf16 (optional) the rows times ``w_next`` (the weight of the norm that follows)."""
        self._need(ids, "ids", torch.int32, 1); self._need(table, "table", None, 2); self._need(x, "x", torch.float32, 2)
        T, (V, H) = ids.numel(), table.shape
        if tuple(x.shape) != (T, H):
            raise KernelError(f"embed: x is {tuple(x.shape)}, expected {(T, H)}")
        if ssq is not None:
            self._need(ssq, "ssq", torch.float32, 2)
            if tuple(ssq.shape) != (T, 1):
                raise KernelError(f"embed: ssq is {tuple(ssq.shape)}, expected {(T, 1)}")
        if xw is not None:
            self._need(xw, "xw", torch.bfloat16, 2); self._need(w_next, "w_next", torch.float32, 1)
            if tuple(xw.shape) != (T, H) or w_next.numel() != H:
                raise KernelError(f"embed: xw {tuple(xw.shape)} / w_next {tuple(w_next.shape)} do not fit {(T, H)}")
        if not self._admit("embed", T * H * (table.element_size() + 4)): return
        self._check(self.lib.cima_embed(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), x.data_ptr(),
                                        T, H, V, scale, _ptr(ssq), _ptr(w_next) if xw is not None else None, _ptr(xw),
                                        self._stream()), "embed")

    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        self._need(x, "x", torch.float32, 2); self._need(w, "w", torch.float32, 1); self._need(out, "out", None, 2)
        T, H = x.shape
        if w.numel() != H or tuple(out.shape) != (T, H):
            raise KernelError(f"rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if not self._admit("rmsnorm", T * H * (4 + out.element_size())): return
        self._check(self.lib.cima_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(out.dtype),
                                          T, H, eps, self._stream()), "rmsnorm")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor, act: int = 0, limit: float = 0.0) -> None:
        """out = act(gate) * up of ``gate_up`` = [gate | up]; ``act`` one of ``ACTIVATIONS``' codes (``limit`` goes with
        "swish_clamped")."""
        self._need(gate_up, "gate_up", None, 2); self._need(out, "out", gate_up.dtype, 2)
        T, I2 = gate_up.shape
        if I2 % 2 or tuple(out.shape) != (T, I2 // 2):
            raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} and out {tuple(out.shape)} do not agree")
        if not self._admit("swiglu", T * (I2 + I2 // 2) * out.element_size()): return
        self._check(self.lib.cima_swiglu(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), T, I2 // 2, act, limit,
                                         self._stream()), "swiglu")

    def add_residual(self, x: torch.Tensor, delta: torch.Tensor) -> None:
        self._need(x, "x", torch.float32); self._need(delta, "delta")
        if x.shape != delta.shape:
            raise KernelError(f"add_residual: x {tuple(x.shape)} and delta {tuple(delta.shape)} differ")
        if not self._admit("add_residual", x.numel() * (8 + delta.element_size())): return
        self._check(self.lib.cima_add_residual(x.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype),
                                               x.numel(), self._stream()), "add_residual")

    def add_rmsnorm(self, x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        """x += delta (float32 sum), then out = RMSNorm(x; w, eps): the two kernels' results in one pass."""
        self._need(x, "x", torch.float32, 2); self._need(delta, "delta", None, 2); self._need(w, "w", torch.float32, 1)
        self._need(out, "out", delta.dtype, 2)
        T, H = x.shape
        if delta.shape != x.shape or out.shape != x.shape or w.numel() != H:
            raise KernelError(f"add_rmsnorm: x {tuple(x.shape)}, delta {tuple(delta.shape)}, out {tuple(out.shape)}, "
                              f"w {tuple(w.shape)} do not agree")
        if not self._admit("add_rmsnorm", T * H * (8 + 2 * delta.element_size())): return
        self._check(self.lib.cima_add_rmsnorm(x.data_ptr(), delta.data_ptr(), w.data_ptr(), out.data_ptr(),
                                              dtype_code(delta.dtype), T, H, eps, self._stream()), "add_rmsnorm")

    def gather_rows(self, x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        self._need(x, "x", torch.float32, 2); self._need(rows, "rows", torch.int32, 1); self._need(out, "out", torch.float32, 2)
        if tuple(out.shape) != (rows.numel(), x.shape[1]):
            raise KernelError(f"gather_rows: out is {tuple(out.shape)}, expected {(rows.numel(), x.shape[1])}")
        if not self._admit("gather_rows", rows.numel() * x.shape[1] * 8): return
        self._check(self.lib.cima_gather_rows(x.data_ptr(), rows.data_ptr(), out.data_ptr(), rows.numel(),
                                              x.shape[1], self._stream()), "gather_rows")

    def decode_advance(self, chosen: torch.Tensor, tokens: torch.Tensor, row_pos: torch.Tensor, seq_len: torch.Tensor) -> None:
        """tokens = chosen; every row's position and every sequence's length + 1 (one token per sequence)."""
        B = tokens.numel()
        for n, t in (("chosen", chosen), ("tokens", tokens), ("row_pos", row_pos), ("seq_len", seq_len)):
            self._need(t, n, torch.int32, 1)
            if t.numel() != B:
                raise KernelError(f"decode_advance: {n} has {t.numel()} entries, expected {B}")
        if not self._admit("decode_advance", 16 * B): return
        self._check(self.lib.cima_decode_advance(chosen.data_ptr(), tokens.data_ptr(), row_pos.data_ptr(),
                                                 seq_len.data_ptr(), B, self._stream()), "decode_advance")

    # ------------------------------------------------------------------ matrix products
    def linear_plain(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     accumulate: bool = False) -> None:
        """out = a @ w.T (+ bias), or out += ... when ``accumulate`` (out float32)."""
        self._need(a, "a", None, 2); self._need(w, "w", None, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear_plain: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError(f"linear_plain: bias has {bias.numel()} entries, expected {N}")
        if not self._admit("linear_plain", w.numel() * w.element_size() + (M * K + M * N) * 4, 2.0 * M * N * K): return
        # one launch takes up to 65535 * 64 rows; cut above that
        step = 65535 * 64
        for m0 in range(0, M, step):
            m1 = min(M, m0 + step)
            self._check(self.lib.cima_linear_plain(a[m0:m1].data_ptr(), dtype_code(a.dtype), w.data_ptr(),
                                                   dtype_code(w.dtype), _ptr(bias), out[m0:m1].data_ptr(),
                                                   dtype_code(out.dtype), 1 if accumulate else 0, m1 - m0, N, K,
                                                   K, N, self._stream()), "linear_plain")

    def linear_skinny(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                      mode: int, ssq_out: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None,
                      xw_out: Optional[torch.Tensor] = None, act: int = 0, limit: float = 0.0) -> None:
        """Few rows (<= 8), bf16 operands; ``mode`` is one of SK_*.  For SK_SWIGLU ``w`` is [2N, K].
        With SK_ACCUM, ``ssq_out`` [M, ceil(N / 16)] receives partial sums of squares of the updated rows and
        ``xw_out`` [M, N] bf16 the updated rows times ``w_next`` (the weight of the norm that follows)."""
        self._need(a, "a", torch.bfloat16, 2); self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode in (SK_ACCUM, SK_STORE_F32) else torch.bfloat16
        if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"linear_skinny(mode {mode}): a {tuple(a.shape)}, w {tuple(w.shape)}, "
                              f"out {tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError(f"linear_skinny: bias has {bias.numel()} entries, expected {N}")
        if ssq_out is not None:
            self._need(ssq_out, "ssq_out", torch.float32, 2)
            if mode != SK_ACCUM or tuple(ssq_out.shape) != (M, -(-N // 16)):
                raise KernelError(f"linear_skinny: ssq_out {tuple(ssq_out.shape)} goes with the accumulating mode and "
                                  f"must be {(M, -(-N // 16))}")
        if xw_out is not None:
            self._need(xw_out, "xw_out", torch.bfloat16, 2); self._need(w_next, "w_next", torch.float32, 1)
            if ssq_out is None or tuple(xw_out.shape) != (M, N) or w_next.numel() != N:
                raise KernelError("linear_skinny: xw_out goes with ssq_out and must be [rows, N], w_next [N]")
        if not self._admit(f"linear_skinny[{mode}]", w.numel() * 2 + M * K * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_linear_skinny(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode,
                                                M, N, K, K, N, _ptr(ssq_out), _ptr(w_next) if xw_out is not None else None,
                                                _ptr(xw_out), act, limit, self._stream()), "linear_skinny")

    def linear_skinny_norm(self, xw: torch.Tensor, ssq: torch.Tensor, eps: float, w: torch.Tensor,
                           bias: Optional[torch.Tensor], out: torch.Tensor, mode: int, act: int = 0) -> None:
        """``linear_skinny`` of RMSNorm(x) for at most 8 rows: ``xw`` [M, K] bf16 = bf16(x * norm weight) and
        ``ssq`` [M, parts], the partial sums of squares of the rows x, as ``embed`` or an accumulating
        ``linear_skinny`` left them."""
        self._need(xw, "xw", torch.bfloat16, 2); self._need(ssq, "ssq", torch.float32, 2)
        self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = xw.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode == SK_STORE_F32 else torch.bfloat16
        if w.shape[1] != K or ssq.shape[0] != M or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"linear_skinny_norm(mode {mode}): xw {tuple(xw.shape)}, w {tuple(w.shape)}, ssq "
                              f"{tuple(ssq.shape)}, out {tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        if not self._admit(f"linear_skinny_norm[{mode}]", w.numel() * 2 + M * K * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_linear_skinny_norm(xw.data_ptr(), ssq.data_ptr(), ssq.shape[1], eps, w.data_ptr(),
                                                     _ptr(bias), out.data_ptr(), mode, M, N, K, K, N, act, self._stream()),
                    "linear_skinny_norm")

    def qkv_rope(self, a, w: torch.Tensor, bias: Optional[torch.Tensor], qkv: torch.Tensor, inv_freq: torch.Tensor,
                 row_pos, row_seq, seq_slot, kv, n_heads: int, n_kv_heads: int, head_dim: int, norm=None) -> None:
        """The q/k/v projection of a decode step (at most 8 rows) with rotation and cache append in its
        epilogue: the rotated q lands in ``qkv`` [rows, (heads + 2 kv_heads) * head_dim], k and v in the layer's
        pages.  ``a``: bf16 activations, or with ``norm = (ssq, eps)`` the rows bf16(x * norm weight) and
        the partial sums of squares of x: the RMSNorm is folded in."""
        self._need(w, "w", torch.bfloat16, 2); self._need(qkv, "qkv", torch.bfloat16, 2)
        self._need(inv_freq, "inv_freq", torch.float32, 1)
        M, K = a.shape
        N = (n_heads + 2 * n_kv_heads) * head_dim
        if tuple(w.shape) != (N, K) or tuple(qkv.shape) != (M, N) or inv_freq.numel() != head_dim // 2:
            raise KernelError(f"qkv_rope: a {tuple(a.shape)}, w {tuple(w.shape)}, qkv {tuple(qkv.shape)}, inv_freq "
                              f"{tuple(inv_freq.shape)} do not agree with {n_heads}+2x{n_kv_heads} heads of {head_dim}")
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        if tuple(kv.storage.shape[1:]) != (2, n_kv_heads, kv.page_size, head_dim):
            raise KernelError(f"qkv_rope: cache pages are {tuple(kv.storage.shape)}")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        self._need(a, "a", torch.bfloat16, 2)
        if norm is None:
            head = (a.data_ptr(), None, 0, 0.0)
        else:
            ssq, eps = norm
            self._need(ssq, "ssq", torch.float32, 2)
            if ssq.shape[0] != M:
                raise KernelError(f"qkv_rope: ssq {tuple(ssq.shape)} does not fit {M} rows")
            head = (a.data_ptr(), ssq.data_ptr(), ssq.shape[1], eps)
        if not self._admit("qkv_rope_skinny", w.numel() * 2 + M * K * 2 + M * N * 2, 2.0 * M * N * K): return
        self._check(self.lib.cima_qkv_rope_skinny(*head, w.data_ptr(), _ptr(bias), qkv.data_ptr(), M, K, K, N,
                                                  inv_freq.data_ptr(), row_pos.data_ptr(), row_seq.data_ptr(),
                                                  seq_slot.data_ptr(), kv.storage.data_ptr(), kv.block_table.data_ptr(),
                                                  kv.block_table.shape[1], kv.ring_pages, kv.page_size, n_heads,
                                                  n_kv_heads, head_dim, self._stream()), "qkv_rope_skinny")

    def gemm_tc_pair(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                     mode: int, act: int = 0, limit: float = 0.0) -> None:
        """out = epilogue(a @ w.T) on the tcgen05 tensor cores, for many rows: bf16 operands by TMA, float32
        accumulation in tensor memory, pairs of SMs on tiles of 256 x 256 (cta_group::2; each SM of a pair stages
        only half of the weight tile).  ``mode`` as for ``linear_skinny`` (SK_*); for SK_SWIGLU ``w`` is [2N, K]."""
        self._need(a, "a", torch.bfloat16, 2); self._need(w, "w", torch.bfloat16, 2); self._need(out, "out", None, 2)
        M, K = a.shape
        N = w.shape[0] // 2 if mode == SK_SWIGLU else w.shape[0]
        want = torch.float32 if mode in (SK_ACCUM, SK_STORE_F32) else torch.bfloat16
        if w.shape[1] != K or tuple(out.shape) != (M, N) or out.dtype is not want:
            raise KernelError(f"gemm_tc_pair(mode {mode}): a {tuple(a.shape)}, w {tuple(w.shape)}, out "
                              f"{tuple(out.shape)} {out.dtype} do not agree")
        if bias is not None:
            self._need(bias, "bias", torch.float32, 1)
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=a.device)
        if not self._admit(f"gemm_tcgen05_pair[{mode}]", (w.numel() + M * K) * 2 + M * N * out.element_size(), 2.0 * M * w.shape[0] * K): return
        self._check(self.lib.cima_gemm_tcgen05_pair(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, M,
                                                    w.shape[0], K, N, N if mode == SK_SWIGLU else 0, act, limit,
                                                    self._error_flag.data_ptr(), self._stream()), "gemm_tcgen05_pair")

    def error_flag(self, device) -> torch.Tensor:
        """The int32 word that kernels with bounded waits set when a wait runs out (``device_errors`` reads it)."""
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        return self._error_flag

    def device_errors(self) -> int:
        """The error flag that a bounded wait inside a kernel sets when it runs out (synchronises).  Reading it
        clears it: a later, sound step is not blamed for an earlier one."""
        if self._error_flag is None:
            return 0
        v = int(self._error_flag.item())
        if v:
            self._error_flag.zero_()
        return v

    # ------------------------------------------------------------------ attention
    def rope_append(self, qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, row_pos, row_seq, seq_slot,
                    seq_len, kv, n_heads: int, n_kv_heads: int, head_dim: int, v_heads: Optional[int] = None,
                    qk_norm=None, amplitude: float = 1.0) -> None:
        """Rotate q and k of ``qkv`` in place and append k, v to the layer's pages (``kv`` a LayerKV or None).
        ``v_heads``: value heads of a row where they are fewer than the key heads (neighbouring key heads share one; the
        pages' value plane holds them in its first heads).  ``qk_norm = (wq, wk, dim, eps)``: before the rotation the first
        ``dim`` values of every q (k) head are divided by their root mean square and multiplied by wq (wk) [dim].
        ``amplitude``: a factor of every sine and cosine."""
        self._need(qkv, "qkv", None, 2); self._need(inv_freq, "inv_freq", torch.float32, 1)
        for n, t in (("row_pos", row_pos), ("row_seq", row_seq), ("seq_slot", seq_slot), ("seq_len", seq_len)):
            self._need(t, n, torch.int32, 1)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError(f"rope_append: inv_freq has {inv_freq.numel()} entries, expected {rotary_dim // 2}")
        T = qkv.shape[0]
        if row_pos.numel() < T or row_seq.numel() < T:
            raise KernelError("rope_append: the rows' positions do not cover the rows")
        if kv is not None:
            self._need(kv.storage, "cache", qkv.dtype, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
            if tuple(kv.storage.shape[1:]) != (2, n_kv_heads, kv.page_size, head_dim):
                raise KernelError(f"rope_append: cache pages are {tuple(kv.storage.shape)}, expected "
                                  f"[*, 2, {n_kv_heads}, {kv.page_size}, {head_dim}]")
            args = (kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.ring_pages, kv.page_size)
        else:
            args = (None, None, 0, 0, 0)
        nv = n_kv_heads if v_heads is None else int(v_heads)
        norm = (None, None, 0, 0.0)
        if qk_norm is not None:
            wq, wk, nd, eps = qk_norm
            self._need(wq, "wq", torch.float32, 1); self._need(wk, "wk", torch.float32, 1)
            if wq.numel() != nd or wk.numel() != nd:
                raise KernelError(f"rope_append: the norm's weights have {wq.numel()} and {wk.numel()} values, expected {nd}")
            norm = (wq.data_ptr(), wk.data_ptr(), int(nd), float(eps))
        if not self._admit("rope_append", 2 * qkv.numel() * qkv.element_size()): return
        step = 65535 if (qk_norm is not None or nv != n_kv_heads) else T       # the general kernel takes a row a block of grid.y
        for r0 in range(0, T, step):
            r1 = min(T, r0 + step)
            self._check(self.lib.cima_rope_append(qkv[r0:r1].data_ptr(), dtype_code(qkv.dtype), qkv.shape[1], inv_freq.data_ptr(),
                                                  rotary_dim, row_pos[r0:r1].data_ptr(), row_seq[r0:r1].data_ptr(), seq_slot.data_ptr(),
                                                  seq_len.data_ptr(), *args, r1 - r0, n_heads, n_kv_heads, head_dim, nv, *norm,
                                                  float(amplitude), self._stream()), "rope_append")

    def attention_plain(self, qkv: torch.Tensor, kv, row_pos, row_seq, seq_slot, seq_first_row, out: torch.Tensor,
                        n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int,
                        from_cache: bool, sink: float = 0.0, keep_first: int = 0, v_group: int = 1, head_sink=None) -> None:
        self._need(qkv, "qkv", None, 2); self._need(out, "out", qkv.dtype, 2)
        self._need_head_sink(head_sink, n_heads)
        T = qkv.shape[0]
        if tuple(out.shape) != (T, n_heads * head_dim):
            raise KernelError(f"attention: out is {tuple(out.shape)}, expected {(T, n_heads * head_dim)}")
        if from_cache:
            if kv is None:
                raise KernelError("attention: decoding needs the layer's cache")
            self._need(kv.storage, "cache", qkv.dtype, 5)
            args = (kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.ring_pages, kv.page_size)
        else:
            args = (None, None, 0, 0, 1)
        planes = int(getattr(kv, "planes", 2)) if from_cache else 2
        if not self._admit("attention_plain", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim, planes)): return
        self._check(self.lib.cima_attention_plain(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[1], *args,
                                                  row_pos.data_ptr(), row_seq.data_ptr(), seq_slot.data_ptr(),
                                                  seq_first_row.data_ptr(), out.data_ptr(), out.shape[1], T,
                                                  n_heads, n_kv_heads, head_dim, scale, window,
                                                  1 if from_cache else 0, planes, sink, keep_first, v_group, _ptr(head_sink),
                                                  self._stream()), "attention_plain")

    def _need_head_sink(self, head_sink, n_heads: int) -> None:
        if head_sink is not None:
            self._need(head_sink, "head_sink", torch.float32, 1)
            if head_sink.numel() != n_heads:
                raise KernelError(f"attention: head_sink has {head_sink.numel()} values, expected one for each of {n_heads} heads")

    def _attention_work(self, qkv, n_heads, n_kv_heads, head_dim, planes: int = 2):
        """(bytes, operations) of an attention launch while a step is profiled: the keys and values of the step's
        sequences (``profile.kv_tokens``: positions that the step's rows read, each once) and the products over the
        (query, key) pairs (``profile.qk_pairs``); the step's maker states both."""
        p = self.profile
        if p is None:
            return 0, 0
        elt = qkv.element_size()
        return (float(planes) * p.kv_tokens * n_kv_heads * head_dim * elt + 2.0 * qkv.shape[0] * n_heads * head_dim * elt,
                4.0 * p.qk_pairs * n_heads * head_dim)

    def library_mm(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """out = a @ w.T (+ bias) by the library's matrix product (cuBLAS through torch), where the reference calls
        its library too; ``out`` may be float32 for bfloat16 operands (the head).  Counted apart from this
        library's own launches."""
        if not self._admit("library_mm", (w.numel() + a.numel()) * a.element_size() + out.numel() * out.element_size(),
                           2.0 * a.shape[0] * w.shape[0] * w.shape[1]):
            return
        self.library_launches += 1
        if out.dtype is not a.dtype:
            torch.mm(a, w.t(), out_dtype=out.dtype, out=out)
            if bias is not None:
                out += bias
        elif bias is not None:
            torch.addmm(bias, a, w.t(), out=out)
        else:
            torch.mm(a, w.t(), out=out)

    def attention(self, qkv: torch.Tensor, kv, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                  head_dim: int, scale: float, window: int, from_cache: bool, after_append: bool = False,
                  sink: float = 0.0, keep_first: int = 0, v_group: int = 1, head_sink=None) -> None:
        """Attention of a step's rows: over the step's own keys (a prompt from position 0) or over the
        cache.  Chooses the kernel; every choice computes the same function.  ``after_append``: the kernel
        launched just before wrote nothing but ``qkv`` and the newest position of each sequence in the cache.
        ``sink``: that many entries of score 0 that carry no value join every row's denominator (0: an ordinary softmax).
        ``keep_first``: with a window, the first so many positions of a sequence stay visible below it.  ``v_group``: that
        many neighbouring key heads share one value head (a step's rows and the pages' value plane hold
        n_kv_heads / v_group value heads).  ``head_sink`` (float32 [n_heads], instead of ``sink``): head h's denominator
        also holds exp(head_sink[h]), an entry that is not scaled and carries no value."""
        general = keep_first > 0 or v_group > 1        # the tcgen05 kernels take neither
        if (from_cache and qkv.dtype is torch.bfloat16 and kv.page_size == 64 and head_dim % 16 == 0
                and head_dim <= 128 and batch.n_rows == batch.n_seqs):
            return self.attention_decode(qkv, kv, batch.seq_slot, batch.seq_len, out, n_heads, n_kv_heads, head_dim,
                                         scale, window, batch.max_len, early=after_append, sink=sink,
                                         keep_first=keep_first, v_group=v_group, head_sink=head_sink)
        many = (not general and qkv.dtype is torch.bfloat16 and head_dim in (64, 128) and qkv.shape[1] % 8 == 0
                and getattr(batch, "n_q_tiles_tc", 0) > 0 and getattr(batch, "max_rows", 0) >= TC_ATTENTION_MIN_LEN)
        if from_cache and many and kv.page_size == 64 and kv.storage.numel() // head_dim < 2 ** 31:
            return self.attention_prefill_tc(qkv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, kv=kv, sink=sink,
                                             head_sink=head_sink)
        if (from_cache and qkv.dtype is torch.bfloat16 and kv.page_size == 64 and head_dim % 16 == 0
                and head_dim <= 128 and qkv.shape[1] % 8 == 0 and getattr(batch, "n_q_tiles", 0) > 0):
            return self.attention_extend(qkv, kv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, sink=sink,
                                         keep_first=keep_first, v_group=v_group, head_sink=head_sink)
        if not from_cache and many:
            return self.attention_prefill_tc(qkv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, sink=sink,
                                             head_sink=head_sink)
        if (not from_cache and qkv.dtype is torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128
                and qkv.shape[1] % 8 == 0 and getattr(batch, "n_q_tiles", 0) > 0):
            return self.attention_prefill(qkv, batch.q_tile_seq, batch.q_tile_row0, batch.seq_first_row, out,
                                          n_heads, n_kv_heads, head_dim, scale, window, sink=sink,
                                          keep_first=keep_first, v_group=v_group, head_sink=head_sink)
        self.attention_plain(qkv, kv, batch.row_pos, batch.row_seq, batch.seq_slot, batch.seq_first_row, out,
                             n_heads, n_kv_heads, head_dim, scale, window, from_cache, sink=sink, keep_first=keep_first,
                             v_group=v_group, head_sink=head_sink)

    def attention_prefill(self, qkv: torch.Tensor, tile_seq, tile_row0, seq_first_row, out: torch.Tensor,
                          n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, sink: float = 0.0,
                          keep_first: int = 0, v_group: int = 1, head_sink=None) -> None:
        """Flash attention of ragged prompts that start at position 0 (bf16, head_dim <= 128);
        ``tile_seq``/``tile_row0`` list the blocks of 64 query rows."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        for n, t in (("tile_seq", tile_seq), ("tile_row0", tile_row0), ("seq_first_row", seq_first_row)):
            self._need(t, n, torch.int32, 1)
        T = qkv.shape[0]
        self._need_head_sink(head_sink, n_heads)
        if tuple(out.shape) != (T, n_heads * head_dim) or tile_seq.numel() != tile_row0.numel():
            raise KernelError(f"attention_prefill: out {tuple(out.shape)} or the block list do not fit")
        if not self._admit("attention_prefill", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim)): return
        self._check(self.lib.cima_attention_prefill(qkv.data_ptr(), qkv.shape[1], tile_seq.data_ptr(), tile_row0.data_ptr(),
                                                    seq_first_row.data_ptr(), out.data_ptr(), out.shape[1], T,
                                                    tile_seq.numel(), n_heads, n_kv_heads, head_dim, scale, window, sink,
                                                    keep_first, v_group, _ptr(head_sink), self._stream()), "attention_prefill")

    def attention_extend(self, qkv: torch.Tensor, kv, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: int, sink: float = 0.0, keep_first: int = 0,
                         v_group: int = 1, head_sink=None) -> None:
        """Flash attention of sequences that bring several rows to a cache that already holds keys (bf16, pages of
        64, head_dim <= 128): the rows of sequence s stand at positions seq_len[s] - rows .. seq_len[s] - 1, and all
        keys, the step's own included, are read from the layer's pages.  ``batch`` brings the blocks of 64 rows."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        T = qkv.shape[0]
        self._need_head_sink(head_sink, n_heads)
        if tuple(out.shape) != (T, n_heads * head_dim) or batch.q_tile_seq.numel() != batch.q_tile_row0.numel():
            raise KernelError(f"attention_extend: out {tuple(out.shape)} or the block list do not fit")
        if not self._admit("attention_extend", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim, kv.planes)): return
        self._check(self.lib.cima_attention_extend(
            qkv.data_ptr(), qkv.shape[1], batch.q_tile_seq.data_ptr(), batch.q_tile_row0.data_ptr(),
            batch.seq_first_row.data_ptr(), kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
            kv.ring_pages, kv.page_size, batch.seq_slot.data_ptr(), batch.seq_len.data_ptr(), out.data_ptr(), out.shape[1],
            T, batch.q_tile_seq.numel(), n_heads, n_kv_heads, head_dim, scale, window, kv.planes, sink, keep_first, v_group,
            _ptr(head_sink), self._stream()), "attention_extend")

    def attention_prefill_tc(self, qkv: torch.Tensor, batch, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                             head_dim: int, scale: float, window: int, kv=None, sink: float = 0.0, head_sink=None) -> None:
        """Flash attention of ragged prompts on the tcgen05 tensor cores (bf16, head_dim 64 or 128): blocks of 128
        query rows, both products with their results in tensor memory.  ``batch`` brings the blocks
        (``q_tile_tc_*``).  Without ``kv`` the sequences start at position 0 and the keys are the step's own rows;
        with ``kv`` (a layer's pages, to which the step has appended) the rows of sequence s stand at positions
        seq_len[s] - rows .. seq_len[s] - 1 and all keys come from the pages."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        T = qkv.shape[0]
        self._need_head_sink(head_sink, n_heads)
        if tuple(out.shape) != (T, n_heads * head_dim) or batch.n_q_tiles_tc <= 0:
            raise KernelError(f"attention_prefill_tc: out {tuple(out.shape)} or the block list do not fit")
        if self._error_flag is None:
            self._error_flag = torch.zeros(1, dtype=torch.int32, device=qkv.device)
        if not self._admit("attention_prefill_tc", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim, kv.planes if kv is not None else 2)): return
        if kv is not None:
            self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
            self._check(self.lib.cima_attention_extend_tc(
                qkv.data_ptr(), qkv.shape[1], batch.q_tile_tc_seq.data_ptr(), batch.q_tile_tc_row0.data_ptr(),
                batch.seq_first_row.data_ptr(), kv.storage.data_ptr(), kv.storage.shape[0], kv.block_table.data_ptr(),
                kv.block_table.shape[1], kv.ring_pages, kv.page_size, batch.seq_slot.data_ptr(), batch.seq_len.data_ptr(),
                out.data_ptr(), out.shape[1], T, batch.n_q_tiles_tc, n_heads, n_kv_heads, head_dim, scale, window,
                self._error_flag.data_ptr(), kv.planes, sink, _ptr(head_sink), self._stream()), "attention_extend_tc")
            return
        self._check(self.lib.cima_attention_prefill_tc(
            qkv.data_ptr(), qkv.shape[1], batch.q_tile_tc_seq.data_ptr(), batch.q_tile_tc_row0.data_ptr(),
            batch.seq_first_row.data_ptr(), out.data_ptr(),
            out.shape[1], T, batch.n_q_tiles_tc, n_heads, n_kv_heads, head_dim, scale, window,
            self._error_flag.data_ptr(), sink, _ptr(head_sink), self._stream()), "attention_prefill_tc")

    def attention_decode(self, qkv: torch.Tensor, kv, seq_slot, seq_len, out: torch.Tensor, n_heads: int,
                         n_kv_heads: int, head_dim: int, scale: float, window: int, max_len: int = 0,
                         n_splits: Optional[int] = None, early: bool = False, sink: float = 0.0, keep_first: int = 0,
                         v_group: int = 1, head_sink=None) -> None:
        """One query per sequence over the paged cache (bf16, pages of 64, head_dim <= 128), keys split
        over ``n_splits`` blocks per (sequence, kv head).  ``max_len`` (0 = unknown) only bounds the
        number of splits chosen here.  ``early``: the kernel launched just before this one wrote neither
        ``seq_slot``, ``seq_len``, the block table nor a page before the one of a sequence's newest position,
        so the first pages may be fetched while it finishes."""
        self._need(qkv, "qkv", torch.bfloat16, 2); self._need(out, "out", torch.bfloat16, 2)
        self._need(kv.storage, "cache", torch.bfloat16, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        B = qkv.shape[0]
        self._need_head_sink(head_sink, n_heads)
        if tuple(out.shape) != (B, n_heads * head_dim) or seq_slot.numel() < B or seq_len.numel() < B:
            raise KernelError(f"attention_decode: out {tuple(out.shape)} / sequences do not fit {B} rows")
        if n_splits is None:
            mtiles = -(-(n_heads // n_kv_heads) // 16)
            # one wave of blocks (two of them fit an SM): never a second, nearly empty wave; beyond 8 splits
            # only while the GPU would otherwise stay mostly idle.  The splits are merged by a second kernel: merging
            # inside a thread-block cluster (clusters of 8 blocks with 100 KB of shared memory each are slow to
            # place) and merging in the last block to finish (a fence and a ticket per block) were both measured
            # slower inside the decode step
            base = B * n_kv_heads * mtiles
            # 32 splits at most, 64 where even 32 leave SMs without a block (one sequence of 4 kv heads: measured at
            # the 7B shape 19 to 25 us against 28 to 31 at 30,000 positions, 15 against 19 at 16,384, the same up to
            # 6,000; with two sequences 32 are the best again)
            n_splits = max(1, min(64 if base * 32 < SPLIT_FEW_BLOCKS else 32, SPLIT_BLOCKS // base))
            if n_splits > 8 and base * 8 >= SPLIT_FEW_BLOCKS:
                n_splits = 8
            if max_len > 0:
                seen = max_len if window <= 0 else min(max_len, window + 64 + -(-keep_first // 64) * 64)      # positions whose pages a row reads
                n_splits = min(n_splits, -(-seen // 64))
                # a short context is a few pages: one block reads them in less time than the merge of splits takes
                if max_len <= short_context(head_dim):
                    n_splits = 1
        if not self._admit(f"attention_decode[{n_splits} splits]", *self._attention_work(qkv, n_heads, n_kv_heads, head_dim, kv.planes)): return
        part_o = part_ml = None
        if n_splits > 1:
            part_o = self._scratch("attn_o", B * n_heads * n_splits * head_dim, qkv.device)
            part_ml = self._scratch("attn_ml", B * n_heads * n_splits * 2, qkv.device)
        self._check(self.lib.cima_attention_decode(
            qkv.data_ptr(), qkv.shape[1], kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
            kv.ring_pages, kv.page_size, seq_slot.data_ptr(), seq_len.data_ptr(), _ptr(part_o), _ptr(part_ml),
            out.data_ptr(), out.shape[1], B, n_heads, n_kv_heads, head_dim, scale, window, n_splits, int(early),
            kv.planes, sink, keep_first, v_group, _ptr(head_sink), self._stream()), "attention_decode")
        if n_splits > 1:
            self.launches += 1

    def _scratch(self, name: str, numel: int, device) -> torch.Tensor:
        """Float32 scratch that lives as long as this object (grown on demand, outside graph capture:
        a captured step always follows an eager one of the same sizes).  A buffer that a larger one replaces is
        kept, not freed: a captured step holds the address it was recorded with and goes on writing there."""
        t = self._scratch_bufs.get(name)
        if t is None or t.numel() < numel or t.device != torch.device(device):
            if t is not None:
                self._retired.append(t)
            t = self._scratch_bufs[name] = torch.empty(numel, dtype=torch.float32, device=device)
        return t

    # ------------------------------------------------------------------ short convolution, depth average, latents
    def short_conv(self, h: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], batch, out: torch.Tensor,
                   rows_per_thread: int = 0, add_input: bool = True, act: int = -1) -> None:
        """out[t] = h[t] + sum_j w[j, :] * h[t - taps + 1 + j] per channel, causal within each sequence of the
        step; what lies before the step's rows comes from ``state`` [slots, taps - 1, C] (the sequences' last
        inputs), which is brought up to date.  ``w`` [taps, C] float32 (tap by tap); h, out, state of one dtype.
        ``add_input`` False leaves h[t] out of the sum (a plain convolution); ``act`` >= 0 applies that entry of
        ``ACTIVATIONS`` to the sum."""
        self._need(h, "h", None, 2); self._need(w, "w", torch.float32, 2); self._need(out, "out", h.dtype, 2)
        T, C = h.shape
        taps = w.shape[0]
        if w.shape[1] != C or out.shape != h.shape:
            raise KernelError(f"short_conv: h {tuple(h.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if taps > 1:
            self._need(state, "state", h.dtype, 3)
            if tuple(state.shape[1:]) != (taps - 1, C):
                raise KernelError(f"short_conv: state is {tuple(state.shape)}, expected [slots, {taps - 1}, {C}]")
        one_row = batch.n_rows == batch.n_seqs
        if not self._admit("short_conv", 2 * T * C * h.element_size()): return
        self._check(self.lib.cima_short_conv(h.data_ptr(), dtype_code(h.dtype), w.data_ptr(), _ptr(state if taps > 1 else None),
                                             batch.row_seq.data_ptr(), batch.seq_slot.data_ptr(), batch.seq_first_row.data_ptr(),
                                             out.data_ptr(), T, batch.n_seqs, C, taps, int(one_row), rows_per_thread,
                                             int(add_input), act, self._stream()), "short_conv")
        if not one_row and taps > 1:
            self.launches += 1

    def depth_average(self, stack: torch.Tensor, n: int, a: torch.Tensor, x: torch.Tensor,
                      w: Optional[torch.Tensor] = None, eps: float = 0.0, y: Optional[torch.Tensor] = None,
                      conv=None) -> None:
        """x = sum_{j < n} a[j] * stack[j] (float32 [planes, T, H]); with ``w`` also y = RMSNorm(x; w, eps).
        ``x`` may be a plane of ``stack`` beyond the first n.  ``conv = (cw, state, seq_slot, u)``, for a step of one
        row a sequence: also u = ``short_conv`` of y (weights cw [taps, H], the sequences' state brought up to date)."""
        self._need(stack, "stack", torch.float32, 3); self._need(a, "a", torch.float32, 1); self._need(x, "x", torch.float32, 2)
        P, T, H = stack.shape
        if not (1 <= n <= P) or a.numel() != n or tuple(x.shape) != (T, H):
            raise KernelError(f"depth_average: stack {tuple(stack.shape)}, {n} streams, a {tuple(a.shape)}, x {tuple(x.shape)} do not agree")
        if (w is None) != (y is None):
            raise KernelError("depth_average: the norm's weight and its output go together")
        if w is not None:
            self._need(w, "w", torch.float32, 1); self._need(y, "y", None, 2)
            if w.numel() != H or tuple(y.shape) != (T, H):
                raise KernelError(f"depth_average: w {tuple(w.shape)} / y {tuple(y.shape)} do not fit {(T, H)}")
        extra = (None, 0, None, None, None)
        if conv is not None:
            cw, state, seq_slot, u = conv
            self._need(cw, "cw", torch.float32, 2); self._need(seq_slot, "seq_slot", torch.int32, 1)
            taps = cw.shape[0]
            if y is None or cw.shape[1] != H or seq_slot.numel() != T or tuple(u.shape) != (T, H) or u.dtype is not y.dtype:
                raise KernelError("depth_average: the convolution goes with the norm, one row a sequence, and an output like y")
            self._need(u, "u", y.dtype, 2)
            if taps > 1:
                self._need(state, "state", y.dtype, 3)
                if tuple(state.shape[1:]) != (taps - 1, H):
                    raise KernelError(f"depth_average: state is {tuple(state.shape)}, expected [slots, {taps - 1}, {H}]")
            extra = (cw.data_ptr(), taps, _ptr(state if taps > 1 else None), seq_slot.data_ptr(), u.data_ptr())
        if not self._admit("depth_average", T * H * (4 * (n + 1) + ((2 if conv else 1) * y.element_size() if y is not None else 0))): return
        self._check(self.lib.cima_depth_average(stack.data_ptr(), T * H, a.data_ptr(), n, x.data_ptr(), _ptr(w), _ptr(y),
                                                dtype_code(y.dtype) if y is not None else F32, T, H, eps, *extra,
                                                self._stream()), "depth_average")

    def latent_append(self, raw: torch.Tensor, g: torch.Tensor, eps: float, kv, batch) -> None:
        """c = RMSNorm(raw; g, eps) per row, written to the row's position in the layer's pages (one plane, one
        head of raw.shape[1] values).  ``raw`` [T, R] may be a column slice of a wider matrix."""
        self._need(g, "g", torch.float32, 1); self._need(kv.storage, "cache", raw.dtype, 5)
        T, R = raw.shape
        if raw.stride(1) != 1 or g.numel() != R or tuple(kv.storage.shape[1:]) != (1, 1, kv.page_size, R):
            raise KernelError(f"latent_append: raw {tuple(raw.shape)}, g {tuple(g.shape)}, pages {tuple(kv.storage.shape)} do not agree")
        if not self._admit("latent_append", 2 * T * R * raw.element_size()): return
        self._check(self.lib.cima_latent_append(raw.data_ptr(), dtype_code(raw.dtype), raw.stride(0), g.data_ptr(), eps,
                                                kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1],
                                                kv.ring_pages, kv.page_size, batch.row_pos.data_ptr(), batch.row_seq.data_ptr(),
                                                batch.seq_slot.data_ptr(), T, R, self._stream()), "latent_append")

    FUSED_APPEND_ROWS = 8       # a step of at most this many rows appends its latents in the launch of its first head product

    def head_linear(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, append=None, a_head: Optional[int] = None,
                    out_head: Optional[int] = None) -> None:
        """out[t, h, :] = a[t, h, :] @ w[h].T for every head: a [T, heads * K] (rows may be slices of a wider
        matrix), w [heads, N, K], out [T, heads * N]; one dtype.  ``append = (raw, g, eps, kv, batch)``: the arguments
        of ``latent_append`` for the same rows, done by the same launch (a decode step's few rows) or, for more rows,
        by a launch of its own first.  ``a_head`` / ``out_head``: values from one head's start to the next in a row of
        ``a`` / ``out`` where a head there is wider than K / N (the product reads a head's first K values and writes its
        first N; what lies behind them is left alone)."""
        if a_head is not None or out_head is not None:
            return self._head_linear_strided(a, w, out, int(a_head or w.shape[2]), int(out_head or w.shape[1]))
        if append is not None and (a.shape[0] > self.FUSED_APPEND_ROWS or a.shape[0] * (w.shape[2] + 3) * 4 > 48 * 1024):
            self.latent_append(*append)
            append = None
        self._need(w, "w", a.dtype, 3); self._need(out, "out", a.dtype, 2)
        heads, N, K = w.shape
        T = a.shape[0]
        if a.dim() != 2 or a.stride(1) != 1 or a.shape[1] != heads * K or tuple(out.shape) != (T, heads * N):
            raise KernelError(f"head_linear: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
        if not self._admit("head_linear", (w.numel() + a.numel() + out.numel()) * a.element_size(), 2.0 * T * heads * N * K): return
        if a.dtype is torch.bfloat16 and T > 8:
            # many bfloat16 rows: the library's batched product, as for the other products of more than 8 rows
            self.library_launches += 1
            torch.bmm(a.view(T, heads, K).transpose(0, 1), w.transpose(1, 2), out=out.view(T, heads, N).transpose(0, 1))
            return
        if append is not None:
            raw, g, eps, kv, batch = append
            self._need(g, "g", torch.float32, 1); self._need(kv.storage, "cache", raw.dtype, 5)
            R = raw.shape[1]
            if (raw.dtype is not a.dtype or raw.shape[0] != T or raw.stride(1) != 1 or g.numel() != R
                    or tuple(kv.storage.shape[1:]) != (1, 1, kv.page_size, R)):
                raise KernelError(f"head_linear: the latents to append, raw {tuple(raw.shape)}, g {tuple(g.shape)}, pages "
                                  f"{tuple(kv.storage.shape)}, do not agree with {T} rows")
            self._check(self.lib.cima_head_linear_append(
                a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype), T, heads, N, K, a.stride(0), out.stride(0),
                raw.data_ptr(), raw.stride(0), g.data_ptr(), eps, kv.storage.data_ptr(), kv.block_table.data_ptr(),
                kv.block_table.shape[1], kv.ring_pages, kv.page_size, batch.row_pos.data_ptr(), batch.row_seq.data_ptr(),
                batch.seq_slot.data_ptr(), R, self._stream()), "head_linear_append")
            return
        self._check(self.lib.cima_head_linear(a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype), T, heads, N, K,
                                              a.stride(0), out.stride(0), K, N, self._stream()), "head_linear")

    def _head_linear_strided(self, a, w, out, a_head: int, out_head: int) -> None:
        self._need(w, "w", a.dtype, 3)
        heads, N, K = w.shape
        T = a.shape[0]
        if (a.dim() != 2 or out.dim() != 2 or a.stride(1) != 1 or out.stride(1) != 1 or out.dtype is not a.dtype or out.shape[0] != T
                or a_head < K or out_head < N or a.shape[1] < (heads - 1) * a_head + K or out.shape[1] < (heads - 1) * out_head + N):
            raise KernelError(f"head_linear: a {tuple(a.shape)} in heads of {a_head}, w {tuple(w.shape)}, out {tuple(out.shape)} in heads "
                              f"of {out_head} do not agree")
        if not self._admit("head_linear", (w.numel() + T * heads * (K + N)) * a.element_size(), 2.0 * T * heads * N * K): return
        if a.dtype is torch.bfloat16 and T > 8:
            # many bfloat16 rows: the library's batched product over the heads' columns
            self.library_launches += 1
            av = torch.as_strided(a, (heads, T, K), (a_head, a.stride(0), 1))
            ov = torch.as_strided(out, (heads, T, N), (out_head, out.stride(0), 1))
            ov.copy_(torch.bmm(av, w.transpose(1, 2)))
            return
        self._check(self.lib.cima_head_linear(a.data_ptr(), w.data_ptr(), out.data_ptr(), dtype_code(a.dtype), T, heads, N, K,
                                              a.stride(0), out.stride(0), a_head, out_head, self._stream()), "head_linear")

    def latent_prepare(self, ql: torch.Tensor, first: int, q_norm, cq, c_norm: torch.Tensor, eps: float, rank: int, rot: int,
                       inv_freq, amplitude: float, interleaved: bool, kv, batch, step_rows=None) -> None:
        """What stands between a latent attention's first product and its attention, for every row of ``ql`` =
        [``first`` values | ``rank`` | ``rot``]: with ``cq`` [T, first] the first part is a query latent, cq = rms(part) * q_norm;
        c = rms(second part) * c_norm; the third part is rotated at the row's position (pairs of neighbours where
        ``interleaved``, else (i, i + rot / 2); sine and cosine times ``amplitude``); [c | rotated part] goes to the row's
        place in the layer's one-plane pages (unless a later row of the step takes that place of a ring) and, with
        ``step_rows`` = (buffer [T, ld], column), to columns column .. column + rank + rot and once more behind them (a
        prompt's attention reads its keys and its values there).  Sums of squares, norms and angles are float32."""
        self._need(ql, "ql", None, 2); self._need(c_norm, "c_norm", torch.float32, 1)
        T, ld = ql.shape
        kd = rank + rot
        q_rank = 0
        if cq is not None:
            self._need(cq, "cq", ql.dtype, 2); self._need(q_norm, "q_norm", torch.float32, 1)
            q_rank = first
            if tuple(cq.shape) != (T, first) or q_norm.numel() != first:
                raise KernelError(f"latent_prepare: cq {tuple(cq.shape)} / q_norm {tuple(q_norm.shape)} do not fit a query latent of {first}")
        if ld < first + kd or c_norm.numel() != rank or rot % 2:
            raise KernelError(f"latent_prepare: rows of {ld} values do not hold {first} + {rank} + {rot}, or the norm's weight does not fit")
        if rot:
            self._need(inv_freq, "inv_freq", torch.float32, 1)
            if inv_freq.numel() != rot // 2:
                raise KernelError(f"latent_prepare: inv_freq has {inv_freq.numel()} entries, expected {rot // 2}")
        self._need(kv.storage, "cache", ql.dtype, 5); self._need(kv.block_table, "block_table", torch.int32, 2)
        if tuple(kv.storage.shape[1:]) != (1, 1, kv.page_size, kd):
            raise KernelError(f"latent_prepare: cache pages are {tuple(kv.storage.shape)}, expected [*, 1, 1, {kv.page_size}, {kd}]")
        sr, sr_ld, sr_col = (None, 0, 0)
        if step_rows is not None:
            buf, sr_col = step_rows
            self._need(buf, "step_rows", ql.dtype, 2)
            if buf.shape[0] != T or buf.shape[1] < sr_col + 2 * kd:
                raise KernelError(f"latent_prepare: step rows {tuple(buf.shape)} do not hold two copies of {kd} values from column {sr_col} on")
            sr, sr_ld = buf.data_ptr(), buf.stride(0)
        if not self._admit("latent_prepare", T * (ld + q_rank + (3 if sr else 1) * kd) * ql.element_size()): return
        self._check(self.lib.cima_latent_prepare(
            ql.data_ptr(), dtype_code(ql.dtype), ld, first, _ptr(q_norm) if cq is not None else None, _ptr(cq), q_rank,
            c_norm.data_ptr(), eps, rank, rot, _ptr(inv_freq) if rot else None, float(amplitude), int(bool(interleaved)),
            kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.ring_pages, kv.page_size,
            batch.row_pos.data_ptr(), batch.row_seq.data_ptr(), batch.seq_slot.data_ptr(), batch.seq_len.data_ptr(),
            sr, sr_ld, sr_col, T, self._stream()), "latent_prepare")

    def rope_rows(self, q: torch.Tensor, q_off: int, q_head: int, out: torch.Tensor, o_off: int, o_head: int, heads: int, rot: int,
                  inv_freq: torch.Tensor, amplitude: float, interleaved: bool, row_pos: torch.Tensor) -> None:
        """out[t, h * o_head + o_off + j] = the j-th of the ``rot`` values q[t, h * q_head + q_off ...] rotated at row t's
        position, for every head (pairs as in ``latent_prepare``); float32 angles, one rounding at the store."""
        self._need(q, "q", None, 2); self._need(out, "out", q.dtype, 2); self._need(inv_freq, "inv_freq", torch.float32, 1)
        self._need(row_pos, "row_pos", torch.int32, 1)
        T = q.shape[0]
        if (out.shape[0] != T or rot % 2 or inv_freq.numel() != rot // 2 or q.shape[1] < (heads - 1) * q_head + q_off + rot
                or out.shape[1] < (heads - 1) * o_head + o_off + rot or row_pos.numel() < T):
            raise KernelError(f"rope_rows: q {tuple(q.shape)}, out {tuple(out.shape)}, {heads} heads of {rot} rotating values do not agree")
        if not self._admit("rope_rows", 2 * T * heads * rot * q.element_size()): return
        self._check(self.lib.cima_rope_rows(q.data_ptr(), dtype_code(q.dtype), q.stride(0), q_off, q_head, out.data_ptr(), out.stride(0),
                                            o_off, o_head, heads, rot, inv_freq.data_ptr(), float(amplitude), int(bool(interleaved)),
                                            row_pos.data_ptr(), T, self._stream()), "rope_rows")

    # ------------------------------------------------------------------ several copies of the stream, ungated activation
    def hyper_connect(self, xs: torch.Tensor, y, C, b, mult: float, a_next, w_next, eps: float, h, spread: bool = False) -> None:
        """The streams xs [T, S, W] (float32, in place) take a sublayer's output and are read for the next one:
            with y [T, W] float32:   X_t <- sum_s C[s, t] X_s + mult * b[t] * y   for all t from the old X
            (``spread``: X_t <- y for all t; C and b are not read)
            with a_next [S]:         u = sum_s a_next[s] X_s (the new X);  h = u / sqrt(mean(u^2) + eps) * w_next
        ``h`` [T, W] in float32 or bfloat16.  Either half may be absent.  Everything is float32; one rounding at the
        store of h."""
        self._need(xs, "xs", torch.float32, 3)
        T, S, W = xs.shape
        if y is not None:
            self._need(y, "y", torch.float32, 2)
            if tuple(y.shape) != (T, W):
                raise KernelError(f"hyper_connect: y is {tuple(y.shape)}, expected {(T, W)}")
            if not spread:
                self._need(C, "C", torch.float32); self._need(b, "b", torch.float32)
                if C.numel() != S * S or b.numel() != S:
                    raise KernelError(f"hyper_connect: C has {C.numel()} and b {b.numel()} values for {S} streams")
        if a_next is not None:
            self._need(a_next, "a_next", torch.float32); self._need(w_next, "w_next", torch.float32, 1); self._need(h, "h", None, 2)
            if a_next.numel() != S or w_next.numel() != W or tuple(h.shape) != (T, W):
                raise KernelError(f"hyper_connect: a_next {tuple(a_next.shape)}, w_next {tuple(w_next.shape)}, h {tuple(h.shape)} do not fit {(T, S, W)}")
        if T == 0:
            return
        nbytes = T * W * ((2 * S if y is not None and not spread else S) * 4 + (4 if y is not None else 0)
                          + (h.element_size() if a_next is not None else 0))
        if not self._admit("hyper_connect", nbytes): return
        self._check(self.lib.cima_hyper_connect(xs.data_ptr(), _ptr(y), _ptr(C) if not spread else None, _ptr(b) if not spread else None,
                                                float(mult), int(bool(spread)), _ptr(a_next), _ptr(w_next) if a_next is not None else None,
                                                float(eps), _ptr(h) if a_next is not None else None,
                                                dtype_code(h.dtype) if a_next is not None else F32, T, S, W, self._stream()), "hyper_connect")

    def activate(self, z: torch.Tensor, act: int) -> None:
        """z <- act(z) in place, ``act`` one of ``UNGATED_ACTIVATIONS``' codes; float32 inside, one rounding at the store."""
        self._need(z, "z")
        if z.numel() == 0:
            return
        if not self._admit("activate", 2 * z.numel() * z.element_size()): return
        self._check(self.lib.cima_activate(z.data_ptr(), dtype_code(z.dtype), z.numel(), int(act), self._stream()), "activate")

    # ------------------------------------------------------------------ Dynamic Tanh, bigram embedding
    def dyt(self, x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
        """out = tanh(alpha * x) * w + b: x float32 [T, H], alpha one float32 value on the device, w and b [H]."""
        self._need(x, "x", torch.float32, 2); self._need(alpha, "alpha", torch.float32); self._need(w, "w", torch.float32, 1)
        self._need(b, "b", torch.float32, 1); self._need(out, "out", None, 2)
        T, H = x.shape
        if alpha.numel() != 1 or w.numel() != H or b.numel() != H or tuple(out.shape) != (T, H):
            raise KernelError(f"dyt: x {tuple(x.shape)}, alpha {tuple(alpha.shape)}, w {tuple(w.shape)}, b {tuple(b.shape)}, out "
                              f"{tuple(out.shape)} do not agree")
        if not self._admit("dyt", T * H * (4 + out.element_size())): return
        self._check(self.lib.cima_dyt(x.data_ptr(), alpha.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(),
                                      dtype_code(out.dtype), T, H, self._stream()), "dyt")

    def dyt_add(self, x: torch.Tensor, y: torch.Tensor, norm, mult: float, next_norm=None, h: Optional[torch.Tensor] = None) -> None:
        """x += mult * (tanh(a1 * y) * w1 + b1) with ``norm`` = (a1, w1, b1); with ``next_norm`` = (a2, w2, b2) also
        h = tanh(a2 * x) * w2 + b2 of the updated rows.  x and y float32 [T, H]."""
        self._need(x, "x", torch.float32, 2); self._need(y, "y", torch.float32, 2)
        T, H = x.shape
        a1, w1, b1 = norm
        for n, t in (("alpha", a1), ("w", w1), ("b", b1)):
            self._need(t, n, torch.float32)
        if y.shape != x.shape or a1.numel() != 1 or w1.numel() != H or b1.numel() != H:
            raise KernelError(f"dyt_add: x {tuple(x.shape)}, y {tuple(y.shape)} and the norm's tensors do not agree")
        second = (None, None, None, None, F32)
        if next_norm is not None:
            a2, w2, b2 = next_norm
            for n, t in (("alpha", a2), ("w", w2), ("b", b2)):
                self._need(t, n, torch.float32)
            self._need(h, "h", None, 2)
            if a2.numel() != 1 or w2.numel() != H or b2.numel() != H or tuple(h.shape) != (T, H):
                raise KernelError("dyt_add: the second norm's tensors and its output do not fit the rows")
            second = (a2.data_ptr(), w2.data_ptr(), b2.data_ptr(), h.data_ptr(), dtype_code(h.dtype))
        if not self._admit("dyt_add", T * H * (12 + (h.element_size() if h is not None else 0))): return
        self._check(self.lib.cima_dyt_add(x.data_ptr(), y.data_ptr(), a1.data_ptr(), w1.data_ptr(), b1.data_ptr(), mult,
                                          *second, T, H, self._stream()), "dyt_add")

    def embed_bigram(self, batch, table: torch.Tensor, bigram: torch.Tensor, x: torch.Tensor, scale: float, buckets: int,
                     mul_prev: int, mul_cur: int, prev_state: torch.Tensor) -> None:
        """x[t] = scale * table[tok_t] + bigram[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets], row ``buckets`` at a
        sequence's first position; the token before a step's rows is ``prev_state`` [slots] int32, brought up to date."""
        self._need(table, "table", None, 2); self._need(bigram, "bigram", table.dtype, 2); self._need(x, "x", torch.float32, 2)
        self._need(prev_state, "prev_state", torch.int32, 1)
        T, (V, H) = batch.n_rows, table.shape
        if tuple(x.shape) != (T, H) or tuple(bigram.shape) != (buckets + 1, H):
            raise KernelError(f"embed_bigram: x {tuple(x.shape)}, table {tuple(table.shape)}, bigram {tuple(bigram.shape)} and "
                              f"{buckets} buckets do not agree")
        one_row = batch.n_rows == batch.n_seqs
        if not self._admit("embed_bigram", T * H * (2 * table.element_size() + 4)): return
        self._check(self.lib.cima_embed_bigram(batch.tokens.data_ptr(), table.data_ptr(), bigram.data_ptr(), dtype_code(table.dtype),
                                               x.data_ptr(), T, batch.n_seqs, H, scale, buckets, mul_prev, mul_cur,
                                               batch.row_pos.data_ptr(), batch.row_seq.data_ptr(), batch.seq_slot.data_ptr(),
                                               batch.seq_first_row.data_ptr(), prev_state.data_ptr(), int(one_row),
                                               self._stream()), "embed_bigram")
        if not one_row:
            self.launches += 1

    # ------------------------------------------------------------------ recurrent mixers
    def recurrence(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, batch, out: torch.Tensor,
                   heads: int, kv_heads: int, dim: int, vdim: int, g: Optional[torch.Tensor] = None,
                   beta: Optional[torch.Tensor] = None, decay: Optional[torch.Tensor] = None, gate=None) -> None:
        """A linear recurrence over the step's rows, sequence by sequence, with the state S [slots, heads, dim, vdim]
        (float32) carried on.  With ``decay`` [heads]: S <- d S + k v^T, o = S^T q, and q, k, v (one dtype) pass SiLU.
        With ``g`` [T, heads * dim] and ``beta`` [T, heads]: the gated delta rule on prepared float32 q and k
        ([T, kv_heads * dim]).  With ``gate`` = (bias, lower), both float32 [heads * dim]: the gate rule, S <- diag(f) S +
        (1 - f) v^T with f = lower + (1 - lower) * sigmoid(k + bias) made from the projection that ``k`` holds, o = S^T silu(q),
        v as it is (q, k, v of one dtype, kv_heads = heads).  q, k, v may be column slices of wider matrices; out
        [T, heads * vdim] float32."""
        if gate is not None:
            return self._recurrence_gate(q, k, v, state, batch, out, heads, kv_heads, dim, vdim, *gate)
        delta = g is not None
        self._need(state, "state", torch.float32, 4); self._need(out, "out", torch.float32, 2)
        T = batch.n_rows
        for n, t in (("q", q), ("k", k), ("v", v)):
            if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != T or not t.is_cuda:
                raise KernelError(f"recurrence: {n} {tuple(t.shape)} must be GPU rows of the step with unit column stride")
        if (tuple(state.shape[1:]) != (heads, dim, vdim) or tuple(out.shape) != (T, heads * vdim) or q.shape[1] != kv_heads * dim
                or k.shape[1] != kv_heads * dim or v.shape[1] != heads * vdim or q.dtype is not k.dtype):
            raise KernelError(f"recurrence: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, state {tuple(state.shape)}, "
                              f"out {tuple(out.shape)} do not agree with {heads} heads on {kv_heads} of {dim} x {vdim}")
        if delta:
            self._need(g, "g", torch.float32, 2); self._need(beta, "beta", torch.float32, 2)
            if q.dtype is not torch.float32 or tuple(g.shape) != (T, heads * dim) or tuple(beta.shape) != (T, heads):
                raise KernelError("recurrence: the delta rule takes float32 q and k, g [T, heads * dim] and beta [T, heads]")
        else:
            self._need(decay, "decay", torch.float32, 1)
            if decay.numel() != heads or q.dtype is not v.dtype:
                raise KernelError("recurrence: the decay rule takes q, k, v of one dtype and one decay a head")
        if not self._admit("recurrence[delta]" if delta else "recurrence[decay]",
                           batch.n_seqs * heads * dim * vdim * 8 + T * (2 * kv_heads * dim * q.element_size() + heads * vdim * (4 + v.element_size())
                                                                        + (heads * dim * 4 if delta else 0)),
                           (8.0 if delta else 5.0) * T * heads * dim * vdim): return
        self._check(self.lib.cima_recurrence(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                             dtype_code(v.dtype), _ptr(g), _ptr(beta), _ptr(decay), state.data_ptr(),
                                             batch.seq_slot.data_ptr(), batch.seq_first_row.data_ptr(), out.data_ptr(), T,
                                             batch.n_seqs, heads, kv_heads, dim, vdim, int(delta), self._stream()), "recurrence")

    def _recurrence_gate(self, q, k, v, state, batch, out, heads, kv_heads, dim, vdim, bias, lower) -> None:
        self._need(state, "state", torch.float32, 4); self._need(out, "out", torch.float32, 2)
        self._need(bias, "bias", torch.float32, 1); self._need(lower, "lower", torch.float32, 1)
        T = batch.n_rows
        for n, t in (("q", q), ("k", k), ("v", v)):
            if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != T or not t.is_cuda or t.dtype is not v.dtype:
                raise KernelError(f"recurrence: {n} {tuple(t.shape)} must be GPU rows of the step, one dtype, unit column stride")
        if (heads != kv_heads or tuple(state.shape[1:]) != (heads, dim, vdim) or tuple(out.shape) != (T, heads * vdim)
                or q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim
                or bias.numel() != heads * dim or lower.numel() != heads * dim):
            raise KernelError(f"recurrence: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}, state {tuple(state.shape)}, "
                              f"out {tuple(out.shape)} and the gate's vectors do not agree with {heads} heads of {dim} x {vdim}")
        if not self._admit("recurrence[gate]", batch.n_seqs * heads * dim * vdim * 8 + T * heads * ((2 * dim + vdim) * v.element_size() + vdim * 4),
                           5.0 * T * heads * dim * vdim): return
        self._check(self.lib.cima_recurrence(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                             dtype_code(v.dtype), bias.data_ptr(), None, lower.data_ptr(), state.data_ptr(),
                                             batch.seq_slot.data_ptr(), batch.seq_first_row.data_ptr(), out.data_ptr(), T,
                                             batch.n_seqs, heads, kv_heads, dim, vdim, 2, self._stream()), "recurrence")

    def delta_prepare(self, qk: torch.Tensor, a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor,
                      qn: torch.Tensor, kn: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, heads: int, kv_heads: int,
                      dim: int) -> None:
        """What the gated delta rule needs of a token besides v, in float32: q and k as unit vectors per head (q also
        times dim^-1/2), g = exp(-exp(A_log[h]) * softplus(a + dt_bias)) per head and key channel, beta = sigmoid(b).
        ``qk`` [T, >= 2 * kv_heads * dim] holds q's heads and then k's; qk, a, b of one dtype, rows may be slices."""
        T = qk.shape[0]
        for n, t in (("qk", qk), ("a", a), ("b", b)):
            if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != T or t.dtype is not qk.dtype or not t.is_cuda:
                raise KernelError(f"delta_prepare: {n} {tuple(t.shape)} {t.dtype} must be GPU rows of one dtype with unit column stride")
        for n, t, shape in (("qn", qn, (T, kv_heads * dim)), ("kn", kn, (T, kv_heads * dim)), ("g", g, (T, heads * dim)),
                            ("beta", beta, (T, heads))):
            self._need(t, n, torch.float32, 2)
            if tuple(t.shape) != shape:
                raise KernelError(f"delta_prepare: {n} is {tuple(t.shape)}, expected {shape}")
        self._need(A_log, "A_log", torch.float32, 1); self._need(dt_bias, "dt_bias", torch.float32, 1)
        if (qk.shape[1] < 2 * kv_heads * dim or a.shape[1] != heads * dim or b.shape[1] != heads or A_log.numel() != heads
                or dt_bias.numel() != heads * dim):
            raise KernelError("delta_prepare: the inputs' widths do not agree with the heads and the key size")
        if not self._admit("delta_prepare", T * (2 * kv_heads * dim + heads * dim + heads) * (4 + qk.element_size())): return
        self._check(self.lib.cima_delta_prepare(qk.data_ptr(), qk.stride(0), a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                                dtype_code(qk.dtype), A_log.data_ptr(), dt_bias.data_ptr(), qn.data_ptr(),
                                                kn.data_ptr(), g.data_ptr(), beta.data_ptr(), T, heads, kv_heads, dim,
                                                self._stream()), "delta_prepare")

    def group_rmsnorm_gate(self, o: torch.Tensor, w: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, groups: int,
                           eps: float) -> None:
        """out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) over each of ``groups`` equal parts of a row: o float32
        [T, groups * n]; w [n] (one weight for all groups) or [groups * n]; gate [T, groups * n] in out's dtype (rows may
        be slices) or None."""
        self._need(o, "o", torch.float32, 2); self._need(w, "w", torch.float32, 1); self._need(out, "out", None, 2)
        T, W = o.shape
        if groups <= 0 or W % groups or out.shape != o.shape or w.numel() not in (W // groups, W):
            raise KernelError(f"group_rmsnorm_gate: o {tuple(o.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, {groups} groups do not agree")
        n = W // groups
        if gate is not None and (gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (T, W) or gate.dtype is not out.dtype):
            raise KernelError(f"group_rmsnorm_gate: the gate {tuple(gate.shape)} {gate.dtype} must match the output")
        shared = int(w.numel() == n and groups > 1)
        if not self._admit("group_rmsnorm_gate", T * W * (4 + 2 * out.element_size())): return
        self._check(self.lib.cima_group_rmsnorm_gate(o.data_ptr(), w.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                                     out.data_ptr(), dtype_code(out.dtype), T, groups, n, shared, eps,
                                                     self._stream()), "group_rmsnorm_gate")

    def rms_mean(self, ys, ws, x: torch.Tensor, eps: float, assign: bool = False) -> None:
        """x += mean over the branches b of  y_b / sqrt(mean(y_b^2) + eps) * w_b:  y_b float32 [T, H], w_b [H], at most 4.
        ``assign``: x = instead of x +=."""
        self._need(x, "x", torch.float32, 2)
        T, H = x.shape
        if not (1 <= len(ys) <= 4) or len(ws) != len(ys):
            raise KernelError(f"rms_mean: {len(ys)} branches with {len(ws)} weights; 1 to 4 of each are possible")
        for y, w in zip(ys, ws):
            self._need(y, "y", torch.float32, 2); self._need(w, "w", torch.float32, 1)
            if y.shape != x.shape or w.numel() != H:
                raise KernelError(f"rms_mean: a branch {tuple(y.shape)} / its weight {tuple(w.shape)} do not fit {tuple(x.shape)}")
        if not self._admit("rms_mean", T * H * 4 * (len(ys) + 2)): return
        yp = (ctypes.c_void_p * len(ys))(*[y.data_ptr() for y in ys])
        wp = (ctypes.c_void_p * len(ws))(*[w.data_ptr() for w in ws])
        self._check(self.lib.cima_rms_mean(yp, wp, len(ys), x.data_ptr(), T, H, eps, int(assign), self._stream()), "rms_mean")

    def diff_combine(self, att: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, heads: int, rep: int,
                     head_dim: int, v_dim: int, lam: float, post: float, eps: float) -> None:
        """The end of a differential attention.  ``att`` [T, 2 * heads * head_dim] holds two softmax maps over the same
        values for every head, in blocks of 2 * rep heads (a key-head pair's map 1 of its rep heads, then map 2 of the
        same); out[t, h] = rms(a1 - lam * a2) * post * sigmoid(gate[t, h]) over the first ``v_dim`` values of a head,
        [T, heads * v_dim].  ``gate`` [T, heads] (rows may be slices) or None."""
        self._need(att, "att", None, 2); self._need(out, "out", att.dtype, 2)
        T = att.shape[0]
        if att.shape[1] != 2 * heads * head_dim or tuple(out.shape) != (T, heads * v_dim):
            raise KernelError(f"diff_combine: att {tuple(att.shape)} and out {tuple(out.shape)} do not agree with {heads} heads of {head_dim} / {v_dim}")
        if gate is not None and (gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (T, heads) or gate.dtype is not att.dtype):
            raise KernelError(f"diff_combine: the gate {tuple(gate.shape)} {gate.dtype} must be [rows, heads] of att's dtype")
        if not self._admit("diff_combine", (att.numel() + out.numel()) * att.element_size()): return
        self._check(self.lib.cima_diff_combine(att.data_ptr(), att.shape[1], _ptr(gate), gate.stride(0) if gate is not None else 0,
                                               out.data_ptr(), dtype_code(att.dtype), T, heads, rep, head_dim, v_dim, lam, post, eps,
                                               self._stream()), "diff_combine")

    def scale_add_group_rmsnorm(self, x: torch.Tensor, y: Optional[torch.Tensor], alpha: float, w: torch.Tensor, groups: int,
                                eps: float, h: Optional[torch.Tensor] = None) -> None:
        """x <- N(alpha * x + y): x, y float32 [T, W] (y None: N(alpha * x)); N divides each of the row's ``groups`` equal
        consecutive parts by its own root mean square (eps inside the root) and multiplies the whole by w [W].  ``h``
        (optional, any dtype of the library) receives the new rows too."""
        self._need(x, "x", torch.float32, 2); self._need(w, "w", torch.float32, 1)
        T, W = x.shape
        if groups <= 0 or W % groups or w.numel() != W:
            raise KernelError(f"scale_add_group_rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)} and {groups} groups do not agree")
        if y is not None:
            self._need(y, "y", torch.float32, 2)
            if y.shape != x.shape:
                raise KernelError(f"scale_add_group_rmsnorm: y {tuple(y.shape)} is not x's {tuple(x.shape)}")
        if h is not None:
            self._need(h, "h", None, 2)
            if h.shape != x.shape:
                raise KernelError(f"scale_add_group_rmsnorm: h {tuple(h.shape)} is not x's {tuple(x.shape)}")
        if not self._admit("scale_add_group_rmsnorm", T * W * (8 + (4 if y is not None else 0) + (h.element_size() if h is not None else 0))): return
        self._check(self.lib.cima_scale_add_group_rmsnorm(x.data_ptr(), _ptr(y), alpha, w.data_ptr(), _ptr(h),
                                                          dtype_code(h.dtype) if h is not None else F32, T, groups, W // groups, eps,
                                                          self._stream()), "scale_add_group_rmsnorm")

    def cast_rows(self, x: torch.Tensor, h: torch.Tensor) -> None:
        """h = x (float32) in h's dtype."""
        self._need(x, "x", torch.float32); self._need(h, "h")
        if h.shape != x.shape:
            raise KernelError(f"cast_rows: h {tuple(h.shape)} is not x's {tuple(x.shape)}")
        if not self._admit("cast_rows", x.numel() * (4 + h.element_size())): return
        self._check(self.lib.cima_cast_rows(x.data_ptr(), h.data_ptr(), dtype_code(h.dtype), x.numel(), self._stream()), "cast_rows")

    def softcap(self, logits: torch.Tensor, cap: float) -> None:
        """logits <- cap * tanh(logits / cap), in place (float32)."""
        self._need(logits, "logits", torch.float32)
        if not self._admit("softcap", logits.numel() * 8): return
        self._check(self.lib.cima_softcap(logits.data_ptr(), logits.numel(), cap, self._stream()), "softcap")

    # ------------------------------------------------------------------ routed feed-forward
    ROUTE_SORT_ROWS = 64        # a step of at most this many rows orders its pairs by expert in the routing launch

    def moe_route(self, scores: torch.Tensor, top: int, groups: int, keep: int, scale: float, idx: torch.Tensor,
                  wgt: torch.Tensor, order: bool = False, experts: Optional[int] = None, softmax: bool = False, correction=None):
        """``scores`` float32 [T, E] holds the router's logits (it is scratch afterwards).  s = sigmoid(logits); the
        experts form ``groups`` equal groups of neighbours, a group's score is the sum of its two best, the best
        ``keep`` groups stay, and the ``top`` best experts among them are chosen: idx [T, top] int32, and their weights
        s / (sum of the chosen s + 1e-20) * scale in wgt [T, top] float32.  ``order`` (at most ``ROUTE_SORT_ROWS`` rows): the
        same launch also orders the pairs by expert; what it returns goes to ``moe_experts`` as ``ordered``.
        ``experts``: the first so many columns of ``scores`` are the experts' (default: all; further columns are left alone).
        ``softmax``: s = softmax(logits) over the experts instead of the sigmoid.  ``correction`` (float32 [experts]): added to s
        where groups and experts are compared; the weights are made of s itself."""
        self._need(scores, "scores", torch.float32, 2); self._need(idx, "idx", torch.int32, 2); self._need(wgt, "wgt", torch.float32, 2)
        T, ld = scores.shape
        E = ld if experts is None else int(experts)
        if not (0 < E <= ld):
            raise KernelError(f"moe_route: {E} experts in rows of {ld} scores")
        if correction is not None:
            self._need(correction, "correction", torch.float32, 1)
            if correction.numel() != E:
                raise KernelError(f"moe_route: the correction has {correction.numel()} values for {E} experts")
        if tuple(idx.shape) != (T, top) or tuple(wgt.shape) != (T, top):
            raise KernelError(f"moe_route: idx {tuple(idx.shape)} / wgt {tuple(wgt.shape)} are not {(T, top)}")
        meta = None
        if order and T <= self.ROUTE_SORT_ROWS:
            meta = torch.empty(2 * (E + 1) + T * top, dtype=torch.int32, device=scores.device)
        if not self._admit("moe_route", T * (E * 8 + top * 8)): return meta
        parts = (meta[:E + 1].data_ptr(), meta[E + 1:2 * (E + 1)].data_ptr(), meta[2 * (E + 1):].data_ptr()) if meta is not None else (None, None, None)
        self._check(self.lib.cima_moe_route(scores.data_ptr(), T, E, ld, top, groups, keep, scale, int(bool(softmax)), _ptr(correction),
                                            idx.data_ptr(), wgt.data_ptr(), *parts, self._stream()), "moe_route")
        return meta

    def moe_experts(self, h: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, idx: torch.Tensor, wgt: torch.Tensor,
                    x: torch.Tensor, act: int = 0, assign: bool = False, ordered: Optional[torch.Tensor] = None,
                    limit: float = 0.0, shared=None) -> None:
        """x[t] += (with ``assign``: =) sum_j wgt[t, j] * W_down[e] (act(W_gate[e] h[t]) * (W_up[e] h[t])), e = idx[t, j], ascending j.
        gate_up [E, 2 ff, H] (an expert's gate rows, then its up rows), down [E, H, ff]; x float32 [T, H].  Four launches:
        the pairs sorted by expert, the two grouped products over tiles of one expert's pairs, the weighted sum.  The
        products take one of three roads by the step's size and dtype alone (``MOE_TC_PAIRS``, ``MOE_FEW_PAIRS``): tcgen05
        tiles of 256 pairs, a warp a feature for the few pairs of a decode step, or the plain tiles (any dtype and size).
        ``limit`` goes with the clamped form of the middle.  ``shared = (rows, gate, col)``: float32 rows [T, H] (a shared
        expert's output) that join the weighted sum in its launch, each row times sigmoid(gate[t, col]) (gate float32
        [T, n]; None: unweighted)."""
        tail = (None, None, 0)
        if shared is not None:
            srows, sgate, scol = shared
            self._need(srows, "shared rows", torch.float32, 2)
            if tuple(srows.shape) != tuple(x.shape):
                raise KernelError(f"moe_experts: the shared rows are {tuple(srows.shape)}, expected {tuple(x.shape)}")
            if sgate is not None:
                self._need(sgate, "shared gate", torch.float32, 2)
                if sgate.shape[0] != x.shape[0] or not (0 <= scol < sgate.shape[1]):
                    raise KernelError(f"moe_experts: the shared gate {tuple(sgate.shape)} has no column {scol} for {x.shape[0]} rows")
                tail = (srows.data_ptr(), sgate[:, scol:].data_ptr(), sgate.stride(0))
            else:
                tail = (srows.data_ptr(), None, 0)
        self._need(h, "h", None, 2); self._need(gate_up, "gate_up", None, 3); self._need(down, "down", gate_up.dtype, 3)
        self._need(idx, "idx", torch.int32, 2); self._need(wgt, "wgt", torch.float32, 2); self._need(x, "x", torch.float32, 2)
        T, H = h.shape
        E, ff2, _ = gate_up.shape
        ff, top = ff2 // 2, idx.shape[1]
        if (gate_up.shape[2] != H or tuple(down.shape) != (E, H, ff) or idx.shape[0] != T or wgt.shape != idx.shape
                or tuple(x.shape) != (T, H)):
            raise KernelError(f"moe_experts: h {tuple(h.shape)}, gate_up {tuple(gate_up.shape)}, down {tuple(down.shape)}, idx "
                              f"{tuple(idx.shape)}, x {tuple(x.shape)} do not agree")
        P = T * top
        dev = h.device
        bf16 = h.dtype is torch.bfloat16 and gate_up.dtype is torch.bfloat16 and H % 8 == 0 and ff % 8 == 0 and h.stride(0) % 8 == 0
        if bf16 and P >= self.MOE_TC_PAIRS:
            return self._moe_experts_tc(h, gate_up, down, idx, wgt, x, act, assign, limit, tail)
        few = bf16 and P <= self.MOE_FEW_PAIRS
        meta = ordered if ordered is not None else torch.empty(2 * (E + 1) + P, dtype=torch.int32, device=dev)
        offsets, tiles, perm = meta[:E + 1], meta[E + 1:2 * (E + 1)], meta[2 * (E + 1):]
        z = torch.empty((P, ff), dtype=h.dtype, device=dev)
        y = torch.empty((P, H), dtype=torch.float32, device=dev)
        wb = gate_up.element_size()
        touched = min(E, P)
        if ordered is None and self._admit("moe_sort", P * 8):
            self._check(self.lib.cima_moe_sort(idx.data_ptr(), P, E, offsets.data_ptr(), tiles.data_ptr(), perm.data_ptr(),
                                               self._stream()), "moe_sort")
        name = "moe_few" if few else "moe_gemm"
        if self._admit(f"{name}[gate|up]", touched * 2 * ff * H * wb + P * (H + ff) * h.element_size(), 4.0 * P * ff * H):
            if few:
                self._check(self.lib.cima_moe_few(h.data_ptr(), h.stride(0), gate_up.data_ptr(), z.data_ptr(), offsets.data_ptr(),
                                                  tiles.data_ptr(), perm.data_ptr(), P, E, top, ff, H, 0, act, limit, self._stream()), "moe_few")
            else:
                self._check(self.lib.cima_moe_gemm(h.data_ptr(), dtype_code(h.dtype), h.stride(0), gate_up.data_ptr(),
                                                   dtype_code(gate_up.dtype), z.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
                                                   perm.data_ptr(), P, E, top, ff, H, 0, act, limit, self._stream()), "moe_gemm")
        if self._admit(f"{name}[down]", touched * ff * H * wb + P * (ff * h.element_size() + H * 4), 2.0 * P * ff * H):
            if few:
                self._check(self.lib.cima_moe_few(z.data_ptr(), ff, down.data_ptr(), y.data_ptr(), offsets.data_ptr(),
                                                  tiles.data_ptr(), perm.data_ptr(), P, E, top, H, ff, 1, 0, 0.0, self._stream()), "moe_few")
            else:
                self._check(self.lib.cima_moe_gemm(z.data_ptr(), dtype_code(z.dtype), ff, down.data_ptr(), dtype_code(down.dtype),
                                                   y.data_ptr(), offsets.data_ptr(), tiles.data_ptr(), perm.data_ptr(), P, E, top,
                                                   H, ff, 1, 0, 0.0, self._stream()), "moe_gemm")
        if self._admit("moe_combine", P * H * 4 + T * H * 8):
            self._check(self.lib.cima_moe_combine(y.data_ptr(), wgt.data_ptr(), None, x.data_ptr(), T, top, H, int(assign), *tail,
                                                  self._stream()), "moe_combine")

    MOE_TC_PAIRS = 1024      # from this many (row, choice) pairs on, bfloat16 experts run on the tcgen05 tiles of 256 pairs
    MOE_FEW_PAIRS = 128      # up to this many, a warp computes a feature for the pairs of an expert (a decode step)

    def _moe_experts_tc(self, h, gate_up, down, idx, wgt, x, act, assign=False, limit: float = 0.0, tail=(None, None, 0)) -> None:
        """Many pairs in bfloat16: every expert's pairs are laid out from a multiple of 256 rows on (the rows of h copied
        there), so that each tile of the tcgen05 product multiplies with one expert's matrix."""
        T, H = h.shape
        E, ff2, _ = gate_up.shape
        ff, top = ff2 // 2, idx.shape[1]
        P, dev, TILE = T * top, h.device, 256
        n_tiles = -(-P // TILE) + E
        meta = torch.empty(n_tiles + P, dtype=torch.int32, device=dev)
        tile_expert, pos = meta[:n_tiles], meta[n_tiles:]
        hs = torch.empty((n_tiles * TILE, H), dtype=h.dtype, device=dev)
        z = torch.empty((n_tiles * TILE, ff), dtype=h.dtype, device=dev)
        y = torch.empty((n_tiles * TILE, H), dtype=torch.float32, device=dev)
        flag = self.error_flag(dev)
        if not h.is_contiguous():
            raise KernelError("moe_experts: the rows of h must be contiguous for the many-pairs road")
        if self._admit("moe_sort_tiles", P * 8):
            self._check(self.lib.cima_moe_sort_tiles(idx.data_ptr(), P, E, TILE, n_tiles, tile_expert.data_ptr(), pos.data_ptr(),
                                                     self._stream()), "moe_sort_tiles")
        if self._admit("moe_gather_rows", 2 * P * H * 2):
            self._check(self.lib.cima_moe_gather_rows(h.data_ptr(), pos.data_ptr(), hs.data_ptr(), P, top, H * 2, self._stream()),
                        "moe_gather_rows")
        if self._admit("gemm_tcgen05_pair_grouped[gate|up]", E * 2 * ff * H * 2 + P * (H + ff) * 2, 4.0 * P * ff * H):
            self._check(self.lib.cima_gemm_tcgen05_pair_grouped(hs.data_ptr(), gate_up.data_ptr(), z.data_ptr(), SK_SWIGLU,
                                                                n_tiles * TILE, 2 * ff, E, H, ff, ff, act, limit, tile_expert.data_ptr(),
                                                                flag.data_ptr(), self._stream()), "gemm_tcgen05_pair_grouped")
        if self._admit("gemm_tcgen05_pair_grouped[down]", E * ff * H * 2 + P * (ff * 2 + H * 4), 2.0 * P * ff * H):
            self._check(self.lib.cima_gemm_tcgen05_pair_grouped(z.data_ptr(), down.data_ptr(), y.data_ptr(), SK_STORE_F32,
                                                                n_tiles * TILE, H, E, ff, H, 0, 0, 0.0, tile_expert.data_ptr(),
                                                                flag.data_ptr(), self._stream()), "gemm_tcgen05_pair_grouped")
        if self._admit("moe_combine", P * H * 4 + T * H * 8):
            self._check(self.lib.cima_moe_combine(y.data_ptr(), wgt.data_ptr(), pos.data_ptr(), x.data_ptr(), T, top, H,
                                                  int(assign), *tail, self._stream()), "moe_combine")

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits: torch.Tensor, tokens: torch.Tensor) -> None:
        self._need(logits, "logits", torch.float32, 2); self._need(tokens, "tokens", torch.int32, 1)
        n, V = logits.shape
        if tokens.numel() < n:
            raise KernelError(f"argmax: {tokens.numel()} token places for {n} rows")
        if not self._admit("argmax", n * V * 4): return
        self._check(self.lib.cima_argmax(logits.data_ptr(), V, n, V, tokens.data_ptr(), self._stream()), "argmax")

    def sample(self, logits: torch.Tensor, row_slot: torch.Tensor, params: torch.Tensor, rng: torch.Tensor,
               ring: torch.Tensor, count: torch.Tensor, work: torch.Tensor, tokens: torch.Tensor,
               all_greedy: bool = False, general: bool = False) -> None:
        """The whole sampling chain per row; per-slot state (rng, ring, count) is read and advanced.
        ``all_greedy`` (no row penalises or draws) takes the argmax kernel and leaves the state alone.
        ``general``: the one-block-per-row kernel whatever the size (it otherwise serves only vocabularies too long
        for the fast kernel's shared memory)."""
        self._need(logits, "logits", torch.float32, 2); self._need(tokens, "tokens", torch.int32, 1)
        n, V = logits.shape
        if tokens.numel() < n:
            raise KernelError(f"sample: {tokens.numel()} token places for {n} rows")
        if not self._admit("argmax" if all_greedy else "sample", n * V * 4): return
        if all_greedy:
            self._check(self.lib.cima_argmax(logits.data_ptr(), V, n, V, tokens.data_ptr(), self._stream()), "argmax")
            return
        self._need(row_slot, "row_slot", torch.int32, 1); self._need(params, "params", torch.float32, 2)
        self._need(rng, "rng", torch.int64); self._need(ring, "ring", torch.int32, 2); self._need(count, "count", torch.int32)
        self._need(work, "work", torch.float32, 2)
        if params.shape != (n, 4) or ring.shape[1] != 64 or work.shape[0] < n or work.shape[1] != V:
            raise KernelError("sample: params must be [rows, 4], the ring [slots, 64], the scratch [>= rows, vocab]")
        fn = self.lib.cima_sample_general if general else self.lib.cima_sample
        self._check(fn(logits.data_ptr(), V, n, V, row_slot.data_ptr(), params.data_ptr(), rng.data_ptr(),
                       ring.data_ptr(), count.data_ptr(), work.data_ptr(), tokens.data_ptr(), self._stream()), "sample")
