"""Python faces of the CUDA kernels: each takes torch CUDA tensors, checks them, and calls
the C function on the current stream. Nothing here computes; there is no fallback."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load as load_library

F32, BF16 = 0, 1
PAGE_SIZE = 64  # positions per cache page; checked against the library's own number when it is loaded
KERNEL_CHOICES = ("fast", "plain")
# activations of a gated feed-forward, by the numbers the kernels know them by (Activation in csrc/common.cuh)
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1}
# the reference's phases (src/model.h:38-41, src/model.c:312-328); the ones that have no counterpart here stay 0
PHASES = ("embed", "norm", "qkv", "rope", "attention", "attn_out", "ffn_up", "activation", "attn_quant", "ffn_down",
          "routing", "residual", "logits")


class KernelError(RuntimeError):
    """A kernel refused its arguments (the message names the size) or CUDA reported an error."""


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, what: str, dtype=None, ndim=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what} must have {ndim} dimensions, got {t.dim()}")
    return t


def _stream() -> ctypes.c_void_p:
    # (the raw handle: building torch's Stream object for every launch cost 3.4 us of the ~12 a launch takes on the host,
    # and the prefill of a small model is bound by the host's launches)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


class NormedRows:
    """The rows of a float residual under RMSNorm, not computed yet. A product over a handful
    of tokens takes the norm as its prologue; everything else asks for ``tensor()``, which
    runs the norm kernel once."""

    def __init__(self, ops: "Ops", residual: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                 rows: Optional[torch.Tensor] = None):
        self.ops, self.residual, self.weight, self.eps, self.out_dtype, self.rows = ops, residual, weight, eps, out_dtype, rows
        self.done: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return (self.residual.shape[0] if self.rows is None else self.rows.numel(), self.residual.shape[1])

    def tensor(self) -> torch.Tensor:
        if self.done is None:
            self.done = self.ops.rmsnorm(self.residual, self.weight, self.eps, self.out_dtype, self.rows)
        return self.done


class FusedLayerRecord(ctypes.Structure):
    """One layer of the fused decode step, as the kernel library lays it out (``sm::FusedLayer``)."""

    _fields_ = [(name, ctypes.c_void_p) for name in ("w_qkv", "b_qkv", "w_o", "w_gate_up", "w_down", "norm1", "norm2",
                                                     "k_pool", "v_pool", "page_table", "cos_table", "sin_table")] + \
               [("table_stride", ctypes.c_int), ("ring", ctypes.c_int), ("window", ctypes.c_int),
                ("eps1", ctypes.c_float), ("eps2", ctypes.c_float), ("pad_", ctypes.c_int)]


class PhaseTimes:
    """Device time per phase of the forward pass, measured with CUDA events between ``lap`` calls (the reference's
    ``lap()``: src/model.c:312-328). Events only mark the stream; nothing computed changes."""

    def __init__(self) -> None:
        self.marks = []          # (phase or None, event): the time up to an event is charged to its phase

    def lap(self, phase: Optional[str]) -> None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        self.marks.append((phase, event))

    def seconds(self) -> dict:
        """Synchronises and returns seconds per phase (every phase of ``PHASES``, zeros included)."""
        torch.cuda.synchronize()
        out = {name: 0.0 for name in PHASES}
        for (_, before), (phase, event) in zip(self.marks, self.marks[1:]):
            if phase is not None:
                out[phase] = out.get(phase, 0.0) + before.elapsed_time(event) / 1000.0
        return out


class Ops:
    """The kernel library, loaded (and built if needed) at construction. ``kernels="plain"`` routes everything to
    the plain kernels (CUDA-core products, one-warp-per-query attention) whatever the dtype: the slow side of an
    A/B comparison, as the reference's ``--scalar`` is of its SIMD kernels (src/main.c:109)."""

    def __init__(self, kernels: str = "fast") -> None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this library runs on an NVIDIA B200 only (no CPU fallback)")
        if kernels not in KERNEL_CHOICES:
            raise KernelError(f"kernels must be one of {KERNEL_CHOICES}, got {kernels!r}")
        self.lib = load_library()
        if int(self.lib.sm_page_size()) != PAGE_SIZE:
            raise KernelError(f"the kernel library pages the cache by {int(self.lib.sm_page_size())} positions, "
                              f"the host by {PAGE_SIZE}")
        self.lib.sm_gemm_tc_workspace_bytes.restype = ctypes.c_longlong
        self.lib.sm_launch_count.restype = ctypes.c_longlong
        fast = kernels == "fast"
        self.kernels = kernels
        self.phase_times: Optional[PhaseTimes] = None   # set to time the phases of the forward pass
        self.use_tensor_cores = fast  # False routes bfloat16 products to the CUDA-core kernel
        self.skinny_most_rounds = 2   # plain rows over a longer K go to the tcgen05 kernel (see _skinny_ok)
        self.use_fast_attention = fast  # False routes bfloat16 attention to the plain kernel
        self.use_tcgen05_attention = True  # False routes prefill attention to the mma.sync kernel
        self.use_skinny = fast  # False routes products over a handful of tokens to the general kernels
        # True runs a decode step of standard layers (up to 16 sequences) as ONE persistent kernel. Off: as measured
        # on a B200 it is correct but slower than the chain of separate kernels (see csrc/decode_fused.cu).
        self.use_fused_decode = False
        self._fused_barriers = []     # barrier words of the fused decode steps, put back to zero after an error
        # more tokens than this go to the tcgen05 kernel (the weight-streaming kernel itself takes up to 32; measured
        # on a B200 at 24 and 32 tokens it is 20-35% behind on every shape from 0.5B to 7B)
        self.skinny_max_tokens = 16
        # Steps of up to this many tokens that go on from the cache attend with the decode kernel, a row a token (measured
        # on the 0.5B sizes against the tiled kernel: 100 tokens onto 2,000 1.60 against 2.65 ms a step, 256 onto 6,000
        # 3.69 against 5.97, 512 onto 2,000 3.50 against 3.54, 768 onto 2,000 4.50 against 3.82).
        self.extend_rows_as_decode = 512 if fast else 0
        # ... and up to this many where the tcgen05 attention can read its keys from the cache (head sizes 64 and 128, no
        # window): 160 tokens onto 2,000 take 2.15 ms either way, 300 tokens 2.93 as rows against 2.56 as tiles, 512 onto
        # 8,000 6.85 against 4.43
        self.extend_rows_as_decode_tc = 176 if fast else 0
        self.extend_tc_variant = -1     # that kernel with one CTA an SM (0), two (1, head size 64), or as the launcher chooses
        self.skinny_single_round_above_8 = True
        self.error_flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.lib.sm_set_error_word.restype = None
        self.lib.sm_set_error_word(_ptr(self.error_flag))
        # scratch of the greedy choice: one word per row, all ones when idle, and arrival counters
        self.argmax_scratch = torch.full((4096,), -1, dtype=torch.int64, device="cuda")
        self.argmax_counters = torch.zeros(4096, dtype=torch.int32, device="cuda")

    def _check(self, status: int) -> None:
        if status:
            raise KernelError(self.lib.sm_last_error().decode("utf-8", "replace"))

    def lap(self, phase: Optional[str]) -> None:
        """Charges the device time since the last lap to ``phase`` (None: to nothing). A no-op unless
        ``phase_times`` is set."""
        if self.phase_times is not None:
            self.phase_times.lap(phase)

    # ---- elementwise -------------------------------------------------------------------
    def embedding(self, table: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
        _need(table, "embedding table", ndim=2)
        _need(tokens, "tokens", torch.int32, 1)
        out = torch.empty((tokens.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
        self._check(self.lib.sm_embedding(_ptr(table), _dt(table), _ptr(tokens), _ptr(out), tokens.numel(),
                                          table.shape[1], table.shape[0], _ptr(status), _stream()))
        return out

    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        _need(x, "norm input", torch.float32, 2)
        _need(weight, "norm weight", ndim=1)
        if weight.numel() != x.shape[1]:
            raise KernelError(f"norm weight has {weight.numel()} elements, rows have {x.shape[1]}")
        n = x.shape[0] if rows is None else _need(rows, "rows", torch.int32, 1).numel()
        out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
        self._check(self.lib.sm_rmsnorm(_ptr(x), _ptr(weight), _dt(weight), ctypes.c_float(eps), _ptr(out), _dt(out),
                                        _ptr(rows), n, x.shape[1], _stream()))
        return out

    def rmsnorm_lazy(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                     rows: Optional[torch.Tensor] = None) -> NormedRows:
        return NormedRows(self, x, weight, eps, out_dtype, rows)

    def swiglu(self, gate_up: torch.Tensor, out_dtype: torch.dtype, activation: str = "silu") -> torch.Tensor:
        _need(gate_up, "gate_up", torch.float32, 2)
        hidden = gate_up.shape[1] // 2
        out = torch.empty((gate_up.shape[0], hidden), dtype=out_dtype, device=gate_up.device)
        self._check(self.lib.sm_swiglu(_ptr(gate_up), _ptr(out), _dt(out), gate_up.shape[0], hidden,
                                       self.activation_code(activation), _stream()))
        return out

    @staticmethod
    def activation_code(name: str) -> int:
        if name not in ACTIVATIONS:
            raise KernelError(f"unknown activation {name!r}: the kernels know {', '.join(sorted(ACTIVATIONS))}")
        return ACTIVATIONS[name]

    # ---- steps of a model that belong to no layer ------------------------------------------
    def scale_(self, x: torch.Tensor, scale: float) -> torch.Tensor:
        """x *= scale, in place (float)."""
        _need(x, "x", torch.float32)
        self._check(self.lib.sm_scale_inplace(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(scale), _stream()))
        return x

    def softcap_(self, x: torch.Tensor, cap: float) -> torch.Tensor:
        """x = cap * tanh(x / cap), in place (float)."""
        _need(x, "x", torch.float32)
        self._check(self.lib.sm_softcap_inplace(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()))
        return x

    def add_rows_(self, x: torch.Tensor, table: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """x[t, :] += table[rows[t], :], in place (x float)."""
        _need(x, "x", torch.float32, 2)
        _need(table, "table", ndim=2)
        _need(rows, "rows", torch.int32, 1)
        if table.shape[1] != x.shape[1] or rows.numel() != x.shape[0]:
            raise KernelError(f"add_rows shapes do not agree: x {tuple(x.shape)}, table {tuple(table.shape)}, rows {rows.numel()}")
        self._check(self.lib.sm_add_rows(_ptr(x), _ptr(table), _dt(table), _ptr(rows), x.shape[0], x.shape[1], table.shape[0],
                                         _stream()))
        return x

    def rope_store(self, qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim, rotary_dim, out_dtype,
                   want_packed, k_pool=None, v_pool=None, page_table=None, ring=0, token_slot=None, token_end=None):
        """Returns (q, k_packed, v_packed); the packed keys and values are None unless asked for."""
        _need(qkv, "qkv", torch.float32, 2)
        T = qkv.shape[0]
        if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
            raise KernelError(f"qkv rows have {qkv.shape[1]} elements, expected {(heads + 2 * kv_heads) * head_dim}")
        _need(positions, "positions", torch.int32, 1)
        _need(cos_table, "cos table", torch.float32, 2)
        _need(sin_table, "sin table", torch.float32, 2)
        if cos_table.shape[1] != rotary_dim // 2:
            raise KernelError("cos/sin tables do not match rotary_dim")
        q = torch.empty((T, heads, head_dim), dtype=out_dtype, device=qkv.device)
        kp = vp = None
        if want_packed:
            kp = torch.empty((T, kv_heads, head_dim), dtype=out_dtype, device=qkv.device)
            vp = torch.empty_like(kp)
        table_stride = 0
        if k_pool is not None:
            _need(k_pool, "key pool", out_dtype)
            _need(v_pool, "value pool", out_dtype)
            _need(page_table, "page table", torch.int32, 2)
            _need(token_slot, "token_slot", torch.int32, 1)
            _need(token_end, "token_end", torch.int32, 1)
            table_stride = page_table.shape[1]
        self._check(self.lib.sm_rope_store(
            _ptr(qkv), T, heads, kv_heads, head_dim, rotary_dim, _ptr(positions), _ptr(cos_table), _ptr(sin_table),
            _ptr(q), _ptr(kp), _ptr(vp), _dt(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), table_stride, ring,
            _ptr(token_slot), _ptr(token_end), _stream()))
        return q, kp, vp

    def qkv_rope_store_many(self, x, w_qkv, b_qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim, rotary_dim,
                            want_packed, k_pool=None, v_pool=None, page_table=None, ring=0, token_slot=None, token_end=None):
        """The q/k/v product of many tokens with bias, rotation and the cache write in its epilogue (what ``linear`` and
        ``rope_store`` do in two launches through a float copy of q, k and v). Returns (q, k_packed, v_packed) like
        ``rope_store``, or None, having done nothing, where the kernel does not take the product (160 tokens or
        fewer, other head sizes than 64 and 128, a partial rotation, float operands): the caller then goes the
        other way."""
        if x.shape[0] <= 160 and rotary_dim == head_dim:
            # few tokens: the small tcgen05 kernel's epilogue does the same (head sizes that divide 128)
            got = self.qkv_rope_store_fused(x, w_qkv, b_qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim,
                                            rotary_dim, k_pool, v_pool, page_table, ring, token_slot, want_packed=True,
                                            token_end=token_end)
            return got if got is None or want_packed else (got[0], None, None)
        if (not self.use_tensor_cores or w_qkv.dtype != torch.bfloat16 or self._dtype_of(x) != torch.bfloat16
                or x.shape[0] <= 160 or head_dim not in (64, 128) or rotary_dim != head_dim):
            return None
        x = self.materialize(x)
        _need(x, "x", torch.bfloat16, 2)
        _need(w_qkv, "w_qkv", torch.bfloat16, 2)
        T, K = x.shape
        if w_qkv.shape != ((heads + 2 * kv_heads) * head_dim, K):
            raise KernelError(f"q/k/v weights are {tuple(w_qkv.shape)}, expected {((heads + 2 * kv_heads) * head_dim, K)}")
        _need(positions, "positions", torch.int32, 1)
        _need(cos_table, "cos table", torch.float32, 2)
        _need(sin_table, "sin table", torch.float32, 2)
        if cos_table.shape[1] != head_dim // 2:
            raise KernelError("cos/sin tables do not match head_dim")
        q = torch.empty((T, heads, head_dim), dtype=torch.bfloat16, device=x.device)
        kp = vp = None
        if want_packed and kv_heads:
            kp = torch.empty((T, kv_heads, head_dim), dtype=torch.bfloat16, device=x.device)
            vp = torch.empty_like(kp)
        table_stride = 0
        if k_pool is not None:
            _need(k_pool, "key pool", torch.bfloat16)
            _need(v_pool, "value pool", torch.bfloat16)
            _need(page_table, "page table", torch.int32, 2)
            _need(token_slot, "token_slot", torch.int32, 1)
            _need(token_end, "token_end", torch.int32, 1)
            table_stride = page_table.shape[1]
        taken = ctypes.c_int(0)
        self._check(self.lib.sm_gemm_pair_qkv(
            _ptr(x), _ptr(w_qkv), T, K, _ptr(b_qkv), _dt(b_qkv) if b_qkv is not None else F32, heads, kv_heads, head_dim,
            _ptr(positions), _ptr(cos_table), _ptr(sin_table), _ptr(q), _ptr(kp), _ptr(vp), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), table_stride, ring, _ptr(token_slot), _ptr(token_end), _ptr(self.error_flag),
            ctypes.byref(taken), _stream()))
        return (q, kp, vp) if taken.value else None

    # ---- matrix products ---------------------------------------------------------------
    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                  accumulate: bool = False) -> torch.Tensor:
        _need(x, "x", ndim=2)
        _need(w, "w", ndim=2)
        _need(out, "out", ndim=2)
        T, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (T, N):
            raise KernelError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if bias is not None and _need(bias, "bias", ndim=1).numel() != N:
            raise KernelError(f"bias has {bias.numel()} elements, expected {N}")
        self._check(self.lib.sm_gemm_simt(_ptr(x), _dt(x), _ptr(w), _dt(w), _ptr(bias),
                                          _dt(bias) if bias is not None else F32, _ptr(out), _dt(out), T, N, K,
                                          int(accumulate), _stream()))
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
               out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
        """out (+)= x @ w.T + bias. float32 operands run on the CUDA cores in float; bfloat16
        operands run on the tensor cores where the shape allows, else on the CUDA cores."""
        if out is None:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype or self._dtype_of(x), device=w.device)
        if self._skinny_ok(x, w) and (not accumulate or out.dtype == torch.float32):
            return self.gemm_skinny(x, w, bias, out, mode=1 if accumulate else 0)
        x = self.materialize(x)
        if self._tensor_core_ok(x, w) and (not accumulate or out.dtype == torch.float32):
            return self.gemm_tc(x, w, bias, out, mode=1 if accumulate else 0)
        return self.gemm_simt(x, w, bias, out, accumulate)

    def gated_linear(self, x, w_gate_up: torch.Tensor, hidden: int, out_dtype: torch.dtype,
                     activation: str = "silu") -> torch.Tensor:
        """act(x @ w_gate.T) * (x @ w_up.T) with w_gate_up = [w_gate; w_up]."""
        act = self.activation_code(activation)
        if self._skinny_ok(x, w_gate_up, gated=True):
            out = torch.empty((x.shape[0], hidden), dtype=out_dtype, device=w_gate_up.device)
            return self.gemm_skinny(x, w_gate_up, None, out, mode=2, up_offset=hidden, activation=act)
        x = self.materialize(x)
        if self._tensor_core_ok(x, w_gate_up):
            out = torch.empty((x.shape[0], hidden), dtype=out_dtype, device=x.device)
            return self.gemm_tc(x, w_gate_up, None, out, mode=2, up_offset=hidden, activation=act)
        gate_up = self.linear(x, w_gate_up, None, out_dtype=torch.float32)
        self.lap("ffn_up")
        out = self.swiglu(gate_up, out_dtype, activation)
        self.lap("activation")
        return out

    # ---- rows under a norm that has not been computed yet -------------------------------
    @staticmethod
    def materialize(x) -> torch.Tensor:
        return x.tensor() if isinstance(x, NormedRows) else x

    @staticmethod
    def _dtype_of(x) -> torch.dtype:
        return x.out_dtype if isinstance(x, NormedRows) else x.dtype

    def _skinny_ok(self, x, w: torch.Tensor, gated: bool = False) -> bool:
        """A handful of tokens and bfloat16 weights: the weight-streaming kernel, which also
        takes the norm as its prologue."""
        if not self.use_skinny or w.dtype != torch.bfloat16 or x.shape[0] > self.skinny_max_tokens:
            return False
        if x.shape[0] > 8 and self.skinny_single_round_above_8 and self.lib.sm_gemm_skinny_rounds(
                x.shape[0], w.shape[0] // 2 if gated else w.shape[0], x.shape[1], int(gated)) > 1:
            return False   # its CTAs would take their weights in rounds: the tcgen05 kernel streams them better
        if isinstance(x, NormedRows):
            if x.rows is not None or x.out_dtype != torch.bfloat16 or x.done is not None:
                return False
        elif x.dtype != torch.bfloat16:
            return False
        elif (self.use_tensor_cores and self.lib.sm_gemm_tc_supports(x.shape[0], w.shape[0], x.shape[1])
              and self.lib.sm_gemm_skinny_rounds(x.shape[0], w.shape[0] // 2 if gated else w.shape[0], x.shape[1],
                                                 int(gated)) >= self.skinny_most_rounds + 1):
            # rows that need no norm and a K so long that a CTA takes its weights in three rounds or more: the tcgen05
            # kernel's clusters stream them better (3,584 x 18,944 at 8 tokens: 26 against 39 us; at two rounds the
            # weight-streaming kernel still wins, 1,536 x 8,960: 8 against 11 us)
            return False
        if (self.use_tensor_cores and self.lib.sm_gemm_tc_supports(x.shape[0], w.shape[0], x.shape[1])
                and self._row_tiles_fill_the_gpu(w.shape[0])):
            return False   # enough row tiles to keep every SM streaming on the tcgen05 kernel without any split of K
        return bool(self.lib.sm_gemm_skinny_supports(x.shape[0], w.shape[0], x.shape[1]))

    def _row_tiles_fill_the_gpu(self, rows: int) -> bool:
        """Whether a product with this many weight rows gives the tcgen05 kernel a full wave of its 128-row tiles at
        two CTAs an SM without any split of K (measured on 148 SMs: at 296 tiles, 37,888 x 3,584, it takes 45 us against
        the weight-streaming kernel's 53; at 1,187 tiles, 151,936 x 896, it streams 5.0 TB/s against 3.1)."""
        if not hasattr(self, "_sm_count"):
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return (rows + 127) // 128 >= 2 * self._sm_count

    def gemm_skinny(self, x, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int = 0,
                    up_offset: int = 0, activation: int = 0) -> torch.Tensor:
        """mode 0: out = x w^T + bias; 1: float out += x w^T; 2: gated (see gemm_tc)."""
        norm_w, eps, src = (x.weight, x.eps, x.residual) if isinstance(x, NormedRows) else (None, 0.0, x)
        _need(src, "x", torch.float32 if norm_w is not None else torch.bfloat16, 2)
        _need(w, "w", torch.bfloat16, 2)
        _need(out, "out", ndim=2)
        T, K = src.shape
        N = out.shape[1]
        if w.shape[1] != K or out.shape[0] != T or w.shape[0] != (up_offset + N if mode == 2 else N):
            raise KernelError(f"gemm shapes do not agree: x {tuple(src.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if mode == 1 and out.dtype != torch.float32:
            raise KernelError("accumulation needs a float32 output")
        self._check(self.lib.sm_gemm_skinny(
            _ptr(src), _ptr(norm_w), _dt(norm_w) if norm_w is not None else F32, ctypes.c_float(eps), _ptr(w), T, N, K,
            mode | (activation << 8), _ptr(bias), _dt(bias) if bias is not None else F32, _ptr(out), _dt(out), up_offset, _stream()))
        return out

    def qkv_rope_store_fused(self, x, w_qkv, b_qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim,
                             rotary_dim, k_pool, v_pool, page_table, ring, token_slot, want_packed=False, token_end=None):
        """For up to 160 tokens: q/k/v product, bias, rotation and cache write in one launch (the weight-streaming
        kernel with the norm as its prologue for a handful of tokens, else the small tcgen05 kernel).
        Returns q [T, heads, head_dim], or with ``want_packed`` (q, k_packed, v_packed) for a step that attends over
        its own packed keys; ``token_end`` keeps positions that a ring has no place for out of the cache; ``k_pool``
        None writes nothing to the cache. None when the shapes are not the fused kernels'."""
        if head_dim % 16 or rotary_dim != head_dim or (k_pool is not None and k_pool.dtype != torch.bfloat16):
            return None
        if k_pool is None and not want_packed:
            return None
        if not self._skinny_ok(x, w_qkv):
            return self._qkv_rope_store_tc(x, w_qkv, b_qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim,
                                           k_pool, v_pool, page_table, ring, token_slot, want_packed, token_end)
        norm_w, eps, src = (x.weight, x.eps, x.residual) if isinstance(x, NormedRows) else (None, 0.0, x)
        T, K = src.shape
        q = torch.empty((T, heads, head_dim), dtype=torch.bfloat16, device=src.device)
        kp = vp = None
        if want_packed and kv_heads:
            kp = torch.empty((T, kv_heads, head_dim), dtype=torch.bfloat16, device=src.device)
            vp = torch.empty_like(kp)
        self._check(self.lib.sm_gemm_skinny_qkv(
            _ptr(src), _ptr(norm_w), _dt(norm_w) if norm_w is not None else F32, ctypes.c_float(eps), _ptr(w_qkv), T, K,
            _ptr(b_qkv), _dt(b_qkv) if b_qkv is not None else F32, heads, kv_heads, head_dim, rotary_dim,
            _ptr(positions), _ptr(cos_table), _ptr(sin_table), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
            page_table.shape[1], ring, _ptr(token_slot), _ptr(kp), _ptr(vp), _ptr(token_end), _stream()))
        return (q, kp, vp) if want_packed else q

    def _qkv_rope_store_tc(self, x, w_qkv, b_qkv, positions, cos_table, sin_table, heads, kv_heads, head_dim, k_pool, v_pool,
                           page_table, ring, token_slot, want_packed=False, token_end=None):
        """The same for up to 160 tokens on the tcgen05 kernel, whose split-K clusters do bias, rotation and cache
        write where they add their sums up. Returns q, or with ``want_packed`` (q, k_packed, v_packed) for a step that
        attends over its own packed keys; ``token_end`` keeps positions that a ring has no place for out of the cache.
        None when the shape is not taken."""
        T, K = x.shape
        if (T > 160 or 128 % head_dim or not self.use_tensor_cores or w_qkv.dtype != torch.bfloat16
                or self._dtype_of(x) != torch.bfloat16 or not self.lib.sm_gemm_tc_supports(T, w_qkv.shape[0], K)
                or (k_pool is not None and k_pool.dtype != torch.bfloat16)):
            return None
        rows = self.materialize(x)
        q = torch.empty((T, heads, head_dim), dtype=torch.bfloat16, device=rows.device)
        kp = vp = None
        if want_packed and kv_heads:
            kp = torch.empty((T, kv_heads, head_dim), dtype=torch.bfloat16, device=rows.device)
            vp = torch.empty_like(kp)
        taken = ctypes.c_int(0)
        self._check(self.lib.sm_gemm_tc_qkv(
            _ptr(rows), _ptr(w_qkv), T, K, _ptr(b_qkv), _dt(b_qkv) if b_qkv is not None else F32, heads, kv_heads,
            head_dim, head_dim, _ptr(positions), _ptr(cos_table), _ptr(sin_table), _ptr(q), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), page_table.shape[1], ring, _ptr(token_slot), _ptr(kp), _ptr(vp), _ptr(token_end),
            _ptr(self.error_flag), ctypes.byref(taken), _stream()))
        if not taken.value:
            return None
        return (q, kp, vp) if want_packed else q

    def _tensor_core_ok(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        return (self.use_tensor_cores and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and bool(self.lib.sm_gemm_tc_supports(x.shape[0], w.shape[0], x.shape[1])))

    def gemm_tc(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int = 0,
                up_offset: int = 0, activation: int = 0) -> torch.Tensor:
        """The tcgen05 product. mode 0: out = x w^T + bias; 1: float out += x w^T;
        2: out = act(x w[:N]^T) * (x w[up_offset:up_offset+N]^T)."""
        _need(x, "x", torch.bfloat16, 2)
        _need(w, "w", torch.bfloat16, 2)
        _need(out, "out", ndim=2)
        T, K = x.shape
        N = out.shape[1]
        rows_needed = up_offset + N if mode == 2 else N
        if w.shape[1] != K or out.shape[0] != T or w.shape[0] != rows_needed:
            raise KernelError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if mode == 1 and out.dtype != torch.float32:
            raise KernelError("accumulation needs a float32 output")
        if bias is not None and _need(bias, "bias", ndim=1).numel() != N:
            raise KernelError(f"bias has {bias.numel()} elements, expected {N}")
        if T == 0:
            return out
        paired = self.lib.sm_gemm_pair_takes(_ptr(x), _ptr(w), _ptr(out), _dt(out), T, N, K, mode)
        need = 0 if paired else int(self.lib.sm_gemm_tc_workspace_bytes(T, N, K, int(mode == 2)))
        workspace = torch.empty((need // 4,), dtype=torch.float32, device=x.device) if need else None
        self._check(self.lib.sm_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), _dt(bias) if bias is not None else F32, _ptr(out),
                                        _dt(out), T, N, K, mode | (activation << 8), up_offset, _ptr(workspace), _ptr(self.error_flag),
                                        _stream()))
        return out

    def gemm_pair_enable(self, on: bool) -> None:
        """Whether products of more than 160 tokens go to the two-CTA kernel (the default) or stay on the one-CTA
        kernel: for comparisons of the two."""
        self.lib.sm_gemm_pair_enable(int(bool(on)))

    def check_error_flag(self) -> None:
        """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            for words in self._fused_barriers:
                words.zero_()
            raise KernelError(f"a kernel's bounded wait ran out (code {code}); its output is not valid")

    # ---- attention ---------------------------------------------------------------------
    def attention_plain(self, q, positions, scale, window, *, k_packed=None, v_packed=None, token_seq_start=None,
                        k_pool=None, v_pool=None, page_table=None, ring=0, token_slot=None, kv_heads=None):
        _need(q, "q", ndim=3)
        T, heads, head_dim = q.shape
        _need(positions, "positions", torch.int32, 1)
        out = torch.empty_like(q)
        table_stride = 0
        if k_packed is not None:
            _need(k_packed, "packed keys", q.dtype, 3)
            _need(v_packed, "packed values", q.dtype, 3)
            _need(token_seq_start, "token_seq_start", torch.int32, 1)
            kv_heads = k_packed.shape[1]
        if k_pool is not None:
            _need(k_pool, "key pool", q.dtype)
            _need(v_pool, "value pool", q.dtype)
            _need(page_table, "page table", torch.int32, 2)
            _need(token_slot, "token_slot", torch.int32, 1)
            table_stride = page_table.shape[1]
        self._check(self.lib.sm_attention_plain(
            _ptr(q), _ptr(out), _dt(q), T, heads, kv_heads, head_dim, ctypes.c_float(scale), int(window or 0),
            _ptr(positions), _ptr(k_packed), _ptr(v_packed), _ptr(token_seq_start), _ptr(k_pool), _ptr(v_pool),
            _ptr(page_table), table_stride, ring, _ptr(token_slot), _stream()))
        return out

    def attention_prefill(self, q, k_packed, v_packed, step, scale, window):
        """Causal attention of whole prompts over their own keys (sequences start at 0)."""
        if self.use_fast_attention and q.dtype == torch.bfloat16 and step.prefill_tiles is not None:
            if self.use_tcgen05_attention and self.lib.sm_attention_prefill_tc_supports(q.shape[1], k_packed.shape[1], q.shape[2]):
                return self.attention_prefill_tcgen05(q, k_packed, v_packed, step.prefill_tiles, scale, window,
                                                      longest=step.max_seq_len)
            if self.lib.sm_attention_prefill_supports(q.shape[2]):
                return self.attention_prefill_mma(q, k_packed, v_packed, step.prefill_tiles, scale, window)
        return self.attention_plain(q, step.positions, scale, window, k_packed=k_packed, v_packed=v_packed,
                                    token_seq_start=step.token_seq_start)

    def _prefill_operands(self, q, k_packed, v_packed, tiles):
        _need(q, "q", torch.bfloat16, 3)
        _need(k_packed, "packed keys", torch.bfloat16, 3)
        _need(v_packed, "packed values", torch.bfloat16, 3)
        _need(tiles, "tiles", torch.int32, 2)
        return torch.empty_like(q)

    def attention_prefill_mma(self, q, k_packed, v_packed, tiles, scale, window):
        """The mma.sync kernel: head sizes in steps of 16 up to 128."""
        out = self._prefill_operands(q, k_packed, v_packed, tiles)
        self._check(self.lib.sm_attention_prefill(_ptr(q), _ptr(k_packed), _ptr(v_packed), _ptr(out), _ptr(tiles),
                                                  tiles.shape[0], q.shape[1], k_packed.shape[1], q.shape[2],
                                                  ctypes.c_float(scale), int(window or 0), _stream()))
        return out

    def attention_prefill_tcgen05(self, q, k_packed, v_packed, tiles, scale, window, longest=0, variant=-1):
        """The tcgen05 kernel: head sizes 64 and 128. ``longest``: the longest sequence, if known; ``variant``:
        0 one CTA an SM, 1 two (head size 64), -1 the launcher's choice."""
        out = self._prefill_operands(q, k_packed, v_packed, tiles)
        self._check(self.lib.sm_attention_prefill_tc(_ptr(q), _ptr(k_packed), _ptr(v_packed), _ptr(out), _ptr(tiles),
                                                     tiles.shape[0], q.shape[0], q.shape[1], k_packed.shape[1], q.shape[2],
                                                     ctypes.c_float(scale), int(window or 0), int(longest), int(variant),
                                                     _ptr(self.error_flag), _stream()))
        return out

    def kv_store(self, k_packed, v_packed, step, cache) -> None:
        """This step's packed keys and values into the cache (what ``rope_store`` does beside its rotation, for
        steps whose attention had to read the ring before its rows are replaced)."""
        _need(k_packed, "packed keys", cache.k_pool.dtype, 3)
        _need(v_packed, "packed values", cache.k_pool.dtype, 3)
        T, kv_heads, head_dim = k_packed.shape
        self._check(self.lib.sm_kv_store(_ptr(k_packed), _ptr(v_packed), _dt(k_packed), T, kv_heads, head_dim,
                                         _ptr(cache.k_pool), _ptr(cache.v_pool), _ptr(step.positions),
                                         _ptr(cache.page_table), cache.page_table.shape[1], cache.ring,
                                         _ptr(step.token_slot), _ptr(step.token_end), _stream()))

    def attention_extend(self, q, k_packed, v_packed, step, scale, window, cache, cache_written=False):
        """Causal attention of sequences that go on from the cache by any number of tokens: keys and values of
        earlier positions from the cache, the step's own from the packed tensors (the cache need not hold them yet)."""
        from_cache = (self.use_fast_attention and q.dtype == torch.bfloat16 and cache.ring == 0 and cache_written
                      and cache.k_pool.dtype == torch.bfloat16)
        tiles_from_cache = (from_cache and self.use_tcgen05_attention and step.extend_tiles is not None and not window
                            and self.lib.sm_attention_extend_tc_supports(q.shape[1], k_packed.shape[1], q.shape[2],
                                                                         ctypes.c_longlong(cache.k_pool.shape[0])))
        rows_limit = self.extend_rows_as_decode_tc if tiles_from_cache else self.extend_rows_as_decode
        if (from_cache and q.shape[0] <= rows_limit
                and self.lib.sm_attention_decode_supports(q.shape[1], k_packed.shape[1], q.shape[2])):
            # a few tokens onto a live sequence: every token as a row of the decode kernel, which shares a row's keys
            # out among the CTAs of a cluster (the tiled kernels below have one CTA per 64 or 128 queries and head, each
            # with the whole chain of keys to itself: 8 tokens onto 2,000 took 2.0 ms a step that way)
            return self.attention_decode(q, step.positions, step.token_slot, scale, window, cache.k_pool, cache.v_pool,
                                         cache.page_table, cache.ring, k_packed.shape[1], step.max_seq_len, late=True)
        if tiles_from_cache:
            # many tokens onto the cache (prompt portions): the tcgen05 kernel, with every key from the paged pools
            _need(q, "q", torch.bfloat16, 3)
            _need(step.extend_tiles, "tiles", torch.int32, 2)
            _need(cache.page_table, "page table", torch.int32, 2)
            out = torch.empty_like(q)
            self._check(self.lib.sm_attention_extend_tc(
                _ptr(q), _ptr(out), _ptr(step.extend_tiles), step.extend_tiles.shape[0], q.shape[0], q.shape[1],
                k_packed.shape[1], q.shape[2], ctypes.c_float(scale), int(window or 0), _ptr(cache.k_pool), _ptr(cache.v_pool),
                _ptr(cache.page_table), cache.page_table.shape[1], ctypes.c_longlong(cache.k_pool.shape[0]),
                int(step.max_seq_len), int(self.extend_tc_variant), _ptr(self.error_flag), _stream()))
            return out
        if (self.use_fast_attention and q.dtype == torch.bfloat16 and step.extend_tiles is not None
                and self.lib.sm_attention_prefill_supports(q.shape[2])):
            out = self._prefill_operands(q, k_packed, v_packed, step.extend_tiles)
            _need(cache.k_pool, "key pool", torch.bfloat16)
            _need(cache.v_pool, "value pool", torch.bfloat16)
            _need(cache.page_table, "page table", torch.int32, 2)
            self._check(self.lib.sm_attention_extend(
                _ptr(q), _ptr(k_packed), _ptr(v_packed), _ptr(out), _ptr(step.extend_tiles), step.extend_tiles.shape[0],
                q.shape[1], k_packed.shape[1], q.shape[2], ctypes.c_float(scale), int(window or 0), _ptr(cache.k_pool),
                _ptr(cache.v_pool), _ptr(cache.page_table), cache.page_table.shape[1], cache.ring, _stream()))
            return out
        return self.attention_plain(q, step.positions, scale, window, k_packed=k_packed, v_packed=v_packed,
                                    token_seq_start=step.token_seq_start, k_pool=cache.k_pool, v_pool=cache.v_pool,
                                    page_table=cache.page_table, ring=cache.ring, token_slot=step.token_slot)

    def attention_cached(self, q, step, scale, window, cache, kv_heads):
        """Attention of this step's tokens over the keys and values in the cache."""
        if (self.use_fast_attention and q.dtype == torch.bfloat16 and step.mode == "decode"
                and self.lib.sm_attention_decode_supports(q.shape[1], kv_heads, q.shape[2])):
            return self.attention_decode(q, step.positions, step.slot_ids, scale, window, cache.k_pool, cache.v_pool,
                                         cache.page_table, cache.ring, kv_heads, step.max_seq_len)
        return self.attention_plain(q, step.positions, scale, window, k_pool=cache.k_pool, v_pool=cache.v_pool,
                                    page_table=cache.page_table, ring=cache.ring, token_slot=step.token_slot,
                                    kv_heads=kv_heads)

    def attention_decode(self, q, positions, slots, scale, window, k_pool, v_pool, page_table, ring, kv_heads, max_len,
                         late=False):
        """One new token per sequence (row b of q belongs to slots[b] at positions[b]). ``late``: the rows are several
        new positions of a sequence, all of them in the cache already (a short later message onto a live sequence);
        each row attends over the cache up to its own position."""
        _need(q, "q", torch.bfloat16, 3)
        B, heads, head_dim = q.shape
        _need(positions, "positions", torch.int32, 1)
        _need(slots, "slots", torch.int32, 1)
        _need(k_pool, "key pool", torch.bfloat16)
        _need(v_pool, "value pool", torch.bfloat16)
        _need(page_table, "page table", torch.int32, 2)
        out = torch.empty_like(q)
        self._check(self.lib.sm_attention_decode(
            _ptr(q), _ptr(out), B, heads, kv_heads, head_dim, ctypes.c_float(scale), int(window or 0), _ptr(positions),
            _ptr(slots), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), page_table.shape[1], ring, int(max_len),
            ctypes.c_longlong(k_pool.shape[0]), int(bool(late)), _stream()))
        return out

    # ---- a whole decode step in one kernel ------------------------------------------------
    def decode_fused_refusal(self, T, D, H, heads, kv_heads, head_dim, V) -> Optional[str]:
        """None if the fused decode kernel takes these sizes, else the sizes it takes."""
        if self.lib.sm_decode_fused_refusal(T, D, H, heads, kv_heads, head_dim, V):
            return self.lib.sm_last_error().decode("utf-8", "replace")
        return None

    def decode_fused_scratch(self, D, H, heads, kv_heads, head_dim, V, device) -> dict:
        """The buffers a model's fused decode steps share (for up to 16 tokens)."""
        if ctypes.sizeof(FusedLayerRecord) != int(self.lib.sm_decode_fused_layer_bytes()):
            raise KernelError("the layer record of the fused decode step is laid out differently in the library")
        T = 16
        out = {
            "residual": torch.empty((T, D), dtype=torch.float32, device=device),
            "q": torch.empty((T, heads * head_dim), dtype=torch.bfloat16, device=device),
            "att": torch.empty((T, heads * head_dim), dtype=torch.bfloat16, device=device),
            "h": torch.empty((T, H), dtype=torch.bfloat16, device=device),
            "att_parts": torch.empty((T * kv_heads * 16 * 16 * (head_dim + 2),), dtype=torch.float32, device=device),
            "att_counters": torch.zeros((T * kv_heads,), dtype=torch.int32, device=device),
            "barrier": torch.zeros((4,), dtype=torch.int32, device=device),
            "logits": torch.empty((T, V), dtype=torch.float32, device=device),
        }
        self._fused_barriers.append(out["barrier"])
        return out

    def decode_fused_maps(self, weights, sizes: dict, device) -> tuple:
        """The tensor maps of a model's weight matrices for the fused decode step, in the order the kernel uses them
        (``weights``: per layer q/k/v, o, gate/up, down; then the head), as a device tensor, and the blocks of K a
        copy of each kind of product brings."""
        bk = (ctypes.c_int * 5)()
        self._check(self.lib.sm_decode_fused_blocks(sizes["D"], sizes["H"], sizes["heads"], sizes["kv_heads"],
                                                     sizes["head_dim"], sizes["V"], bk))
        host = ctypes.create_string_buffer(128 * len(weights) + 64)
        base = (ctypes.addressof(host) + 63) // 64 * 64
        for i, w in enumerate(weights):
            _need(w, "weight", torch.bfloat16, 2)
            kind = 4 if i == len(weights) - 1 else i % 4
            self._check(self.lib.sm_decode_fused_encode_map(ctypes.c_void_p(base + 128 * i), _ptr(w),
                                                             ctypes.c_longlong(w.shape[0]), w.shape[1], bk[kind]))
        raw = ctypes.string_at(base, 128 * len(weights))
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device), [int(x) for x in bk]

    def decode_fused(self, layers: torch.Tensor, maps: torch.Tensor, bk, n_layers: int, sizes: dict, embed, head, norm_f, eps_f: float, scale: float,
                     tokens, positions, token_slot, rows: Optional[torch.Tensor], scratch: dict,
                     status: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """One decode step of ``n_layers`` standard layers (records in ``layers``, a uint8 device tensor) with final
        norm and output head; returns float logits ``[len(rows), V]`` (a view of the scratch) or None."""
        T = tokens.numel()
        n_rows = 0 if rows is None else rows.numel()
        _need(tokens, "tokens", torch.int32, 1)
        _need(positions, "positions", torch.int32, 1)
        _need(token_slot, "token_slot", torch.int32, 1)
        if rows is not None:
            _need(rows, "rows", torch.int32, 1)
        splits = int(self.lib.sm_decode_fused_splits(T, sizes["kv_heads"]))
        self._check(self.lib.sm_decode_fused(
            _ptr(layers), _ptr(maps), (ctypes.c_int * 5)(*bk), n_layers, T, sizes["D"], sizes["H"], sizes["heads"], sizes["kv_heads"], sizes["head_dim"], sizes["V"],
            _ptr(embed), _ptr(head), _ptr(norm_f), ctypes.c_float(eps_f), ctypes.c_float(scale), _ptr(tokens), _ptr(positions),
            _ptr(token_slot), _ptr(rows), n_rows, splits, _ptr(scratch["residual"]), _ptr(scratch["q"]), _ptr(scratch["att"]),
            _ptr(scratch["h"]), _ptr(scratch["att_parts"]), _ptr(scratch["att_counters"]), _ptr(scratch["barrier"]),
            _ptr(scratch["logits"]), _ptr(self.error_flag), _ptr(status), _ptr(scratch.get("trace")), _stream()))
        return scratch["logits"][:n_rows] if n_rows else None

    # ---- sampling ----------------------------------------------------------------------
    def argmax(self, logits: torch.Tensor, banned: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
        _need(logits, "logits", torch.float32, 2)
        if banned is not None:
            _need(banned, "banned", torch.uint8, 1)
        if out is None:
            out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        if logits.shape[0] > self.argmax_scratch.numel():
            raise KernelError(f"argmax takes at most {self.argmax_scratch.numel()} rows a call")
        self._check(self.lib.sm_argmax(_ptr(logits), _ptr(banned), _ptr(out), logits.shape[0], logits.shape[1],
                                       _ptr(self.argmax_scratch), _ptr(self.argmax_counters), _stream()))
        return out

    def sample(self, logits, rng_state, temperature, top_k, top_p, banned=None, out=None):
        _need(logits, "logits", torch.float32, 2)
        _need(rng_state, "rng_state", torch.int32, 1)  # xorshift32 words, one per row
        if rng_state.numel() != logits.shape[0]:
            raise KernelError("one rng state per row is needed")
        if banned is not None:
            _need(banned, "banned", torch.uint8, 1)
        if out is None:
            out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        self._check(self.lib.sm_sample(_ptr(logits), _ptr(banned), _ptr(out), _ptr(rng_state), logits.shape[0],
                                       logits.shape[1], ctypes.c_float(temperature), int(top_k), ctypes.c_float(top_p),
                                       _stream()))
        return out


_ops: dict = {}


def get_ops(kernels: str = "fast") -> Ops:
    """The shared instance for a choice of kernels."""
    if kernels not in _ops:
        _ops[kernels] = Ops(kernels)
    return _ops[kernels]
