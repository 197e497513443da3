"""ctypes binding of libquic_b200.so plus per-op wrappers shaped like the reference's
kernel getters.

The reference loads one JIT torch extension per op through getters that return a module
with a ``forward`` (kernels/__init__.py:42-115: ``gemm() rmsnorm() rope() swiglu() sampler()
flash_attn_decode() marlin()``).  Here one ahead-of-time library built for sm_100a carries
every op behind a C ABI (include/quic_b200.h); the getters below return small objects with
the same ``forward`` call shapes, so model code written against the reference's loader
keeps working.  There is no CPU or eager fallback: a missing library or a call with CPU
tensors raises.
"""

from __future__ import annotations

import ctypes as C
import functools
import os
from types import SimpleNamespace

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libquic_b200.so")

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, INTER, GROUP, QKV_N = 896, 14, 2, 64, 4864, 128, 1152
ROWS_NATURAL, ROWS_ROPE_PAIRS = 0, 1
# M >= TENSOR_MIN_ROWS runs the tcgen05 GEMM when True; the dequant GEMV in row chunks otherwise.
TENSOR_PATH = True
TENSOR_MIN_ROWS = 2


class W4(C.Structure):
    """quic_w4_t"""

    _fields_ = [
        ("qw", C.c_void_p),
        ("sc", C.c_void_p),
        ("zp", C.c_void_p),
        ("bias", C.c_void_p),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("w16", C.c_void_p),
    ]


class Layer(C.Structure):
    """quic_layer_t"""

    _fields_ = [
        ("qkv", W4),
        ("o", W4),
        ("gate_up", W4),
        ("down", W4),
        ("ln1", C.c_void_p),
        ("ln2", C.c_void_p),
    ]


class Model(C.Structure):
    """quic_model_t"""

    _fields_ = [
        ("n_layers", C.c_int32),
        ("vocab", C.c_int32),
        ("eps", C.c_float),
        ("max_pos", C.c_int32),
        ("layers", C.POINTER(Layer)),
        ("embed", C.c_void_p),
        ("final_norm", C.c_void_p),
        ("rope_cos", C.c_void_p),
        ("rope_sin", C.c_void_p),
    ]


class Decode(C.Structure):
    """quic_decode_t"""

    _fields_ = [
        ("kv", C.c_void_p),
        ("n_slots", C.c_int32),
        ("s_max", C.c_int32),
        ("tok", C.c_void_p),
        ("pos", C.c_void_p),
        ("rows", C.c_void_p),
        ("batch", C.c_int32),
        ("out_tokens", C.c_void_p),
        ("ring", C.c_int32),
        ("step_counter", C.c_void_p),
        ("logits", C.c_void_p),
        ("scratch", C.c_void_p),
        ("attn_splits", C.c_int32),
        ("ctx_hint", C.c_int32),
    ]


class Prefill(C.Structure):
    """quic_prefill_t"""

    _fields_ = [
        ("ids", C.c_void_p),
        ("row_slot", C.c_void_p),
        ("row_pos", C.c_void_p),
        ("seq_start", C.c_void_p),
        ("seq_len", C.c_void_p),
        ("seq_slot", C.c_void_p),
        ("rows", C.c_int32),
        ("n_seq", C.c_int32),
        ("max_len", C.c_int32),
        ("kv", C.c_void_p),
        ("n_slots", C.c_int32),
        ("s_max", C.c_int32),
        ("tok", C.c_void_p),
        ("pos", C.c_void_p),
        ("first_tokens", C.c_void_p),
        ("logits", C.c_void_p),
        ("scratch", C.c_void_p),
        ("seq_off", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol declared in include/quic_b200.h
_P, _I32, _I64, _F = C.c_void_p, C.c_int32, C.c_int64, C.c_float
SIGNATURES = {
    "quic_last_error": (C.c_char_p, []),
    "quic_abi_version": (C.c_int, []),
    "quic_set_pdl": (None, [C.c_int]),
    "quic_w4_prepack": (C.c_int, [_P, _P, _P, _I32, _I32, _I32, _I32, _I32, _P, _P, _P, _P]),
    "quic_w4_dequant": (C.c_int, [C.POINTER(W4), _P, _P]),
    "quic_w4a16_linear": (C.c_int, [_P, C.POINTER(W4), _P, _I32, _I32, _P, _P]),
    "quic_w4a16_workspace_bytes": (_I64, [_I32, _I32, _I32]),
    "quic_w4a16_tensor_status": (C.c_int, []),
    "quic_w4a16_tensor_test_hook": (None, [C.c_uint32, _I32]),
    "quic_attn_stream_test_hook": (None, [_I32]),
    "quic_rmsnorm": (C.c_int, [_P, _P, _P, _F, _P, _P, _I32, _P]),
    "quic_rope_table_init": (C.c_int, [_P, _I32, _P, _P, _P]),
    "quic_rope": (C.c_int, [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _P]),
    "quic_qkv_rope_append": (C.c_int, [_P, _P, _P, _P, _P, _I32, _P, _P, _P, _I32, _I32, _I32, _P]),
    "quic_attn_prefill": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, C.c_float, _P, _P]),
    "quic_swiglu": (C.c_int, [_P, _P, _P, _I32, _P]),
    "quic_swiglu_fused": (C.c_int, [_P, _P, _I32, _P]),
    "quic_argmax": (C.c_int, [_P, _I32, _I32, _P, _P]),
    "quic_gemm_f16": (C.c_int, [_P, _P, _P, _P, _I32, _I32, _I32, _P]),
    "quic_lm_head_argmax": (C.c_int, [_P, _P, _F, _P, _I32, _I32, _P, _P, _P, _P]),
    "quic_lm_head_scratch_bytes": (_I64, [_I32, _I32]),
    "quic_attn_decode": (C.c_int, [_P, _P, _P, _I64, _I64, _P, _P, _I32, _F, _P, _I32, _I32, _P, _P]),
    "quic_attn_decode_noalloc": (C.c_int, [_P, _P, _P, _I64, _I64, _P, _P, _I32, _F, _P, _I32, _I32, _P]),
    "quic_attn_decode_noalloc_max_bytes": (_I64, []),
    "quic_attn_decode_cta": (C.c_int, [_P, _P, _P, _I64, _I64, _P, _P, _I32, _F, _P, _I32, _P]),
    "quic_attn_decode_cta_max_tokens": (_I32, []),
    "quic_attn_pick_splits": (_I32, [_I32, _I32]),
    "quic_attn_scratch_bytes": (_I64, [_I32, _I32]),
    "quic_set_tensor_min_batch": (None, [_I32]),
    "quic_set_prefill_tensor_attention": (None, [C.c_int]),
    "quic_set_mma_chain_min_batch": (None, [_I32]),
    "quic_decode_pick_splits": (_I32, [_I32, _I32]),
    "quic_decode_scratch_bytes": (_I64, [_I32, _I32, _I32]),
    "quic_decode_launch_count": (_I32, [C.POINTER(Model), C.POINTER(Decode)]),
    "quic_decode_step": (C.c_int, [C.POINTER(Model), C.POINTER(Decode), _P]),
    "quic_prefill_scratch_bytes": (_I64, [_I32, _I32, _I32]),
    "quic_prefill": (C.c_int, [C.POINTER(Model), C.POINTER(Prefill), _P]),
    "quic_decode_graph_create": (C.c_int, [C.POINTER(Model), C.POINTER(Decode), _I32, _P, C.POINTER(_P)]),
    "quic_graph_launch": (C.c_int, [_P, _P]),
    "quic_graph_run_host": (C.c_int, [_P, _P, _P, _P, C.c_int32, _P, _P, C.c_int32]),
    "quic_graph_destroy": (C.c_int, [_P]),
    "quic_persist_max_rows": (_I32, []),
    "quic_persist_stream_bytes": (_I64, [_I32]),
    "quic_persist_sync_bytes": (_I64, []),
    "quic_persist_pick_splits": (_I32, [_I32, _I32]),
    "quic_persist_pack": (C.c_int, [C.POINTER(Model), _P, _P]),
    "quic_decode_persist": (C.c_int, [C.POINTER(Model), C.POINTER(Decode), _P, _P, _I32, _P]),
    "quic_decode_persist_status": (C.c_int, [_P, _P, C.POINTER(_I32)]),
    "quic_decode_persist_run_host": (C.c_int, [C.POINTER(Model), C.POINTER(Decode), _P, _P, _I32, _P, _P, _P, _I32,
                                               _P, _P, _I32, _P]),
}


@functools.cache
def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback)."""
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()); this package has no CPU or eager fallback"
        )
    handle = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def check(rc: int, what: str = "") -> None:
    """Turns a negative return code into RuntimeError, the reference's error convention
    (TORCH_CHECK -> RuntimeError, e.g. kernels/cuda/flash_attn_decode.cu:136-161)."""
    if rc != 0:
        msg = lib().quic_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"quic_b200 {what} failed ({rc}): {msg}")


def stream_ptr() -> int:
    """Raw handle of torch's current CUDA stream on the current device."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
    except AttributeError:
        return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("quic_b200: CUDA tensors required (no CPU path)")


def _need_half(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.float16:
            raise RuntimeError("quic_b200: fp16 tensors required")


# ---------------------------------------------------------------------------------
# W4A16 weights on the device
# ---------------------------------------------------------------------------------
class W4Weight:
    """One (possibly fused) W4A16 matrix in the device layout of quic_w4_t.

    Built from checkpoint tensors (reference layout, src/quant/checkpoint.py:23-36) by the
    GPU repack kernel; replaces MarlinWeight (src/quant/marlin.py:128)."""

    def __init__(self, n: int, k: int, device, bias: torch.Tensor | None = None):
        if n % 32 or k % GROUP:
            raise RuntimeError("W4Weight: N must be a multiple of 32 and K of 128")
        self.size_n, self.size_k = n, k
        self.qw = torch.empty(k // 8, n, dtype=torch.int32, device=device)
        self.sc = torch.empty(k // GROUP, n, dtype=torch.float16, device=device)
        self.zp = torch.empty(k // GROUP, n // 2, dtype=torch.uint8, device=device)
        self.bias = bias
        self._workspace: torch.Tensor | None = None

    def put(self, packed: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor,
            row_offset: int = 0, row_order: int = ROWS_NATURAL) -> None:
        """Repacks one checkpoint layer into columns [row_offset, row_offset + N_layer)."""
        dev = self.qw.device
        packed = packed.to(dev, torch.int32).contiguous()
        scale = scale.to(dev, torch.float16).contiguous()
        zero_point = zero_point.to(dev, torch.int32).contiguous()
        n, k8 = packed.shape
        if k8 * 8 != self.size_k or scale.shape != (n, self.size_k // GROUP) or \
                zero_point.shape != (n // 8, self.size_k // GROUP):
            raise RuntimeError("W4Weight.put: checkpoint tensor shapes do not match")
        check(lib().quic_w4_prepack(ptr(packed), ptr(scale), ptr(zero_point), n, self.size_k,
                                    row_order, row_offset, self.size_n, ptr(self.qw), ptr(self.sc),
                                    ptr(self.zp), stream_ptr()), "w4_prepack")

    def struct(self) -> W4:
        return W4(ptr(self.qw), ptr(self.sc), ptr(self.zp), ptr(self.bias), self.size_n, self.size_k, None)

    def dequant(self) -> torch.Tensor:
        out = torch.empty(self.size_n, self.size_k, dtype=torch.float16, device=self.qw.device)
        s = self.struct()
        check(lib().quic_w4_dequant(C.byref(s), ptr(out), stream_ptr()), "w4_dequant")
        return out

    def workspace(self, m: int) -> torch.Tensor:
        """Split-K workspace, shared by every weight on the device (calls on one stream are ordered)."""
        need = lib().quic_w4a16_workspace_bytes(m, self.size_n, self.size_k)
        key = self.qw.device.index
        ws = _linear_workspace.get(key)
        if ws is None or ws.numel() * 4 < need:
            ws = torch.zeros((max(need, 1 << 22) + 3) // 4, dtype=torch.float32, device=self.qw.device)
            _linear_workspace[key] = ws
        return ws

    @property
    def weight_bytes(self) -> int:
        return self.qw.numel() * 4 + self.sc.numel() * 2 + self.zp.numel()


class F16Weight:
    """One (possibly fused) DENSE fp16 matrix [N, K] of the un-quantised model, in the form the
    kernels read through quic_w4_t.w16: K contiguous, rows in the order W4Weight gives its
    columns.  The second execution path of the reference (src/model.py:35-41: a linear
    without a packed weight runs kernels/cuda/gemm.cu:36)."""

    def __init__(self, n: int, k: int, device, bias: torch.Tensor | None = None):
        if n % 8 or k % 8:
            raise RuntimeError("F16Weight: N and K must be multiples of 8")
        self.size_n, self.size_k = n, k
        self.w = torch.empty(n, k, dtype=torch.float16, device=device)
        self.bias = bias

    def put(self, weight: torch.Tensor, row_offset: int = 0, row_order: int = ROWS_NATURAL) -> None:
        """Places one checkpoint layer [N_layer, K] at rows [row_offset, row_offset + N_layer)."""
        w = weight.to(self.w.device, torch.float16)
        n, k = w.shape
        if k != self.size_k or row_offset + n > self.size_n:
            raise RuntimeError("F16Weight.put: checkpoint tensor shape does not match")
        if row_order == ROWS_ROPE_PAIRS:  # (0,32,1,33,...) inside every head of 64 rows
            w = w.view(-1, 2, 32, k).transpose(1, 2).reshape(n, k)
        self.w[row_offset:row_offset + n] = w

    def struct(self) -> W4:
        return W4(None, None, None, ptr(self.bias), self.size_n, self.size_k, ptr(self.w))

    def dequant(self) -> torch.Tensor:
        return self.w

    def workspace(self, m: int):
        return None

    @property
    def weight_bytes(self) -> int:
        return self.w.numel() * 2


_linear_workspace: dict = {}
MAX_LINEAR_ROWS = 8192  # rows per launch; longer inputs are processed in chunks to bound scratch memory


def w4a16_linear(w, x: torch.Tensor, use_tensor: bool | None = None) -> torch.Tensor:
    """y = x · dequant(W)^T + bias.  Replaces marlin_linear (src/quant/marlin.py:190); with an
    F16Weight the dense linear of the un-quantised model (_linear, src/model.py:35-41)."""
    _need_cuda(x)
    _need_half(x)
    x2 = x.contiguous().reshape(-1, w.size_k)
    m = x2.shape[0]
    y = torch.empty(m, w.size_n, dtype=torch.float16, device=x.device)
    if use_tensor is None:
        use_tensor = TENSOR_PATH and m >= TENSOR_MIN_ROWS
    s = w.struct()
    for r0 in range(0, m, MAX_LINEAR_ROWS):
        rows = min(MAX_LINEAR_ROWS, m - r0)
        check(lib().quic_w4a16_linear(ptr(x2[r0:r0 + rows]), C.byref(s), ptr(y[r0:r0 + rows]), rows,
                                      int(bool(use_tensor)), ptr(w.workspace(rows)), stream_ptr()), "w4a16_linear")
    return y.reshape(*x.shape[:-1], w.size_n)


# ---------------------------------------------------------------------------------
# Per-op getters with the reference's forward() call shapes
# ---------------------------------------------------------------------------------
def _rmsnorm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float,
                     residual: torch.Tensor | None = None):
    """rmsnorm.forward(x fp16 [...,896], weight fp16 [896], eps) -> fp16 (rmsnorm.cu:100).
    With ``residual`` returns (normed, x + residual)."""
    _need_cuda(x, weight, residual)
    _need_half(x, weight, residual)
    if x.shape[-1] != HIDDEN or weight.numel() != HIDDEN:
        raise RuntimeError("rmsnorm: hidden size must be 896")
    x = x.contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // HIDDEN
    if rows == 0:
        return y if residual is None else (y, torch.empty_like(x))
    total = None
    if residual is not None:
        residual = residual.contiguous()
        total = torch.empty_like(x)
    check(lib().quic_rmsnorm(ptr(x), ptr(residual), ptr(weight.contiguous()), float(eps), ptr(y),
                             ptr(total), rows, stream_ptr()), "rmsnorm")
    return y if residual is None else (y, total)


def _rope_init_table(inv_freq: torch.Tensor, max_seq_len: int):
    """rope.init_table(inv_freq fp32 cuda [32], max_seq_len) -> [cos, sin] fp16 [max,32]
    (rope.cu:125)."""
    _need_cuda(inv_freq)
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != 32:
        raise RuntimeError("rope.init_table: inv_freq must be fp32 with 32 elements")
    cos = torch.empty(max_seq_len, 32, dtype=torch.float16, device=inv_freq.device)
    sin = torch.empty_like(cos)
    check(lib().quic_rope_table_init(ptr(inv_freq.contiguous()), int(max_seq_len), ptr(cos), ptr(sin),
                                     stream_ptr()), "rope_table_init")
    return [cos, sin]


def _rope_forward(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """rope.forward(x fp16 [B,H,S,64] contiguous, cos, sin fp16 [S,32] or [B,S,32]) (rope.cu:85)."""
    _need_cuda(x, cos, sin)
    _need_half(x, cos, sin)
    if x.dim() != 4 or not x.is_contiguous() or x.shape[3] != HEAD_DIM:
        raise RuntimeError("rope: x must be contiguous [B, H, S, 64]")
    b, h, s, _ = x.shape
    if cos.shape != sin.shape or not (cos.is_contiguous() and sin.is_contiguous()):
        raise RuntimeError("rope: cos/sin must be contiguous and of equal shape")
    if cos.dim() == 3:
        if tuple(cos.shape) != (b, s, 32):
            raise RuntimeError("rope: per-row cos/sin must be [B, S, 32]")
        stride = s * 32
    elif cos.dim() == 2 and tuple(cos.shape) == (s, 32):
        stride = 0
    else:
        raise RuntimeError("rope: shared cos/sin must be [S, 32]")
    y = torch.empty_like(x)
    check(lib().quic_rope(ptr(x), ptr(cos), ptr(sin), ptr(y), b, h, s, stride, stream_ptr()), "rope")
    return y


def _swiglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """swiglu.forward(gate, up fp16 [rows,4864]) -> fp16 (swiglu.cu:37)."""
    _need_cuda(gate, up)
    _need_half(gate, up)
    if gate.dim() != 2 or gate.shape[1] != INTER or gate.shape != up.shape:
        raise RuntimeError("swiglu: gate/up must be [rows, 4864] of equal shape")
    gate, up = gate.contiguous(), up.contiguous()
    y = torch.empty_like(gate)
    check(lib().quic_swiglu(ptr(gate), ptr(up), ptr(y), gate.shape[0], stream_ptr()), "swiglu")
    return y


def qkv_rope_append(qkv: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor,
                    sin: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor) -> torch.Tensor:
    """Prefill: rotates and scatters the fused QKV output of ``rows`` tokens.  ``slots`` /
    ``positions`` int32 [rows]; ``kcache`` / ``vcache`` one layer's planes [n_slots, 2, s_max,
    64].  Returns the rotated queries fp16 [14, rows, 64] (the reference's _heads + rope +
    cache update, src/model.py:138-160, in one kernel)."""
    _need_cuda(qkv, slots, positions, cos, sin, kcache, vcache)
    _need_half(qkv, cos, sin, kcache, vcache)
    rows = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != QKV_N or slots.numel() != rows or positions.numel() != rows:
        raise RuntimeError("qkv_rope_append: qkv must be [rows, 1152] with one slot and position per row")
    if slots.dtype != torch.int32 or positions.dtype != torch.int32:
        raise RuntimeError("qkv_rope_append: slots / positions must be int32")
    if not (kcache.is_contiguous() and vcache.is_contiguous()) or kcache.shape[1:] != (KV_HEADS, kcache.shape[2], HEAD_DIM):
        raise RuntimeError("qkv_rope_append: cache planes must be contiguous [n_slots, 2, s_max, 64]")
    q = torch.empty(HEADS, rows, HEAD_DIM, dtype=torch.float16, device=qkv.device)
    check(lib().quic_qkv_rope_append(ptr(qkv.contiguous()), ptr(slots), ptr(positions), ptr(cos), ptr(sin),
                                     cos.shape[0], ptr(q), ptr(kcache), ptr(vcache), kcache.shape[2],
                                     kcache.shape[0], rows, stream_ptr()), "qkv_rope_append")
    return q


def attn_prefill(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, seq_start: torch.Tensor,
                 seq_len: torch.Tensor, seq_slot: torch.Tensor, max_len: int, scale: float = -1.0,
                 seq_off: torch.Tensor | None = None) -> torch.Tensor:
    """Causal prefill attention of several sequences in one launch.  ``q`` fp16 [14, rows, 64]
    (from qkv_rope_append); ``seq_start`` / ``seq_len`` / ``seq_slot`` int32 [n_seq] on the
    device; keys and values are read from the slots.  Returns fp16 [rows, 896]."""
    _need_cuda(q, kcache, vcache, seq_start, seq_len, seq_slot)
    _need_half(q, kcache, vcache)
    if q.dim() != 3 or q.shape[0] != HEADS or q.shape[2] != HEAD_DIM or not q.is_contiguous():
        raise RuntimeError("attn_prefill: q must be contiguous [14, rows, 64]")
    if any(t.dtype != torch.int32 for t in (seq_start, seq_len, seq_slot)):
        raise RuntimeError("attn_prefill: sequence tables must be int32")
    rows, n_seq = q.shape[1], seq_len.numel()
    out = torch.empty(rows, HEADS * HEAD_DIM, dtype=torch.float16, device=q.device)
    if seq_off is not None and (seq_off.dtype != torch.int32 or seq_off.numel() != n_seq or not seq_off.is_cuda):
        raise RuntimeError("attn_prefill: seq_off must be a CUDA int32 tensor with one entry per sequence")
    check(lib().quic_attn_prefill(ptr(q), ptr(kcache), ptr(vcache), ptr(seq_start), ptr(seq_len), ptr(seq_slot),
                                  ptr(seq_off), n_seq, int(max_len), rows, kcache.shape[2], kcache.shape[0], float(scale), ptr(out),
                                  stream_ptr()),
          "attn_prefill")
    return out


def _flash_attn_prefill_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = True,
                                softmax_scale: float = -1.0, pad_lens: torch.Tensor | None = None) -> torch.Tensor:
    """flash_attn_prefill.forward(Q fp16 [B,14,N,64], K, V fp16 [B,14 or 2,N,64], is_causal,
    softmax_scale, pad_lens int32 [B] or None) -> fp16 [B,14,N,64]: the reference's prefill
    attention call (kernels/cuda/flash_attn_prefill.cu:520, kernels/flash_attn_prefill_pytorch.py:10)
    on left-padded batches.  The rows are repacked without their padding, run through
    ``attn_prefill`` in one launch and scattered back; rows inside the padding come back as zeros
    (the reference lets them attend to themselves; nothing reads them)."""
    _need_cuda(q, k, v, pad_lens)
    _need_half(q, k, v)
    if not is_causal:
        raise RuntimeError("flash_attn_prefill: only the causal form is built")
    b, nh, n, d = q.shape
    if nh != HEADS or d != HEAD_DIM or k.shape != v.shape or k.shape[0] != b or k.shape[2] != n or \
            k.shape[1] not in (HEADS, KV_HEADS):
        raise RuntimeError("flash_attn_prefill: expected Q [B,14,N,64] and K, V [B,14|2,N,64]")
    if k.shape[1] == HEADS:  # repeat_kv layout: query head h reads kv head h // 7
        k, v = k[:, :: HEADS // KV_HEADS], v[:, :: HEADS // KV_HEADS]
    pads = [0] * b if pad_lens is None else [int(p) for p in pad_lens.tolist()]
    lens = [n - p for p in pads]
    if any(l < 0 for l in lens):
        raise RuntimeError("flash_attn_prefill: a pad length exceeds the sequence length")
    dev = q.device
    pos = torch.arange(n, device=dev)
    pad_t = torch.tensor(pads, device=dev)
    keep = pos[None, :] >= pad_t[:, None]                                    # [B, N] real tokens
    src = torch.clamp(pos[None, :] + pad_t[:, None], max=n - 1)              # token t of the sequence sits at pad + t
    idx = src[:, None, :, None].expand(b, KV_HEADS, n, d)
    kc, vc = k.gather(2, idx).contiguous(), v.gather(2, idx).contiguous()    # [B, 2, N, 64], sequences at position 0
    q_rows = q.permute(1, 0, 2, 3)[:, keep].contiguous()                     # [14, rows, 64]
    starts, total = [], 0
    for l in lens:
        starts.append(total)
        total += l
    live = [i for i, l in enumerate(lens) if l > 0]
    out = torch.zeros(b, nh, n, d, dtype=torch.float16, device=dev)
    if not live:
        return out
    table = torch.tensor([[starts[i] for i in live], [lens[i] for i in live], live], dtype=torch.int32, device=dev)
    rows = attn_prefill(q_rows, kc, vc, table[0], table[1], table[2], max(lens), float(softmax_scale))
    out.permute(0, 2, 1, 3)[keep] = rows.view(total, nh, d)
    return out


def swiglu_fused(gu: torch.Tensor) -> torch.Tensor:
    """silu(gu[:, :4864]) * gu[:, 4864:] on the fused gate|up linear output, fp16 [rows, 9728]
    -> fp16 [rows, 4864] (the reference's _MLP, src/model.py:96-105, without slicing copies)."""
    _need_cuda(gu)
    _need_half(gu)
    if gu.dim() != 2 or gu.shape[1] != 2 * INTER:
        raise RuntimeError("swiglu_fused: expected [rows, 9728]")
    gu = gu.contiguous()
    y = torch.empty(gu.shape[0], INTER, dtype=torch.float16, device=gu.device)
    if gu.shape[0]:
        check(lib().quic_swiglu_fused(ptr(gu), ptr(y), gu.shape[0], stream_ptr()), "swiglu_fused")
    return y


def _sampler_forward(logits: torch.Tensor) -> torch.Tensor:
    """sampler.forward(logits fp16 [B,1,V]) -> int64 [B,1] (sampler.cu:52)."""
    _need_cuda(logits)
    _need_half(logits)
    if logits.dim() != 3 or logits.shape[1] != 1:
        raise RuntimeError("sampler: expected [B,1,V]")
    logits = logits.contiguous()
    b, _, v = logits.shape
    out = torch.empty(b, 1, dtype=torch.int64, device=logits.device)
    check(lib().quic_argmax(ptr(logits), b, v, ptr(out), stream_ptr()), "argmax")
    return out


def _gemm_forward(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """gemm.forward(x fp16 [...,K], w fp16 [N,K], bias fp16 [N] or None) -> [...,N] (gemm.cu:36)."""
    _need_cuda(x, w, bias)
    _need_half(x, w, bias)
    k = x.shape[-1]
    n = w.shape[0]
    if w.dim() != 2 or w.shape[1] != k:
        raise RuntimeError("gemm: weight must be [N, K]")
    x2 = x.contiguous().reshape(-1, k)
    y = torch.empty(x2.shape[0], n, dtype=torch.float16, device=x.device)
    check(lib().quic_gemm_f16(ptr(x2), ptr(w.contiguous()), ptr(bias), ptr(y), x2.shape[0], n, k,
                              stream_ptr()), "gemm_f16")
    return y.reshape(*x.shape[:-1], n)


_attn_scratch: dict = {}
_lm_scratch: dict = {}


def lm_head_argmax(x: torch.Tensor, embed: torch.Tensor, norm_weight: torch.Tensor | None = None,
                   eps: float = 1e-6, want_logits: bool = False):
    """Final norm (optional) + tied lm_head + greedy argmax in one kernel.
    x fp16 [B, 896] -> (tokens int64 [B], logits fp16 [B, V] or None)."""
    _need_cuda(x, embed, norm_weight)
    _need_half(x, embed, norm_weight)
    x = x.contiguous().view(-1, HIDDEN)
    b, vocab = x.shape[0], embed.shape[0]
    need = lib().quic_lm_head_scratch_bytes(b, vocab)
    key = (x.device.index, torch.cuda.current_stream().cuda_stream)
    scratch = _lm_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        scratch = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=x.device)
        _lm_scratch[key] = scratch
    out = torch.empty(b, dtype=torch.int64, device=x.device)
    logits = torch.empty(b, vocab, dtype=torch.float16, device=x.device) if want_logits else None
    check(lib().quic_lm_head_argmax(ptr(x), ptr(norm_weight), float(eps), ptr(embed), vocab, b,
                                    ptr(logits), ptr(out), ptr(scratch), stream_ptr()), "lm_head_argmax")
    return out, logits


def _flash_attn_decode_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                               softmax_scale: float = -1.0, pad_lens: torch.Tensor | None = None,
                               splits: int = 0, cta_merge: bool = False) -> torch.Tensor:
    """flash_attn_decode.forward(Q fp16 [B,nh,1,64], K, V fp16 [B,n_kv,S,64], softmax_scale,
    pad_lens int32 [B] or None) -> fp16 [B,nh,1,64] (flash_attn_decode.cu:133-198)."""
    _need_cuda(q, k, v, pad_lens)
    _need_half(q, k, v)
    if q.dim() != 4 or q.shape[2] != 1 or q.shape[3] != HEAD_DIM:
        raise RuntimeError("flash_attn_decode: Q must be [B, nh, 1, 64]")
    b, nh = q.shape[0], q.shape[1]
    if nh != HEADS or k.shape[1] != KV_HEADS:
        raise RuntimeError("flash_attn_decode: built for 14 query heads / 2 KV heads")
    if k.shape[0] != b or v.shape != k.shape or k.shape[3] != HEAD_DIM:
        raise RuntimeError("flash_attn_decode: K/V shape mismatch")
    s = k.shape[2]
    if pad_lens is not None and not (pad_lens.dtype == torch.int32 and pad_lens.dim() == 1 and
                                     pad_lens.shape[0] == b and pad_lens.is_contiguous()):
        raise RuntimeError("flash_attn_decode: pad_lens must be a contiguous CUDA int32 tensor of shape [B]")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty(b, nh, 1, HEAD_DIM, dtype=torch.float16, device=q.device)
    if s == 0:
        return out.zero_()
    scale = float(softmax_scale) if softmax_scale and softmax_scale > 0 else HEAD_DIM ** -0.5
    if cta_merge:  # CTAs of 512 tokens merged through (distributed) shared memory: no scratch
        check(lib().quic_attn_decode_cta(ptr(q), ptr(k), ptr(v), KV_HEADS * s * HEAD_DIM, s * HEAD_DIM,
                                         ptr(pad_lens), None, s, scale, ptr(out), b, stream_ptr()),
              "attn_decode_cta")
        return out
    asked = splits
    if splits <= 0:  # the library chooses (the same count, or its streamed kernel, which needs no scratch)
        splits = lib().quic_attn_pick_splits(b, s)
    scratch = None
    if splits > 1:
        need = lib().quic_attn_scratch_bytes(b, splits)
        key = (q.device.index, torch.cuda.current_stream().cuda_stream)
        scratch = _attn_scratch.get(key)
        if scratch is None or scratch.numel() < need:
            scratch = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=q.device)
            _attn_scratch[key] = scratch
    check(lib().quic_attn_decode(ptr(q), ptr(k), ptr(v), KV_HEADS * s * HEAD_DIM, s * HEAD_DIM,
                                 ptr(pad_lens), None, s, scale, ptr(out), b, splits if asked > 0 else 0, ptr(scratch),
                                 stream_ptr()), "attn_decode")
    return out


@functools.cache
def rmsnorm():
    lib()
    return SimpleNamespace(forward=_rmsnorm_forward)


@functools.cache
def rope():
    lib()
    return SimpleNamespace(forward=_rope_forward, init_table=_rope_init_table)


@functools.cache
def swiglu():
    lib()
    return SimpleNamespace(forward=_swiglu_forward)


@functools.cache
def sampler():
    lib()
    return SimpleNamespace(forward=_sampler_forward)


@functools.cache
def gemm():
    lib()
    return SimpleNamespace(forward=_gemm_forward)


@functools.cache
def flash_attn_decode():
    lib()
    return SimpleNamespace(forward=_flash_attn_decode_forward)


@functools.cache
def flash_attn_prefill():
    """Same getter as the reference's (kernels/__init__.py:76-85)."""
    lib()
    return SimpleNamespace(forward=_flash_attn_prefill_forward)


@functools.cache
def w4a16():
    """Replaces the reference's ``marlin()`` getter: ``forward(weight, x)``."""
    lib()
    return SimpleNamespace(forward=w4a16_linear)
