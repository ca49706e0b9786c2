"""Python side of the CUDA kernel library: one thin function per launcher.

The role of ``engine/ops_cuda.py`` + ``kernels/bindings.cpp`` in
davidjoyme/flashdecode-cuda (bindings.cpp:24-63,79-164), without an op
registry or an alternative backend: these functions are the only
implementation, they check what the kernels assume (device, dtype,
contiguity) and raise with the kernel library's own message when a launcher
refuses a size.  There is no CPU path; importing this module on a machine
without the built library builds it, and calling any function without a CUDA
device fails.

Tensors are passed as raw pointers on torch's current stream, so launches are
ordered with torch's own work and can be captured into a CUDA graph.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

STATUS_BAD_TOKEN = 1
STATUS_BAD_BLOCK = 2
STATUS_BAD_POSITION = 4
STATUS_WAIT_TIMEOUT = 8
_STATUS_TEXT = {
    STATUS_BAD_TOKEN: "a token id lies outside the embedding table",
    STATUS_BAD_BLOCK: "a cached token maps to no allocated block",
    STATUS_BAD_POSITION: "a position lies beyond the rotation table",
    STATUS_WAIT_TIMEOUT: "a bounded wait inside a kernel ran out",
}

_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A launcher refused its arguments or a launch failed."""


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t}")


def lib() -> ctypes.CDLL:
    """The loaded kernel library; built on first use if it is missing or stale."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover - environment failure
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from e
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    L.fd_last_error.restype = ctypes.c_char_p
    L.fd_last_error.argtypes = []
    sigs = {
        "fd_device_arch": [],
        "fd_set_pdl": [I],
        "fd_sm_count": [],
        "fd_embed": [P, P, I, P, I, I, I, I, F, P, P],
        "fd_add_rmsnorm": [P, I, I, LL, P, I, P, I, F, P, I, P, I, I, F, P],
        "fd_silu_mul": [P, P, I, I, I, I, P],
        "fd_rope_append": [P, I, I, LL, P, I, P, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
        "fd_gemv_qkv_rope": [P, P, P, I, P, I, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P, c_ulonglong, P],
        "fd_gemm_tc_supported": [I, I, I],
        "fd_gemm_tc_set_wide": [I],
        "fd_attn_prefill_set_form": [I],
        "fd_attn_decode_set_form": [I],
        "fd_gemm_tc": [P, P, P, I, P, I, I, I, I, P, P],
        "fd_gemm_tc_qkv_rope": [P, P, P, I, P, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
        "fd_gemm_stream_splits": [I, I, I],
        "fd_gemm_stream_force_2d": [I],
        "fd_gemm_stream_set_pdl": [I],
        "fd_gemm_stream_last_map3d": [],
        "fd_gemm_stream": [P, P, P, I, P, I, I, I, I, I, P, P],
        "fd_gemm_stream_qkv_rope": [P, P, P, I, P, I, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
        "fd_tc_test_hook": [LL, I],
        "fd_gemv_splits": [I, I, I, I, I],
        "fd_gemv": [P, P, P, I, P, I, I, I, I, I, P, c_ulonglong, P],
        "fd_gemm_simt": [P, P, P, P, I, I, I, I, I, I, P],
        "fd_attn_simt_qt": [I],
        "fd_attn_decode_group": [I, I, I],
        "fd_attention_simt": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, I, I, P, P, P],
        "fd_attention": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, I, I, P, P, P, P, c_ulonglong, P],
        "fd_attention_mma_sync": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, I, I, P, P, P, P],
        "fd_conv_rope_append": [P, I, I, P, P, P, P, P, I, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, I, P, P, F, I, I, P],
        "fd_attention_ext": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, I, I, P, P, F, I, P, I, I, I, P, P],
        "fd_attn_head_mix": [P, P, P, I, I, I, I, I, I, F, P],
        "fd_add_dyn_tanh": [P, I, P, I, P, P, F, P, I, P, I, I, P],
        "fd_quad_exp_act": [P, P, I, P, LL, P],
        "fd_scale_f32": [P, LL, F, P],
        "fd_axpy_f32": [P, P, I, LL, F, I, P],
        "fd_linear_scan": [P, I, I, I, I, I, P, P, I, P, P, P, P, I, I, F, P, P, P, P, I, I, I, I, I, P, I, I, P, LL, P, I, F, F, P],
        "fd_head_norm_gate": [P, P, P, I, P, I, I, I, I, I, F, F, P],
        "fd_low_rank_expand": [P, I, P, P, P, I, I, I, I, P],
        "fd_conv_state_update": [P, I, I, P, P, P, P, I, I, I, P],
        "fd_gate_mul": [P, P, I, P, I, I, I, P],
        "fd_add_concat": [P, I, P, P, P, I, I, I, P],
        "fd_relu2": [P, P, I, LL, P],
        "fd_moe_tile_rows": [I, I],
        "fd_moe_route": [P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
        "fd_glu_mul": [P, P, I, I, I, I, I, F, P],
        "fd_softcap": [P, LL, F, P],
        "fd_lanes_norm": [P, I, I, LL, P, P, P, P, I, P, P, F, P, I, P, I, I, I, P],
        "fd_lanes_fill": [P, P, I, I, I, P],
        "fd_lanes_sum": [P, I, P, P, P, P, P, I, I, I, P],
        "fd_norm_append": [P, I, P, I, P, P, F, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, I, I, P, P],
        "fd_head_gemm": [P, P, P, I, I, I, I, I, P],
        "fd_moe_align": [P, I, I, P, P, P, P, I, I, P],
        "fd_moe_gemm": [P, P, P, I, I, P, P, P, I, I, I, I, I, F, I, P],
        "fd_add_cast": [P, I, P, P, I, I, I, F, P],
        "fd_side_gate_mul": [P, P, P, I, I, I, P, I, I, I, P, P],
        "fd_token_side_row": [P, I, P, F, P, P, I, I, I, P, P, P, I, F, P, P, I, I, I, I, P, P],
        "fd_add_row_vector": [P, I, P, P, I, I, F, P],
        "fd_moe_combine": [P, P, P, P, P, P, P, I, I, I, I, I, P],
        "fd_moe_gather": [P, P, P, P, I, I, I, I, P],
        "fd_gemm_tc_grouped": [P, P, P, I, I, I, I, I, P, P, F, P, P],
        "fd_sample": [P, I, I, P, P, P, c_ulonglong, P, P, P, P],
        "fd_copy_h2d_async": [P, P, LL, P],
        "fd_copy_d2h_sync": [P, P, LL, P],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = I
    L.fd_attn_scratch_floats.argtypes = [I, I, I, I]
    L.fd_launch_count.restype = c_ulonglong
    L.fd_launch_count.argtypes = []
    L.fd_attn_scratch_floats.restype = LL
    L.fd_linear_scan_segment.argtypes = []
    L.fd_linear_scan_segment.restype = I
    L.fd_linear_scan_scratch_floats.argtypes = [I, I, I, I, I]
    L.fd_linear_scan_scratch_floats.restype = LL
    L.fd_sample_scratch_words.argtypes = [I, I]
    L.fd_sample_scratch_words.restype = LL


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def launch_count() -> int:
    """Kernels of this library launched so far by this process, counted where they are launched (a kernel
    captured into a graph counts once, at capture)."""
    return int(lib().fd_launch_count())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  torch's own accessor for the raw handle costs a fraction of a microsecond;
    ``torch.cuda.current_stream()`` builds a Stream object each time (about 5 us), which in a prompt step of some
    250 launches was a sixth of the host's time."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return t.data_ptr()


def require_device() -> None:
    """Fail loudly unless a CUDA device of compute capability 10.x is current."""
    if not torch.cuda.is_available():
        raise KernelError("flashdecode_cuda_b200 needs a CUDA device (B200, sm_100a); none is available "
                          "and there is no CPU fallback")
    arch = lib().fd_device_arch()
    if arch < 0:
        _check(arch)
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a only; this device is sm_{arch}")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for this library's kernels: a kernel may start, and fetch
    weights, while the previous one is still finishing.  Off by default: measured on B200 inside
    the captured decode graph every programmatic edge made the step slower (all kernels: 2.34
    against 1.46 ms at batch 8; a single kind of product per layer: 1.50 to 1.62 ms)."""
    lib().fd_set_pdl(int(on))


def copy_h2d_async(dst: torch.Tensor, src_pinned: torch.Tensor, n_elements: int) -> None:
    """dst[:n] <- src[:n] from pinned host memory, asynchronously on the current stream."""
    rc = lib().fd_copy_h2d_async(dst.data_ptr(), src_pinned.data_ptr(), n_elements * dst.element_size(), _stream())
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def copy_d2h_sync(dst_pinned: torch.Tensor, src: torch.Tensor, n_elements: int) -> None:
    """dst[:n] <- src[:n] into pinned host memory on the current stream, waited for."""
    rc = lib().fd_copy_d2h_sync(dst_pinned.data_ptr(), src.data_ptr(), n_elements * src.element_size(), _stream())
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def sm_count() -> int:
    return lib().fd_sm_count()


def status_message(word: int) -> str:
    return "; ".join(text for bit, text in _STATUS_TEXT.items() if word & bit) or "ok"


# ---------------------------------------------------------------------------

def embed(tokens: torch.Tensor, table: torch.Tensor, resid: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """resid[t] = float(table[tokens[t]]) * scale; tokens int32 [T], resid float32 [T, H] - or [T, lanes * H], a
    residual stream of several lanes, every one of which receives the row."""
    T = tokens.numel()
    V, H = table.shape
    assert tokens.dtype == torch.int32 and resid.dtype == torch.float32 and resid.shape[-1] % H == 0
    _check(lib().fd_embed(_ptr(tokens), _ptr(table), _dt(table.dtype), _ptr(resid), T, H, V, resid.shape[-1] // H,
                          float(scale), _ptr(status), _stream()))


def add_rmsnorm(delta: Optional[torch.Tensor], resid: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                write_resid: bool = True, n_parts: int = 1, delta_scale: float = 1.0) -> None:
    """out[j] = rmsnorm(resid[r] + delta_scale * delta[r]) * weight with r = rows[j] (or j);
    resid[r] takes the sum when ``write_resid``.  ``delta`` None: plain norm.
    ``delta`` [parts, rows, H] (or ``n_parts`` > 1) holds partial sums, added in order."""
    H = resid.shape[-1]
    if delta is not None and delta.dim() == 3:
        n_parts = delta.shape[0]
    if n_out is None:
        n_out = rows.numel() if rows is not None else resid.numel() // H
    assert resid.dtype == torch.float32 and out.shape[-1] == H and weight.numel() == H
    part_stride = 0
    if delta is not None and n_parts > 1:
        part_stride = delta.numel() // n_parts
    _check(lib().fd_add_rmsnorm(_ptr(delta), _dt(delta.dtype) if delta is not None else _dt(out.dtype),
                                n_parts, part_stride, _ptr(resid), int(write_resid), _ptr(weight),
                                _dt(weight.dtype), float(eps), _ptr(out), _dt(out.dtype), _ptr(rows),
                                n_out, H, float(delta_scale), _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, tiled: bool = False) -> None:
    """out[m, i] = silu(gate_i) * up_i.  ``gate_up`` [M, 2I] is [gate | up], or
    with ``tiled`` tiles of 16 columns: 8 gate values then the 8 up values."""
    M, I2 = gate_up.shape
    assert out.shape == (M, I2 // 2) and out.dtype == gate_up.dtype
    _check(lib().fd_silu_mul(_ptr(gate_up), _ptr(out), _dt(out.dtype), M, I2 // 2, int(tiled), _stream()))


GLU_SILU, GLU_GELU_TANH, GLU_CLAMPED = 0, 1, 2
GLU_KINDS = {"silu": GLU_SILU, "gelu_tanh": GLU_GELU_TANH, "clamped_swish": GLU_CLAMPED}


def glu_mul(gate_up: torch.Tensor, out: torch.Tensor, kind: int, limit: float = 0.0, tiled: bool = False) -> None:
    """out[m, i] = act(gate_i, up_i) with ``gate_up`` [M, 2I] = [gate | up] (or tiles of 8 + 8 columns).  ``kind``:
    GLU_SILU g sigmoid(g) u; GLU_GELU_TANH the tanh form of GELU of g, times u; GLU_CLAMPED g' sigmoid(1.702 g') (u' + 1)
    with g' = min(g, limit) and u' = clamp(u, -limit, limit).  Float arithmetic, one rounding."""
    M, I2 = gate_up.shape
    assert out.shape == (M, I2 // 2) and out.dtype == gate_up.dtype
    _check(lib().fd_glu_mul(_ptr(gate_up), _ptr(out), _dt(out.dtype), M, I2 // 2, int(tiled), int(kind), float(limit),
                            _stream()))


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place; x float32."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().fd_softcap(_ptr(x), x.numel(), float(cap), _stream()))


def lanes_norm(y: Optional[torch.Tensor], gain: Optional[torch.Tensor], mix: Optional[torch.Tensor],
               back: Optional[torch.Tensor], lanes: torch.Tensor, read: Optional[torch.Tensor], weight: torch.Tensor,
               eps: float, out: torch.Tensor, n_lanes: int, rows: Optional[torch.Tensor] = None,
               n_out: Optional[int] = None, write_lanes: bool = True) -> None:
    """The step between two sub-layers on a residual stream of ``n_lanes`` lanes, ``lanes`` [T, n_lanes * H] float32:
    first the pending update X'[t] = sum_s mix[s, t] X[s] + back[t] * gain * y (``y`` [T, H], or float partial sums
    [parts, T, H]; None: nothing pending), written back when ``write_lanes``; then out[j] = rmsnorm(sum_s read[s]
    X'[s]) * weight for row j (or rows[j]).  gain [H], mix [S, S], back [S], read [S]: float32 or None (ones, the unit
    matrix)."""
    H = weight.numel()
    assert lanes.dtype == torch.float32 and lanes.shape[-1] == n_lanes * H and out.shape[-1] == H
    for t in (gain, mix, back, read, weight):
        assert t is None or t.dtype == torch.float32
    n_parts, part_stride = 1, 0
    if y is not None and y.dim() == 3:
        n_parts, part_stride = y.shape[0], y.shape[1] * y.shape[2]
    if n_out is None:
        n_out = rows.numel() if rows is not None else lanes.shape[0]
    _check(lib().fd_lanes_norm(_ptr(y), _dt(y.dtype) if y is not None else _dt(out.dtype), n_parts, part_stride,
                               _ptr(gain), _ptr(mix), _ptr(back), _ptr(lanes), int(write_lanes), _ptr(read), _ptr(weight),
                               float(eps), _ptr(out), _dt(out.dtype), _ptr(rows), n_out, H, n_lanes, _stream()))


def lanes_fill(src: torch.Tensor, lanes: torch.Tensor, n_lanes: int) -> None:
    """Every lane of ``lanes`` [T, n_lanes * H] <- ``src`` [T, H]; float32."""
    T, H = src.shape
    assert src.dtype == lanes.dtype == torch.float32 and lanes.shape == (T, n_lanes * H)
    _check(lib().fd_lanes_fill(_ptr(src), _ptr(lanes), T, H, n_lanes, _stream()))


def lanes_sum(y: Optional[torch.Tensor], gain: Optional[torch.Tensor], mix: Optional[torch.Tensor],
              back: Optional[torch.Tensor], lanes: torch.Tensor, out: torch.Tensor, n_lanes: int) -> None:
    """out [T, H] float32 = the lanes added up, after the pending update (as in ``lanes_norm``) if ``y`` is given."""
    T, H = out.shape
    assert lanes.dtype == out.dtype == torch.float32 and lanes.shape == (T, n_lanes * H)
    assert y is None or y.shape == (T, H)
    _check(lib().fd_lanes_sum(_ptr(y), _dt(y.dtype) if y is not None else 0, _ptr(gain), _ptr(mix), _ptr(back),
                              _ptr(lanes), _ptr(out), T, H, n_lanes, _stream()))


def norm_append(proj: torch.Tensor, q_out: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                k_weight: Optional[torch.Tensor], eps: float, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: Optional[torch.Tensor], block_table: torch.Tensor,
                n_kv: int, write_kv: bool, status: torch.Tensor, k_rows: Optional[torch.Tensor] = None,
                q_count: int = 0, k_count: int = 0) -> None:
    """``proj`` [T, >= nq + nk + nv] = [q | k | v]: q (normed over all its nq columns with ``q_weight``, or as it is) to
    ``q_out`` [T, nq]; k (normed over all its nk columns with ``k_weight``, or as it is) and v to the pools at each
    token's position.  ``v_pool`` None: nothing but the keys is kept.  ``q_out`` None: the rows hold no q.  ``k_rows``
    [T, nk]: receives the (normed) k once more as plain rows.  ``q_count`` / ``k_count``: how many of q's and k's
    columns are real where heads are zero-padded to multiples of 8 (the norms' means run over these; 0: all).  Norm
    weights float32."""
    T, ld = proj.shape
    nq = 0 if q_out is None else q_out.shape[1]
    num_blocks, kvh, block_size, d = k_pool.shape
    nk = n_kv * d
    nv = 0 if v_pool is None else n_kv * v_pool.shape[-1]
    assert kvh == n_kv and proj.dtype == k_pool.dtype and proj.is_contiguous() and (q_out is None or q_out.dtype == proj.dtype)
    assert k_rows is None or (k_rows.shape == (T, nk) and k_rows.dtype == proj.dtype and k_rows.is_contiguous())
    assert q_weight is None or (q_weight.dtype == torch.float32 and q_weight.numel() == nq)
    assert k_weight is None or (k_weight.dtype == torch.float32 and k_weight.numel() == nk)
    _check(lib().fd_norm_append(_ptr(proj), ld, _ptr(q_out), _dt(proj.dtype), _ptr(q_weight), _ptr(k_weight), float(eps),
                                _ptr(tok_row), _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool),
                                _ptr(block_table), block_table.shape[1], num_blocks, block_size, T, nq, nk, nv, n_kv,
                                int(write_kv), _ptr(k_rows), int(q_count), int(k_count), _ptr(status), _stream()))


HEAD_GEMM_LIBRARY_ROWS = 64      # from this many rows on, the per-head products of bfloat16 steps go to the library's batched product


def head_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h, :] = w[h] a[t, h, :]: a [T, heads * K], w [heads, N, K], out [T, heads * N]; float accumulation.
    float32: the library's own CUDA-core kernel with k ascending (no bit of a row depends on the step's other rows);
    bfloat16: a warp per output column for steps of up to 16 rows, cuBLAS's strided batched product for prompts."""
    heads, N, Kd = w.shape
    T = a.shape[0]
    assert a.shape == (T, heads * Kd) and out.shape == (T, heads * N) and a.dtype == w.dtype == out.dtype
    assert a.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    if a.dtype == torch.bfloat16 and T >= HEAD_GEMM_LIBRARY_ROWS:
        torch.bmm(a.view(T, heads, Kd).transpose(0, 1), w.transpose(1, 2), out=out.view(T, heads, N).transpose(0, 1))
        return
    _check(lib().fd_head_gemm(_ptr(a), _ptr(w), _ptr(out), _dt(a.dtype), T, heads, N, Kd, _stream()))


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                tok_row: torch.Tensor, tok_pos: torch.Tensor, row_slot: torch.Tensor,
                k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor,
                bias: Optional[torch.Tensor] = None, paired: bool = False) -> None:
    """Rotate q and k of every token at its position; append k and v to the
    paged pools [num_blocks, n_kv, block_size, d] (unless ``write_kv`` is off).
    ``qkv`` is [T, (n_q + 2 n_kv) d], or [parts, T, ...] float32 partial sums of
    a split-K product that are added up here, with ``bias`` added on top.
    ``paired``: the columns of each q and k head come in tiles of 8 dims + their
    8 rotation partners (the order ``gemv_qkv_rope`` wants the rows of W in)."""
    n_parts = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.shape[-1] == (n_q + 2 * n_kv) * head_dim and q_out.shape == (T, n_q * head_dim)
    assert cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2
    assert k_pool.dtype == q_out.dtype and (n_parts == 1 or qkv.dtype == torch.float32)
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_rope_append(_ptr(qkv), _dt(qkv.dtype), n_parts, qkv.numel() // n_parts, _ptr(bias),
                                _dt(bias.dtype) if bias is not None else 0, _ptr(q_out), _dt(q_out.dtype),
                                _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row), _ptr(tok_pos), _ptr(row_slot),
                                _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], num_blocks,
                                block_size, T, n_q, n_kv, head_dim, int(write_kv), int(paired), _ptr(status),
                                _stream()))


def gemv_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                  row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                  n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor, n_splits: int = 1,
                  prefetch: Optional[torch.Tensor] = None) -> None:
    """The q/k/v projection of a decode step (M <= 64 rows, bfloat16) with bias,
    rotary encoding and the append to the paged cache in its epilogue.  ``w``
    and ``bias`` are in the paired row order (see ``rope_append``).  ``prefetch``: a
    tensor that a later kernel streams (the output projection's weights); the kernel
    asks L2 for it once its own loads are through."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemv_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                  _ptr(q_out), M, K, n_splits, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                  _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                  block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim, int(write_kv),
                                  _ptr(status), *_prefetch_args(prefetch, 1 << 62), _stream()))


GEMV_PARTIAL, GEMV_BF16, GEMV_F32, GEMV_GATED = 0, 1, 2, 3
GEMV_GATED_GELU = 6      # gated with the tanh form of GELU instead of SiLU; both take a bias on gate and up


def gemm_tc_set_wide(on) -> None:
    """Which tiling ``gemm_tc`` and ``gemm_tc_qkv_rope`` use from now on where N >= 256: 2 = two SMs per
    256 x 256 tile (``tcgen05.mma.cta_group::2``), 1 / True = one persistent CTA per SM with 128 x 256
    tiles, or with 128 x 128 tiles where those number no more than the SMs, 3 = 128 x 256 tiles
    always, 0 / False = 128 x 128 tiles, one per CTA, everywhere.  For tests and measurements."""
    lib().fd_gemm_tc_set_wide(int(on))


def attn_prefill_set_form(form: int) -> None:
    """Which form the tcgen05 prompt attention takes from now on: 1 = a CTA takes 256 queries as two query
    tiles that share every key tile; 2 = a CTA takes 128 queries and deals their key tiles to its two groups
    of softmax warps, which add up their results at the end (half the chain of key tiles per query tile:
    for prompts too short to fill the GPU); 0 = the launcher chooses by the number of CTAs.  For tests and
    measurements."""
    lib().fd_attn_prefill_set_form(int(form))


def attn_decode_set_form(form: int) -> None:
    """Which form the tensor-core decode attention takes from now on: 0 = the launcher chooses (keys as
    the rows of the MMAs for groups of up to 8 query heads, CTAs of eight warps where all of them fit the
    GPU at one per SM); bit 0: the heads as rows always; bit 1: four warps always; bit 2: eight warps
    always.  For tests and measurements."""
    lib().fd_attn_decode_set_form(int(form))


def gemm_tc_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                     cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                     row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                     n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor) -> None:
    """The q/k/v projection of a prompt step on the tcgen05 tensor cores with
    bias, rotary encoding and the append to the paged cache in its epilogue.
    ``w`` and ``bias`` in the paired row order (see ``rope_append``)."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemm_tc_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                     _ptr(q_out), M, K, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                     _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                     block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim,
                                     int(write_kv), _ptr(status), _stream()))


def gemm_tc_supported(M: int, N: int, K: int) -> bool:
    return bool(lib().fd_gemm_tc_supported(M, N, K))


GEMM_RELU2 = 5


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, gated: bool = False,
            status: Optional[torch.Tensor] = None, relu2: bool = False) -> None:
    """out = x w^T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulator in
    tensor memory); bfloat16 operands, ``out`` bfloat16 or float32 [M, N], or
    with ``gated`` (w rows in tiles of 8 gate + 8 up) bfloat16 [M, N / 2] =
    silu(gate) * up, or with ``relu2`` bfloat16 [M, N] = max(x w^T, 0)^2.  Any M and N; K a multiple of 8."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
        mode = GEMV_GATED_GELU if gated == "gelu_tanh" else GEMV_GATED
    elif relu2:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N)
        mode = GEMM_RELU2
    else:
        assert out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
        mode = GEMV_BF16 if out.dtype == torch.bfloat16 else GEMV_F32
    _check(lib().fd_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                            _ptr(out), mode, M, N, K, _ptr(status), _stream()))


def gemm_stream_splits(M: int, N: int, K: int) -> int:
    """CTAs per cluster (splits of K) the streaming tcgen05 product would use; 0 if it does not take
    the sizes (more than 128 rows of x, K not a multiple of 8)."""
    return int(lib().fd_gemm_stream_splits(M, N, K))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, gated: bool = False,
                splits: int = 0, status: Optional[torch.Tensor] = None) -> None:
    """Weight-streaming product for up to 128 rows of x on the tcgen05 tensor cores (W tiles as the
    M side, the rows of x as the N side, K split over a thread-block cluster for narrow W):
    out = x w^T (+ bias), bfloat16 or float32 [M, N], or with ``gated`` (w rows in tiles of 8 gate +
    8 up) bfloat16 [M, N / 2] = silu(gate) * up.  ``splits`` 0: chosen by the launcher."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
        mode = GEMV_GATED_GELU if gated == "gelu_tanh" else GEMV_GATED
    else:
        assert out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
        mode = GEMV_BF16 if out.dtype == torch.bfloat16 else GEMV_F32
    _check(lib().fd_gemm_stream(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                _ptr(out), mode, M, N, K, splits, _ptr(status), _stream()))


def gemm_stream_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                         cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                         row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                         n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor,
                         splits: int = 0) -> None:
    """The q/k/v projection of a step of up to 128 tokens on the streaming tcgen05 product, with bias,
    rotary encoding and the append to the paged cache in its epilogue.  ``w`` and ``bias`` in the
    paired row order (see ``rope_append``)."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemm_stream_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                         _ptr(q_out), M, K, splits, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                         _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                         block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim,
                                         int(write_kv), _ptr(status), _stream()))


def gemm_stream_set_pdl(on: bool) -> None:
    """Whether the streaming product is launched with the programmatic-dependent-launch attribute (the
    default): it may then start and fetch its first weights while the kernel before it in the stream
    still runs, and waits for that kernel before it reads x or writes anything."""
    lib().fd_gemm_stream_set_pdl(int(on))


def gemm_stream_force_2d(on: bool) -> None:
    """Tests: make the streaming product read its operands through two-dimensional tensor maps (one copy per
    k-block) even where K is a multiple of 64 and one three-dimensional copy per stage would do."""
    lib().fd_gemm_stream_force_2d(int(on))


def gemm_stream_last_map3d() -> bool:
    """Whether the last streaming product read its operands through three-dimensional tensor maps."""
    return bool(lib().fd_gemm_stream_last_map3d())


def tc_test_hook(wait_ns: int = 0, skip_last: bool = False) -> None:
    """Tests only.  The limit of every bounded wait of the TMA + tcgen05 kernels (0: the default of
    0.2 s) and whether their producers leave out their very last copy, so that a wait runs out and the
    kernel reports ``STATUS_WAIT_TIMEOUT`` and returns."""
    lib().fd_tc_test_hook(int(wait_ns), int(skip_last))


def gemv_splits(M: int, N: int, K: int, target_ctas: int, allow_split: bool = True) -> int:
    """Splits of K the decode matrix product would use; 0 if it does not take the sizes."""
    return int(lib().fd_gemv_splits(M, N, K, target_ctas, int(allow_split)))


def _prefetch_args(t: Optional[torch.Tensor], limit: int):
    """(pointer, bytes) of the leading ``limit`` bytes of a tensor that a kernel is to ask L2 for.  It is a hint:
    a tensor the kernels cannot take it from (not on the device, not contiguous, not 16-byte aligned) is passed over."""
    if t is None or limit <= 0 or not t.is_cuda or not t.is_contiguous() or t.data_ptr() % 16 != 0:
        return None, 0
    return t.data_ptr(), min(int(limit), t.numel() * t.element_size()) & ~15


def gemv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int,
         n_splits: int = 1, prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 1 << 62) -> None:
    """Weight-streaming product for M <= 64 rows (bfloat16): out = x w^T.
    mode GEMV_PARTIAL: out float32 [n_splits, M, N]; GEMV_BF16 / GEMV_F32: out
    [M, N] (+ bias), with ``n_splits`` <= 8 splits of K added inside a
    thread-block cluster; GEMV_GATED: w rows in tiles of 8 gate + 8 up, out
    bfloat16 [M, N / 2] = silu(gate) * up.  ``prefetch``: a tensor that a later kernel
    streams; the kernel asks L2 for its first ``prefetch_bytes`` once its own loads are through."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    want = {GEMV_PARTIAL: (torch.float32, n_splits * M * N), GEMV_BF16: (torch.bfloat16, M * N),
            GEMV_F32: (torch.float32, M * N), GEMV_GATED: (torch.bfloat16, M * N // 2),
            GEMV_GATED_GELU: (torch.bfloat16, M * N // 2)}[mode]
    assert out.dtype == want[0] and out.numel() == want[1], (out.dtype, out.shape, mode)
    _check(lib().fd_gemv(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                         _ptr(out), mode, M, N, K, n_splits, *_prefetch_args(prefetch, prefetch_bytes), _stream()))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] w[N, K]^T + bias on the CUDA cores (fixed k order)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and w.dtype == x.dtype
    _check(lib().fd_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dt(x.dtype),
                              _dt(bias.dtype) if bias is not None else 0, _dt(out.dtype), M, N, K, _stream()))


def attention_decode_heads(n_q: int, n_kv: int, head_dim: int, v_dim: int) -> int:
    """Key/value heads as the tensor-core decode kernel counts them: a group of more than 16 query heads on one
    key/value head is cut into several smaller groups that read the same cached head."""
    g = int(lib().fd_attn_decode_group(n_q // n_kv, head_dim, v_dim))
    return n_q // g if g > 0 else n_kv


def attention_scratch_floats(n_tokens: int, n_q: int, head_dim: int, n_splits: int) -> int:
    return int(lib().fd_attn_scratch_floats(n_tokens, n_q, head_dim, n_splits))


_attn_counters = {}      # per device: zeroed ints the decode kernel counts arriving splits in (kept alive for good)


def _counters(device, n: int) -> torch.Tensor:
    bufs = _attn_counters.setdefault(device, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]


def _attention(fn_name, q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start, row_q_len,
               row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits, split_len,
               scratch, status, prefetch=None, prefetch_bytes=0, chunk=0) -> None:
    T = q.shape[0]
    num_blocks, _, block_size, _ = k_pool.shape
    v_dim = v_pool.shape[-1]
    assert q.dtype == k_pool.dtype == out.dtype and k_pool.shape[-1] == head_dim and out.shape[-1] == n_q * v_dim
    assert v_pool.shape[:3] == k_pool.shape[:3]
    if n_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= attention_scratch_floats(T, n_q, v_dim, n_splits)
    args = [_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _dt(q.dtype), _ptr(block_table), block_table.shape[1],
            num_blocks, block_size, _ptr(tok_row), _ptr(row_slot), _ptr(row_q_start), _ptr(row_q_len),
            _ptr(row_ctx_len), n_rows, T, max_q_len, n_q, n_kv, head_dim, float(scale), int(window), int(v_dim),
            int(chunk), n_splits, split_len, _ptr(scratch)]
    if fn_name != "fd_attention_simt":
        fused = n_splits > 1 and max_q_len == 1 and q.dtype == torch.bfloat16
        # (a large group of query heads may be cut into several: at most one counter per query head)
        args.append(_ptr(_counters(q.device, n_rows * n_q)) if fused else None)
    args.append(_ptr(status))
    if fn_name == "fd_attention":
        args += list(_prefetch_args(prefetch, prefetch_bytes))
    args.append(_stream())
    _check(getattr(lib(), fn_name)(*args))


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
              block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
              row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
              n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
              window: int = 0, n_splits: int = 1, split_len: int = 0,
              scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
              prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 0, chunk: int = 0) -> None:
    """Causal GQA attention of the step's tokens over the paged cache, by the
    fastest kernel that takes the sizes (tensor cores for bfloat16 decode steps
    with head size 64 or 128; the CUDA-core kernel otherwise).  ``window`` > 0: a query
    sees the last ``window`` keys only; ``chunk`` > 0: only the keys of its own chunk of
    ``chunk`` positions, counted from the start of the sequence.  The size of a value head
    is that of ``v_pool`` (the tensor-core kernels take it equal to the key's).  ``prefetch``: a
    tensor that a later kernel streams; the tensor-core decode kernel asks L2 for its
    first ``prefetch_bytes`` when its own reads are through (the other kernels do not)."""
    _attention("fd_attention", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start, row_q_len,
               row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits, split_len,
               scratch, status, prefetch, prefetch_bytes, chunk=chunk)


def attention_mma_sync(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                       block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
                       row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
                       n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                       window: int = 0, n_splits: int = 1, split_len: int = 0,
                       scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                       chunk: int = 0) -> None:
    """The same with prompts on the mma.sync kernel even at head size 128, where
    ``attention`` takes the tcgen05 kernel."""
    _attention("fd_attention_mma_sync", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start,
               row_q_len, row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits,
               split_len, scratch, status, chunk=chunk)


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                   block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
                   row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
                   n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                   window: int = 0, n_splits: int = 1, split_len: int = 0,
                   scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                   chunk: int = 0) -> None:
    """The same on the CUDA cores for every size (the true 32-bit path)."""
    _attention("fd_attention_simt", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start,
               row_q_len, row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits,
               split_len, scratch, status, chunk=chunk)


def attention_ext(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                  block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
                  row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
                  n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                  window: int = 0, n_splits: int = 1, split_len: int = 0,
                  scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, chunk: int = 0,
                  softcap: float = 0.0, keep_first: int = 0, sink: Optional[torch.Tensor] = None,
                  all_value_heads: bool = False, tensor_cores: bool = True) -> None:
    """Attention with more options, on the CUDA cores; prompt steps in bfloat16 whose key and value heads both have 64
    or 128 dimensions run on the tensor cores unless ``tensor_cores`` is False, and so do decode steps in bfloat16 whose
    only option is ``sink`` (the split-keys decode kernel, at the sizes it takes).  ``softcap`` > 0: the scaled scores
    become softcap * tanh(score / softcap).  ``keep_first``: with a window, keys at positions below it stay
    visible.  ``sink`` [n_q] float32: exp(sink[h]) is one more term of head h's softmax denominator; it has
    no key and no value.  ``all_value_heads``: every query head's weights are applied to each of the ``n_kv``
    value heads; ``out`` is then float32 [T, n_q, n_kv, dv] (for ``attn_head_mix``).  Otherwise ``out`` is
    [T, n_q * dv] in q's dtype, or float32 if it is given so."""
    T = q.shape[0]
    num_blocks, _, block_size, _ = k_pool.shape
    v_dim = v_pool.shape[-1]
    v_rep = n_kv if all_value_heads else 1
    assert q.dtype == k_pool.dtype == v_pool.dtype and k_pool.shape[-1] == head_dim
    assert out.dtype in (q.dtype, torch.float32) and out.numel() == T * n_q * v_rep * v_dim
    assert not all_value_heads or out.dtype == torch.float32
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_q)
    if n_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= attention_scratch_floats(T, n_q * v_rep, v_dim, n_splits)
    # a bfloat16 decode step whose only option is the keyless term may run on the tensor-core decode kernel, which
    # merges its own splits when it is given counters
    fused = (n_splits > 1 and max_q_len == 1 and q.dtype == torch.bfloat16 and tensor_cores and sink is not None
             and not softcap and not (keep_first and window) and not all_value_heads and out.dtype == q.dtype)
    _check(lib().fd_attention_ext(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _dt(q.dtype), _ptr(block_table), block_table.shape[1],
        num_blocks, block_size, _ptr(tok_row), _ptr(row_slot), _ptr(row_q_start), _ptr(row_q_len), _ptr(row_ctx_len),
        n_rows, T, max_q_len, n_q, n_kv, head_dim, float(scale), int(window), int(v_dim), int(chunk), n_splits,
        split_len, _ptr(scratch), _ptr(status), float(softcap), int(keep_first), _ptr(sink), v_rep,
        int(out.dtype == torch.float32 and q.dtype != torch.float32 or all_value_heads), int(tensor_cores),
        _ptr(_counters(q.device, n_rows * n_q)) if fused else None, _stream()))


def _col_ptr(t: torch.Tensor, first_col: int) -> int:
    assert t.is_contiguous() and t.dim() == 2 and 0 <= first_col < t.shape[1]
    return _ptr(t) + first_col * t.element_size()


def attn_head_mix(o: torch.Tensor, mix: torch.Tensor, out: torch.Tensor, first_col: int, n_q: int, n_kv: int,
                  v_head_dim: int, scale: float = 1.0) -> None:
    """out[t, first_col + h dv + j] = scale * sum_g mix[h, g] o[t, g, h // (n_q / n_kv), j]: the heads' attention
    weights mixed after the softmax, each head on the values of its own key/value head.  ``o`` float32
    [T, n_q, n_kv, dv] from ``attention_ext(all_value_heads=True)``; ``mix`` float32 [n_q, n_q]; ``out`` [T, ld]."""
    T, dv = o.shape[0], v_head_dim
    assert o.dtype == torch.float32 and o.numel() == T * n_q * n_kv * dv and mix.dtype == torch.float32
    assert mix.shape == (n_q, n_q) and out.shape[0] == T and first_col + n_q * dv <= out.shape[1]
    _check(lib().fd_attn_head_mix(_ptr(o), _ptr(mix), _col_ptr(out, first_col), out.shape[1], _dt(out.dtype), T, n_q,
                                  n_kv, dv, float(scale), _stream()))


def add_dyn_tanh(delta: Optional[torch.Tensor], resid: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                 alpha: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                 write_resid: bool = True) -> None:
    """resid[r] += delta[r]; out[j] = tanh(alpha * resid[r]) * weight + bias with r = rows[j] (or j).  No mean, no
    variance.  ``resid``, ``weight`` and ``bias`` float32; ``delta`` [*, H] float32 or bfloat16, or None."""
    H = resid.shape[-1]
    if n_out is None:
        n_out = rows.numel() if rows is not None else resid.numel() // H
    assert resid.dtype == weight.dtype == bias.dtype == torch.float32 and weight.numel() == bias.numel() == H
    assert out.shape[-1] == H and (delta is None or (delta.dim() == 2 and delta.shape[-1] == H))
    _check(lib().fd_add_dyn_tanh(_ptr(delta), _dt(delta.dtype) if delta is not None else 0, _ptr(resid), int(write_resid),
                                 _ptr(weight), _ptr(bias), float(alpha), _ptr(out), _dt(out.dtype), _ptr(rows), n_out, H,
                                 _stream()))


def quad_exp_act(x: torch.Tensor, pq: torch.Tensor, out: torch.Tensor) -> None:
    """out = softplus(p) z^2 + z / 2 where z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 elsewhere; ``pq`` float32
    [2] = (p, q) on the device.  Float arithmetic, one rounding."""
    assert x.shape == out.shape and x.dtype == out.dtype and pq.dtype == torch.float32 and pq.numel() == 2
    _check(lib().fd_quad_exp_act(_ptr(x), _ptr(out), _dt(x.dtype), _ptr(pq), x.numel(), _stream()))


def scale_(x: torch.Tensor, s: float) -> None:
    """x <- x * s in place; x float32."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().fd_scale_f32(_ptr(x), x.numel(), float(s), _stream()))


def axpy_f32(y: torch.Tensor, x: torch.Tensor, s: float, accumulate: bool = True) -> None:
    """y <- s * x (+ y if ``accumulate``); y float32, x float32 or bfloat16 of the same shape."""
    assert y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous()
    _check(lib().fd_axpy_f32(_ptr(y), _ptr(x), _dt(x.dtype), y.numel(), float(s), int(accumulate), _stream()))


SCAN_DECAY, SCAN_GATED, SCAN_CHANNEL_DECAY = 0, 1, 2


def linear_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, state: torch.Tensor, out: torch.Tensor,
                mode: int, row_slot: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
                row_ctx_len: torch.Tensor, n_rows: int, n_heads: int, head_dim: int, v_head_dim: int,
                write_state: bool, status: torch.Tensor, decay: Optional[torch.Tensor] = None,
                lower: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                sin: Optional[torch.Tensor] = None, rot_dims: int = 0, k_scale: float = 1.0, max_q_len: int = 0,
                scratch: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_col: int = 0,
                q_scale: float = 1.0, tau: float = 1.0) -> None:
    """The recurrence S_t = diag(a_t) S_(t-1) + b_t v_t^T, o_t = S_t^T q_t per sequence and head over the step's
    tokens, from ``state`` [slots, heads, head_dim, v_head_dim] (float32, updated when ``write_state``) to ``out``
    [T, heads * v_head_dim] (float32).  q, k and v are column ranges of ``proj`` [T, ld].  ``SCAN_DECAY``: a = decay[h],
    b = rotated k times ``k_scale``, q rotated (the first ``rot_dims`` dimensions, i paired with i + rot_dims / 2).
    ``SCAN_GATED``: the k columns hold the gate's pre-activation z; a = lower + (1 - lower) sigmoid(z), b = 1 - a,
    q = silu of the q columns.  ``SCAN_CHANNEL_DECAY``: a = sigmoid(z)^(1 / tau) per key channel with z the columns
    ``gate_col ...`` of ``gate`` [T, ldg] (float32), b = the k columns, q = the q columns times ``q_scale``.  With ``scratch`` (float32, ``linear_scan_scratch_floats`` elements) and ``max_q_len`` (the
    longest portion of the step), portions longer than two segments are cut into segments that run side by side."""
    T = proj.shape[0]
    assert state.dtype == out.dtype == torch.float32 and state.shape[1:] == (n_heads, head_dim, v_head_dim)
    assert out.shape == (T, n_heads * v_head_dim) and proj.is_contiguous()
    assert max(q_col, k_col) + n_heads * head_dim <= proj.shape[1] and v_col + n_heads * v_head_dim <= proj.shape[1]
    if mode == SCAN_DECAY:
        assert decay is not None and decay.dtype == torch.float32 and decay.numel() == n_heads
        if rot_dims:
            assert cos.dtype == torch.float32 and cos.shape[1] == rot_dims // 2 and sin.shape == cos.shape
    elif mode == SCAN_GATED:
        assert lower is not None and lower.dtype == torch.float32 and lower.numel() == n_heads * head_dim
        rot_dims = 0
    else:
        assert gate is not None and gate.dtype == torch.float32 and gate.shape[0] == T and gate.is_contiguous()
        assert gate_col + n_heads * head_dim <= gate.shape[1] and tau > 0
        rot_dims = 0
    _check(lib().fd_linear_scan(_ptr(proj), proj.shape[1], _dt(proj.dtype), q_col, k_col, v_col, _ptr(state), _ptr(out),
                                mode, _ptr(decay), _ptr(lower), _ptr(cos) if rot_dims else None,
                                _ptr(sin) if rot_dims else None, cos.shape[0] if rot_dims else 0, rot_dims,
                                float(k_scale), _ptr(row_slot), _ptr(row_q_start), _ptr(row_q_len), _ptr(row_ctx_len),
                                n_rows, n_heads, head_dim, v_head_dim, int(write_state), _ptr(status), T, int(max_q_len),
                                _ptr(scratch) if scratch is not None else None,
                                scratch.numel() if scratch is not None else 0,
                                _col_ptr(gate, gate_col) if gate is not None else None,
                                gate.shape[1] if gate is not None else 0, float(q_scale), 1.0 / float(tau), _stream()))


def linear_scan_segment() -> int:
    """Tokens of a segment of ``linear_scan``; portions longer than two of them run in segments."""
    return lib().fd_linear_scan_segment()


def linear_scan_scratch_floats(T: int, n_rows: int, n_heads: int, head_dim: int, v_head_dim: int) -> int:
    """float32 elements of scratch memory with which ``linear_scan`` runs a step of T tokens in n_rows sequences in segments."""
    return int(lib().fd_linear_scan_scratch_floats(T, n_rows, n_heads, head_dim, v_head_dim))


LOW_RANK_EXPAND_MAX = 64        # widest vector ``low_rank_expand`` takes


def low_rank_expand(x: torch.Tensor, first_col: int, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t, c] = bias[c] + sum_r w[c, r] * x[t, first_col + r]; x [T, ld] and w [N, R] in the model's dtype (R at most
    ``LOW_RANK_EXPAND_MAX``), bias float32 [N] or None, out float32 [T, N].  Float sums in the order r = 0, 1, ..."""
    T, (N, R) = x.shape[0], w.shape
    assert x.dtype == w.dtype and out.dtype == torch.float32 and out.shape == (T, N) and first_col + R <= x.shape[1]
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    _check(lib().fd_low_rank_expand(_col_ptr(x, first_col), x.shape[1], _ptr(w), _ptr(bias), _ptr(out), _dt(x.dtype),
                                    T, N, R, _stream()))


def head_norm_gate(o: torch.Tensor, out: torch.Tensor, first_col: int, n_heads: int, v_head_dim: int, eps: float,
                   weight: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_col: int = 0,
                   scale: float = 1.0) -> None:
    """out[t, first_col + h dv + j] = scale * o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) [* weight[j]]
    [* silu(gate[t, gate_col + h dv + j])].  ``o`` float32 [T, heads * dv]; ``weight`` float32 [dv]; ``gate`` a packed
    projection [T, ldg] in out's dtype."""
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.shape == (T, n_heads * v_head_dim) and out.shape[0] == T
    assert first_col + n_heads * v_head_dim <= out.shape[1]
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == v_head_dim)
    assert gate is None or (gate.dtype == out.dtype and gate.shape[0] == T and gate_col + n_heads * v_head_dim <= gate.shape[1])
    _check(lib().fd_head_norm_gate(_ptr(o), _ptr(weight), _col_ptr(gate, gate_col) if gate is not None else None,
                                   gate.shape[1] if gate is not None else 0, _col_ptr(out, first_col), out.shape[1],
                                   _dt(out.dtype), T, n_heads, v_head_dim, float(eps), float(scale), _stream()))


# ---------------------------------------------------------------------------
# short convolution + partial rotation + cache append; gates; routed experts

def conv_rope_append(proj: torch.Tensor, conv_w: torch.Tensor, state: Optional[torch.Tensor], q_out: torch.Tensor,
                     cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot_dims: int, tok_row: torch.Tensor,
                     tok_pos: torch.Tensor, row_slot: torch.Tensor, row_q_start: torch.Tensor, row_q_len: torch.Tensor,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, n_q: int, n_kv: int,
                     head_dim: int, v_head_dim: int, write_kv: bool, update_state: bool, status: torch.Tensor,
                     interleaved: bool = False, first_col: int = 0, q_norm: Optional[torch.Tensor] = None,
                     k_norm: Optional[torch.Tensor] = None, norm_eps: float = 0.0, norm_count: int = 0,
                     values_from_keys: bool = False) -> None:
    """For every token: the causal convolution over time of each q, k and v channel of ``proj``
    [T, >= C] (C = (n_q + n_kv) head_dim + n_kv v_head_dim leading columns) with ``conv_w`` [C, taps]
    (float32), earlier steps' values taken from ``state`` [slots, taps - 1, C] (float32); rotation of
    the first ``rot_dims`` dimensions of every q and k head (i paired with i + rot_dims / 2); q to
    ``q_out`` [T, n_q head_dim], k and v to the paged pools.  ``update_state``: rows that bring one
    token move their state on in the same kernel (use ``conv_state_update`` for the others).
    ``interleaved``: the rotation pairs dimension 2i with 2i + 1.  ``first_col``: the column of ``proj``
    at which the C channels start (an even number).  ``q_norm`` / ``k_norm`` [head_dim] float32: every q / k head is
    RMS-normed with that weight (``norm_eps``; the mean over ``norm_count`` dimensions, default head_dim) after the
    convolution and before the rotation.  ``values_from_keys``: ``proj`` has no v columns (C = (n_q + n_kv) head_dim)
    and the value pool receives the convolved keys as they are before norm and rotation."""
    T = proj.shape[0]
    taps = conv_w.shape[1]
    C = (n_q + n_kv) * head_dim + (0 if values_from_keys else n_kv * v_head_dim)
    for nw in (q_norm, k_norm):
        assert nw is None or (nw.dtype == torch.float32 and nw.numel() == head_dim)
    assert conv_w.dtype == torch.float32 and conv_w.shape == (C, taps) and proj.shape[1] >= first_col + C
    assert first_col % 2 == 0 and proj.is_contiguous()
    assert state is None or (state.dtype == torch.float32 and state.shape[1:] == (taps - 1, C))
    assert proj.dtype == q_out.dtype == k_pool.dtype == v_pool.dtype and q_out.shape == (T, n_q * head_dim)
    assert k_pool.shape[-1] == head_dim and v_pool.shape[-1] == v_head_dim
    if rot_dims:
        assert cos.dtype == torch.float32 and cos.shape[1] == rot_dims // 2 and sin.shape == cos.shape
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_conv_rope_append(_ptr(proj) + first_col * proj.element_size(), proj.shape[1], _dt(proj.dtype),
                                     _ptr(conv_w), _ptr(state), _ptr(q_out),
                                     _ptr(cos) if rot_dims else None, _ptr(sin) if rot_dims else None,
                                     cos.shape[0] if rot_dims else 0, rot_dims, _ptr(tok_row), _ptr(tok_pos),
                                     _ptr(row_slot), _ptr(row_q_start), _ptr(row_q_len), _ptr(k_pool), _ptr(v_pool),
                                     _ptr(block_table), block_table.shape[1], num_blocks, block_size, T, n_q, n_kv,
                                     head_dim, v_head_dim, taps, int(write_kv), int(update_state), _ptr(status),
                                     int(interleaved), _ptr(q_norm), _ptr(k_norm), float(norm_eps),
                                     int(norm_count or head_dim), int(values_from_keys), _stream()))


def conv_state_update(proj: torch.Tensor, state: torch.Tensor, row_slot: torch.Tensor, row_q_start: torch.Tensor,
                      row_q_len: torch.Tensor, n_rows: int, first_col: int = 0) -> None:
    """``state`` [slots, taps - 1, C] of every row's sequence <- its last taps - 1 projected values after the step
    (the C columns of ``proj`` from ``first_col`` on)."""
    hist, C = state.shape[1], state.shape[2]
    assert state.dtype == torch.float32 and proj.shape[1] >= first_col + C and proj.is_contiguous()
    _check(lib().fd_conv_state_update(_ptr(proj) + first_col * proj.element_size(), proj.shape[1], _dt(proj.dtype),
                                      _ptr(state), _ptr(row_slot),
                                      _ptr(row_q_start), _ptr(row_q_len), n_rows, C, hist + 1, _stream()))


def gate_mul(a: torch.Tensor, packed: torch.Tensor, first_col: int, out: torch.Tensor) -> None:
    """out = a * sigmoid(g) with g the columns ``first_col ...`` of ``packed`` [M, ld]; a, out [M, C]."""
    M, C = a.shape
    assert out.shape == a.shape and a.dtype == out.dtype == packed.dtype and packed.shape[0] == M
    assert first_col + C <= packed.shape[1] and packed.is_contiguous()
    g_ptr = packed.data_ptr() + first_col * packed.element_size()
    _check(lib().fd_gate_mul(_ptr(a), g_ptr, packed.shape[1], _ptr(out), _dt(a.dtype), M, C, _stream()))


def add_concat(delta: Optional[torch.Tensor], resid: torch.Tensor, other: torch.Tensor, out: torch.Tensor) -> None:
    """resid += delta (if given); out [T, 2H] = [resid | other] in out's dtype; resid and other float32 [T, H]."""
    T, H = resid.shape
    assert resid.dtype == other.dtype == torch.float32 and out.shape == (T, 2 * H) and other.shape == resid.shape
    assert delta is None or delta.shape == resid.shape
    _check(lib().fd_add_concat(_ptr(delta), _dt(delta.dtype) if delta is not None else 0, _ptr(resid), _ptr(other),
                               _ptr(out), _dt(out.dtype), T, H, _stream()))


def add_cast(delta: Optional[torch.Tensor], resid: torch.Tensor, out: torch.Tensor, delta_scale: float = 1.0) -> None:
    """resid += delta_scale * delta (if given); out [T, H] = resid rounded to out's dtype; resid float32 [T, H]."""
    T, H = resid.shape
    assert resid.dtype == torch.float32 and out.shape == (T, H) and (delta is None or delta.shape == (T, H))
    _check(lib().fd_add_cast(_ptr(delta), _dt(delta.dtype) if delta is not None else 0, _ptr(resid), _ptr(out),
                             _dt(out.dtype), T, H, float(delta_scale), _stream()))


def side_gate_mul(z: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, first_col: int, g: torch.Tensor,
                  status: torch.Tensor) -> None:
    """g[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], first_col + j]; z float32 [T, dim], g [T, dim] in the table's
    dtype."""
    T, dim = z.shape
    assert z.dtype == torch.float32 and g.shape == (T, dim) and g.dtype == table.dtype and tokens.dtype == torch.int32
    _check(lib().fd_side_gate_mul(_ptr(z), _ptr(tokens), _ptr(table), table.shape[1], first_col, table.shape[0], _ptr(g),
                                  _dt(g.dtype), T, dim, _ptr(status), _stream()))


TOKEN_SIDE_ROW_MAX_FLOATS = 12000 - 48      # floats of shared memory the one-launch form has for a row and its gate values


def token_side_row(delta: Optional[torch.Tensor], resid: torch.Tensor, delta_scale: float, tokens: torch.Tensor,
                   table: torch.Tensor, first_col: int, gate_w: torch.Tensor, proj_w: torch.Tensor,
                   norm_w: torch.Tensor, eps: float, out: torch.Tensor, status: torch.Tensor,
                   scratch: Optional[torch.Tensor] = None) -> None:
    """In two launches made for steps of few tokens: resid += delta_scale * delta; g = gelu_tanh(gate_w x) *
    table[token, first_col ...]; y = proj_w g; out = y / sqrt(mean(y^2) + eps) * norm_w (float32 [T, H]).  gate_w
    [dim, H], proj_w [H, dim]; ``scratch`` float32 [T, dim] holds g between the launches."""
    T, H = resid.shape
    dim = gate_w.shape[0]
    if scratch is None:
        scratch = torch.empty(T, dim, dtype=torch.float32, device=resid.device)
    assert scratch.dtype == torch.float32 and scratch.numel() >= T * dim
    assert resid.dtype == out.dtype == torch.float32 and out.shape == (T, H) and gate_w.shape == (dim, H)
    assert proj_w.shape == (H, dim) and gate_w.dtype == proj_w.dtype == table.dtype and norm_w.numel() == H
    _check(lib().fd_token_side_row(_ptr(delta), _dt(delta.dtype) if delta is not None else 0, _ptr(resid),
                                   float(delta_scale), _ptr(tokens), _ptr(table), table.shape[1], first_col, table.shape[0],
                                   _ptr(gate_w), _ptr(proj_w), _ptr(norm_w), _dt(norm_w.dtype), float(eps), _ptr(scratch),
                                   _ptr(out), _dt(gate_w.dtype), T, H, dim, _ptr(status), _stream()))


def add_row_vector(delta: Optional[torch.Tensor], resid: torch.Tensor, vec: torch.Tensor, delta_scale: float = 1.0) -> None:
    """resid <- resid + delta_scale * delta + vec; resid float32 [T, H], vec float32 [H], delta [T, H] or None."""
    T, H = resid.shape
    assert resid.dtype == vec.dtype == torch.float32 and vec.numel() == H and (delta is None or delta.shape == (T, H))
    _check(lib().fd_add_row_vector(_ptr(delta), _dt(delta.dtype) if delta is not None else 0, _ptr(resid), _ptr(vec),
                                   T, H, float(delta_scale), _stream()))


def relu2(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0)^2."""
    assert x.shape == out.shape and x.dtype == out.dtype
    _check(lib().fd_relu2(_ptr(x), _ptr(out), _dt(x.dtype), x.numel(), _stream()))


def moe_tile_rows(dtype: torch.dtype = torch.float32, n_pairs: int = 0, n_experts: int = 1, k_sizes=()) -> int:
    """Rows of a tile of the grouped products: 32, or 128 for bfloat16 steps with many (token, choice) pairs per
    expert (prompts).  ``k_sizes``: the inner sizes of the products; one that is no multiple of 8 keeps the products
    on the CUDA cores, whose tiles have 32 rows."""
    if dtype != torch.bfloat16 or any(k % 8 for k in k_sizes):
        return int(lib().fd_moe_tile_rows(0, 0))
    return int(lib().fd_moe_tile_rows(1, n_pairs // max(1, n_experts)))


def moe_grouped_rows(n_pairs: int, n_experts: int, mt: int) -> int:
    """Rows of the grouped buffers that hold ``n_pairs`` (token, choice) pairs of ``n_experts`` experts whatever the
    routing: every expert's group is padded to whole tiles of ``mt`` rows."""
    worst = n_pairs + min(n_experts, n_pairs) * (mt - 1)
    return -(-worst // mt) * mt


ROUTE_FUSED_MAX_ROW = 8192      # widest row of x the routing kernel takes into shared memory to make its own logits


def moe_route(x: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], ids: torch.Tensor,
              wts: torch.Tensor, logits: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
              sigmoid_scores: bool = False, n_groups: int = 1, keep_groups: int = 1,
              weight_scale: Optional[float] = None) -> None:
    """Per row of x [T, H]: softmax scores over the rows of ``router`` [n_out, H] (float arithmetic), the ``top``
    outputs with the largest score + correction into ``ids`` [T, top] (int32), and their scores over their sum
    (+ 1e-20) into ``wts`` [T, top] (float32).  ``logits`` [T, n_out] float32: the router's outputs made by a matrix
    product beforehand (steps of many tokens); without them the kernel makes them itself, a token per CTA.
    ``bias`` [n_out] float32 is added to the logits before the softmax.  The chosen scores over their sum are the
    softmax over the chosen logits alone.  ``sigmoid_scores``: the scores are sigmoid(logit) instead of the softmax.
    ``n_groups`` > ``keep_groups``: the outputs form ``n_groups`` equal groups of neighbours, a group ranks by the sum of
    its two largest score + correction, and only outputs of the best ``keep_groups`` groups can be chosen.
    ``weight_scale``: the weights are the chosen scores times this constant, not divided by their sum."""
    T, H = x.shape
    n_out, top = router.shape[0], ids.shape[1]
    assert router.shape == (n_out, H) and router.dtype == x.dtype and ids.dtype == torch.int32
    assert wts.dtype == torch.float32 and wts.shape == ids.shape == (T, top)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == n_out)
    assert logits is None or (logits.dtype == torch.float32 and logits.shape == (T, n_out))
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == n_out)
    _check(lib().fd_moe_route(_ptr(x), _ptr(router), _dt(x.dtype), _ptr(logits), _ptr(correction), _ptr(bias), _ptr(ids),
                              _ptr(wts), T, H, n_out, top, int(sigmoid_scores), int(n_groups), int(keep_groups),
                              int(weight_scale is None), float(weight_scale or 0.0), _stream()))


def moe_align(ids: torch.Tensor, n_experts: int, pair_pos: torch.Tensor, sorted_pair: torch.Tensor,
              tile_expert: torch.Tensor, n_tiles: torch.Tensor, mt: int) -> None:
    """Group the (token, choice) pairs of ``ids`` by expert, every group padded to whole tiles of ``mt`` rows
    (outputs >= ``n_experts`` are left out: pair_pos -1)."""
    P = ids.numel()
    cap = sorted_pair.numel()
    assert all(t.dtype == torch.int32 for t in (ids, pair_pos, sorted_pair, tile_expert, n_tiles))
    assert pair_pos.numel() >= P and tile_expert.numel() * mt >= cap
    _check(lib().fd_moe_align(_ptr(ids), P, n_experts, _ptr(pair_pos), _ptr(sorted_pair), _ptr(tile_expert),
                              _ptr(n_tiles), cap, mt, _stream()))


def moe_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, down: bool, sorted_pair: torch.Tensor,
             tile_expert: torch.Tensor, n_tiles: torch.Tensor, top: int, mt: int, plain: bool = False,
             gated_limit: Optional[float] = None, gated_act: Optional[int] = None) -> None:
    """Grouped product with the experts' stacked matrices w [E, N, K].  ``down`` False: a = x [T, K] (rows gathered
    through the grouping), out [cap, N] = relu(x w_e^T)^2 in a's dtype; True: a = the grouped activations [cap, K],
    out [cap, N] in a's dtype.  ``plain`` (with ``down`` False): no activation, out = x w_e^T (a gated activation follows
    in a kernel of its own).  ``mt``: the tile rows the grouping was made with.  bfloat16 with K a multiple of 8 runs on
    the tensor cores, everything else on the CUDA cores (tiles of 32 rows only).  ``gated_limit`` (clamped swish with
    that limit) or ``gated_act`` (GLU_SILU, GLU_GELU_TANH): w's rows are tiles of 8 gate + 8 up rows and out [cap, N / 2]
    is the gated activation of each pair."""
    E, N, Kd = w.shape
    cap = sorted_pair.numel()
    gated = gated_limit is not None or gated_act is not None
    act = GLU_CLAMPED if gated_limit is not None else (gated_act or 0)
    assert a.dtype == w.dtype and a.shape[1] == Kd and out.shape == (cap, N // 2 if gated else N)
    assert out.dtype == a.dtype and (not down or a.shape[0] == cap) and not (gated and (down or plain))
    mode = 1 if down else (3 if gated else (2 if plain else 0))
    _check(lib().fd_moe_gemm(_ptr(a), _ptr(w), _ptr(out), _dt(a.dtype), mode, _ptr(sorted_pair), _ptr(tile_expert),
                             _ptr(n_tiles), cap, mt, top, N, Kd, float(gated_limit or 0.0), int(act), _stream()))


def moe_gather(x: torch.Tensor, xs: torch.Tensor, sorted_pair: torch.Tensor, n_tiles: torch.Tensor, top: int,
               mt: int) -> None:
    """xs [cap, K] <- the rows of x [T, K] in grouped order (zeros in padding rows; rows beyond the tiles that exist are
    left alone): the operand of ``gemm_tc_grouped``, which reads through a tensor map."""
    cap, Kd = xs.shape
    assert x.dtype == xs.dtype == torch.bfloat16 and x.shape[1] == Kd and sorted_pair.numel() == cap
    _check(lib().fd_moe_gather(_ptr(x), _ptr(xs), _ptr(sorted_pair), _ptr(n_tiles), cap, mt, top, Kd, _stream()))


def gemm_tc_grouped_supported(N: int, K: int) -> bool:
    """Whether the grouped tcgen05 product takes matrices [N, K]."""
    return N >= 256 and gemm_tc_supported(128, N, K)


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, relu2: bool, tile_expert: torch.Tensor,
                    n_tiles: torch.Tensor, status: Optional[torch.Tensor] = None,
                    gated_limit: Optional[float] = None, gated_act: Optional[int] = None) -> None:
    """Grouped product on the tcgen05 tensor cores: x [cap, K] in row tiles of 128 of which the first ``n_tiles``
    exist, tile t times matrix ``tile_expert[t]`` of the stack w [E, N, K] (both device tensors).  ``relu2``: out
    bfloat16 [cap, N] = max(x w_e^T, 0)^2; else out bfloat16 or float32 [cap, N]."""
    cap, Kd = x.shape
    E, N, _ = w.shape
    # w rows in tiles of 8 gate + 8 up: out bfloat16 [cap, N / 2] = clamped swish(gate) (up + 1) with ``gated_limit``, or
    # ``gated_act`` (GLU_SILU, GLU_GELU_TANH) of gate, times up
    gated = gated_limit is not None or gated_act is not None
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[2] == Kd and cap % 128 == 0
    assert out.shape == (cap, N // 2 if gated else N) and not (gated and relu2)
    assert out.dtype in ((torch.bfloat16,) if relu2 or gated else (torch.bfloat16, torch.float32)) and tile_expert.numel() * 128 >= cap
    mode = 5 if relu2 else (1 if out.dtype == torch.bfloat16 else 2)
    if gated:
        mode = 7 if gated_limit is not None else (8 if gated_act == GLU_SILU else 9)
    _check(lib().fd_gemm_tc_grouped(_ptr(x), _ptr(w), _ptr(out), mode, cap, N, Kd, E, _ptr(tile_expert),
                                    _ptr(n_tiles), float(gated_limit or 0.0), _ptr(status), _stream()))


def moe_combine(y: Optional[torch.Tensor], x: torch.Tensor, shared: Optional[torch.Tensor], ids: torch.Tensor,
                wts: torch.Tensor, pair_pos: torch.Tensor, out: torch.Tensor, n_experts: int) -> None:
    """out[t] = sum_c wts[t, c] * (y[pair_pos[t, c]] if ids[t, c] < n_experts else x[t]) + shared[t]."""
    T, H = x.shape
    top = ids.shape[1]
    assert out.shape == x.shape and out.dtype == x.dtype and (shared is None or shared.shape == x.shape)
    assert y is None or (y.dtype == x.dtype and y.shape[1] == H)
    _check(lib().fd_moe_combine(_ptr(y), _ptr(x), _ptr(shared), _ptr(ids), _ptr(wts), _ptr(pair_pos), _ptr(out),
                                _dt(x.dtype), T, H, top, n_experts, _stream()))


_sample_scratch = {}


def sample_scratch_words(n: int, V: int) -> int:
    return int(lib().fd_sample_scratch_words(n, V))


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           request: Optional[torch.Tensor] = None, step: Optional[torch.Tensor] = None, seed: int = 0,
           scratch: Optional[torch.Tensor] = None, seed_tensor: Optional[torch.Tensor] = None) -> None:
    """out[i] = argmax (greedy) or a Gumbel-max draw from softmax(logits[i] / T_i).
    ``scratch``: int32 tensor of ``sample_scratch_words(n, V)`` entries for large
    vocabularies; when omitted a per-device buffer is kept and reused.  ``seed_tensor``:
    a one-element int64 tensor on the device that holds the seed (its 64 bits) instead of
    ``seed``, so that a captured graph serves any seed."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and request.dtype == torch.int64 and step.dtype == torch.int32
    words = sample_scratch_words(n, V)
    if words and scratch is None:
        key = logits.device
        scratch = _sample_scratch.get(key)
        if scratch is None or scratch.numel() < words:
            scratch = torch.empty(max(words, 4096), dtype=torch.int32, device=logits.device)
            _sample_scratch[key] = scratch
    if words:
        assert scratch.dtype == torch.int32 and scratch.numel() >= words
    assert seed_tensor is None or (seed_tensor.dtype == torch.int64 and seed_tensor.numel() == 1)
    _check(lib().fd_sample(_ptr(logits), n, V, _ptr(temperature), _ptr(request), _ptr(step),
                           seed & 0xFFFFFFFFFFFFFFFF, _ptr(seed_tensor), _ptr(out), _ptr(scratch) if words else None,
                           _stream()))
