"""Python entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors, checks what the kernel assumes, and launches
on the current stream.  There is no other implementation behind them: a tensor
that is not on a CUDA device, or a library that cannot be built or loaded, is
an error.  Model parts call these as ``kernels.<name>(...)``.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from kairyu_b200.kernels.build import KernelBuildError, load_library

# The library products (cuBLAS through torch) may otherwise add split-K partial sums in
# bfloat16; this engine's products accumulate and reduce in fp32.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

c_int = ctypes.c_int
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p

FLAG_BAD_PAGE = 1
FLAG_BAD_TOKEN = 2
FLAG_BAD_ROW = 4
FLAG_BAD_POS = 8
FLAG_TIMEOUT = 16
FLAG_MISALIGNED = 32

_CODES = {
    -1: "bad argument",
    -2: "a size this kernel does not support",
    -3: "a required pointer is null",
}


class KernelError(RuntimeError):
    pass


launch_count = 0  # kernel launches made through this module (library products not counted)


def _check(code: int, what: str, launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code < 0:
        raise KernelError(f"{what}: {_CODES.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current stream of the current device.  The raw accessor costs a fraction of a
    microsecond; building a torch Stream object for every launch cost 15 (a step launches hundreds)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _need_cuda(what: str, *tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError(
                f"{what}: tensor on {tensor.device}; the kernels of kairyu_b200 run on CUDA "
                "devices only and have no CPU implementation"
            )


def _is_bf16(tensor: torch.Tensor, what: str) -> int:
    if tensor.dtype == torch.bfloat16:
        return 1
    if tensor.dtype == torch.float32:
        return 0
    raise KernelError(f"{what}: dtype {tensor.dtype} is not supported (float32 or bfloat16)")


def _need_i32(what: str, *tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and (tensor.dtype != torch.int32 or not tensor.is_contiguous()):
            raise KernelError(f"{what}: index tensors must be contiguous int32")


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str, argtypes: list) -> ctypes._CFuncPtr:
    function = _functions.get(name)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = c_int
        _functions[name] = function
    return function


# ----------------------------------------------------------------------------- elementwise


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, flag: Optional[torch.Tensor] = None, *, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale as fp32."""
    _need_cuda("embedding", table, ids, out, flag)
    _need_i32("embedding", ids)
    V, H = table.shape
    if out.dtype != torch.float32 or out.shape != (ids.numel(), H) or not out.is_contiguous():
        raise KernelError("embedding: out must be contiguous fp32 [tokens, hidden]")
    if not table.is_contiguous():
        raise KernelError("embedding: table must be contiguous")
    fn = _fn("elementwise", "kb_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(table.data_ptr(), _is_bf16(table, "embedding"), ids.data_ptr(), out.data_ptr(), ids.numel(), H, V, float(scale), _ptr(flag), _stream()), "embedding")


def add_positions(table: torch.Tensor, positions: torch.Tensor, x: torch.Tensor, flag: Optional[torch.Tensor] = None) -> None:
    """x[t] += table[positions[t]] on the fp32 residual (learned absolute positions)."""
    _need_cuda("add_positions", table, positions, x, flag)
    _need_i32("add_positions", positions)
    P, H = table.shape
    if x.dtype != torch.float32 or x.shape != (positions.numel(), H) or not x.is_contiguous() or not table.is_contiguous():
        raise KernelError("add_positions: x must be contiguous fp32 [tokens, hidden] and the table contiguous [positions, hidden]")
    fn = _fn("elementwise", "kb_add_positions", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(table.data_ptr(), _is_bf16(table, "add_positions"), positions.data_ptr(), x.data_ptr(), positions.numel(), H, P, _ptr(flag), _stream()), "add_positions")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) element by element (``out`` may be ``x``): ``relu2`` = relu(x)^2, ``gelu_tanh``, ``silu``."""
    _need_cuda("activation", x, out)
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: unknown kind {kind!r} ({', '.join(ACTIVATIONS)})")
    if x.shape != out.shape or x.dtype != out.dtype or not (x.is_contiguous() and out.is_contiguous()):
        raise KernelError("activation: contiguous tensors of one shape and dtype")
    fn = _fn("elementwise", "kb_activation", [c_void_p, c_void_p, c_int, ctypes.c_longlong, c_int, c_void_p])
    _check(fn(x.data_ptr(), out.data_ptr(), _is_bf16(x, "activation"), x.numel(), ACTIVATIONS[kind], _stream()), "activation")


def patch_tokens(ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor, flag: Optional[torch.Tensor] = None) -> None:
    """ids[t] = sampled[source[t]] wherever source[t] >= 0 (tokens the host has not seen yet)."""
    _need_cuda("patch_tokens", ids, source, sampled, flag)
    _need_i32("patch_tokens", ids, source, sampled)
    if source.numel() != ids.numel() or not (ids.is_contiguous() and source.is_contiguous() and sampled.is_contiguous()):
        raise KernelError("patch_tokens: ids and source must be contiguous and of one length")
    fn = _fn("elementwise", "kb_patch_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(fn(ids.data_ptr(), source.data_ptr(), sampled.data_ptr(), ids.numel(), sampled.numel(), _ptr(flag), _stream()), "patch_tokens")


def rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    *,
    delta: Optional[torch.Tensor] = None,
    rows: Optional[torch.Tensor] = None,
) -> None:
    """``x += delta`` (if given and ``rows`` is None), ``out = rmsnorm(x) * weight``.

    With ``rows`` only the listed rows of x (+delta) are normed, into
    out[0..len(rows)), and x is not modified.
    """
    _need_cuda("rmsnorm", x, weight, out, delta, rows)
    _need_i32("rmsnorm", rows)
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.shape[0]
    if not x.is_contiguous() or not out.is_contiguous() or (delta is not None and not delta.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    if weight.numel() != H or out.shape[-1] != H or out.shape[0] < R:
        raise KernelError("rmsnorm: shape mismatch")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != x.shape):
        raise KernelError("rmsnorm: delta must have the activation dtype and x's shape")
    fn = _fn("elementwise", "kb_rmsnorm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(
        fn(x.data_ptr(), _is_bf16(x, "rmsnorm"), _ptr(delta), weight.data_ptr(), _is_bf16(weight, "rmsnorm"), out.data_ptr(), _is_bf16(out, "rmsnorm"), _ptr(rows), R, H, float(eps), 1, _stream()),
        "rmsnorm",
    )


def layernorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    *,
    delta: Optional[torch.Tensor] = None,
    delta2: Optional[torch.Tensor] = None,
    rows: Optional[torch.Tensor] = None,
) -> None:
    """``x += delta + delta2`` (those given; not with ``rows``), ``out = (x - mean) * rsqrt(var + eps) * weight + bias`` with the
    variance the mean of the squared deviations, all in 32-bit.  ``x`` is the fp32 residual.  With ``rows`` only the listed rows
    of x (+ the sums) are normed, into out[0..len(rows)), and x is not modified."""
    _need_cuda("layernorm", x, weight, bias, out, delta, delta2, rows)
    _need_i32("layernorm", rows)
    H = x.shape[-1]
    R = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: the residual must be contiguous fp32 and the output contiguous")
    if weight.numel() != H or bias.numel() != H or weight.dtype != bias.dtype or out.shape[-1] != H or out.shape[0] < R:
        raise KernelError("layernorm: shape mismatch, or weight and bias of different dtypes")
    for pending in (delta, delta2):
        if pending is not None and (pending.dtype != out.dtype or pending.shape != x.shape or not pending.is_contiguous()):
            raise KernelError("layernorm: a pending sum must be contiguous, in the activation dtype and of x's shape")
    fn = _fn("layernorm", "kb_layernorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(fn(x.data_ptr(), _ptr(delta), _ptr(delta2), weight.data_ptr(), bias.data_ptr(), _is_bf16(weight, "layernorm"), out.data_ptr(),
              _is_bf16(out, "layernorm"), _ptr(rows), R, H, float(eps), _stream()), "layernorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda("swiglu", gate_up, out)
    T, two_i = gate_up.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: shape or dtype mismatch")
    if not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError("swiglu: tensors must be contiguous")
    fn = _fn("elementwise", "kb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(gate_up.data_ptr(), out.data_ptr(), _is_bf16(out, "swiglu"), T, two_i // 2, _stream()), "swiglu")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda("gather_rows", src, rows, out)
    _need_i32("gather_rows", rows)
    if src.dtype != out.dtype or out.shape != (rows.numel(), src.shape[1]):
        raise KernelError("gather_rows: shape or dtype mismatch")
    if not src.is_contiguous() or not out.is_contiguous():
        raise KernelError("gather_rows: tensors must be contiguous")
    fn = _fn("elementwise", "kb_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(src.data_ptr(), rows.data_ptr(), out.data_ptr(), _is_bf16(src, "gather_rows"), rows.numel(), src.shape[1], _stream()), "gather_rows")


# ----------------------------------------------------------------------------- rope + cache write


def qk_norm_rope_kv_write(
    qkv: torch.Tensor,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    eps: float = 0.0,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    block_table: Optional[torch.Tensor] = None,
    write_from: Optional[torch.Tensor] = None,
    k_cache: Optional[torch.Tensor] = None,
    v_cache: Optional[torch.Tensor] = None,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """In place on the packed ``qkv`` rows: per-head norm of q and k (if weights
    are given), rotation (if tables are given), then k and v into the paged
    cache (if caches are given)."""
    _need_cuda("qk_norm_rope_kv_write", qkv, positions, row_ids, q_norm_weight, k_norm_weight, cos, sin, block_table, write_from, k_cache, v_cache, flag)
    _need_i32("qk_norm_rope_kv_write", positions, row_ids, block_table, write_from)
    T = qkv.shape[0]
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError(f"qk_norm_rope_kv_write: qkv must be [tokens, {width}] with unit inner stride")
    rot_half = 0
    max_pos = 0
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32:
            raise KernelError("qk_norm_rope_kv_write: cos and sin must be fp32 tables of one shape")
        if not cos.is_contiguous() or not sin.is_contiguous():
            raise KernelError("qk_norm_rope_kv_write: cos and sin must be contiguous")
        max_pos, rot_half = cos.shape
    norm_bf16 = 0
    if q_norm_weight is not None:
        if k_norm_weight is None or q_norm_weight.dtype != k_norm_weight.dtype:
            raise KernelError("qk_norm_rope_kv_write: q and k norm weights come together, in one dtype")
        norm_bf16 = _is_bf16(q_norm_weight, "qk_norm_rope_kv_write")
    page_size = num_pages = max_pages = 0
    if k_cache is not None:
        if v_cache is None or k_cache.shape != v_cache.shape or k_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv_write: caches must match each other and the qkv dtype")
        if not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise KernelError("qk_norm_rope_kv_write: caches must be contiguous")
        num_pages, page_size, kv_heads, dim = k_cache.shape
        if kv_heads != num_kv_heads or dim != head_dim:
            raise KernelError("qk_norm_rope_kv_write: cache geometry does not match the heads")
        if block_table is None or write_from is None:
            raise KernelError("qk_norm_rope_kv_write: a cache write needs block_table and write_from")
        max_pages = block_table.shape[1]
    fn = _fn(
        "rope_kv",
        "kb_qk_norm_rope_kv_write",
        [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            qkv.data_ptr(), _is_bf16(qkv, "qk_norm_rope_kv_write"), T, qkv.stride(0), num_q_heads, num_kv_heads, head_dim,
            _ptr(q_norm_weight), _ptr(k_norm_weight), norm_bf16, float(eps), _ptr(cos), _ptr(sin), rot_half, max_pos,
            positions.data_ptr(), row_ids.data_ptr(), _ptr(block_table), max_pages, _ptr(write_from),
            _ptr(k_cache), _ptr(v_cache), page_size, num_pages, _ptr(flag), _stream(),
        ),
        "qk_norm_rope_kv_write",
    )


def projection_norm_rope_write(
    packed: torch.Tensor,
    *,
    num_q_heads: int,
    num_kv_heads: int,
    head_dim: int,
    value_dim: int,
    k_offset: int,
    v_offset: int,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    q_norm_weight: Optional[torch.Tensor] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    eps: float = 0.0,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    interleaved: bool = False,
    block_table: Optional[torch.Tensor] = None,
    write_from: Optional[torch.Tensor] = None,
    k_cache: Optional[torch.Tensor] = None,
    v_cache: Optional[torch.Tensor] = None,
    flag: Optional[torch.Tensor] = None,
    per_head_norm: bool = False,
    v_cos: Optional[torch.Tensor] = None,
    v_sin: Optional[torch.Tensor] = None,
) -> None:
    """On the packed rows ``[q | ... k at k_offset ... v at v_offset ...]``: RMS norm of q over all its ``heads * dim``
    columns at once and of k over all of its (if weights of those sizes are given; with ``per_head_norm`` the statistics
    are a head's and the weights ``dim`` entries that the heads share), rotation of the first
    ``2 * cos.shape[1]`` columns of every head (pairs (i, i + half), or (2i, 2i + 1) when ``interleaved``), q back in place, k
    into ``k_cache`` [pages, page, kv_heads, dim] and v into ``v_cache`` [pages, page, kv_heads, value_dim]; with ``v_cos`` /
    ``v_sin`` (tables of as many positions) the first ``2 * v_cos.shape[1]`` columns of every value head turn too."""
    what = "projection_norm_rope_write"
    _need_cuda(what, packed, positions, row_ids, q_norm_weight, k_norm_weight, cos, sin, block_table, write_from, k_cache, v_cache, flag, v_cos, v_sin)
    _need_i32(what, positions, row_ids, block_table, write_from)
    q_size, k_size, v_size = num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * value_dim
    if packed.stride(1) != 1 or k_offset < q_size or k_offset + k_size > packed.shape[1] or v_offset < 0 or v_offset + v_size > packed.shape[1]:
        raise KernelError(f"{what}: the packed rows do not hold q, k and v where the offsets say")
    rot_half = max_pos = 0
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32 or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError(f"{what}: cos and sin must be contiguous fp32 tables of one shape")
        max_pos, rot_half = cos.shape
        if 2 * rot_half > head_dim:
            raise KernelError(f"{what}: {2 * rot_half} rotated columns in a head of {head_dim}")
    v_rot_half = 0
    if v_cos is not None:
        if v_sin is None or v_cos.shape != v_sin.shape or v_cos.dtype != torch.float32 or v_sin.dtype != torch.float32 or not (v_cos.is_contiguous() and v_sin.is_contiguous()):
            raise KernelError(f"{what}: the values' cos and sin must be contiguous fp32 tables of one shape")
        if cos is not None and v_cos.shape[0] != max_pos:
            raise KernelError(f"{what}: the values' table must hold as many positions as the keys'")
        max_pos, v_rot_half = v_cos.shape
        if 2 * v_rot_half > value_dim:
            raise KernelError(f"{what}: {2 * v_rot_half} rotated columns in a value head of {value_dim}")
    w_bf16 = 0
    if q_norm_weight is not None:
        want_q, want_k = (head_dim, head_dim) if per_head_norm else (q_size, k_size)
        if num_kv_heads == 0:  # queries alone: the key weight is not used
            want_k = k_norm_weight.numel() if k_norm_weight is not None else 0
        if k_norm_weight is None or q_norm_weight.dtype != k_norm_weight.dtype or q_norm_weight.numel() != want_q or k_norm_weight.numel() != want_k \
                or not (q_norm_weight.is_contiguous() and k_norm_weight.is_contiguous()):
            raise KernelError(f"{what}: q and k norm weights come together, in one dtype, one entry a projection column (a head's column with per_head_norm)")
        w_bf16 = _is_bf16(q_norm_weight, what)
    page_size = num_pages = max_pages = num_rows = 0
    if k_cache is not None:
        if v_cache is None or k_cache.dtype != packed.dtype or v_cache.dtype != packed.dtype or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise KernelError(f"{what}: contiguous caches in the activations' dtype")
        num_pages, page_size = k_cache.shape[:2]
        if tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) or tuple(v_cache.shape) != (num_pages, page_size, num_kv_heads, value_dim):
            raise KernelError(f"{what}: cache geometry does not match the heads")
        if block_table is None:
            raise KernelError(f"{what}: a cache write needs the block table")
        num_rows, max_pages = block_table.shape
    fn = _fn("projection_rope", "kb_projection_norm_rope_write",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_int,
              c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(packed.data_ptr(), packed.stride(0), _is_bf16(packed, what), packed.shape[0], int(k_offset), int(v_offset), num_q_heads, num_kv_heads,
              head_dim, value_dim, _ptr(q_norm_weight), _ptr(k_norm_weight), w_bf16, float(eps), 1 if per_head_norm else 0, _ptr(cos), _ptr(sin),
              rot_half, max_pos, 1 if interleaved else 0, _ptr(v_cos), _ptr(v_sin), v_rot_half, positions.data_ptr(), row_ids.data_ptr(), _ptr(block_table), max_pages, _ptr(write_from), _ptr(k_cache),
              _ptr(v_cache), page_size, num_pages, num_rows, _ptr(flag), _stream()), what)


def rotate_heads(x: torch.Tensor, *, heads: int, head_dim: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
                 interleaved: bool = False, inverse: bool = False, flag: Optional[torch.Tensor] = None) -> None:
    """In place on ``x`` [tokens, heads * head_dim]: the first ``2 * cos.shape[1]`` columns of every head turn by the
    token's position (``inverse``: by minus it), pairs (i, i + half) or (2i, 2i + 1) when ``interleaved``; 32-bit arithmetic."""
    what = "rotate_heads"
    _need_cuda(what, x, cos, sin, positions, flag)
    _need_i32(what, positions)
    if x.stride(1) != 1 or x.shape[1] < heads * head_dim or positions.numel() != x.shape[0]:
        raise KernelError(f"{what}: rows of at least heads * head_dim columns with unit inner stride, a position a row")
    if cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32 or not (cos.is_contiguous() and sin.is_contiguous()):
        raise KernelError(f"{what}: cos and sin must be contiguous fp32 tables of one shape")
    max_pos, rot_half = cos.shape
    if 2 * rot_half > head_dim:
        raise KernelError(f"{what}: {2 * rot_half} rotated columns in a head of {head_dim}")
    fn = _fn("projection_rope", "kb_rotate_heads",
             [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(x.data_ptr(), x.stride(0), _is_bf16(x, what), x.shape[0], heads, head_dim, cos.data_ptr(), sin.data_ptr(), rot_half, max_pos,
              1 if interleaved else 0, 1 if inverse else 0, positions.data_ptr(), _ptr(flag), _stream()), what)


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float, out: torch.Tensor) -> None:
    """``out = scale_a * a + scale_b * b``, formed in 32-bit with one rounding."""
    _need_cuda("scaled_sum", a, b, out)
    if a.shape != b.shape or a.shape != out.shape or a.dtype != b.dtype or a.dtype != out.dtype or not (a.is_contiguous() and b.is_contiguous() and out.is_contiguous()):
        raise KernelError("scaled_sum: three contiguous tensors of one shape and dtype")
    fn = _fn("elementwise", "kb_scaled_sum", [c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, ctypes.c_longlong, c_void_p])
    _check(fn(a.data_ptr(), float(scale_a), b.data_ptr(), float(scale_b), out.data_ptr(), _is_bf16(a, "scaled_sum"), a.numel(), _stream()), "scaled_sum")


# ----------------------------------------------------------------------------- attention


def paged_attention_generic(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    flag: Optional[torch.Tensor] = None,
    sinks: Optional[torch.Tensor] = None,
    value_dim: Optional[int] = None,
    out_head_stride: Optional[int] = None,
) -> None:
    """fp32-arithmetic attention of every token in ``q`` over its request's pages.

    ``q``: [tokens, >= heads*dim] (a view into the packed qkv rows is fine);
    ``out``: [tokens, heads*out_head_stride].  ``sinks``: fp32 [heads], a logit a head that joins the
    softmax's denominator (a term exp(sink) there and nothing else).  ``value_dim`` (default: dim): how many
    leading columns of a value row are used; with ``v_cache`` the key cache itself, a row's first
    ``value_dim`` columns are its value.  ``out_head_stride`` (default: value_dim): where head h's
    output starts in its token's row, h * out_head_stride (the columns behind value_dim stay as they are).
    """
    _need_cuda("paged_attention_generic", q, out, k_cache, v_cache, positions, row_ids, block_table, flag, sinks)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_q_heads or not sinks.is_contiguous()):
        raise KernelError("paged_attention_generic: sinks must be contiguous fp32, one a query head")
    _need_i32("paged_attention_generic", positions, row_ids, block_table)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if q.dtype != k_cache.dtype or out.dtype != q.dtype or v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention_generic: dtype or cache shape mismatch")
    if q.stride(1) != 1 or out.stride(1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("paged_attention_generic: inner strides must be 1 and caches contiguous")
    if head_dim > 1024:
        raise KernelError(f"paged_attention_generic: head_dim {head_dim} > 1024 is not supported")
    if num_q_heads % num_kv_heads:
        raise KernelError("paged_attention_generic: query heads must be a multiple of KV heads")
    T = q.shape[0]
    fn = _fn(
        "attention_generic",
        "kb_paged_attention_generic",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    )
    value_dim = int(head_dim if value_dim is None else value_dim)
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            _is_bf16(q, "paged_attention_generic"), positions.data_ptr(), row_ids.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], T, num_q_heads, num_kv_heads, head_dim, page_size, num_pages, float(scale),
            int(window), _ptr(sinks), value_dim, int(value_dim if out_head_stride is None else out_head_stride), _ptr(flag), _stream(),
        ),
        "paged_attention_generic",
    )


def paged_kv_write(
    packed: torch.Tensor,
    k_offset: int,
    v_offset: int,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    block_table: torch.Tensor,
    write_from: Optional[torch.Tensor] = None,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """Columns of a step's packed rows into the pages: a key row (all key/value heads side by side)
    from ``k_offset`` on, a value row from ``v_offset`` on; the two may differ in width."""
    _need_cuda("paged_kv_write", packed, k_cache, v_cache, positions, row_ids, block_table, write_from, flag)
    _need_i32("paged_kv_write", positions, row_ids, block_table, write_from)
    num_pages, page_size = k_cache.shape[:2]
    k_width = k_cache.shape[2] * k_cache.shape[3]
    v_width = v_cache.shape[2] * v_cache.shape[3]
    if packed.dtype != k_cache.dtype or v_cache.dtype != k_cache.dtype or packed.stride(1) != 1 or v_cache.shape[:2] != k_cache.shape[:2]:
        raise KernelError("paged_kv_write: one dtype, unit inner stride, caches of one page geometry")
    if not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("paged_kv_write: caches must be contiguous")
    if min(k_offset, v_offset) < 0 or k_offset + k_width > packed.shape[1] or v_offset + v_width > packed.shape[1]:
        raise KernelError("paged_kv_write: the key or value columns lie outside the packed rows")
    fn = _fn("diff_attention", "kb_paged_kv_write", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(fn(packed.data_ptr(), packed.stride(0), _is_bf16(packed, "paged_kv_write"), packed.shape[0], int(k_offset), k_width, int(v_offset),
              v_width, k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(), row_ids.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], _ptr(write_from), page_size, num_pages, _ptr(flag), _stream()), "paged_kv_write")


def _check_diff_attention(what: str, q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_q_heads: int,
                          maps: int) -> tuple[int, int, int, int, int]:
    num_pages, page_size, num_kv_heads, key_width = k_cache.shape
    if maps not in (1, 2) or key_width % maps:
        raise KernelError(f"{what}: {maps} maps over key rows of {key_width}")
    dim, vdim = key_width // maps, v_cache.shape[3]
    if v_cache.shape[:3] != k_cache.shape[:3] or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError(f"{what}: caches must be contiguous and of one page geometry")
    if q.dtype != k_cache.dtype or out.dtype != q.dtype or v_cache.dtype != q.dtype or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"{what}: one dtype and unit inner strides")
    if num_q_heads % num_kv_heads or q.shape[1] < num_q_heads * key_width or out.shape[1] < num_q_heads * vdim:
        raise KernelError(f"{what}: heads or widths do not fit")
    return num_pages, page_size, num_kv_heads, dim, vdim


def _check_sinks_gate(what: str, q: torch.Tensor, out: torch.Tensor, num_q_heads: int, sinks: Optional[torch.Tensor],
                      gate: Optional[torch.Tensor]) -> None:
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_q_heads or not sinks.is_contiguous()):
        raise KernelError(f"{what}: sinks must be contiguous fp32, one a query head")
    if gate is not None and (gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != q.shape[0] or gate.shape[1] < out.shape[1]):
        raise KernelError(f"{what}: the gate must hold a column for every output column, in the activations' dtype")


def diff_attention_generic(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    block_table: torch.Tensor,
    num_q_heads: int,
    maps: int,
    scale: float,
    softcap: float = 0.0,
    window: int = 0,
    lam: float = 0.0,
    head_norm_eps: Optional[float] = None,
    out_scale: float = 1.0,
    flag: Optional[torch.Tensor] = None,
    sinks: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
) -> None:
    """Attention with ``maps`` softmax maps a head over the same values, every token of the step, in 32-bit
    arithmetic.  ``q``: [tokens, >= heads * maps * dim], a head's maps side by side; the key cache
    [pages, page, kv_heads, maps * dim] the same way; values [pages, page, kv_heads, vdim].  Scores
    q.k * scale, capped as softcap * tanh(s / softcap) when softcap > 0; a token sees itself and the
    ``window - 1`` before it (0: all).  o = a_1 - lam * a_2; with ``head_norm_eps`` each head's o is divided
    by its root mean square (eps inside the root) and multiplied by ``out_scale``.  ``out``: [tokens, heads * vdim].
    ``sinks``: fp32 [heads], a logit a head that joins every map's denominator (a term exp(sink) there and nothing else).
    ``gate``: [tokens, >= heads * vdim] in the activations' dtype (a view into the packed rows is fine): the output
    is multiplied by sigmoid(gate), last of all."""
    what = "diff_attention_generic"
    _need_cuda(what, q, out, k_cache, v_cache, positions, row_ids, block_table, flag, sinks, gate)
    _check_sinks_gate(what, q, out, num_q_heads, sinks, gate)
    _need_i32(what, positions, row_ids, block_table)
    num_pages, page_size, num_kv_heads, dim, vdim = _check_diff_attention(what, q, out, k_cache, v_cache, num_q_heads, maps)
    if dim > 256 or vdim > 256:
        raise KernelError(f"{what}: key width {dim} or value width {vdim} > 256 is not supported")
    fn = _fn("diff_attention", "kb_diff_attention_generic",
             [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
              c_int, c_int, c_int, c_float, c_float, c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), _is_bf16(q, what),
              positions.data_ptr(), row_ids.data_ptr(), block_table.data_ptr(), block_table.shape[1], q.shape[0], num_q_heads, num_kv_heads,
              int(maps), dim, vdim, page_size, num_pages, float(scale), float(softcap), int(window), float(lam),
              0 if head_norm_eps is None else 1, float(head_norm_eps or 0.0), float(out_scale), _ptr(sinks), _ptr(gate),
              gate.stride(0) if gate is not None else 0, _ptr(flag), _stream()), what)


DIFF_ATTENTION_TILE = 64  # queries a tile of the tensor-core kernel for prompt portions


DIFF_ATTENTION_MMA_MAPS = (2,)  # how many softmax maps a head the tensor-core kernel is built for


def diff_attention_mma_supported(head_dim: int, value_dim: int, num_q_heads: int, num_kv_heads: int, maps: int = 2) -> bool:
    """Sizes the tensor-core kernel of differential attention takes (bfloat16; key and value widths multiples of 16
    up to 128, up to 64 query heads a key/value head); others use the 32-bit-arithmetic kernel."""
    return (maps in DIFF_ATTENTION_MMA_MAPS and head_dim % 16 == 0 and 16 <= head_dim <= 128 and value_dim % 16 == 0 and 16 <= value_dim <= 128
            and num_kv_heads >= 1 and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 64)


def diff_attention_mma(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    ctx: object,
    block_table: torch.Tensor,
    num_q_heads: int,
    maps: int,
    scale: float,
    softcap: float = 0.0,
    window: int = 0,
    lam: float = 0.0,
    head_norm_eps: Optional[float] = None,
    out_scale: float = 1.0,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """``diff_attention_generic`` on tensor cores (bfloat16, two maps): the step's prompt portions go tile by
    tile (``ctx.tiles[DIFF_ATTENTION_TILE]``), its single-token rows a key/value head at a time
    (``ctx.decode_rows``), in two launches of one kernel.  ``ctx``: the step's description."""
    what = "diff_attention_mma"
    _need_cuda(what, q, out, k_cache, v_cache, block_table, flag)
    _need_i32(what, block_table)
    num_pages, page_size, num_kv_heads, dim, vdim = _check_diff_attention(what, q, out, k_cache, v_cache, num_q_heads, maps)
    if maps != 2 or q.dtype != torch.bfloat16 or not diff_attention_mma_supported(dim, vdim, num_q_heads, num_kv_heads):
        raise KernelError(f"{what}: bfloat16, two maps, sizes as diff_attention_mma_supported says")
    fn = _fn("diff_attention_mma", "kb_diff_attention_mma",
             [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_float, c_int, c_float, c_float, c_void_p, c_void_p])

    def launch(rows: torch.Tensor, second: torch.Tensor, count: int, single: int) -> None:
        _check(fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), ctx.qo_indptr.data_ptr(),
                  ctx.seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], rows.data_ptr(), second.data_ptr(), int(count), single,
                  num_q_heads, num_kv_heads, dim, vdim, page_size, num_pages, float(scale), float(softcap), int(window), float(lam),
                  0 if head_norm_eps is None else 1, float(head_norm_eps or 0.0), float(out_scale), _ptr(flag), _stream()), what)

    num_tiles, tile_rows, tile_starts = ctx.tiles[DIFF_ATTENTION_TILE]
    if num_tiles:
        launch(tile_rows, tile_starts, num_tiles, 0)
    if ctx.num_decode_rows:
        launch(ctx.decode_rows, ctx.decode_tokens, ctx.num_decode_rows, 1)


ATTENTION_MMA_SINKS = True  # the tensor-core attention kernels take sink logits, in the step that divides a row's result

DECODE_SPLIT = 128  # keys per split of the split-KV kernel (csrc/attention_mma.cu: DEC_SPLIT)


def attention_mma_supported(head_dim: int, num_q_heads: int, num_kv_heads: int) -> bool:
    """Sizes the tensor-core attention kernels take; others use the generic kernel."""
    return (
        head_dim % 16 == 0
        and 16 <= head_dim <= 256
        and num_kv_heads >= 1
        and num_q_heads % num_kv_heads == 0
        and num_q_heads // num_kv_heads <= 16
    )


def attention_prefill_tile_rows(head_dim: int) -> int:
    """Queries per tile the prefill attention kernel expects in its tile list
    (csrc/attention_mma.cuh: prefill_tile_rows)."""
    return 128 if head_dim <= 128 else 64


def attention_prefill_wide_tile_rows(head_dim: int) -> Optional[int]:
    """Queries per tile of the second list the prefill attention takes for long portions (the kernel
    that walks two 128-query tiles a block, csrc/attention_prefill_tc5.cu), or None for head sizes
    it does not cover."""
    return 256 if head_dim == 128 else None


def _check_sinks(what: str, num_q_heads: int, sinks: Optional[torch.Tensor]) -> None:
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_q_heads or not sinks.is_contiguous()):
        raise KernelError(f"{what}: sinks must be contiguous fp32, one a query head")


def _check_mma_gate(what: str, q: torch.Tensor, gate: Optional[torch.Tensor]) -> None:
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.dim() != 2 or gate.shape[0] != q.shape[0] or gate.stride(1) != 1
                             or gate.data_ptr() % 4 or gate.stride(0) % 2):
        raise KernelError(f"{what}: the gate must be bf16, a row a token, inner stride 1, rows aligned to 4 bytes")


def _check_mma_common(what: str, q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError(f"{what}: bf16 only")
    if k_cache.shape != v_cache.shape or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError(f"{what}: caches must be contiguous and of one shape")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"{what}: inner strides must be 1")
    if q.data_ptr() % 16 or (q.stride(0) * 2) % 16 or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16:
        raise KernelError(f"{what}: q rows and caches must be 16-byte aligned")


def attention_prefill_mma(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    qo_indptr: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    tile_rows: torch.Tensor,
    tile_starts: torch.Tensor,
    num_tiles: int,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    flag: Optional[torch.Tensor] = None,
    max_seq_len: int = 0,
    workspace: object = None,
    num_splits: Optional[int] = None,
    wide_tiles: Optional[tuple[int, torch.Tensor, torch.Tensor]] = None,
    two_tiles: Optional[bool] = None,
    sinks: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
) -> None:
    """Flash attention over query tiles (``attention_prefill_tile_rows`` queries each) of
    rows with several tokens (bf16).

    With ``workspace`` and ``max_seq_len`` (a bound on the rows' lengths) given, the tcgen05 kernel
    may share a tile's keys among several blocks when the tiles alone would leave most of the device
    idle (a short portion of a long prompt); their results meet in fp32 scratch of the workspace and a
    second kernel combines them.  ``num_splits`` overrides the choice (tests).

    ``wide_tiles`` (count, rows, starts of tiles of ``attention_prefill_wide_tile_rows`` queries over the
    same portions): long portions of head size 128 go to the kernel that takes two query tiles a block
    when its grid makes two waves or more; ``two_tiles`` overrides that choice (tests).

    ``sinks``: fp32 [heads], a logit a head whose exp joins the softmax's denominator.  ``gate``: bf16 [tokens, >= heads *
    head_dim], columns laid out as ``out``'s; the result is multiplied by its sigmoid.  Every kernel here takes both, in its
    last step (the tcgen05 kernels a gate whose rows are whole 16-byte groups)."""
    what = "attention_prefill_mma"
    _need_cuda(what, q, out, k_cache, v_cache, qo_indptr, seq_lens, block_table, tile_rows, tile_starts, sinks, gate)
    _check_sinks(what, num_q_heads, sinks)
    _check_mma_gate(what, q, gate)
    _need_i32(what, qo_indptr, seq_lens, block_table, tile_rows, tile_starts)
    _check_mma_common(what, q, out, k_cache, v_cache)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if not attention_mma_supported(head_dim, num_q_heads, num_kv_heads):
        raise KernelError(f"{what}: head_dim {head_dim} with {num_q_heads}/{num_kv_heads} heads is not supported")
    gate_by_16 = gate is None or (gate.stride(0) % 8 == 0 and gate.data_ptr() % 16 == 0)  # the tcgen05 kernel reads it in 16-byte groups
    if gate_by_16 and _prefill_tc5_ok(q, out, k_cache, v_cache):  # tcgen05 + TMA: S and O in tensor memory
        fn = _fn(
            "attention_prefill_tc5",
            "kb_attention_prefill_tc5",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        )
        merged = bool(_fn("attention_prefill_tc5", "kb_attention_prefill_tc5_merged", [c_int, c_int])(head_dim, page_size))
        splits = 1
        if workspace is not None and num_tiles > 0:
            if num_splits is not None:
                splits = int(num_splits)
            elif max_seq_len > 0:
                longest = min(int(max_seq_len), int(window) + 128) if window > 0 else int(max_seq_len)
                splits = _fn("attention_prefill_tc5", "kb_attention_prefill_tc5_splits", [c_int, c_int, c_int, c_int])(head_dim, num_q_heads, int(num_tiles), longest)
        use_two = False
        if wide_tiles is not None and wide_tiles[0] > 0 and head_dim == 128 and splits == 1:
            if two_tiles is None:
                use_two = bool(_fn("attention_prefill_tc5", "kb_attention_prefill_tc5_two_tiles", [c_int] * 5)(
                    head_dim, num_q_heads, int(wide_tiles[0]), page_size, int(max_seq_len)))
            else:
                use_two = bool(two_tiles)
            if use_two:
                _need_cuda(what, wide_tiles[1], wide_tiles[2])
                _need_i32(what, wide_tiles[1], wide_tiles[2])
        part_o = part_ml = None
        if splits > 1:
            slots = splits * int(num_tiles) * 128 * num_q_heads
            part_o = workspace.flat("attn.prefill.part_o", slots * head_dim, torch.float32)
            part_ml = workspace.flat("attn.prefill.part_ml", slots * 2, torch.float32)
        _check(
            fn(
                _tensor_map(q, 128), _cache_map(k_cache), _cache_map(v_cache, bands=merged), out.data_ptr(), out.stride(0),
                qo_indptr.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                tile_rows.data_ptr(), tile_starts.data_ptr(), int(num_tiles), num_q_heads, num_kv_heads, head_dim,
                page_size, num_pages, float(scale), int(window), splits, _ptr(part_o), _ptr(part_ml),
                wide_tiles[1].data_ptr() if use_two else None, wide_tiles[2].data_ptr() if use_two else None,
                int(wide_tiles[0]) if use_two else 0, 1 if use_two else 0, _ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0,
                _ptr(flag), _stream(),
            ),
            what,
            launches=2 if splits > 1 else 1,
        )
        return
    fn = _fn(
        "attention_mma",
        "kb_attention_prefill_mma",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            qo_indptr.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1],
            tile_rows.data_ptr(), tile_starts.data_ptr(), int(num_tiles), num_q_heads, num_kv_heads, head_dim,
            page_size, num_pages, float(scale), int(window), _ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(flag), _stream(),
        ),
        what,
    )


def attention_decode_mma(
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    decode_rows: torch.Tensor,
    decode_tokens: torch.Tensor,
    num_rows: int,
    max_seq_len: int,
    num_q_heads: int,
    scale: float,
    window: int = 0,
    workspace: object,
    flag: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    sinks: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
) -> None:
    """Split-KV attention of rows that carry one token (bf16), then the merge.

    ``sinks``: fp32 [heads], a logit a head whose exp joins the softmax's denominator.  ``gate``: bf16 [tokens, >= heads *
    head_dim]; the result is multiplied by its sigmoid.  Both act where a row's result is divided (the merge, or the TMA-fed
    kernel itself when it runs one split).

    ``max_seq_len`` bounds every row's length; it sizes the grid and the scratch
    (``workspace.flat`` gives persistent fp32 buffers).  ``num_splits`` overrides the
    number of splits of the TMA-fed kernel (tests use it to make a block stream many tiles).
    """
    what = "attention_decode_mma"
    _need_cuda(what, q, out, k_cache, v_cache, seq_lens, block_table, decode_rows, decode_tokens, sinks, gate)
    _check_sinks(what, num_q_heads, sinks)
    _check_mma_gate(what, q, gate)
    _need_i32(what, seq_lens, block_table, decode_rows, decode_tokens)
    _check_mma_common(what, q, out, k_cache, v_cache)
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    if not attention_mma_supported(head_dim, num_q_heads, num_kv_heads):
        raise KernelError(f"{what}: head_dim {head_dim} with {num_q_heads}/{num_kv_heads} heads is not supported")
    if _decode_tma_ok(k_cache, v_cache):  # tiled TMA copies of whole runs of key rows, streamed through a ring
        splits_fn = _fn("attention_decode_tma", "kb_attention_decode_tma_splits", [c_int, c_int, c_int, c_int])
        if num_splits is None:
            num_splits = splits_fn(int(num_rows), num_kv_heads, head_dim, max(1, int(max_seq_len)))
        if num_splits < 1:
            raise KernelError(f"{what}: choosing the number of splits failed with code {num_splits}")
        part_o = workspace.flat("attn.part_o", num_rows * num_q_heads * num_splits * head_dim, torch.float32)
        part_ml = workspace.flat("attn.part_ml", num_rows * num_q_heads * num_splits * 2, torch.float32)
        fn = _fn(
            "attention_decode_tma",
            "kb_attention_decode_tma",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
        )
        joined = _joined_cache_map(k_cache, v_cache)  # keys and values in one copy where the cache allows
        map_k = joined or _cache_map(k_cache, bands=True)
        map_v = joined or _cache_map(v_cache, bands=True)
        _check(
            fn(
                map_k, map_v, q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
                seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], decode_rows.data_ptr(),
                decode_tokens.data_ptr(), int(num_rows), num_q_heads, num_kv_heads, head_dim, page_size, num_pages,
                float(scale), int(window), num_splits, part_o.data_ptr(), part_ml.data_ptr(), 1 if joined else 0, _ptr(sinks), _ptr(gate),
                gate.stride(0) if gate is not None else 0, _ptr(flag), _stream(),
            ),
            what,
            launches=_fn("attention_decode_tma", "kb_attention_decode_tma_launches", [c_int])(num_splits),
        )
        return
    num_splits = max(1, -(-int(max_seq_len) // DECODE_SPLIT))
    part_o = workspace.flat("attn.part_o", num_rows * num_q_heads * num_splits * head_dim, torch.float32)
    part_ml = workspace.flat("attn.part_ml", num_rows * num_q_heads * num_splits * 2, torch.float32)
    fn = _fn(
        "attention_mma",
        "kb_attention_decode_mma",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(
            q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            seq_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], decode_rows.data_ptr(),
            decode_tokens.data_ptr(), int(num_rows), num_q_heads, num_kv_heads, head_dim, page_size, num_pages,
            float(scale), int(window), num_splits, part_o.data_ptr(), part_ml.data_ptr(), _ptr(sinks), _ptr(gate),
            gate.stride(0) if gate is not None else 0, _ptr(flag), _stream(),
        ),
        what,
        launches=2,
    )


def _prefill_tc5_ok(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> bool:
    head_dim = k_cache.shape[3]
    return (
        head_dim in (64, 128)
        and _decode_tma_ok(k_cache, v_cache)
        and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
        and out.stride(1) == 1 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
    )


def _decode_tma_ok(k_cache: torch.Tensor, v_cache: torch.Tensor) -> bool:
    num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
    return (
        head_dim in (64, 128, 192, 256)
        and page_size >= 8 and page_size & (page_size - 1) == 0
        and all(t.stride(3) == 1 and all(t.stride(i) % 8 == 0 for i in range(3)) and t.data_ptr() % 16 == 0 for t in (k_cache, v_cache))
    )


def _cache_map(cache: torch.Tensor, bands: bool = False) -> int:
    """Host address of a cached TMA descriptor of one layer's key (or value) pages: boxes of one
    64-column band (the prefill kernel's), or with ``bands`` of every band at once (the decode kernel's)."""
    key = ("cache", cache.data_ptr(), tuple(cache.shape), tuple(cache.stride()), bands)
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        ll = ctypes.c_longlong
        fn = _fn("attention_decode_tma", "kb_attention_encode_cache_map", [c_void_p, c_void_p, ll, c_int, c_int, c_int, ll, ll, ll, c_int])
        num_pages, page_size, num_kv_heads, head_dim = cache.shape
        code = fn(address, cache.data_ptr(), num_pages, page_size, num_kv_heads, head_dim, cache.stride(0), cache.stride(1), cache.stride(2), 1 if bands else 0)
        if code != 0:
            raise KernelError(f"tensor map encoding of the cache failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


def _joined_cache_map(k_cache: torch.Tensor, v_cache: torch.Tensor) -> int:
    """Host address of a cached TMA descriptor over the keys AND the values of one layer's pages, or 0
    where there is none: head size 64, and values that lie a fixed distance behind the keys with the same
    shape and strides (the cache storage allocates them so).  One copy then brings a run of key rows and
    the value rows of the same positions: at 128 bytes a row the decode kernel is bound by how many
    copies an SM can issue, not by their bytes."""
    if k_cache.shape[3] != 64 or k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        return 0
    gap_bytes = v_cache.data_ptr() - k_cache.data_ptr()
    if gap_bytes <= 0 or gap_bytes % 16 != 0 or gap_bytes >= 1 << 40:
        return 0
    key = ("joined", k_cache.data_ptr(), gap_bytes, tuple(k_cache.shape), tuple(k_cache.stride()))
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        ll = ctypes.c_longlong
        fn = _fn("attention_decode_tma", "kb_attention_encode_joined_map", [c_void_p, c_void_p, ll, ll, c_int, c_int, c_int, ll, ll, ll])
        num_pages, page_size, num_kv_heads, head_dim = k_cache.shape
        code = fn(address, k_cache.data_ptr(), gap_bytes // 2, num_pages, page_size, num_kv_heads, head_dim,
                  k_cache.stride(0), k_cache.stride(1), k_cache.stride(2))
        if code != 0:
            raise KernelError(f"tensor map encoding of the cache's keys and values failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


# ----------------------------------------------------------------------------- matrix products


def linear(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor], *,
           fold: Optional["ResidualNorm"] = None) -> None:
    """out = x @ weight.T (+ bias).

    float32: this package's own FMA kernel (true 32-bit, fixed summation order).
    bfloat16: the weight-streaming kernel up to 8 rows, else the library product (cuBLAS
    through torch), as the reference's ``F.linear`` is (kairyu/models/packed_linear.py:217);
    accumulation is fp32, ``out`` may be bfloat16 or float32.

    ``x`` may be a :class:`PreNormed` (its rows are scaled in the epilogue) and ``fold`` a
    :class:`ResidualNorm` (the result goes into the residual and towards the next norm instead
    of ``out``); both need the weight-streaming kernel (``fused_norm_shapes_ok``).
    """
    scale_by = x if isinstance(x, PreNormed) else None
    if scale_by is not None or fold is not None:
        values = scale_by.values if scale_by is not None else x
        _need_cuda("linear", values, weight, bias, out)
        if fold is None and (out is None or out.shape != (values.shape[0], weight.shape[0])):
            raise KernelError("linear: out does not fit")
        probe = out if out is not None else fold.values
        if values.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != values.shape[1] or not _skinny_ok(values, weight, bias, probe):
            raise KernelError("linear: a fused norm needs bf16 operands that the weight-streaming kernel takes (at most 16 rows, sizes in steps of 16)")
        if fold is not None and (fold.residual.dtype != torch.float32 or fold.residual.shape != (values.shape[0], weight.shape[0])
                                 or fold.values.shape != fold.residual.shape or fold.values.dtype != torch.bfloat16
                                 or fold.sumsq.numel() < 16 * skinny_blocks(values.shape[0], weight.shape[0])):
            raise KernelError("linear: the residual, values and partial sums of a folded norm do not fit the product")
        _gemm_skinny(values, weight, bias, out, gated=False, scale_by=scale_by, fold=fold)
        return
    _need_cuda("linear", x, weight, bias, out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path needs fp32 weights and output")
        if bias is not None and bias.dtype != torch.float32:
            raise KernelError("linear: the 32-bit path needs an fp32 bias")
        if x.stride(1) != 1 or weight.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear: inner strides must be 1")
        fn = _fn("gemm_f32", "kb_gemm_f32", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), M, N, K, _stream()), "linear")
        return
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtypes {x.dtype} / {weight.dtype} are not supported")
    if M == 0:
        return
    if few_rows(M, max(K, N)) and _skinny_ok(x, weight, bias, out):
        _gemm_skinny(x, weight, bias, out, gated=False)
        return
    if out.dtype == torch.bfloat16:
        if bias is not None:
            torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            out.add_(bias)
    else:
        raise KernelError(f"linear: output dtype {out.dtype} is not supported")


SKINNY_MAX_ROWS = 16  # token rows the weight-streaming product takes (csrc/gemm_skinny.cu)
# ... and up to which the engine uses it.  With two token tiles (9 to 16 rows) the step is 5-7 % faster
# on the library product (plain) and the tcgen05 product (gated) with the norms and the position
# encoding as kernels of their own (measured at 9, 12 and 16 rows; a two-tile variant without
# register spills, one k step a batch, was no faster).
SKINNY_FAST_ROWS = 8
# A narrow model is the exception: at width 2,048 a layer's products are 8 to 67 MB and take 5-15 us each, so
# the three launches a layer that the fusions save weigh more than the second token tile costs (16 layers of
# that width, 12 rows: 1.08 -> 0.96 ms a step; 16 rows: 1.14 -> 1.04).
SKINNY_NARROW_WIDTH = 2048


def few_rows(rows: int, width: Optional[int] = None) -> bool:
    """Whether a step of this many token rows runs on the weight-streaming product and its fusions;
    ``width``: the larger side of the product, or the residual's width for a layer's chain of products."""
    if 1 <= rows <= SKINNY_FAST_ROWS:
        return True
    return width is not None and 1 <= rows <= SKINNY_MAX_ROWS and width <= SKINNY_NARROW_WIDTH


def _skinny_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        M <= SKINNY_MAX_ROWS
        and K % 16 == 0
        and x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
        and x.stride(0) % 16 == 0 and weight.stride(0) % 16 == 0
        and x.data_ptr() % 32 == 0 and weight.data_ptr() % 32 == 0
        and out.dtype in (torch.bfloat16, torch.float32)
        and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))
    )


def _gemm_skinny(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor], *, gated: bool,
                 scale_by: Optional["PreNormed"] = None, fold: Optional["ResidualNorm"] = None) -> None:
    M, K = x.shape
    N = weight.shape[0]
    if scale_by is None and fold is None:
        fn = _fn("gemm_skinny", "kb_gemm_skinny", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
        _check(
            fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(),
               1 if out.dtype == torch.float32 else 0, out.stride(0), M, N, K, 1 if gated else 0, _stream()),
            "gemm_skinny",
        )
        return
    fn = _fn(
        "gemm_skinny", "kb_gemm_skinny_fused",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
         c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), _ptr(out),
           1 if out is not None and out.dtype == torch.float32 else 0, out.stride(0) if out is not None else 0, M, N, K, 1 if gated else 0,
           _ptr(scale_by.sumsq) if scale_by is not None else None, scale_by.sumsq.shape[0] if scale_by is not None else 0,
           scale_by.hidden if scale_by is not None else 0, float(scale_by.eps) if scale_by is not None else 0.0,
           fold.residual.data_ptr() if fold is not None else None, fold.residual.stride(0) if fold is not None else 0,
           fold.weight.data_ptr() if fold is not None else None, 1 if fold is not None and fold.weight.dtype == torch.bfloat16 else 0,
           fold.values.data_ptr() if fold is not None else None, fold.values.stride(0) if fold is not None else 0,
           fold.sumsq.data_ptr() if fold is not None else None, _stream()),
        "gemm_skinny",
    )


def linear_weight_streaming(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, gated: bool = False) -> None:
    """The weight-streaming kernel itself, for up to 16 bf16 rows (``linear`` and ``linear_swiglu``
    choose it up to ``SKINNY_FAST_ROWS``); ``gated``: out = silu(x.Wg^T) * (x.Wu^T)."""
    _need_cuda("linear_weight_streaming", x, weight, bias, out)
    n_out = weight.shape[0] // 2 if gated else weight.shape[0]
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != x.shape[1] or out.shape != (x.shape[0], n_out) or not _skinny_ok(x, weight, bias, out):
        raise KernelError("linear_weight_streaming: needs bf16 operands, at most 16 rows, sizes in steps of 16, 32-byte aligned rows")
    _gemm_skinny(x, weight, bias, out, gated=gated)


def linear_rope_ok(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, num_q_heads: int,
                   num_kv_heads: int, head_dim: int, cos: Optional[torch.Tensor], k_cache: Optional[torch.Tensor]) -> bool:
    """Whether ``linear_rope`` takes this q | k | v product: bf16, at most 16 rows (the weight-streaming
    kernel), a rotation over the whole head, bf16 caches."""
    values = x.values if isinstance(x, PreNormed) else x
    if cos is None or not values.is_cuda or values.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        return False
    if head_dim % 16 or cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] * 2 != head_dim or not cos.is_contiguous():
        return False
    if weight.shape[0] != (num_q_heads + 2 * num_kv_heads) * head_dim or out.shape != (values.shape[0], weight.shape[0]):
        return False
    if k_cache is not None and (k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous()):
        return False
    return _skinny_ok(values, weight, bias, out)


def linear_rope(x, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, num_q_heads: int, num_kv_heads: int,
                head_dim: int, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, row_ids: torch.Tensor,
                block_table: Optional[torch.Tensor], write_from: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                v_cache: Optional[torch.Tensor], flag: Optional[torch.Tensor] = None) -> None:
    """The q | k | v product of attention for a few rows with the position encoding and the cache
    write in its epilogue (csrc/gemm_skinny.cu, rope): the q columns of ``out`` get the rotated
    queries; rotated keys and the values go straight to their cache pages (``out``'s k and v
    columns are left as they were).  ``x`` may be a :class:`PreNormed`.  Same arithmetic as
    ``linear`` then ``qk_norm_rope_kv_write`` without per-head norms, except that the product is
    not rounded to bf16 before it is rotated."""
    scale_by = x if isinstance(x, PreNormed) else None
    values = scale_by.values if scale_by is not None else x
    _need_cuda("linear_rope", values, weight, bias, out, cos, sin, positions, row_ids, block_table, write_from, k_cache, v_cache, flag)
    _need_i32("linear_rope", positions, row_ids, *(t for t in (block_table, write_from) if t is not None))
    if not linear_rope_ok(x, weight, bias, out, num_q_heads=num_q_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, cos=cos, k_cache=k_cache):
        raise KernelError("linear_rope: operands the fused kernel does not take (see linear_rope_ok)")
    if sin.shape != cos.shape or sin.dtype != torch.float32 or not sin.is_contiguous():
        raise KernelError("linear_rope: sin must match cos")
    M, K = values.shape
    if positions.numel() != M or row_ids.numel() != M:
        raise KernelError("linear_rope: one position and one row id per token")
    page_size = num_pages = max_pages = 0
    if k_cache is not None:
        if v_cache is None or block_table is None or write_from is None or v_cache.shape != k_cache.shape or v_cache.dtype != k_cache.dtype or not v_cache.is_contiguous():
            raise KernelError("linear_rope: a cache write needs both caches, the block table and write_from")
        if tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) or block_table.dim() != 2 or not block_table.is_contiguous():
            raise KernelError("linear_rope: cache or block table layout")
        num_pages, page_size = k_cache.shape[0], k_cache.shape[1]
        max_pages = block_table.shape[1]
    fn = _fn(
        "gemm_skinny", "kb_gemm_skinny_rope",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float,
         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_void_p, c_void_p],
    )
    _check(
        fn(values.data_ptr(), values.stride(0), weight.data_ptr(), weight.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), M, weight.shape[0], K,
           _ptr(scale_by.sumsq) if scale_by is not None else None, scale_by.sumsq.shape[0] if scale_by is not None else 0,
           scale_by.hidden if scale_by is not None else 0, float(scale_by.eps) if scale_by is not None else 0.0,
           cos.data_ptr(), sin.data_ptr(), cos.shape[0], num_q_heads, num_kv_heads, head_dim, positions.data_ptr(), row_ids.data_ptr(),
           _ptr(block_table), max_pages, _ptr(write_from), _ptr(k_cache), _ptr(v_cache), page_size, num_pages, _ptr(flag), _stream()),
        "linear_rope",
    )


# ---- RMSNorm inside the products around it (decode: a norm kernel of its own costs as much as
# a third of the q/k/v product it feeds)


@dataclass
class PreNormed:
    """Rows on their way into an RMSNorm whose work is split between two products: ``values`` =
    bf16(x * norm weight), not yet scaled; ``sumsq[b, m]`` = partial sums of x[m]^2, one per block
    of the product that wrote them.  The product that reads it scales row m by
    rsqrt(sum_b sumsq[b, m] / hidden + eps)."""

    values: torch.Tensor
    sumsq: torch.Tensor
    hidden: int
    eps: float

    @property
    def shape(self) -> torch.Size:
        return self.values.shape


@dataclass
class ResidualNorm:
    """What a product does with its result instead of writing it: add it to the fp32 ``residual`` in
    place, and leave ``values`` and ``sumsq`` of a :class:`PreNormed` for the norm (weight, eps) that follows."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float
    values: torch.Tensor
    sumsq: torch.Tensor

    def result(self) -> PreNormed:
        return PreNormed(self.values, self.sumsq, self.residual.shape[1], self.eps)


def fused_norm_available() -> bool:
    """The products of this module can take the RMSNorm around them into their epilogues."""
    return True


def skinny_blocks(rows: int, out_features: int, gated: bool = False) -> int:
    """Blocks the skinny product is launched with: partial sums per row a ``ResidualNorm`` needs room for."""
    fn = _fn("gemm_skinny", "kb_gemm_skinny_blocks", [c_int, c_int, c_int])
    return int(fn(int(rows), int(out_features), 1 if gated else 0))


def fused_norm_shapes_ok(rows: int, hidden: int, *feature_sizes: int) -> bool:
    """Whether products between ``hidden`` (the width of the residual, which the folding products
    write) and these other sizes can all take the fused path.  The product that scales adds one
    partial sum per block of the product that folded: a residual so wide that the folding product
    is launched with more blocks than it can add up keeps the norm kernel."""
    if not few_rows(rows, hidden) or hidden % 16 != 0 or any(size % 16 != 0 for size in feature_sizes):
        return False
    fits = _fold_fits.get((rows, hidden))
    if fits is None:
        limit = int(_fn("gemm_skinny", "kb_gemm_skinny_max_sum_blocks", [])())
        fits = _fold_fits[(rows, hidden)] = skinny_blocks(rows, hidden) <= limit
    return fits


_fold_fits: dict[tuple[int, int], bool] = {}


TC5_MAX_ROWS = 64  # token rows the tcgen05 weight-streaming product takes (csrc/gemm_tc5.cu)
# Encoded TMA descriptors by what they describe.  A caller takes the host addresses of several of
# them before it launches, so none may be freed while a call is being put together: when the table
# is full it is set aside whole (and only dropped when the next one is full, thousands of
# descriptors later) instead of being cleared.
_TENSOR_MAP_LIMIT = 4096
_tensor_maps: dict[tuple, ctypes.Array] = {}
_tensor_maps_before: dict[tuple, ctypes.Array] = {}


def _keep_map(key: tuple, held: ctypes.Array) -> None:
    global _tensor_maps, _tensor_maps_before
    if len(_tensor_maps) >= _TENSOR_MAP_LIMIT:
        _tensor_maps_before = _tensor_maps
        _tensor_maps = {}
    _tensor_maps[key] = held


def _held_map(key: tuple) -> Optional[ctypes.Array]:
    held = _tensor_maps.get(key)
    if held is None:
        held = _tensor_maps_before.get(key)
        if held is not None:
            _keep_map(key, held)  # in use again: it moves to the current table
    return held


_tc5_scratch: list[torch.Tensor] = []  # old buffers stay alive: captured graphs may still point at them


def _tensor_map(tensor: torch.Tensor, box_rows: int) -> int:
    """Host address of a cached TMA descriptor of a row-major bf16 matrix (boxes of [box_rows, 64])."""
    key = (tensor.data_ptr(), tensor.shape[0], tensor.shape[1], tensor.stride(0), box_rows)
    held = _held_map(key)
    if held is None:
        held = ctypes.create_string_buffer(128 + 64)
        address = (ctypes.addressof(held) + 63) & ~63
        fn = _fn("gemm_tc5", "kb_tc5_encode_map", [c_void_p, c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, c_int])
        code = fn(address, tensor.data_ptr(), tensor.shape[0], tensor.shape[1], tensor.stride(0), box_rows)
        if code != 0:
            raise KernelError(f"tensor map encoding failed with code {code}")
        _keep_map(key, held)
    return (ctypes.addressof(held) + 63) & ~63


# The tcgen05 product takes a gated weight from this size on.  Measured at 12 to 64 rows against the library
# product followed by the gate kernel: 201 to 524 MB (hidden 4,096 and 5,120) it is level or up to 5 % ahead,
# at 50 to 100 MB (hidden 2,048 to 3,072: 48 to 72 weight rows a block) it takes 18-32 us where the pair
# takes 12-20: a k step costs it about 600 ns however few rows a block owns, and neither more stages in the
# same shared memory nor another order of the k steps nor other cache hints changed that.
TC5_MIN_WEIGHT_BYTES = 160 << 20


def _tc5_ok(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    M, K = x.shape
    return (
        M <= TC5_MAX_ROWS
        and K % 8 == 0
        and x.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1
        and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
        and out.dtype in (torch.bfloat16, torch.float32)
        and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))
    )


def _gemm_tc5(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, gated: bool,
              flag: Optional[torch.Tensor] = None) -> None:
    M, K = x.shape
    N = weight.shape[0]
    n_out = N // 2 if gated else N
    splits_fn = _fn("gemm_tc5", "kb_gemm_tc5_splits", [c_int, c_int, c_int])
    splits = splits_fn(n_out, K, 1 if gated else 0)
    partial = None
    if splits > 1:
        need = splits * M * n_out
        if not _tc5_scratch or _tc5_scratch[-1].numel() < need or _tc5_scratch[-1].device != x.device:
            _tc5_scratch.append(torch.empty(max(need, 8 * 1024 * 1024), dtype=torch.float32, device=x.device))
        partial = _tc5_scratch[-1]
    box = 16 if M <= 16 else (32 if M <= 32 else 64)
    rows_fn = _fn("gemm_tc5", "kb_gemm_tc5_rows", [c_int, c_int, c_int])
    rows_per_block = rows_fn(n_out, K, 1 if gated else 0)
    fn = _fn("gemm_tc5", "kb_gemm_tc5", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(_tensor_map(weight, rows_per_block), _tensor_map(x, box), out.data_ptr(), 1 if out.dtype == torch.float32 else 0, out.stride(0),
           _ptr(bias), _ptr(partial), M, N, K, 1 if gated else 0, rows_per_block, _ptr(flag), _stream()),
        "gemm_tc5",
        launches=2 if splits > 1 else 1,
    )


def linear_swiglu(x, weight_gate_up: torch.Tensor, out: torch.Tensor, scratch: object) -> None:
    """out = silu(x @ Wg.T) * (x @ Wu.T) with ``weight_gate_up`` = [Wg; Wu] stacked by rows.

    For up to 64 bf16 token rows this is one weight-streaming kernel with the gate in its
    epilogue: the mma.sync skinny kernel up to 8 rows (csrc/gemm_skinny.cu; measured on the
    decode step at 8 rows it is 2 % of the step faster than the tcgen05 kernel, whose fixed
    costs - barrier and tensor-memory set-up, the accumulator read-back - weigh more on a 40 us
    kernel), the tcgen05 + TMA kernel from 9 to 64 rows (csrc/gemm_tc5.cu) where the weight is large
    enough for it (``TC5_MIN_WEIGHT_BYTES``); otherwise a product into ``scratch.buffer(...)`` and the
    gate kernel.
    """
    if isinstance(x, PreNormed):  # its rows are scaled in the epilogue, before the gate
        _need_cuda("linear_swiglu", x.values, weight_gate_up, out)
        if (x.values.dtype != torch.bfloat16 or weight_gate_up.dtype != torch.bfloat16 or out.dtype != torch.bfloat16
                or out.shape != (x.values.shape[0], weight_gate_up.shape[0] // 2) or not _skinny_ok(x.values, weight_gate_up, None, out)):
            raise KernelError("linear_swiglu: a fused norm needs bf16 operands that the weight-streaming kernel takes")
        _gemm_skinny(x.values, weight_gate_up, None, out, gated=True, scale_by=x)
        return
    _need_cuda("linear_swiglu", x, weight_gate_up, out)
    M = x.shape[0]
    two_i = weight_gate_up.shape[0]
    if two_i % 2 or out.shape != (M, two_i // 2):
        raise KernelError("linear_swiglu: shape mismatch")
    if M == 0:
        return
    if x.dtype == torch.bfloat16 and weight_gate_up.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        if few_rows(M, x.shape[1]) and _skinny_ok(x, weight_gate_up, None, out):
            _gemm_skinny(x, weight_gate_up, None, out, gated=True)
            return
        if _tc5_ok(x, weight_gate_up, None, out) and weight_gate_up.numel() * 2 >= TC5_MIN_WEIGHT_BYTES:
            _gemm_tc5(x, weight_gate_up, None, out, gated=True)
            return
    gate_up = scratch.buffer("ffn.gate_up", M, two_i, x.dtype)
    linear(x, weight_gate_up, None, gate_up)
    swiglu(gate_up, out)


# ----------------------------------------------------------------------------- sampling


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda("argmax", logits, out)
    _need_i32("argmax", out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be fp32 with unit inner stride")
    n, V = logits.shape
    fn = _fn("sampling", "kb_argmax", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), n, V, out.data_ptr(), _stream()), "argmax")


def edit_logits(
    logits: torch.Tensor,
    rows: torch.Tensor,
    tokens: torch.Tensor,
    mul: torch.Tensor,
    sub: torch.Tensor,
    mask: torch.Tensor,
) -> None:
    _need_cuda("edit_logits", logits, rows, tokens, mul, sub, mask)
    _need_i32("edit_logits", rows, tokens, mask)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("edit_logits: logits must be fp32 with unit inner stride")
    E = rows.numel()
    if not (tokens.numel() == mul.numel() == sub.numel() == mask.numel() == E):
        raise KernelError("edit_logits: entry arrays must have one length")
    if mul.dtype != torch.float32 or sub.dtype != torch.float32:
        raise KernelError("edit_logits: mul and sub must be fp32")
    fn = _fn("sampling", "kb_edit_logits", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(), tokens.data_ptr(), mul.data_ptr(), sub.data_ptr(), mask.data_ptr(), E, _stream()), "edit_logits")


def logprob_report(
    logits: torch.Tensor,
    rows: torch.Tensor,
    tokens: torch.Tensor,
    k: int,
    values: torch.Tensor,
    indices: torch.Tensor,
    *,
    tokens_by_row: bool,
) -> None:
    """For report r over row ``rows[r]`` of the raw logits: ``values[r, 0]`` = log-softmax of its
    token (``tokens[rows[r]]`` when ``tokens_by_row``, else ``tokens[r]``), ``values[r, 1 + i]`` and
    ``indices[r, i]`` the i-th largest log-softmax value and its token id (ties: the lower id)."""
    _need_cuda("logprob_report", logits, rows, tokens, values, indices)
    _need_i32("logprob_report", rows, tokens, indices)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logprob_report: logits must be fp32 with unit inner stride")
    reports = rows.numel()
    n, V = logits.shape
    k = int(k)
    if k < 0 or values.dtype != torch.float32 or not values.is_contiguous() or values.shape != (reports, k + 1):
        raise KernelError("logprob_report: values must be contiguous fp32 [reports, k + 1]")
    if not indices.is_contiguous() or indices.shape != (reports, k):
        raise KernelError("logprob_report: indices must be contiguous int32 [reports, k]")
    if tokens.numel() < (n if tokens_by_row else reports):
        raise KernelError("logprob_report: too few tokens")
    if reports == 0:
        return
    need_fn = _fn("sampling", "kb_logprob_report_scratch_floats", [c_int, c_int, c_int])
    need_fn.restype = ctypes.c_longlong
    scratch = torch.empty(max(1, int(need_fn(reports, V, k))), dtype=torch.float32, device=logits.device)  # the chunks' candidates
    fn = _fn("sampling", "kb_logprob_report", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(logits.data_ptr(), logits.stride(0), n, V, rows.data_ptr(), tokens.data_ptr(), 1 if tokens_by_row else 0, reports, k,
           values.data_ptr(), indices.data_ptr() if k else None, scratch.data_ptr(), _stream()),
        "logprob_report",
        launches=2,
    )


def sample_work_floats(rows: int, vocab: int) -> int:
    """Scratch floats ``sample`` needs: the rows' probabilities and the state of its three stages."""
    fn = _fn("sampling", "kb_sample_extra_floats", [c_int])
    return rows * vocab + 1 + int(fn(int(rows)))


def sample(
    logits: torch.Tensor,
    work: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    min_p: torch.Tensor,
    seeds: torch.Tensor,
    out: torch.Tensor,
) -> None:
    """One draw per row; ``seeds`` are int64 bit patterns of the per-position seeds."""
    _need_cuda("sample", logits, work, temperature, top_k, top_p, min_p, seeds, out)
    _need_i32("sample", top_k, out)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be fp32 with unit inner stride")
    if work.dtype != torch.float32 or not work.is_contiguous() or work.numel() < sample_work_floats(n, V) or work.data_ptr() % 8:
        raise KernelError("sample: work must be contiguous fp32 with at least sample_work_floats(rows, vocab) elements")
    if seeds.dtype != torch.int64 or temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or min_p.dtype != torch.float32:
        raise KernelError("sample: parameter dtypes are fp32 (temperature, top_p, min_p), int32 (top_k), int64 (seeds)")
    fn = _fn("sampling", "kb_sample", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(logits.data_ptr(), logits.stride(0), work.data_ptr(), n, V, temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(), seeds.data_ptr(), out.data_ptr(), _stream()),
        "sample",
    )


__all__ = [
    "few_rows",
    "linear_weight_streaming",
    "linear_rope",
    "linear_rope_ok",
    "logprob_report",
    "KernelBuildError",
    "KernelError",
    "PreNormed",
    "ResidualNorm",
    "argmax",
    "attention_decode_mma",
    "attention_mma_supported",
    "attention_prefill_tile_rows",
    "attention_prefill_wide_tile_rows",
    "attention_prefill_mma",
    "edit_logits",
    "embedding",
    "fused_norm_available",
    "fused_norm_shapes_ok",
    "gather_rows",
    "linear",
    "linear_swiglu",
    "patch_tokens",
    "paged_attention_generic",
    "qk_norm_rope_kv_write",
    "rmsnorm",
    "sample",
    "sample_work_floats",
    "skinny_blocks",
    "swiglu",
]


# ----------------------------------------------------------------------------- norm on a sub-layer's output


@dataclass
class PendingSums:
    """What a layer whose sub-layers run side by side leaves for the next norm: two outputs still to be added to the
    residual (the mixer's, then the feed-forward's).  A norm that takes two pending sums adds both in its own kernel."""

    first: torch.Tensor
    second: torch.Tensor

    @property
    def shape(self) -> torch.Size:
        return self.first.shape


@dataclass
class ResidualCopy:
    """What a block that norms its sub-layers' OUTPUTS hands to the block after it: the residual's
    rows in the activation dtype (the sub-layers read the stream itself, so the next one wants them
    as product operands).  Nothing is left to add: ``pending_delta`` is None."""

    values: torch.Tensor
    pending_delta = None


@dataclass
class WeightedRows:
    """A sub-layer's output as K rows a token and their weights (a mixture of experts before the
    sum): ``rows`` [tokens * K, width], ``weights`` [tokens, K] fp32; row k of token t is
    ``rows[t * K + k]``, or ``rows[at[t * K + k]]`` where ``at`` (int32) is given."""

    rows: torch.Tensor
    weights: torch.Tensor
    at: Optional[torch.Tensor] = None


def output_norm_add(residual: torch.Tensor, y, weight: torch.Tensor, eps: float, copy: Optional[torch.Tensor]) -> None:
    """``residual += rmsnorm(y) * weight`` and ``copy = residual`` in the activation dtype (when given).
    ``y``: rows of the residual's shape, or a :class:`WeightedRows` whose K rows a token are summed
    first, weighted, in the order of k."""
    mix = at = None
    K = 1
    rows = y
    if isinstance(y, WeightedRows):
        rows, mix, at = y.rows, y.weights, y.at
        K = mix.shape[1]
        _need_i32("output_norm_add", at)
        if at is not None and at.numel() != mix.numel():
            raise KernelError("output_norm_add: the index of weighted rows must have one entry a row")
        if mix.dtype != torch.float32 or not mix.is_contiguous() or mix.shape[0] != residual.shape[0]:
            raise KernelError("output_norm_add: the weights of weighted rows must be contiguous fp32 [tokens, K]")
    _need_cuda("output_norm_add", residual, rows, weight, copy, mix, at)
    T, H = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous() or not rows.is_contiguous() or rows.shape != (T * K, H):
        raise KernelError("output_norm_add: the residual must be contiguous fp32 and the rows of its width")
    if weight.numel() != H or (copy is not None and (copy.shape != (T, H) or not copy.is_contiguous())):
        raise KernelError("output_norm_add: shape mismatch")
    fn = _fn("sublayer_norm", "kb_output_norm_add", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(
        fn(residual.data_ptr(), rows.data_ptr(), _is_bf16(rows, "output_norm_add"), _ptr(mix), _ptr(at), K, weight.data_ptr(),
           _is_bf16(weight, "output_norm_add"), _ptr(copy), _is_bf16(copy, "output_norm_add") if copy is not None else 0, T, H,
           float(eps), _stream()),
        "output_norm_add",
    )


@dataclass
class PendingNormed:
    """What a block that norms its sub-layers' outputs may leave for the norm that reads the stream next:
    ``residual += rmsnorm(values) * weight`` is still to be done, and that norm's kernel does it on its way."""

    values: torch.Tensor
    weight: torch.Tensor
    eps: float

    @property
    def shape(self) -> torch.Size:
        return self.values.shape


def sandwich_norm(residual: torch.Tensor, pending: Optional[PendingNormed], weight: Optional[torch.Tensor], eps: float,
                  out: Optional[torch.Tensor], *, rows: Optional[torch.Tensor] = None) -> None:
    """``residual += rmsnorm(pending.values) * pending.weight`` (when given), then ``out = rmsnorm(residual) * weight``
    (when given), in one kernel.  With ``rows`` only the listed rows are produced and the residual is not written."""
    what = "sandwich_norm"
    y = pending.values if pending is not None else None
    wy = pending.weight if pending is not None else None
    _need_cuda(what, residual, y, wy, weight, out, rows)
    _need_i32(what, rows)
    T, H = residual.shape
    R = rows.numel() if rows is not None else T
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError(f"{what}: the residual must be contiguous fp32")
    if y is not None and (y.shape != (T, H) or not y.is_contiguous() or wy.numel() != H or (out is not None and y.dtype != out.dtype)):
        raise KernelError(f"{what}: the pending rows must have the residual's shape and the activation dtype, their weight its width")
    if out is not None and (out.shape[1] != H or out.shape[0] < R or not out.is_contiguous() or weight is None or weight.numel() != H):
        raise KernelError(f"{what}: the output or its weight does not fit")
    if y is None and out is None:
        return
    weights = [w for w in (wy, weight) if w is not None]
    if any(w.dtype != weights[0].dtype or not w.is_contiguous() for w in weights):
        raise KernelError(f"{what}: contiguous weights of one dtype")
    act = out if out is not None else y
    fn = _fn("sublayer_norm", "kb_sandwich_norm", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(residual.data_ptr(), _ptr(y), _ptr(wy), float(pending.eps) if pending is not None else 0.0, _ptr(weight), float(eps), _ptr(out),
              _is_bf16(act, what), _is_bf16(weights[0], what), _ptr(rows), R, H, _stream()), what)


def residual_copy(residual: torch.Tensor, copy: torch.Tensor) -> None:
    """copy = residual in bfloat16."""
    _need_cuda("residual_copy", residual, copy)
    if residual.dtype != torch.float32 or copy.dtype != torch.bfloat16 or residual.shape != copy.shape or not (residual.is_contiguous() and copy.is_contiguous()):
        raise KernelError("residual_copy: needs a contiguous fp32 source and a bfloat16 copy of its shape")
    fn = _fn("sublayer_norm", "kb_residual_copy", [c_void_p, c_void_p, ctypes.c_longlong, c_void_p])
    _check(fn(residual.data_ptr(), copy.data_ptr(), residual.numel(), _stream()), "residual_copy")


# ----------------------------------------------------------------------------- latent attention


def latent_norm_write(
    packed: torch.Tensor,
    offset: int,
    rank: int,
    weight: torch.Tensor,
    eps: float,
    cache: Optional[torch.Tensor],
    *,
    positions: torch.Tensor,
    row_ids: torch.Tensor,
    block_table: Optional[torch.Tensor],
    write_from: Optional[torch.Tensor],
    flag: Optional[torch.Tensor] = None,
    rot_dim: int = 0,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    interleaved: bool = True,
    q_out: Optional[torch.Tensor] = None,
    num_heads: int = 0,
    q_head_width: int = 0,
) -> None:
    """Columns [offset, offset + rank) of every row of ``packed`` are RMS-normed (32-bit) and written,
    in the cache's dtype, at the token's place in its request's pages.  ``cache``: [pages, page_size, 1, rank + rot_dim].

    ``rot_dim`` > 0: the ``rot_dim`` columns behind the latent's are one key part shared by all heads; it is
    rotated by the token's position (``cos``/``sin`` [positions, rot_dim/2] fp32; pairs (2i, 2i+1) when
    ``interleaved``, else (i, i + rot_dim/2)) and stored behind the latent.  With ``q_out``
    [tokens, heads * (rank + rot_dim)] the last ``rot_dim`` of every head's ``q_head_width`` columns of the
    packed query (columns [0, heads * q_head_width)) are rotated into columns [rank, rank + rot_dim) of the
    head's row of ``q_out``.  ``cache=None``: only the queries' part is produced (a call that writes no cache)."""
    _need_cuda("latent_norm_write", packed, weight, cache, positions, row_ids, block_table, write_from, flag, cos, sin, q_out)
    _need_i32("latent_norm_write", positions, row_ids, block_table, write_from)
    width = rank + rot_dim
    num_pages = page_size = 1
    if cache is not None:
        num_pages, page_size, heads, cache_width = cache.shape
        if heads != 1 or cache_width != width or not cache.is_contiguous() or cache.dtype != packed.dtype:
            raise KernelError("latent_norm_write: the cache must be contiguous [pages, page_size, 1, rank + rot_dim] in the activations' dtype")
        if block_table is None:
            raise KernelError("latent_norm_write: a cache write needs the block table")
    if packed.stride(1) != 1 or offset < 0 or offset + width > packed.shape[1] or weight.numel() != rank:
        raise KernelError("latent_norm_write: the packed rows do not hold the latent's columns")
    max_pos = 0
    if rot_dim:
        if cos is None or sin is None or cos.shape != sin.shape or cos.shape[1] * 2 != rot_dim or cos.dtype != torch.float32 or sin.dtype != torch.float32 \
                or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError("latent_norm_write: cos and sin must be contiguous fp32 [positions, rot_dim / 2]")
        max_pos = cos.shape[0]
        if q_out is not None:
            if q_out.dtype != packed.dtype or q_out.stride(1) != 1 or q_out.shape[1] != num_heads * width or q_out.shape[0] != packed.shape[0] \
                    or q_head_width < rot_dim or num_heads * q_head_width > packed.shape[1]:
                raise KernelError("latent_norm_write: q_out must be [tokens, heads * (rank + rot_dim)] beside a packed query of heads * q_head_width columns")
    elif q_out is not None:
        raise KernelError("latent_norm_write: q_out comes with a rotated part")
    fn = _fn("latent_cache", "kb_latent_norm_write",
             [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(packed.data_ptr(), packed.stride(0), int(offset), int(rank), _is_bf16(packed, "latent_norm_write"), weight.data_ptr(),
           _is_bf16(weight, "latent_norm_write"), float(eps), positions.data_ptr(), row_ids.data_ptr(), _ptr(block_table),
           block_table.shape[1] if block_table is not None else 0, _ptr(write_from), _ptr(cache), page_size, num_pages,
           block_table.shape[0] if block_table is not None else 0, packed.shape[0], int(rot_dim), _ptr(cos), _ptr(sin), max_pos,
           1 if interleaved else 0, int(num_heads), int(q_head_width), _ptr(q_out), q_out.stride(0) if q_out is not None else 0,
           1 if cache is not None else 0, _ptr(flag), _stream()),
        "latent_norm_write",
    )


def heads_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """A product per head: ``out[t, h, :] = weight[h] @ x[t, h, :]``.  ``x`` [tokens, heads, K] and
    ``out`` [tokens, heads, N] may be views with any row and head stride (inner stride 1: a head's columns
    may be part of a wider run); ``weight`` is
    contiguous [heads, N, K].  bfloat16: the library's batched product (fp32 accumulation);
    float32: this package's FMA product, one launch a head."""
    _need_cuda("heads_linear", x, weight, out)
    T, H, K = x.shape
    N = weight.shape[1]
    if weight.shape != (H, N, K) or out.shape != (T, H, N) or not weight.is_contiguous():
        raise KernelError(f"heads_linear: shapes x{tuple(x.shape)} w{tuple(weight.shape)} out{tuple(out.shape)} do not agree")
    if x.stride(2) != 1 or out.stride(2) != 1 or x.stride(1) < K or out.stride(1) < N:
        raise KernelError("heads_linear: a head's columns must lie side by side, and heads must not overlap")
    if T == 0:
        return
    if x.dtype == torch.float32:
        if weight.dtype != torch.float32 or out.dtype != torch.float32:
            raise KernelError("heads_linear: the 32-bit path needs fp32 weights and output")
        fn = _fn("gemm_f32", "kb_gemm_f32", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        for h in range(H):
            _check(fn(x.data_ptr() + 4 * h * x.stride(1), x.stride(0), weight.data_ptr() + 4 * h * N * K, K, None, out.data_ptr() + 4 * h * out.stride(1),
                      out.stride(0), T, N, K, _stream()), "heads_linear")
        return
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("heads_linear: bfloat16 or float32 throughout")
    torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))


# ----------------------------------------------------------------------------- gated delta rule


def delta_prepare(
    packed: torch.Tensor,
    gates: torch.Tensor,
    taps: torch.Tensor,
    conv_state: Optional[torch.Tensor],
    *,
    row_ids: torch.Tensor,
    qo_indptr: torch.Tensor,
    state_slots: torch.Tensor,
    a_log: torch.Tensor,
    dt_bias: torch.Tensor,
    kv_heads: int,
    dim: int,
    heads: int,
    vdim: int,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    beta: torch.Tensor,
    decay: torch.Tensor,
    flag: Optional[torch.Tensor] = None,
    channel_a: Optional[torch.Tensor] = None,
) -> None:
    """Convolution + silu of the packed q|k|v columns, unit norms of q and k, beta and the decay, all
    to fp32; then the step's last inputs become the requests' kept inputs (``conv_state``
    [slots, taps - 1, channels] fp32).  ``gates`` [tokens, 2 * heads]: beta's logits, then the decay's input a head
    (``dt_bias`` and ``decay`` a head).  With ``channel_a`` [tokens, heads * dim] the decay is one number a head and
    key channel: ``gates`` is then [tokens, heads], ``dt_bias`` [heads * dim] and ``decay`` [tokens, heads * dim]."""
    _need_cuda("delta_prepare", packed, gates, taps, conv_state, row_ids, qo_indptr, state_slots, a_log, dt_bias, q, k, v, beta, decay, flag, channel_a)
    _need_i32("delta_prepare", row_ids, qo_indptr, state_slots)
    T = packed.shape[0]
    channels = 2 * kv_heads * dim + heads * vdim
    n = taps.shape[1]
    for tensor in (gates, taps, a_log, dt_bias, q, k, v, beta, decay) + ((conv_state,) if conv_state is not None else ()) + ((channel_a,) if channel_a is not None else ()):
        if tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError("delta_prepare: everything but the packed projection is contiguous fp32")
    per = 1 if channel_a is None else dim  # decays a head
    if packed.stride(1) != 1 or packed.shape[1] < channels or taps.shape[0] != channels or gates.shape != (T, (2 if channel_a is None else 1) * heads):
        raise KernelError("delta_prepare: the packed projection, the taps or the gates do not fit the sizes")
    if (channel_a is not None and channel_a.shape != (T, heads * dim)) or dt_bias.numel() != heads * per or a_log.numel() != heads:
        raise KernelError("delta_prepare: the decay's inputs do not fit the sizes")
    if conv_state is not None and tuple(conv_state.shape[1:]) != (n - 1, channels):
        raise KernelError("delta_prepare: the kept inputs must be [slots, taps - 1, channels]")
    if q.numel() != T * kv_heads * dim or k.numel() != q.numel() or v.numel() != T * heads * vdim or beta.numel() != T * heads or decay.numel() != T * heads * per:
        raise KernelError("delta_prepare: an output does not fit")
    fn = _fn("delta_rule", "kb_delta_prepare",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(packed.data_ptr(), packed.stride(0), _is_bf16(packed, "delta_prepare"), gates.data_ptr(), _ptr(channel_a), taps.data_ptr(), n, _ptr(conv_state),
           row_ids.data_ptr(), qo_indptr.data_ptr(), state_slots.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), kv_heads, dim, heads,
           vdim, q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), decay.data_ptr(), qo_indptr.numel() - 1, T, _ptr(flag), _stream()),
        "delta_prepare",
        launches=2 if n > 1 else 1,
    )


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, states: torch.Tensor,
                     out: torch.Tensor, *, qo_indptr: torch.Tensor, state_slots: torch.Tensor, kv_heads: int, dim: int, heads: int,
                     vdim: int, channel_decay: bool = False) -> None:
    """Every row's tokens in order through S <- g S + k (beta (v - g S^T k))^T, o = S^T q; ``states``
    [slots, heads, vdim, dim] fp32 (S column by column) is read and left updated.  ``decay``: [tokens, heads], or
    [tokens, heads * dim] with ``channel_decay``: one decay a key channel (g then scales the rows of S)."""
    _need_cuda("delta_recurrence", q, k, v, beta, decay, states, out, qo_indptr, state_slots)
    _need_i32("delta_recurrence", qo_indptr, state_slots)
    for tensor in (q, k, v, beta, decay, states, out):
        if tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError("delta_recurrence: contiguous fp32 tensors only")
    if tuple(states.shape[1:]) != (heads, vdim, dim) or out.numel() != v.numel():
        raise KernelError("delta_recurrence: the state must be [slots, heads, vdim, dim] and the output as large as v")
    if dim > 512:
        raise KernelError(f"delta_recurrence: dim {dim} > 512 is not supported")
    if decay.numel() != q.shape[0] * heads * (dim if channel_decay else 1):
        raise KernelError("delta_recurrence: the decay is one number a token and head, or with channel_decay one a token, head and key channel")
    channel = 1 if channel_decay else 0
    fn = _fn("delta_rule", "kb_delta_recurrence",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    rows = qo_indptr.numel() - 1
    _check(
        fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), decay.data_ptr(), states.data_ptr(), qo_indptr.data_ptr(),
           state_slots.data_ptr(), kv_heads, dim, heads, vdim, out.data_ptr(), rows, 1 if q.shape[0] == rows else 0, channel, _stream()),
        "delta_recurrence",
    )


def delta_gated_norm(o: torch.Tensor, packed: torch.Tensor, gate_offset: int, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
                     heads: int, vdim: int, gate_activation: str = "silu") -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * act(gate[t, h]); the gate is columns
    [gate_offset, gate_offset + heads * vdim) of ``packed`` (the packed projection, or a tensor of the gate's
    own); ``gate_activation``: ``silu`` or ``sigmoid``."""
    _need_cuda("delta_gated_norm", o, packed, weight, out)
    T = packed.shape[0]
    if gate_activation not in ("silu", "sigmoid"):
        raise KernelError(f"delta_gated_norm: unknown gate activation {gate_activation!r} (silu, sigmoid)")
    if o.dtype != torch.float32 or weight.dtype != torch.float32 or not o.is_contiguous() or not out.is_contiguous() or out.dtype != packed.dtype:
        raise KernelError("delta_gated_norm: o and the weight are fp32, the output has the projection's dtype")
    if out.shape != (T, heads * vdim) or o.numel() != T * heads * vdim or weight.numel() != vdim or gate_offset + heads * vdim > packed.shape[1] or packed.stride(1) != 1:
        raise KernelError("delta_gated_norm: shape mismatch")
    fn = _fn("delta_rule", "kb_delta_gated_norm", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(fn(o.data_ptr(), packed.data_ptr() + int(gate_offset) * packed.element_size(), packed.stride(0), 1 if gate_activation == "sigmoid" else 0,
              _is_bf16(packed, "delta_gated_norm"), weight.data_ptr(), float(eps), heads, vdim, out.data_ptr(), T, _stream()), "delta_gated_norm")


# ----------------------------------------------------------------------------- selective state-space mixer


def ssm_prepare(
    packed: torch.Tensor,
    dt_raw: torch.Tensor,
    taps: torch.Tensor,
    conv_bias: Optional[torch.Tensor],
    conv_state: Optional[torch.Tensor],
    *,
    row_ids: torch.Tensor,
    qo_indptr: torch.Tensor,
    state_slots: torch.Tensor,
    a_log: torch.Tensor,
    dt_bias: torch.Tensor,
    groups: int,
    state: int,
    heads: int,
    vdim: int,
    x: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    dt: torch.Tensor,
    decay: torch.Tensor,
    flag: Optional[torch.Tensor] = None,
) -> None:
    """Convolution (+ bias) + silu of the columns ``x | B | C`` of ``packed`` (a view that starts at x) to fp32;
    ``dt = softplus(dt_raw + dt_bias)`` and ``decay = exp(-exp(a_log) * dt)`` a token and head; then the step's last
    inputs become the requests' kept inputs (``conv_state`` [slots, taps - 1, channels] fp32)."""
    what = "ssm_prepare"
    _need_cuda(what, packed, dt_raw, taps, conv_bias, conv_state, row_ids, qo_indptr, state_slots, a_log, dt_bias, x, b, c, dt, decay, flag)
    _need_i32(what, row_ids, qo_indptr, state_slots)
    T = packed.shape[0]
    channels = heads * vdim + 2 * groups * state
    n = taps.shape[1]
    for tensor in (dt_raw, taps, a_log, dt_bias, x, b, c, dt, decay) + tuple(t for t in (conv_state, conv_bias) if t is not None):
        if tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError(f"{what}: everything but the packed projection is contiguous fp32")
    if packed.stride(1) != 1 or packed.shape[1] < channels or taps.shape[0] != channels or dt_raw.shape != (T, heads) or (conv_bias is not None and conv_bias.numel() != channels):
        raise KernelError(f"{what}: the packed projection, the taps, the bias or the step sizes do not fit the sizes")
    if conv_state is not None and tuple(conv_state.shape[1:]) != (n - 1, channels):
        raise KernelError(f"{what}: the kept inputs must be [slots, taps - 1, channels]")
    if x.numel() != T * heads * vdim or b.numel() != T * groups * state or c.numel() != b.numel() or dt.numel() != T * heads or decay.numel() != T * heads \
            or a_log.numel() != heads or dt_bias.numel() != heads:
        raise KernelError(f"{what}: an output or a per-head constant does not fit")
    fn = _fn("ssm", "kb_ssm_prepare",
             [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check(
        fn(packed.data_ptr(), packed.stride(0), _is_bf16(packed, what), dt_raw.data_ptr(), taps.data_ptr(), _ptr(conv_bias), n, _ptr(conv_state),
           row_ids.data_ptr(), qo_indptr.data_ptr(), state_slots.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), groups, state, heads, vdim,
           x.data_ptr(), b.data_ptr(), c.data_ptr(), dt.data_ptr(), decay.data_ptr(), qo_indptr.numel() - 1, T, _ptr(flag), _stream()),
        what,
        launches=2 if n > 1 else 1,
    )


def ssm_recurrence(c: torch.Tensor, b: torch.Tensor, x: torch.Tensor, dt: torch.Tensor, decay: torch.Tensor, states: torch.Tensor,
                   out: torch.Tensor, *, qo_indptr: torch.Tensor, state_slots: torch.Tensor, groups: int, state: int, heads: int, vdim: int) -> None:
    """Every row's tokens in order through S <- decay S + dt B x^T, y = S^T C; ``states`` [slots, heads, vdim, state]
    fp32 (S column by column) is read and left updated."""
    what = "ssm_recurrence"
    _need_cuda(what, c, b, x, dt, decay, states, out, qo_indptr, state_slots)
    _need_i32(what, qo_indptr, state_slots)
    for tensor in (c, b, x, dt, decay, states, out):
        if tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError(f"{what}: contiguous fp32 tensors only")
    if tuple(states.shape[1:]) != (heads, vdim, state) or out.numel() != x.numel() or state > 512:
        raise KernelError(f"{what}: the state must be [slots, heads, vdim, state <= 512] and the output as large as x")
    rows = qo_indptr.numel() - 1
    fn = _fn("ssm", "kb_ssm_recurrence",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(c.data_ptr(), b.data_ptr(), x.data_ptr(), dt.data_ptr(), decay.data_ptr(), states.data_ptr(), qo_indptr.data_ptr(), state_slots.data_ptr(),
              groups, state, heads, vdim, out.data_ptr(), rows, 1 if x.shape[0] == rows else 0, _stream()), what)


def ssm_gated_norm(y: torch.Tensor, x: torch.Tensor, skip: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
                   heads: int, vdim: int, norm_groups: int) -> None:
    """``out = groupnorm((y + skip[h] * x) * silu(z)) * weight``: the RMS norm runs over ``norm_groups`` equal parts of a
    token's ``heads * vdim`` columns, each by its own root mean square.  ``z`` may be a view of a wider row."""
    what = "ssm_gated_norm"
    _need_cuda(what, y, x, skip, z, weight, out)
    T, inner = out.shape
    for tensor in (y, x, skip, weight):
        if tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError(f"{what}: y, x, the skip weights and the norm weight are contiguous fp32")
    if inner != heads * vdim or y.numel() != T * inner or x.numel() != T * inner or skip.numel() != heads or weight.numel() != inner or inner % norm_groups \
            or z.shape != (T, inner) or z.stride(1) != 1 or z.dtype != out.dtype or not out.is_contiguous():
        raise KernelError(f"{what}: shape mismatch")
    fn = _fn("ssm", "kb_ssm_gated_norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_float, c_int, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(fn(y.data_ptr(), x.data_ptr(), skip.data_ptr(), z.data_ptr(), z.stride(0), _is_bf16(z, what), weight.data_ptr(), float(eps), heads, vdim,
              norm_groups, out.data_ptr(), T, _stream()), what)


# ----------------------------------------------------------------------------- mixture of experts


def moe_max_tiles(pairs: int, experts: int) -> int:
    """Upper bound of the tiles ``moe_plan`` cuts ``pairs`` (token, expert) pairs into (csrc/moe.cu: MOE_TM = 64)."""
    return -(-pairs // 64) + experts


def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top: int, ids: torch.Tensor, weights: torch.Tensor) -> None:
    """The ``top`` largest of logits + bias per token and the softmax over them (fp32)."""
    _need_cuda("moe_route", logits, bias, ids, weights)
    T, E = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous() or weights.dtype != torch.float32 or ids.dtype != torch.int32:
        raise KernelError("moe_route: fp32 logits and weights, int32 ids")
    if ids.shape != (T, top) or weights.shape != (T, top) or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("moe_route: ids and weights must be contiguous [tokens, top]")
    if bias is not None and (bias.numel() != E or not bias.is_contiguous()):
        raise KernelError("moe_route: the bias must have one entry an expert")
    fn = _fn("moe", "kb_moe_route", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(logits.data_ptr(), _ptr(bias), _is_bf16(bias, "moe_route") if bias is not None else 0, E, int(top), ids.data_ptr(),
              weights.data_ptr(), T, _stream()), "moe_route")


def moe_route_scores(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, ids: torch.Tensor, weights: torch.Tensor, *,
                     groups: int = 1, keep: int = 1, scale: float = 1.0, score: str = "softmax") -> None:
    """Routing by scores (fp32): s = softmax(logits) over all outputs (``score="sigmoid"``: s = sigmoid(logit), each output by
    itself); the choice runs on s + correction within the ``keep`` best of ``groups`` equal groups of neighbours (a group's
    value: its largest s + correction); the ``top`` best are chosen (ties: the lower index) and weigh s * scale, not
    renormalised.  ``logits`` may be the leading columns of wider rows (a view ``[:, :n]``)."""
    _need_cuda("moe_route_scores", logits, correction, ids, weights)
    T, n = logits.shape
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route_scores: unknown score function {score!r} (softmax, sigmoid)")
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or weights.dtype != torch.float32 or ids.dtype != torch.int32:
        raise KernelError("moe_route_scores: fp32 logits and weights, int32 ids")
    if ids.shape != (T, top) or weights.shape != (T, top) or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("moe_route_scores: ids and weights must be contiguous [tokens, top]")
    if correction is not None and (correction.numel() != n or not correction.is_contiguous()):
        raise KernelError("moe_route_scores: the correction must have one entry a router output")
    fn = _fn("moe", "kb_moe_route_scores", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(logits.data_ptr(), _ptr(correction), _is_bf16(correction, "moe_route_scores") if correction is not None else 0, n, int(top),
              int(groups), int(keep), float(scale), 1 if score == "sigmoid" else 0, logits.stride(0) if T > 1 else n, ids.data_ptr(),
              weights.data_ptr(), T, _stream()), "moe_route_scores")


def moe_scale_rows(src: torch.Tensor, scale: torch.Tensor, out: torch.Tensor, *, rows: Optional[torch.Tensor] = None, per: int = 1,
                   index: Optional[torch.Tensor] = None) -> None:
    """out[i] = src[rows[i]] * scale[index[i]] (``rows=None``: src[i // per]; ``index=None``: scale[i]), 32-bit with one
    rounding: the input rows of experts whose router weight multiplies their input.  ``scale``: flat fp32."""
    _need_cuda("moe_scale_rows", src, scale, out, rows, index)
    _need_i32("moe_scale_rows", rows, index)
    R, H = out.shape
    if src.dtype != out.dtype or src.shape[1] != H or not (src.is_contiguous() and out.is_contiguous()):
        raise KernelError("moe_scale_rows: contiguous rows of one width and dtype")
    if scale.dtype != torch.float32 or not scale.is_contiguous() or (index is None and scale.numel() < R) or (rows is not None and rows.numel() < R) \
            or (index is not None and index.numel() < R) or (rows is None and (R + per - 1) // per > src.shape[0]):
        raise KernelError("moe_scale_rows: a weight and a source row for every output row")
    fn = _fn("moe", "kb_moe_scale_rows", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(src.data_ptr(), _is_bf16(src, "moe_scale_rows"), _ptr(rows), int(per), scale.data_ptr(), _ptr(index), out.data_ptr(), R, H,
              _stream()), "moe_scale_rows")


def moe_plan(ids: torch.Tensor, experts: int, plan: torch.Tensor) -> dict:
    """Sort a step's (token, expert) pairs by expert and cut the runs into tiles.  ``ids`` [tokens, top];
    ``plan``: int32 scratch of at least ``moe_plan_size(pairs, experts)`` entries; returns views into it:
    ``sorted`` (the pairs run by run), ``token_of`` (their tokens), ``place_of`` (where each pair stands),
    ``ends`` (where each expert's run ends) and the tile lists."""
    _need_cuda("moe_plan", ids, plan)
    _need_i32("moe_plan", ids, plan)
    top = ids.shape[1]
    pairs = ids.numel()
    tiles = moe_max_tiles(pairs, experts)
    if plan.numel() < moe_plan_size(pairs, experts):
        raise KernelError("moe_plan: the scratch is too small")
    views: dict = {"max_tiles": tiles}
    at = 0
    for name, count in (("sorted", pairs), ("token_of", pairs), ("place_of", pairs), ("ends", experts), ("tile_expert", tiles),
                        ("tile_first", tiles), ("tile_pairs", tiles), ("num_tiles", 1)):
        views[name] = plan[at : at + count]
        at += count
    fn = _fn("moe", "kb_moe_plan", [c_void_p, c_int, c_int, c_int] + [c_void_p] * 9)
    _check(fn(ids.data_ptr(), pairs, int(experts), int(top), views["sorted"].data_ptr(), views["token_of"].data_ptr(), views["place_of"].data_ptr(),
              views["ends"].data_ptr(), views["tile_expert"].data_ptr(), views["tile_first"].data_ptr(), views["tile_pairs"].data_ptr(),
              views["num_tiles"].data_ptr(), _stream()), "moe_plan")
    return views


def moe_plan_size(pairs: int, experts: int) -> int:
    return 3 * pairs + experts + 3 * moe_max_tiles(pairs, experts) + 1


def moe_library_products_ok(hidden: int, intermediate: int, dtype: torch.dtype) -> bool:
    """Whether the experts' products can go to the library's grouped product (bfloat16, fp32
    accumulation, group sizes read on the device): it wants every row 16-byte aligned."""
    return dtype == torch.bfloat16 and hidden % 8 == 0 and intermediate % 8 == 0 and hasattr(torch, "_grouped_mm")


def moe_library_product(a: torch.Tensor, weight: torch.Tensor, ends: torch.Tensor) -> torch.Tensor:
    """Rows of ``a`` [pairs, K], sorted by expert, times their experts' weights ``weight`` [experts, N, K]:
    [pairs, N] bfloat16.  ``ends`` (int32, on the device) gives where each expert's rows end."""
    _need_cuda("moe_library_product", a, weight, ends)
    if a.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not a.is_contiguous() or not weight.is_contiguous():
        raise KernelError("moe_library_product: contiguous bfloat16 operands only")
    return torch._grouped_mm(a, weight.transpose(1, 2), offs=ends)


def moe_activation(gate_up: torch.Tensor, out: torch.Tensor, *, limit: float, alpha: float = 1.702, shift: float = 1.0) -> None:
    """out = a * sigmoid(alpha a) * (b + shift), a = min(gate, limit), b = clamp(up, -limit, limit); ``gate_up`` rows hold
    the gate columns and then the up columns.  An infinite limit, alpha 1 and shift 0 give silu(gate) * up."""
    _need_cuda("moe_activation", gate_up, out)
    rows, wide = gate_up.shape
    if wide % 2 or out.shape != (rows, wide // 2) or out.dtype != gate_up.dtype or not (gate_up.is_contiguous() and out.is_contiguous()):
        raise KernelError("moe_activation: shape or dtype mismatch")
    fn = _fn("moe", "kb_moe_activation", [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(fn(gate_up.data_ptr(), out.data_ptr(), _is_bf16(out, "moe_activation"), rows, wide // 2, float(limit), float(alpha), float(shift), _stream()), "moe_activation")


def moe_grouped(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, plan: dict, *, top: int, gated: bool, limit: float = 0.0,
                alpha: float = 1.702, shift: float = 1.0) -> None:
    """The experts' products over a planned step.  ``gated``: ``a`` [tokens, K] activations, ``weight``
    [experts, 2 * N, K] (gate rows, then up rows), ``out`` [pairs, N] in the activations' dtype, rows
    in the plan's sorted order, after the experts' activation.  Otherwise ``a`` is such an ``out``,
    ``weight`` [experts, N, K] and ``out`` fp32 [pairs, N] with row t * top + k for token t's k-th expert."""
    _need_cuda("moe_grouped", a, weight, out)
    experts, rows, K = weight.shape
    N = rows // 2 if gated else rows
    pairs = plan["sorted"].numel()
    if a.dtype != weight.dtype or a.shape[1] != K or a.stride(1) != 1 or not weight.is_contiguous() or not out.is_contiguous():
        raise KernelError("moe_grouped: operands must share a dtype and K, the weight and the output be contiguous")
    if out.shape != (pairs, N) or out.dtype != (a.dtype if gated else torch.float32):
        raise KernelError("moe_grouped: the output does not fit")
    fn = _fn("moe", "kb_moe_grouped", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_float, c_float, c_float, c_int, c_void_p, c_void_p])
    _check(fn(a.data_ptr(), a.stride(0), plan["sorted"].data_ptr(), int(top), weight.data_ptr(), N, K, _is_bf16(a, "moe_grouped"), 1 if gated else 0,
              plan["tile_expert"].data_ptr(), plan["tile_first"].data_ptr(), plan["tile_pairs"].data_ptr(), plan["num_tiles"].data_ptr(),
              plan["max_tiles"], float(limit), float(alpha), float(shift), experts, out.data_ptr(), _stream()), "moe_grouped")


# The few-pairs kernel is taken for up to this many tokens a step, in models this narrow: measured against the
# library's grouped product (32 experts, 4 a token; gate/up + down, microseconds with about 17 of overhead in each
# figure): width 2,048 and 1,024 rows an expert 53+33 / 65+38 / 69+44 / 77+52 against 52+41 / 69+51 / 78+57 / 87+65 at
# 1 / 4 / 8 / 16 tokens; at width 4,096 and 2,048 rows an expert it is behind at every size (132+60 against 64+46 at
# one token: four experts are 128 blocks of a megabyte each, too few loads in flight), and at 64 tokens everywhere.
MOE_SKINNY_MAX_TOKENS = 16
MOE_SKINNY_MAX_WIDTH = 2048


def moe_skinny_ok(tokens: int, hidden: int, intermediate: int, dtype: torch.dtype) -> bool:
    """Whether a step's experts run on the weight-streaming kernel for few pairs an expert: bfloat16, rows of whole
    16 bytes, a decode-sized step of a narrow model."""
    return (dtype == torch.bfloat16 and tokens <= MOE_SKINNY_MAX_TOKENS and hidden % 8 == 0 and intermediate % 8 == 0
            and max(hidden, intermediate) <= MOE_SKINNY_MAX_WIDTH)


def moe_skinny(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, plan: dict, *, top: int, gated: bool, limit: float = 0.0,
               alpha: float = 1.702, shift: float = 1.0) -> None:
    """``moe_grouped`` for few pairs an expert (bfloat16): the weight rows are the tensor cores' M side, up to 8
    pairs at a time the N side, and the weights are read straight from global memory.  Same operands and results."""
    _need_cuda("moe_skinny", a, weight, out)
    experts, rows, K = weight.shape
    N = rows // 2 if gated else rows
    pairs = plan["sorted"].numel()
    if a.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or a.shape[1] != K or a.stride(1) != 1 or not weight.is_contiguous() or not out.is_contiguous():
        raise KernelError("moe_skinny: bfloat16 operands of one K, the weight and the output contiguous")
    if out.shape != (pairs, N) or out.dtype != (torch.bfloat16 if gated else torch.float32):
        raise KernelError("moe_skinny: the output does not fit")
    fn = _fn("moe", "kb_moe_skinny", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_float, c_float, c_float, c_int, c_void_p, c_void_p])
    _check(fn(a.data_ptr(), a.stride(0), plan["sorted"].data_ptr(), int(top), weight.data_ptr(), N, K, 1 if gated else 0,
              plan["tile_expert"].data_ptr(), plan["tile_first"].data_ptr(), plan["tile_pairs"].data_ptr(), plan["num_tiles"].data_ptr(),
              plan["max_tiles"], float(limit), float(alpha), float(shift), experts, out.data_ptr(), _stream()), "moe_skinny")


def moe_combine(rows: torch.Tensor, weights: Optional[torch.Tensor], out: torch.Tensor, at: Optional[torch.Tensor] = None, *,
                ids: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None, experts: int = 0, top: Optional[int] = None,
                extra: Optional[torch.Tensor] = None, extra_gate: Optional[torch.Tensor] = None) -> None:
    """out[t] = sum_k weights[t, k] * rows[t * K + k] (or rows[at[t * K + k]]): fp32 sum, in the order of k.  With ``ids``
    [tokens, K], ``x`` [tokens, H] (out's dtype) and ``experts``: a pair whose id is ``experts`` or more is an identity
    expert and contributes the token's own row ``x[t]``.  ``weights=None`` (then ``top`` names K): a plain sum.  ``extra``
    [tokens, H] (out's dtype): an always-on expert's rows, added last, times sigmoid(``extra_gate[t]``) when that
    (fp32, one number a token, any row stride) is given."""
    _need_cuda("moe_combine", rows, weights, out, at, ids, x, extra, extra_gate)
    _need_i32("moe_combine", at, ids)
    T, H = out.shape
    if weights is None:
        if top is None:
            raise KernelError("moe_combine: a plain sum needs the number of rows a token")
        K = int(top)
    else:
        K = weights.shape[1]
        if weights.dtype != torch.float32 or weights.shape[0] != T or not weights.is_contiguous():
            raise KernelError("moe_combine: weights must be contiguous fp32 [tokens, K]")
    if ids is not None and (x is None or x.dtype != out.dtype or x.shape != out.shape or not x.is_contiguous() or ids.shape != (T, K)):
        raise KernelError("moe_combine: identity experts need the tokens' rows in the output's dtype and shape, and ids [tokens, K]")
    if rows.shape != (T * K, H) or not (rows.is_contiguous() and out.is_contiguous()):
        raise KernelError("moe_combine: shape or dtype mismatch")
    if extra is not None and (extra.dtype != out.dtype or extra.shape != out.shape or not extra.is_contiguous()):
        raise KernelError("moe_combine: the extra rows must have the output's dtype and shape")
    if extra_gate is not None and (extra is None or extra_gate.dtype != torch.float32 or extra_gate.shape[0] != T):
        raise KernelError("moe_combine: the extra rows' gate is fp32, one number a token")
    fn = _fn("moe", "kb_moe_combine", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(rows.data_ptr(), _is_bf16(rows, "moe_combine"), _ptr(weights), _ptr(at), K, H, out.data_ptr(), _is_bf16(out, "moe_combine"), T,
              _ptr(ids), _ptr(x), int(experts), _ptr(extra), _ptr(extra_gate), extra_gate.stride(0) if extra_gate is not None else 0,
              _stream()), "moe_combine")
