"""Python launchers of the CUDA kernels: thin, checked, allocation-free where the caller gives the output.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes), launches on the current stream and raises :class:`KernelError`
with the CUDA error text if the launch failed.  There is no CPU path: on a machine
without a GPU, or without the compiled libraries, these functions raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import Structure, byref, c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import List, Optional, Sequence, Tuple

import torch

from .build import load_library

ODI_ERR_UNSUPPORTED = 10001
ODI_ERR_ARGUMENT = 10002


class KernelError(RuntimeError):
    pass


def _cuda_error_text(code: int) -> str:
    if code == ODI_ERR_UNSUPPORTED:
        return "the kernel does not take these sizes or this alignment"
    if code == ODI_ERR_ARGUMENT:
        return "inconsistent arguments"
    try:
        rt = ctypes.CDLL("libcudart.so.12")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return f"CUDA error {code}"


# Kernels of this library launched so far in this process (library matrix products are
# counted apart); the benchmark reads the difference over its timed region.
LAUNCHES = {"own": 0, "library": 0}


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_cuda_error_text(code)} (code {code})")
    LAUNCHES["own"] += kernels


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


# the raw handle of the current stream without building a Stream object (several microseconds a launch)
_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    if _raw_current_stream is not None:
        return c_void_p(_raw_current_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _require(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


# ------------------------------------------------------------------------------ elementwise


def embed(table: torch.Tensor, ids: torch.Tensor, hidden: torch.Tensor) -> None:
    """hidden[t, :] = table[ids[t], :] into the fp32 residual stream."""
    _require(table, "table", ndim=2)
    _require(ids, "ids", torch.int32, 1)
    _require(hidden, "hidden", torch.float32, 2)
    if hidden.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"hidden is {tuple(hidden.shape)}, expected {(ids.numel(), table.shape[1])}")
    lib = load_library("elementwise")
    _check(lib.odi_embed(_ptr(table), _ptr(ids), _ptr(hidden), c_int(ids.numel()), c_int(table.shape[1]),
                         c_int(dtype_code(table.dtype)), _stream()), "embed")


def embed_sinusoid(table: torch.Tensor, ids: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, hidden: torch.Tensor,
                   scale: float) -> None:
    """hidden[t, j] = table[ids[t], j] * scale + (sin for even j, cos for odd j)(pos[t] * inv_freq[j // 2]), fp32."""
    _require(table, "table", ndim=2)
    _require(ids, "ids", torch.int32, 1)
    _require(pos, "pos", torch.int32, 1)
    _require(inv_freq, "inv_freq", torch.float32, 1)
    _require(hidden, "hidden", torch.float32, 2)
    H = table.shape[1]
    if hidden.shape != (ids.numel(), H) or pos.numel() != ids.numel() or inv_freq.numel() != (H + 1) // 2:
        raise KernelError(f"embed_sinusoid sizes disagree: hidden {tuple(hidden.shape)}, table {tuple(table.shape)}")
    lib = load_library("elementwise")
    _check(lib.odi_embed_sinusoid(_ptr(table), _ptr(ids), _ptr(pos), _ptr(inv_freq), _ptr(hidden), c_int(ids.numel()),
                                  c_int(H), c_float(scale), c_int(dtype_code(table.dtype)), _stream()), "embed_sinusoid")


def rmsnorm_adds(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: torch.Tensor) -> bool:
    """Whether :func:`rmsnorm` can take ``add`` for these tensors (the vector form: a width that is a multiple of 4
    and at most 8,192, aligned tensors, ``add`` in the dtype of ``out``)."""
    if add.dtype != out.dtype or add.shape != x.shape or not add.is_contiguous():
        return False
    lib = load_library("elementwise")
    return bool(lib.odi_rmsnorm_adds(_ptr(x), _ptr(weight), _ptr(out), _ptr(add), c_int(x.shape[1])))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None) -> None:
    """out[i] = weight * cast(x[r_i] * rsqrt(mean(x[r_i]^2) + eps)), r_i = rows[i] or i.

    ``add`` ([tokens, H] in the dtype of ``out``, without ``rows``; see :func:`rmsnorm_adds`): first x += add, in
    place, then the norm of the sum: the residual add of a product and the norm after it in one pass."""
    _require(x, "x", torch.float32, 2)
    _require(weight, "weight", torch.float32, 1)
    _require(out, "out", ndim=2)
    n = out.shape[0]
    H = x.shape[1]
    if weight.numel() != H or out.shape[1] != H:
        raise KernelError(f"rmsnorm sizes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _require(rows, "rows", torch.int32, 1)
        if rows.numel() != n:
            raise KernelError("rows and out disagree")
    elif x.shape[0] != n:
        raise KernelError("x and out disagree")
    if add is not None:
        _require(add, "add", out.dtype, 2)
        if rows is not None or add.shape != x.shape:
            raise KernelError("rmsnorm: add goes without rows and has the shape of x")
    lib = load_library("elementwise")
    _check(lib.odi_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), _ptr(rows), _ptr(add), c_int(n), c_int(H), c_float(eps),
                           c_int(dtype_code(out.dtype)), _stream()), "rmsnorm")


class _HeadPrepArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("page_start", c_void_p), ("page_ids", c_void_p),
                ("n_tokens", c_int), ("nq", c_int), ("nkv", c_int), ("d", c_int), ("rot_dim", c_int),
                ("page_size", c_int), ("ring_pages", c_int), ("write_kv", c_int), ("eps", c_float)]


def rope_table(inv_freq: torch.Tensor, tok_pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
               magnitude: float = 1.0) -> None:
    """cos_t/sin_t[t, i] = magnitude * cos/sin(tok_pos[t] * inv_freq[i]) in fp32."""
    _require(inv_freq, "inv_freq", torch.float32, 1)
    _require(tok_pos, "tok_pos", torch.int32, 1)
    _require(cos_t, "cos_t", torch.float32, 2)
    _require(sin_t, "sin_t", torch.float32, 2)
    n, half = tok_pos.numel(), inv_freq.numel()
    if cos_t.shape != (n, half) or sin_t.shape != (n, half):
        raise KernelError("rope tables must be [tokens, rot_dim / 2]")
    lib = load_library("elementwise")
    _check(lib.odi_rope_table(_ptr(inv_freq), _ptr(tok_pos), _ptr(cos_t), _ptr(sin_t), c_int(n), c_int(half),
                              c_float(magnitude), _stream()), "rope_table")


def head_prep(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, cos_t, sin_t, tok_seq, tok_pos, page_start,
              page_ids, *, nq: int, nkv: int, d: int, rot_dim: int, page_size: int, ring_pages: int,
              write_kv: bool, eps: float) -> None:
    """Per-head Q/K RMSNorm (optional), rotary embedding (optional) and cache write, fused.

    With ``qkv=None`` nothing runs: the checked argument block is returned, for the tensor-core product
    that does the same in its epilogue (``gemm_bf16(..., EPI_HEAD_PREP, head_prep=...)``; bf16 only)."""
    _require(q_out, "q_out", torch.bfloat16 if qkv is None else qkv.dtype, 2)
    n = q_out.shape[0]
    if qkv is not None:
        _require(qkv, "qkv", ndim=2)
        if qkv.shape[0] != n or qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError(f"head_prep sizes disagree: qkv {tuple(qkv.shape)}, nq={nq}, nkv={nkv}, d={d}")
    if q_out.numel() != n * nq * d:
        raise KernelError(f"head_prep sizes disagree: q_out {tuple(q_out.shape)}, nq={nq}, d={d}")
    if write_kv:
        _require(k_pool, "k_pool", q_out.dtype)
        _require(v_pool, "v_pool", q_out.dtype)
    for name, w in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w)):
        if w is not None:
            _require(w, name, torch.float32, 1)
            if w.numel() != d:
                raise KernelError(f"{name} has {w.numel()} entries, head_dim is {d}")
    if cos_t is not None:
        _require(cos_t, "cos_t", torch.float32, 2)
        _require(sin_t, "sin_t", torch.float32, 2)
        if cos_t.shape != (n, rot_dim // 2) or sin_t.shape != cos_t.shape:
            raise KernelError("rope tables must be [tokens, rot_dim / 2]")
    args = _HeadPrepArgs(_ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w), _ptr(k_norm_w),
                         _ptr(cos_t), _ptr(sin_t), _ptr(tok_seq), _ptr(tok_pos), _ptr(page_start), _ptr(page_ids),
                         n, nq, nkv, d, rot_dim, page_size, ring_pages, 1 if write_kv else 0, eps)
    if qkv is None:
        return args
    lib = load_library("elementwise")
    _check(lib.odi_head_prep(byref(args), c_int(dtype_code(qkv.dtype)), _stream()), "head_prep")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _require(gate_up, "gate_up", ndim=2)
    _require(out, "out", gate_up.dtype, 2)
    n, I = out.shape
    if gate_up.shape != (n, 2 * I):
        raise KernelError(f"silu_mul sizes disagree: {tuple(gate_up.shape)} -> {tuple(out.shape)}")
    lib = load_library("elementwise")
    _check(lib.odi_silu_mul(_ptr(gate_up), _ptr(out), c_int(n), c_int(I), c_int(dtype_code(out.dtype)), _stream()),
           "silu_mul")


def residual_add(hidden: torch.Tensor, y: torch.Tensor) -> None:
    """hidden (fp32) += y."""
    _require(hidden, "hidden", torch.float32)
    _require(y, "y")
    if hidden.numel() != y.numel():
        raise KernelError("residual_add sizes disagree")
    lib = load_library("elementwise")
    _check(lib.odi_residual_add(_ptr(hidden), _ptr(y), c_long(hidden.numel()), c_int(dtype_code(y.dtype)), _stream()),
           "residual_add")


def bias_add(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t, n] += bias[n] in place (y bf16 or fp32, bias fp32), rounded once to the dtype of y.  For the
    products that the tensor-core kernels refuse and the vendor library computes."""
    _require(y, "y", ndim=2)
    _require_bias(bias, y.shape[1])
    lib = load_library("elementwise")
    _check(lib.odi_bias_add(_ptr(y), _ptr(bias), c_long(y.shape[0]), c_int(y.shape[1]), c_int(dtype_code(y.dtype)),
                            _stream()), "bias_add")


def widen(x: torch.Tensor, out: torch.Tensor) -> None:
    _require(x, "x", torch.bfloat16)
    _require(out, "out", torch.float32)
    lib = load_library("elementwise")
    _check(lib.odi_widen(_ptr(x), _ptr(out), c_long(x.numel()), _stream()), "widen")


# ------------------------------------------------------------------------------ matrix products


def _require_bias(bias: Optional[torch.Tensor], rows: int) -> None:
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
        if bias.numel() != rows:
            raise KernelError(f"bias has {bias.numel()} entries, the weight has {rows} rows")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] w[N,K]^T (+ bias[N]) (+ residual) in true fp32; residual may be ``out`` itself."""
    _require(a, "a", torch.float32, 2)
    _require(w, "w", torch.float32, 2)
    _require(out, "out", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm sizes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if residual is not None:
        _require(residual, "residual", torch.float32, 2)
        if residual.shape != out.shape:
            raise KernelError("residual and out disagree")
    _require_bias(bias, N)
    lib = load_library("gemm_f32")
    _check(lib.odi_gemm_f32(_ptr(a), _ptr(w), _ptr(out), _ptr(residual), _ptr(bias), c_int(M), c_int(N), c_int(K),
                            c_int(K), c_int(K), c_int(N), c_int(N), _stream()), "gemm_f32")


EPI_STORE_BF16, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU, EPI_HEAD_PREP, EPI_GELU = 0, 1, 2, 3, 4, 5

_gemm_state = {}

# Scratch that the wrappers keep per device is handed to kernels by address, and a captured CUDA graph keeps
# replaying with the address it saw.  So a buffer that has to grow is not freed: it is put aside here for
# the life of the process, where a graph that still writes to it does no harm.
_outgrown = []


def _gemm_buffers(device, scratch_floats: int):
    """Scratch for split partials, tile tickets (kept zero between launches) and the error word."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    state = _gemm_state.setdefault(device, {})
    if "tickets" not in state:
        state["tickets"] = torch.zeros(16384, dtype=torch.int32, device=device)
        state["status"] = torch.zeros(4, dtype=torch.int32, device=device)
        state["scratch"] = torch.empty(1 << 22, dtype=torch.float32, device=device)
    if state["scratch"].numel() < scratch_floats:
        _outgrown.append(state["scratch"])
        state["scratch"] = torch.empty(int(scratch_floats * 1.25), dtype=torch.float32, device=device)
    return state["scratch"], state["tickets"], state["status"]


def kernel_status_word(device) -> torch.Tensor:
    """The error word of the kernels that wait on barriers, as a one-element int32 tensor on ``device``
    (0 = fine).  Whoever already copies a step's result to the host can take it along and call
    :func:`raise_on_kernel_fault` when it is not zero."""
    _, _, status = _gemm_buffers(torch.device(device), 0)
    return status[:1]


def gemm_status(device=None) -> int:
    """The error word of the tensor-core GEMM (0 = fine); reading it synchronises the device."""
    codes = [int(s["status"][0].item()) for d, s in _gemm_state.items() if "status" in s and (device is None or d == device)]
    return next((c for c in codes if c), 0)


def raise_on_kernel_fault() -> None:
    code = gemm_status()
    if code:
        names = {1: "gemm_tcgen05: the TMA producer", 2: "gemm_tcgen05: the MMA issuer", 3: "gemm_tcgen05: the epilogue",
                 21: "gemm_prefill_tcgen05: the TMA producer", 22: "gemm_prefill_tcgen05: the MMA issuer",
                 23: "gemm_prefill_tcgen05: the epilogue",
                 11: "attention_tcgen05: the TMA producer", 12: "attention_tcgen05: the MMA issuer",
                 13: "attention_tcgen05: the softmax warps",
                 31: "attention_mma (decode, TMA-fed): the TMA producer", 32: "attention_mma (decode, TMA-fed): a compute warp"}
        for state in _gemm_state.values():
            state["status"].zero_()
        if code == 33:
            raise KernelError("attention_mma (decode): the host's list of key blocks ends before a sequence's keys do "
                              "(the lengths on the device are not those the list was made for); its result is invalid")
        raise KernelError(f"a kernel gave up waiting on a barrier ({names.get(code, code)}); its result is invalid")


# Token tile for 33 to 64 tokens: 64 (one tile), or 32 (two tiles side by side, which keep the norm prologue,
# the head preparation and the sums of squares that only tiles up to 32 have).
TILE_ABOVE_32 = int(os.environ.get("ODI_GEMM_TILE_ABOVE_32", "64"))


def gemm_bf16_plan(tokens: int, n_out: int, K: int, epi: int):
    """(tile, splits) for a shape: tiles of 128 features x `tile` tokens, with enough K splits for about
    384 CTAs (at most 8, a cluster), each split at least four k-blocks of 64."""
    total_kb = -(-K // 64)
    bn = next((b for b in (16, 32) if tokens <= b), TILE_ABOVE_32 if tokens <= 64 else 64)
    tiles = -(-n_out // 128) * -(-tokens // bn)
    # measured on whole decode steps on B200: about 384 CTAs (three of 72 KB per SM) stream best,
    # in clusters of up to 8 splits (192: +7 %, 288: +2 %, 512: +7 % step time)
    target = 384
    splits = max(1, min(total_kb // 4, int(target / tiles + 0.5), 8)) if tiles < target else 1
    return bn, splits


def gemm_bf16_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return K % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_bf16_sumsq_parts(n_out: int) -> int:
    """Rows of the ``sumsq_out`` a residual product over ``n_out`` features fills: one per tile of 128."""
    return -(-n_out // 128)


def gemm_bf16_fuses_norm(tokens: int, n_out: int, K: int, epi: int) -> bool:
    """Whether the planned form of this product can take its operand through the norm prologue."""
    bn, _ = gemm_bf16_plan(tokens, n_out, K, epi)
    return bn <= 32 and tokens <= 64 and epi in (EPI_STORE_BF16, EPI_SWIGLU, EPI_HEAD_PREP)


def gemm_bf16_fuses_head_prep(tokens: int, n_out: int, K: int, *, d: int, rot_dim: int, rotated: bool,
                              write_kv: bool) -> bool:
    """Whether the planned form of the q/k/v product can prepare the heads in its epilogue: heads of 128
    (a tile of the product is a head), whole-head rotation or none, keys and values written, decode widths."""
    bn, splits = gemm_bf16_plan(tokens, n_out, K, EPI_STORE_BF16)
    return (bn <= 32 and tokens <= 64 and splits <= 8 and d == 128 and n_out % 128 == 0 and write_kv
            and (not rotated or rot_dim == d))


MERGE_SMEM_LIMIT = 96 * 1024


def gemm_bf16_fuses_merge(tokens: int, n_out: int, K: int, *, splits: int, nq: int, d: int) -> bool:
    """Whether the planned form of this residual product can take the unmerged splits of a decode attention
    (``splits`` partials per token and head, ``nq`` heads of ``d``) as its operand: decode widths, heads of a
    multiple of 64, K all the heads, and shared memory for the token tiles of a CTA's share of K."""
    bn, k_splits = gemm_bf16_plan(tokens, n_out, K, EPI_RESIDUAL)
    if bn > 32 or tokens > 64 or k_splits > 8 or not 1 <= splits <= 32 or d % 64 or nq * d != K:
        return False
    kb_cap = -(-(K // 64) // k_splits)
    heads = -(-kb_cap * 64 // d) + 1
    smem = 3 * 128 * 64 * 2 + 1024 + kb_cap * bn * 64 * 2 + bn * heads * (splits + 2) * 4
    return smem <= MERGE_SMEM_LIMIT


class _MergeArgs(Structure):
    _fields_ = [("partial", c_void_p), ("past", c_void_p), ("plan", c_void_p), ("splits", c_int), ("nq", c_int),
                ("d", c_int)]


def gemm_bf16_gives_sumsq(tokens: int, n_out: int, K: int) -> bool:
    """Whether the planned form of this residual product can leave the rows' sums of squares."""
    bn, splits = gemm_bf16_plan(tokens, n_out, K, EPI_RESIDUAL)
    return bn <= 64 and splits <= 8


def gemm_bf16(x: Optional[torch.Tensor], w: torch.Tensor, out: Optional[torch.Tensor], epi: int, *,
              bn: Optional[int] = None, splits: Optional[int] = None, cluster: bool = True,
              norm: Optional[tuple] = None, sumsq_out: Optional[torch.Tensor] = None, head_prep=None,
              bias: Optional[torch.Tensor] = None, merge: Optional[tuple] = None) -> None:
    """Tensor-core product out = epilogue(x w^T): x [tokens, K] bf16, w [rows, K] bf16.

    ``EPI_STORE_BF16`` / ``EPI_STORE_F32``: out [tokens, rows]; ``EPI_RESIDUAL``: out (fp32) += product;
    ``EPI_SWIGLU``: w holds the gate rows then the up rows, out [tokens, rows / 2] = silu(gate) * up;
    ``EPI_GELU``: out [tokens, rows] = gelu(product) in bf16 (the exact erf form).
    ``cluster``: let 2..8 K splits exchange their partials inside a thread-block cluster (else, and for
    more splits, through global scratch and a ticket).
    ``norm = (rows, weight, parts, eps)`` instead of ``x``: the operand is RMSNorm(rows) * weight with the
    roundings of :func:`rmsnorm`, made inside the kernel from the fp32 ``rows`` [tokens, K]; ``parts``
    [pieces, tokens] holds sums of squares of pieces of each row (what ``sumsq_out`` of the product that
    wrote the rows received).  Decode form only (``gemm_bf16_fuses_norm``).
    ``sumsq_out`` (fp32 [gemm_bf16_sumsq_parts(features), tokens]) with ``EPI_RESIDUAL``: receives, per tile
    of 128 features, the sums of squares of the rows the product leaves in ``out``.
    ``EPI_HEAD_PREP`` with ``head_prep`` (the block that ``head_prep(None, ...)`` returns) and ``out=None``:
    w holds query, key and value heads of 128 rows each; the epilogue rounds the projections to bf16 and
    does what :func:`head_prep` does with them (``gemm_bf16_fuses_head_prep`` says when).
    ``bias`` (fp32, one per row of w): added to the fp32 product before the epilogue's own work and rounding.
    ``merge = (partial, past, plan, splits, nq, d)`` instead of ``x``, with ``EPI_RESIDUAL``: the operand is the
    output of a decode attention whose ``splits`` partials per token and head are still apart in ``partial``
    (:func:`attention_mma` with ``combine=False``; ``plan``: its ``tiles_per_split`` or None); the kernel merges
    them as the combine kernel would, bit for bit (``gemm_bf16_fuses_merge`` says when it can).
    """
    merge_args = None
    if merge is not None:
        if x is not None or norm is not None or epi != EPI_RESIDUAL:
            raise KernelError("gemm_bf16 takes merge instead of x and norm, with EPI_RESIDUAL")
        partial, past, plan, m_splits, m_nq, m_d = merge
        _require(partial, "merge partial", torch.float32)
        _require(past, "merge past", torch.int32, 1)
        if plan is not None:
            _require(plan, "merge plan", torch.int32, 1)
        tokens = past.numel()
        if partial.numel() < tokens * m_nq * m_splits * (m_d + 2):
            raise KernelError("merge partial is smaller than tokens x heads x splits x (d + 2)")
        if not gemm_bf16_fuses_merge(tokens, w.shape[0], m_nq * m_d, splits=m_splits, nq=m_nq, d=m_d):
            raise KernelError("this product cannot take unmerged attention splits (see gemm_bf16_fuses_merge)")
        merge_args = _MergeArgs(_ptr(partial), _ptr(past), _ptr(plan), m_splits, m_nq, m_d)
        x_like = torch.empty((tokens, m_nq * m_d), dtype=torch.bfloat16, device="meta")
    if norm is not None:
        if x is not None:
            raise KernelError("gemm_bf16 takes either x or norm")
        rows, norm_w, parts, eps = norm
        _require(rows, "norm rows", torch.float32, 2)
        _require(norm_w, "norm weight", torch.float32, 1)
        _require(parts, "norm parts", torch.float32, 2)
        if norm_w.numel() != rows.shape[1] or parts.shape[1] != rows.shape[0]:
            raise KernelError(f"norm operands disagree: rows {tuple(rows.shape)}, weight {tuple(norm_w.shape)}, "
                              f"parts {tuple(parts.shape)}")
        x_like = rows
    elif merge is None:
        _require(x, "x", torch.bfloat16, 2)
        x_like = x
    _require(w, "w", torch.bfloat16, 2)
    tokens, K = x_like.shape
    w_rows = w.shape[0]
    n_out = w_rows // 2 if epi == EPI_SWIGLU else w_rows
    if epi == EPI_HEAD_PREP:
        if out is not None or head_prep is None:
            raise KernelError("EPI_HEAD_PREP takes head_prep and no out")
        if w.shape[1] != K:
            raise KernelError(f"gemm sizes disagree: x {tuple(x_like.shape)}, w {tuple(w.shape)}")
    else:
        _require(out, "out", torch.bfloat16 if epi in (EPI_STORE_BF16, EPI_SWIGLU, EPI_GELU) else torch.float32, 2)
        if w.shape[1] != K or out.shape != (tokens, n_out) or (epi == EPI_SWIGLU and w_rows % 2):
            raise KernelError(f"gemm sizes disagree: x {tuple(x_like.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if sumsq_out is not None:
        _require(sumsq_out, "sumsq_out", torch.float32, 2)
        if epi != EPI_RESIDUAL or sumsq_out.shape != (gemm_bf16_sumsq_parts(n_out), tokens):
            raise KernelError("sumsq_out goes with EPI_RESIDUAL and has one row per tile of 128 features")
    if not gemm_bf16_supported(w if merge is not None else x_like, w):
        raise KernelError(f"gemm_tcgen05 needs K a multiple of 8 and 16-byte aligned operands (K={K})")
    _require_bias(bias, w_rows)
    plan_bn, plan_splits = gemm_bf16_plan(tokens, n_out, K, epi)
    bn = plan_bn if bn is None else bn
    splits = plan_splits if splits is None else splits
    lib = load_library("gemm_tcgen05")
    lib.odi_gemm_bf16_scratch_floats.restype = c_long
    need = lib.odi_gemm_bf16_scratch_floats(c_int(tokens), c_int(n_out), c_int(bn), c_int(splits),
                                            c_int(1 if epi == EPI_SWIGLU else 0))
    tiles = -(-n_out // 128) * -(-tokens // bn)
    scratch, tickets, status = _gemm_buffers(w.device, need)
    if splits > 1 and tiles > tickets.numel() // 2:      # the upper half belongs to the many-token kernel's tile flags
        raise KernelError("too many tiles for a split product")
    if norm is not None:
        norm_args = (_ptr(norm[0]), _ptr(norm[1]), _ptr(norm[2]), c_int(norm[2].shape[0]), c_float(norm[3]))
    else:
        norm_args = (_ptr(None), _ptr(None), _ptr(None), c_int(0), c_float(0.0))
    _check(lib.odi_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(tokens), c_int(n_out), c_int(K), c_int(w_rows),
                             c_int(n_out), c_int(epi), c_int(bn), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch), _ptr(tickets), _ptr(status), *norm_args,
                             _ptr(sumsq_out), byref(head_prep) if head_prep is not None else _ptr(None), _ptr(bias),
                             c_int(0), byref(merge_args) if merge_args is not None else _ptr(None), _stream()),
           "gemm_tcgen05")


SELFTEST_WAIT_CYCLES = 20_000_000        # about ten milliseconds of SM clock


def selftest_bounded_wait(device="cuda:0") -> int:
    """Make one wait of the tensor-core GEMM run out, safely, and return the code the kernel recorded.

    One tile is launched from a build of ``gemm_tcgen05.cu`` whose waits last about ten milliseconds
    (``ODI_WAIT_CYCLES``) with a producer that requests no copy at all, so nothing is in flight: the MMA role
    gives up on its first wait, every role leaves its loop, tensor memory is freed and the kernel returns.
    The error word then holds the MMA role's code (2) and :func:`raise_on_kernel_fault` raises naming it.
    The product's own build and its two-second limit are not involved."""
    device = torch.device(device)
    x = torch.zeros((16, 256), dtype=torch.bfloat16, device=device)
    w = torch.zeros((128, 256), dtype=torch.bfloat16, device=device)
    out = torch.zeros((16, 128), dtype=torch.float32, device=device)
    scratch, tickets, status = _gemm_buffers(device, 0)
    lib = load_library("gemm_tcgen05", {"ODI_WAIT_CYCLES": SELFTEST_WAIT_CYCLES})
    none = _ptr(None)
    with torch.cuda.device(device):
        _check(lib.odi_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(16), c_int(128), c_int(256), c_int(128), c_int(128),
                                 c_int(EPI_STORE_F32), c_int(16), c_int(1), c_int(0), _ptr(scratch), _ptr(tickets),
                                 _ptr(status), none, none, none, c_int(0), c_float(0.0), none, none, none, c_int(1),
                                 none, _stream()), "gemm_tcgen05 (bounded-wait self-test)")
        torch.cuda.synchronize(device)
    return int(status[0].item())


def gemm_prefill_supported(x: torch.Tensor, w: torch.Tensor, n_out: int, out_dtype: torch.dtype) -> bool:
    """Whether :func:`gemm_prefill_bf16` takes these operands: K a multiple of 8, 16-byte aligned operands, and
    output rows that start on 16-byte boundaries (they leave through TMA stores)."""
    elem = 4 if out_dtype == torch.float32 else 2
    return gemm_bf16_supported(x, w) and (n_out * elem) % 16 == 0


PREFILL_BALANCE = int(os.environ.get("ODI_PREFILL_BALANCE", "1"))     # 0 whole tiles, 1 parts when they pay, 2..4 that many


def gemm_prefill_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], epi: int, *, head_prep=None,
                      bias: Optional[torch.Tensor] = None, balance: Optional[int] = None) -> None:
    """The persistent two-CTA tensor-core product for many tokens (``csrc/gemm_prefill_tcgen05.cu``): clusters
    of two CTAs own tiles of 256 tokens x 256 features (tcgen05.mma.cta_group::2), two accumulators in tensor
    memory so that a tile's epilogue runs under the next tile's MMAs, output by TMA store or fp32 reduce-add.
    ``balance`` (default ``ODI_PREFILL_BALANCE``, 1): with ``EPI_RESIDUAL``, cut every tile's k-blocks into up to four
    parts that different CTA pairs add into the residual, in a fixed order, when that shortens the walk (128 tiles
    on 74 pairs: two rounds whole, 1.75 in quarters); 0 whole tiles always, 2..4 that many parts.
    Same operands and epilogues as :func:`gemm_bf16`; with ``EPI_HEAD_PREP`` (``out=None``, ``head_prep`` the block
    that ``head_prep(None, ...)`` returns) a thread of the epilogue finishes a token's row of a head."""
    _require(x, "x", torch.bfloat16, 2)
    _require(w, "w", torch.bfloat16, 2)
    tokens, K = x.shape
    w_rows = w.shape[0]
    n_out = w_rows // 2 if epi == EPI_SWIGLU else w_rows
    if epi == EPI_HEAD_PREP:
        if out is not None or head_prep is None or w.shape[1] != K:
            raise KernelError("EPI_HEAD_PREP takes head_prep, no out, and weights as wide as x")
        if not gemm_bf16_supported(x, w):
            raise KernelError(f"gemm_prefill_tcgen05 needs K a multiple of 8 and 16-byte aligned operands (K={K})")
    else:
        if epi not in (EPI_STORE_BF16, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU, EPI_GELU):
            raise KernelError(f"gemm_prefill_bf16 has no epilogue {epi}")
        _require(out, "out", torch.bfloat16 if epi in (EPI_STORE_BF16, EPI_SWIGLU, EPI_GELU) else torch.float32, 2)
        if w.shape[1] != K or out.shape != (tokens, n_out) or (epi == EPI_SWIGLU and w_rows % 2):
            raise KernelError(f"gemm sizes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if not gemm_prefill_supported(x, w, n_out, out.dtype):
            raise KernelError(f"gemm_prefill_tcgen05 needs K a multiple of 8, 16-byte aligned operands and output rows "
                              f"(K={K}, {n_out} {out.dtype} per row)")
    _require_bias(bias, w_rows)
    _, tickets, status = _gemm_buffers(w.device, 0)
    # the upper half of the ticket array serves as the tiles' flags (the few-token kernel counts tiles in the lower)
    flags = tickets[tickets.numel() // 2:]
    lib = load_library("gemm_prefill_tcgen05")
    _check(lib.odi_gemm_prefill_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(tokens), c_int(n_out), c_int(K), c_int(w_rows),
                                     c_int(n_out), c_int(epi), byref(head_prep) if head_prep is not None else _ptr(None),
                                     _ptr(bias), _ptr(status), _ptr(flags), c_int(flags.numel()),
                                     c_int(PREFILL_BALANCE if balance is None else balance), _stream()),
           "gemm_prefill_tcgen05")


# ------------------------------------------------------------------------------ attention


class _AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("out", c_void_p),
                ("partial", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int), ("page_size", c_int),
                ("ring_pages", c_int), ("window", c_int), ("splits", c_int), ("bq", c_int),
                ("head_chunks", c_int), ("scale", c_float), ("softcap", c_float), ("sink", c_int), ("keep", c_int)]


SIMT_HEAD_DIMS = tuple(range(16, 513, 16))


def attention_simt(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                   nq: int, nkv: int, d: int, page_size: int, ring_pages: int, window: int, scale: float,
                   splits: int = 1, partial: Optional[torch.Tensor] = None, dv: Optional[int] = None,
                   shared_kv: bool = False, softcap: float = 0.0, sink: bool = False, keep: int = 0) -> None:
    """Causal GQA over the paged cache for any mixture of prompt and decode sequences.  ``softcap`` c > 0:
    scores (times ``scale``) become c tanh(score / c) before the softmax.  ``sink``: the softmax has one more
    term of score 0 and no value, p_j = exp(s_j) / (1 + sum_k exp(s_k)).  ``keep`` > 0 with a window: the first
    ``keep`` positions of a sequence stay visible beyond the window (a ring then has their pages pinned in front).

    ``dv`` (default ``d``): width of the value rows and of the output.  ``shared_kv``: a cached row is key and
    value at once (the value is its first ``dv`` lanes; ``v_pool`` is None), as in attention over a latent
    cache; ``d`` may then be any multiple of 4."""
    dv = d if dv is None else dv
    plain = dv == d and not shared_kv and (d in SIMT_HEAD_DIMS or d % 4 != 0 or d > 1024)
    if plain and d not in SIMT_HEAD_DIMS:
        raise KernelError(f"attention takes head sizes in steps of 16 up to 512, not {d}")
    if not plain and (d % 4 != 0 or not 4 <= d <= 1024 or dv <= 0 or (shared_kv and dv > d)):
        raise KernelError(f"attention with a value width of its own takes key widths in steps of 4 up to 1024 "
                          f"and values no wider than a shared row (d={d}, dv={dv})")
    _require(q, "q")
    _require(out, "out", q.dtype)
    _require(k_pool, "k_pool", q.dtype)
    if shared_kv:
        if v_pool is not None:
            raise KernelError("attention over shared rows takes no value pool")
    else:
        _require(v_pool, "v_pool", q.dtype)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != n_tokens * nq * dv:
        raise KernelError("q and out disagree")
    if splits > 1:
        need = n_tokens * nq * splits * (dv + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    args = _AttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(partial), _ptr(cu_q), _ptr(past),
                     _ptr(page_start), _ptr(page_ids), n_seqs, nq, nkv, page_size, ring_pages, window, splits,
                     0, 0, scale, softcap, 1 if sink else 0, keep)
    defines = {"ODI_HEAD_DIM": d}
    if not plain:
        defines.update({"ODI_VALUE_DIM": dv, "ODI_SHARED_KV": 1 if shared_kv else 0})
    lib = load_library("attention_simt", defines)
    _check(lib.odi_attention_simt(byref(args), c_int(max_q_len), c_int(n_tokens), c_int(dtype_code(q.dtype)),
                                  _stream()), "attention_simt", 2 if splits > 1 else 1)


class _LatentAttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("pool", c_void_p), ("out", c_void_p), ("partial", c_void_p), ("cu_q", c_void_p),
                ("past", c_void_p), ("page_start", c_void_p), ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int),
                ("ring_pages", c_int), ("window", c_int), ("splits", c_int), ("bq", c_int), ("head_chunks", c_int),
                ("scale", c_float)]


def attention_latent_supported(dtype: torch.dtype, d: int, dv: int, page_size: int) -> bool:
    """Whether :func:`attention_latent` takes these rows: bfloat16, rows in steps of 16 up to 1024 lanes, values in
    steps of 16 up to 512 lanes and no wider than a row, pages of 64."""
    return (dtype == torch.bfloat16 and page_size == 64 and d % 16 == 0 and dv % 16 == 0 and 16 <= d <= 1024
            and 16 <= dv <= min(d, 512))


def attention_latent(q, pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int, nq: int, d: int,
                     dv: int, page_size: int, ring_pages: int, window: int, scale: float, splits: int = 1,
                     partial: Optional[torch.Tensor] = None) -> None:
    """bf16 causal attention over shared rows on the tensor cores: a cached row of ``d`` lanes is the key of every
    query head and its first ``dv`` lanes are the value, as in attention over a latent cache.  Any mixture of single
    tokens and portions of prompts; ``window`` 0 for none (the cache may be a ring of pages); with ``splits`` > 1
    each sequence's visible keys are cut into that many ranges and ``partial`` (fp32, tokens * nq * splits * (dv + 2))
    holds their results for the combine kernel."""
    if not attention_latent_supported(q.dtype, d, dv, page_size):
        raise KernelError(f"attention_latent takes bfloat16 rows in steps of 16 up to 1024, values up to 512 and pages "
                          f"of 64 (d={d}, dv={dv}, page_size={page_size})")
    _require(q, "q", torch.bfloat16)
    _require(out, "out", torch.bfloat16)
    _require(pool, "pool", torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != n_tokens * nq * dv or pool.shape[-1] != d:
        raise KernelError("attention_latent sizes disagree")
    if splits > 1:
        need = n_tokens * nq * splits * (dv + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    args = _LatentAttnArgs(_ptr(q), _ptr(pool), _ptr(out), _ptr(partial), _ptr(cu_q), _ptr(past), _ptr(page_start),
                           _ptr(page_ids), n_seqs, nq, ring_pages, window, splits, 0, 0, scale)
    lib = load_library("attention_latent_mma", {"ODI_HEAD_DIM": d, "ODI_VALUE_DIM": dv})
    _check(lib.odi_attention_latent_mma(byref(args), c_int(max_q_len), c_int(n_tokens), c_int(page_size), _stream()),
           "attention_latent", 2 if splits > 1 else 1)


class _MmaAttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("out", c_void_p),
                ("partial", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int), ("splits", c_int),
                ("head_chunks", c_int), ("scale", c_float), ("clustered", c_int), ("tickets", c_void_p),
                ("tiles_per_split", c_void_p), ("pool_rows", c_long), ("status", c_void_p), ("items", c_int),
                ("skip_combine", c_int)]


MMA_HEAD_DIMS = tuple(range(16, 257, 16))

_attention_state = {}


def _attention_tickets(device, count: int) -> torch.Tensor:
    """Counters of the split-key decode attention, one per (sequence, block row); kept zero between launches."""
    have = _attention_state.get(device)
    if have is None or have.numel() < count:
        if have is not None:
            _outgrown.append(have)
        have = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _attention_state[device] = have
    return have


DECODE_ATTENTION_BLOCKS = 296     # blocks of the split-key decode kernel that a B200 holds at once (148 SMs x 2)
ROUND_FILL_CUTS = 6               # the most cuts per sequence when whole sequences already run in rounds


def plan_key_splits(kv_lens: Sequence[int], block_rows: int, *, blocks: int = DECODE_ATTENTION_BLOCKS,
                    min_tiles: int = 2, max_splits: int = 32) -> Tuple[int, int]:
    """How the split-key decode attention cuts unequal sequences: ``(tiles_per_split, splits)``.

    ``kv_lens`` are the keys that each sequence sees, ``block_rows`` the blocks that one split of one
    sequence launches (kv heads x chunks of 16 query heads).  Every block takes ``tiles_per_split`` tiles
    of 64 keys, so a long sequence gets more blocks than a short one and all blocks end together; the
    size is the smallest (from ``min_tiles`` up) with which all blocks are on the GPU at once, or the
    longest sequence whole when even that is too many.  ``splits`` is what the longest sequence needs; more
    than 32 measured slower even where they would fill the GPU exactly (one sequence of 131,072 keys, 8 kv
    heads: 95 us with 32, 103 with 37, 108 with 64), since every split adds to the merge."""
    tiles = [max(1, -(-int(n) // 64)) for n in kv_lens]
    longest, total = max(tiles), sum(tiles)
    per = max(min_tiles, -(-total * block_rows // blocks), -(-longest // max_splits))
    for _ in range(64):
        if per >= longest or sum(-(-t // per) for t in tiles) * block_rows <= blocks:
            break
        per += max(1, per // 8)
    per = min(per, longest)
    if per == longest and len(tiles) * block_rows > blocks:
        # More whole sequences than the GPU holds blocks: they run in rounds, and the last round may be nearly
        # empty (40 sequences x 8 kv heads: 320 blocks on 296 places, two rounds for 1.08).  A few cuts per
        # sequence fill the rounds better.  Estimate: rounds x (tiles of a block + 4 for its start and end), plus
        # 6 for the merge when there are cuts; measured at 2,048 keys (us, whole / best cut): 40 sequences 80 /
        # 69 (3 to 5 cuts), 48: 83 / 76 (3 cuts), 56: 85 / 90, 64: 87 / 101 (whole sequences stay).
        def estimate(size: int) -> float:
            count = sum(-(-t // size) for t in tiles) * block_rows
            return -(-count // blocks) * (size + 4) + (6 if size < longest else 0)
        best, best_cost = longest, estimate(longest)
        for cuts in range(2, min(max_splits, ROUND_FILL_CUTS) + 1):
            size = -(-longest // cuts)
            if size < min_tiles:
                break
            cost = estimate(size)
            if cost < best_cost:
                best, best_cost = size, cost
        per = best
    return per, -(-longest // per)


def key_split_capacity(n_seqs: int, block_rows: int, *, blocks: int = DECODE_ATTENTION_BLOCKS, max_splits: int = 32) -> int:
    """The most (sequence, split) pairs that :func:`plan_key_splits` gives ``n_seqs`` sequences, whatever their
    lengths: what fills the GPU once, or every sequence whole; with more whole sequences than the GPU holds
    blocks, every sequence may be cut ``ROUND_FILL_CUTS`` times."""
    if n_seqs * block_rows > blocks:
        return n_seqs * min(max_splits, ROUND_FILL_CUTS)
    return min(n_seqs * max_splits, max(n_seqs, blocks // block_rows))


def key_split_list(kv_lens: Sequence[int], tiles_per_split: int, capacity: int) -> List[int]:
    """The decode attention's list of blocks for sequences of ``kv_lens`` keys cut every ``tiles_per_split`` tiles
    of 64: ``[tiles_per_split, n, entry...]`` padded with zeros to ``2 + capacity``.  An entry is
    ``sequence << 8 | 128 if it is the sequence's last | split``; blocks with the most tiles come first, so that
    when the blocks run in more than one round the short ones fill the end.  The list holds for every bound on
    the splits that the longest sequence fits (``splits * tiles_per_split`` tiles)."""
    per = max(1, int(tiles_per_split))
    entries = []
    for seq, n in enumerate(kv_lens):
        tiles = max(1, -(-int(n) // 64))
        count = -(-tiles // per)
        if count > 128:
            raise KernelError(f"{count} blocks for one sequence; an entry of the list holds up to 128")
        entries.extend((-per, seq, split, False) for split in range(count - 1))
        entries.append((-(tiles - (count - 1) * per), seq, count - 1, True))
    if len(entries) > capacity:
        raise KernelError(f"{len(entries)} blocks of keys for a list of {capacity}: the plan and the graph disagree")
    entries.sort()
    packed = [(seq << 8) | (128 if last else 0) | split for _, seq, split, last in entries]
    return [per, len(packed)] + packed + [0] * (capacity - len(packed))


def attention_mma(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                  nq: int, nkv: int, d: int, page_size: int, scale: float, splits: int = 1,
                  partial: Optional[torch.Tensor] = None, cluster: bool = False, merge_in_kernel: bool = False,
                  tiles_per_split: Optional[torch.Tensor] = None, combine: bool = True) -> None:
    """bf16 causal GQA on the tensor cores: the prefill kernel for any q_len, the split-key
    decode kernel when every sequence brings exactly one token.  No window.

    Decode with ``tiles_per_split`` (int32 on the device, written by the host; see
    :func:`plan_key_splits`): every block takes that many tiles of 64 keys and ``splits`` only bounds the
    count per sequence; whatever the number says, ``splits`` blocks cover every sequence.  With one element the
    grid has ``splits`` blocks for every sequence and those without keys leave at once; with more it is a
    :func:`key_split_list`, the grid is as long as the list's capacity (or ``n_seqs * splits`` if that is less),
    and a list that does not cover the lengths on the device is reported through the kernels' status word.  Without it every sequence is cut into
    ``splits`` equal ranges.

    Decode splits go through the fp32 ``partial`` buffer and a combine kernel; ``combine=False`` leaves them in
    ``partial`` unmerged (``out`` may then be None) for a product that takes them as its operand
    (:func:`gemm_bf16` with ``merge``).  ``merge_in_kernel=True``
    lets the block that finishes a (sequence, kv head) last merge them instead (an atomic ticket; the same
    bits); on B200 that measured slower (20.1 against 17.5 us at 8 x 2048 with 4 splits, 17.1 against 10.8 us
    at 1 x 2048 with 16: the fence, the ticket and the merge lengthen the slowest block).  ``cluster=True``
    merges 2..8 splits inside a thread-block cluster instead (no scratch, no second kernel); on
    B200 that measured no faster (19.4 against 19.3 us at 8 x 2048, slower at other split counts:
    the co-scheduling of 104 KB blocks costs what the saved launch gains), so it is not the default."""
    if d not in MMA_HEAD_DIMS:
        raise KernelError(f"the tensor-core attention takes head sizes in steps of 16 up to 256, not {d}")
    if page_size != 64:
        raise KernelError("the tensor-core attention works on pages of 64 positions")
    _require(q, "q", torch.bfloat16)
    _require(k_pool, "k_pool", torch.bfloat16)
    _require(v_pool, "v_pool", torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    decode = max_q_len == 1
    if not decode:
        splits = 1
    clustered = cluster and 1 < splits <= 8
    if not combine and (not decode or splits == 1 or clustered or merge_in_kernel):
        raise KernelError("combine=False belongs to the decode kernel with more than one split and global partials")
    if combine or out is not None:
        _require(out, "out", torch.bfloat16)
        if out.numel() != q.numel():
            raise KernelError("q and out disagree")
    if splits > 1 and not clustered:
        need = n_tokens * nq * splits * (d + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    tickets = None
    if decode and splits > 1 and not clustered and merge_in_kernel:
        tickets = _attention_tickets(q.device, n_seqs * nkv * (-(-(nq // nkv) // 16)))
    if tiles_per_split is not None:
        if not decode or clustered or tickets is not None:
            raise KernelError("tiles_per_split belongs to the decode kernel with the combine kernel")
        _require(tiles_per_split, "tiles_per_split", torch.int32)
        if tiles_per_split.numel() == 2:
            raise KernelError("tiles_per_split is one number or a list of 2 + capacity")
    # the grid: as long as the list, but no longer than `splits` blocks for every sequence, which no list exceeds
    # (blocks behind the list's end leave at once, yet each costs a place on an SM for a moment: 64 whole
    # sequences on a grid for six cuts each measured 4 % more per step)
    items = min(tiles_per_split.numel() - 2, n_seqs * splits) if tiles_per_split is not None and tiles_per_split.numel() > 1 else 0
    # what the TMA-fed decode form needs besides: the pools' extent (rows of d) and the error word of its bounded waits
    pool_rows = k_pool.numel() // d if k_pool.numel() == v_pool.numel() else 0
    _, _, status = _gemm_buffers(q.device, 0)
    args = _MmaAttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(partial), _ptr(cu_q), _ptr(past),
                        _ptr(page_start), _ptr(page_ids), n_seqs, nq, nkv, splits, 0, scale, 1 if clustered else 0,
                        _ptr(tickets), _ptr(tiles_per_split if decode else None), pool_rows, _ptr(status), items,
                        0 if combine else 1)
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_mma(byref(args), c_int(max_q_len), c_int(n_tokens), c_int(1 if decode else 0),
                                 _stream()), "attention_mma",
           2 if (splits > 1 and not clustered and tickets is None and combine) else 1)


def attention_mma_combine(partial: torch.Tensor, out: torch.Tensor, past: torch.Tensor, *, nq: int, d: int, splits: int,
                          tiles_per_split: Optional[torch.Tensor] = None) -> None:
    """Merge the ``splits`` partials per token and head that :func:`attention_mma` left with ``combine=False``
    into ``out`` [tokens, nq * d] (the kernel that the launch would have run itself)."""
    _require(partial, "partial", torch.float32)
    _require(out, "out", torch.bfloat16)
    _require(past, "past", torch.int32, 1)
    tokens = past.numel()
    if d not in MMA_HEAD_DIMS or out.numel() != tokens * nq * d or partial.numel() < tokens * nq * splits * (d + 2):
        raise KernelError("attention_mma_combine: sizes disagree")
    if tiles_per_split is not None:
        _require(tiles_per_split, "tiles_per_split", torch.int32)
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_mma_combine(_ptr(partial), _ptr(out), c_int(tokens), c_int(nq), c_int(splits), _ptr(past),
                                         _ptr(tiles_per_split), _stream()), "attention_mma_combine")


class _TcAttnArgs(Structure):
    _fields_ = [("out", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("status", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int),
                ("scale", c_float), ("window", c_int), ("ring_pages", c_int), ("softcap", c_float), ("sink", c_int),
                ("keep", c_int)]


TCGEN05_ATTENTION_HEAD_DIMS = (64, 128)


def attention_tcgen05(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                      nq: int, nkv: int, d: int, page_size: int, scale: float, heads_per_cta: int = 0, window: int = 0,
                      ring_pages: int = 0, softcap: float = 0.0, sink: bool = False, keep: int = 0) -> None:
    """bf16 causal GQA for prefill on tcgen05: scores and outputs in tensor memory, TMA-fed pages.
    ``sink``: one more term of score 0 and no value in the softmax.
    ``window`` > 0 keeps the last ``window`` keys visible (``ring_pages`` > 0: the page lists are rings);
    ``softcap`` c > 0 squashes the scores (times ``scale``) by c tanh(score / c).
    ``heads_per_cta``: 1, or 2 (two heads of a key/value group share a CTA and its K/V pages; needs an
    even group size), or 0 for the library's choice."""
    if d not in TCGEN05_ATTENTION_HEAD_DIMS:
        raise KernelError(f"the tcgen05 attention takes head sizes {TCGEN05_ATTENTION_HEAD_DIMS}, not {d}")
    if page_size != 64:
        raise KernelError("the tcgen05 attention works on pages of 64 positions")
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _require(t, name, torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != q.numel() or k_pool.shape != v_pool.shape or k_pool.dim() != 4:
        raise KernelError("attention_tcgen05: q/out or the pools disagree")
    _, _, status = _gemm_buffers(q.device, 0)
    args = _TcAttnArgs(_ptr(out), _ptr(cu_q), _ptr(past), _ptr(page_start), _ptr(page_ids), _ptr(status),
                       n_seqs, nq, nkv, scale, window, ring_pages, softcap, 1 if sink else 0, keep)
    lib = load_library("attention_tcgen05", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), byref(args), c_int(n_tokens),
                                     c_int(max_q_len), c_long(k_pool.shape[0]), c_int(heads_per_cta), _stream()),
           "attention_tcgen05")


# ------------------------------------------------------------------------------ norms and activations in fp32


def rmsnorm_scaled(x: torch.Tensor, scale: torch.Tensor, eps: float, out: torch.Tensor,
                   rows: Optional[torch.Tensor] = None) -> None:
    """out[i] = cast(x[r_i] * rsqrt(mean(x[r_i]^2) + eps) * scale): the scaling in fp32, one rounding."""
    _require(x, "x", torch.float32, 2)
    _require(scale, "scale", torch.float32, 1)
    _require(out, "out", ndim=2)
    n, H = out.shape
    if scale.numel() != H or x.shape[1] != H:
        raise KernelError(f"rmsnorm sizes disagree: x {tuple(x.shape)}, scale {tuple(scale.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _require(rows, "rows", torch.int32, 1)
        if rows.numel() != n:
            raise KernelError("rows and out disagree")
    elif x.shape[0] != n:
        raise KernelError("x and out disagree")
    lib = load_library("elementwise")
    _check(lib.odi_rmsnorm_scaled(_ptr(x), _ptr(scale), _ptr(out), _ptr(rows), c_int(n), c_int(H), c_float(eps),
                                  c_int(dtype_code(out.dtype)), _stream()), "rmsnorm_scaled")


def gated_clamp(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), for
    ``gate_up`` [tokens, 2 F] (gate lanes, then up lanes)."""
    _require(gate_up, "gate_up", ndim=2)
    _require(out, "out", gate_up.dtype, 2)
    rows, F = out.shape
    if gate_up.shape != (rows, 2 * F):
        raise KernelError(f"gated_clamp sizes disagree: {tuple(gate_up.shape)} -> {tuple(out.shape)}")
    lib = load_library("moe")
    _check(lib.odi_gated_clamp(_ptr(gate_up), _ptr(out), c_int(rows), c_int(F), c_float(limit), c_float(alpha),
                               c_int(dtype_code(out.dtype)), _stream()), "gated_clamp")


# ------------------------------------------------------------------------------ latent attention


class _LatentPrepArgs(Structure):
    _fields_ = [("proj", c_void_p), ("q_abs", c_void_p), ("pool", c_void_p), ("norm_w", c_void_p),
                ("cos_t", c_void_p), ("sin_t", c_void_p), ("tok_seq", c_void_p), ("tok_pos", c_void_p),
                ("page_start", c_void_p), ("page_ids", c_void_p),
                ("n_tokens", c_int), ("ld", c_int), ("heads", c_int), ("d", c_int), ("r", c_int), ("R", c_int),
                ("rot_dims", c_int), ("interleaved", c_int), ("page_size", c_int), ("ring_pages", c_int),
                ("write_cache", c_int), ("eps", c_float), ("latent_out", c_void_p), ("key_rot_out", c_void_p),
                ("row", c_int), ("down", c_void_p), ("ld_down", c_int), ("has_down", c_int)]


def latent_prep(proj: torch.Tensor, q_abs: torch.Tensor, pool: torch.Tensor, norm_w: torch.Tensor, cos_t, sin_t,
                tok_seq, tok_pos, page_start, page_ids, *, heads: int, d: int, r: int, R: int, rot_dims: int,
                interleaved: bool, page_size: int, ring_pages: int, write_cache: bool, eps: float,
                latent_out: Optional[torch.Tensor] = None, key_rot_out: Optional[torch.Tensor] = None,
                row: Optional[int] = None, down: Optional[torch.Tensor] = None, has_down: bool = True,
                trailing: int = 0) -> None:
    """From the fused query / down projection ``proj`` [tokens, heads (d + r) + R + r]: the normed latent and the
    rotated shared key lanes into the token's cache row, each head's rotated query lanes into lanes R.. of
    ``q_abs`` [tokens, heads, row] (see ``csrc/latent.cu``).  ``row`` (default R + r) is the width of a cache row and
    of a head's absorbed query; lanes beyond R + r are left as they are (zero).  With ``down`` ([tokens, >= R + r],
    the down projection in its first lanes) ``proj`` holds the queries only; ``has_down`` False (a layer that reads
    another layer's cache rows) prepares the queries and nothing else.  ``trailing``: lanes of ``proj`` behind all
    of these that belong to somebody else (a gate computed by the same product)."""
    row = R + r if row is None else row
    _require(proj, "proj", ndim=2)
    _require(q_abs, "q_abs", proj.dtype)
    n = proj.shape[0]
    apart = down is not None or not has_down
    if has_down:
        _require(pool, "pool", proj.dtype)
        _require(norm_w, "norm_w", torch.float32, 1)
        if norm_w.numel() != R or pool.shape[-1] != row:
            raise KernelError("latent_prep sizes disagree")
    elif write_cache or latent_out is not None:
        raise KernelError("latent_prep without a down projection writes no cache rows")
    if down is not None:
        _require(down, "down", proj.dtype, 2)
        if down.shape[0] != n or down.shape[1] < R + r:
            raise KernelError("latent_prep: down is [tokens, >= R + r]")
    if (proj.shape[1] != heads * (d + r) + (0 if apart else R + r) + trailing or trailing < 0 or q_abs.numel() != n * heads * row or row < R + r):
        raise KernelError("latent_prep sizes disagree")
    if rot_dims > 0:
        _require(cos_t, "cos_t", torch.float32, 2)
        _require(sin_t, "sin_t", torch.float32, 2)
        if cos_t.shape != (n, rot_dims // 2) or sin_t.shape != cos_t.shape:
            raise KernelError("rotary tables do not fit the tokens")
    if (latent_out is None) != (key_rot_out is None):
        raise KernelError("latent_out and key_rot_out go together")
    if latent_out is not None:
        _require(latent_out, "latent_out", proj.dtype, 2)
        _require(key_rot_out, "key_rot_out", proj.dtype, 2)
        if latent_out.shape != (n, R) or key_rot_out.shape != (n, r):
            raise KernelError("latent_out is [tokens, R] and key_rot_out [tokens, r]")
    args = _LatentPrepArgs(_ptr(proj), _ptr(q_abs), _ptr(pool), _ptr(norm_w), _ptr(cos_t), _ptr(sin_t), _ptr(tok_seq),
                           _ptr(tok_pos), _ptr(page_start), _ptr(page_ids), n, proj.shape[1], heads, d, r, R, rot_dims,
                           1 if interleaved else 0, page_size, ring_pages, 1 if write_cache else 0, eps,
                           _ptr(latent_out), _ptr(key_rot_out), row, _ptr(down), 0 if down is None else down.shape[1],
                           1 if has_down else 0)
    lib = load_library("latent")
    _check(lib.odi_latent_prep(byref(args), c_int(dtype_code(proj.dtype)), _stream()), "latent_prep")


def slice_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, col: int = 0) -> None:
    """out[t] = cast(x[t, col : col + Q] / sqrt(mean of squares + eps) * weight), Q = len(weight): the RMS norm of a
    slice of a wider product, statistics and scaling in fp32, one rounding."""
    _require(x, "x", ndim=2)
    _require(weight, "weight", torch.float32, 1)
    _require(out, "out", x.dtype, 2)
    Q = weight.numel()
    if out.shape != (x.shape[0], Q) or col < 0 or col + Q > x.shape[1]:
        raise KernelError(f"slice_norm sizes disagree: x {tuple(x.shape)}, col {col}, weight {Q}, out {tuple(out.shape)}")
    lib = load_library("latent")
    _check(lib.odi_slice_norm(_ptr(x), _ptr(weight), _ptr(out), c_int(x.shape[0]), c_int(x.shape[1]), c_int(col), c_int(Q),
                              c_float(eps), c_int(dtype_code(x.dtype)), _stream()), "slice_norm")


def gate_heads(x: torch.Tensor, gate: torch.Tensor, *, heads: int, dv: int, lanes: int, col: int = 0,
               per_head: bool = False) -> None:
    """x[t, h, i] *= sigmoid(gate[t, col + h dv + i]) for i < dv, in place; ``x`` is [tokens, heads * lanes]
    (lanes >= dv; the lanes beyond stay), ``gate`` a product whose rows hold the gate's lanes from ``col`` on.
    ``per_head``: the gate has one lane per head, gate[t, col + h], for all of the head's lanes."""
    _require(x, "x", ndim=2)
    _require(gate, "gate", x.dtype, 2)
    n = x.shape[0]
    if (x.shape[1] != heads * lanes or gate.shape[0] != n or lanes < dv or col < 0
            or col + heads * (1 if per_head else dv) > gate.shape[1]):
        raise KernelError(f"gate_heads sizes disagree: x {tuple(x.shape)}, gate {tuple(gate.shape)}, heads={heads}, dv={dv}")
    lib = load_library("latent")
    _check(lib.odi_gate_heads(_ptr(x), _ptr(gate), c_int(n), c_int(heads), c_int(dv), c_int(lanes), c_int(gate.shape[1]),
                              c_int(col), c_int(1 if per_head else 0), c_int(dtype_code(x.dtype)), _stream()), "gate_heads")


class _LatentExpandArgs(Structure):
    _fields_ = [("proj", c_void_p), ("q_abs", c_void_p), ("k_plain", c_void_p), ("key_rot", c_void_p), ("v", c_void_p),
                ("q_full", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("tok_seq", c_void_p),
                ("cu_q", c_void_p), ("page_start", c_void_p),
                ("n_tokens", c_int), ("ld", c_int), ("heads", c_int), ("d", c_int), ("r", c_int), ("R", c_int),
                ("dv", c_int), ("Dh", c_int), ("page_size", c_int), ("row", c_int)]


def latent_expand(proj, q_abs, k_plain, key_rot, v, q_full, k_pool, v_pool, tok_seq, cu_q, page_start, *, heads: int,
                  d: int, r: int, R: int, dv: int, Dh: int, page_size: int, row: Optional[int] = None) -> None:
    """Whole heads of ``Dh`` lanes for prompts that start their sequences (``csrc/latent.cu``): queries into ``q_full``
    [tokens, heads, Dh], keys and values into pools [pages, heads, page_size, Dh] where sequence s holds the pages
    from ``page_start[s]`` on, in order."""
    n = proj.shape[0]
    for name, t in (("proj", proj), ("q_abs", q_abs), ("k_plain", k_plain), ("key_rot", key_rot), ("v", v),
                    ("q_full", q_full), ("k_pool", k_pool), ("v_pool", v_pool)):
        _require(t, name, proj.dtype)
    if (k_plain.shape != (n, heads * d) or v.shape != (n, heads * dv) or key_rot.shape != (n, r)
            or q_full.numel() != n * heads * Dh or k_pool.shape[1:] != (heads, page_size, Dh) or v_pool.shape != k_pool.shape):
        raise KernelError("latent_expand sizes disagree")
    args = _LatentExpandArgs(_ptr(proj), _ptr(q_abs), _ptr(k_plain), _ptr(key_rot), _ptr(v), _ptr(q_full), _ptr(k_pool),
                             _ptr(v_pool), _ptr(tok_seq), _ptr(cu_q), _ptr(page_start), n, proj.shape[1], heads, d, r, R,
                             dv, Dh, page_size, R + r if row is None else row)
    lib = load_library("latent")
    _check(lib.odi_latent_expand(byref(args), c_int(dtype_code(proj.dtype)), _stream()), "latent_expand")


# ------------------------------------------------------------------------------ grouped products and routing


class _GroupedArgs(Structure):
    _fields_ = [("A", c_void_p), ("W", c_void_p), ("C", c_void_p), ("row_index", c_void_p), ("tile_group", c_void_p),
                ("tile_row0", c_void_p), ("tile_rows", c_void_p), ("n_tiles", c_void_p),
                ("a_group_off", ctypes.c_longlong), ("w_group_stride", ctypes.c_longlong), ("c_group_off", ctypes.c_longlong),
                ("lda", c_int), ("ldw", c_int), ("ldc", c_int), ("M", c_int), ("N", c_int), ("K", c_int),
                ("groups", c_int), ("index_div", c_int), ("epi", c_int), ("limit", c_float), ("alpha", c_float)]


GROUPED_STORE, GROUPED_STORE_F32, GROUPED_GATED_CLAMP, GROUPED_GELU_ERF, GROUPED_GELU_TANH, GROUPED_RELU2 = 0, 1, 2, 3, 4, 5


FEW_ROWS = 4      # row tile of the grouped product's form for single-token steps (weights through registers only)


def grouped_rows_tile(rows_per_group: float, few_rows_ok: bool = False) -> int:
    """Row tile of the grouped product for groups of about this many rows: 4 (if the operands allow the form for
    few rows), 16 or 64."""
    if few_rows_ok and rows_per_group <= FEW_ROWS:
        return FEW_ROWS
    return 64 if rows_per_group > 32 else 16


def grouped_few_rows_ok(K_values: Sequence[int], dtype: torch.dtype) -> bool:
    """Whether products over these inner sizes can take the form for few rows (multiples of 8, and four rows of
    floats within the shared memory of a block)."""
    return all(K % 8 == 0 and 4 * FEW_ROWS * K <= 200 * 1024 for K in K_values)


def grouped_gemm_heads(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, *, a_col: int, a_stride: int, c_col: int,
                       c_stride: int, K: int, out_f32: bool = False) -> None:
    """One product per head in one launch: for head g, ``c[:, c_col + g c_stride : +N] = a[:, a_col + g a_stride :
    +K] w[g]^T`` with ``w`` [heads, N, K]; ``a`` and ``c`` are 2-D and contiguous, fp32 accumulation in k order."""
    _require(a, "a", w.dtype, 2)
    _require(w, "w", ndim=3)
    _require(c, "c", torch.float32 if out_f32 else w.dtype, 2)
    groups, N, Kw = w.shape
    M = a.shape[0]
    if Kw != K or c.shape[0] != M or a_col + (groups - 1) * a_stride + K > a.shape[1] \
            or c_col + (groups - 1) * c_stride + N > c.shape[1]:
        raise KernelError(f"grouped product sizes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    args = _GroupedArgs(a.data_ptr() + a_col * a.element_size(), _ptr(w), c.data_ptr() + c_col * c.element_size(),
                        None, None, None, None, None, a_stride, N * K, c_stride, a.shape[1], K, c.shape[1], M, N, K,
                        groups, 1, GROUPED_STORE_F32 if out_f32 else GROUPED_STORE, 0.0, 0.0)
    lib = load_library("grouped_gemm")
    # up to four rows: the form that streams the weights; five to eight rows too when the inner size is long (the
    # tile form would walk it in a few blocks per head), in two row tiles; else tiles of 16 or 64 rows
    few = M <= 2 * FEW_ROWS and (M <= FEW_ROWS or K >= 256) and bool(lib.odi_grouped_gemm_takes_few_rows(byref(args)))
    tm = FEW_ROWS if few else grouped_rows_tile(M)
    _check(lib.odi_grouped_gemm(byref(args), c_int(0), c_int(tm), c_int(dtype_code(w.dtype)), _stream()), "grouped_gemm")


def grouped_gemm_routed(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, table: "RoutingTable", *, gather: bool,
                        epi: int, limit: float = 0.0, alpha: float = 0.0) -> None:
    """The product of each routed row with its expert's matrix ``w[e]`` ([experts, rows, K]; with
    ``GROUPED_GATED_CLAMP`` rows = N gate rows then N up rows).  Rows are taken in ``table``'s sorted order; with
    ``gather`` row i reads ``a[perm[i] // top]`` (the token's input), else ``a[i]``; row i of ``c`` is written."""
    _require(a, "a", w.dtype, 2)
    _require(w, "w", ndim=3)
    _require(c, "c", torch.float32 if epi == GROUPED_STORE_F32 else w.dtype, 2)
    experts, w_rows, K = w.shape
    N = w_rows // 2 if epi == GROUPED_GATED_CLAMP else w_rows
    if a.shape[1] != K or c.shape != (table.n_pairs, N) or experts != table.n_experts:
        raise KernelError(f"routed product sizes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)}")
    args = _GroupedArgs(_ptr(a), _ptr(w), _ptr(c), _ptr(table.perm) if gather else None, _ptr(table.tile_group),
                        _ptr(table.tile_row0), _ptr(table.tile_rows), _ptr(table.n_tiles), 0, w_rows * K, 0,
                        K, K, N, 0, N, K, experts, table.top if gather else 1, epi, limit, alpha)
    lib = load_library("grouped_gemm")
    _check(lib.odi_grouped_gemm(byref(args), c_int(table.max_tiles), c_int(table.tm), c_int(dtype_code(w.dtype)),
                                _stream()), "grouped_gemm")


class _RouteArgs(Structure):
    _fields_ = [("logits", c_void_p), ("correction", c_void_p), ("ids", c_void_p), ("weights", c_void_p),
                ("n_tokens", c_int), ("n_all", c_int), ("n_groups", c_int), ("keep", c_int), ("top", c_int),
                ("sigmoid", c_int)]


def moe_route(logits: torch.Tensor, correction: Optional[torch.Tensor], ids: torch.Tensor, weights: torch.Tensor, *,
              n_groups: int, keep: int, sigmoid: bool = False) -> None:
    """Grouped top-k routing of fp32 ``logits`` [tokens, outputs] (see ``csrc/moe.cu``): ``ids`` and ``weights``
    [tokens, top] receive the chosen outputs, best first, and their scores: the softmax over the outputs, or with
    ``sigmoid`` the logistic function of each logit for itself."""
    _require(logits, "logits", torch.float32, 2)
    _require(ids, "ids", torch.int32, 2)
    _require(weights, "weights", torch.float32, 2)
    n, n_all = logits.shape
    if ids.shape[0] != n or weights.shape != ids.shape:
        raise KernelError("routing outputs do not fit the tokens")
    if correction is not None:
        _require(correction, "correction", torch.float32, 1)
        if correction.numel() != n_all:
            raise KernelError("the correction has one entry per router output")
    args = _RouteArgs(_ptr(logits), _ptr(correction), _ptr(ids), _ptr(weights), n, n_all, n_groups, keep, ids.shape[1],
                      1 if sigmoid else 0)
    lib = load_library("moe")
    _check(lib.odi_moe_route(byref(args), _stream()), "moe_route")


class _GroupingArgs(Structure):
    _fields_ = [("ids", c_void_p), ("counts", c_void_p), ("rank", c_void_p), ("offsets", c_void_p), ("pos", c_void_p),
                ("perm", c_void_p), ("tile_group", c_void_p), ("tile_row0", c_void_p), ("tile_rows", c_void_p),
                ("n_tiles", c_void_p), ("n_pairs", c_int), ("n_experts", c_int), ("tm", c_int), ("max_tiles", c_int)]


class RoutingTable:
    """The (token, choice) pairs of a step sorted by expert, made on the device by :func:`moe_group`: ``perm`` the
    sorted order, ``pos`` each pair's place in it, and the table of row tiles the grouped products walk."""

    def __init__(self, n_tokens: int, top: int, n_experts: int, device, few_rows_ok: bool = False) -> None:
        self.n_pairs, self.top, self.n_experts = n_tokens * top, top, n_experts
        self.tm = grouped_rows_tile(self.n_pairs / max(n_experts, 1), few_rows_ok)
        self.max_tiles = -(-self.n_pairs // self.tm) + n_experts
        ints = torch.empty(3 * self.n_pairs + n_experts + 1 + 3 * self.max_tiles + 1, dtype=torch.int32, device=device)
        cuts = [self.n_pairs, self.n_pairs, self.n_pairs, n_experts + 1, self.max_tiles, self.max_tiles, self.max_tiles, 1]
        (self.rank, self.pos, self.perm, self.offsets, self.tile_group, self.tile_row0, self.tile_rows,
         self.n_tiles) = torch.split(ints, cuts)


def moe_group(ids: torch.Tensor, counts: torch.Tensor, table: RoutingTable) -> None:
    """Fill ``table`` from the chosen outputs ``ids`` [tokens, top]; outputs >= ``table.n_experts`` (identity
    outputs) and -1 take no place.  ``counts`` [experts] int32 must be zero and is zero again afterwards."""
    _require(ids, "ids", torch.int32, 2)
    _require(counts, "counts", torch.int32, 1)
    if ids.numel() != table.n_pairs or counts.numel() != table.n_experts:
        raise KernelError("the routing table was made for other sizes")
    args = _GroupingArgs(_ptr(ids), _ptr(counts), _ptr(table.rank), _ptr(table.offsets), _ptr(table.pos),
                         _ptr(table.perm), _ptr(table.tile_group), _ptr(table.tile_row0), _ptr(table.tile_rows),
                         _ptr(table.n_tiles), table.n_pairs, table.n_experts, table.tm, table.max_tiles)
    lib = load_library("moe")
    _check(lib.odi_moe_group(byref(args), _stream()), "moe_group", 1 if table.n_pairs <= 2048 and table.n_experts <= 4096 else 3)


def moe_gather(x: torch.Tensor, table: RoutingTable, out: torch.Tensor, weights: Optional[torch.Tensor] = None) -> None:
    """out[i] = x[perm[i] // top] for every taken place i of ``table``'s sorted order (other rows are left alone);
    with ``weights`` (fp32 [tokens, top]) the row is multiplied by the weight of its (token, choice) pair."""
    _require(x, "x", ndim=2)
    _require(out, "out", x.dtype, 2)
    if out.shape != (table.n_pairs, x.shape[1]):
        raise KernelError("moe_gather sizes disagree")
    if weights is not None:
        _require(weights, "weights", torch.float32, 2)
        if weights.numel() != table.n_pairs:
            raise KernelError("moe_gather: one weight per (token, choice) pair")
    lib = load_library("moe")
    _check(lib.odi_moe_gather(_ptr(x), _ptr(table.perm), _ptr(table.offsets), _ptr(out), c_int(table.n_pairs),
                              c_int(x.shape[1]), c_int(table.top), c_int(table.n_experts), _ptr(weights),
                              c_int(dtype_code(x.dtype)), _stream()), "moe_gather")


class _CombineArgs(Structure):
    _fields_ = [("residual", c_void_p), ("expert_out", c_void_p), ("input", c_void_p), ("ids", c_void_p),
                ("weights", c_void_p), ("pos", c_void_p), ("n_tokens", c_int), ("H", c_int), ("top", c_int),
                ("n_experts", c_int), ("out_is_t", c_int), ("assign", c_int)]


def moe_combine(residual: torch.Tensor, expert_out: torch.Tensor, x: torch.Tensor, ids: torch.Tensor,
                weights: Optional[torch.Tensor], table: RoutingTable, assign: bool = False) -> None:
    """residual[t] += sum_k weights[t, k] * (row pos[t, k] of ``expert_out``, or ``x[t]`` for an identity output);
    ``weights`` None: every chosen row counts once.
    ``expert_out`` is fp32, or in the dtype of ``x``.  ``assign``: the sums replace the rows of ``residual``."""
    _require(residual, "residual", torch.float32, 2)
    _require(expert_out, "expert_out", ndim=2)
    _require(x, "x", ndim=2)
    if expert_out.dtype not in (torch.float32, x.dtype):
        raise KernelError("expert_out is float32 or has the dtype of x")
    n, H = residual.shape
    if x.shape != (n, H) or expert_out.shape != (table.n_pairs, H) or ids.numel() != table.n_pairs:
        raise KernelError("moe_combine sizes disagree")
    args = _CombineArgs(_ptr(residual), _ptr(expert_out), _ptr(x), _ptr(ids), _ptr(weights), _ptr(table.pos), n, H,
                        table.top, table.n_experts, 0 if expert_out.dtype == torch.float32 else 1, 1 if assign else 0)
    lib = load_library("moe")
    _check(lib.odi_moe_combine(byref(args), c_int(dtype_code(x.dtype)), _stream()), "moe_combine")


def moe_table_route(table: torch.Tensor, token_ids: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, *,
                    n_experts: int, weight: float) -> None:
    """Routing without a router: ``ids[t]`` = row ``token_ids[t]`` of the int32 ``table`` [vocab, top] (entries
    outside the experts become -1), ``weights`` all ``weight``."""
    _require(table, "table", torch.int32, 2)
    _require(token_ids, "token_ids", torch.int32, 1)
    _require(ids, "ids", torch.int32, 2)
    _require(weights, "weights", torch.float32, 2)
    n, top = ids.shape
    if token_ids.numel() != n or table.shape[1] != top or weights.shape != ids.shape:
        raise KernelError("table routing sizes disagree")
    lib = load_library("moe")
    _check(lib.odi_moe_table_route(_ptr(table), _ptr(token_ids), _ptr(ids), _ptr(weights), c_int(n), c_int(top),
                                   c_int(table.shape[0]), c_int(n_experts), c_float(weight), _stream()), "moe_table_route")


# ------------------------------------------------------------------------------ rotated unit heads, activations, norm-and-add


class _RotUnitArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
                ("cos_t", c_void_p), ("sin_t", c_void_p), ("tok_seq", c_void_p), ("tok_pos", c_void_p),
                ("page_start", c_void_p), ("page_ids", c_void_p), ("n_tokens", c_int), ("nq", c_int), ("nkv", c_int),
                ("d", c_int), ("dv", c_int), ("rot_dim", c_int), ("page_size", c_int), ("ring_pages", c_int),
                ("write_kv", c_int), ("unit", c_int), ("d_store", c_int), ("eps", c_float), ("v_from_k", c_int),
                ("q_w", c_void_p), ("k_w", c_void_p)]


def rot_unit_prep(qkv, q_out, k_pool, v_pool, cos_t, sin_t, tok_seq, tok_pos, page_start, page_ids, *, nq: int,
                  nkv: int, d: int, dv: int, rot_dim: int, page_size: int, ring_pages: int, write_kv: bool,
                  unit_eps: Optional[float], d_store: Optional[int] = None, v_from_k: bool = False,
                  q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None) -> None:
    """Head preparation of an attention that rotates first and norms afterwards: q and k heads (``d`` lanes) of
    ``qkv`` [tokens, nq d + nkv d + nkv dv] are rotated over their first ``rot_dim`` lanes (lane 2i with 2i + 1;
    ``cos_t`` None: not at all) and, with ``unit_eps`` not None, divided by sqrt(mean of squares + eps); q goes to
    ``q_out``, k and the v heads (``dv`` lanes, as they are) to the token's row of their cache pages.  Stored q
    and k heads have ``d_store`` >= ``d`` lanes (default ``d``), the ones beyond ``d`` zero.  ``v_from_k``: ``qkv``
    holds no v lanes ([tokens, nq d + nkv d]); the value of a head is its key as projected, before the rotation.
    ``q_weight`` / ``k_weight`` (fp32 [d], with ``unit_eps``): after the division every query resp. key head is
    multiplied by it lane by lane (an RMS norm per head with a weight that the heads share)."""
    d_store = d if d_store is None else d_store
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _require(w, name, torch.float32, 1)
            if w.numel() != d or unit_eps is None:
                raise KernelError(f"{name} has one entry per lane of a head and goes with unit_eps")
    if v_from_k and dv != d:
        raise KernelError("values that are the keys have the keys' width")
    _require(qkv, "qkv", ndim=2)
    _require(q_out, "q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    if qkv.shape[1] != (nq + nkv) * d + (0 if v_from_k else nkv * dv) or q_out.shape != (n, nq * d_store):
        raise KernelError(f"rot_unit_prep sizes disagree: qkv {tuple(qkv.shape)}, q_out {tuple(q_out.shape)}, "
                          f"nq={nq}, nkv={nkv}, d={d}, dv={dv}")
    if write_kv:
        _require(k_pool, "k_pool", qkv.dtype)
        _require(v_pool, "v_pool", qkv.dtype)
        if k_pool.shape[-1] != d_store or v_pool.shape[-1] != dv:
            raise KernelError("the cache pools do not have the heads' widths")
    if cos_t is not None:
        _require(cos_t, "cos_t", torch.float32, 2)
        _require(sin_t, "sin_t", torch.float32, 2)
        if cos_t.shape != (n, rot_dim // 2) or sin_t.shape != cos_t.shape:
            raise KernelError("rope tables must be [tokens, rot_dim / 2]")
    args = _RotUnitArgs(_ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(cos_t), _ptr(sin_t), _ptr(tok_seq),
                        _ptr(tok_pos), _ptr(page_start), _ptr(page_ids), n, nq, nkv, d, dv, rot_dim, page_size, ring_pages,
                        1 if write_kv else 0, 0 if unit_eps is None else 1, d_store, 0.0 if unit_eps is None else unit_eps,
                        1 if v_from_k else 0, _ptr(q_weight), _ptr(k_weight))
    lib = load_library("capped")
    _check(lib.odi_rot_unit_prep(byref(args), c_int(dtype_code(qkv.dtype)), _stream()), "rot_unit_prep")


class _CappedAttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("out", c_void_p), ("cu_q", c_void_p),
                ("past", c_void_p), ("page_start", c_void_p), ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int),
                ("nkv", c_int), ("ring_pages", c_int), ("window", c_int), ("scale", c_float), ("softcap", c_float),
                ("sink", c_int), ("keep", c_int)]


def attention_capped_supported(dtype: torch.dtype, d: int, dv: int) -> bool:
    """Whether :func:`attention_capped` takes these heads: bfloat16, key and value widths in steps of 16 up to 256."""
    return dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0 and 16 <= d <= 256 and 16 <= dv <= 256


def attention_capped(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int, nq: int,
                     nkv: int, d: int, dv: int, page_size: int, ring_pages: int, window: int, scale: float,
                     softcap: float = 0.0, sink: bool = False, keep: int = 0) -> None:
    """bf16 causal GQA on the tensor cores with squashed scores (``softcap`` c > 0: c tanh(score / c)), a window
    (0: none; the cache may be a ring of pages) and value rows of ``dv`` lanes, for any mixture of sequences.
    ``sink``: one more term of score 0 and no value in the softmax.  ``keep`` > 0 with a window: the first ``keep``
    positions of a sequence stay visible beyond the window."""
    if not attention_capped_supported(q.dtype, d, dv) or page_size != 64:
        raise KernelError(f"attention_capped takes bfloat16 heads in steps of 16 up to 256 and pages of 64 (d={d}, dv={dv})")
    _require(q, "q", torch.bfloat16)
    _require(out, "out", torch.bfloat16)
    _require(k_pool, "k_pool", torch.bfloat16)
    _require(v_pool, "v_pool", torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != n_tokens * nq * dv or k_pool.shape[-1] != d or v_pool.shape[-1] != dv:
        raise KernelError("attention_capped sizes disagree")
    args = _CappedAttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(cu_q), _ptr(past), _ptr(page_start),
                           _ptr(page_ids), n_seqs, nq, nkv, ring_pages, window, scale, softcap, 1 if sink else 0, keep)
    lib = load_library("attention_capped_mma", {"ODI_HEAD_DIM": d, "ODI_VALUE_DIM": dv})
    _check(lib.odi_attention_capped(byref(args), c_int(max_q_len), _stream()), "attention_capped")


def attention_capped_decode(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, nq: int, nkv: int,
                            d: int, dv: int, page_size: int, ring_pages: int, window: int, scale: float,
                            softcap: float = 0.0, splits: int = 1, partial: Optional[torch.Tensor] = None,
                            sink: bool = False, keep: int = 0) -> None:
    """:func:`attention_capped` for steps in which every sequence brings one token: each sequence's visible keys
    are cut into ``splits`` ranges that blocks of their own take; ``partial`` (fp32, tokens * nq * splits * (dv + 2))
    holds their results for the combine kernel."""
    if not attention_capped_supported(q.dtype, d, dv) or page_size != 64:
        raise KernelError(f"attention_capped takes bfloat16 heads in steps of 16 up to 256 and pages of 64 (d={d}, dv={dv})")
    _require(q, "q", torch.bfloat16)
    _require(out, "out", torch.bfloat16)
    _require(k_pool, "k_pool", torch.bfloat16)
    _require(v_pool, "v_pool", torch.bfloat16)
    if q.numel() != n_seqs * nq * d or out.numel() != n_seqs * nq * dv or k_pool.shape[-1] != d or v_pool.shape[-1] != dv:
        raise KernelError("attention_capped_decode sizes disagree (one token per sequence)")
    if splits > 1:
        need = n_seqs * nq * splits * (dv + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    args = _CappedAttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(cu_q), _ptr(past), _ptr(page_start),
                           _ptr(page_ids), n_seqs, nq, nkv, ring_pages, window, scale, softcap, 1 if sink else 0, keep)
    lib = load_library("attention_capped_mma", {"ODI_HEAD_DIM": d, "ODI_VALUE_DIM": dv})
    _check(lib.odi_attention_capped_decode(byref(args), _ptr(partial), c_int(splits), _stream()), "attention_capped_decode",
           2 if splits > 1 else 1)


ACTIVATIONS = {"gelu_erf": 0, "gelu_tanh": 1, "relu2": 2}      # relu2: the square of max(x, 0)


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) elementwise (fp32 arithmetic, one rounding); ``kind`` one of ``ACTIVATIONS``."""
    _require(x, "x")
    _require(out, "out", x.dtype)
    if kind not in ACTIVATIONS or out.numel() != x.numel():
        raise KernelError(f"activation {kind!r} on {tuple(x.shape)} -> {tuple(out.shape)}")
    lib = load_library("capped")
    _check(lib.odi_activation(_ptr(x), _ptr(out), c_long(x.numel()), c_int(ACTIVATIONS[kind]), c_int(dtype_code(x.dtype)),
                              _stream()), "activation")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (fp32)."""
    _require(x, "x", torch.float32)
    lib = load_library("capped")
    _check(lib.odi_softcap(_ptr(x), c_long(x.numel()), c_float(cap), _stream()), "softcap")


def concat_cast(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] ; b[t]] for fp32 ``a`` and ``b`` [tokens, H], in the dtype of ``out`` [tokens, 2 H]."""
    _require(a, "a", torch.float32, 2)
    _require(b, "b", torch.float32, 2)
    _require(out, "out", ndim=2)
    n, H = a.shape
    if b.shape != (n, H) or out.shape != (n, 2 * H):
        raise KernelError("concat_cast sizes disagree")
    lib = load_library("capped")
    _check(lib.odi_concat_cast(_ptr(a), _ptr(b), _ptr(out), c_long(n), c_int(H), c_int(dtype_code(out.dtype)), _stream()),
           "concat_cast")


def rmsnorm_add(hidden: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """hidden[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * weight, all fp32: the norm of a sublayer's output and the
    residual add in one pass."""
    _require(hidden, "hidden", torch.float32, 2)
    _require(y, "y", torch.float32, 2)
    _require(weight, "weight", torch.float32, 1)
    n, H = hidden.shape
    if y.shape != (n, H) or weight.numel() != H:
        raise KernelError("rmsnorm_add sizes disagree")
    lib = load_library("capped")
    _check(lib.odi_rmsnorm_add(_ptr(hidden), _ptr(y), _ptr(weight), c_int(n), c_int(H), c_float(eps), _stream()), "rmsnorm_add")


def rmsnorm_add_norm(hidden: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, next_weight: torch.Tensor,
                     next_eps: float, out: torch.Tensor) -> bool:
    """:func:`rmsnorm_add` followed by the norm of the sum for the next sublayer, in one pass over the row:
    hidden[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * weight, then out[t] = cast(hidden[t] * rsqrt(mean(hidden[t]^2)
    + next_eps) * next_weight) (scaled in fp32, one rounding).  Returns False, having done nothing, for widths the
    fused kernel does not take (no multiple of 4, or above 8,192)."""
    _require(hidden, "hidden", torch.float32, 2)
    _require(y, "y", torch.float32, 2)
    _require(weight, "weight", torch.float32, 1)
    _require(next_weight, "next_weight", torch.float32, 1)
    _require(out, "out", ndim=2)
    n, H = hidden.shape
    if y.shape != (n, H) or weight.numel() != H or next_weight.numel() != H or out.shape != (n, H):
        raise KernelError("rmsnorm_add_norm sizes disagree")
    lib = load_library("capped")
    code = lib.odi_rmsnorm_add_norm(_ptr(hidden), _ptr(y), _ptr(weight), c_float(eps), _ptr(next_weight), c_float(next_eps),
                                    _ptr(out), c_int(n), c_int(H), c_int(dtype_code(out.dtype)), _stream())
    if code == ODI_ERR_UNSUPPORTED:
        return False
    _check(code, "rmsnorm_add_norm")
    return True


def gated_row_add(acc: torch.Tensor, y: torch.Tensor, x: torch.Tensor, gate: torch.Tensor) -> None:
    """acc[t] += sigmoid(x[t] . gate) * y[t]: ``acc`` fp32 [tokens, H], ``y`` fp32 or in the dtype of ``x``,
    ``x`` [tokens, K] and ``gate`` [K] in the compute dtype; the dot product and the sigmoid in fp32."""
    _require(acc, "acc", torch.float32, 2)
    _require(y, "y", ndim=2)
    _require(x, "x", ndim=2)
    _require(gate, "gate", x.dtype)
    n, H = acc.shape
    if y.shape != (n, H) or x.shape[0] != n or gate.numel() != x.shape[1] or y.dtype not in (torch.float32, x.dtype):
        raise KernelError("gated_row_add sizes disagree")
    lib = load_library("capped")
    _check(lib.odi_gated_row_add(_ptr(acc), _ptr(y), _ptr(x), _ptr(gate), c_int(n), c_int(H), c_int(x.shape[1]),
                                 c_int(0 if y.dtype == torch.float32 else 1), c_int(dtype_code(x.dtype)), _stream()),
           "gated_row_add")


# ------------------------------------------------------------------------------ the gated delta rule


class _DeltaArgs(Structure):
    _fields_ = [("proj", c_void_p), ("taps", c_void_p), ("conv_state", c_void_p), ("conv_out", c_void_p),
                ("decay_in", c_void_p), ("a_log", c_void_p), ("dt_bias", c_void_p), ("qkg", c_void_p), ("beta", c_void_p),
                ("state", c_void_p), ("o", c_void_p), ("norm_w", c_void_p), ("out", c_void_p), ("cu_q", c_void_p),
                ("tok_seq", c_void_p), ("slots", c_void_p),
                ("n_tokens", c_int), ("n_seqs", c_int), ("ld_proj", c_int), ("ld_decay", c_int), ("heads", c_int),
                ("kv_heads", c_int), ("dv", c_int), ("taps_n", c_int), ("C", c_int), ("eps", c_float),
                ("unit_eps", c_float)]


DELTA_MAX_DIM = 480     # the recurrence stages 8 tokens of q, k and decay in 48 KB of shared memory


def delta_rule(proj: torch.Tensor, decay_in: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor,
               dt_bias: torch.Tensor, norm_w: torch.Tensor, conv_state: Optional[torch.Tensor], state: torch.Tensor,
               out: torch.Tensor, cu_q, tok_seq, slots, *, n_seqs: int, heads: int, kv_heads: int, d: int, dv: int,
               eps: float, unit_eps: float) -> None:
    """The channel-wise gated delta rule between its input products and its output product (``csrc/delta.cu``).

    ``proj`` [tokens, C + heads]: q, k and v channels before their convolutions (C = 2 kv_heads d + heads dv), then
    one beta logit per head.  ``decay_in`` fp32 [tokens, heads d + heads dv]: the decay's inner term per head and
    key channel, then the output gate's logits.  ``taps`` fp32 [C, K].  ``conv_state`` fp32 [slots, K - 1, C] and
    ``state`` fp32 [slots, heads, d, dv] are read and advanced for the sequences ``slots``.  ``out`` [tokens,
    heads dv] receives the gated, normed read-outs in the dtype of ``proj``."""
    _require(proj, "proj", ndim=2)
    _require(decay_in, "decay_in", torch.float32, 2)
    _require(taps, "taps", torch.float32, 2)
    _require(state, "state", torch.float32)
    _require(out, "out", proj.dtype, 2)
    n = proj.shape[0]
    C, K = taps.shape
    if not 1 <= d <= DELTA_MAX_DIM:
        raise KernelError(f"the delta rule takes key sizes up to {DELTA_MAX_DIM}, not {d}")
    if (C != 2 * kv_heads * d + heads * dv or proj.shape[1] != C + heads or decay_in.shape != (n, heads * (d + dv))
            or out.shape != (n, heads * dv) or a_log.numel() != heads or dt_bias.numel() != heads * d
            or norm_w.numel() != dv or tuple(state.shape[1:]) != (heads, d, dv)):
        raise KernelError("delta_rule sizes disagree")
    if K > 1:
        _require(conv_state, "conv_state", torch.float32)
        if tuple(conv_state.shape[1:]) != (K - 1, C):
            raise KernelError("the convolution state does not fit the taps")
    dev = proj.device
    conv_out = torch.empty((n, C), dtype=proj.dtype, device=dev)
    qkg = torch.empty((n, heads, 3, d), dtype=torch.float32, device=dev)
    beta = torch.empty((n, heads), dtype=torch.float32, device=dev)
    o = torch.empty((n, heads * dv), dtype=torch.float32, device=dev)
    args = _DeltaArgs(_ptr(proj), _ptr(taps), _ptr(conv_state), _ptr(conv_out), _ptr(decay_in), _ptr(a_log),
                      _ptr(dt_bias), _ptr(qkg), _ptr(beta), _ptr(state), _ptr(o), _ptr(norm_w), _ptr(out), _ptr(cu_q),
                      _ptr(tok_seq), _ptr(slots), n, n_seqs, proj.shape[1], decay_in.shape[1], heads, kv_heads, dv, K, C,
                      eps, unit_eps)
    lib = load_library("delta", {"ODI_DELTA_DIM": d})
    _check(lib.odi_delta_rule(byref(args), c_int(dtype_code(proj.dtype)), _stream()), "delta_rule", 6 if K > 1 else 5)


# ------------------------------------------------------------------------------ sampling

_sample_state = {}


def _sample_buffers(device, rows: int, chunks: int):
    """Per-chunk partial results (16 bytes each) and one ticket per row (kept zero between launches)."""
    state = _sample_state.setdefault(device, {})
    if state.get("rows", 0) < rows:
        _outgrown.append(state.get("tickets"))
        state["tickets"] = torch.zeros(max(rows, 256), dtype=torch.int32, device=device)
        state["rows"] = state["tickets"].numel()
    if state.get("entries", 0) < rows * chunks:
        _outgrown.append(state.get("partials"))
        state["partials"] = torch.empty(max(rows * chunks, 4096) * 4, dtype=torch.float32, device=device)
        state["entries"] = state["partials"].numel() // 4
    return state["partials"], state["tickets"]


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, seed: int = 0,
           streams: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, *,
           advance_pos: Optional[torch.Tensor] = None, advance_past: Optional[torch.Tensor] = None,
           active: Optional[torch.Tensor] = None) -> None:
    """out[i] = argmax(logits[i]) if temperature == 0 else a draw from softmax(logits[i] / temperature).

    With ``active`` (int32 0/1 per row) the kernel also adds ``active[i]`` to ``advance_pos[i]``,
    ``advance_past[i]`` and ``steps[i]``: the bookkeeping of a decode loop that stays on the device."""
    _require(logits, "logits", torch.float32, 2)
    _require(out, "out", torch.int32, 1)
    n, V = logits.shape
    if out.numel() < n:
        raise KernelError("out is shorter than the number of rows")
    if temperature > 0:
        _require(streams, "streams", torch.int32, 1)
        _require(steps, "steps", torch.int32, 1)
    if active is not None:
        for name, t in (("active", active), ("advance_pos", advance_pos), ("advance_past", advance_past)):
            _require(t, name, torch.int32, 1)
    lib = load_library("sampling")
    partials, tickets = _sample_buffers(logits.device, n, int(lib.odi_sample_chunks(c_int(V))))
    _check(lib.odi_sample(_ptr(logits), _ptr(out), c_int(n), c_int(V), c_int(V), c_float(temperature),
                          c_ulonglong(seed & ((1 << 64) - 1)), _ptr(streams), _ptr(steps), _ptr(advance_pos),
                          _ptr(advance_past), _ptr(active), _ptr(partials), _ptr(tickets), _stream()), "sample")



# ------------------------------------------------------------------------------ parallel block, polynomial activation


class _CanonArgs(Structure):
    _fields_ = [("x", c_void_p), ("g", c_void_p), ("taps_w", c_void_p), ("state", c_void_p), ("tok_seq", c_void_p),
                ("cu_q", c_void_p), ("slots", c_void_p), ("h_out", c_void_p), ("hc_out", c_void_p), ("n_tokens", c_int),
                ("n_seqs", c_int), ("W", c_int), ("taps", c_int), ("eps", c_float)]


CANON_MAX_TAPS = 64       # the plain kernel keeps the taps' factors in shared memory; up to 8 taps take the 16-byte forms


def _canon_args(x, g, taps_w, state, tok_seq, cu_q, slots, h_out, hc_out, eps) -> _CanonArgs:
    _require(x, "x", torch.float32, 2)
    _require(g, "g", torch.float32)
    _require(taps_w, "taps_w", torch.float32, 2)
    n, W = x.shape
    taps = taps_w.shape[1]
    if g.numel() != 1 or taps_w.shape[0] != W or not 1 <= taps <= CANON_MAX_TAPS:
        raise KernelError(f"canon: one norm weight, taps [width, 1..{CANON_MAX_TAPS}] (got {tuple(g.shape)}, {tuple(taps_w.shape)})")
    if taps > 1:
        _require(state, "state", torch.float32, 3)
        if state.shape[1:] != (taps - 1, W):
            raise KernelError(f"canon: the state is [slots, taps - 1, width], not {tuple(state.shape)}")
    for name, t in (("tok_seq", tok_seq), ("cu_q", cu_q), ("slots", slots)):
        _require(t, name, torch.int32, 1)
    return _CanonArgs(_ptr(x), _ptr(g), _ptr(taps_w), _ptr(state if taps > 1 else None), _ptr(tok_seq), _ptr(cu_q),
                      _ptr(slots), _ptr(h_out), _ptr(hc_out), n, slots.numel(), W, taps, eps)


def canon_norm(x, g, eps: float, taps_w, state, tok_seq, cu_q, slots, h_out, hc_out) -> None:
    """h = x / sqrt(mean(x^2) + eps) * g (``g`` one number) per token into ``h_out``, and h + conv(h) into ``hc_out``
    (both in the compute dtype), conv(h)_t = sum_j taps_w[:, j] h_(t - taps + 1 + j) over the sequence's earlier
    tokens: those of this step, and before them ``state[slot]`` [taps - 1, width] (fp32: h of the sequence's last
    positions, zero before its start).  The state of a sequence that brings one token is moved on in the same
    launch; :func:`canon_state` moves on the others afterwards."""
    args = _canon_args(x, g, taps_w, state, tok_seq, cu_q, slots, h_out, hc_out, eps)
    _require(h_out, "h_out", ndim=2)
    _require(hc_out, "hc_out", h_out.dtype, 2)
    if h_out.shape != x.shape or hc_out.shape != x.shape or tok_seq.numel() != x.shape[0]:
        raise KernelError("canon_norm: outputs and tok_seq follow the tokens of x")
    lib = load_library("parallel")
    _check(lib.odi_canon_norm(byref(args), c_int(dtype_code(h_out.dtype)), _stream()), "canon_norm")


def canon_state(x, g, eps: float, taps_w, state, tok_seq, cu_q, slots) -> None:
    """After :func:`canon_norm` and before ``x`` changes: ``state[slot]`` becomes h of the last taps - 1 positions
    of every sequence that brought more than one token (rows of the old state move up where it brought fewer than
    taps - 1); a step of single tokens needs no call."""
    if taps_w.shape[1] <= 1:
        return
    args = _canon_args(x, g, taps_w, state, tok_seq, cu_q, slots, None, None, eps)
    lib = load_library("parallel")
    _check(lib.odi_canon_state(byref(args), _stream()), "canon_state")


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e per row, N(v) = v / sqrt(mean(v^2) + eps), (a, b, c, e) = ``coef``
    (fp32); powers, means and the sum in fp32, one rounding."""
    _require(z, "z", ndim=2)
    _require(out, "out", z.dtype, 2)
    _require(coef, "coef", torch.float32, 1)
    if out.shape != z.shape or coef.numel() != 4:
        raise KernelError(f"poly_norm sizes disagree: {tuple(z.shape)} -> {tuple(out.shape)}, coef {tuple(coef.shape)}")
    lib = load_library("parallel")
    _check(lib.odi_poly_norm(_ptr(z), _ptr(coef), _ptr(out), c_int(z.shape[0]), c_int(z.shape[1]), c_float(eps),
                             c_int(dtype_code(z.dtype)), _stream()), "poly_norm")


def scaled_add(x: torch.Tensor, y: torch.Tensor, m: float) -> None:
    """x += m * y (fp32, in place)."""
    _require(x, "x", torch.float32)
    _require(y, "y", torch.float32)
    if x.shape != y.shape:
        raise KernelError(f"scaled_add sizes disagree: {tuple(x.shape)} and {tuple(y.shape)}")
    lib = load_library("parallel")
    _check(lib.odi_scaled_add(_ptr(x), _ptr(y), c_long(x.numel()), c_float(m), _stream()), "scaled_add")


# ------------------------------------------------------------------------------ block with two norms and scaled outputs


def dual_norm(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float, out1: torch.Tensor, out2: torch.Tensor) -> None:
    """out1 = cast(x r w1), out2 = cast(x r w2) with r = 1 / sqrt(mean(x^2) + eps) per row: two RMS norms of the same
    fp32 rows in one pass (``w1``, ``w2``: what multiplies each lane, fp32)."""
    _require(x, "x", torch.float32, 2)
    _require(w1, "w1", torch.float32, 1)
    _require(w2, "w2", torch.float32, 1)
    _require(out1, "out1", ndim=2)
    _require(out2, "out2", out1.dtype, 2)
    n, H = x.shape
    if w1.numel() != H or w2.numel() != H or out1.shape != (n, H) or out2.shape != (n, H):
        raise KernelError("dual_norm sizes disagree")
    lib = load_library("scaled_block")
    _check(lib.odi_dual_norm(_ptr(x), _ptr(w1), _ptr(w2), _ptr(out1), _ptr(out2), c_int(n), c_int(H), c_float(eps),
                             c_int(dtype_code(out1.dtype)), _stream()), "dual_norm")


def scaled_add2(x: torch.Tensor, a: torch.Tensor, s1: torch.Tensor, b: Optional[torch.Tensor] = None,
                s2: Optional[torch.Tensor] = None, copy: Optional[torch.Tensor] = None) -> None:
    """x += a * s1 (+ b * s2) on fp32 rows, ``s1`` and ``s2`` one number per lane; ``copy`` (optional, any compute
    dtype) receives the new rows once more."""
    _require(x, "x", torch.float32, 2)
    _require(a, "a", torch.float32, 2)
    _require(s1, "s1", torch.float32, 1)
    n, H = x.shape
    if a.shape != (n, H) or s1.numel() != H:
        raise KernelError("scaled_add2 sizes disagree")
    if b is not None:
        _require(b, "b", torch.float32, 2)
        _require(s2, "s2", torch.float32, 1)
        if b.shape != (n, H) or s2.numel() != H:
            raise KernelError("scaled_add2 sizes disagree")
    if copy is not None:
        _require(copy, "copy", ndim=2)
        if copy.shape != (n, H):
            raise KernelError("scaled_add2: the copy has the shape of x")
    lib = load_library("scaled_block")
    _check(lib.odi_scaled_add2(_ptr(x), _ptr(a), _ptr(s1), _ptr(b), _ptr(s2), _ptr(copy), c_long(n), c_int(H),
                               c_int(0 if copy is None else dtype_code(copy.dtype)), _stream()), "scaled_add2")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = cast(x) for fp32 ``x``, into the compute dtype of ``out`` (same shape)."""
    _require(x, "x", torch.float32)
    _require(out, "out")
    if out.shape != x.shape:
        raise KernelError("cast_rows sizes disagree")
    lib = load_library("scaled_block")
    _check(lib.odi_cast_rows(_ptr(x), _ptr(out), c_long(x.numel()), c_int(dtype_code(out.dtype)), _stream()), "cast_rows")


def weighted_sum(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, ca: float, cb: float) -> None:
    """out = ca * a + cb * b on fp32 tensors of one shape (``out`` may be ``a`` or ``b``)."""
    for name, t in (("out", out), ("a", a), ("b", b)):
        _require(t, name, torch.float32)
    if a.shape != out.shape or b.shape != out.shape:
        raise KernelError("weighted_sum sizes disagree")
    lib = load_library("scaled_block")
    _check(lib.odi_weighted_sum(_ptr(out), _ptr(a), _ptr(b), c_long(out.numel()), c_float(ca), c_float(cb), _stream()),
           "weighted_sum")


def gated_lookup(z: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, col: int) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col + j] for ``z`` and ``out`` [tokens, dim] and ``table``
    [rows, >= col + dim], all in one compute dtype (fp32 arithmetic, one rounding)."""
    _require(z, "z", ndim=2)
    _require(table, "table", z.dtype, 2)
    _require(ids, "ids", torch.int32, 1)
    _require(out, "out", z.dtype, 2)
    n, dim = z.shape
    if out.shape != (n, dim) or ids.numel() != n or col < 0 or col + dim > table.shape[1]:
        raise KernelError("gated_lookup sizes disagree")
    lib = load_library("scaled_block")
    _check(lib.odi_gated_lookup(_ptr(z), _ptr(table), _ptr(ids), _ptr(out), c_long(n), c_int(dim), c_int(table.shape[1]),
                                c_int(col), c_int(dtype_code(z.dtype)), _stream()), "gated_lookup")


# ------------------------------------------------------------------------------ state-space mixer


class _SsdArgs(Structure):
    _fields_ = [("proj", c_void_p), ("conv_w", c_void_p), ("conv_b", c_void_p), ("dt_bias", c_void_p), ("a_log", c_void_p),
                ("d_skip", c_void_p), ("norm_w", c_void_p), ("conv_state", c_void_p), ("state", c_void_p), ("xbc", c_void_p),
                ("y", c_void_p), ("out", c_void_p), ("cu_q", c_void_p), ("tok_seq", c_void_p), ("slots", c_void_p),
                ("n_tokens", c_int), ("n_seqs", c_int), ("ld", c_int), ("heads", c_int), ("P", c_int), ("N", c_int),
                ("G", c_int), ("taps", c_int), ("norm_groups", c_int), ("eps", c_float)]


SSD_MAX_STATE, SSD_MAX_TAPS = 256, 16


def ssd_mix(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
            d_skip: torch.Tensor, norm_w: torch.Tensor, conv_state: Optional[torch.Tensor], state: torch.Tensor,
            out: torch.Tensor, cu_q, tok_seq, slots, *, n_seqs: int, heads: int, head_dim: int, state_dim: int,
            groups: int, norm_groups: int, eps: float) -> None:
    """The state-space mixer between its projections (``csrc/ssd.cu``): ``proj`` [tokens, 2 inner + 2 G N + heads]
    = [z | x | B | C | dt] in the compute dtype, ``out`` [tokens, inner] in the same; ``conv_state``
    [slots, taps - 1, inner + 2 G N] and ``state`` [slots, heads, N, P] are fp32 rows of the cache, advanced in place
    over all tokens that each sequence brings."""
    _require(proj, "proj", ndim=2)
    _require(out, "out", proj.dtype, 2)
    n = proj.shape[0]
    inner, C = heads * head_dim, heads * head_dim + 2 * groups * state_dim
    taps = conv_w.shape[1]
    for name, t, shape in (("conv_w", conv_w, (C, taps)), ("conv_b", conv_b, (C,)), ("dt_bias", dt_bias, (heads,)),
                           ("a_log", a_log, (heads,)), ("d_skip", d_skip, (heads,)), ("norm_w", norm_w, (inner,))):
        _require(t, name, torch.float32)
        if tuple(t.shape) != shape:
            raise KernelError(f"ssd_mix: {name} is {tuple(t.shape)}, expected {shape}")
    _require(state, "state", torch.float32)
    if proj.shape[1] != inner + C + heads or out.shape != (n, inner) or tuple(state.shape[1:]) != (heads, state_dim, head_dim):
        raise KernelError(f"ssd_mix sizes disagree: proj {tuple(proj.shape)}, out {tuple(out.shape)}, state {tuple(state.shape)}")
    if taps > 1:
        _require(conv_state, "conv_state", torch.float32)
        if tuple(conv_state.shape[1:]) != (taps - 1, C):
            raise KernelError("ssd_mix: the convolution state is [slots, taps - 1, channels]")
    xbc = torch.empty((n, C), dtype=torch.float32, device=proj.device)
    y = torch.empty((n, inner), dtype=torch.float32, device=proj.device)
    args = _SsdArgs(_ptr(proj), _ptr(conv_w), _ptr(conv_b), _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(norm_w),
                    _ptr(conv_state if taps > 1 else None), _ptr(state), _ptr(xbc), _ptr(y), _ptr(out), _ptr(cu_q),
                    _ptr(tok_seq), _ptr(slots), n, n_seqs, proj.shape[1], heads, head_dim, state_dim, groups, taps,
                    norm_groups, eps)
    lib = load_library("ssd")
    _check(lib.odi_ssd(byref(args), c_int(dtype_code(proj.dtype)), _stream()), "ssd_mix", 4 if taps > 1 else 3)
