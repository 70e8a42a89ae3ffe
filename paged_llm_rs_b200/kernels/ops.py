"""Python side of the CUDA kernels: argument checks, then the C entry point.

Every function takes torch tensors that live on the GPU, checks dtype, shape and
contiguity, and launches on torch's current stream.  There is no fallback: if
the kernel library cannot be built or loaded, or a tensor is not on a CUDA
device, a ``KernelError`` is raised.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import KernelError

_F32, _BF16 = 0, 1
_ERRORS = {
    -1: "dtype is neither float32 nor bfloat16",
    -2: "a size the kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "a size beyond the kernel's stated maximum",
}

_lib = None
LAUNCHES = 0  # kernels of this library launched so far (library matrix products are not counted)
c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def lib():
    global _lib
    if _lib is None:
        L = load_library()
        P = c_void_p
        sig = {
            "pllm_embed": [c_int, P, P, P, c_int, c_int, c_int, P, P],
            "pllm_rmsnorm": [c_int, P, P, P, P, P, P, c_int, c_int, c_float, P],
            "pllm_swiglu": [c_int, P, P, c_int, c_int, P],
            "pllm_qk_norm_rope_kv": [c_int, P, P, P, P, c_float, P, P, c_int, c_int, P, P, P, P,
                                     c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P],
            "pllm_attention_generic": [c_int, P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_float, P, P],
            "pllm_attention_generic_tile_tokens": [c_int, c_int],
            "pllm_attention_reduce": [c_int, P, P, P, P, c_int, P, c_int, c_int, c_int, P],
            "pllm_sample": [P, c_int, c_int, c_ll, P, P, P, P, P],
            "pllm_sample_scratch_floats": [c_int, c_int],
            "pllm_skinny_gemm_supports": [c_int, c_int, c_int],
            "pllm_skinny_gemm": [P, P, P, c_int, c_int, c_int, c_int, P],
            "pllm_skinny_gemm_glu_supports": [c_int, c_int, c_int],
            "pllm_skinny_gemm_glu": [P, P, P, c_int, c_int, c_int, P],
            "pllm_sm_count": [],
            "pllm_attention_mma_supports": [c_int, c_int, c_int, c_int],
            "pllm_attention_mma_tile_tokens": [c_int, c_int],
            "pllm_attention_mma": [P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_float, c_int, c_int, P, P],
            "pllm_attention_decode_tma_supports": [c_int, c_int, c_int, c_int, c_int, c_int],
            "pllm_attention_decode_tma": [P, P, P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, P, P],
        }
        sig["pllm_set_pdl"] = [c_int]
        sig["pllm_attention_decode_tma_fused"] = [P, P, P, c_float, P, P, c_int, P, P, P, P, P, c_int, P, P, P] + [c_int] * 6 + [c_float, P, P]
        sig["pllm_attention_prefill_tcgen05_tile_tokens"] = [c_int, c_int]
        sig["pllm_attention_prefill_tcgen05_supports"] = [c_int] * 6
        sig["pllm_attention_prefill_tcgen05"] = [P] * 10 + [c_int] * 7 + [c_float, c_int, P, P]
        sig["pllm_gemm_tcgen05_supports"] = [c_int, c_int, c_int, c_int]
        sig["pllm_gemm_tcgen05"] = [P, P, P, c_int, c_int, c_int, c_int, P, P]
        sig["pllm_pack_decode_step"] = [P, c_int, c_int, P, P, P, P, P] + [c_int] * 16 + [P, P]
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        # The kernels are launched with programmatic dependent launch: a kernel's CTAs
        # may take their places while the one before it drains (the long kernels let
        # them in after their main loops; every kernel waits for its predecessors
        # before it touches memory).  A decode step measured 11% faster with it;
        # PAGED_LLM_PDL=0 turns it off.
        L.pllm_set_pdl(0 if os.environ.get("PAGED_LLM_PDL", "1") == "0" else 1)
        _lib = L
    return _lib


def _check(code: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += launches
        return
    if code < 0:
        raise KernelError(f"{what}: refused, {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {t.dtype} is not handled: the kernels take float32 and bfloat16")


def _dev(*tensors) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("a tensor is not on a CUDA device: there is no CPU path")
        if not t.is_contiguous():
            raise KernelError("a tensor is not contiguous")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _i32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


def _f32(t: Optional[torch.Tensor], name: str):
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{name} must be float32, got {t.dtype}")


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]]; tokens int32 [T], table [V, H], out [T, H]."""
    _dev(tokens, table, out, status)
    _i32(tokens, "tokens")
    T, (V, H) = tokens.numel(), table.shape
    if out.shape != (T, H) or out.dtype != table.dtype:
        raise KernelError(f"embed: out is {tuple(out.shape)} {out.dtype}, expected {(T, H)} {table.dtype}")
    _check(lib().pllm_embed(_code(table), _ptr(tokens), _ptr(table), _ptr(out), T, H, V, _ptr(status), _stream()),
           "embed")
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, residual_out: Optional[torch.Tensor] = None,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rmsnorm(x[r] (+ delta[r])) * gain with r = rows[i] or i; when
    residual_out is given the sum is stored to residual_out[r] (may alias x)."""
    _dev(x, gain, out, delta, residual_out, rows)
    _f32(gain, "gain")
    _i32(rows, "rows")
    W = x.shape[-1]
    n = rows.numel() if rows is not None else x.numel() // W
    if gain.numel() != W:
        raise KernelError(f"rmsnorm: gain has {gain.numel()} entries for rows of width {W}")
    if out.numel() != n * W or out.dtype != x.dtype:
        raise KernelError("rmsnorm: out does not fit")
    for t in (delta, residual_out):
        if t is not None and (t.shape != x.shape or t.dtype != x.dtype):
            raise KernelError("rmsnorm: delta / residual_out must have x's shape and dtype")
    _check(lib().pllm_rmsnorm(_code(x), _ptr(x), _ptr(delta), _ptr(residual_out), _ptr(gain), _ptr(out),
                              _ptr(rows), n, W, float(eps), _stream()), "rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, I] = silu(gate_up[n, :I]) * gate_up[n, I:]."""
    _dev(gate_up, out)
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("swiglu: out must be [n, I] for an input [n, 2I] of the same dtype")
    _check(lib().pllm_swiglu(_code(gate_up), _ptr(gate_up), _ptr(out), n, two_i // 2, _stream()), "swiglu")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, q_gain, k_gain, eps: float, cos, sin,
                    rotary_dim: int, positions: torch.Tensor, slots: torch.Tensor, k_pool, v_pool,
                    num_heads: int, num_kv_heads: int, head_dim: int, status: torch.Tensor,
                    swizzled: bool = False) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation, q to q_out, k and v into the paged
    pools [pages, kv_heads, page_size, head_dim] at ``slots`` (a negative slot, or
    k_pool None, writes nothing).  ``swizzled``: the pools keep each row's 16-byte
    chunks at chunk ^ (offset in page & 7), the layout of ``pool_is_swizzled``."""
    _dev(qkv, q_out, q_gain, k_gain, cos, sin, positions, slots, k_pool, v_pool, status)
    _f32(q_gain, "q_gain"); _f32(k_gain, "k_gain"); _f32(cos, "cos"); _f32(sin, "sin")
    _i32(positions, "positions"); _i32(slots, "slots")
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (T, width):
        raise KernelError(f"qk_norm_rope_kv: qkv is {tuple(qkv.shape)}, expected {(T, width)}")
    if q_out.numel() != T * num_heads * head_dim or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_kv: q_out does not fit")
    if positions.numel() < T or slots.numel() < T:
        raise KernelError("qk_norm_rope_kv: positions / slots shorter than the tokens")
    max_pos, page_size, n_pages = 0, 1, 0
    if cos is not None:
        if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
            raise KernelError("qk_norm_rope_kv: cos/sin must be [max_positions, rotary_dim/2]")
        max_pos = cos.shape[0]
    if k_pool is not None:
        if k_pool.shape != v_pool.shape or k_pool.dtype != qkv.dtype or k_pool.dim() != 4 \
                or k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim:
            raise KernelError(f"qk_norm_rope_kv: pools must be [pages, {num_kv_heads}, page_size, {head_dim}] "
                              f"of {qkv.dtype}, got {tuple(k_pool.shape)} {k_pool.dtype}")
        n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    for g in (q_gain, k_gain):
        if g is not None and g.numel() != head_dim:
            raise KernelError("qk_norm_rope_kv: a head gain must have head_dim entries")
    _check(lib().pllm_qk_norm_rope_kv(_code(qkv), _ptr(qkv), _ptr(q_out), _ptr(q_gain), _ptr(k_gain), float(eps),
                                      _ptr(cos), _ptr(sin), rotary_dim, max_pos, _ptr(positions), _ptr(slots),
                                      _ptr(k_pool), _ptr(v_pool), T, num_heads, num_kv_heads, head_dim, page_size,
                                      n_pages, 1 if swizzled else 0, _ptr(status), _stream()), "qk_norm_rope_kv")
    return q_out


def attention_uses_tensor_cores(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether paged_attention runs the mma kernel for this shape (bfloat16, head
    sizes 64 and 128) or the generic one."""
    if dtype != torch.bfloat16:
        return False
    return bool(lib().pllm_attention_mma_supports(_BF16, num_heads, num_kv_heads, head_dim))


TMA_KINDS = int(os.environ.get("PAGED_LLM_TMA_KINDS", "3"))  # which items the bulk-copy attention kernel takes where it applies: 1 single tokens, 2 portions, 3 both


def pool_is_swizzled(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whether the cache pools of such layers keep each row's 16-byte chunks at
    chunk ^ (offset in page & 7).  True exactly where the tensor-core attention
    kernels run: they read that layout from shared memory without bank conflicts,
    and the decode kernel copies whole pages there as they lie."""
    return attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim)


def swizzle_pool_(pool: torch.Tensor) -> torch.Tensor:
    """Rearrange a plain pool [pages, kv_heads, page_size, head_dim] into the swizzled
    layout in place (its own inverse); for tests and tools."""
    pages, nkv, ps, hd = pool.shape
    epc = 16 // pool.element_size()
    ch = hd // epc
    if ch % 8:
        raise KernelError("swizzle_pool_: a row must hold a multiple of eight 16-byte chunks")
    v = pool.view(pages, nkv, ps, ch, epc)
    o = torch.arange(ps, device=pool.device)[:, None] & 7
    c = torch.arange(ch, device=pool.device)[None, :]
    idx = (c ^ o)[None, None, :, :, None].expand_as(v)
    pool.copy_(torch.gather(v.clone(), 3, idx).view_as(pool))
    return pool


# Prompt portions (work items of several tokens) in bfloat16 over swizzled pages: the tcgen05 kernel
# (csrc/attention_prefill_tcgen05.cu), 128 rows an item (PAGED_LLM_TCGEN05_ATTN=0: the mma.sync kernels).
TCGEN05_ATTN = os.environ.get("PAGED_LLM_TCGEN05_ATTN", "1") != "0"


def attention_prefill_uses_tcgen05(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: Optional[int],
                                   window: int) -> bool:
    if not TCGEN05_ATTN or page_size is None or not pool_is_swizzled(dtype, num_heads, num_kv_heads, head_dim):
        return False
    return bool(lib().pllm_attention_prefill_tcgen05_supports(_BF16, num_heads, num_kv_heads, head_dim, int(page_size),
                                                              int(window or 0)))


def attention_tile_tokens(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32,
                          head_dim: int = 0, page_size: Optional[int] = None, window: int = 0) -> int:
    """The most query tokens one attention work item may hold, for the kernel that
    paged_attention picks for this dtype, shape and (when given) cache layout."""
    if attention_prefill_uses_tcgen05(dtype, num_heads, num_kv_heads, head_dim, page_size, window):
        return lib().pllm_attention_prefill_tcgen05_tile_tokens(num_heads, num_kv_heads)
    if attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim):
        return lib().pllm_attention_mma_tile_tokens(num_heads, num_kv_heads)
    return lib().pllm_attention_generic_tile_tokens(num_heads, num_kv_heads)


# PAGED_LLM_MIXED_BESIDE=0: in a step of decoded tokens beside prompt portions the tcgen05 kernel takes the
# single tokens too (one launch) instead of the bulk-copy kernel running beside it on a second stream.
MIXED_BESIDE = os.environ.get("PAGED_LLM_MIXED_BESIDE", "1") != "0"
MIXED_BESIDE_MIN_REQUESTS = 9       # rows of the step's block tables (a captured step's capacity)
MIXED_BESIDE_CALLS = 0              # how often that route was taken (for tests)
_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index or 0
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]


def sm_count() -> int:
    """Streaming multiprocessors of the current device (the kernels size their grids by it)."""
    return int(lib().pllm_sm_count())


def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor, w,
                    out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                    status: torch.Tensor, swizzled: bool = False) -> torch.Tensor:
    """Attention of the step's tokens over the paged cache, then the reduction of
    split items.  ``w`` is the group's ``AttentionWork`` (parts/base.py): work items
    int32 [>=max_work, 8], reductions int32 [>=max_red, 4], how many are live as
    int32 scalars on the device, the scratch for partial results, and ``kinds``,
    what the work items are (1 single decoded tokens only, 2 portions of several
    tokens only, 3 both), so that only the kernels with work are launched.
    ``swizzled`` says how the pools are laid out (see ``pool_is_swizzled``)."""
    work, n_work, max_work, red, n_red, max_red = w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red
    part_o, part_ml, kinds = w.part_o, w.part_ml, w.kinds
    _dev(q, k_pool, v_pool, block_tables, work, n_work, out, part_o, part_ml, red, n_red, status)
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml")
    if k_pool.dtype != q.dtype or out.dtype != q.dtype or k_pool.shape != v_pool.shape:
        raise KernelError("paged_attention: q, pools and out must share one dtype, pools one shape")
    if k_pool.dim() != 4 or k_pool.shape[1] != num_kv_heads or k_pool.shape[3] != head_dim:
        raise KernelError(f"paged_attention: pools must be [pages, {num_kv_heads}, page_size, {head_dim}]")
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"paged_attention: head_dim {head_dim} is not a multiple of 16 up to 256")
    if num_heads % num_kv_heads:
        raise KernelError(f"paged_attention: {num_heads} heads do not group over {num_kv_heads} kv heads")
    if work.numel() < max_work * 8 or red.numel() < max_red * 4:
        raise KernelError("paged_attention: work / red lists shorter than their maxima")
    if part_o.shape[1:] != (num_heads, head_dim) or part_ml.shape[1:] != (num_heads, 2):
        raise KernelError("paged_attention: the scratch for partial results is not [rows, heads, head_dim] and [rows, heads, 2]")
    n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    L = lib()
    if attention_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim):
        # The bulk-copy kernel where the cache layout allows it (swizzled rows, pages of a power
        # of two tokens, no window); TMA_KINDS says which items it takes there: 1 single decoded
        # tokens, 2 portions of several tokens, 3 both.  The cp.async kernel takes the rest.
        tma_ok = swizzled and bool(L.pllm_attention_decode_tma_supports(_BF16, num_heads, num_kv_heads, head_dim,
                                                                        page_size, int(window)))
        # portions of several tokens go to the tcgen05 kernel where the layout allows it
        multi_tc = bool(kinds & 2) and swizzled and attention_prefill_uses_tcgen05(q.dtype, num_heads, num_kv_heads, head_dim,
                                                                                   page_size, int(window))
        # (worth the two edges without programmatic launch from some eight requests on: 0.6B shape, a layer of a
        # step of 1 / 8 / 64 decoded tokens at 4096 beside a portion: +9 / -3 / -10 us)
        beside = bool(MIXED_BESIDE and multi_tc and kinds == 3 and tma_ok and (TMA_KINDS & 1)
                      and block_tables.shape[0] >= MIXED_BESIDE_MIN_REQUESTS)
        if beside:
            # A step of decoded tokens beside prompt portions: the single tokens go to the bulk-copy kernel and
            # the portions to the tcgen05 kernel, on two streams that meet again before the reduction.  Neither
            # kernel reads what the other writes, a CTA of one does not fit an SM beside a CTA of the other, and
            # the single tokens' long key ranges no longer queue behind tiles of 128 rows with two of them live.
            global MIXED_BESIDE_CALLS
            MIXED_BESIDE_CALLS += 1
            main, side = torch.cuda.current_stream(), _side_stream(q.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                _check(L.pllm_attention_decode_tma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                                   _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                                   num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                                   block_tables.shape[-1], float(scale), 1, _ptr(status), _stream()),
                       "paged_attention (bulk copy, beside)")
        if multi_tc:
            _check(L.pllm_attention_prefill_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                                    _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                                    q.shape[0], num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                                    block_tables.shape[-1], float(scale), 1 if (kinds == 3 and not beside) else 0,
                                                    _ptr(status), _stream()),
                   "paged_attention (tcgen05)")
            if beside:
                torch.cuda.current_stream().wait_stream(_side_stream(q.device))
            # (else) beside portions it takes the single decoded tokens too: one launch a layer, not two
            kinds = 0 if kinds == 3 else kinds & ~2
        take = (kinds & TMA_KINDS) if tma_ok else 0
        rest = kinds & ~take
        if take:
            _check(L.pllm_attention_decode_tma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                               _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                               num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                               block_tables.shape[-1], float(scale), take, _ptr(status), _stream()),
                   "paged_attention (bulk copy)")
        if rest:
            _check(L.pllm_attention_mma(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables), _ptr(work),
                                        _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml), num_heads,
                                        num_kv_heads, head_dim, page_size, n_pages, block_tables.shape[-1], int(window),
                                        float(scale), 1 if swizzled else 0, rest, _ptr(status), _stream()),
                   "paged_attention (mma)")
    else:
        if swizzled:
            raise KernelError("paged_attention: the generic kernel reads plain pools, not swizzled ones")
        _check(L.pllm_attention_generic(_code(q), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_tables),
                                        _ptr(work), _ptr(n_work), max_work, _ptr(out), _ptr(part_o), _ptr(part_ml),
                                        num_heads, num_kv_heads, head_dim, page_size, n_pages,
                                        block_tables.shape[-1], int(window), float(scale), _ptr(status), _stream()),
               "paged_attention")
    _check(L.pllm_attention_reduce(_code(q), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red,
                                   _ptr(out), num_heads, head_dim, 1 if w.many_splits else 0, _stream()), "attention_reduce")
    return out


# A step of single decoded tokens: the q/k norm, the rotation and the cache write are done by the
# attention kernel itself (PAGED_LLM_FUSE_QK=0: by their own kernel before it, as for prompt portions).
FUSE_QK = os.environ.get("PAGED_LLM_FUSE_QK", "1") != "0"


def decode_attention_fuses(dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int,
                           rotary_dim: int, swizzled: bool) -> bool:
    """Whether ``decode_attention_fused`` takes a step of single tokens of this shape: the bulk-copy
    kernel's conditions, and a rotation over the whole head or none."""
    if not FUSE_QK or not swizzled or not (TMA_KINDS & 1) or rotary_dim not in (0, head_dim):
        return False
    if not attention_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim):
        return False
    return bool(lib().pllm_attention_decode_tma_supports(_BF16, num_heads, num_kv_heads, head_dim, int(page_size),
                                                         int(window or 0)))


def decode_attention_fused(qkv: torch.Tensor, q_gain, k_gain, eps: float, cos, sin, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, block_tables: torch.Tensor, w, out: torch.Tensor, num_heads: int,
                           num_kv_heads: int, head_dim: int, scale: float, status: torch.Tensor) -> torch.Tensor:
    """Attention of a step of single decoded tokens straight from the projection's output
    ``qkv`` [tokens, (heads + 2 kv heads) * head_dim]: per-head norm of q and k, rotation at each
    token's position (the work item's), the token's key and value written to its cache slot
    (found through the block table), attention over the cache, reduction of split items.
    ``w``: the group's ``AttentionWork``."""
    work, n_work, max_work, red, n_red, max_red, part_o, part_ml = (w.work, w.n_work, w.max_work, w.red, w.n_red, w.max_red,
                                                                    w.part_o, w.part_ml)
    _dev(qkv, k_pool, v_pool, block_tables, work, n_work, out, part_o, part_ml, red, n_red, status, q_gain, k_gain, cos, sin)
    _f32(q_gain, "q_gain"); _f32(k_gain, "k_gain"); _f32(cos, "cos"); _f32(sin, "sin")
    _f32(part_o, "part_o"); _f32(part_ml, "part_ml")
    for t, n in ((block_tables, "block_tables"), (work, "work"), (n_work, "n_work"), (red, "red"), (n_red, "n_red")):
        _i32(t, n)
    if qkv.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention_fused: bfloat16 only")
    if qkv.shape[-1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("decode_attention_fused: qkv's width is not (heads + 2 kv heads) * head_dim")
    if (cos is None) != (sin is None) or (cos is not None and cos.shape[-1] * 2 != head_dim):
        raise KernelError("decode_attention_fused: the rotation must span the whole head (or be absent)")
    n_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    L = lib()
    _check(L.pllm_attention_decode_tma_fused(_ptr(qkv), _ptr(q_gain), _ptr(k_gain), float(eps), _ptr(cos), _ptr(sin),
                                             cos.shape[0] if cos is not None else 0, _ptr(k_pool), _ptr(v_pool),
                                             _ptr(block_tables), _ptr(work), _ptr(n_work), max_work, _ptr(out),
                                             _ptr(part_o), _ptr(part_ml), num_heads, num_kv_heads, head_dim, page_size,
                                             n_pages, block_tables.shape[-1], float(scale), _ptr(status), _stream()),
           "decode_attention_fused")
    _check(L.pllm_attention_reduce(_code(out), _ptr(part_o), _ptr(part_ml), _ptr(red), _ptr(n_red), max_red,
                                   _ptr(out), num_heads, head_dim, 1 if w.many_splits else 0, _stream()), "attention_reduce")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """tokens[i] = argmax(logits[i]) where temperature[i] <= 0, else a draw from
    softmax(logits[i] / temperature[i]) at uniform[i], walking ids upward."""
    _dev(logits, temperature, uniform, tokens)
    _f32(logits, "logits"); _f32(temperature, "temperature"); _f32(uniform, "uniform"); _i32(tokens, "tokens")
    n, V = logits.shape
    if min(temperature.numel(), uniform.numel(), tokens.numel()) < n:
        raise KernelError("sample: per-row arguments shorter than the rows")
    L = lib()
    # per chunk of a row (max, first index of it, sum): scratch between the two launches
    scratch = torch.empty(L.pllm_sample_scratch_floats(n, V), dtype=torch.float32, device=logits.device)
    _check(L.pllm_sample(_ptr(logits), n, V, logits.stride(0), _ptr(temperature), _ptr(uniform), _ptr(tokens),
                         _ptr(scratch), _stream()), "sample", launches=2)
    return tokens


SKINNY_GEMM = True  # few rows in bfloat16 go to this library's weight-streaming kernel
FUSE_GLU = os.environ.get("PAGED_LLM_FUSE_GLU", "1") != "0"     # ... with the gated activation in its epilogue


def skinny_gemm_takes(x: torch.Tensor, weight: torch.Tensor, k: Optional[int] = None) -> bool:
    """Whether ``linear`` runs the weight-streaming kernel for this product."""
    if not SKINNY_GEMM or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    N, K = weight.shape
    return x.shape[0] <= SKINNY_MAX_M and bool(lib().pllm_skinny_gemm_supports(x.shape[0], N, K if k is None else k))


# Measured on a B200 inside a captured step (0.6B shapes, microseconds, skinny / cuBLAS):
#   rows 1-8:  qkv 3.5-3.8 / 5.0   o 3.1 / 6.4-7.5   gate_up 4.6-4.8 / 5.1   down 3.9-4.2 / 8.9-9.6
#   rows 64:   qkv 12.3 / 4.9      o 6.3 / 5.4        gate_up 12.6 / 5.3      down 8.4 / 6.6
# so the kernel (which takes up to 64 rows) is used up to 16, and up to a width where the
# library's head product is the faster one (151936 x 1024: 66 / 54).
SKINNY_MAX_M = 16
SKINNY_MAX_N = 32768


# The many rows of a prompt portion in bfloat16: this library's tcgen05 product (csrc/gemm_tcgen05.cu)
# where it is the faster one.  Measured on a B200 at 2048 rows (us, this kernel / cuBLAS):
#   gate/up 6144 x 1024 with silu(gate)*up in the epilogue 25.2 / 24.3 + 10.8 for the activation's own pass
#   qkv 4096 x 1024   18.5 / 17.7      o 1024 x 2048   17.4 / 10.7      down 1024 x 3072   19.5 / 12.6
# so the gated product takes it and the plain ones stay with the library (PAGED_LLM_TCGEN05=0: none,
# =2: the plain ones too).  One CTA's tcgen05.mma reads both operands from shared memory, whose
# bandwidth bounds a 128 x 256 tile at two thirds of the tensor peak; pairs of CTAs are the next step.
TCGEN05_GEMM = int(os.environ.get("PAGED_LLM_TCGEN05", "1"))
TCGEN05_MIN_M = 64     # below this the tiles of 128 rows are mostly padding
_gemm_status: dict = {}


def gemm_status(device) -> torch.Tensor:
    """The status word the tcgen05 product raises bit 64 in when one of its bounded waits
    ran out (one int32 per device; the engine reads it with its own status word)."""
    key = str(device)
    if key not in _gemm_status:
        _gemm_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _gemm_status[key]


def gemm_tcgen05_takes(x, weight: torch.Tensor, n_out: int, glu: bool) -> bool:
    if not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    return x.is_contiguous() and weight.is_contiguous() and bool(
        lib().pllm_gemm_tcgen05_supports(x.shape[0], n_out, weight.shape[1], 1 if glu else 0))


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, glu: bool = False, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x W^T on the tcgen05 tensor cores (bfloat16, float accumulation); with ``glu`` W is
    [gate rows; up rows] and the result is silu(x Wg^T) * (x Wu^T)."""
    M, K = x.shape
    n_out = weight.shape[0] // 2 if glu else weight.shape[0]
    if weight.shape[1] != K or not gemm_tcgen05_takes(x, weight, n_out, glu):
        raise KernelError(f"gemm_tcgen05: does not take x {tuple(x.shape)} {x.dtype}, W {tuple(weight.shape)} {weight.dtype}")
    _dev(x, weight)
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    st = status if status is not None else gemm_status(x.device)
    _check(lib().pllm_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), M, n_out, K, 1 if glu else 0, _ptr(st), _stream()),
           "gemm_tcgen05")
    return out


def skinny_glu_takes(x, weight: torch.Tensor, n_out: int) -> bool:
    """Whether the weight-streaming kernel takes the gate/up product with the activation in its epilogue."""
    if not SKINNY_GEMM or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    return n_out <= SKINNY_MAX_N and bool(lib().pllm_skinny_gemm_glu_supports(x.shape[0], n_out, weight.shape[1]))


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None, gated: bool = False,
           out_dtype: Optional[torch.dtype] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T with W stored [out, in].

    Few rows (a decode step) in bfloat16 run this library's weight-streaming
    kernel.  With ``gated`` the input is [g | u] of twice W's width and the
    product is taken of silu(g) * u, formed by the activation kernel first.
    Everything else is the library matrix product (cuBLAS through torch), which
    is where the reference uses a library too
    (crates/pagedllm/src/model/layers.rs:27-35).  float32 inputs run in true
    float32: the engine switches TF32 off."""
    N, K = weight.shape
    if not x.is_cuda:
        raise KernelError("linear: input is not on a CUDA device: there is no CPU path")
    if x.shape[-1] != (2 * K if gated else K):
        raise KernelError(f"linear: input width {x.shape[-1]} does not fit a weight of {tuple(weight.shape)}")
    want = out_dtype or x.dtype
    if gated:
        # Forming silu(g) * u inside the product that consumes it repeats it in every CTA
        # (measured 31 us against 3.4 + 6 us at batch 8, 3072 -> 1024): a pass of its own here,
        # or the epilogue of the product that makes [g | u] (linear_glu).
        act = torch.empty((x.shape[0], K), dtype=x.dtype, device=x.device)
        swiglu(x, act)
        x = act
    # The widest products (the output head) stay with the library, which is faster there
    # (measured 54 us against 66 us at 151936 x 1024, batch 8).
    if skinny_gemm_takes(x, weight, K) and N <= SKINNY_MAX_N and want in (torch.bfloat16, torch.float32):
        _dev(x, weight, out)
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=want, device=x.device)
        elif out.shape != (M, N) or out.dtype != want:
            raise KernelError("linear: out does not fit")
        _check(lib().pllm_skinny_gemm(_ptr(x), _ptr(weight), _ptr(out), M, N, K,
                                      1 if want == torch.float32 else 0, _stream()), "skinny_gemm")
        return out
    if TCGEN05_GEMM >= 2 and out is None and want == torch.bfloat16 and x.shape[0] >= TCGEN05_MIN_M \
            and gemm_tcgen05_takes(x, weight, N, False):
        return gemm_tcgen05(x, weight, status=status)
    if want != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=want)
    return torch.matmul(x, weight.t(), out=out) if out is not None else torch.matmul(x, weight.t())


def linear_glu(x: torch.Tensor, w_gate_up: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] stacked [2I, K]: the gated
    feed-forward's first half (crates/pagedllm/src/model/layers.rs:93-99).  Few
    rows in bfloat16: one kernel whose CTAs hold the same columns of both halves;
    many rows: the tcgen05 product with the activation in its epilogue; otherwise
    the product, then the activation kernel."""
    two_i, K = w_gate_up.shape
    if two_i % 2:
        raise KernelError("linear_glu: the stacked weight needs an even number of rows")
    inter = two_i // 2
    if x.shape[-1] != K:
        raise KernelError(f"linear_glu: input width {x.shape[-1]} does not fit a weight of {tuple(w_gate_up.shape)}")
    if FUSE_GLU and skinny_glu_takes(x, w_gate_up, inter):
        _dev(x, w_gate_up)
        out = torch.empty((x.shape[0], inter), dtype=torch.bfloat16, device=x.device)
        _check(lib().pllm_skinny_gemm_glu(_ptr(x), _ptr(w_gate_up), _ptr(out), x.shape[0], inter, K, _stream()),
               "skinny_gemm_glu")
        return out
    if TCGEN05_GEMM >= 1 and x.shape[0] >= TCGEN05_MIN_M and gemm_tcgen05_takes(x, w_gate_up, inter, True):
        return gemm_tcgen05(x, w_gate_up, glu=True, status=status)
    gu = linear(x, w_gate_up)
    act = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
    return swiglu(gu, act)
