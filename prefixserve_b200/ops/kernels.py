"""Host-side faces of the kernels: argument checks, output allocation, launch.

Tensors are handed to the C ABI as raw device pointers on the current CUDA
stream.  Everything here refuses CPU tensors: there is no CPU path.
"""

from __future__ import annotations

import math

import torch

from .deferred import Affine, NormedRows, PendingProduct, PostNormed
from .library import KernelError, check, lib, stream_handle

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not one of float32, bfloat16") from None


def _dev(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what} is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous, strides are {t.stride()}")
    return t


def _i32(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, is {t.dtype}")
    return _dev(t, what)


def _stream() -> int:
    return stream_handle()


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """h[t] = float32(table[ids[t]]) * scale (the product in float32)."""
    _i32(ids, "token ids")
    _dev(table, "embedding table")
    t, (v, h) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((t, h), dtype=torch.float32, device=ids.device)
    if scale != 1.0:
        check(lib().psb_embedding_pos(ids.data_ptr(), None, table.data_ptr(), None, _code(table, "embedding table"), out.data_ptr(),
                                      t, h, v, 0, float(scale), _stream()), "embedding_pos")
        return out
    check(lib().psb_embedding(ids.data_ptr(), table.data_ptr(), _code(table, "embedding table"), out.data_ptr(),
                              t, h, v, _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
    """h += delta (float32, in place, unless ``rows``); returns gain * rmsnorm(h) for all or the chosen rows."""
    dscale = dshift = None
    if isinstance(delta, Affine):  # joins the stream as (y + shift) * scale
        delta, dscale, dshift = delta.y, delta.scale, delta.shift
    if isinstance(delta, PendingProduct):
        delta = delta.tensor()
    _dev(h, "residual stream")
    if h.dtype != torch.float32 or h.dim() != 2:
        raise KernelError(f"residual stream must be float32 [T, H], is {h.dtype} {tuple(h.shape)}")
    width = h.shape[1]
    if gain.dtype != torch.float32 or gain.numel() != width:
        raise KernelError(f"norm gain must be float32 [{width}], is {gain.dtype} {tuple(gain.shape)}")
    _dev(gain, "norm gain")
    dcode = F32
    if delta is not None:
        _dev(delta, "sublayer output")
        if delta.shape != h.shape:
            raise KernelError(f"sublayer output {tuple(delta.shape)} does not match the stream {tuple(h.shape)}")
        dcode = _code(delta, "sublayer output")
        for what, v in (("scale", dscale), ("shift", dshift)):
            if v is not None:
                _f32_vector(v, width, f"the sublayer output's {what}")
    n = h.shape[0]
    if rows is not None:
        _i32(rows, "row index")
        n = rows.numel()
    x = torch.empty((n, width), dtype=out_dtype, device=h.device)
    check(lib().psb_add_rmsnorm(h.data_ptr(), _ptr(delta), dcode, gain.data_ptr(), _ptr(rows), x.data_ptr(),
                                _code(x, "norm output"), n, width, float(eps), 0 if rows is not None else 1, _ptr(dscale),
                                _ptr(dshift), _stream()),
          "add_rmsnorm")
    return x


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """a[M,K] @ w[N,K]^T with float32 multiply-adds on the CUDA cores."""
    _dev(a, "left operand")
    _dev(w, "weight")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"cannot multiply {tuple(a.shape)} by the transpose of {tuple(w.shape)}")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    check(lib().psb_gemm_nt(a.data_ptr(), _code(a, "left operand"), w.data_ptr(), _code(w, "weight"), out.data_ptr(),
                            _code(out, "product"), m, n, k, k, k, n, 1 if accumulate else 0, _stream()), "gemm_nt")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x[M,K] @ w[N,K]^T, accumulated in float32.

    bfloat16 x bfloat16 goes to the tensor-core path; every other mix (all of
    the 32-bit path, and weights a checkpoint stores in float32) goes to the
    float32 CUDA-core kernel, so that path never touches a reduced-precision
    matrix mode.
    """
    if isinstance(x, NormedRows):
        if x.fusable and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            from .tensorcore import norm_linear_bf16
            y = norm_linear_bf16(x, w, out_dtype or x.dtype)
            if y is not None:
                return y
        if (out_dtype or x.dtype) == torch.bfloat16 and w.dtype == torch.bfloat16:
            from .tensorcore import fewrows_behind_norm
            y = fewrows_behind_norm(x, w, "plain")
            if y is not None:
                return y
        x = x.tensor()
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from .tensorcore import linear_bf16
        return linear_bf16(x, w, out_dtype)
    return gemm_nt_simt(x, w, out_dtype)


def last_product(x: torch.Tensor, w: torch.Tensor, ctx=None):
    """A sublayer's last product, x @ w^T, whose only reader is the residual sum in front of the next norm.  Where the
    step says that every norm downstream takes one (``ctx.extras["lazy_products"]``) and the rows are few enough for
    the kernel that can carry that sum and the norm's share in its epilogue, the product is handed on unrun
    (``PendingProduct``); otherwise it runs now."""
    extras = getattr(ctx, "extras", None)
    if extras is not None and extras.get("lazy_products") and x.dim() == 2 and x.is_cuda:
        from .tensorcore import fewrows_lazy_ok
        if fewrows_lazy_ok(x, w):
            return PendingProduct(x, w)
    return linear(x, w)


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}  # the codes the kernels know (PsbAct in common.cuh)


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} is not built (one of {sorted(ACTIVATIONS)})") from None


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T) for W = [gate rows; up rows]: fused for bfloat16 rows, else product then activation."""
    code = activation_code(activation)
    if isinstance(x, NormedRows):
        if x.fusable and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
            from .tensorcore import norm_gated_linear_bf16
            act = norm_gated_linear_bf16(x, w_gate_up, code)
            if act is not None:
                return act
        if w_gate_up.dtype == torch.bfloat16:
            from .tensorcore import fewrows_behind_norm
            act = fewrows_behind_norm(x, w_gate_up, "gated", activation=code)
            if act is not None:
                return act
        x = x.tensor()
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
        from .tensorcore import gated_linear_bf16
        _dev(x, "left operand"), _dev(w_gate_up, "weight")
        act = gated_linear_bf16(x, w_gate_up, activation=code)
        if act is not None:
            return act
    return act_mul(linear(x, w_gate_up), activation)


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor, cos: torch.Tensor | None,
                sin: torch.Tensor | None, table: torch.Tensor | None, kv: torch.Tensor | None, *, num_heads: int,
                num_kv_heads: int, head_dim: int, page_size: int, write_kv: bool, paired: bool = False,
                rotary_dim: int | None = None, interleaved: bool = False) -> torch.Tensor:
    """Rotates queries (and keys); stores rotated keys and values in the pages. Returns q [T, hq, D].

    ``paired``: every query and key head comes (and goes) with its elements in the pair-interleaved order of
    ``pair_interleaved_order``; the rotary kernel's header says why that is harmless.
    ``rotary_dim``: only the first so many elements of a head turn (default: all; the tables then hold
    rotary_dim/2 angles); ``interleaved``: element 2j turns with 2j+1 instead of j with j + rotary_dim/2."""
    _dev(qkv, "projection output")
    t = qkv.shape[0]
    hkv_in = num_kv_heads if write_kv else 0
    want = (num_heads + 2 * hkv_in) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] != want:
        raise KernelError(f"projection output must be [T, {want}], is {tuple(qkv.shape)}")
    _i32(positions, "positions")
    _i32(token_item, "token-to-item map")
    rotate = cos is not None
    max_pos = 0
    rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
    if rotary_dim < 2 or rotary_dim > head_dim or rotary_dim % 2:
        raise KernelError(f"rotary_dim {rotary_dim} must be even and within the head size {head_dim}")
    if paired and (rotary_dim != head_dim or interleaved):
        raise KernelError("the paired element order goes with the split-half rotation of a whole head only")
    if rotate:
        assert sin is not None
        _dev(cos, "cos table"), _dev(sin, "sin table")
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2:
            raise KernelError(f"angle tables must be float32 [positions, {rotary_dim // 2}], are {cos.dtype} {tuple(cos.shape)}")
        max_pos = cos.shape[0]
    width = num_pages = 0
    kv_code = _code(qkv, "projection output")
    if write_kv:
        if kv is None or table is None:
            raise KernelError("appending to the cache needs the cache entry and the page table")
        _dev(kv, "cache entry"), _i32(table, "page table")
        if kv.dim() != 5 or tuple(kv.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
            raise KernelError(f"cache entry must be [pages, 2, {num_kv_heads}, {page_size}, {head_dim}], is {tuple(kv.shape)}")
        num_pages, width, kv_code = kv.shape[0], table.shape[1], _code(kv, "cache entry")
    q = torch.empty((t, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    check(lib().psb_rope_append(qkv.data_ptr(), _code(qkv, "projection output"), positions.data_ptr(),
                                token_item.data_ptr(), _ptr(cos), _ptr(sin), _ptr(table) if write_kv else None, width,
                                _ptr(kv) if write_kv else None, kv_code, q.data_ptr(), t, num_heads, hkv_in, head_dim,
                                page_size, num_pages, max_pos, 1 if rotate else 0, 1 if write_kv else 0, 1 if paired else 0,
                                rotary_dim, 1 if interleaved else 0, _stream()),
          "rope_append")
    return q


def pair_interleaved_order(head_dim: int) -> list[int]:
    """For a head size that is a multiple of 16: natural element index for each stored index when 8 elements of the
    first half are followed by the 8 elements they are rotated with (split-half rotation pairs d with d + D/2)."""
    if head_dim % 16:
        raise KernelError(f"a head size of {head_dim} cannot be pair-interleaved (multiples of 16 only)")
    order: list[int] = []
    for block in range(head_dim // 16):
        order += list(range(8 * block, 8 * block + 8)) + list(range(head_dim // 2 + 8 * block, head_dim // 2 + 8 * block + 8))
    return order


def qkv_rope_append(x: NormedRows, w_qkv: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor,
                    cos: torch.Tensor | None, sin: torch.Tensor | None, table: torch.Tensor, kv: torch.Tensor, *,
                    num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> torch.Tensor | None:
    """rmsnorm(h + pending) @ w_qkv^T, rotation and append to the pages, for bfloat16 tokens and a projection whose
    query and key rows are pair-interleaved: one kernel for few tokens (the norm folded in as well), the norm's kernel
    and one product that rotates and stores in its epilogue for many.  Returns q [T, hq, D], or None when neither kernel
    takes the case (the caller then runs the product and ``rope_append(..., paired=True)``)."""
    from .tensorcore import norm_qkv_rope_bf16, tcgen05_qkv_rope_bf16
    if not (x.rows is None and x.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
            and kv.dtype == torch.bfloat16 and head_dim % 16 == 0 and page_size & (page_size - 1) == 0):
        return None
    _i32(positions, "positions"), _i32(token_item, "token-to-item map"), _i32(table, "page table"), _dev(kv, "cache entry")
    if kv.dim() != 5 or tuple(kv.shape[1:]) != (2, num_kv_heads, page_size, head_dim):
        raise KernelError(f"cache entry must be [pages, 2, {num_kv_heads}, {page_size}, {head_dim}], is {tuple(kv.shape)}")
    if w_qkv.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"projection has {w_qkv.shape[0]} rows, not {(num_heads + 2 * num_kv_heads) * head_dim}")
    if cos is not None and (sin is None or cos.dtype != torch.float32 or cos.shape != sin.shape or cos.dim() != 2
                            or cos.shape[1] != head_dim // 2):
        raise KernelError(f"angle tables must be float32 [positions, {head_dim // 2}]")
    if x.fusable:
        q = norm_qkv_rope_bf16(x, w_qkv, positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads, head_dim, page_size)
        if q is not None:
            return q
    from .tensorcore import fewrows_behind_norm
    q = fewrows_behind_norm(x, w_qkv, "rope", rope=(positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads, head_dim, page_size))
    if q is not None:
        return q
    return tcgen05_qkv_rope_bf16(x.tensor(), w_qkv, positions, token_item, cos, sin, table, kv, num_heads, num_kv_heads,
                                 head_dim, page_size)


def attention_generic(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                      token_item: torch.Tensor, *, window: int | None, scale: float, sink: torch.Tensor | None = None) -> torch.Tensor:
    _dev(q, "queries"), _dev(kv, "cache entry")
    _i32(table, "page table"), _i32(positions, "positions"), _i32(token_item, "token-to-item map")
    t, hq, d = q.shape
    _, two, hkv, page, dk = kv.shape
    if two != 2 or dk != d:
        raise KernelError(f"cache entry {tuple(kv.shape)} does not fit queries {tuple(q.shape)}")
    out = torch.empty((t, hq * d), dtype=q.dtype, device=q.device)
    check(lib().psb_attention_generic(q.data_ptr(), _code(q, "queries"), kv.data_ptr(), _code(kv, "cache entry"),
                                      table.data_ptr(), table.shape[1], positions.data_ptr(), token_item.data_ptr(),
                                      out.data_ptr(), t, hq, hkv, d, page, int(window or 0), float(scale), _ptr(sink), _stream()),
          "attention")
    return out


def attention(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
              token_item: torch.Tensor, *, window: int | None = None, scale: float | None = None,
              ctx=None, sink: torch.Tensor | None = None) -> torch.Tensor:
    """Causal grouped-query attention of the step's tokens over their requests' pages -> [T, hq*D].  ``sink`` (float32
    [hq]): a score per head that joins every row's softmax denominator without a key or a value."""
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != q.shape[1] or not sink.is_cuda or not sink.is_contiguous()):
        raise KernelError(f"sinks must be float32 [{q.shape[1]}] on the device")
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and ctx is not None:
        from .tensorcore import attention_bf16
        _dev(q, "queries"), _dev(kv, "cache entry"), _i32(table, "page table")
        if q.shape[1] % kv.shape[2] or kv.shape[4] != q.shape[2] or kv.shape[1] != 2:
            raise KernelError(f"cache entry {tuple(kv.shape)} does not fit queries {tuple(q.shape)}")
        extras = getattr(ctx, "extras", None)
        fast = attention_bf16(q, kv, table, ctx.item_start, ctx.kv_len, None, None, window=window, scale=scale,
                              static_kv_len=extras.get("static_kv_len") if extras is not None else None,
                              plans=extras, items=ctx.items, token_item=_i32(token_item, "token-to-item map"), sink=sink)
        if fast is not None:
            return fast
    return attention_generic(q, kv, table, positions, token_item, window=window, scale=scale, sink=sink)


def act_mul(gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    """[T, 2I] -> act(first half) * second half, [T, I]."""
    _dev(gate_up, "gate/up projection")
    t, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"gate/up projection must have an even width, has {two_i}")
    out = torch.empty((t, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(lib().psb_silu_mul(gate_up.data_ptr(), _code(gate_up, "gate/up projection"), out.data_ptr(), t, two_i // 2,
                             activation_code(activation), _stream()), "silu_mul")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] -> silu(first half) * second half, [T, I]."""
    return act_mul(gate_up, "silu")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h += delta in place (h float32, delta float32 or bfloat16 of the same shape); returns h."""
    if isinstance(delta, PostNormed):  # a result that brings its own norm: h += gain * rmsnorm(y)
        norm_add_norm(h, delta.y, delta.gain, delta.eps)
        return h
    if isinstance(delta, PendingProduct):
        delta = delta.tensor()
    _dev(h, "residual stream"), _dev(delta, "sublayer output")
    if h.dtype != torch.float32 or delta.shape != h.shape:
        raise KernelError(f"residual stream must be float32 and the output must match it: {h.dtype} {tuple(h.shape)} vs {tuple(delta.shape)}")
    check(lib().psb_residual_add(h.data_ptr(), delta.data_ptr(), _code(delta, "sublayer output"), h.numel(), _stream()), "residual_add")
    return h


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seed: torch.Tensor | None = None,
           position: torch.Tensor | None = None) -> torch.Tensor:
    """Arg max (temperature absent or 0) or Gumbel-max sampling per row -> int32 [S]."""
    _dev(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError(f"logits must be float32 [S, V], are {logits.dtype} {tuple(logits.shape)}")
    s, v = logits.shape
    if temperature is not None:
        if seed is None or position is None:
            raise KernelError("temperature sampling needs seed and position per row")
        _dev(temperature, "temperature"), _dev(seed, "seed"), _i32(position, "position")
        if temperature.dtype != torch.float32 or seed.dtype != torch.int64:
            raise KernelError("temperature must be float32 and seed int64")
        if temperature.numel() != s or seed.numel() != s or position.numel() != s:
            raise KernelError("temperature, seed and position need one entry per logits row")
    out = torch.empty((s,), dtype=torch.int32, device=logits.device)
    need = lib().psb_sample_scratch_bytes(s, v)
    scratch = torch.empty((need,), dtype=torch.uint8, device=logits.device) if need else None
    check(lib().psb_sample(logits.data_ptr(), _ptr(temperature), _ptr(seed), _ptr(position), out.data_ptr(),
                           _ptr(scratch), s, v, _stream()), "sample")
    return out


def sample_slots(logits: torch.Tensor, records: torch.Tensor, row_slot: torch.Tensor) -> torch.Tensor:
    """The same choice with each row's temperature, seed and position read on the device from the record of the row's
    request slot (``records`` int32 [num_slots, words]: position, temperature bits, seed low, seed high) -> int32 [S]."""
    _dev(logits, "logits"), _i32(records, "slot records"), _i32(row_slot, "slot of each row")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError(f"logits must be float32 [S, V], are {logits.dtype} {tuple(logits.shape)}")
    s, v = logits.shape
    if records.dim() != 2 or records.shape[1] < 4 or row_slot.numel() != s:
        raise KernelError(f"slot records must be [slots, >=4] and one slot per logits row is needed, got {tuple(records.shape)}, "
                          f"{row_slot.numel()} slots for {s} rows")
    out = torch.empty((s,), dtype=torch.int32, device=logits.device)
    need = lib().psb_sample_scratch_bytes(s, v)
    scratch = torch.empty((need,), dtype=torch.uint8, device=logits.device) if need else None
    check(lib().psb_sample_slots(logits.data_ptr(), records.data_ptr(), row_slot.data_ptr(), records.shape[1], out.data_ptr(),
                                 _ptr(scratch), s, v, _stream()), "sample")
    return out


def scatter_words(resident: torch.Tensor, pairs: torch.Tensor, count: int) -> None:
    """resident[pairs[2i]] = pairs[2i+1] for i < count (int32 arrays on the device; every index at most once)."""
    _i32(resident, "resident array"), _i32(pairs, "index/value pairs")
    if count < 0 or pairs.numel() < 2 * count:
        raise KernelError(f"{count} pairs do not fit in {pairs.numel()} words")
    check(lib().psb_scatter_words(resident.data_ptr(), pairs.data_ptr(), count, resident.numel(), _stream()), "scatter_words")


def step_prepare(records: torch.Tensor | None, kv_len: torch.Tensor | None, slots: torch.Tensor, rows: torch.Tensor | None,
                 out: torch.Tensor | None) -> None:
    """out[i, :] = rows[slots[i], :width] (the page table of a step from the rows that stay on the device, padded
    with -1 beyond their width), and records[slots[i]].position = kv_len[i].  Either half may be left out."""
    _i32(slots, "slots")
    b = slots.numel()
    num_slots = record_words = row_width = width = 0
    if records is not None:
        _i32(records, "slot records"), _i32(kv_len, "kv_len")
        if records.dim() != 2 or kv_len.numel() != b:
            raise KernelError("slot records must be [slots, words] and kv_len needs one entry per item")
        num_slots, record_words = records.shape
    if rows is not None:
        _i32(rows, "resident page table"), _i32(out, "page table of the step")
        if rows.dim() != 2 or out.dim() != 2 or out.shape[0] != b:
            raise KernelError(f"page tables must be [slots, pages] and [{b}, width], are {tuple(rows.shape)} and {tuple(out.shape)}")
        num_slots, row_width = rows.shape
        width = out.shape[1]
    if records is None and rows is None:
        return
    check(lib().psb_step_prepare(_ptr(records), record_words, _ptr(kv_len), slots.data_ptr(), _ptr(rows), row_width, _ptr(out),
                                 width, b, num_slots, _stream()), "step_prepare")


_BMM_INTO_VIEW = True   # cleared if this torch refuses ``out=`` with a result type of its own
PER_HEAD_LIBRARY_ROWS = 128  # per-head products of bfloat16 rows: from this many rows on, the library's batched product


def linear_per_head(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """out[t, h, :] = w[h] @ a[t, h, :] for a [T, heads, K] (a view whose last axis is contiguous and whose head axis
    has a fixed stride: a slice of a wider [T, heads, more] tensor will do), w [heads, N, K] contiguous, out
    [T, heads, N] (again possibly a slice of a wider tensor).  Per-head and block-diagonal matrices; float32 sums."""
    _dev(w, "per-head weight")
    if a.dim() != 3 or w.dim() != 3 or a.shape[1] != w.shape[0] or a.shape[2] != w.shape[2] or a.stride(2) != 1 or not a.is_cuda:
        raise KernelError(f"cannot multiply rows {tuple(a.shape)} (strides {a.stride()}) by per-head matrices {tuple(w.shape)}")
    t, heads, k = a.shape
    n = w.shape[1]
    if out is None:
        out = torch.empty((t, heads, n), dtype=out_dtype or a.dtype, device=a.device)
    if tuple(out.shape) != (t, heads, n) or out.stride(2) != 1 or not out.is_cuda:
        raise KernelError(f"per-head product output must be [{t}, {heads}, {n}] with a contiguous last axis")
    if t >= PER_HEAD_LIBRARY_ROWS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        # many rows: the library's batched product on the tensor cores (as ``linear`` sends its mid-sized products
        # there), sums in float32 when the output is
        global _BMM_INTO_VIEW
        if _BMM_INTO_VIEW:  # straight into out's [heads, T, N] view: the library takes a leading dimension and a batch stride
            try:
                if out.dtype == torch.float32:
                    torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32, out=out.transpose(0, 1))
                else:
                    torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
                return out
            except (TypeError, RuntimeError):
                if torch.cuda.is_current_stream_capturing():
                    raise
                _BMM_INTO_VIEW = False
        y = torch.bmm(a.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32) if out.dtype == torch.float32 \
            else torch.bmm(a.transpose(0, 1), w.transpose(1, 2))
        out.copy_(y.transpose(0, 1))
        return out
    check(lib().psb_gemm_nt_batched(a.data_ptr(), _code(a, "left operand"), w.data_ptr(), _code(w, "weight"), out.data_ptr(),
                                    _code(out, "product"), t, n, k, a.stride(0), k, out.stride(0), heads, a.stride(1),
                                    n * k, out.stride(1), _stream()), "gemm_nt_batched")
    return out


def hashed_embedding(ids: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor, item_start: torch.Tensor,
                     slots: torch.Tensor, last_token: torch.Tensor, table: torch.Tensor, pair_table: torch.Tensor, *,
                     mul_prev: int, mul_cur: int, copy_dtype: torch.dtype | None = None):
    """h[t] = float32(table[ids[t]]) + float32(pair_table[(prev * mul_prev + ids[t] * mul_cur) mod buckets]), the last
    row of pair_table at position 0; ``prev`` of a portion's first token comes from ``last_token`` [num_slots], which is
    then set to the portion's last token.  Returns (h float32, a copy in ``copy_dtype`` or None)."""
    for what, x in (("token ids", ids), ("positions", positions), ("token-to-item map", token_item), ("item offsets", item_start),
                    ("slots", slots), ("last tokens", last_token)):
        _i32(x, what)
    _dev(table, "embedding table"), _dev(pair_table, "pair table")
    t, (v, h) = ids.numel(), table.shape
    if pair_table.dim() != 2 or pair_table.shape[1] != h or pair_table.shape[0] < 2 or pair_table.dtype != table.dtype:
        raise KernelError(f"pair table {tuple(pair_table.shape)} {pair_table.dtype} does not fit the embedding table {tuple(table.shape)} {table.dtype}")
    out = torch.empty((t, h), dtype=torch.float32, device=ids.device)
    copy = torch.empty((t, h), dtype=copy_dtype, device=ids.device) if copy_dtype not in (None, torch.float32) else None
    check(lib().psb_hashed_embedding(ids.data_ptr(), positions.data_ptr(), token_item.data_ptr(), item_start.data_ptr(),
                                     slots.data_ptr(), last_token.data_ptr(), table.data_ptr(), pair_table.data_ptr(),
                                     _code(table, "embedding table"), out.data_ptr(), _ptr(copy),
                                     _code(copy, "copy") if copy is not None else F32, t, slots.numel(), h, v,
                                     pair_table.shape[0] - 1, int(mul_prev), int(mul_cur), last_token.numel(), _stream()),
          "hashed_embedding")
    return out, copy


def gated_norm_add(h: torch.Tensor, y: torch.Tensor, gate: torch.Tensor | None, gate_bias: torch.Tensor | None,
                   gain: torch.Tensor, eps: float, mult: float, copy_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """h += mult * gain * rmsnorm(y * sigmoid(gate + gate_bias)) in place (h float32; without ``gate`` the norm is taken
    of y itself).  Returns the new h in ``copy_dtype`` (None when that is float32 or not asked for: read h)."""
    if isinstance(y, PendingProduct):
        y = y.tensor()
    _dev(h, "residual stream"), _dev(y, "sublayer output"), _dev(gain, "norm gain")
    if h.dtype != torch.float32 or h.dim() != 2 or y.shape != h.shape:
        raise KernelError(f"residual stream must be float32 [T, H] and the output must match it: {h.dtype} {tuple(h.shape)} vs {tuple(y.shape)}")
    rows, width = h.shape
    if gain.dtype != torch.float32 or gain.numel() != width:
        raise KernelError(f"norm gain must be float32 [{width}]")
    if gate is not None:
        _dev(gate, "gate")
        if gate.shape != h.shape:
            raise KernelError(f"gate {tuple(gate.shape)} does not match the stream {tuple(h.shape)}")
        if gate_bias is not None and (gate_bias.dtype != torch.float32 or gate_bias.numel() != width or not gate_bias.is_cuda):
            raise KernelError(f"gate bias must be float32 [{width}] on the device")
    copy = torch.empty((rows, width), dtype=copy_dtype, device=h.device) if copy_dtype not in (None, torch.float32) else None
    check(lib().psb_gated_norm_add(h.data_ptr(), y.data_ptr(), _code(y, "sublayer output"), _ptr(gate),
                                   _code(gate, "gate") if gate is not None else F32, _ptr(gate_bias) if gate is not None else None,
                                   gain.data_ptr(), _ptr(copy), _code(copy, "copy") if copy is not None else F32, rows, width,
                                   float(eps), float(mult), _stream()), "gated_norm_add")
    return copy


UNARY_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "xielu": 2, "relu2": 3}  # the codes of activation.cu; xielu takes two learned numbers


def activation(x: torch.Tensor, name: str, params: torch.Tensor | None = None) -> torch.Tensor:
    """act(x) element by element; ``params``: float32 numbers of the activation on the device (xielu: p, q)."""
    try:
        code = UNARY_ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} is not built (one of {sorted(UNARY_ACTIVATIONS)})") from None
    _dev(x, "activation input")
    if name == "xielu":
        if params is None or params.dtype != torch.float32 or params.numel() != 2 or not params.is_cuda:
            raise KernelError("xielu needs its two numbers as float32 on the device")
    out = torch.empty_like(x)
    check(lib().psb_unary_act(x.data_ptr(), _code(x, "activation input"), out.data_ptr(), x.numel(), code, _ptr(params), _stream()),
          "unary_act")
    return out


def latent_prepare(proj: torch.Tensor, positions: torch.Tensor, token_item: torch.Tensor, table: torch.Tensor,
                   cos: torch.Tensor | None, sin: torch.Tensor | None, gain_q: torch.Tensor, gain_kv: torch.Tensor,
                   cache: torch.Tensor, *, q_rank: int, rank: int, rot: int, rot_dims: int, heads: int, page_size: int,
                   eps: float):
    """One row of the fused projection [query latent | key/value latent | rotated key part | head gates] -> (normed query
    latent [T, q_rank], sigmoid of the gates float32 [T, heads]); the normed key/value latent and the rotated key part
    go to the token's row of the cache [pages, page_size, rank + rot]."""
    _dev(cache, "cache entry")
    _i32(positions, "positions"), _i32(token_item, "token-to-item map"), _i32(table, "page table")
    t = proj.shape[0]
    if not proj.is_cuda or proj.dim() != 2 or proj.shape[1] != q_rank + rank + rot + heads or proj.stride(1) != 1:
        raise KernelError(f"projection output must be [T, {q_rank + rank + rot + heads}] on the device (rows may be part of wider ones), is {tuple(proj.shape)}")
    if cache.numel() % (page_size * (rank + rot)) or cache.shape[-1] != rank + rot or cache.shape[-2] != page_size:
        raise KernelError(f"cache entry must be [pages, .., {page_size}, {rank + rot}], is {tuple(cache.shape)}")
    for what, g, n in (("query latent gain", gain_q, q_rank), ("key/value latent gain", gain_kv, rank)):
        if n == 0 and g is None:  # no query latent in the row (queries projected directly)
            continue
        if g.dtype != torch.float32 or g.numel() != n or not g.is_cuda:
            raise KernelError(f"{what} must be float32 [{n}] on the device")
    max_pos = 0
    if rot_dims:
        if cos is None or sin is None or cos.dtype != torch.float32 or cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rot_dims // 2:
            raise KernelError(f"angle tables must be float32 [positions, {rot_dims // 2}]")
        _dev(cos, "cos table"), _dev(sin, "sin table")
        max_pos = cos.shape[0]
    cq = torch.empty((t, q_rank), dtype=proj.dtype, device=proj.device)
    gate = torch.empty((t, heads), dtype=torch.float32, device=proj.device)
    check(lib().psb_latent_prepare(proj.data_ptr(), _code(proj, "projection output"), positions.data_ptr(), token_item.data_ptr(),
                                   table.data_ptr(), table.shape[1], _ptr(cos), _ptr(sin), _ptr(gain_q), gain_kv.data_ptr(),
                                   cq.data_ptr(), gate.data_ptr(), cache.data_ptr(), _code(cache, "cache entry"), t, q_rank, rank,
                                   rot, rot_dims, heads, page_size, cache.shape[0], max_pos, float(eps), int(proj.stride(0)), _stream()),
          "latent_prepare")
    return cq, gate


def latent_query_rotate(q: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
                        q_lat: torch.Tensor, *, heads: int, plain: int, rot: int, rot_dims: int, rank: int) -> None:
    """q [T, heads * (plain + rot)]: every head's rotated part, turned by the token's position, into q_lat[:, :, rank:]
    (float32 [T, heads, rank + rot])."""
    _dev(q_lat, "latent queries"), _i32(positions, "positions")
    t = q.shape[0]
    if not q.is_cuda or q.dim() != 2 or q.stride(1) != 1 or q.shape[1] != heads * (plain + rot) or q_lat.dtype != torch.float32 or tuple(q_lat.shape) != (t, heads, rank + rot):
        raise KernelError(f"queries {tuple(q.shape)} / latent queries {q_lat.dtype} {tuple(q_lat.shape)} do not fit {heads} heads of {plain}+{rot} and a latent of {rank}")
    check(lib().psb_latent_query_rotate(q.data_ptr(), _code(q, "queries"), positions.data_ptr(), _ptr(cos), _ptr(sin), q_lat.data_ptr(),
                                        t, heads, plain, rot, rot_dims, rank, cos.shape[0] if cos is not None else 0, int(q.stride(0)),
                                        _stream()),
          "latent_query_rotate")


def gate_mul(x: torch.Tensor, gate: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x * gate element by element (gate float32, e.g. a sigmoid already taken; the product in float32), in ``out_dtype``."""
    _dev(x, "gated values"), _dev(gate, "gate")
    if gate.dtype != torch.float32 or gate.numel() != x.numel():
        raise KernelError(f"the gate must be float32 with {x.numel()} numbers, is {gate.dtype} {tuple(gate.shape)}")
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    check(lib().psb_gate_mul(x.data_ptr(), _code(x, "gated values"), gate.data_ptr(), out.data_ptr(), _code(out, "gated output"),
                             x.numel(), _stream()), "gate_mul")
    return out


BAND_MIN_TOKENS = 64    # portions from this many tokens on take the banded form of latent attention (bfloat16, with a window)
BAND_CHUNK = 256        # tokens of a portion whose band of keys is handled by one set of products
BAND_MAX_WINDOW = 8192  # wider windows stay with the kernel that walks the keys


def latent_attention(q_lat: torch.Tensor, cache: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
                     token_item: torch.Tensor, gate: torch.Tensor | None, *, rank: int, page_size: int, window: int | None,
                     scale: float, out_dtype: torch.dtype, items=None, key_hint: int = 0,
                     sink: torch.Tensor | None = None, static_shapes: bool = False) -> torch.Tensor:
    """Softmax attention of latent-space queries [T, heads, rank + rot] (float32) over the cached rows
    [pages, page_size, rank + rot]; returns sum_j p_j c_j times the head's gate, [T, heads, rank].

    ``items`` (the step's host-side item list): portions of ``BAND_MIN_TOKENS`` tokens or more of a bfloat16 cache with
    a window go through the banded form (the keys a run of tokens can see gathered into a matrix, scores and weighted
    sums as products on the tensor cores, softmax in float32 between them); single tokens and short portions through
    the kernel that walks the keys.  Which form a token takes depends on its portion's length only.

    Without a window the band of a run of tokens is every key up to the run's last token: as wide as the run's own
    positions say in a step that runs at once, as wide as the step's class of lengths (``key_hint``, with
    ``static_shapes``) in a step whose launches are captured for later steps of other positions.

    ``sink`` (float32 [heads]): a score per head whose exponential joins the softmax denominator once, without a key or
    a value."""
    _dev(q_lat, "latent queries"), _dev(cache, "cache entry")
    _i32(table, "page table"), _i32(positions, "positions"), _i32(token_item, "token-to-item map")
    t, heads, d = q_lat.shape
    if q_lat.dtype != torch.float32 or cache.shape[-1] != d or cache.shape[-2] != page_size or d < rank:
        raise KernelError(f"latent queries {q_lat.dtype} {tuple(q_lat.shape)} do not fit the cache entry {tuple(cache.shape)}")
    if gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (t, heads) or not gate.is_cuda):
        raise KernelError(f"head gates must be float32 [{t}, {heads}]")
    if sink is not None:
        _f32_vector(sink, heads, "sinks")
    out = torch.empty((t, heads, rank), dtype=out_dtype, device=q_lat.device)
    banded = []
    reach = window or (key_hint if static_shapes else max((it.end for it in items), default=0) if items is not None else 0)
    if (items is not None and 0 < reach <= BAND_MAX_WINDOW and cache.dtype == torch.bfloat16 and d % 8 == 0 and rank % 8 == 0):
        banded = [(it.first_token, it.end - it.start, it.start) for it in items if it.end - it.start >= BAND_MIN_TOKENS]
    at = 0
    for first, n, _ in banded + [(t, 0, 0)]:   # the tokens between the banded portions: runs for the kernel that walks the keys
        if first > at:
            _latent_attention_walk(q_lat[at:first], cache, table, positions[at:first], token_item[at:first],
                                   None if gate is None else gate[at:first], out[at:first], rank, page_size, window, scale,
                                   key_hint=int(window or key_hint), sink=sink)
        at = first + n
    if banded:
        q16 = torch.empty((t, heads, d), dtype=torch.bfloat16, device=q_lat.device)
        lo_t, hi_t = banded[0][0], banded[-1][0] + banded[-1][1]
        check(lib().psb_split_pairs(q_lat[lo_t:hi_t].data_ptr(), q16[lo_t:hi_t].data_ptr(), None,
                                    (hi_t - lo_t) * heads * d, _stream()), "split_pairs")
        for first, n, start in banded:
            for c0 in range(first, first + n, BAND_CHUNK):
                nc = min(BAND_CHUNK, first + n - c0)
                # no window: the band reaches back to the sequence's first key (the chunk's last position + 1 keys)
                reach = window or (key_hint if static_shapes else start + (c0 - first) + nc)
                _latent_attention_band(q16, cache, table, positions, token_item, gate, out, c0, nc, rank, page_size, reach, scale, sink)
    return out


# The kernel that reads rows side by side holds a (token, head pair)'s sums in registers (234 a thread with two heads): one
# block of eight warps an SM.  Its blocks walk their keys in a chain of dependent loads, so a launch costs (rounds of blocks
# over the SMs) x (keys a block + a fixed share); the keys of a (token, heads) are split among as many blocks as makes that
# least (8 tokens of 16 heads over 2,048 keys: 64 units x 2 blocks in one round, 1,024 keys each, instead of 64 x 5 in three
# rounds of 410: 105 -> 86 us a layer).
ROWS_BLOCK_SHARE = 96      # what a block costs beyond its keys, in keys
ROWS_KEYS_PER_SPLIT = 128  # no block of that kernel is given fewer keys than this by splitting


def _rows_splits(blocks: int, keys: int, slots: int) -> int:
    best, best_cost = 1, None
    for s in range(1, 9):
        if s > 1 and keys // s < ROWS_KEYS_PER_SPLIT:
            break
        cost = -(-blocks * s // slots) * (keys / s + ROWS_BLOCK_SHARE)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def _latent_attention_walk(q_lat, cache, table, positions, token_item, gate, out, rank, page_size, window, scale,
                           key_hint: int = 0, sink=None) -> None:
    """Tokens that walk their keys.  ``key_hint``: about how many keys the longest walk has (the window, or the step's
    longest sequence), for the choice of how many blocks share a (token, head)."""
    t, heads, d = q_lat.shape
    hp, splits, partial = 1, 1, None
    if lib().psb_latent_attention_rows_supported(_code(cache, "cache entry"), rank, d - rank):
        if heads % 2 == 0 and d <= 768:
            hp = 2  # two heads of a token share a block and every row it loads
        blocks = t * heads // hp
        if key_hint >= 2 * ROWS_KEYS_PER_SPLIT:
            from .tensorcore import _sms
            splits = _rows_splits(blocks, key_hint, _sms(q_lat.device))
        if splits > 1:
            partial = torch.empty((t, heads, splits, rank + 2), dtype=torch.float32, device=q_lat.device)
    check(lib().psb_latent_attention(q_lat.data_ptr(), cache.data_ptr(), _code(cache, "cache entry"), table.data_ptr(), table.shape[1],
                                     positions.data_ptr(), token_item.data_ptr(), _ptr(gate), out.data_ptr(), _code(out, "output"),
                                     t, heads, rank, d - rank, page_size, cache.shape[0], int(window or 0), float(scale), hp, splits,
                                     _ptr(partial), _ptr(sink), _stream()),
          "latent_attention")


def _latent_attention_band(q16, cache, table, positions, token_item, gate, out, t0, n, rank, page_size, window, scale, sink=None) -> None:
    """Tokens t0 .. t0+n-1 (consecutive tokens of one request) against the window + n - 1 keys they can see."""
    _, heads, d = q16.shape
    kp = -(-(window + n - 1) // 8) * 8
    dev = q16.device
    band = torch.empty((kp, d), dtype=cache.dtype, device=dev)
    values2 = torch.empty((2 * kp, rank), dtype=cache.dtype, device=dev)
    check(lib().psb_latent_band_gather(cache.data_ptr(), _code(cache, "cache entry"), table.data_ptr(), table.shape[1],
                                       positions.data_ptr(), token_item.data_ptr(), band.data_ptr(), values2.data_ptr(), t0, n, kp,
                                       d, rank, page_size, cache.shape[0], window, _stream()), "latent_band_gather")
    rows = n * heads
    scores = torch.mm(q16[t0:t0 + n].view(rows, d), band.t(), out_dtype=torch.float32)
    weights = torch.empty((rows, 2 * kp), dtype=torch.bfloat16, device=dev)
    check(lib().psb_latent_band_softmax(scores.data_ptr(), positions.data_ptr(), weights.data_ptr(), t0, n, heads, kp, window,
                                        float(scale), _ptr(sink), _stream()), "latent_band_softmax")
    mixed = torch.mm(weights, values2, out_dtype=torch.float32)
    check(lib().psb_latent_band_finish(mixed.data_ptr(), None if gate is None else gate[t0:t0 + n].data_ptr(),
                                       out[t0:t0 + n].data_ptr(), _code(out, "output"), rank, rows * rank, _stream()),
          "latent_band_finish")


SCAN_CHUNK = 64  # tokens of a chunk when the recurrence cuts long portions into chunks that run side by side


def causal_conv(proj: torch.Tensor, bias_x: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, state: torch.Tensor,
                ctx) -> torch.Tensor:
    """proj [T, 2W] (gate branch, convolution branch): u[t] = conv over the branch's last K inputs (+ biases), inputs from
    before the portion read from ``state`` [num_slots, K, W] (rows 0..K-2)."""
    _dev(proj, "projection output"), _dev(state, "recurrent state")
    t, two_w = proj.shape
    w = two_w // 2
    k = conv_w.shape[1]
    if two_w != 2 * w or tuple(conv_w.shape) != (w, k) or state.dtype != torch.float32 or tuple(state.shape[1:]) != (k, w):
        raise KernelError(f"projection {tuple(proj.shape)}, taps {tuple(conv_w.shape)} and state {state.dtype} {tuple(state.shape)} do not fit")
    for what, x, n in (("branch bias", bias_x, w), ("tap weights", conv_w, w * k), ("tap bias", conv_b, w)):
        if x.dtype != torch.float32 or x.numel() != n or not x.is_cuda or not x.is_contiguous():
            raise KernelError(f"{what} must be float32 with {n} numbers on the device")
    u = torch.empty((t, w), dtype=proj.dtype, device=proj.device)
    check(lib().psb_causal_conv(proj.data_ptr(), _code(proj, "projection output"), bias_x.data_ptr(), conv_w.data_ptr(),
                                conv_b.data_ptr(), state.data_ptr(), _i32(ctx.positions, "positions").data_ptr(),
                                _i32(ctx.token_item, "token-to-item map").data_ptr(), _i32(ctx.item_start, "item offsets").data_ptr(),
                                _i32(ctx.slots, "slots").data_ptr(), u.data_ptr(), t, w, k, state.shape[0], _stream()), "causal_conv")
    return u


def recurrence_scan(proj: torch.Tensor, u: torch.Tensor, gates: torch.Tensor, bias_y: torch.Tensor, bias_x: torch.Tensor,
                    bias_r: torch.Tensor, bias_i: torch.Tensor, lam: torch.Tensor, state: torch.Tensor, ctx, *, blocks: int,
                    decay: float) -> torch.Tensor:
    """The gated linear recurrence over every portion of the step, from and to ``state`` [num_slots, K, W] (row K-1; the
    rows before it receive the portion's last convolution inputs).  gates float32 [T, blocks, 2 * W/blocks]."""
    _dev(proj, "projection output"), _dev(u, "convolved branch"), _dev(gates, "gate pre-activations"), _dev(state, "recurrent state")
    t, w = u.shape
    k = state.shape[1]
    if proj.shape != (t, 2 * w) or u.dtype != proj.dtype or gates.dtype != torch.float32 or gates.numel() != t * 2 * w \
            or state.dtype != torch.float32 or state.shape[2] != w or w % blocks:
        raise KernelError("recurrence: projection, convolved branch, gates and state do not fit one another")
    for what, x in (("gate-branch bias", bias_y), ("convolution-branch bias", bias_x), ("recurrence-gate bias", bias_r),
                    ("input-gate bias", bias_i), ("decay parameter", lam)):
        if x.dtype != torch.float32 or x.numel() != w or not x.is_cuda or not x.is_contiguous():
            raise KernelError(f"{what} must be float32 [{w}] on the device")
    out = torch.empty((t, w), dtype=proj.dtype, device=proj.device)
    # portions of more than a few chunks run their chunks side by side (two passes); short ones in one piece
    chunk = SCAN_CHUNK if ctx.max_new_tokens > 2 * SCAN_CHUNK else max(t, 1)
    carry = torch.empty((t // chunk + ctx.num_items, w, 2), dtype=torch.float32, device=proj.device) if chunk < t else None
    check(lib().psb_recurrence_scan(proj.data_ptr(), u.data_ptr(), _code(proj, "projection output"), gates.data_ptr(),
                                    bias_y.data_ptr(), bias_x.data_ptr(), bias_r.data_ptr(), bias_i.data_ptr(), lam.data_ptr(),
                                    state.data_ptr(), _i32(ctx.item_start, "item offsets").data_ptr(),
                                    _i32(ctx.slots, "slots").data_ptr(), _ptr(carry), out.data_ptr(), ctx.num_items, t, w, k,
                                    blocks, state.shape[0], chunk, float(decay), _stream()), "recurrence_scan")
    return out


def embedding_positions(ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, pos_table: torch.Tensor,
                        scale: float) -> torch.Tensor:
    """h[t] = float32(table[ids[t]]) * scale + float32(pos_table[positions[t]])."""
    _i32(ids, "token ids"), _i32(positions, "positions"), _dev(table, "embedding table"), _dev(pos_table, "position table")
    t, (v, h) = ids.numel(), table.shape
    if pos_table.dim() != 2 or pos_table.shape[1] != h or pos_table.dtype != table.dtype or positions.numel() != t:
        raise KernelError(f"position table {tuple(pos_table.shape)} {pos_table.dtype} does not fit the embedding table {tuple(table.shape)} {table.dtype}")
    out = torch.empty((t, h), dtype=torch.float32, device=ids.device)
    check(lib().psb_embedding_pos(ids.data_ptr(), positions.data_ptr(), table.data_ptr(), pos_table.data_ptr(),
                                  _code(table, "embedding table"), out.data_ptr(), t, h, v, pos_table.shape[0], float(scale),
                                  _stream()), "embedding_pos")
    return out


def norm_add_norm(h: torch.Tensor, y: torch.Tensor, gain_post: torch.Tensor, eps_post: float,
                  gain_pre: torch.Tensor | None = None, eps_pre: float = 0.0, out_dtype: torch.dtype | None = None,
                  rows: torch.Tensor | None = None) -> torch.Tensor | None:
    """h += gain_post * rmsnorm(y) in place (h float32), and, with ``gain_pre``, returns gain_pre * rmsnorm(new h) in
    ``out_dtype``: the norm behind one sublayer and the norm in front of the next in one pass.  With ``rows`` only those
    rows are computed and returned and h is left as it was (the last use of the stream)."""
    if isinstance(y, PendingProduct):
        y = y.tensor()
    _dev(h, "residual stream"), _dev(y, "sublayer output"), _dev(gain_post, "norm gain")
    if h.dtype != torch.float32 or h.dim() != 2 or y.shape != h.shape:
        raise KernelError(f"residual stream must be float32 [T, H] and the output must match it: {h.dtype} {tuple(h.shape)} vs {tuple(y.shape)}")
    n, width = h.shape
    for g in (gain_post, gain_pre):
        if g is not None and (g.dtype != torch.float32 or g.numel() != width or not g.is_cuda):
            raise KernelError(f"norm gain must be float32 [{width}] on the device")
    if rows is not None:
        if gain_pre is None:
            raise KernelError("chosen rows need the second norm")
        _i32(rows, "row index")
        n = rows.numel()
    x = torch.empty((n, width), dtype=out_dtype or torch.float32, device=h.device) if gain_pre is not None else None
    check(lib().psb_norm_add_norm(h.data_ptr(), y.data_ptr(), _code(y, "sublayer output"), gain_post.data_ptr(), _ptr(gain_pre),
                                  _ptr(rows), _ptr(x), _code(x, "norm output") if x is not None else F32, n, width,
                                  float(eps_post), float(eps_pre), _stream()), "norm_add_norm")
    return x


BIASED_TILE_MIN_TOKENS = 16  # portions from this many tokens on go to the kernels that stage keys for a tile of tokens
BIASED_MMA = True            # ... the tensor-core one where the sizes allow (multiples of 8 up to 128), else the CUDA-core one
# The tensor-core kernel also takes single tokens and short portions: its blocks bring keys and values in with wide,
# coalesced loads of all threads, which is what a decode step is bound by (the rows of its tile that have no token idle).
BIASED_MMA_MIN_TOKENS = 1
# Steps in which every item is a single token: the kernel that walks the keys, with the runs of a (token, head) shared out
# among up to 16 blocks and a merge kernel behind them (a step of 8 tokens is 128 blocks of one warp's work each otherwise,
# every one of them a chain of a thousand keys).  BIASED_BLOCKS_WANTED blocks keep every SM busy; no share below 128 keys.
BIASED_SPLIT_DECODE = True
BIASED_BLOCKS_WANTED = 2368


def biased_attention(qkv: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                     dim: int, vdim: int, page_size: int, scale: float, window: int | None = None, chunk: int | None = None,
                     bias: torch.Tensor | None = None, sink: torch.Tensor | None = None) -> torch.Tensor:
    """The fused projection [T, hq*dim + hkv*dim + hkv*vdim] -> keys and values appended to the pages
    ([pages, 1, hkv, page_size, dim + vdim]) and causal attention with an optional window, chunk mask, distance bias
    (float32 [heads, reach]) and sink (float32 [heads]) -> [T, hq * vdim]."""
    _dev(qkv, "projection output"), _dev(kv, "cache entry"), _i32(table, "page table")
    positions, token_item = _i32(ctx.positions, "positions"), _i32(ctx.token_item, "token-to-item map")
    t = qkv.shape[0]
    want = num_heads * dim + num_kv_heads * (dim + vdim)
    if qkv.dim() != 2 or qkv.shape[1] != want:
        raise KernelError(f"projection output must be [T, {want}], is {tuple(qkv.shape)}")
    if kv.dim() != 5 or tuple(kv.shape[1:]) != (1, num_kv_heads, page_size, dim + vdim):
        raise KernelError(f"cache entry must be [pages, 1, {num_kv_heads}, {page_size}, {dim + vdim}], is {tuple(kv.shape)}")
    q = torch.empty((t, num_heads, dim), dtype=qkv.dtype, device=qkv.device)
    check(lib().psb_attention_biased_append(qkv.data_ptr(), _code(qkv, "projection output"), positions.data_ptr(),
                                            token_item.data_ptr(), table.data_ptr(), table.shape[1], kv.data_ptr(),
                                            _code(kv, "cache entry"), q.data_ptr(), t, num_heads, num_kv_heads, dim, vdim,
                                            page_size, kv.shape[0], _stream()), "attention_biased_append")
    return attention_over_rows(q, kv, table, ctx, num_heads=num_heads, num_kv_heads=num_kv_heads, dim=dim, vdim=vdim,
                               page_size=page_size, scale=scale, window=window, chunk=chunk, bias=bias, sink=sink)


def attention_over_rows(q: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                        dim: int, vdim: int, page_size: int, scale: float, window: int | None = None, chunk: int | None = None,
                        bias: torch.Tensor | None = None, sink: torch.Tensor | None = None, keep_first: int = 0) -> torch.Tensor:
    """Causal attention of queries [T, hq, dim] over a cache entry that holds one row per token and key/value head, the
    key and then the value ([pages, 1, hkv, page_size, dim + vdim]; the step's own rows already appended), with an
    optional window, chunk mask, distance bias (float32 [heads, reach]) and sink (float32 [heads]: a score per head
    that joins the softmax denominator without a value) -> [T, hq * vdim].  ``keep_first`` (with a window): the first so
    many keys of a sequence stay visible to every later query."""
    keep_first = int(keep_first or 0)
    if keep_first and (not window or chunk):
        raise KernelError("kept first keys go with a window and no chunk mask")
    _dev(q, "queries"), _dev(kv, "cache entry"), _i32(table, "page table")
    positions, token_item = _i32(ctx.positions, "positions"), _i32(ctx.token_item, "token-to-item map")
    t = q.shape[0]
    if q.dim() != 3 or tuple(q.shape[1:]) != (num_heads, dim):
        raise KernelError(f"queries must be [T, {num_heads}, {dim}], are {tuple(q.shape)}")
    if kv.dim() != 5 or tuple(kv.shape[1:]) != (1, num_kv_heads, page_size, dim + vdim):
        raise KernelError(f"cache entry must be [pages, 1, {num_kv_heads}, {page_size}, {dim + vdim}], is {tuple(kv.shape)}")
    reach = 0
    if bias is not None:
        if bias.dtype != torch.float32 or bias.dim() != 2 or bias.shape[0] != num_heads or not bias.is_cuda or not bias.is_contiguous():
            raise KernelError(f"distance bias must be float32 [{num_heads}, reach] on the device")
        reach = bias.shape[1]
    if sink is not None and (sink.dtype != torch.float32 or sink.numel() != num_heads or not sink.is_cuda):
        raise KernelError(f"sinks must be float32 [{num_heads}] on the device")
    out = torch.empty((t, num_heads * vdim), dtype=q.dtype, device=q.device)
    win, chk = int(window or 0), int(chunk or 0)
    # Portions of a bfloat16 step go tile by tile; what is left (single tokens, short portions) walks its keys.  Which
    # kernel a token gets depends on the length of its portion only (decided on the device from the item offsets, so
    # the launches have the same shape whatever the step holds).
    item_start = _i32(ctx.item_start, "item offsets")
    both16 = q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16
    if BIASED_SPLIT_DECODE and ctx.max_new_tokens == 1:
        extras = getattr(ctx, "extras", None) or {}
        keys = int(extras.get("static_kv_len") or ctx.max_kv_len)  # a captured step is sized for its class of lengths
        if win:
            keys = min(keys, win + keep_first)
        if chk:
            keys = min(keys, chk)
        splits = max(1, min(16, -(-BIASED_BLOCKS_WANTED // max(t * num_heads, 1)), keys // 128))
        partial = torch.empty((t, num_heads, splits, vdim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
        check(lib().psb_attention_biased(q.data_ptr(), _code(q, "queries"), kv.data_ptr(), _code(kv, "cache entry"),
                                         table.data_ptr(), table.shape[1], positions.data_ptr(), token_item.data_ptr(),
                                         _ptr(bias), _ptr(sink), out.data_ptr(), t, num_heads, num_kv_heads, dim, vdim,
                                         page_size, win, chk, reach, float(scale), item_start.data_ptr(), 0, keep_first,
                                         _ptr(partial), splits, _stream()), "attention_biased")
        return out
    on_tensor_cores = both16 and BIASED_MMA and bool(lib().psb_attention_biased_mma_supported(num_heads, num_kv_heads, dim, vdim))
    least = BIASED_MMA_MIN_TOKENS if on_tensor_cores else BIASED_TILE_MIN_TOKENS
    long_portions = both16 and ctx.max_new_tokens >= least
    tiled = long_portions and (on_tensor_cores or bool(lib().psb_attention_biased_tile_supported(num_heads, num_kv_heads, dim, vdim)))
    if not (tiled and (ctx.num_items == 1 or least <= 1)):  # nothing for the walking kernel when every portion is tiled
        check(lib().psb_attention_biased(q.data_ptr(), _code(q, "queries"), kv.data_ptr(), _code(kv, "cache entry"),
                                         table.data_ptr(), table.shape[1], positions.data_ptr(), token_item.data_ptr(),
                                         _ptr(bias), _ptr(sink), out.data_ptr(), t, num_heads, num_kv_heads, dim, vdim,
                                         page_size, win, chk, reach, float(scale), item_start.data_ptr(),
                                         least if tiled else 0, keep_first, None, 1, _stream()), "attention_biased")
    if tiled:
        entry = lib().psb_attention_biased_mma if on_tensor_cores else lib().psb_attention_biased_tiles
        check(entry(q.data_ptr(), kv.data_ptr(), table.data_ptr(), table.shape[1], positions.data_ptr(), item_start.data_ptr(),
                    ctx.num_items, t, least, _ptr(bias), _ptr(sink), out.data_ptr(), num_heads, num_kv_heads, dim,
                    vdim, page_size, win, chk, reach, float(scale), keep_first, _stream()),
              "attention_biased_mma" if on_tensor_cores else "attention_biased_tiles")
    return out


DELTA_LONG_PORTION = 32  # steps whose longest portion has this many tokens take DELTA_LONG_LANES lanes a column of the state, else 4
DELTA_LONG_LANES = 16   # measured: 32 lanes (a column a warp) took 807 us for a 2,048-token portion with 16 heads of 128 x 128, 16 lanes 716


def delta_rule(proj: torch.Tensor, ba: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               gain: torch.Tensor, state: torch.Tensor, ctx, *, groups: int, heads: int, dim: int, vdim: int, eps: float) -> torch.Tensor:
    """The gated delta rule over every portion of the step.  proj [T, 2*groups*dim + 2*heads*vdim] (queries, keys,
    values, output gate; compute type), ba float32 [T, 2*heads] (write strength, decay pre-activations), taps float32
    [2*groups*dim + heads*vdim, K], state float32 [num_slots, (K-1)*channels + heads*dim*vdim].  Returns the normed,
    gated read-out [T, heads*vdim] in the compute type."""
    _dev(proj, "projection output"), _dev(ba, "gate pre-activations"), _dev(state, "recurrent state")
    t = proj.shape[0]
    c = 2 * groups * dim + heads * vdim
    k = taps.shape[1]
    slot_floats = (k - 1) * c + heads * dim * vdim
    if proj.dim() != 2 or proj.shape[1] != c + heads * vdim or ba.dtype != torch.float32 or tuple(ba.shape) != (t, 2 * heads):
        raise KernelError(f"delta rule: projection {tuple(proj.shape)} / gates {ba.dtype} {tuple(ba.shape)} do not fit the sizes")
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != slot_floats:
        raise KernelError(f"delta rule: state must be float32 [slots, {slot_floats}], is {state.dtype} {tuple(state.shape)}")
    for what, x, n in (("taps", taps, c * k), ("decay rates", a_log, heads), ("decay bias", dt_bias, heads), ("read-out gain", gain, vdim)):
        if x.dtype != torch.float32 or x.numel() != n or not x.is_cuda or not x.is_contiguous():
            raise KernelError(f"delta rule: {what} must be float32 with {n} numbers on the device")
    dev = proj.device
    qkv = torch.empty((t, c), dtype=torch.float32, device=dev)
    bd = torch.empty((t, 5 * heads), dtype=torch.float32, device=dev)   # beta, decay and three state-free dot products per head
    positions, token_item = _i32(ctx.positions, "positions"), _i32(ctx.token_item, "token-to-item map")
    item_start, slots = _i32(ctx.item_start, "item offsets"), _i32(ctx.slots, "slots")
    check(lib().psb_delta_prepare(proj.data_ptr(), _code(proj, "projection output"), ba.data_ptr(), taps.data_ptr(), a_log.data_ptr(),
                                  dt_bias.data_ptr(), state.data_ptr(), positions.data_ptr(), token_item.data_ptr(),
                                  item_start.data_ptr(), slots.data_ptr(), qkv.data_ptr(), bd.data_ptr(), t, groups, heads, dim, vdim,
                                  k, state.shape[0], slot_floats, _stream()), "delta_prepare")
    o = torch.empty((t, heads, vdim), dtype=torch.float32, device=dev)
    lanes = DELTA_LONG_LANES if ctx.max_new_tokens >= DELTA_LONG_PORTION and dim >= DELTA_LONG_LANES else 4
    check(lib().psb_delta_rule(qkv.data_ptr(), bd.data_ptr(), proj.data_ptr(), _code(proj, "projection output"), state.data_ptr(),
                               item_start.data_ptr(), slots.data_ptr(), o.data_ptr(), ctx.num_items, groups, heads, dim, vdim, k,
                               state.shape[0], slot_floats, lanes, _stream()), "delta_rule")
    out = torch.empty((t, heads * vdim), dtype=proj.dtype, device=dev)
    check(lib().psb_delta_finish(o.data_ptr(), proj.data_ptr(), _code(proj, "projection output"), gain.data_ptr(), out.data_ptr(), t,
                                 groups, heads, dim, vdim, float(eps), _stream()), "delta_finish")
    return out


def moe_route(z: torch.Tensor, correction: torch.Tensor | None, *, experts: int, top: int, groups: int, keep: int,
              scale: float, scores: str = "sigmoid", group_score: str = "top2", normalize: bool = True):
    """Router logits float32 [T, >= experts] (further columns are ignored) -> (chosen int32 [T, top], weights float32
    [T, top]): scores (``scores``: "sigmoid", or "softmax" over all experts), choice by score + correction among the
    experts of the ``keep`` best of ``groups`` groups (``group_score``: a group counts by the sum of its two largest
    choice scores, "top2", or by its largest, "max"), weights = chosen scores / their sum * scale, or with
    ``normalize`` False the chosen scores * scale as they are."""
    if scores not in ("sigmoid", "softmax") or group_score not in ("top2", "max"):
        raise KernelError(f"router: scores {scores!r} (sigmoid, softmax) / group score {group_score!r} (top2, max) not built")
    _dev(z, "router logits")
    if z.dtype != torch.float32 or z.dim() != 2 or z.shape[1] < experts:
        raise KernelError(f"router logits must be float32 [T, >= {experts}], are {z.dtype} {tuple(z.shape)}")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != experts or not correction.is_cuda):
        raise KernelError(f"router correction must be float32 [{experts}] on the device")
    t = z.shape[0]
    chosen = torch.empty((t, top), dtype=torch.int32, device=z.device)
    weight = torch.empty((t, top), dtype=torch.float32, device=z.device)
    check(lib().psb_moe_route(z.data_ptr(), z.shape[1], _ptr(correction), chosen.data_ptr(), weight.data_ptr(), t, experts, top,
                              groups, keep, float(scale), 1 if scores == "softmax" else 0, 1 if group_score == "max" else 0,
                              1 if normalize else 0, _stream()), "moe_route")
    return chosen, weight


MOE_ACTIVATIONS = {None: 0, "relu2": 1}
MOE_TCGEN05 = True            # bfloat16 experts on the grouped tcgen05 product
MOE_TCGEN05_MIN_PAIRS = 256   # with fewer (token, expert) pairs in a step the 64-row tiles of the mma.sync kernel waste less


def moe_experts(x: torch.Tensor, chosen: torch.Tensor, weight: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, *,
                activation: str | None = "relu2", shared: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None, glu: tuple[float, float, float] | None = None) -> torch.Tensor:
    """sum over a token's chosen experts of weight * down_e(act(up_e x)) (+ sigmoid(shared_gate) * shared), for
    w_up [E, ff, H], w_down [E, H, ff].  ``shared_gate``: float32 column view [T, 1] (its row stride may be wider);
    without it the shared expert's output is added as it is.

    ``glu`` = (limit, alpha, offset): gated experts.  w_up is then [E, 2 ff, H], an expert's gate rows followed by its
    up rows, ``activation`` is None, and between the two products g * sigmoid(alpha g) * (u + offset) is taken with
    g = min(gate, limit), u = clamp(up, -limit, limit)."""
    _dev(x, "expert input"), _dev(w_up, "expert up matrices"), _dev(w_down, "expert down matrices")
    _i32(chosen, "chosen experts"), _dev(weight, "expert weights")
    t, h = x.shape
    e, ff, _ = w_up.shape
    top = chosen.shape[1]
    ff_in = ff  # columns of the first product
    if glu is not None:
        if activation is not None or ff % 2:
            raise KernelError("gated experts: the gate is the activation, and the first matrices hold gate rows and up rows")
        ff = ff // 2
    if tuple(w_up.shape) != (e, ff_in, h) or tuple(w_down.shape) != (e, h, ff) or tuple(weight.shape) != (t, top) or weight.dtype != torch.float32:
        raise KernelError(f"experts: up {tuple(w_up.shape)}, down {tuple(w_down.shape)}, weights {tuple(weight.shape)} do not fit {t} tokens of {h}")
    if activation not in MOE_ACTIVATIONS:
        raise KernelError(f"experts: activation {activation!r} is not built (one of {sorted(k for k in MOE_ACTIVATIONS if k)})")
    dev, pairs = x.device, t * top
    # bfloat16 with rows the tensor map takes: the experts' rows start at multiples of 128 and both products run on the
    # tcgen05 kernel, every 128-row tile against its own expert's matrix; otherwise tiles of 64 rows on mma.sync or FFMA
    grouped = (MOE_TCGEN05 and x.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
               and h % 8 == 0 and ff % 8 == 0 and pairs >= MOE_TCGEN05_MIN_PAIRS)
    pad = 128 if grouped else 1
    room = -(-(pairs + e * (pad - 1)) // pad) * pad
    offsets = torch.empty((e + 1,), dtype=torch.int32, device=dev)
    row_pair = torch.empty((max(room, 1),), dtype=torch.int32, device=dev)
    pair_row = torch.empty((max(pairs, 1),), dtype=torch.int32, device=dev)
    tile_expert = torch.empty((room // pad,), dtype=torch.int32, device=dev) if grouped else None
    check(lib().psb_moe_group(chosen.data_ptr(), offsets.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(), _ptr(tile_expert),
                              pairs, e, pad, room, _stream()), "moe_group")
    if grouped:
        from .tensorcore import _sms
        sms = _sms(dev)
        rows = torch.empty((room, h), dtype=torch.bfloat16, device=dev)
        check(lib().psb_moe_gather(x.data_ptr(), row_pair.data_ptr(), rows.data_ptr(), room, h, top, _stream()), "moe_gather")
        if glu is not None:  # both branches and the gate in one product's epilogue
            mid = torch.empty((room, ff), dtype=torch.bfloat16, device=dev)
            check(lib().psb_gemm_tcgen05_grouped_gated_clipped(rows.data_ptr(), w_up.data_ptr(), mid.data_ptr(), room, ff, h, e,
                                                               tile_expert.data_ptr(), float(glu[0]), float(glu[1]), float(glu[2]),
                                                               sms, _stream()), "gemm_tcgen05_grouped_gated_clipped")
        else:
            mid = torch.empty((room, ff_in), dtype=torch.bfloat16, device=dev)
            check(lib().psb_gemm_tcgen05_grouped(rows.data_ptr(), w_up.data_ptr(), mid.data_ptr(), room, ff_in, h, e, tile_expert.data_ptr(),
                                                 MOE_ACTIVATIONS[activation], sms, _stream()), "gemm_tcgen05_grouped")
        y = torch.empty((room, h), dtype=torch.bfloat16, device=dev)
        check(lib().psb_gemm_tcgen05_grouped(mid.data_ptr(), w_down.data_ptr(), y.data_ptr(), room, h, ff, e, tile_expert.data_ptr(),
                                             0, sms, _stream()), "gemm_tcgen05_grouped")
    else:
        mid = torch.empty((room, ff_in), dtype=x.dtype, device=dev)
        check(lib().psb_moe_gemm(x.data_ptr(), _code(x, "expert input"), w_up.data_ptr(), _code(w_up, "expert up matrices"), mid.data_ptr(),
                                 _code(mid, "expert activations"), offsets.data_ptr(), row_pair.data_ptr(), room, e, ff_in, h, top, 1,
                                 MOE_ACTIVATIONS[activation], 0, 0.0, 0.0, 0.0, _stream()), "moe_gemm")
        # gated experts: the second product takes the clipped gate of a row's two halves as it reads the row
        lim, alpha, off = (float(v) for v in glu) if glu is not None else (0.0, 0.0, 0.0)
        y = torch.empty((room, h), dtype=torch.float32, device=dev)
        check(lib().psb_moe_gemm(mid.data_ptr(), _code(mid, "expert activations"), w_down.data_ptr(), _code(w_down, "expert down matrices"),
                                 y.data_ptr(), F32, offsets.data_ptr(), row_pair.data_ptr(), room, e, h, ff, top, 0, 0,
                                 1 if glu is not None else 0, lim, alpha, off, _stream()), "moe_gemm")
    out = torch.empty((t, h), dtype=out_dtype or x.dtype, device=dev)
    ldg = 0
    if shared is not None:
        _dev(shared, "shared expert output")
        if shared.shape != x.shape:
            raise KernelError("experts: the shared expert's output must match the input")
        if shared_gate is not None:
            if shared_gate.dtype != torch.float32 or shared_gate.shape[0] != t or not shared_gate.is_cuda:
                raise KernelError("experts: the shared expert's gate must be a float32 column on the device")
            ldg = shared_gate.stride(0)
    check(lib().psb_moe_combine(y.data_ptr(), _code(y, "experts' outputs"), pair_row.data_ptr(), weight.data_ptr(), _ptr(shared),
                                _code(shared, "shared expert output") if shared is not None else F32,
                                _ptr(shared_gate) if shared is not None else None, ldg, out.data_ptr(), _code(out, "experts' sum"),
                                t, h, top, _stream()), "moe_combine")
    return out


def _f32_vector(x: torch.Tensor, n: int, what: str) -> torch.Tensor:
    if x.dtype != torch.float32 or x.numel() != n or not x.is_cuda or not x.is_contiguous():
        raise KernelError(f"{what} must be float32 with {n} numbers on the device, is {x.dtype} {tuple(x.shape)} on {x.device}")
    return x


def _slot_rows(state: torch.Tensor, width: int, what: str) -> int:
    """A per-slot float32 state [num_slots, >= width] whose rows may be part of wider ones; returns the row stride."""
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != width or not state.is_cuda or state.stride(1) != 1:
        raise KernelError(f"{what} must be float32 [slots, {width}] on the device with unit stride along a row, is "
                          f"{state.dtype} {tuple(state.shape)} strides {state.stride()}")
    return int(state.stride(0))


FUSE_NORM_SHIFT = True  # steps of single tokens: the residual sum, the norm in front and the shift in one kernel


def token_shift(x, mix: torch.Tensor, state: torch.Tensor, ctx) -> torch.Tensor:
    """y_t = x_t + (x_(t-1) - x_t) * mix per channel, with x_(t-1) the row before (zero in front of a sequence's first
    token); the row before a portion's first token comes from ``state`` [num_slots, W] (float32; rows may be strided),
    which receives the portion's last row.  ``x`` may be an ``ops.NormedRows`` that nobody has computed yet: in a step
    of single tokens the residual sum and the norm then run in the same kernel as the shift."""
    t, w = x.shape
    stride = _slot_rows(state, w, "token-shift state")
    _f32_vector(mix, w, "token-shift weights")
    if isinstance(x, NormedRows):
        if (FUSE_NORM_SHIFT and ctx.max_new_tokens == 1 and x._x is None and not x._settled and x.rows is None and w % 8 == 0
                and stride % 4 == 0 and state.data_ptr() % 16 == 0):
            pending = x.pending.tensor() if isinstance(x.pending, PendingProduct) else x.pending
            if pending is None or (pending.is_contiguous() and pending.shape == x.h.shape and pending.data_ptr() % 16 == 0):
                _dev(x.h, "residual stream")
                y = torch.empty((t, w), dtype=x.dtype, device=x.h.device)
                check(lib().psb_add_rmsnorm_shift(x.h.data_ptr(), _ptr(pending), _code(pending, "sublayer output") if pending is not None else F32,
                                                  x.gain.data_ptr(), x.eps, mix.data_ptr(), state.data_ptr(), stride,
                                                  _i32(ctx.positions, "positions").data_ptr(), _i32(ctx.token_item, "token-to-item map").data_ptr(),
                                                  _i32(ctx.slots, "slots").data_ptr(), y.data_ptr(), _code(y, "shifted rows"), t, w,
                                                  state.shape[0], _stream()), "add_rmsnorm_shift")
                x.fused(None)
                return y
        x = x.tensor()
    _dev(x, "shifted rows")
    y = torch.empty_like(x)
    check(lib().psb_token_shift(x.data_ptr(), _code(x, "shifted rows"), mix.data_ptr(), state.data_ptr(), stride,
                                _i32(ctx.positions, "positions").data_ptr(), _i32(ctx.token_item, "token-to-item map").data_ptr(),
                                _i32(ctx.item_start, "item offsets").data_ptr(), _i32(ctx.slots, "slots").data_ptr(), y.data_ptr(),
                                t, w, state.shape[0], _stream()), "token_shift")
    return y


def normed_pair_sum(a: torch.Tensor, b: torch.Tensor, gain_a: torch.Tensor, gain_b: torch.Tensor, eps: float,
                    weight: float = 1.0) -> torch.Tensor:
    """(gain_a * rmsnorm(a) + gain_b * rmsnorm(b)) * weight, row by row, as float32 [T, W]."""
    _dev(a, "left result"), _dev(b, "right result")
    if isinstance(a, PendingProduct) or a.dim() != 2 or a.shape != b.shape or a.dtype != b.dtype:
        raise KernelError(f"the two results must have one shape and type: {a.dtype} {tuple(a.shape)} vs {b.dtype} {tuple(b.shape)}")
    t, w = a.shape
    _f32_vector(gain_a, w, "left gain"), _f32_vector(gain_b, w, "right gain")
    out = torch.empty((t, w), dtype=torch.float32, device=a.device)
    check(lib().psb_normed_pair_sum(a.data_ptr(), b.data_ptr(), _code(a, "left result"), gain_a.data_ptr(), gain_b.data_ptr(),
                                    out.data_ptr(), t, w, float(eps), float(weight), _stream()), "normed_pair_sum")
    return out


def attention_prepare(proj: torch.Tensor, kv: torch.Tensor, table: torch.Tensor, ctx, *, num_heads: int, num_kv_heads: int,
                      dim: int, vdim: int, page_size: int, cos: torch.Tensor | None = None, sin: torch.Tensor | None = None,
                      rotary_dim: int | None = None, interleaved: bool = False, unit_norm_eps: float | None = None,
                      head_factor: torch.Tensor | None = None, values_are_keys: bool = False,
                      split_planes: bool = False, bias: torch.Tensor | None = None, write_kv: bool = True) -> torch.Tensor:
    """One pass over the fused projection [T, q | k | v] (or [T, q | k] with ``values_are_keys``): optional rotation of
    the first ``rotary_dim`` elements of query and key heads by position (``cos``/``sin`` float32 [positions,
    rotary_dim/2]), optional division of every query and key head by its root mean square (``unit_norm_eps``), an
    optional float32 factor per query head; keys and values appended to the cache entry [pages, 1, hkv, page_size,
    dim + vdim], or with ``split_planes`` (vdim == dim) [pages, 2, hkv, page_size, dim]: keys in plane 0, values in
    plane 1.  Returns the queries [T, hq, dim].

    ``bias`` (float32, one number per column of the projection): added to the projection in float32 before anything
    else.  ``write_kv`` False: the projection holds queries only and nothing is appended (a layer that reads the keys
    and values another layer has stored); ``kv`` and ``table`` may then be None."""
    t = proj.shape[0]
    want = num_heads * dim + (num_kv_heads * dim + (0 if values_are_keys else num_kv_heads * vdim) if write_kv else 0)
    if bias is not None:
        _f32_vector(bias, want, "projection bias")
    if not write_kv:
        if not proj.is_cuda or proj.dim() != 2 or proj.shape[1] != want or proj.stride(1) != 1:
            raise KernelError(f"query projection must be [T, {want}] on the device, is {tuple(proj.shape)}")
        max_pos = 0
        rotary_dim = dim if rotary_dim is None else int(rotary_dim)
        if cos is not None:
            if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2 \
                    or rotary_dim % 2 or not 2 <= rotary_dim <= dim:
                raise KernelError(f"angle tables must be float32 [positions, {rotary_dim // 2}] for {rotary_dim} rotated elements of {dim}")
            _dev(cos, "cosines"), _dev(sin, "sines")
            max_pos = cos.shape[0]
            if ctx.max_kv_len > max_pos:
                raise KernelError(f"a position of this step ({ctx.max_kv_len - 1}) lies beyond the angle tables ({max_pos} positions)")
        if head_factor is not None:
            _f32_vector(head_factor, num_heads, "per-head factors")
        q = torch.empty((t, num_heads, dim), dtype=proj.dtype, device=proj.device)
        check(lib().psb_attention_prepare(proj.data_ptr(), int(proj.stride(0)), _code(proj, "projection output"), _i32(ctx.positions, "positions").data_ptr(),
                                          _i32(ctx.token_item, "token-to-item map").data_ptr(), None, 0, _ptr(cos), _ptr(sin),
                                          _ptr(head_factor), None, _code(proj, "projection output"), q.data_ptr(), t, num_heads, num_kv_heads, dim, vdim,
                                          1, 0, max_pos, rotary_dim, 1 if interleaved else 0,
                                          -1.0 if unit_norm_eps is None else float(unit_norm_eps), 0, 0, _ptr(bias), 0, _stream()),
              "attention_prepare")
        return q
    _dev(kv, "cache entry"), _i32(table, "page table")
    if not proj.is_cuda or proj.dim() != 2 or proj.shape[1] != want or proj.stride(1) != 1:
        raise KernelError(f"projection output must be [T, {want}] on the device (rows may be part of wider ones), is {tuple(proj.shape)}")
    entry = (2, num_kv_heads, page_size, dim) if split_planes else (1, num_kv_heads, page_size, dim + vdim)
    if kv.dim() != 5 or tuple(kv.shape[1:]) != entry or not kv.is_contiguous():
        raise KernelError(f"cache entry must be [pages, {', '.join(map(str, entry))}], is {tuple(kv.shape)}")
    if split_planes and vdim != dim:
        raise KernelError(f"keys and values in planes of their own need vdim == dim, not {vdim} and {dim}")
    if values_are_keys and vdim != dim:
        raise KernelError(f"keys that serve as values need vdim == dim, not {vdim} and {dim}")
    max_pos = 0
    rotary_dim = dim if rotary_dim is None else int(rotary_dim)
    if cos is not None:
        if sin is None or cos.shape != sin.shape or cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] != rotary_dim // 2 \
                or rotary_dim % 2 or not 2 <= rotary_dim <= dim:
            raise KernelError(f"angle tables must be float32 [positions, {rotary_dim // 2}] for {rotary_dim} rotated elements of {dim}")
        _dev(cos, "cosines"), _dev(sin, "sines")
        max_pos = cos.shape[0]
        if ctx.max_kv_len > max_pos:
            raise KernelError(f"a position of this step ({ctx.max_kv_len - 1}) lies beyond the angle tables ({max_pos} positions)")
    if head_factor is not None:
        _f32_vector(head_factor, num_heads, "per-head factors")
    q = torch.empty((t, num_heads, dim), dtype=proj.dtype, device=proj.device)
    check(lib().psb_attention_prepare(proj.data_ptr(), int(proj.stride(0)), _code(proj, "projection output"), _i32(ctx.positions, "positions").data_ptr(),
                                      _i32(ctx.token_item, "token-to-item map").data_ptr(), table.data_ptr(), table.shape[1],
                                      _ptr(cos), _ptr(sin), _ptr(head_factor), kv.data_ptr(), _code(kv, "cache entry"), q.data_ptr(),
                                      t, num_heads, num_kv_heads, dim, vdim, page_size, kv.shape[0], max_pos, rotary_dim,
                                      1 if interleaved else 0, -1.0 if unit_norm_eps is None else float(unit_norm_eps),
                                      1 if values_are_keys else 0, 1 if split_planes else 0, _ptr(bias), 1, _stream()), "attention_prepare")
    return q


# Portions of more than four times this many tokens run as chunks side by side.  32: a 2,048-token portion at width 2,048
# gives 2,112 blocks of two warps, 28 warps an SM; with chunks of 64 an SM held 14 and the two passes took 24 + 35 us.
MIN_GRU_CHUNK = 32


def min_gru(proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor, ctx, *, width: int) -> torch.Tensor:
    """The minGRU recurrence over every portion of the step.  proj [T, >= 3W]: update-gate, candidate and output-gate
    pre-activations in its first 3W columns (the tensor may be a column slice of a wider one); biases float32 [W];
    state float32 [num_slots, W] (rows may be strided), read and brought up to date.  Returns S_t * silu(g_t) [T, W]."""
    if not proj.is_cuda or proj.dim() != 2 or proj.shape[1] < 3 * width or proj.stride(1) != 1:
        raise KernelError(f"minGRU: projection must be [T, >= {3 * width}] on the device with unit column stride, is {tuple(proj.shape)}")
    t = proj.shape[0]
    stride = _slot_rows(state, width, "minGRU state")
    _f32_vector(bias_z, width, "update-gate bias"), _f32_vector(bias_x, width, "candidate bias")
    out = torch.empty((t, width), dtype=proj.dtype, device=proj.device)
    two_pass = ctx.max_new_tokens > 4 * MIN_GRU_CHUNK
    chunk = MIN_GRU_CHUNK if two_pass else max(t, 1)
    carry = start = None
    if two_pass:
        carry = torch.empty((t // chunk + ctx.num_items, width, 2), dtype=torch.float32, device=proj.device)
        start = torch.empty((ctx.num_items, width), dtype=torch.float32, device=proj.device)
    check(lib().psb_min_gru(proj.data_ptr(), int(proj.stride(0)), _code(proj, "projection output"), bias_z.data_ptr(),
                            bias_x.data_ptr(), state.data_ptr(), stride, _i32(ctx.item_start, "item offsets").data_ptr(),
                            _i32(ctx.slots, "slots").data_ptr(), _ptr(carry), _ptr(start), out.data_ptr(), ctx.num_items, t, width,
                            state.shape[0], chunk, 1 if two_pass else 0, _stream()), "min_gru")
    return out


CLIPPED_FUSED_MIN_ROWS = 65  # from here on no product folds the norm in front of it into itself, so nothing is lost by asking for the rows


def clipped_gated_linear(x, w_gate_up: torch.Tensor, limit: float, alpha: float = 1.702, offset: float = 1.0) -> torch.Tensor:
    """g * sigmoid(alpha g) * (u + offset) with g = min(x Wg^T, limit), u = clamp(x Wu^T, -limit, limit) for W = [gate rows;
    up rows].  bfloat16: a few rows in the streaming product's epilogue (with the norm in front, if ``x`` still carries
    it), many in the tcgen05 product's; between the two, and in float32, product (which may fold the norm in front
    into itself) and then the activation.  Every way rounds the two products to the compute type before they are clipped."""
    both16 = x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    if both16 and isinstance(x, NormedRows) and x.fusable:   # few rows: the norm in front, both products and the gate in one kernel
        from .tensorcore import norm_gated_linear_bf16
        act = norm_gated_linear_bf16(x, w_gate_up, clip=(limit, alpha, offset))
        if act is not None:
            return act
    if both16 and (x.shape[0] >= CLIPPED_FUSED_MIN_ROWS or not isinstance(x, NormedRows)):
        from .tensorcore import clipped_gated_linear_bf16
        rows = x.tensor() if isinstance(x, NormedRows) else x
        _dev(rows, "left operand"), _dev(w_gate_up, "weight")
        act = clipped_gated_linear_bf16(rows, w_gate_up, limit, alpha, offset)
        if act is not None:
            return act
        x = rows
    return clipped_glu(linear(x, w_gate_up), limit, alpha, offset)


def clipped_glu(gate_up: torch.Tensor, limit: float, alpha: float = 1.702, offset: float = 1.0) -> torch.Tensor:
    """[T, 2I] -> g * sigmoid(alpha * g) * (u + offset) with g = min(first half, limit), u = clamp(second half, +-limit)."""
    _dev(gate_up, "gate/up projection")
    t, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"gate/up projection must have an even width, has {two_i}")
    out = torch.empty((t, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(lib().psb_clipped_glu(gate_up.data_ptr(), _code(gate_up, "gate/up projection"), out.data_ptr(), t, two_i // 2,
                                float(limit), float(alpha), float(offset), _stream()), "clipped_glu")
    return out
