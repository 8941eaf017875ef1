"""The kernels as Python functions on torch tensors.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, sizes that index arithmetic relies on), passes raw pointers and the
current stream to the launcher and raises KernelError when the launcher refuses
or the launch fails.  Nothing here computes with torch: if the extension cannot
be built or loaded, every call fails.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

import torch

from ..errors import KernelError
from . import build

PAGE_SIZE = 64  # tokens per cache page; the attention kernels' key tile

_F32, _BF16 = 0, 1
_DT = {torch.float32: _F32, torch.bfloat16: _BF16}

c_int, c_ll, c_float, c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is neither float32 nor bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(t: torch.Tensor, what: str, dtype=None, contiguous=True) -> torch.Tensor:
    _need(isinstance(t, torch.Tensor), f"{what}: not a tensor")
    _need(t.is_cuda, f"{what}: tensor is on {t.device}, the kernels run on CUDA only")
    if dtype is not None:
        _need(t.dtype == dtype, f"{what}: dtype {t.dtype}, expected {dtype}")
    if contiguous:
        _need(t.is_contiguous(), f"{what}: tensor is not contiguous")
    return t


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    _need(t.dim() == 2 and t.stride(1) == 1, f"{what}: expected a 2-D tensor with dense rows")
    return t.stride(0)


def _p(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far in this process (replayed graph nodes included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(lib, rc: int, name: str, kernels: int = 1) -> None:
    global _launches
    _launches += kernels
    if rc != 0:
        text = lib.rl_error_text().decode("utf-8", "replace")
        kind = "refused its arguments" if rc < 0 else f"failed to launch (CUDA error {rc})"
        raise KernelError(f"{name} {kind}: {text}")


# ------------------------------------------------------------------ row kernels
def embed_gather(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale as float32.  Token ids must already be known to lie in the table."""
    _cuda(tokens, "embed_gather tokens", torch.int32)
    _cuda(table, "embed_gather table")
    _need(tokens.dim() == 1 and table.dim() == 2, "embed_gather: tokens[T] and table[V, d] expected")
    T, d = tokens.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, d), dtype=torch.float32, device=table.device)
    _cuda(out, "embed_gather out", torch.float32)
    _need(tuple(out.shape) == (T, d), "embed_gather: out has the wrong shape")
    _need(table.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0, "embed_gather: tensors must be 16-byte aligned")
    lib = build.load("elementwise")
    rc = lib.rl_embed_gather(_p(tokens), _p(table), c_int(_dt(table, "embed_gather table")), _p(out), c_int(T), c_int(d), c_float(scale), _stream())
    _check(lib, rc, "embed_gather")
    return out


def add_rmsnorm(
    x: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: Optional[torch.Tensor],
    eps: float,
    act_dtype: torch.dtype,
    rows: Optional[torch.Tensor] = None,
    write_x: bool = True,
    out: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """x (float32 [T, d]) += sum of delta parts; returns rmsnorm(x) * weight in `act_dtype`.

    delta: None, [T, d] or [parts, T, d], in `act_dtype` or in float32 (partial sums of a product
    split over k).  weight None: only the sum.
    rows: int32 indices of the rows to produce (all rows if None).
    """
    _cuda(x, "add_rmsnorm x", torch.float32)
    _need(x.dim() == 2, "add_rmsnorm: x must be [T, d]")
    T, d = x.shape
    n_parts, part_stride = 0, 0
    delta_dt = _DT[act_dtype]
    if delta is not None:
        _cuda(delta, "add_rmsnorm delta")
        _need(delta.dtype in (act_dtype, torch.float32), f"add_rmsnorm: delta is {delta.dtype} in a run of {act_dtype}")
        delta_dt = _DT[delta.dtype]
        if delta.dim() == 2:
            _need(tuple(delta.shape) == (T, d), f"add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
            n_parts = 1
        else:
            _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (T, d), f"add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
            n_parts, part_stride = delta.shape[0], T * d
    n_rows = T
    if rows is not None:
        _cuda(rows, "add_rmsnorm rows", torch.int32)
        n_rows = rows.numel()
    w_dt = _F32
    if weight is not None:
        _cuda(weight, "add_rmsnorm weight")
        _need(tuple(weight.shape) == (d,), f"add_rmsnorm: weight {tuple(weight.shape)} does not match d={d}")
        w_dt = _dt(weight, "add_rmsnorm weight")
        if out is None:
            out = torch.empty((n_rows, d), dtype=act_dtype, device=x.device)
        _cuda(out, "add_rmsnorm out", act_dtype)
        _need(tuple(out.shape) == (n_rows, d), "add_rmsnorm: out has the wrong shape")
    else:
        _need(delta is not None, "add_rmsnorm: neither a delta nor a weight, nothing to do")
        out = None
    if n_rows == 0:
        return out
    for name, t in (("x", x), ("delta", delta), ("weight", weight), ("out", out)):
        _need(t is None or t.data_ptr() % 16 == 0, f"add_rmsnorm: {name} is not 16-byte aligned")
    lib = build.load("elementwise")
    rc = lib.rl_add_rmsnorm(
        _p(x), _p(delta), c_int(delta_dt), c_int(n_parts), c_ll(part_stride), _p(weight), c_int(w_dt), _p(out),
        c_int(_DT[act_dtype]), _p(rows), c_int(n_rows), c_int(d), c_float(eps), c_int(1 if write_x else 0), _stream(),
    )
    _check(lib, rc, "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h[t, i] = silu(gate_up[t, i]) * gate_up[t, ff + i]."""
    _cuda(gate_up, "swiglu input")
    _need(gate_up.dim() == 2 and gate_up.shape[1] % 2 == 0, "swiglu: input must be [T, 2*ff]")
    T, ff = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((T, ff), dtype=gate_up.dtype, device=gate_up.device)
    _cuda(out, "swiglu out", gate_up.dtype)
    _need(tuple(out.shape) == (T, ff), "swiglu: out has the wrong shape")
    lib = build.load("elementwise")
    rc = lib.rl_swiglu(_p(gate_up), _p(out), c_int(_dt(gate_up, "swiglu")), c_int(T), c_int(ff), _stream())
    _check(lib, rc, "swiglu")
    return out


# ------------------------------------------------------------------ per-sequence records
SEQ_FIELDS = 4  # a record: positions held, tokens decoded, the most it may decode, flags
SEQ_LEN, SEQ_DECODED, SEQ_MAX_NEW, SEQ_FLAGS = 0, 1, 2, 3


def seq_begin_decode(state: torch.Tensor, slot_ids: torch.Tensor, tok_pos: torch.Tensor, seq_pos0: torch.Tensor, seq_len: torch.Tensor) -> None:
    """A decode step's positions from the records on the device (int32 [slots, 4]): row i of the batch, which belongs
    to slot slot_ids[i], stands at position record.len; the record moves on by one position and one decoded token."""
    _cuda(state, "seq_begin_decode state", torch.int32)
    _need(state.dim() == 2 and state.shape[1] == SEQ_FIELDS, f"seq_begin_decode: records must be [slots, {SEQ_FIELDS}]")
    S = slot_ids.numel()
    for name, t in (("slot_ids", slot_ids), ("tok_pos", tok_pos), ("seq_pos0", seq_pos0), ("seq_len", seq_len)):
        _cuda(t, f"seq_begin_decode {name}", torch.int32)
        _need(t.numel() == S, f"seq_begin_decode: {name} has {t.numel()} entries for {S} sequences")
    lib = build.load("elementwise")
    rc = lib.rl_seq_begin_decode(_p(state), _p(slot_ids), c_int(S), _p(tok_pos), _p(seq_pos0), _p(seq_len), _stream())
    _check(lib, rc, "seq_begin_decode")


def seq_set_len(state: torch.Tensor, slot_ids: torch.Tensor, seq_len: torch.Tensor) -> None:
    """record.len = seq_len[i] for the sequences of a step whose positions the host gave."""
    _cuda(state, "seq_set_len state", torch.int32)
    _need(state.dim() == 2 and state.shape[1] == SEQ_FIELDS, f"seq_set_len: records must be [slots, {SEQ_FIELDS}]")
    _cuda(slot_ids, "seq_set_len slot_ids", torch.int32)
    _cuda(seq_len, "seq_set_len seq_len", torch.int32)
    _need(slot_ids.numel() == seq_len.numel(), "seq_set_len: one length per sequence")
    lib = build.load("elementwise")
    rc = lib.rl_seq_set_len(_p(state), _p(slot_ids), _p(seq_len), c_int(slot_ids.numel()), _stream())
    _check(lib, rc, "seq_set_len")


# ------------------------------------------------------------------ position encoding + cache write
def rope_kv_write(
    qkv: torch.Tensor,
    tok_pos: torch.Tensor,
    tok_seq: torch.Tensor,
    block_table: Optional[torch.Tensor],
    k_pages: Optional[torch.Tensor],
    v_pages: Optional[torch.Tensor],
    inv_freq: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    interleaved: bool,
    write_kv: bool = True,
) -> None:
    """Rotate q (in place) and k, store k and v at each token's place in the paged cache.

    qkv: [T, >= (H + 2K) * hd] rows holding q heads, k heads, v heads.
    k_pages, v_pages: [pages, K, PAGE_SIZE, hd] of qkv's dtype.
    """
    _cuda(qkv, "rope_kv_write qkv", contiguous=False)
    stride = _rows(qkv, "rope_kv_write qkv")
    T = qkv.shape[0]
    _cuda(tok_pos, "rope_kv_write tok_pos", torch.int32)
    _cuda(tok_seq, "rope_kv_write tok_seq", torch.int32)
    _need(tok_pos.numel() == T and tok_seq.numel() == T, "rope_kv_write: one position and one sequence index per token")
    width = 0
    if write_kv:
        _cuda(block_table, "rope_kv_write block_table", torch.int32)
        _need(block_table.dim() == 2, "rope_kv_write: block_table must be [S, width]")
        width = block_table.shape[1]
        for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
            _cuda(pages, f"rope_kv_write {name}", qkv.dtype)
            _need(
                pages.dim() == 4 and tuple(pages.shape[1:]) == (num_kv_heads, PAGE_SIZE, head_dim),
                f"rope_kv_write: {name} {tuple(pages.shape)} is not [pages, {num_kv_heads}, {PAGE_SIZE}, {head_dim}]",
            )
        _need(qkv.shape[1] >= (num_heads + 2 * num_kv_heads) * head_dim, "rope_kv_write: qkv rows too short")
    _need(qkv.data_ptr() % 16 == 0, "rope_kv_write: qkv is not 16-byte aligned")
    if rotary_dim:
        _cuda(inv_freq, "rope_kv_write inv_freq", torch.float32)
        _need(inv_freq.numel() == rotary_dim // 2, "rope_kv_write: inv_freq must hold rotary_dim/2 values")
    lib = build.load("rope")
    rc = lib.rl_rope_kv_write(
        _p(qkv), c_int(_dt(qkv, "rope_kv_write")), c_int(stride), _p(tok_pos), _p(tok_seq), _p(block_table), c_int(width),
        _p(k_pages), _p(v_pages), _p(inv_freq), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
        c_int(rotary_dim), c_int(1 if interleaved else 0), c_int(PAGE_SIZE), c_int(1 if write_kv else 0), _stream(),
    )
    _check(lib, rc, "rope_kv_write")


# ------------------------------------------------------------------ attention
def _check_pages(k_pages, v_pages, dtype, K, hd, what):
    for name, pages in (("k_pages", k_pages), ("v_pages", v_pages)):
        _cuda(pages, f"{what} {name}", dtype)
        _need(
            pages.dim() == 4 and tuple(pages.shape[1:]) == (K, PAGE_SIZE, hd),
            f"{what}: {name} {tuple(pages.shape)} is not [pages, {K}, {PAGE_SIZE}, {hd}]",
        )


def attn_generic(
    q: torch.Tensor, k_pages, v_pages, block_table, tok_seq, tok_pos, num_heads: int, num_kv_heads: int,
    head_dim: int, window: int = 0, scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of each token over its sequence's cached keys 0..pos; any head size up to 256, both dtypes.

    q: [T, >= H*hd] rows (the q part of the fused projection may be passed as is)."""
    _cuda(q, "attn_generic q", contiguous=False)
    qs = _rows(q, "attn_generic q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "attn_generic: q rows too short")
    _check_pages(k_pages, v_pages, q.dtype, num_kv_heads, head_dim, "attn_generic")
    _cuda(block_table, "attn_generic block_table", torch.int32)
    _cuda(tok_seq, "attn_generic tok_seq", torch.int32)
    _cuda(tok_pos, "attn_generic tok_pos", torch.int32)
    _need(tok_seq.numel() == T and tok_pos.numel() == T and block_table.dim() == 2, "attn_generic: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _cuda(out, "attn_generic out", q.dtype)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    lib = build.load("attention_generic")
    rc = lib.rl_attn_generic(
        _p(q), c_int(_dt(q, "attn_generic")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), _p(tok_seq), _p(tok_pos), _p(out), c_int(out.stride(0)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _stream(),
    )
    _check(lib, rc, "attn_generic")
    return out


ATTN_DECODE_TMA_HEAD_DIMS = (64, 128)  # head sizes the TMA-fed decode kernel is built for


def _check_sink(sink, num_heads: int, what: str) -> None:
    if sink is not None:
        _cuda(sink, f"{what} sink", torch.float32)
        _need(sink.numel() == num_heads, f"{what}: one sink per head")


def attn_decode_scratch_floats(n_seqs: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return n_seqs * num_heads * n_splits * (head_dim + 2)


def attn_decode(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_len, num_heads: int, num_kv_heads: int, head_dim: int,
    n_splits: int, scratch: torch.Tensor, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None, impl: str = "auto", fuse: int = 0,
    inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False,
    counters: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0,
) -> torch.Tensor:
    """One query token per sequence over keys 0..seq_len-1, the key range cut into `n_splits`.

    sink: None, or float32 [H]: exp(sink_h) joins the softmax's denominator of head h and nothing else.
    chunk, softcap (the "tma" kernel only): 0, or the size of the chunks of positions outside of which the query sees nothing,
    and 0, or the cap c of s <- c tanh(s / c) on the scaled scores.

    counters (the "tma" kernel only): int32 zeros, one per sequence and group of 8 query heads of a kv
    head; with them the splits are added up by the block that finishes last instead of by a second
    kernel, and the counters are zeros again afterwards.

    fuse (the "tma" kernel only): 0 = q is position-encoded and the new key and value are in the cache
    (what `rope_kv_write` leaves); 1 = q's rows are raw projections, the kernel turns the queries by
    `inv_freq` / `rotary_dim` / `interleaved`; 2 = as 1, and the kernel also takes the new token's key and
    value from q's rows, turns the key and stores both into the cache (k_pages and v_pages are written).

    scratch: float32 tensor of at least attn_decode_scratch_floats(...) elements.
    impl: "warp" = one-warp blocks that copy their own tiles, "tma" = four-warp blocks on a TMA-fed
    ring of whole pages (head sizes 64 and 128), "auto" = "tma" where it applies, else "warp"."""
    q_parts = None
    if q.dim() == 3:
        # the projection as float32 partial sums [parts, S, columns] (a product that was split over k): the
        # fused TMA kernel adds them up as it reads them
        _cuda(q, "attn_decode q (partial sums)", torch.float32, contiguous=False)
        _need(fuse > 0, "attn_decode: partial sums of the projection need fuse > 0")
        _need(q.stride(2) == 1 and q.stride(1) % 4 == 0 and q.stride(0) % 4 == 0, "attn_decode: partial sums must have dense, 16-byte aligned rows")
        q_parts, act = q, k_pages.dtype
        qs, S, q_cols = q.stride(1), q.shape[1], q.shape[2]
    else:
        _cuda(q, "attn_decode q", contiguous=False)
        qs, act = _rows(q, "attn_decode q"), q.dtype
        S, q_cols = q.shape
    _need(q_cols >= num_heads * head_dim, "attn_decode: q rows too short")
    _need(q.data_ptr() % 16 == 0, "attn_decode: q is not 16-byte aligned")
    _check_pages(k_pages, v_pages, act, num_kv_heads, head_dim, "attn_decode")
    _cuda(block_table, "attn_decode block_table", torch.int32)
    _cuda(seq_len, "attn_decode seq_len", torch.int32)
    _need(block_table.dim() == 2 and block_table.shape[0] >= S and seq_len.numel() == S, "attn_decode: metadata sizes")
    _cuda(scratch, "attn_decode scratch", torch.float32)
    need = attn_decode_scratch_floats(S, num_heads, head_dim, n_splits)
    _need(scratch.numel() >= need, f"attn_decode: scratch holds {scratch.numel()} floats, {need} needed")
    if out is None:
        out = torch.empty((S, num_heads * head_dim), dtype=act, device=q.device)
    _cuda(out, "attn_decode out", act, contiguous=False)
    _need(_rows(out, "attn_decode out") >= num_heads * head_dim and tuple(out.shape) == (S, num_heads * head_dim), "attn_decode: out must be [S, H head_dim] rows")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    n_o = S * num_heads * n_splits * head_dim
    part_o = c_void_p(scratch.data_ptr())
    part_ml = c_void_p(scratch.data_ptr() + 4 * n_o)
    _need(impl in ("auto", "warp", "tma"), f"attn_decode: unknown impl {impl!r}")
    if impl == "auto":
        impl = "tma" if (head_dim in ATTN_DECODE_TMA_HEAD_DIMS and act == torch.bfloat16) else "warp"
    _need(fuse in (0, 1, 2), f"attn_decode: fuse={fuse}")
    if fuse:
        _need(impl == "tma", "attn_decode: only the TMA kernel fuses the position encoding")
        if rotary_dim:
            _cuda(inv_freq, "attn_decode inv_freq", torch.float32)
            _need(inv_freq.numel() >= rotary_dim // 2, "attn_decode: too few angles for the rotary size")
        if fuse == 2:
            _need(q_cols >= (num_heads + 2 * num_kv_heads) * head_dim, "attn_decode: q rows hold no key and value")
    if counters is not None:
        _need(impl == "tma", "attn_decode: only the TMA kernel adds the splits up itself")
        _cuda(counters, "attn_decode counters", torch.int32)
        groups = num_kv_heads * ((num_heads // num_kv_heads + 7) // 8)
        _need(counters.numel() >= S * groups, f"attn_decode: {counters.numel()} counters, {S * groups} needed")
    _need(q_parts is None or impl == "tma", "attn_decode: only the TMA kernel takes partial sums")
    _check_sink(sink, num_heads, "attn_decode")
    if impl == "tma":
        _need(act == torch.bfloat16, "attn_decode: the TMA kernel is bfloat16 only")
        status = _tc_status_word(q.device)
        lib = build.load("attention_decode_tma")
        rc = lib.rl_attn_decode_tma(
            c_void_p(0) if q_parts is not None else _p(q), c_int(qs), _p(k_pages), _p(v_pages), c_int(k_pages.shape[0]), _p(block_table),
            c_int(block_table.shape[1]), _p(seq_len), part_o, part_ml, _p(out), c_int(out.stride(0)), c_int(S),
            c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale),
            c_int(n_splits), _p(status), c_int(fuse), _p(inv_freq) if (fuse and rotary_dim) else c_void_p(0), c_int(rotary_dim if fuse else 0),
            c_int(1 if interleaved else 0), _p(counters) if counters is not None else c_void_p(0),
            _p(q_parts) if q_parts is not None else c_void_p(0), c_int(0 if q_parts is None else q_parts.shape[0]),
            c_ll(0 if q_parts is None else q_parts.stride(0)), *_wt(), _p(sink), c_int(chunk), c_float(softcap), _stream(),
        )
        _check(lib, rc, "attn_decode_tma", kernels=1 if counters is not None else 2)
        return out
    _need(chunk == 0 and softcap == 0.0, "attn_decode: only the TMA kernel takes chunks and capped scores")
    lib = build.load("attention_decode")
    rc = lib.rl_attn_decode_sink(
        _p(q), c_int(_dt(q, "attn_decode")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), _p(seq_len), part_o, part_ml, _p(out), c_int(out.stride(0)), c_int(S),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale),
        c_int(n_splits), _p(sink), _stream(),
    )
    _check(lib, rc, "attn_decode", kernels=2)
    return out


def flash_prefill(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int,
    num_kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """bfloat16 causal attention of a ragged batch over the paged cache (tensor cores).  sink: None, or float32 [H] (see `attn_decode`)."""
    _cuda(q, "flash_prefill q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "flash_prefill q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "flash_prefill: q rows too short")
    _need(q.data_ptr() % 16 == 0, "flash_prefill: q is not 16-byte aligned")
    _check_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, head_dim, "flash_prefill")
    _cuda(block_table, "flash_prefill block_table", torch.int32)
    _cuda(seq_start, "flash_prefill seq_start", torch.int32)
    _cuda(seq_pos0, "flash_prefill seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_prefill: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    _cuda(out, "flash_prefill out", torch.bfloat16)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    _check_sink(sink, num_heads, "flash_prefill")
    lib = build.load("attention_prefill")
    rc = lib.rl_flash_prefill(
        _p(q), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(seq_start),
        _p(seq_pos0), _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _p(sink), _stream(),
    )
    _check(lib, rc, "flash_prefill")
    return out


FLASH_TC_HEAD_DIMS = (64, 128)  # head sizes the tcgen05 prompt attention is built for


def flash_prefill_tc(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int,
    num_kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0,
) -> torch.Tensor:
    """`flash_prefill` on the tcgen05 tensor cores (TMA-fed, S and P V in tensor memory); head sizes 64 and 128.
    chunk: 0, or the size of the chunks of positions (counted from 0) outside of which a query sees nothing; softcap: 0, or the
    cap c of s <- c tanh(s / c) on the scaled scores."""
    _need(head_dim in FLASH_TC_HEAD_DIMS, f"flash_prefill_tc: head size {head_dim}, this kernel is built for {FLASH_TC_HEAD_DIMS}")
    _cuda(q, "flash_prefill_tc q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "flash_prefill_tc q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * head_dim, "flash_prefill_tc: q rows too short")
    _check_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, head_dim, "flash_prefill_tc")
    _need(k_pages.shape[0] == v_pages.shape[0], "flash_prefill_tc: k and v have different page counts")
    _cuda(block_table, "flash_prefill_tc block_table", torch.int32)
    _cuda(seq_start, "flash_prefill_tc seq_start", torch.int32)
    _cuda(seq_pos0, "flash_prefill_tc seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_prefill_tc: metadata sizes")
    if out is None:
        out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    _cuda(out, "flash_prefill_tc out", torch.bfloat16, contiguous=False)
    _need(_rows(out, "flash_prefill_tc out") % 8 == 0 and tuple(out.shape) == (T, num_heads * head_dim), "flash_prefill_tc: out must be [T, H head_dim] rows at 16-byte steps")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    _check_sink(sink, num_heads, "flash_prefill_tc")
    status = _tc_status_word(q.device)
    lib = build.load("attention_prefill_tc")
    rc = lib.rl_flash_prefill_tc(
        _p(q), c_int(qs), c_int(T), _p(k_pages), _p(v_pages), c_int(k_pages.shape[0]), _p(block_table),
        c_int(block_table.shape[1]), _p(seq_start), _p(seq_pos0), _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_int(PAGE_SIZE), c_int(window), c_float(scale), _p(status), *_wt(), _p(sink),
        c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "flash_prefill_tc")
    return out


# ------------------------------------------------------------------ matrix products
GEMV_MAX_ROWS = 64


def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T in true 32-bit."""
    _cuda(x, "gemm_f32 x", torch.float32, contiguous=False)
    _cuda(w, "gemm_f32 w", torch.float32, contiguous=False)
    ldx, ldw = _rows(x, "gemm_f32 x"), _rows(w, "gemm_f32 w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_f32: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _cuda(out, "gemm_f32 out", torch.float32, contiguous=False)
    _need(tuple(out.shape) == (M, N), "gemm_f32: out has the wrong shape")
    lib = build.load("gemm_f32")
    rc = lib.rl_gemm_f32(_p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_rows(out, "gemm_f32 out")), c_int(M), c_int(N), c_int(K), _stream())
    _check(lib, rc, "gemm_f32")
    return out


GATED_ACTS = ("gelu_tanh",)  # activations of a gate/up product that are named by a string (a pair (alpha, limit) names the clamped form)


def _act(act):
    """(alpha, limit) of a gate/up product's activation as the launchers take it: None is silu(gate) * up.
    "relu2": the code with which a product that is NOT a gate/up product sends its sums through relu(x)^2."""
    if act is None:
        return c_float(1.0), c_float(0.0)
    if act == "relu2":
        return c_float(0.0), c_float(-2.0)
    if act == "gelu_tanh":  # gelu(gate) * up, the tanh form (RL_GATED_GELU_TANH of csrc/common.cuh)
        return c_float(0.0), c_float(-3.0)
    alpha, limit = act
    _need(limit > 0, f"a gated activation with limits needs a positive limit, got {limit}")
    return c_float(alpha), c_float(limit)


def gemm_bf16_any(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu: bool = False, act=None,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for bfloat16 operands of any k and alignment, 32-bit sums on the
    CUDA cores: the slow kernel behind the shapes that the 16-byte-row kernels refuse.

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums."""
    _cuda(x, "gemm_bf16_any x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemm_bf16_any w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemm_bf16_any x"), _rows(w, "gemm_bf16_any w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_bf16_any: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=x.device)
    lib = build.load("gemm_f32")
    rc = lib.rl_gemm_bf16_any(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemm_bf16_any out")), c_int(out.shape[1]),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), *_act(act), _stream(),
    )
    _check(lib, rc, "gemm_bf16_any")
    return out


def gemv_bf16(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1, act=None,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 64 rows, bfloat16 in, 32-bit accumulate.
    (act, here and in the other products with `swiglu`: None for silu(gate) * up, or (alpha, limit) for
    g s(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit).)

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums.
    k_splits > 1: returns float32 [k_splits, M, N], one partial sum per slice of k, for a consumer
    that adds them (`add_rmsnorm`): more blocks in flight when N is small."""
    _cuda(x, "gemv_bf16 x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_bf16 w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemv_bf16 x"), _rows(w, "gemv_bf16 w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemv_bf16: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemv_bf16: operands must be 16-byte aligned")
    n_out = N // 2 if swiglu else N
    if k_splits > 1:
        _need(out_dtype == torch.float32 and not swiglu, "gemv_bf16: partial sums over k slices are float32, without activation")
        if out is None:
            out = torch.empty((k_splits, M, n_out), dtype=torch.float32, device=x.device)
        _cuda(out, "gemv_bf16 out", torch.float32)
        _need(tuple(out.shape) == (k_splits, M, n_out), "gemv_bf16: out has the wrong shape")
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemv_bf16 out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemv_bf16: out has the wrong shape")
        ldo = _rows(out, "gemv_bf16 out")
    lib = build.load("gemv_bf16")
    rc = lib.rl_gemv_bf16(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_bf16 out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), *_act(act), c_int(k_splits), _stream(),
    )
    _check(lib, rc, "gemv_bf16")
    return out


def gemv_stream_slices(M: int, K: int, k_splits: int = 1) -> int:
    """How many slices of k `gemv_stream` produces for these arguments: 1 is a finished result, more
    are float32 partial sums, 0 means that the kernel does not take the shape (more than 16 rows, k
    no multiple of 64).  A slice is at most 4096 long, or 5120 when k is longer than 4096, so longer k always comes in slices."""
    lib = build.load("gemv_stream")
    return int(lib.rl_gemv_stream_slices(c_int(M), c_int(K), c_int(k_splits)))


def gemv_stream_into_stream(
    x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, next_w: torch.Tensor, xw: Optional[torch.Tensor] = None,
    sumsq: Optional[torch.Tensor] = None,
):
    """The product before an RMSNorm that is folded into its neighbours (at most 8 rows, k a multiple of 64 up to 5120):

        resid (float32 [M, N], in place) += x[M, K] . w[N, K]^T
        xw[M, N] = bfloat16(resid * next_w)           the activations of the product after the norm
        sumsq[blocks, 8]                              each block's share of the rows' sum(resid^2)

    Returns (xw, sumsq, blocks); hand them to `gemv_stream(xw, ..., row_scale=(sumsq, blocks, N, eps))`."""
    _cuda(x, "gemv_stream_into_stream x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_stream_into_stream w", torch.bfloat16, contiguous=False)
    _cuda(resid, "gemv_stream_into_stream resid", torch.float32, contiguous=False)
    _cuda(next_w, "gemv_stream_into_stream next_w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(resid.shape) == (M, N) and tuple(next_w.shape) == (N,),
          f"gemv_stream_into_stream: x{tuple(x.shape)} w{tuple(w.shape)} resid{tuple(resid.shape)} next_w{tuple(next_w.shape)} do not fit")
    lib = build.load("gemv_stream")
    blocks = int(lib.rl_gemv_stream_blocks(c_int(N), c_int(K)))
    _need(blocks > 0, f"gemv_stream_into_stream: the kernel does not take N={N}, K={K}")
    if xw is None:
        xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if sumsq is None:
        sumsq = torch.empty(blocks * 8, dtype=torch.float32, device=x.device)
    _cuda(xw, "gemv_stream_into_stream xw", torch.bfloat16, contiguous=False)
    _cuda(sumsq, "gemv_stream_into_stream sumsq", torch.float32)
    _need(tuple(xw.shape) == (M, N) and sumsq.numel() >= blocks * 8, "gemv_stream_into_stream: xw or sumsq of the wrong size")
    used = c_int(0)
    status = _tc_status_word(x.device)
    rc = lib.rl_gemv_stream_into_stream(
        _p(x), c_int(_rows(x, "gemv_stream_into_stream x")), _p(w), c_int(_rows(w, "gemv_stream_into_stream w")), _p(resid),
        c_int(_rows(resid, "gemv_stream_into_stream resid")), _p(next_w), c_int(_dt(next_w, "gemv_stream_into_stream next_w")), _p(xw),
        c_int(_rows(xw, "gemv_stream_into_stream xw")), _p(sumsq), c_int(M), c_int(N), c_int(K), ctypes.byref(used), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemv_stream_into_stream")
    _need(used.value == blocks, f"gemv_stream_into_stream: the kernel ran {used.value} blocks, the wrapper planned {blocks}")
    return xw, sumsq, blocks


def gemv_stream(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1, row_scale=None, act=None,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T for M <= 16 rows: the persistent weight-streaming kernel of
    decode steps (bulk copies into a ring of shared memory, one block per SM).

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit sums.
    k_splits > 1: returns float32 [slices, M, N] partial sums over slices of k (`gemv_stream_slices`
    says how many: each is a multiple of 1024 and at most 5120 long), for a consumer that adds them up.
    row_scale = (sumsq, blocks, norm_k, eps), as left by `gemv_stream_into_stream`: an RMSNorm folded into this
    product, whose x is then `xw`; every row's sums are multiplied by 1 / sqrt(sum(shares) / norm_k + eps) before
    they are stored or go through the activation (at most 8 rows, k in one slice)."""
    _cuda(x, "gemv_stream x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemv_stream w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemv_stream x"), _rows(w, "gemv_stream w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemv_stream: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    n_out = N // 2 if swiglu else N
    used = c_int(1)
    _need(act in GATED_ACTS or not isinstance(act, str) or (not swiglu and k_splits == 1 and row_scale is None),
          "gemv_stream: an activation of one argument goes with a plain product and whole sums")
    _need(act not in GATED_ACTS or swiglu, "gemv_stream: a gate's activation goes with a gate/up product")
    slices = max(1, gemv_stream_slices(M, K, k_splits))  # (0: the launcher says what it does not take)
    _need(k_splits > 1 or slices == 1, f"gemv_stream: k = {K} comes in {slices} slices, whose float32 partial sums have to be asked for (k_splits > 1)")
    if k_splits > 1 and slices > 1:
        _need(out is None and out_dtype == torch.float32 and not swiglu, "gemv_stream: partial sums over k slices are float32, without activation")
        out = torch.empty((slices, M, n_out), dtype=torch.float32, device=x.device)
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemv_stream out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemv_stream: out has the wrong shape")
        ldo = _rows(out, "gemv_stream out")
    status = _tc_status_word(x.device)
    lib = build.load("gemv_stream")
    if row_scale is not None:
        sumsq, blocks, norm_k, eps = row_scale
        _cuda(sumsq, "gemv_stream row_scale", torch.float32)
        _need(k_splits == 1 and slices == 1 and sumsq.numel() >= blocks * 8, "gemv_stream: a row scale goes with whole sums and needs its shares")
        rc = lib.rl_gemv_stream_scaled(
            _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_stream out")), c_int(ldo), c_int(M), c_int(N), c_int(K),
            c_int(1 if swiglu else 0), *_act(act), _p(sumsq), c_int(blocks), c_int(norm_k), c_float(eps), _p(status), *_wt(), _stream(),
        )
        _check(lib, rc, "gemv_stream")
        return out
    rc = lib.rl_gemv_stream(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemv_stream out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), *_act(act), c_int(k_splits), ctypes.byref(used), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemv_stream")
    _need(used.value == slices, f"gemv_stream: kernel used {used.value} slices, the wrapper planned {slices}")
    return out


_tc_status = {}
_wait_test = (0, 0)  # (role code, limit in nanoseconds) handed to the launchers with bounded waits; (0, 0): none


class short_wait:
    """For tests of the give-up paths: inside `with ops.short_wait(code, ns):` the kernels with bounded waits
    let the role whose status code is `code` wait `ns` nanoseconds instead of a second (every other role keeps
    its limit, and so do the waits that keep a block alive until its copies have landed).  The codes are the
    ones `tc_status_check` names."""

    def __init__(self, role_code: int, limit_ns: int):
        self.value = (int(role_code), int(limit_ns))

    def __enter__(self):
        global _wait_test
        self.before, _wait_test = _wait_test, self.value
        return self

    def __exit__(self, *exc):
        global _wait_test
        _wait_test = self.before
        return False


def _wt():
    return c_int(_wait_test[0]), ctypes.c_uint(_wait_test[1])


def _tc_status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _tc_status:
        _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[key]


_STATUS_NAMES = {
    1: "gemm_tc: the TMA producer (for a free stage)", 2: "gemm_tc: the tensor-core issuer (for a stage's data)",
    3: "gemm_tc: an epilogue warp (for a finished accumulator)", 4: "gemm_tc: the tensor-core issuer (for a free accumulator)",
    11: "flash_prefill_tc: the TMA producer (for a free key stage)", 12: "flash_prefill_tc: the TMA producer (for a free value stage)",
    13: "flash_prefill_tc: the tensor-core issuer (for the queries)", 14: "flash_prefill_tc: the tensor-core issuer (for a key tile)",
    15: "flash_prefill_tc: the tensor-core issuer (for the probabilities)", 16: "flash_prefill_tc: the tensor-core issuer (for a value tile)",
    17: "flash_prefill_tc: a softmax warp (for the scores)", 18: "flash_prefill_tc: a softmax warp (for the product before a rescale)",
    20: "flash_prefill_tc: a softmax warp (for the last product)",
    23: "flash_prefill_tc: shared memory not aligned",
    32: "gemv_stream: the copying lane (for a free stage)", 34: "gemv_stream: a product warp (for a stage's weights)",
    35: "gemv_stream: a storing warp (for an item's sums)", 36: "gemv_stream: shared memory not aligned",
    37: "gemv_stream: a product warp (for a free sum buffer)",
    51: "attn_decode_tma: the copying lane (for a free stage)", 52: "attn_decode_tma: a product warp (for a page)",
    56: "attn_decode_tma: shared memory not aligned",
}


def tc_status_check() -> None:
    """Raise if a bounded wait inside a TMA / tensor-core kernel expired since the last check (synchronises);
    the status word is zero again afterwards."""
    for word in _tc_status.values():
        code = int(word.item())
        if code:
            word.zero_()
            who = _STATUS_NAMES.get(code, "a role")
            raise KernelError(f"{who} gave up waiting on a barrier (code {code}); results of that step are not valid")


def gemm_tc(
    x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None,
    swiglu: bool = False, k_splits: int = 1, tile_n: int = 0, act=None,
) -> torch.Tensor:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory).

    tile_n: 0 (the launcher chooses), or the width of the output tiles, a multiple of 16 up to 256.

    swiglu: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up, from the 32-bit accumulators.
    k_splits > 1: returns float32 [slices, M, N] partial sums over slices of k (at most k_splits of
    them), for a consumer that adds them up: more blocks at work when the output has few tiles."""
    _cuda(x, "gemm_tc x", torch.bfloat16, contiguous=False)
    _cuda(w, "gemm_tc w", torch.bfloat16, contiguous=False)
    ldx, ldw = _rows(x, "gemm_tc x"), _rows(w, "gemm_tc w")
    M, K = x.shape
    N = w.shape[0]
    _need(w.shape[1] == K, f"gemm_tc: x[{M}, {K}] against w[{N}, {w.shape[1]}]")
    n_out = N // 2 if swiglu else N
    used = c_int(1)
    if k_splits > 1:
        _need(out is None and out_dtype == torch.float32 and not swiglu, "gemm_tc: partial sums over k slices are float32, without activation")
        slices = (K + 63) // 64
        per = (slices + min(k_splits, slices) - 1) // min(k_splits, slices)
        k_splits = (slices + per - 1) // per
        out = torch.empty((k_splits, M, n_out), dtype=torch.float32, device=x.device)
        ldo = n_out
    else:
        if out is None:
            out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _cuda(out, "gemm_tc out", out_dtype, contiguous=False)
        _need(tuple(out.shape) == (M, n_out), "gemm_tc: out has the wrong shape")
        ldo = _rows(out, "gemm_tc out")
    status = _tc_status_word(x.device)
    lib = build.load("gemm_tc")
    rc = lib.rl_gemm_tc(
        _p(x), c_int(ldx), _p(w), c_int(ldw), _p(out), c_int(_dt(out, "gemm_tc out")), c_int(ldo),
        c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), *_act(act), c_int(k_splits), ctypes.byref(used), c_int(tile_n), _p(status), *_wt(), _stream(),
    )
    _check(lib, rc, "gemm_tc")
    if k_splits > 1:
        _need(used.value == k_splits, f"gemm_tc: kernel used {used.value} slices, the wrapper planned {k_splits}")
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit of each row, the last one among equals."""
    _cuda(logits, "argmax logits", torch.float32, contiguous=False)
    stride = _rows(logits, "argmax logits")
    R, n = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "argmax out", torch.int32)
    lib = build.load("sampling")
    rc = lib.rl_argmax(_p(logits), c_ll(stride), c_int(R), c_int(n), _p(out), _stream())
    _check(lib, rc, "argmax")
    return out


def sample(
    logits: torch.Tensor, temperature: float, top_p: float, rng_states: torch.Tensor, rng_index: torch.Tensor,
    scratch: torch.Tensor, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature), cut to the top-p nucleus when 0 < top_p < 1.

    rng_states: int64 tensor of xorshift64* states; row r uses and advances rng_states[rng_index[r]].
    scratch: float32, at least rows * vocabulary elements."""
    _cuda(logits, "sample logits", torch.float32, contiguous=False)
    stride = _rows(logits, "sample logits")
    R, n = logits.shape
    _cuda(rng_states, "sample rng_states", torch.int64)
    _cuda(rng_index, "sample rng_index", torch.int32)
    _need(rng_index.numel() == R, "sample: one random-state index per row")
    _cuda(scratch, "sample scratch", torch.float32)
    _need(scratch.numel() >= R * n, f"sample: scratch holds {scratch.numel()} floats, {R * n} needed")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "sample out", torch.int32)
    lib = build.load("sampling")
    rc = lib.rl_sample(
        _p(logits), c_ll(stride), c_int(R), c_int(n), c_float(temperature), c_float(top_p), _p(rng_states),
        _p(rng_index), _p(scratch), _p(out), _stream(),
    )
    _check(lib, rc, "sample")
    return out


SAMPLE_HISTORY_MAX = 1024


def sample_chain(
    logits: torch.Tensor, temperature: float, top_p: float, top_k: int, min_p: float, repeat_penalty: float,
    last_n: int, frequency_penalty: float, presence_penalty: float, rng_states: torch.Tensor, slot_of_row: torch.Tensor,
    history: torch.Tensor, history_count: torch.Tensor, work: torch.Tensor, out: Optional[torch.Tensor] = None,
    mirostat: int = 0, mirostat_tau: float = 5.0, mirostat_eta: float = 0.1, mirostat_mu: Optional[torch.Tensor] = None,
    xtc_probability: float = 0.0, xtc_threshold: float = 0.1, xtc_states: Optional[torch.Tensor] = None,
    dry_multiplier: float = 0.0, dry_base: float = 1.75, dry_allowed_length: int = 2, dry_last_n: int = 0,
    dry_breakers: Sequence[int] = (),
) -> torch.Tensor:
    """One token per row through penalties -> top-k -> top-p -> min-p -> temperature -> draw (temperature 0:
    the argmax of the penalised logits, no draw).

    Row r belongs to slot slot_of_row[r]: it uses and advances rng_states[slot], reads the last `last_n`
    chosen tokens of history[slot] (int32 [slots, 1024] with history_count[slot] tokens written so far) for
    the penalties and appends its choice.  work: float32, at least rows * 2 * (vocabulary rounded up to 4).
    mirostat 1 or 2: penalties -> temperature -> mirostat's own cut and draw; mirostat_mu: float32 [slots], NaN
    for a sequence that has not drawn yet.  xtc_probability > 0: the "exclude top choices" filter after min-p, with
    a generator of its own per slot (xtc_states, int64 like rng_states).  dry_multiplier > 0: the DRY penalty
    after the other penalties, over the last dry_last_n chosen tokens, with up to 8 breaker tokens.
    history[slot] is a ring over all 1024 places (the p-th chosen token at p % 1024), whatever the windows."""
    _cuda(logits, "sample_chain logits", torch.float32, contiguous=False)
    stride = _rows(logits, "sample_chain logits")
    R, n = logits.shape
    _cuda(rng_states, "sample_chain rng_states", torch.int64)
    _cuda(slot_of_row, "sample_chain slot_of_row", torch.int32)
    _need(slot_of_row.numel() == R, "sample_chain: one slot per row")
    _cuda(history, "sample_chain history", torch.int32)
    _cuda(history_count, "sample_chain history_count", torch.int32)
    _need(history.dim() == 2 and history.shape[1] == SAMPLE_HISTORY_MAX and history.shape[0] == history_count.numel(),
          f"sample_chain: history must be [slots, {SAMPLE_HISTORY_MAX}] with one count per slot")
    _cuda(work, "sample_chain work", torch.float32)
    need = R * 2 * ((n + 3) // 4 * 4)
    _need(work.numel() >= need, f"sample_chain: work holds {work.numel()} floats, {need} needed")
    _need(work.data_ptr() % 16 == 0, "sample_chain: work must be 16-byte aligned")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _cuda(out, "sample_chain out", torch.int32)
    if mirostat:
        _need(mirostat_mu is not None, "sample_chain: mirostat needs its state")
        _cuda(mirostat_mu, "sample_chain mirostat_mu", torch.float32)
        _need(mirostat_mu.numel() == history_count.numel(), "sample_chain: one mirostat state per slot")
    if xtc_probability > 0.0:
        _need(xtc_states is not None, "sample_chain: XTC needs its random states")
        _cuda(xtc_states, "sample_chain xtc_states", torch.int64)
        _need(xtc_states.numel() == history_count.numel(), "sample_chain: one XTC state per slot")
    breakers = (ctypes.c_int * max(len(dry_breakers), 1))(*[int(b) for b in dry_breakers])
    lib = build.load("sampling")
    rc = lib.rl_sample_chain(
        _p(logits), c_ll(stride), c_int(R), c_int(n), c_float(temperature), c_float(top_p), c_int(top_k), c_float(min_p),
        c_float(repeat_penalty), c_int(last_n), c_float(frequency_penalty), c_float(presence_penalty), c_int(mirostat),
        c_float(mirostat_tau), c_float(mirostat_eta), c_float(xtc_probability), c_float(xtc_threshold),
        c_float(dry_multiplier), c_float(dry_base), c_int(dry_allowed_length), c_int(dry_last_n), breakers, c_int(len(dry_breakers)),
        _p(rng_states),
        _p(slot_of_row), _p(history), _p(history_count), _p(mirostat_mu) if mirostat_mu is not None else c_void_p(0),
        _p(xtc_states) if xtc_states is not None else c_void_p(0), _p(work), _p(out), _stream(),
    )
    _check(lib, rc, "sample_chain")
    return out


# ------------------------------------------------------------------ sublayer results that are normed before they are added
def normed_add_rmsnorm(
    x: torch.Tensor, delta: torch.Tensor, delta_weight: torch.Tensor, delta_eps: float, weight: Optional[torch.Tensor], eps: float,
    act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, write_x: bool = True, delta_bias: Optional[torch.Tensor] = None,
) -> Optional[torch.Tensor]:
    """x (float32 [T, d]) += rmsnorm(sum of delta parts + delta_bias) * delta_weight; returns rmsnorm(x) * weight in `act_dtype`
    (None without a weight).  delta: [T, d] or [parts, T, d], in `act_dtype` or float32.  Both norm weights have one type.
    delta_bias: None or float32 [d], a row that belongs to every row of the summed delta (a projection's bias)."""
    _cuda(x, "normed_add_rmsnorm x", torch.float32)
    T, d = x.shape
    _cuda(delta, "normed_add_rmsnorm delta")
    _need(delta.dtype in (act_dtype, torch.float32), f"normed_add_rmsnorm: delta is {delta.dtype} in a run of {act_dtype}")
    if delta.dim() == 2:
        _need(tuple(delta.shape) == (T, d), f"normed_add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
        n_parts, part_stride = 1, 0
    else:
        _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (T, d), f"normed_add_rmsnorm: delta {tuple(delta.shape)} does not match x {(T, d)}")
        n_parts, part_stride = delta.shape[0], T * d
    _cuda(delta_weight, "normed_add_rmsnorm delta_weight")
    _need(tuple(delta_weight.shape) == (d,), "normed_add_rmsnorm: delta_weight does not match d")
    n_rows = T if rows is None else rows.numel()
    out = None
    if weight is not None:
        _cuda(weight, "normed_add_rmsnorm weight", delta_weight.dtype)
        _need(tuple(weight.shape) == (d,), "normed_add_rmsnorm: weight does not match d")
        out = torch.empty((n_rows, d), dtype=act_dtype, device=x.device)
    if rows is not None:
        _cuda(rows, "normed_add_rmsnorm rows", torch.int32)
    if delta_bias is not None:
        _cuda(delta_bias, "normed_add_rmsnorm delta_bias", torch.float32)
        _need(tuple(delta_bias.shape) == (d,) and delta_bias.data_ptr() % 16 == 0, "normed_add_rmsnorm: delta_bias must be an aligned row of d numbers")
    if n_rows == 0:
        return out
    lib = build.load("elementwise")
    rc = lib.rl_normed_add_rmsnorm(
        _p(x), _p(delta), c_int(_DT[delta.dtype]), c_int(n_parts), c_ll(part_stride), _p(delta_bias), _p(delta_weight), c_float(delta_eps), _p(weight),
        c_int(_dt(delta_weight, "normed_add_rmsnorm weight")), c_float(eps), _p(out), c_int(_DT[act_dtype]), _p(rows), c_int(n_rows),
        c_int(d), c_int(1 if write_x else 0), _stream(),
    )
    _check(lib, rc, "normed_add_rmsnorm")
    return out


def gated_glu(gate_up: torch.Tensor, act) -> torch.Tensor:
    """h[t, i] = act(gate_up[t, i], gate_up[t, ff + i]) for the activations of a gate/up product (None: silu(gate) * up,
    (alpha, limit): the clamped form, "gelu_tanh": gelu(gate) * up), as a pass of its own behind a plain product."""
    alpha, limit = _act(act)
    return clamped_glu(gate_up, alpha.value, limit.value)


def clamped_glu(gate_up: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """h[t, i] = g * sigmoid(alpha * g) * (u + 1), g = min(gate_up[t, i], limit), u = clamp(gate_up[t, ff + i], -limit, limit)."""
    _cuda(gate_up, "clamped_glu input")
    _need(gate_up.dim() == 2 and gate_up.shape[1] % 2 == 0, "clamped_glu: input must be [T, 2*ff]")
    T, ff = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((T, ff), dtype=gate_up.dtype, device=gate_up.device)
    lib = build.load("elementwise")
    rc = lib.rl_clamped_glu(_p(gate_up), _p(out), c_int(_dt(gate_up, "clamped_glu")), c_int(T), c_int(ff), c_float(alpha), c_float(limit), _stream())
    _check(lib, rc, "clamped_glu")
    return out


# ------------------------------------------------------------------ latent attention
def latent_prep(
    q: torch.Tensor, kv: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor], n_pairs: int,
    magnitude: float, tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor],
    q_cat: torch.Tensor, num_heads: int, dim: int, rot: int, rank: int,
) -> None:
    """Per token: kv's first `rank` values RMS-normed (weight norm_w) and its last `rot` values rotated go into the token's
    place in `pages` [pages, 1, PAGE_SIZE, rank + rot] (kv None: nothing is stored); the rotated part of every head of
    q [T, >= H (dim + rot)] is rotated into q_cat[T, H, rank:]."""
    _cuda(q, "latent_prep q", contiguous=False)
    ldq = _rows(q, "latent_prep q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * (dim + rot), "latent_prep: q rows too short")
    _cuda(q_cat, "latent_prep q_cat", q.dtype)
    _need(tuple(q_cat.shape) == (T, num_heads, rank + rot), "latent_prep: q_cat has the wrong shape")
    _cuda(tok_pos, "latent_prep tok_pos", torch.int32)
    _cuda(tok_seq, "latent_prep tok_seq", torch.int32)
    _need(tok_pos.numel() == T and tok_seq.numel() == T, "latent_prep: one position and one sequence index per token")
    ldkv, width = 0, 0
    if kv is not None:
        _cuda(kv, "latent_prep kv", q.dtype, contiguous=False)
        ldkv = _rows(kv, "latent_prep kv")
        _need(kv.shape[0] == T and kv.shape[1] >= rank + rot, "latent_prep: kv rows do not fit")
        _cuda(pages, "latent_prep pages", q.dtype)
        _need(pages.dim() == 4 and tuple(pages.shape[1:]) == (1, PAGE_SIZE, rank + rot), f"latent_prep: pages {tuple(pages.shape)}")
        _cuda(block_table, "latent_prep block_table", torch.int32)
        _need(block_table.dim() == 2, "latent_prep: block_table must be [S, width]")
        width = block_table.shape[1]
        _cuda(norm_w, "latent_prep norm_w", torch.float32)
        _need(norm_w.numel() == rank, "latent_prep: norm weight does not match the latent size")
    if n_pairs:
        _cuda(freq, "latent_prep freq", torch.float32)
        _need(freq.numel() >= n_pairs, "latent_prep: too few angles")
    lib = build.load("latent_attention")
    rc = lib.rl_latent_prep(
        _p(q), c_int(ldq), _p(kv), c_int(ldkv), c_int(_dt(q, "latent_prep")), _p(norm_w), c_float(eps), _p(freq), c_int(n_pairs),
        c_float(magnitude), _p(tok_pos), _p(tok_seq), _p(block_table) if kv is not None else c_void_p(0), c_int(width),
        _p(pages) if kv is not None else c_void_p(0), c_int(PAGE_SIZE), _p(q_cat), c_int(T), c_int(num_heads), c_int(dim), c_int(rot),
        c_int(rank), _stream(),
    )
    _check(lib, rc, "latent_prep")


def head_linear(
    x: torch.Tensor, x_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int,
    gate: Optional[torch.Tensor] = None, gate_head_stride: int = 0,
) -> torch.Tensor:
    """out[t, h, n] = sum_k x[t, h, k] * w[h, n, k] (optionally times sigmoid(gate[t, h, n])), one small product per head.

    x, out, gate: 2-D [T, row] tensors with dense rows; head h's values start `*_head_stride` * h into a row.  w: [H, N, K]."""
    _cuda(x, "head_linear x", contiguous=False)
    _cuda(w, "head_linear w", x.dtype)
    _cuda(out, "head_linear out", x.dtype, contiguous=False)
    _need(w.dim() == 3, "head_linear: w must be [H, N, K]")
    H, N, K = w.shape
    M = x.shape[0]
    ldx, ldo = _rows(x, "head_linear x"), _rows(out, "head_linear out")
    _need(out.shape[0] == M, "head_linear: x and out have different row counts")
    _need((H - 1) * x_head_stride + K <= x.shape[1] and (H - 1) * out_head_stride + N <= out.shape[1], "head_linear: rows too short for the heads")
    ldg = 0
    if gate is not None:
        _cuda(gate, "head_linear gate", x.dtype, contiguous=False)
        ldg = _rows(gate, "head_linear gate")
        _need(gate.shape[0] == M and (H - 1) * gate_head_stride + N <= gate.shape[1], "head_linear: gate rows do not fit")
    if x.dtype == torch.bfloat16 and grouped_gemm_takes(K, ldx, x_head_stride) and x.data_ptr() % 16 == 0:
        lib = build.load("grouped_gemm")
        rc = lib.rl_head_linear_mma(
            _p(x), c_int(ldx), c_int(x_head_stride), _p(w), _p(out), c_int(ldo), c_int(out_head_stride), _p(gate), c_int(ldg),
            c_int(gate_head_stride), c_int(M), c_int(H), c_int(N), c_int(K), _stream(),
        )
        _check(lib, rc, "head_linear_mma")
        return out
    lib = build.load("latent_attention")
    rc = lib.rl_head_linear(
        _p(x), c_int(ldx), c_int(x_head_stride), _p(w), c_ll(N * K), c_int(K), c_int(1), _p(out), c_int(ldo), c_int(out_head_stride),
        _p(gate), c_int(ldg), c_int(gate_head_stride), c_int(_dt(x, "head_linear")), c_int(M), c_int(H), c_int(N), c_int(K), _stream(),
    )
    _check(lib, rc, "head_linear")
    return out


def latent_attn(
    q_cat: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor,
    sink: Optional[torch.Tensor], rank: int, rot: int, scale: float, window: int = 0, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention of each token's heads q_cat[T, H, rank + rot] over its sequence's cached rows 0..pos of
    pages [pages, 1, PAGE_SIZE, rank + rot]; softmax with a sink per head (float32 [H], or None); returns the
    probability-weighted sums of the rows' first `rank` values, [T, H, rank]."""
    _cuda(q_cat, "latent_attn q_cat")
    _need(q_cat.dim() == 3 and q_cat.shape[2] == rank + rot, "latent_attn: q_cat must be [T, H, rank + rot]")
    T, H = q_cat.shape[0], q_cat.shape[1]
    _cuda(pages, "latent_attn pages", q_cat.dtype)
    _need(pages.dim() == 4 and tuple(pages.shape[1:]) == (1, PAGE_SIZE, rank + rot), f"latent_attn: pages {tuple(pages.shape)}")
    _cuda(block_table, "latent_attn block_table", torch.int32)
    _cuda(tok_seq, "latent_attn tok_seq", torch.int32)
    _cuda(tok_pos, "latent_attn tok_pos", torch.int32)
    _need(tok_seq.numel() == T and tok_pos.numel() == T and block_table.dim() == 2, "latent_attn: metadata sizes")
    if sink is not None:
        _cuda(sink, "latent_attn sink", torch.float32)
        _need(sink.numel() == H, "latent_attn: one sink per head")
    if out is None:
        out = torch.empty((T, H, rank), dtype=q_cat.dtype, device=q_cat.device)
    _cuda(out, "latent_attn out", q_cat.dtype)
    _need(tuple(out.shape) == (T, H, rank), "latent_attn: out has the wrong shape")
    lib = build.load("latent_attention")
    rc = lib.rl_latent_attn(
        _p(q_cat), _p(pages), c_int(_dt(q_cat, "latent_attn")), _p(block_table), c_int(block_table.shape[1]), _p(tok_seq), _p(tok_pos),
        _p(sink), _p(out), c_int(T), c_int(H), c_int(rank), c_int(rot), c_int(PAGE_SIZE), c_int(window), c_float(scale), _stream(),
    )
    _check(lib, rc, "latent_attn")
    return out


# ------------------------------------------------------------------ routed feed-forward
def grouped_gemm_takes(K: int, ldx: int, head_stride: int) -> bool:
    """Whether the tensor-core products of `grouped_gemm.cu` take operands with this k and these strides (in elements)."""
    return bool(build.load("grouped_gemm").rl_grouped_gemm_takes(c_int(K), c_int(ldx), c_int(head_stride)))


def moe_tile_rows() -> int:
    return int(build.load("moe").rl_moe_tile_rows())


def moe_router(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], n_experts: int, top: int, renormalize: bool = False,
               logistic: bool = False, renorm_eps: float = 0.0, weight_scale: float = 1.0):
    """x[T, d], w float32 [E (+1), d] -> (ids int32 [T, top], weights float32 [T, top], gate float32 [T] or None).

    Softmax over the E experts in 32-bit (`logistic`: the logistic function of every logit instead); the `top` largest of
    score + bias are chosen, their weights are their scores (divided by their sum + `renorm_eps` if `renormalize`), times
    `weight_scale`.  A row E of w gives gate = sigmoid(w[E] . x)."""
    _cuda(x, "moe_router x", contiguous=False)
    _cuda(w, "moe_router w", torch.float32)
    T, d = x.shape
    has_gate = w.shape[0] == n_experts + 1
    _need(w.dim() == 2 and w.shape[1] == d and w.shape[0] in (n_experts, n_experts + 1), f"moe_router: w {tuple(w.shape)} for {n_experts} experts of width {d}")
    if bias is not None:
        _cuda(bias, "moe_router bias", torch.float32)
        _need(bias.numel() == n_experts, "moe_router: one bias per expert")
    ids = torch.empty((T, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
    gate = torch.empty((T,), dtype=torch.float32, device=x.device) if has_gate else None
    logits = torch.empty((T, w.shape[0]), dtype=torch.float32, device=x.device)
    lib = build.load("moe")
    rc = lib.rl_moe_router(
        _p(x), c_int(_rows(x, "moe_router x")), c_int(_dt(x, "moe_router")), _p(w), _p(bias), c_int(T), c_int(n_experts), c_int(d), c_int(top),
        c_int(1 if renormalize else 0), c_int(1 if has_gate else 0), _p(logits), _p(ids), _p(weights), _p(gate), c_int(1 if logistic else 0),
        c_float(renorm_eps), c_float(weight_scale), _stream(),
    )
    _check(lib, rc, "moe_router", kernels=2)
    return ids, weights, gate


def moe_table_lookup(tokens: torch.Tensor, table: torch.Tensor, n_experts: int):
    """tokens int32 [T], table int32 [vocab, top] -> (ids int32 [T, top] = table[tokens], weights float32 [T, top] = 1 / top)."""
    _cuda(tokens, "moe_table_lookup tokens", torch.int32)
    _cuda(table, "moe_table_lookup table", torch.int32)
    _need(tokens.dim() == 1 and table.dim() == 2, "moe_table_lookup: tokens[T] and table[vocab, top] expected")
    T, top = tokens.numel(), table.shape[1]
    ids = torch.empty((T, top), dtype=torch.int32, device=tokens.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=tokens.device)
    lib = build.load("moe")
    rc = lib.rl_moe_table_lookup(_p(tokens), _p(table), c_int(top), c_int(T), c_int(n_experts), _p(ids), _p(weights), _stream())
    _check(lib, rc, "moe_table_lookup")
    return ids, weights


MOE_MMA_TILE_ROWS = (32, 128)  # tile heights the tensor-core products are built for


def moe_max_tiles(n_pairs: int, n_experts: int, tile_rows: int = 0) -> int:
    """Upper bound of the row tiles that `moe_plan` makes of n_pairs (token, choice) pairs."""
    rows = tile_rows or moe_tile_rows()
    return min(n_pairs, n_pairs // rows + n_experts)


def moe_plan(ids: torch.Tensor, n_experts: int, tile_rows: int = 0):
    """ids int32 [T, top] -> (order [T top], place [T top], tiles [1 + 3 max_tiles], max_tiles), all on the device.
    tile_rows: the height of a row tile (0: the plain product's)."""
    _cuda(ids, "moe_plan ids", torch.int32)
    n = ids.numel()
    tile_rows = tile_rows or moe_tile_rows()
    max_tiles = moe_max_tiles(n, n_experts, tile_rows)
    order = torch.empty((n,), dtype=torch.int32, device=ids.device)
    place = torch.empty((n,), dtype=torch.int32, device=ids.device)
    tiles = torch.empty((1 + 3 * max_tiles,), dtype=torch.int32, device=ids.device)
    lib = build.load("moe")
    rc = lib.rl_moe_plan(_p(ids), c_int(n), c_int(n_experts), _p(order), _p(place), _p(tiles), c_int(tile_rows), _stream())
    _check(lib, rc, "moe_plan")
    return order, place, tiles, max_tiles


def moe_gemm(
    x: torch.Tensor, w: torch.Tensor, tiles: torch.Tensor, max_tiles: int, n_rows: int, order: Optional[torch.Tensor] = None,
    gather_div: int = 1, w2: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, tile_rows: int = 0, act=None,
) -> torch.Tensor:
    """out[r] = w[expert of r] . x[row of r] for the n_rows rows of a plan's layout; w: [E, N, K].

    order given: row r reads x[order[r] // gather_div], else x[r].  w2 given: out = silu(w x) * (w2 x), or with act = (alpha, limit)
    g s(alpha g) (u + 1), g = min(w x, limit), u = clamp(w2 x, -limit, limit).
    tile_rows: the height of the plan's tiles; bfloat16 operands whose rows can be moved in 16-byte pieces go to the
    tensor cores if it is one of MOE_MMA_TILE_ROWS, everything else to the plain kernel (which wants its own height)."""
    _cuda(x, "moe_gemm x", contiguous=False)
    _cuda(w, "moe_gemm w", x.dtype)
    _need(w.dim() == 3 and w.shape[2] == x.shape[1], f"moe_gemm: w {tuple(w.shape)} against x {tuple(x.shape)}")
    E, N, K = w.shape
    if w2 is not None:
        _cuda(w2, "moe_gemm w2", x.dtype)
        _need(tuple(w2.shape) == (E, N, K), "moe_gemm: w2 does not match w")
    out_dtype = out_dtype or x.dtype
    out = torch.empty((n_rows, N), dtype=out_dtype, device=x.device)
    tile_rows = tile_rows or moe_tile_rows()
    alpha, limit = _act(act)
    if x.dtype == torch.bfloat16 and tile_rows in MOE_MMA_TILE_ROWS and grouped_gemm_takes(K, x.stride(0), 0) and x.data_ptr() % 16 == 0:
        lib = build.load("grouped_gemm")
        rc = lib.rl_moe_gemm_mma(
            _p(x), c_int(x.stride(0)), _p(order), c_int(gather_div), _p(w), _p(w2), _p(out), c_int(_dt(out, "moe_gemm out")), c_int(N),
            _p(tiles), c_int(max_tiles), c_int(tile_rows), c_int(N), c_int(K), alpha, limit, _stream(),
        )
        _check(lib, rc, "moe_gemm_mma")
        return out
    _need(tile_rows == moe_tile_rows(), f"moe_gemm: the plain kernel wants tiles of {moe_tile_rows()} rows, the plan has {tile_rows}")
    lib = build.load("moe")
    rc = lib.rl_moe_gemm(
        _p(x), c_int(_rows(x, "moe_gemm x")), c_int(_dt(x, "moe_gemm")), _p(order), c_int(gather_div), _p(w), _p(w2), _p(out),
        c_int(_dt(out, "moe_gemm out")), c_int(N), _p(tiles), c_int(max_tiles), c_int(N), c_int(K), alpha, limit, _stream(),
    )
    _check(lib, rc, "moe_gemm")
    return out


def moe_combine(
    y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
    out_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * y[place[t, j]] (+ gate[t] * shared[t]); y float32 [T top, d]."""
    _cuda(y, "moe_combine y", torch.float32)
    _cuda(weights, "moe_combine weights", torch.float32)
    _cuda(place, "moe_combine place", torch.int32)
    T, top = weights.shape
    d = y.shape[1]
    _need(y.shape[0] == T * top and place.numel() == T * top, "moe_combine: sizes do not fit")
    shared_dt = _F32
    if shared is not None:
        _cuda(shared, "moe_combine shared")
        _need(tuple(shared.shape) == (T, d), "moe_combine: shared has the wrong shape")
        shared_dt = _dt(shared, "moe_combine shared")
    if gate is not None:
        _cuda(gate, "moe_combine gate", torch.float32)
    out = torch.empty((T, d), dtype=out_dtype, device=y.device)
    lib = build.load("moe")
    rc = lib.rl_moe_combine(
        _p(y), _p(place), _p(weights), c_int(top), _p(shared), c_int(shared_dt), _p(gate), _p(out), c_int(_dt(out, "moe_combine out")),
        c_int(T), c_int(d), _stream(),
    )
    _check(lib, rc, "moe_combine")
    return out


def latent_attn_mma_takes(rank: int, rot: int) -> bool:
    """Whether the tensor-core latent attention is built for these sizes (else `latent_attn` takes them)."""
    return bool(build.load("latent_attention_mma").rl_latent_attn_mma_takes(c_int(rank), c_int(rot)))


def latent_attn_mma_scratch_floats(n_rows: int, rank: int, n_splits: int) -> int:
    return n_rows * n_splits * (rank + 2) if n_splits > 1 else 0


def latent_attn_mma(
    q_cat: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, seq_start: torch.Tensor, seq_pos0: torch.Tensor, max_q_len: int,
    sink: Optional[torch.Tensor], rank: int, rot: int, scale: float, window: int = 0, n_splits: int = 1,
    scratch: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """`latent_attn` on the tensor cores, bfloat16: sequence s brings the tokens seq_start[s] .. seq_start[s+1]-1 of q_cat
    [T, H, rank + rot] at positions seq_pos0[s], seq_pos0[s] + 1, ...; max_q_len: the most tokens one sequence brings.
    n_splits > 1 cuts every sequence's key range into that many parts (float32 scratch of
    `latent_attn_mma_scratch_floats` elements), added up by a second kernel."""
    _cuda(q_cat, "latent_attn_mma q_cat", torch.bfloat16)
    _need(q_cat.dim() == 3 and q_cat.shape[2] == rank + rot, "latent_attn_mma: q_cat must be [T, H, rank + rot]")
    T, H = q_cat.shape[0], q_cat.shape[1]
    _cuda(pages, "latent_attn_mma pages", torch.bfloat16)
    _need(pages.dim() == 4 and tuple(pages.shape[1:]) == (1, PAGE_SIZE, rank + rot), f"latent_attn_mma: pages {tuple(pages.shape)}")
    _need(q_cat.data_ptr() % 16 == 0 and pages.data_ptr() % 16 == 0, "latent_attn_mma: tensors must be 16-byte aligned")
    _cuda(block_table, "latent_attn_mma block_table", torch.int32)
    _cuda(seq_start, "latent_attn_mma seq_start", torch.int32)
    _cuda(seq_pos0, "latent_attn_mma seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "latent_attn_mma: metadata sizes")
    if sink is not None:
        _cuda(sink, "latent_attn_mma sink", torch.float32)
        _need(sink.numel() == H, "latent_attn_mma: one sink per head")
    if n_splits > 1:
        _cuda(scratch, "latent_attn_mma scratch", torch.float32)
        need = latent_attn_mma_scratch_floats(T * H, rank, n_splits)
        _need(scratch.numel() >= need, f"latent_attn_mma: scratch holds {scratch.numel()} floats, {need} needed")
    if out is None:
        out = torch.empty((T, H, rank), dtype=torch.bfloat16, device=q_cat.device)
    _cuda(out, "latent_attn_mma out", torch.bfloat16)
    _need(tuple(out.shape) == (T, H, rank), "latent_attn_mma: out has the wrong shape")
    lib = build.load("latent_attention_mma")
    rc = lib.rl_latent_attn_mma(
        _p(q_cat), _p(pages), _p(block_table), c_int(block_table.shape[1]), _p(seq_start), _p(seq_pos0), _p(sink), _p(out),
        _p(scratch) if n_splits > 1 else c_void_p(0), c_ll(T * H), c_int(S), c_int(max_q_len * H), c_int(H), c_int(rank), c_int(rot),
        c_int(PAGE_SIZE), c_int(window), c_float(scale), c_int(n_splits), _stream(),
    )
    _check(lib, rc, "latent_attn_mma", kernels=2 if n_splits > 1 else 1)
    return out


# ------------------------------------------------------------------ attention with options (csrc/attention_ext.cu)
def _check_kv_pages(k_pages, v_pages, dtype, K, kdim, vdim, what):
    for name, pages, size in (("k_pages", k_pages, kdim), ("v_pages", v_pages, vdim)):
        _cuda(pages, f"{what} {name}", dtype)
        _need(
            pages.dim() == 4 and tuple(pages.shape[1:]) == (K, PAGE_SIZE, size),
            f"{what}: {name} {tuple(pages.shape)} is not [pages, {K}, {PAGE_SIZE}, {size}]",
        )


def qkv_prep(
    qkv: torch.Tensor, bias: Optional[torch.Tensor], tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
    k_pages: torch.Tensor, v_pages: torch.Tensor, inv_freq: Optional[torch.Tensor], magnitude: float, num_heads: int, num_kv_heads: int,
    kdim: int, vdim: int, rotary_dim: int, interleaved: bool, q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None,
    norm_eps: float = 0.0, v_src: Optional[torch.Tensor] = None, v_lambda: Optional[torch.Tensor] = None,
) -> None:
    """qkv[T, >= (H + K) kdim + K vdim]: add `bias` (float32, one number per column, or None), divide every q head (k head) by its
    root mean square and multiply it by `q_norm` (`k_norm`; float32 [kdim], None: no norm), rotate the first `rotary_dim`
    dimensions of every q head (in place) and k head by position * inv_freq, cosines and sines times `magnitude`, and store
    k and v at each token's place in the paged cache (k_pages [pages, K, PAGE_SIZE, kdim], v_pages [..., vdim]).
    v_src ([T, K vdim] rows of qkv's type) with v_lambda (float32, one number on the device): what is stored as the value is
    (1 - lambda) v + lambda v_src[t]."""
    _cuda(qkv, "qkv_prep qkv", contiguous=False)
    stride = _rows(qkv, "qkv_prep qkv")
    T = qkv.shape[0]
    cols = (num_heads + num_kv_heads) * kdim + num_kv_heads * vdim
    _need(qkv.shape[1] >= cols, "qkv_prep: qkv rows too short")
    _cuda(tok_pos, "qkv_prep tok_pos", torch.int32)
    _cuda(tok_seq, "qkv_prep tok_seq", torch.int32)
    _need(tok_pos.numel() == T and tok_seq.numel() == T, "qkv_prep: one position and one sequence index per token")
    _cuda(block_table, "qkv_prep block_table", torch.int32)
    _need(block_table.dim() == 2, "qkv_prep: block_table must be [S, width]")
    _check_kv_pages(k_pages, v_pages, qkv.dtype, num_kv_heads, kdim, vdim, "qkv_prep")
    if bias is not None:
        _cuda(bias, "qkv_prep bias", torch.float32)
        _need(bias.numel() == cols, f"qkv_prep: bias has {bias.numel()} numbers for {cols} columns")
    if rotary_dim:
        _cuda(inv_freq, "qkv_prep inv_freq", torch.float32)
        _need(inv_freq.numel() == rotary_dim // 2, "qkv_prep: inv_freq must hold rotary_dim/2 values")
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None:
            _cuda(w, f"qkv_prep {name}", torch.float32)
            _need(w.numel() == kdim, f"qkv_prep: {name} must hold one weight per number of a head ({kdim})")
    vs_stride = 0
    if v_src is not None:
        _cuda(v_src, "qkv_prep v_src", qkv.dtype, contiguous=False)
        vs_stride = _rows(v_src, "qkv_prep v_src")
        _need(tuple(v_src.shape) == (T, num_kv_heads * vdim), f"qkv_prep: v_src {tuple(v_src.shape)} is not [T, {num_kv_heads * vdim}]")
        _cuda(v_lambda, "qkv_prep v_lambda", torch.float32)
        _need(v_lambda.numel() == 1, "qkv_prep: v_lambda is one number")
    lib = build.load("attention_ext")
    rc = lib.rl_qkv_prep(
        _p(qkv), c_int(_dt(qkv, "qkv_prep")), c_int(stride), _p(bias), _p(tok_pos), _p(tok_seq), _p(block_table), c_int(block_table.shape[1]),
        _p(k_pages), _p(v_pages), _p(inv_freq if rotary_dim else None), c_float(magnitude), _p(q_norm), _p(k_norm), c_float(norm_eps), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(rotary_dim), c_int(1 if interleaved else 0), c_int(PAGE_SIZE),
        _p(v_src), c_int(vs_stride), _p(v_lambda), _stream(),
    )
    _check(lib, rc, "qkv_prep")


def attn_ext(
    q: torch.Tensor, k_pages, v_pages, block_table, tok_seq, tok_pos, num_heads: int, num_kv_heads: int, kdim: int, vdim: int,
    scale: float, window: int = 0, sink: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None, out_scale: float = 1.0, out: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0,
) -> torch.Tensor:
    """Attention of each token over its sequence's cached keys, both element types, prompts and decoding.

    window: 0, or how many of the last positions a query sees.  chunk: 0, or the size of the chunks (counted from position 0)
    outside of which a query sees nothing.  softcap: 0, or the cap c of s <- c tanh(s / c) on the scaled scores.

    q: [T, >= H kdim] rows.  sink: float32 [H] or None.  mix: float32 [H, H] or None (scores of the heads are mixed before the
    softmax).  gate: [T, >= H vdim] rows of q's type or None: the result is multiplied by sigmoid(gate).  out: [T, H vdim] rows
    (a strided view is taken as it is)."""
    _cuda(q, "attn_ext q", contiguous=False)
    qs = _rows(q, "attn_ext q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * kdim, "attn_ext: q rows too short")
    _check_kv_pages(k_pages, v_pages, q.dtype, num_kv_heads, kdim, vdim, "attn_ext")
    _cuda(block_table, "attn_ext block_table", torch.int32)
    _cuda(tok_seq, "attn_ext tok_seq", torch.int32)
    _cuda(tok_pos, "attn_ext tok_pos", torch.int32)
    _need(tok_seq.numel() == T and tok_pos.numel() == T and block_table.dim() == 2, "attn_ext: metadata sizes")
    if sink is not None:
        _cuda(sink, "attn_ext sink", torch.float32)
        _need(sink.numel() == num_heads, "attn_ext: one sink per head")
    if mix is not None:
        _cuda(mix, "attn_ext mix", torch.float32)
        _need(tuple(mix.shape) == (num_heads, num_heads), "attn_ext: the mixing matrix must be [H, H]")
    gs = 0
    if gate is not None:
        _cuda(gate, "attn_ext gate", q.dtype, contiguous=False)
        gs = _rows(gate, "attn_ext gate")
        _need(gate.shape[0] == T and gate.shape[1] >= num_heads * vdim, "attn_ext: gate rows too short")
    if out is None:
        out = torch.empty((T, num_heads * vdim), dtype=q.dtype, device=q.device)
    _cuda(out, "attn_ext out", q.dtype, contiguous=False)
    _need(_rows(out, "attn_ext out") >= num_heads * vdim and tuple(out.shape) == (T, num_heads * vdim), "attn_ext: out must be [T, H vdim]")
    lib = build.load("attention_ext")
    rc = lib.rl_attn_ext(
        _p(q), c_int(_dt(q, "attn_ext")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(tok_seq),
        _p(tok_pos), _p(sink), _p(mix), _p(gate), c_int(gs), c_float(out_scale), _p(out), c_int(out.stride(0)), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(PAGE_SIZE), c_int(window), c_float(scale), c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "attn_ext")
    return out


def sigmoid_attn(
    q: torch.Tensor, k_pages, v_pages, block_table, tok_seq, tok_pos, num_heads: int, num_kv_heads: int, kdim: int, vdim: int,
    scale: float, head_bias: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
    softcap: float = 0.0, window: int = 0, chunk: int = 0, out_scale: float = 1.0, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Attention without a softmax: a visible key's weight is logistic(cap(q . k * scale) + head_bias[h]), nothing is normalised
    over the keys; the heads' weights are mixed by `mix` (w'_h = sum_g mix[h][g] w_g) before head h applies them to the values of
    its kv head; the result of head h is multiplied by logistic(gate[t, h]) and `out_scale`.  Both element types, prompts and
    single tokens, every size; each output is one 32-bit sum in a fixed order.

    q: [T, >= H kdim] rows.  head_bias: float32 [H] or None.  mix: float32 [H, H] or None.  gate: [T, >= H] rows of q's type or
    None.  window, chunk, softcap: as in `attn_ext`.  out: [T, H vdim] rows (a strided view is taken as it is)."""
    _cuda(q, "sigmoid_attn q", contiguous=False)
    qs = _rows(q, "sigmoid_attn q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * kdim, "sigmoid_attn: q rows too short")
    _check_kv_pages(k_pages, v_pages, q.dtype, num_kv_heads, kdim, vdim, "sigmoid_attn")
    _cuda(block_table, "sigmoid_attn block_table", torch.int32)
    _cuda(tok_seq, "sigmoid_attn tok_seq", torch.int32)
    _cuda(tok_pos, "sigmoid_attn tok_pos", torch.int32)
    _need(tok_seq.numel() == T and tok_pos.numel() == T and block_table.dim() == 2, "sigmoid_attn: metadata sizes")
    if head_bias is not None:
        _cuda(head_bias, "sigmoid_attn head_bias", torch.float32)
        _need(head_bias.numel() == num_heads, "sigmoid_attn: one bias per head")
    if mix is not None:
        _cuda(mix, "sigmoid_attn mix", torch.float32)
        _need(tuple(mix.shape) == (num_heads, num_heads), "sigmoid_attn: the mixing matrix must be [H, H]")
    gs = 0
    if gate is not None:
        _cuda(gate, "sigmoid_attn gate", q.dtype, contiguous=False)
        gs = _rows(gate, "sigmoid_attn gate")
        _need(gate.shape[0] == T and gate.shape[1] >= num_heads, "sigmoid_attn: gate rows too short")
    if out is None:
        out = torch.empty((T, num_heads * vdim), dtype=q.dtype, device=q.device)
    _cuda(out, "sigmoid_attn out", q.dtype, contiguous=False)
    _need(_rows(out, "sigmoid_attn out") >= num_heads * vdim and tuple(out.shape) == (T, num_heads * vdim), "sigmoid_attn: out must be [T, H vdim]")
    lib = build.load("attention_sigmoid")
    rc = lib.rl_sigmoid_attn(
        _p(q), c_int(_dt(q, "sigmoid_attn")), c_int(qs), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(tok_seq),
        _p(tok_pos), _p(head_bias), _p(mix), _p(gate), c_int(gs), c_float(out_scale), _p(out), c_int(out.stride(0)), c_int(T), c_int(num_heads),
        c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(PAGE_SIZE), c_int(window), c_float(scale), c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "sigmoid_attn")
    return out


def sigmoid_attn_mma_takes(kdim: int, vdim: int, num_heads: int) -> bool:
    """Whether the tensor-core form of the attention with logistic weights is built for these sizes (bfloat16 only)."""
    return kdim % 8 == 0 and vdim % 8 == 0 and 0 < kdim <= 128 and 0 < vdim <= 128 and num_heads * vdim * 4 <= 48 * 1024


def sigmoid_attn_mma_scratch_floats(n_tokens: int, num_heads: int, num_kv_heads: int, vdim: int, mixed: bool, parts: int) -> int:
    return parts * n_tokens * num_heads * (num_kv_heads if mixed else 1) * vdim


def sigmoid_attn_mma(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int, num_kv_heads: int, kdim: int, vdim: int,
    scale: float, scratch: torch.Tensor, parts: int = 1, head_bias: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None, softcap: float = 0.0, window: int = 0, chunk: int = 0, out_scale: float = 1.0,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """`sigmoid_attn` on the tensor cores, bfloat16, key and value sizes in multiples of 8 up to 128: the sequences' query rows
    (tokens seq_start[i] .. seq_start[i+1] at positions seq_pos0[i] ..) against their cached keys.  parts: into how many runs
    of pages a block's key range is cut (more blocks for a decode step; the partial sums add up in the second kernel).
    scratch: float32, `sigmoid_attn_mma_scratch_floats(...)` numbers."""
    _cuda(q, "sigmoid_attn_mma q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "sigmoid_attn_mma q")
    T = q.shape[0]
    _need(q.shape[1] >= num_heads * kdim, "sigmoid_attn_mma: q rows too short")
    _need(sigmoid_attn_mma_takes(kdim, vdim, num_heads), f"sigmoid_attn_mma: sizes {kdim}, {vdim} with {num_heads} heads are not built")
    _check_kv_pages(k_pages, v_pages, q.dtype, num_kv_heads, kdim, vdim, "sigmoid_attn_mma")
    _cuda(block_table, "sigmoid_attn_mma block_table", torch.int32)
    _cuda(seq_start, "sigmoid_attn_mma seq_start", torch.int32)
    _cuda(seq_pos0, "sigmoid_attn_mma seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] == S, "sigmoid_attn_mma: metadata sizes")
    if head_bias is not None:
        _cuda(head_bias, "sigmoid_attn_mma head_bias", torch.float32)
        _need(head_bias.numel() == num_heads, "sigmoid_attn_mma: one bias per head")
    if mix is not None:
        _cuda(mix, "sigmoid_attn_mma mix", torch.float32)
        _need(tuple(mix.shape) == (num_heads, num_heads), "sigmoid_attn_mma: the mixing matrix must be [H, H]")
    gs = 0
    if gate is not None:
        _cuda(gate, "sigmoid_attn_mma gate", q.dtype, contiguous=False)
        gs = _rows(gate, "sigmoid_attn_mma gate")
        _need(gate.shape[0] == T and gate.shape[1] >= num_heads, "sigmoid_attn_mma: gate rows too short")
    _cuda(scratch, "sigmoid_attn_mma scratch", torch.float32)
    _need(parts >= 1 and scratch.numel() >= sigmoid_attn_mma_scratch_floats(T, num_heads, num_kv_heads, vdim, mix is not None, parts),
          "sigmoid_attn_mma: scratch too small")
    if out is None:
        out = torch.empty((T, num_heads * vdim), dtype=q.dtype, device=q.device)
    _cuda(out, "sigmoid_attn_mma out", q.dtype, contiguous=False)
    _need(_rows(out, "sigmoid_attn_mma out") >= num_heads * vdim and tuple(out.shape) == (T, num_heads * vdim), "sigmoid_attn_mma: out must be [T, H vdim]")
    lib = build.load("attention_sigmoid")
    rc = lib.rl_sigmoid_attn_mma(
        _p(q), c_ll(qs), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(seq_start), _p(seq_pos0), _p(head_bias), _p(mix),
        _p(gate), c_int(gs), c_float(out_scale), _p(scratch), c_int(parts), _p(out), c_int(out.stride(0)), c_int(T), c_int(S), c_int(max_q_len),
        c_int(num_heads), c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(window), c_float(scale), c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "sigmoid_attn_mma", kernels=2)
    return out


# ------------------------------------------------------------------ recurrent mixers (csrc/recurrent.cu)
DECAY_CHUNK = 64  # tokens per chunk of the chunked kernels
DECAY_CHUNKED_MAX_DIM = 256


def decay_attn_chunked_scratch_floats(n_seqs: int, max_q_len: int, num_heads: int, dim: int, vdim: int) -> int:
    return n_seqs * num_heads * ((max_q_len + DECAY_CHUNK - 1) // DECAY_CHUNK) * dim * vdim


def decay_attn(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, slot_ids: torch.Tensor,
    seq_start: torch.Tensor, num_heads: int, dim: int, vdim: int, silu: bool = False, out: Optional[torch.Tensor] = None,
    max_q_len: int = 0, scratch: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Linear attention with a decay per head, S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, through the sequences' states.

    max_q_len, scratch: 0 / None = token by token (equal bits for every cut of a sequence).  With the most tokens that a sequence
    of the step brings and a float32 scratch of `decay_attn_chunked_scratch_floats(...)`, the sequences are worked chunk by chunk,
    all chunks side by side (equal within rounding; key sizes up to 256).

    q, k: [T, H dim], v: [T, H vdim], views of one projection's rows (equal row strides).  decay: float32 [H].
    state: float32 [slots, H, dim, vdim]; sequence i of the step owns state[slot_ids[i]] and the tokens seq_start[i] .. seq_start[i+1].
    silu: the activation is applied to q, k and v as they are read.  Returns float32 [T, H vdim]."""
    for name, t, n in (("q", q, num_heads * dim), ("k", k, num_heads * dim), ("v", v, num_heads * vdim)):
        _cuda(t, f"decay_attn {name}", q.dtype, contiguous=False)
        _need(_rows(t, f"decay_attn {name}") == q.stride(0) and t.shape[1] == n and t.shape[0] == q.shape[0], f"decay_attn: {name} has the wrong shape or stride")
    T = q.shape[0]
    _cuda(decay, "decay_attn decay", torch.float32)
    _need(decay.numel() == num_heads, "decay_attn: one decay per head")
    _cuda(state, "decay_attn state", torch.float32)
    _need(state.dim() == 4 and tuple(state.shape[1:]) == (num_heads, dim, vdim), f"decay_attn: state {tuple(state.shape)} is not [slots, {num_heads}, {dim}, {vdim}]")
    _cuda(slot_ids, "decay_attn slot_ids", torch.int32)
    _cuda(seq_start, "decay_attn seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "decay_attn: seq_start must hold one more entry than there are sequences")
    if out is None:
        out = torch.empty((T, num_heads * vdim), dtype=torch.float32, device=q.device)
    _cuda(out, "decay_attn out", torch.float32)
    _need(tuple(out.shape) == (T, num_heads * vdim), "decay_attn: out has the wrong shape")
    lib = build.load("recurrent")
    if max_q_len > 0 and scratch is not None:
        _cuda(scratch, "decay_attn scratch", torch.float32)
        _need(dim <= DECAY_CHUNKED_MAX_DIM, f"decay_attn: the chunked kernels take key sizes up to {DECAY_CHUNKED_MAX_DIM}")
        _need(scratch.numel() >= decay_attn_chunked_scratch_floats(S, max_q_len, num_heads, dim, vdim), "decay_attn: scratch too small")
        rc = lib.rl_decay_attn_chunked(
            _p(q), _p(k), _p(v), c_int(_dt(q, "decay_attn")), c_int(q.stride(0)), _p(decay), _p(state), _p(slot_ids), _p(seq_start), _p(scratch),
            _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len), c_int(num_heads), c_int(dim), c_int(vdim), c_int(1 if silu else 0), _stream(),
        )
        _check(lib, rc, "decay_attn_chunked", kernels=3)
        return out
    rc = lib.rl_decay_attn(
        _p(q), _p(k), _p(v), c_int(_dt(q, "decay_attn")), c_int(q.stride(0)), _p(decay), _p(state), _p(slot_ids), _p(seq_start), _p(out),
        c_int(out.stride(0)), c_int(S), c_int(num_heads), c_int(dim), c_int(vdim), c_int(1 if silu else 0), _stream(),
    )
    _check(lib, rc, "decay_attn")
    return out


def rms_gate(
    x: torch.Tensor, weight: torch.Tensor, eps: float, gate: Optional[torch.Tensor], act_dtype: torch.dtype, out_scale: float = 1.0,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out = x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate) * out_scale over rows; x float32 [T, n], gate [T, >= n] rows of
    `act_dtype` or None, out [T, n] rows of `act_dtype` (a strided view is taken as it is)."""
    _cuda(x, "rms_gate x", torch.float32, contiguous=False)
    xs = _rows(x, "rms_gate x")
    T, n = x.shape
    _cuda(weight, "rms_gate weight")
    _need(tuple(weight.shape) == (n,), "rms_gate: weight does not match the rows")
    gs = 0
    if gate is not None:
        _cuda(gate, "rms_gate gate", act_dtype, contiguous=False)
        gs = _rows(gate, "rms_gate gate")
        _need(gate.shape[0] == T and gate.shape[1] >= n, "rms_gate: gate rows too short")
    if out is None:
        out = torch.empty((T, n), dtype=act_dtype, device=x.device)
    _cuda(out, "rms_gate out", act_dtype, contiguous=False)
    _need(tuple(out.shape) == (T, n) and _rows(out, "rms_gate out") >= n, "rms_gate: out must be [T, n]")
    lib = build.load("recurrent")
    rc = lib.rl_rms_gate(
        _p(x), c_int(xs), _p(weight), c_int(_dt(weight, "rms_gate weight")), c_float(eps), _p(gate), c_int(gs), c_float(out_scale), _p(out),
        c_int(out.stride(0)), c_int(_DT[act_dtype]), c_int(T), c_int(n), _stream(),
    )
    _check(lib, rc, "rms_gate")
    return out


def min_gru(
    z: torch.Tensor, x: torch.Tensor, g: torch.Tensor, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor], state: torch.Tensor,
    slot_ids: torch.Tensor, seq_start: torch.Tensor, out_scale: float = 1.0, out: Optional[torch.Tensor] = None, max_q_len: int = 0,
) -> torch.Tensor:
    """Element by element S_t = (1 - z_t) S_(t-1) + z_t c_t with z_t = sigmoid(z + z_bias), u = x + x_bias,
    c = u + 1/2 where u >= 0 else sigmoid(u); returns S_t * silu(g) * out_scale in the inputs' type.

    max_q_len: 0 = token by token (equal bits for every cut of a sequence); the most tokens a sequence of the step brings = long
    sequences are cut into stretches that run side by side (equal within rounding).

    z, x, g: [T, width] views of one projection's rows (equal row strides).  state: float32 [slots, width]."""
    T, width = z.shape
    for name, t in (("z", z), ("x", x), ("g", g)):
        _cuda(t, f"min_gru {name}", z.dtype, contiguous=False)
        _need(_rows(t, f"min_gru {name}") == z.stride(0) and tuple(t.shape) == (T, width), f"min_gru: {name} has the wrong shape or stride")
    for name, b in (("z_bias", z_bias), ("x_bias", x_bias)):
        if b is not None:
            _cuda(b, f"min_gru {name}", torch.float32)
            _need(b.numel() == width, f"min_gru: {name} does not match the width")
    _cuda(state, "min_gru state", torch.float32)
    _need(state.dim() == 2 and state.shape[1] == width, f"min_gru: state {tuple(state.shape)} is not [slots, {width}]")
    _cuda(slot_ids, "min_gru slot_ids", torch.int32)
    _cuda(seq_start, "min_gru seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "min_gru: seq_start must hold one more entry than there are sequences")
    if out is None:
        out = torch.empty((T, width), dtype=z.dtype, device=z.device)
    _cuda(out, "min_gru out", z.dtype, contiguous=False)
    _need(tuple(out.shape) == (T, width) and _rows(out, "min_gru out") >= width, "min_gru: out must be [T, width]")
    lib = build.load("recurrent")
    rc = lib.rl_min_gru(
        _p(z), _p(x), _p(g), c_int(_dt(z, "min_gru")), c_int(z.stride(0)), _p(z_bias), _p(x_bias), _p(state), _p(slot_ids), _p(seq_start),
        c_float(out_scale), _p(out), c_int(out.stride(0)), c_int(S), c_int(width), c_int(max_q_len), _stream(),
    )
    _check(lib, rc, "min_gru")
    return out


# ------------------------------------------------------------------ recurrences with gates per token (csrc/gated_recurrent.cu)
def gla_log_decay(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """log a = logsigmoid(z + bias) / tau as float32 [T, n]; z: [T, n] rows of the run's type (a strided view is taken as it is)."""
    _cuda(z, "gla_log_decay z", contiguous=False)
    zs = _rows(z, "gla_log_decay z")
    T, n = z.shape
    if bias is not None:
        _cuda(bias, "gla_log_decay bias", torch.float32)
        _need(bias.numel() == n, "gla_log_decay: one bias per column")
    out = torch.empty((T, n), dtype=torch.float32, device=z.device)
    lib = build.load("gated_recurrent")
    rc = lib.rl_gla_log_decay(_p(z), c_int(_dt(z, "gla_log_decay")), c_int(zs), _p(bias), c_float(tau), _p(out), c_int(T), c_int(n), _stream())
    _check(lib, rc, "gla_log_decay")
    return out


def mlstm_gates(
    gi: torch.Tensor, gf: torch.Tensor, bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor], cap: float, m_state: torch.Tensor,
    slot_ids: torch.Tensor, seq_start: torch.Tensor, scan: bool = False,
):
    """The gates of a matrix memory.  gi, gf: [T, H] views of one projection's rows (the raw input and forget gates); biases float32 [H].
    With i = cap tanh((gi + b_i) / cap), f = logsigmoid(cap tanh((gf + b_f) / cap)) and the running maximum m_t = max(f_t + m_(t-1), i_t)
    carried in m_state float32 [slots, H]: returns (log_a = f + m_(t-1) - m_t, b = exp(i - m_t), m), each float32 [T, H].
    scan: 256 tokens of a sequence at a time, their maps m -> max(m + f, i) composed by a scan (long prompts; equal within rounding);
    else token after token (equal bits however a sequence is cut into steps)."""
    _cuda(gi, "mlstm_gates gi", contiguous=False)
    _cuda(gf, "mlstm_gates gf", gi.dtype, contiguous=False)
    stride = _rows(gi, "mlstm_gates gi")
    _need(_rows(gf, "mlstm_gates gf") == stride and gf.shape == gi.shape, "mlstm_gates: the two gates must be views of the same rows")
    T, H = gi.shape
    for name, b in (("bias_i", bias_i), ("bias_f", bias_f)):
        if b is not None:
            _cuda(b, f"mlstm_gates {name}", torch.float32)
            _need(b.numel() == H, "mlstm_gates: one bias per head")
    _cuda(m_state, "mlstm_gates m_state", torch.float32)
    _need(m_state.dim() == 2 and m_state.shape[1] == H, f"mlstm_gates: m_state {tuple(m_state.shape)} is not [slots, {H}]")
    _cuda(slot_ids, "mlstm_gates slot_ids", torch.int32)
    _cuda(seq_start, "mlstm_gates seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "mlstm_gates: seq_start must hold one more entry than there are sequences")
    log_a, b, m = (torch.empty((T, H), dtype=torch.float32, device=gi.device) for _ in range(3))
    lib = build.load("gated_recurrent")
    rc = lib.rl_mlstm_gates(
        _p(gi), _p(gf), c_int(_dt(gi, "mlstm_gates")), c_int(stride), _p(bias_i), _p(bias_f), c_float(cap), _p(m_state), _p(slot_ids),
        _p(seq_start), _p(log_a), _p(b), _p(m), c_int(S), c_int(H), c_int(1 if scan else 0), _stream(),
    )
    _check(lib, rc, "mlstm_gates")
    return log_a, b, m


def gated_attn(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_decay: torch.Tensor, in_scale: Optional[torch.Tensor], state: torch.Tensor,
    slot_ids: torch.Tensor, seq_start: torch.Tensor, num_heads: int, dim: int, vdim: int, q_scale: float = 1.0, ext: bool = False,
) -> torch.Tensor:
    """S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T, o_t = S_t^T (q_scale q_t) through the sequences' states, token by token.

    q, k: [T, H dim], v: [T, H vdim], views of one projection's rows.  log_decay: float32 [T, H dim] (a per key channel) or [T, H]
    (a per head), a = exp(log_decay).  in_scale: float32 [T, H] (b) or None (1).  ext: the state has one more column, fed with
    v = 1, and so has the result.  state: float32 [slots, H, dim, vdim (+1)].  Returns float32 [T, H (vdim (+1))]."""
    for name, t, n in (("q", q, num_heads * dim), ("k", k, num_heads * dim), ("v", v, num_heads * vdim)):
        _cuda(t, f"gated_attn {name}", q.dtype, contiguous=False)
        _need(_rows(t, f"gated_attn {name}") == q.stride(0) and t.shape[1] == n and t.shape[0] == q.shape[0], f"gated_attn: {name} has the wrong shape or stride")
    T = q.shape[0]
    vcols = vdim + (1 if ext else 0)
    _cuda(log_decay, "gated_attn log_decay", torch.float32)
    per_channel = log_decay.numel() == T * num_heads * dim
    _need(per_channel or log_decay.numel() == T * num_heads, f"gated_attn: log_decay {tuple(log_decay.shape)} is neither [T, H dim] nor [T, H]")
    if in_scale is not None:
        _cuda(in_scale, "gated_attn in_scale", torch.float32)
        _need(in_scale.numel() == T * num_heads, "gated_attn: in_scale must be [T, H]")
    _cuda(state, "gated_attn state", torch.float32)
    _need(state.dim() == 4 and tuple(state.shape[1:]) == (num_heads, dim, vcols), f"gated_attn: state {tuple(state.shape)} is not [slots, {num_heads}, {dim}, {vcols}]")
    _cuda(slot_ids, "gated_attn slot_ids", torch.int32)
    _cuda(seq_start, "gated_attn seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "gated_attn: seq_start must hold one more entry than there are sequences")
    out = torch.empty((T, num_heads * vcols), dtype=torch.float32, device=q.device)
    lib = build.load("gated_recurrent")
    rc = lib.rl_gated_attn(
        _p(q), _p(k), _p(v), c_int(_dt(q, "gated_attn")), c_int(q.stride(0)), _p(log_decay), c_int(1 if per_channel else 0), _p(in_scale),
        c_float(q_scale), _p(state), _p(slot_ids), _p(seq_start), _p(out), c_int(out.stride(0)), c_int(S), c_int(num_heads), c_int(dim),
        c_int(vdim), c_int(1 if ext else 0), _stream(),
    )
    _check(lib, rc, "gated_attn")
    return out


GATED_CHUNK = 64  # tokens per chunk of the chunked recurrence


def gated_attn_chunked_takes(dim: int, vcols: int) -> bool:
    """Whether the chunked form of `gated_attn` is built for these sizes (its last kernel keeps three [64, dim + 1] tiles in shared memory)."""
    tile, later = GATED_CHUNK * (dim + 1), GATED_CHUNK * 64 + GATED_CHUNK * (GATED_CHUNK + 1)
    return dim > 0 and (2 * tile + max(tile, later) + 5 * dim + GATED_CHUNK * 4) * 4 <= 227 * 1024


def gated_attn_chunked_scratch_floats(n_seqs: int, max_q_len: int, num_heads: int, dim: int, vcols: int) -> int:
    """Floats of scratch that `gated_attn_chunked` needs: a [dim, vcols] matrix and a row of dim decays per (sequence, head, chunk)."""
    return n_seqs * num_heads * ((max_q_len + GATED_CHUNK - 1) // GATED_CHUNK) * dim * (vcols + 1)


def gated_attn_chunked(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_decay: torch.Tensor, in_scale: Optional[torch.Tensor], state: torch.Tensor,
    slot_ids: torch.Tensor, seq_start: torch.Tensor, num_heads: int, dim: int, vdim: int, max_q_len: int, scratch: torch.Tensor,
    q_scale: float = 1.0, ext: bool = False,
) -> torch.Tensor:
    """`gated_attn` chunk by chunk (64 tokens, all chunks side by side, 32-bit arithmetic): equal within rounding, for prompts.
    max_q_len: the most tokens a sequence of the step brings; scratch: float32, at least `gated_attn_chunked_scratch_floats(...)`."""
    for name, t, n in (("q", q, num_heads * dim), ("k", k, num_heads * dim), ("v", v, num_heads * vdim)):
        _cuda(t, f"gated_attn_chunked {name}", q.dtype, contiguous=False)
        _need(_rows(t, f"gated_attn_chunked {name}") == q.stride(0) and t.shape[1] == n and t.shape[0] == q.shape[0], f"gated_attn_chunked: {name} has the wrong shape or stride")
    T = q.shape[0]
    vcols = vdim + (1 if ext else 0)
    _need(gated_attn_chunked_takes(dim, vcols), f"gated_attn_chunked: key size {dim} is too large for the chunked kernels")
    _cuda(log_decay, "gated_attn_chunked log_decay", torch.float32)
    per_channel = log_decay.numel() == T * num_heads * dim
    _need(per_channel or log_decay.numel() == T * num_heads, f"gated_attn_chunked: log_decay {tuple(log_decay.shape)} is neither [T, H dim] nor [T, H]")
    if in_scale is not None:
        _cuda(in_scale, "gated_attn_chunked in_scale", torch.float32)
        _need(in_scale.numel() == T * num_heads, "gated_attn_chunked: in_scale must be [T, H]")
    _cuda(state, "gated_attn_chunked state", torch.float32)
    _need(state.dim() == 4 and tuple(state.shape[1:]) == (num_heads, dim, vcols), f"gated_attn_chunked: state {tuple(state.shape)} is not [slots, {num_heads}, {dim}, {vcols}]")
    _cuda(slot_ids, "gated_attn_chunked slot_ids", torch.int32)
    _cuda(seq_start, "gated_attn_chunked seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "gated_attn_chunked: seq_start must hold one more entry than there are sequences")
    _cuda(scratch, "gated_attn_chunked scratch", torch.float32)
    _need(max_q_len >= 1 and scratch.numel() >= gated_attn_chunked_scratch_floats(S, max_q_len, num_heads, dim, vcols), "gated_attn_chunked: scratch too small")
    out = torch.empty((T, num_heads * vcols), dtype=torch.float32, device=q.device)
    lib = build.load("gated_recurrent")
    rc = lib.rl_gated_attn_chunked(
        _p(q), _p(k), _p(v), c_int(_dt(q, "gated_attn_chunked")), c_int(q.stride(0)), _p(log_decay), c_int(1 if per_channel else 0), _p(in_scale),
        c_float(q_scale), _p(state), _p(slot_ids), _p(seq_start), _p(scratch), _p(out), c_int(out.stride(0)), c_int(S), c_int(max_q_len),
        c_int(num_heads), c_int(dim), c_int(vdim), c_int(1 if ext else 0), _stream(),
    )
    _check(lib, rc, "gated_attn_chunked", kernels=3)
    return out


GATE_NONE, GATE_SIGMOID, GATE_SILU = 0, 1, 2


def head_norm_gate(
    x: torch.Tensor, num_heads: int, n: int, weight: Optional[torch.Tensor], eps: float, gate: Optional[torch.Tensor], gate_act: int,
    act_dtype: torch.dtype, m: Optional[torch.Tensor] = None, den_eps: float = 0.0, out_scale: float = 1.0, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Per (row, head): y = v / sqrt(mean(v^2) + eps) * weight * act(gate) * out_scale over the head's n values.

    x: float32 [T, H xh] with xh = n, or n + 1 when m (float32 [T, H]) is given: the head's last number is then its n . q and
    v = x / (max(|n . q|, exp(-m)) + den_eps).  weight: float32 [n] (shared by the heads), [H n] or None.  gate: [T, >= H n] rows of
    `act_dtype` or None; gate_act: GATE_NONE (the gate itself), GATE_SIGMOID, GATE_SILU.  out: [T, H n] rows of `act_dtype`."""
    _cuda(x, "head_norm_gate x", torch.float32, contiguous=False)
    xs = _rows(x, "head_norm_gate x")
    T = x.shape[0]
    xh = n + (1 if m is not None else 0)
    _need(x.shape[1] == num_heads * xh, f"head_norm_gate: x {tuple(x.shape)} is not [T, {num_heads} * {xh}]")
    per_head = 0
    if weight is not None:
        _cuda(weight, "head_norm_gate weight", torch.float32)
        _need(weight.numel() in (n, num_heads * n), "head_norm_gate: weight must hold n or H n numbers")
        per_head = 1 if (weight.numel() == num_heads * n and num_heads > 1) else 0
    if m is not None:
        _cuda(m, "head_norm_gate m", torch.float32)
        _need(m.numel() == T * num_heads, "head_norm_gate: m must be [T, H]")
    gs = 0
    if gate is not None:
        _cuda(gate, "head_norm_gate gate", act_dtype, contiguous=False)
        gs = _rows(gate, "head_norm_gate gate")
        _need(gate.shape[0] == T and gate.shape[1] >= num_heads * n, "head_norm_gate: gate rows too short")
    if out is None:
        out = torch.empty((T, num_heads * n), dtype=act_dtype, device=x.device)
    _cuda(out, "head_norm_gate out", act_dtype, contiguous=False)
    _need(tuple(out.shape) == (T, num_heads * n) and _rows(out, "head_norm_gate out") >= num_heads * n, "head_norm_gate: out must be [T, H n]")
    lib = build.load("gated_recurrent")
    rc = lib.rl_head_norm_gate(
        _p(x), c_int(xs), c_int(xh), _p(m), c_float(den_eps), _p(weight), c_int(per_head), c_float(eps), _p(gate), c_int(gs), c_int(gate_act),
        c_float(out_scale), _p(out), c_int(out.stride(0)), c_int(_DT[act_dtype]), c_int(T), c_int(num_heads), c_int(n), _stream(),
    )
    _check(lib, rc, "head_norm_gate")
    return out



# ------------------------------------------------------------------ gated delta rule (csrc/delta_rule.cu)
SHORT_CONV_MAX_TAPS = 16
DELTA_RULE_MAX_DIM = 256


def short_conv(
    x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], slot_ids: torch.Tensor, seq_start: torch.Tensor, tok_seq: torch.Tensor,
    silu: bool = True,
) -> torch.Tensor:
    """y[t, c] = act(sum_i w[i, c] x[t - taps + 1 + i, c]) over each sequence's tokens, a causal convolution over time per channel.

    x: [T, C] rows (a view of a projection's rows is taken as it is).  w: float32 [taps, C] (tap i of every channel side by side,
    so that neighbouring channels read neighbouring weights), the last row the current token's.
    state: float32 [slots, taps - 1, C], the last taps - 1 inputs of every sequence before this step (zeros at a sequence's
    start); it is moved on to the end of the step's tokens.  Returns [T, C] in x's type."""
    _cuda(x, "short_conv x", contiguous=False)
    xs = _rows(x, "short_conv x")
    T, C = x.shape
    _cuda(w, "short_conv w", torch.float32)
    _need(w.dim() == 2 and w.shape[1] == C, f"short_conv: w {tuple(w.shape)} does not have {C} columns")
    taps = w.shape[0]
    _need(1 <= taps <= SHORT_CONV_MAX_TAPS, f"short_conv: {taps} taps (1 to {SHORT_CONV_MAX_TAPS})")
    _cuda(slot_ids, "short_conv slot_ids", torch.int32)
    _cuda(seq_start, "short_conv seq_start", torch.int32)
    _cuda(tok_seq, "short_conv tok_seq", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1 and tok_seq.numel() == T, "short_conv: metadata sizes")
    if taps > 1:
        _cuda(state, "short_conv state", torch.float32)
        _need(state.dim() == 3 and tuple(state.shape[1:]) == (taps - 1, C), f"short_conv: state {tuple(state.shape)} is not [slots, {taps - 1}, {C}]")
    out = torch.empty((T, C), dtype=x.dtype, device=x.device)
    lib = build.load("delta_rule")
    rc = lib.rl_short_conv(
        _p(x), c_int(_dt(x, "short_conv")), c_int(xs), _p(w), _p(state if taps > 1 else None), _p(slot_ids), _p(seq_start), _p(tok_seq), _p(out),
        c_int(out.stride(0)), c_int(T), c_int(S), c_int(C), c_int(taps), c_int(1 if silu else 0), _stream(),
    )
    _check(lib, rc, "short_conv", kernels=2 if taps > 1 else 1)
    return out


def delta_prep(
    qk: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, num_qk_heads: int, num_heads: int, dim: int,
    unit_eps: float, q_scale: float,
):
    """What the gated delta rule's recurrence takes, all float32: qk [T, 2 G dim] rows (G q heads, then G k heads) -> unit vectors
    qn (times q_scale) and kn [T, G dim], their products kq [T, G]; ba [T, >= 2 H] rows (b, then a) -> beta = logistic(b) and
    decay = exp(-exp(a_log) softplus(a + dt_bias)), both [T, H]."""
    _cuda(qk, "delta_prep qk", contiguous=False)
    _cuda(ba, "delta_prep ba", qk.dtype, contiguous=False)
    T = qk.shape[0]
    G, H = num_qk_heads, num_heads
    _need(qk.shape[1] == 2 * G * dim and ba.shape[0] == T and ba.shape[1] >= 2 * H, "delta_prep: row sizes")
    _cuda(a_log, "delta_prep a_log", torch.float32)
    _cuda(dt_bias, "delta_prep dt_bias", torch.float32)
    _need(a_log.numel() == H and dt_bias.numel() == H, "delta_prep: one A_log and one dt_bias per head")
    f32 = dict(dtype=torch.float32, device=qk.device)
    qn, kn = torch.empty((T, G * dim), **f32), torch.empty((T, G * dim), **f32)
    kq, beta, decay = torch.empty((T, G), **f32), torch.empty((T, H), **f32), torch.empty((T, H), **f32)
    lib = build.load("delta_rule")
    rc = lib.rl_delta_prep(
        _p(qk), c_int(_dt(qk, "delta_prep")), c_int(_rows(qk, "delta_prep qk")), _p(ba), c_int(_rows(ba, "delta_prep ba")), _p(a_log), _p(dt_bias),
        c_float(unit_eps), c_float(q_scale), _p(qn), _p(kn), _p(kq), _p(beta), _p(decay), c_int(T), c_int(G), c_int(H), c_int(dim), _stream(),
    )
    _check(lib, rc, "delta_prep")
    return qn, kn, kq, beta, decay


def delta_rule(
    qn: torch.Tensor, kn: torch.Tensor, kq: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
    slot_ids: torch.Tensor, seq_start: torch.Tensor, num_heads: int, num_qk_heads: int, dim: int, vdim: int,
) -> torch.Tensor:
    """The gated delta rule through the sequences' states, token by token: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  qn, kn: float32 [T, G dim]; kq = k . q: float32 [T, G]; v: [T, H vdim] rows of the run's type; beta, decay:
    float32 [T, H]; state: float32 [slots, H, dim, vdim].  Head h reads q/k head h // (H / G).  Returns float32 [T, H vdim]."""
    T = qn.shape[0]
    H, G = num_heads, num_qk_heads
    for name, t, n in (("qn", qn, G * dim), ("kn", kn, G * dim), ("kq", kq, G), ("beta", beta, H), ("decay", decay, H)):
        _cuda(t, f"delta_rule {name}", torch.float32)
        _need(tuple(t.shape) == (T, n), f"delta_rule: {name} {tuple(t.shape)} is not [{T}, {n}]")
    _cuda(v, "delta_rule v", contiguous=False)
    _need(tuple(v.shape) == (T, H * vdim), "delta_rule: v must be [T, H vdim]")
    _need(dim <= DELTA_RULE_MAX_DIM, f"delta_rule: key size {dim} exceeds {DELTA_RULE_MAX_DIM}")
    _cuda(state, "delta_rule state", torch.float32)
    _need(state.dim() == 4 and tuple(state.shape[1:]) == (H, dim, vdim), f"delta_rule: state {tuple(state.shape)} is not [slots, {H}, {dim}, {vdim}]")
    _cuda(slot_ids, "delta_rule slot_ids", torch.int32)
    _cuda(seq_start, "delta_rule seq_start", torch.int32)
    S = slot_ids.numel()
    _need(seq_start.numel() == S + 1, "delta_rule: seq_start must hold one more entry than there are sequences")
    out = torch.empty((T, H * vdim), dtype=torch.float32, device=qn.device)
    lib = build.load("delta_rule")
    rc = lib.rl_delta_rule(
        _p(qn), _p(kn), _p(kq), _p(v), c_int(_dt(v, "delta_rule v")), c_int(_rows(v, "delta_rule v")), _p(beta), _p(decay), _p(state), _p(slot_ids),
        _p(seq_start), _p(out), c_int(out.stride(0)), c_int(S), c_int(H), c_int(G), c_int(dim), c_int(vdim), _stream(),
    )
    _check(lib, rc, "delta_rule")
    return out


ACT_RELU2 = 1  # relu(x)^2


def unary_act(x: torch.Tensor, kind: int = ACT_RELU2) -> torch.Tensor:
    """y = f(x) element by element in 32-bit, stored in x's type."""
    _cuda(x, "unary_act x")
    out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    lib = build.load("recurrent")
    rc = lib.rl_unary_act(_p(x), _p(out), c_int(_dt(x, "unary_act")), c_ll(x.numel()), c_int(kind), _stream())
    _check(lib, rc, "unary_act")
    return out


# ------------------------------------------------------------------ tensor-core attention with options (csrc/attention_mix_mma.cu)
FLASH_MIX_SMEM_LIMIT = 227 * 1024


def flash_mix_takes(kdim: int, vdim: int, parts: int) -> bool:
    """Whether `flash_mix` is built for these sizes: multiples of 8 up to 256, and the query parts fit shared memory."""
    if kdim % 8 or vdim % 8 or max(kdim, vdim) > 256:
        return False
    hd = max(kdim, vdim)
    hd = 32 if hd <= 32 else 64 if hd <= 64 else 128 if hd <= 128 else 256
    return (3 * 64 + parts * 64) * (hd + 8) * 2 <= FLASH_MIX_SMEM_LIMIT


def fold_queries(q: torch.Tensor, mix: torch.Tensor, num_heads: int, num_kv_heads: int, kdim: int) -> torch.Tensor:
    """out[t, h, c, :] = sum over the heads g of kv head c of mix[h, g] * q[t, g, :] (32-bit sums, bfloat16 result): the queries
    with which head h's mixed score is one product against the keys of all kv heads side by side."""
    _cuda(q, "fold_queries q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "fold_queries q")
    _need(q.shape[1] >= num_heads * kdim, "fold_queries: q rows too short")
    _cuda(mix, "fold_queries mix", torch.float32)
    _need(tuple(mix.shape) == (num_heads, num_heads), "fold_queries: the mixing matrix must be [H, H]")
    T = q.shape[0]
    out = torch.empty((T, num_heads * num_kv_heads * kdim), dtype=torch.bfloat16, device=q.device)
    lib = build.load("attention_mix_mma")
    rc = lib.rl_fold_queries(_p(q), c_int(qs), _p(mix), _p(out), c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(kdim), _stream())
    _check(lib, rc, "fold_queries")
    return out


def flash_mix(
    q: torch.Tensor, k_pages, v_pages, block_table, seq_start, seq_pos0, max_q_len: int, num_heads: int, num_kv_heads: int, kdim: int,
    vdim: int, scale: float, window: int = 0, sink: Optional[torch.Tensor] = None, folded: bool = False, gate: Optional[torch.Tensor] = None,
    out_scale: float = 1.0, out: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0,
) -> torch.Tensor:
    """bfloat16 attention of a ragged batch over the paged cache on the tensor cores, keys of `kdim` and values of `vdim` numbers,
    with a window, chunks (a query sees the keys of its own chunk of positions only), capped scores (s <- c tanh(s / c)), a sink,
    a gate (out *= sigmoid(gate)) and a constant factor.  folded: q is what `fold_queries` made
    ([T, H K kdim]: the heads' scores are mixed); else q holds [T, >= H kdim] rows."""
    _cuda(q, "flash_mix q", torch.bfloat16, contiguous=False)
    qs = _rows(q, "flash_mix q")
    T = q.shape[0]
    parts = num_kv_heads if folded else 1
    _need(q.shape[1] >= num_heads * parts * kdim, "flash_mix: q rows too short")
    _need(flash_mix_takes(kdim, vdim, parts), f"flash_mix: sizes {kdim} / {vdim} with {parts} query parts are not built")
    _check_kv_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, kdim, vdim, "flash_mix")
    _cuda(block_table, "flash_mix block_table", torch.int32)
    _cuda(seq_start, "flash_mix seq_start", torch.int32)
    _cuda(seq_pos0, "flash_mix seq_pos0", torch.int32)
    S = seq_pos0.numel()
    _need(seq_start.numel() == S + 1 and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_mix: metadata sizes")
    _check_sink(sink, num_heads, "flash_mix")
    gs = 0
    if gate is not None:
        _cuda(gate, "flash_mix gate", torch.bfloat16, contiguous=False)
        gs = _rows(gate, "flash_mix gate")
        _need(gate.shape[0] == T and gate.shape[1] >= num_heads * vdim, "flash_mix: gate rows too short")
    if out is None:
        out = torch.empty((T, num_heads * vdim), dtype=torch.bfloat16, device=q.device)
    _cuda(out, "flash_mix out", torch.bfloat16, contiguous=False)
    _need(tuple(out.shape) == (T, num_heads * vdim) and _rows(out, "flash_mix out") >= num_heads * vdim, "flash_mix: out must be [T, H vdim]")
    lib = build.load("attention_mix_mma")
    rc = lib.rl_flash_mix(
        _p(q), c_ll(qs), c_int(parts * kdim), c_int(parts), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]),
        _p(seq_start), _p(seq_pos0), _p(sink), _p(gate), c_int(gs), c_float(out_scale), _p(out), c_int(out.stride(0)), c_int(S),
        c_int(max_q_len), c_int(num_heads), c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(PAGE_SIZE), c_int(window), c_float(scale),
        c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "flash_mix")
    return out


def flash_mix_decode_takes(num_heads: int, num_kv_heads: int, kdim: int, vdim: int) -> bool:
    """Whether `flash_mix_decode` (and `fold_queries` before it) is built for these sizes."""
    if kdim % 8 or vdim % 8 or max(kdim, vdim) > 256 or num_heads > 256:
        return False
    hd = max(kdim, vdim)
    hd = 32 if hd <= 32 else 64 if hd <= 64 else 128 if hd <= 128 else 256
    rows = (num_heads + 15) // 16 * 16
    return ((3 * 64 + num_kv_heads * rows) * (hd + 8) * 2 <= FLASH_MIX_SMEM_LIMIT
            and (num_heads * kdim + num_heads * num_heads) * 4 <= 48 * 1024)


def flash_mix_decode_scratch_floats(n_seqs: int, num_heads: int, vdim: int, n_splits: int) -> int:
    return n_seqs * num_heads * n_splits * (vdim + 2)


def flash_mix_decode(
    qf: torch.Tensor, k_pages, v_pages, block_table, seq_pos0, num_heads: int, num_kv_heads: int, kdim: int, vdim: int, scale: float,
    n_splits: int, scratch: torch.Tensor, window: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
    out_scale: float = 1.0, out: Optional[torch.Tensor] = None, chunk: int = 0, softcap: float = 0.0,
) -> torch.Tensor:
    """One query token per sequence, at position seq_pos0[s], over its sequence's cached keys (its own among them), the key range
    cut into `n_splits` parts; a block's rows are the heads.  qf: folded queries [S, H K kdim] (`fold_queries`, with the identity
    matrix for an attention without mixing).  scratch: float32, `flash_mix_decode_scratch_floats(...)`."""
    _cuda(qf, "flash_mix_decode qf", torch.bfloat16)
    S = qf.shape[0]
    _need(qf.dim() == 2 and qf.shape[1] == num_heads * num_kv_heads * kdim, "flash_mix_decode: qf must be [S, H K kdim]")
    _need(flash_mix_decode_takes(num_heads, num_kv_heads, kdim, vdim), f"flash_mix_decode: sizes {num_heads} / {num_kv_heads} / {kdim} / {vdim} are not built")
    _check_kv_pages(k_pages, v_pages, torch.bfloat16, num_kv_heads, kdim, vdim, "flash_mix_decode")
    _cuda(block_table, "flash_mix_decode block_table", torch.int32)
    _cuda(seq_pos0, "flash_mix_decode seq_pos0", torch.int32)
    _need(seq_pos0.numel() == S and block_table.dim() == 2 and block_table.shape[0] >= S, "flash_mix_decode: metadata sizes")
    _need(1 <= n_splits <= 256, f"flash_mix_decode: {n_splits} splits")
    _check_sink(sink, num_heads, "flash_mix_decode")
    _cuda(scratch, "flash_mix_decode scratch", torch.float32)
    _need(scratch.numel() >= flash_mix_decode_scratch_floats(S, num_heads, vdim, n_splits), "flash_mix_decode: scratch too small")
    gs = 0
    if gate is not None:
        _cuda(gate, "flash_mix_decode gate", torch.bfloat16, contiguous=False)
        gs = _rows(gate, "flash_mix_decode gate")
        _need(gate.shape[0] == S and gate.shape[1] >= num_heads * vdim, "flash_mix_decode: gate rows too short")
    if out is None:
        out = torch.empty((S, num_heads * vdim), dtype=torch.bfloat16, device=qf.device)
    _cuda(out, "flash_mix_decode out", torch.bfloat16, contiguous=False)
    _need(tuple(out.shape) == (S, num_heads * vdim) and _rows(out, "flash_mix_decode out") >= num_heads * vdim, "flash_mix_decode: out must be [S, H vdim]")
    n_o = S * num_heads * n_splits * vdim
    lib = build.load("attention_mix_mma")
    rc = lib.rl_flash_mix_decode(
        _p(qf), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]), _p(seq_pos0), _p(sink), _p(gate), c_int(gs),
        c_float(out_scale), c_void_p(scratch.data_ptr()), c_void_p(scratch.data_ptr() + 4 * n_o), _p(out), c_int(out.stride(0)), c_int(S),
        c_int(num_heads), c_int(num_kv_heads), c_int(kdim), c_int(vdim), c_int(PAGE_SIZE), c_int(window), c_float(scale), c_int(n_splits),
        c_int(chunk), c_float(softcap), _stream(),
    )
    _check(lib, rc, "flash_mix_decode", kernels=2)
    return out
