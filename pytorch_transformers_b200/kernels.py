"""Python face of the sm_100a kernel library: one function per entry point, torch tensors in.

Every function launches on the current CUDA stream of the tensors' device and raises
``KernelError`` if the entry point refuses its arguments. Nothing here computes on the host
and nothing falls back to torch: without a CUDA device, or without the compiled library, the
calls fail.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

PAGE = 64  # tokens of a cache page (PTB_PAGE in csrc/common.cuh)
# names (src/transformers/activations.py:200-228) -> the codes of csrc/common.cuh, the kernels' one table
ACTIVATIONS = {"none": 0, "gelu": 1, "gelu_new": 2, "gelu_pytorch_tanh": 2, "relu": 3, "relu2": 4, "silu": 5}   # relu2: relu(x)^2
NORM_KINDS = {"layernorm": 0, "rmsnorm": 1}
_ERRORS = {1: "unknown dtype code", 2: "a size that the kernel does not take", 3: "the CUDA launch failed",
           4: "a pointer or row size is not aligned as the kernel needs"}


class KernelError(RuntimeError):
    pass


class StepBatchC(ctypes.Structure):
    """Mirror of ``StepBatch`` in csrc/common.cuh."""
    _fields_ = [("tok_seq", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("seq_start", ctypes.c_void_p),
                ("seq_new", ctypes.c_void_p), ("seq_past", ctypes.c_void_p), ("pages", ctypes.c_void_p),
                ("pages_stride", ctypes.c_int), ("n_tokens", ctypes.c_int), ("n_seqs", ctypes.c_int)]


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


launches = 0  # entry points called so far (every one launches one kernel of this library)


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on " + str(t.device))
        if t is not None and not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


def _check_rows(t: torch.Tensor, shape, dtype, what: str) -> None:
    """``t`` is a CUDA tensor [rows, n] of ``dtype`` whose rows are contiguous (the rows themselves may lie wider apart:
    a slice of columns of a wider tensor)."""
    if not t.is_cuda or tuple(t.shape) != tuple(shape) or t.dtype != dtype or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what} must be a CUDA tensor {tuple(shape)} of {dtype} with contiguous rows, got "
                          f"{tuple(t.shape)} of {t.dtype}, strides {t.stride()}")


_configured = False


def lib():
    global _configured
    L = native.library()
    if not _configured:
        for name in ("ptb_gather_rows", "ptb_norm", "ptb_bias_act", "ptb_residual", "ptb_to_float",
                     "ptb_linear_f32", "ptb_split_rotate_store", "ptb_attention_generic", "ptb_sample",
                     "ptb_attention_generic_tile_rows", "ptb_attention_mma", "ptb_attention_mma_kept", "ptb_attention_mma_supports",
                     "ptb_skinny_linear", "ptb_skinny_linear_max_rows", "ptb_skinny_linear_k_multiple",
                     "ptb_rope_table", "ptb_attention_decode", "ptb_attention_tc", "ptb_attention_tc_supports",
                     "ptb_attention_tc_tile_tokens", "ptb_tc_linear", "ptb_tc_linear_max_rows",
                     "ptb_tc_linear_k_multiple", "ptb_attention_decode_tc", "ptb_attention_decode_tc_supports",
                     "ptb_fill_normal", "ptb_selftest_bounded_wait", "ptb_scale", "ptb_selftest_mma_cadence",
                     "ptb_norm_stream", "ptb_add_stream", "ptb_latent_store", "ptb_latent_attention", "ptb_latent_rows",
                     "ptb_rglru_conv", "ptb_rglru_scan", "ptb_block_linear", "ptb_route", "ptb_expert_plan",
                     "ptb_expert_linear", "ptb_expert_combine", "ptb_expert_linear_mma", "ptb_latent_attention_mma",
                     "ptb_latent_attention_mma_supports", "ptb_rglru_scan_chunks", "ptb_block_epilogue", "ptb_latent_gather",
                     "ptb_latent_unfold", "ptb_latent_q_unfold", "ptb_gate_heads", "ptb_linear_attention_scan",
                     "ptb_linear_attention_chunks", "ptb_linear_attention_chunks_supports", "ptb_norm_gate",
                     "ptb_qk_norm_store", "ptb_post_norm_add", "ptb_embed_sum", "ptb_softcap", "ptb_glu_clamp",
                     "ptb_attention_mma_gated", "ptb_linear_attention_chunk_join", "ptb_linear_attention_mma_supports",
                     "ptb_linear_attention_chunks_mma", "ptb_linear_attention_token", "ptb_dyt", "ptb_mlstm_gates",
                     "ptb_mlstm_scan", "ptb_mlstm_max_dim", "ptb_mlstm_state_floats", "ptb_head_norm_gate",
                     "ptb_rope_norm_store", "ptb_talk_mix", "ptb_mlstm_chunks", "ptb_mlstm_chunks_supports",
                     "ptb_mlstm_chunk_tokens", "ptb_embed_rows", "ptb_attention_generic_capped", "ptb_attention_mma_capped",
                     "ptb_qk_prepare_store", "ptb_route_grouped", "ptb_expert_combine_shared", "ptb_glu_act",
                     "ptb_head_norm_gate_act", "ptb_gla_decay", "ptb_gla_walk", "ptb_gla_chunks", "ptb_gla_max_dim",
                     "ptb_gla_chunk_tokens"):
            getattr(L, name).restype = ctypes.c_int
        L.ptb_latent_part_floats.restype = ctypes.c_longlong
        L.ptb_expert_plan_words.restype = ctypes.c_longlong
        L.ptb_mlstm_chunks_scratch_floats.restype = ctypes.c_longlong
        _configured = True
    return L


def generic_tile_rows() -> int:
    return 16  # BQ of csrc/attention_generic.cu (checked against the library in the GPU tests)


# ------------------------------------------------------------------------------------------------
def gather_rows(ids: torch.Tensor, table: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = table[ids[t]] (int32 ids). An id out of range sets bit 0 of ``status``."""
    _need_cuda(ids, table)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    _check(lib().ptb_gather_rows(_dtype_code(table), _ptr(ids), _ptr(table), _ptr(out), ids.numel(),
                                 table.shape[1], table.shape[0], _ptr(status), _stream(table)), "gather_rows")
    return out


def embed_rows(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) * scale (int32 ids; the product in float32): the first value of a float32
    stream in one pass. An id out of range sets bit 0 of ``status``."""
    _need_cuda(ids, table)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    _check(lib().ptb_embed_rows(_dtype_code(table), _ptr(ids), _ptr(table), _ptr(out), ids.numel(), table.shape[1],
                                table.shape[0], ctypes.c_float(scale), _ptr(status), _stream(table)), "embed_rows")
    return out


def norm(x: torch.Tensor, gain: torch.Tensor, bias: Optional[torch.Tensor], eps: float, kind: str = "layernorm",
         gain2: Optional[torch.Tensor] = None, bias2: Optional[torch.Tensor] = None,
         addend: Optional[torch.Tensor] = None):
    """LayerNorm / RMSNorm of rows; with ``gain2`` a second output from the same statistics. With
    ``addend`` the rows normalised are ``x + addend`` (one rounding), and that sum is returned first:
    ``(sum, y)`` or ``(sum, y, y2)``."""
    _need_cuda(x, gain, bias, gain2, bias2, addend)
    n, width = x.shape
    y1 = torch.empty_like(x)
    y2 = torch.empty_like(x) if gain2 is not None else None
    total = torch.empty_like(x) if addend is not None else None
    _check(lib().ptb_norm(_dtype_code(x), _ptr(x), _ptr(addend), _ptr(total), _ptr(gain), _ptr(bias), _ptr(y1),
                          _ptr(gain2), _ptr(bias2), _ptr(y2), n, width, ctypes.c_float(eps), NORM_KINDS[kind],
                          _stream(x)), "norm")
    outs = (y1,) if gain2 is None else (y1, y2)
    if addend is not None:
        return (total,) + outs
    return outs[0] if len(outs) == 1 else outs


def bias_act_(y: torch.Tensor, bias: Optional[torch.Tensor], act: str) -> torch.Tensor:
    """y = act(y + bias) in place."""
    _need_cuda(y, bias)
    _check(lib().ptb_bias_act(_dtype_code(y), _ptr(y), _ptr(bias), y.shape[0], y.shape[1], ACTIVATIONS[act],
                              _stream(y)), "bias_act")
    return y


def residual(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x + (a + b), the sum formed in float32."""
    _need_cuda(x, a, b)
    out = torch.empty_like(x)
    _check(lib().ptb_residual(_dtype_code(x), _ptr(x), _ptr(a), _ptr(b), _ptr(out), ctypes.c_longlong(x.numel()),
                              _stream(x)), "residual")
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32 product, one rounding)."""
    _need_cuda(x)
    _check(lib().ptb_scale(_dtype_code(x), _ptr(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream(x)),
           "scale")
    return x


def to_float(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _check(lib().ptb_to_float(_dtype_code(x), _ptr(x), _ptr(out), ctypes.c_longlong(x.numel()), _stream(x)),
           "to_float")
    return out


def fill_normal(out: torch.Tensor, key: int, std: float, offset: float = 0.0, first: int = 0,
                round_bf16: bool = False) -> torch.Tensor:
    """out.flatten()[i] = offset + std * z(key, first + i): the device twin of weights/generator.py, bit for
    bit. ``round_bf16`` rounds a float32 tensor's values to what a bfloat16 tensor would hold."""
    _need_cuda(out)
    _check(lib().ptb_fill_normal(_dtype_code(out), _ptr(out), ctypes.c_ulonglong(out.numel()),
                                 ctypes.c_ulonglong(first), ctypes.c_ulonglong(key & (2 ** 64 - 1)),
                                 ctypes.c_double(std), ctypes.c_double(offset), 1 if round_bf16 else 0,
                                 _stream(out)), "fill_normal")
    return out


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none"):
    """act(x @ w.T + bias) in true float32 on the CUDA cores."""
    _need_cuda(x, w, bias)
    if x.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("linear_f32 takes float32 tensors")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_f32: x is [{m}, {k}] but w is {list(w.shape)}")
    y = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _check(lib().ptb_linear_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(y), m, n, k, ACTIVATIONS[act], _stream(x)),
           "linear_f32")
    return y


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor, factor: float = 1.0):
    """(cos, sin) of position * inv_freq for every token of a step, each times ``factor`` (a float32 product):
    float32 [tokens, pairs] each."""
    _need_cuda(tok_pos, inv_freq)
    n, pairs = tok_pos.numel(), inv_freq.numel()
    table = torch.empty((2, n, pairs), dtype=torch.float32, device=inv_freq.device)
    _check(lib().ptb_rope_table(_ptr(tok_pos), _ptr(inv_freq), _ptr(table[0]), _ptr(table[1]), n, pairs,
                                ctypes.c_float(factor), _stream(inv_freq)), "rope_table")
    return table[0], table[1]


def split_rotate_store(fused: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       batch: StepBatchC, inv_freq: Optional[torch.Tensor], kv_heads: int, q_per_kv: int,
                       head_dim: int, write_cache: bool = True, rope=None, interleaved: bool = False) -> torch.Tensor:
    """Fused projection -> rotated queries [tokens, heads, head_dim]; K (rotated) and V go to the pools.
    The rotation comes from ``inv_freq`` (angles computed in the kernel) or from ``rope`` = (cos, sin)
    tables of ``rope_table`` for this step's tokens; the pairs are (i, i + pairs) of a head's first
    2 * pairs dims, or (2 i, 2 i + 1) with ``interleaved``."""
    _need_cuda(fused, k_pool, v_pool, inv_freq)
    n = fused.shape[0]
    q = torch.empty((n, kv_heads * q_per_kv, head_dim), dtype=fused.dtype, device=fused.device)
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    pairs = 0 if inv_freq is None else inv_freq.numel()
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        pairs = cos.shape[1]
        inv_freq = None
    _check(lib().ptb_split_rotate_store(_dtype_code(fused), _ptr(fused), _ptr(q), _ptr(k_pool), _ptr(v_pool),
                                        ctypes.byref(batch), _ptr(inv_freq), _ptr(cos), _ptr(sin), pairs, kv_heads,
                                        q_per_kv, head_dim, 1 if write_cache else 0, 1 if interleaved else 0,
                                        _stream(fused)),
           "split_rotate_store")
    return q


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                      tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      slopes: Optional[torch.Tensor], kv_heads: int, scale: float, window: int = 0,
                      sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                      out: Optional[torch.Tensor] = None, keep_first: int = 0, wide: bool = False, softcap: float = 0.0,
                      gate_wide: bool = False) -> torch.Tensor:
    """Causal attention of the step's tokens over the paged cache; returns [tokens, heads * v_dim] (v_dim is
    the V pool's row size). ``sinks`` [heads] float32: one more term exp(sink) in every row's softmax denominator,
    for which nothing is read. ``gate`` [tokens, heads] (a view whose rows may be wider apart): each head's
    output times sigmoid(gate). ``out``: a [tokens, heads * v_dim] view (rows may be wider apart) to write into.
    ``keep_first``: with a window, a sequence's first ``keep_first`` positions stay visible as well. ``wide``: returns
    float32 [tokens, heads, kv_heads, v_dim] instead, every head's softmax weights applied to every K/V head's values
    (what ``talk_mix`` sums when the heads' weights are mixed after the softmax). ``softcap`` > 0: every score becomes
    softcap * tanh(score / softcap) after the scale. ``gate_wide``: ``gate`` is [tokens, heads * v_dim], a number per
    entry of the output."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes, sinks)
    n, heads, head_dim = q.shape
    v_dim = v_pool.shape[-1]
    if wide:
        if gate is not None or sinks is not None or out is not None or out_scale != 1.0 or softcap:
            raise KernelError("attention_generic: the wide form takes no sink, gate, factor, cap or output view")
        res = torch.empty((n, heads, kv_heads, v_dim), dtype=torch.float32, device=q.device)
        _check(lib().ptb_attention_generic(_dtype_code(q), _ptr(q), _ptr(k_pool), _ptr(v_pool), None,
                                           ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(slopes),
                                           heads, kv_heads, head_dim, ctypes.c_float(scale), window, v_dim, None,
                                           None, 0, ctypes.c_float(1.0), 0, int(keep_first), _ptr(res), _stream(q)),
               "attention_generic (wide)")
        return res
    if out is None:
        out = torch.empty((n, heads * v_dim), dtype=q.dtype, device=q.device)
    _check_rows(out, (n, heads * v_dim), q.dtype, "attention_generic: out")
    if gate is not None:
        _check_rows(gate, (n, heads * v_dim if gate_wide else heads), q.dtype, "attention_generic: gate")
    _check(lib().ptb_attention_generic_capped(_dtype_code(q), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out),
                                              ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(slopes),
                                              heads, kv_heads, head_dim, ctypes.c_float(scale), window, v_dim, _ptr(sinks),
                                              _ptr(gate), 0 if gate is None else gate.stride(0), ctypes.c_float(out_scale),
                                              out.stride(0), int(keep_first), None, ctypes.c_float(softcap),
                                              1 if gate_wide else 0, _stream(q)),
           "attention_generic")
    return out


def rope_norm_store(proj: torch.Tensor, bias: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: torch.Tensor,
                    batch: StepBatchC, rope, heads: int, kv_heads: int, dim: int, v_dim: int, eps: float,
                    unit_norm: bool = True, v_first: Optional[torch.Tensor] = None, lam: Optional[torch.Tensor] = None,
                    keep_values: bool = False, write_cache: bool = True, q_gain: Optional[torch.Tensor] = None,
                    k_gain: Optional[torch.Tensor] = None, norm_first: bool = False, q_temp=None):
    """``proj`` [tokens, >= (heads + kv_heads) dim + kv_heads v_dim] holds q, k, v side by side (rows may lie wider
    apart); ``bias`` (float32, as long) is added in float32. Queries and keys: rotation of a head's first entries by
    ``rope`` = (cos, sin) tables [tokens, pairs] (None: none), then, with ``unit_norm``, division by the head's root mean
    square. Values: ``(1 - lam) v + lam v_first`` where ``v_first`` [tokens, kv_heads v_dim] is given (``lam``: one
    float32 on the device). Keys and values go into the paged pools. Returns q [tokens, heads, dim], and with
    ``keep_values`` also this layer's own values [tokens, kv_heads v_dim] as they were before any mixing.
    ``norm_first``: the norm comes before the rotation and multiplies by the gains ``q_gain``, ``k_gain`` (float32 [dim];
    None: no gains). ``q_temp`` = (coef, every): a query at position p is multiplied by
    1 + coef ln(floor((p + 1) / every) + 1) at the end."""
    _need_cuda(k_pool, v_pool, bias, lam, q_gain, k_gain)
    if (q_gain is not None or k_gain is not None) and not (unit_norm and norm_first):
        raise KernelError("rope_norm_store: gains go with a norm before the rotation")
    for g in (q_gain, k_gain):
        if g is not None and (g.dtype != torch.float32 or g.numel() != dim):
            raise KernelError("rope_norm_store: gains are float32 [dim]")
    coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    _check_rows(proj, proj.shape, proj.dtype, "rope_norm_store: proj")
    n = proj.shape[0]
    q = torch.empty((n, heads, dim), dtype=proj.dtype, device=proj.device)
    kept = torch.empty((n, kv_heads * v_dim), dtype=proj.dtype, device=proj.device) if keep_values else None
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    if v_first is not None:
        _check_rows(v_first, (n, kv_heads * v_dim), proj.dtype, "rope_norm_store: v_first")
        if lam is None or lam.dtype != torch.float32:
            raise KernelError("rope_norm_store: the mixing weight is one float32 on the device")
    _check(lib().ptb_qk_prepare_store(_dtype_code(proj), _ptr(proj), proj.stride(0), _ptr(bias), _ptr(q), _ptr(k_pool),
                                      _ptr(v_pool), ctypes.byref(batch), _ptr(cos), _ptr(sin), pairs, heads, kv_heads, dim,
                                      v_dim, ctypes.c_float(eps), 1 if unit_norm else 0, _ptr(v_first),
                                      0 if v_first is None else v_first.stride(0), _ptr(lam if v_first is not None else None),
                                      _ptr(kept), 1 if write_cache else 0, _ptr(q_gain), _ptr(k_gain), 1 if norm_first else 0,
                                      ctypes.c_float(coef), every, _stream(proj)), "rope_norm_store")
    return (q, kept) if keep_values else q


def talk_mix(wide: torch.Tensor, talk: torch.Tensor, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h] = sum_g talk[h, g] * wide[t, g, K/V head of h]: ``wide`` float32 [tokens, heads, kv_heads, v_dim] from
    ``attention_generic(wide=True)``, ``talk`` float32 [heads, heads]. Returns [tokens, heads * v_dim] of ``out_dtype``."""
    _need_cuda(wide, talk)
    n, heads, kv_heads, v_dim = wide.shape
    if wide.dtype != torch.float32 or talk.dtype != torch.float32 or tuple(talk.shape) != (heads, heads):
        raise KernelError("talk_mix takes float32 results [tokens, heads, kv_heads, v_dim] and a float32 matrix [heads, heads]")
    if out is None:
        out = torch.empty((n, heads * v_dim), dtype=out_dtype, device=wide.device)
    _check_rows(out, (n, heads * v_dim), out_dtype, "talk_mix: out")
    _check(lib().ptb_talk_mix(_dtype_code(out), _ptr(wide), _ptr(talk), _ptr(out), out.stride(0), n, heads, kv_heads, v_dim,
                              _stream(wide)), "talk_mix")
    return out


DECODE_SPLITS = (1, 2, 3, 4, 5, 6, 7, 8)   # ptb_attention_decode: the blocks of a split set form one cluster
DECODE_KEY_SPLITS = (1, 2, 4)              # groups of warps that share a page's keys


def decode_max_warps(head_dim: int) -> int:
    """Warps of a block of attention_decode: row warps times key groups."""
    return 10 if head_dim == 64 else 8


def attention_decode(fused: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC, rope,
                     slopes: Optional[torch.Tensor], kv_heads: int, q_per_kv: int, head_dim: int, scale: float,
                     window: int, heads_per_tile: int, warps: int, n_splits: int, write_cache: bool = True,
                     key_split: int = 1, n_teams: int = 1, interleaved: bool = False):
    """One kernel for the attention of a step of single tokens: rotate q and k of each new token, put
    k and v into the cache, attend over the cache (all heads of a K/V group in one tile of ``warps``
    x 16 rows, key pages divided among ``n_splits`` blocks of one cluster, the keys of a page among
    ``key_split`` groups of warps, all joined through (distributed) shared memory; ``n_teams`` such
    clusters share the pages of a long sequence and join through a workspace in global memory).
    Returns [tokens, heads * head_dim]."""
    _need_cuda(fused, k_pool, v_pool, slopes)
    if fused.dtype != torch.bfloat16:
        raise KernelError("attention_decode takes bfloat16 tensors")
    n = fused.shape[0]
    heads = kv_heads * q_per_kv
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    out = torch.empty((n, heads * head_dim), dtype=fused.dtype, device=fused.device)
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    parts = tickets = None
    part_floats = n_tickets = 0
    if n_teams > 1:
        groups = n * kv_heads * ((q_per_kv + heads_per_tile - 1) // heads_per_tile)
        if groups * n_splits > DECODE_TICKETS:
            raise KernelError("attention_decode: too many (sequence, head chunk, split) triples for the ticket buffer")
        part_floats = groups * n_teams * heads_per_tile * (head_dim + 2)
        parts = torch.empty(part_floats, dtype=torch.float32, device=fused.device)
        n_tickets = groups * n_splits
        tickets = _tickets(n_tickets, fused.device)
    _check(lib().ptb_attention_decode(_ptr(fused), _ptr(k_pool), _ptr(v_pool), _ptr(out), ctypes.byref(batch),
                                      _ptr(cos), _ptr(sin), pairs, 1 if interleaved else 0, _ptr(slopes), heads, kv_heads,
                                      head_dim,
                                      heads_per_tile, n_splits, n_teams, warps, key_split, ctypes.c_float(scale),
                                      window, 1 if write_cache else 0, _ptr(parts), ctypes.c_size_t(part_floats),
                                      _ptr(tickets), n_tickets, _stream(fused)),
           "attention_decode")
    return out


def attention_decode_tc_supports(head_dim: int, q_per_kv: int) -> bool:
    return bool(lib().ptb_attention_decode_tc_supports(int(head_dim), int(q_per_kv)))


def attention_decode_tc(fused: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC, rope,
                        kv_heads: int, q_per_kv: int, head_dim: int, scale: float, n_splits: int,
                        write_cache: bool = True, n_teams: int = 1, interleaved: bool = False):
    """The attention of a step of single tokens on the tcgen05 tensor cores, for K/V heads that serve
    33 to 128 query heads of size 64: the query heads of a group are the rows of one tile, S, P and O
    live in tensor memory, pages come by TMA, ``n_splits`` blocks of one cluster share a sequence's
    pages and join through distributed shared memory; ``n_teams`` such clusters share the pages of a
    long sequence and join through a workspace in global memory. No score bias, no window.
    Returns [tokens, heads * head_dim]."""
    _need_cuda(fused, k_pool, v_pool)
    if fused.dtype != torch.bfloat16:
        raise KernelError("attention_decode_tc takes bfloat16 tensors")
    n = fused.shape[0]
    heads = kv_heads * q_per_kv
    if fused.shape[1] != kv_heads * (q_per_kv + 2) * head_dim:
        raise KernelError(f"fused projection has width {fused.shape[1]}, expected "
                          f"{kv_heads * (q_per_kv + 2) * head_dim}")
    if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
        raise KernelError("attention_decode_tc takes the contiguous K and V pools of one cache entry")
    out = torch.empty((n, heads * head_dim), dtype=fused.dtype, device=fused.device)
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    parts = tickets = None
    part_floats = n_tickets = 0
    if n_teams > 1:
        if n * kv_heads * n_splits > DECODE_TICKETS:
            raise KernelError("attention_decode_tc: too many (sequence, K/V head, split) triples for the ticket buffer")
        part_floats = n * kv_heads * n_teams * q_per_kv * (head_dim + 2)
        parts = torch.empty(part_floats, dtype=torch.float32, device=fused.device)
        n_tickets = n * kv_heads * n_splits
        tickets = _tickets(n_tickets, fused.device)
    _check(lib().ptb_attention_decode_tc(_ptr(fused), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(out),
                                         ctypes.byref(batch), _ptr(cos), _ptr(sin), pairs, 1 if interleaved else 0, heads,
                                         kv_heads, head_dim,
                                         n_splits, n_teams, ctypes.c_float(scale), 1 if write_cache else 0,
                                         _ptr(parts), ctypes.c_size_t(part_floats), _ptr(tickets), n_tickets,
                                         _ptr(error_flag(fused.device)), _stream(fused)), "attention_decode_tc")
    return out


DECODE_TICKETS = 8192      # most (sequence, K/V head, split) triples of one decode attention launch
TICKET_ARENA = 1 << 18     # int32 words per device
_ticket_arenas = {}


def _tickets(n: int, device) -> torch.Tensor:
    """``n`` int32 zeros for a launch whose blocks count their arrivals; the kernel leaves them zero.
    Two launches that run at the same time (the two branches of a block, side by side in one graph)
    must not count in the same words, so every launch takes the next stretch of a zeroed arena, which
    wraps around after tens of launches; launches that far apart in a stream or a graph depend on
    one another and never overlap. The arena is allocated at a device's first launch, which is never
    inside a stream capture (a captured step has run once plainly before)."""
    device = torch.device(device)
    arena = _ticket_arenas.get(device)
    if arena is None:
        arena = _ticket_arenas[device] = [torch.zeros(TICKET_ARENA, dtype=torch.int32, device=device), 0]
    n = (n + 31) // 32 * 32
    if n > TICKET_ARENA:
        raise KernelError(f"a launch asks for {n} tickets, more than the arena's {TICKET_ARENA}")
    if arena[1] + n > TICKET_ARENA:
        arena[1] = 0
    out = arena[0][arena[1]:arena[1] + n]
    arena[1] += n
    return out


_error_flags = {}
TC_TILE_TOKENS = 128  # ptb_attention_tc_tile_tokens()


def error_flag(device) -> torch.Tensor:
    """Device int32 word that kernels with bounded waits raise when a wait runs out."""
    device = torch.device(device)
    if device not in _error_flags:
        _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[device]


def check_device_errors(device) -> None:
    """Raise if a kernel has reported that one of its bounded waits ran out (synchronises)."""
    device = torch.device(device)
    flag = _error_flags.get(device)
    if flag is not None:
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise KernelError(f"a kernel gave up waiting inside its pipeline (code {code}): its results are void")


def selftest_mma_cadence(device, n: int, reps: int = 1000, a_in_tmem: bool = False, blocks: int = 1) -> float:
    """Clocks per tcgen05.mma (M = 128, K = 16, N = ``n``) when one thread of each of ``blocks`` blocks issues
    ``4 * reps`` of them back to back on operands that sit in shared (or tensor) memory."""
    device = torch.device(device)
    clocks = torch.zeros(1, dtype=torch.int64, device=device)
    _check(lib().ptb_selftest_mma_cadence(int(n), int(reps), 1 if a_in_tmem else 0, int(blocks), _ptr(clocks),
                                          _ptr(error_flag(device)),
                                          ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)),
           "selftest_mma_cadence")
    return float(clocks.item()) / (4 * reps)


def selftest_bounded_wait(device, tries: int = 1000) -> torch.Tensor:
    """Launch a kernel that waits, at most ``tries`` times, on a barrier at which nobody arrives: the wait
    runs out and raises the device's error flag, as a tcgen05 kernel does whose copy never lands.
    Returns an int32 word that the kernel sets to 1 when it gave up. ``check_device_errors`` then raises."""
    device = torch.device(device)
    gave_up = torch.zeros(1, dtype=torch.int32, device=device)
    _check(lib().ptb_selftest_bounded_wait(int(tries), _ptr(error_flag(device)), _ptr(gave_up),
                                           ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)),
           "selftest_bounded_wait")
    return gave_up


def attention_tc_supports(head_dim: int) -> bool:
    return bool(lib().ptb_attention_tc_supports(int(head_dim)))


def attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, kv_heads: int, scale: float,
                 slopes: Optional[torch.Tensor] = None):
    """Causal prompt attention on tcgen05 tensor cores with accumulators in tensor memory: bfloat16,
    head size 64 or 128, tiles of 128 tokens, no window; ``slopes`` [heads] float32: per-head score
    slopes (ALiBi). Returns [tokens, heads * head_dim]."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_tc takes bfloat16 tensors")
    n, heads, head_dim = q.shape
    out = torch.empty((n, heads * head_dim), dtype=q.dtype, device=q.device)
    if not k_pool.is_contiguous() or not v_pool.is_contiguous() or k_pool.shape != v_pool.shape:
        raise KernelError("attention_tc takes the contiguous K and V pools of one cache entry")
    _check(lib().ptb_attention_tc(_ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(out), ctypes.byref(batch), _ptr(tile_seq),
                                  _ptr(tile_q0), n_tiles, _ptr(slopes), heads, kv_heads, head_dim, ctypes.c_float(scale),
                                  _ptr(error_flag(q.device)), _stream(q)), "attention_tc")
    return out


def attention_tc_pairs(mode) -> None:
    """For measurements and tests. ``attention_tc`` with head size 128 puts two heads of a K/V group in one
    block where the pairs fill the device (mode 1 or True, the default); 0 or False: never; 2: wherever a
    group has two heads or more."""
    lib().ptb_attention_tc_pairs(int(mode))


def attention_mma_supports(head_dim: int) -> bool:
    return bool(lib().ptb_attention_mma_supports(int(head_dim)))


def attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                  tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, slopes: Optional[torch.Tensor],
                  kv_heads: int, scale: float, window: int, tokens_per_tile: int, heads_per_tile: int, warps: int,
                  n_splits: int, scratch: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                  gate: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                  out: Optional[torch.Tensor] = None, wide_weights: bool = False, keep_first: int = 0,
                  wide: bool = False, softcap: float = 0.0, gate_wide: bool = False) -> torch.Tensor:
    """Tensor-core attention over the paged cache (bfloat16). A tile holds ``tokens_per_tile`` tokens
    x ``heads_per_tile`` heads of one K/V group in ``warps`` x 16 rows; with ``n_splits`` > 1 the key
    pages are divided among blocks and joined by a second kernel (``scratch``: float32 workspace).
    ``sinks``, ``gate``, ``out_scale``, ``out``: as attention_generic takes them. ``wide_weights``: the softmax
    weights meet the values as two bfloat16 terms (16 bits of mantissa) instead of one. ``keep_first``: with a window,
    the first positions that stay visible left of it. ``wide``: every head's weights on every K/V head's values, float32
    [tokens, heads, kv_heads, head_dim], as ``attention_generic(wide=True)`` returns them. ``softcap``, ``gate_wide``: as
    attention_generic takes them (a gate per entry starts at a whole 32-bit word, rows an even number of entries apart)."""
    _need_cuda(q, k_pool, v_pool, tile_seq, tile_q0, slopes, scratch, sinks)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_mma takes bfloat16 tensors")
    n, heads, head_dim = q.shape
    out_wide = None
    if wide:
        if sinks is not None or gate is not None or out_scale != 1.0 or out is not None or softcap:
            raise KernelError("attention_mma: the wide form takes no sink, gate, factor, cap or output view")
        out_wide = torch.empty((n, heads, kv_heads, head_dim), dtype=torch.float32, device=q.device)
    else:
        if out is None:
            out = torch.empty((n, heads * head_dim), dtype=q.dtype, device=q.device)
        _check_rows(out, (n, heads * head_dim), q.dtype, "attention_mma: out")
        if out.data_ptr() % 4 or out.stride(0) % 2:
            raise KernelError("attention_mma: output rows must start at whole 32-bit words")
    if gate is not None:
        _check_rows(gate, (n, heads * head_dim if gate_wide else heads), q.dtype, "attention_mma: gate")
        if gate_wide and (gate.data_ptr() % 4 or gate.stride(0) % 2):
            raise KernelError("attention_mma: a gate per entry must start at whole 32-bit words")
    if n_splits > 1:
        need = attention_mma_scratch_floats(n_tiles, heads, kv_heads, heads_per_tile, n_splits, warps, head_dim)
        if wide:
            need *= kv_heads
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        elif scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention_mma: scratch of {need} float32 values needed")
    _check(lib().ptb_attention_mma_capped(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch),
                                          ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(slopes),
                                          heads, kv_heads, head_dim, heads_per_tile, tokens_per_tile, n_splits, warps,
                                          ctypes.c_float(scale), window, _ptr(sinks), _ptr(gate),
                                          0 if gate is None else gate.stride(0), ctypes.c_float(out_scale),
                                          0 if wide else out.stride(0), 1 if wide_weights else 0, int(keep_first),
                                          _ptr(out_wide), ctypes.c_float(softcap), 1 if gate_wide else 0, _stream(q)),
           "attention_mma")
    if n_splits > 1:
        global launches
        launches += 1   # the kernel that joins the splits
    return out_wide if wide else out


def attention_mma_scratch_floats(n_tiles: int, heads: int, kv_heads: int, heads_per_tile: int, n_splits: int,
                                 warps: int, head_dim: int) -> int:
    if n_splits <= 1:
        return 0
    chunks = (heads // kv_heads + heads_per_tile - 1) // heads_per_tile
    return n_tiles * kv_heads * chunks * n_splits * warps * 16 * (head_dim + 2)


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, do_sample: bool, temperature: float = 1.0,
           top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
           history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
           suppress: Optional[torch.Tensor] = None, seed: int = 0, streams: Optional[torch.Tensor] = None,
           counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Select one token per row of float32 logits into ``out`` (int32). ``work`` is scratch of the
    logits' shape; ``streams`` and ``counters`` (int64 per row) key the uniform draw."""
    _need_cuda(logits, work, out, history, history_len, suppress, streams, counters)
    if logits.dtype != torch.float32 or work.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample takes float32 logits and scratch and an int32 output")
    rows, vocab = logits.shape
    if work.numel() < logits.numel() or out.numel() < rows:
        raise KernelError("sample: scratch or output too small")
    if do_sample and (streams is None or counters is None):
        raise KernelError("sample: sampling needs the per-row stream and counter tensors")
    _check(lib().ptb_sample(_ptr(logits), _ptr(work), _ptr(out), rows, vocab, 1 if do_sample else 0,
                            ctypes.c_float(temperature), int(top_k), ctypes.c_float(top_p), ctypes.c_float(min_p),
                            ctypes.c_float(repetition_penalty), _ptr(history), _ptr(history_len),
                            0 if history is None else history.shape[1], _ptr(suppress),
                            0 if suppress is None else suppress.numel(), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                            _ptr(streams), _ptr(counters), _stream(logits)), "sample")
    return out


SKINNY_MAX_ROWS = 32   # ptb_skinny_linear_max_rows()
SKINNY_K_MULTIPLE = 32  # ptb_skinny_linear_k_multiple()


# Rows beyond which the library product is faster inside a step (12 rows: 3.40 against 3.49 ms a step;
# 16 rows: 3.51 against 3.22).
SKINNY_BEST_ROWS = 12
# A matrix of tens of thousands of rows (the vocabulary's) runs alone in the step, and there the library
# reads it faster from 5 rows on (591 MB, float32 out, 8 rows: 92.7 against 86.9 us).
SKINNY_TALL_ROWS = 32768
SKINNY_BEST_ROWS_TALL = 4


def skinny_linear_takes(rows: int, k: int) -> bool:
    return 0 < rows <= SKINNY_MAX_ROWS and k % SKINNY_K_MULTIPLE == 0


def skinny_linear_preferred(rows: int, k: int, n: int = 0) -> bool:
    best = SKINNY_BEST_ROWS_TALL if n >= SKINNY_TALL_ROWS else SKINNY_BEST_ROWS
    return 0 < rows <= best and k % SKINNY_K_MULTIPLE == 0


def skinny_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                  add: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """act(x @ w.T + bias) + add for up to 32 rows of bfloat16 x: one pass over w at memory speed,
    float32 accumulation and epilogue; the result is bfloat16 or float32."""
    _need_cuda(x, w, bias, add)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (add is not None and add.dtype != torch.bfloat16):
        raise KernelError("skinny_linear takes bfloat16 x, w and add")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (add is not None and tuple(add.shape) != (m, n)):
        raise KernelError(f"skinny_linear: shapes x {list(x.shape)}, w {list(w.shape)} do not fit")
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    ybf, yf = (y, None) if out_dtype == torch.bfloat16 else (None, y)
    # where the tiles of w do not divide evenly over the SMs the kernel divides K among several blocks per
    # tile; their partial sums meet in scratch memory, a zeroed ticket per tile says who is last
    need = _skinny_scratch_floats(m, n, k)
    scratch = torch.empty(need, dtype=torch.float32, device=x.device) if need else None
    n_tickets = (n + 15) // 16 if need else 0        # a ticket per tile of weight rows; tiles have 16 rows or more
    tickets = _tickets(n_tickets, x.device) if need else None
    _check(lib().ptb_skinny_linear(_ptr(x), _ptr(w), _ptr(bias), _ptr(add), _ptr(ybf), _ptr(yf), m, n, k,
                                   ACTIVATIONS[act], _ptr(scratch), ctypes.c_size_t(need), _ptr(tickets),
                                   n_tickets, _stream(x)), "skinny_linear")
    return y


_skinny_scratch_cache = {}


def _skinny_scratch_floats(m: int, n: int, k: int) -> int:
    key = (m, n, k)
    if key not in _skinny_scratch_cache:
        fn = lib().ptb_skinny_linear_scratch
        fn.restype = ctypes.c_longlong
        _skinny_scratch_cache[key] = int(fn(m, n, k))
    return _skinny_scratch_cache[key]


_sm_count = {}


def sm_count(device) -> int:
    """Multiprocessors of ``device`` (148 on a B200); without a CUDA device, the B200's count."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return 148
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[device]


# A step of few tokens is bound by the read of the weights, and a mixer's small kernels can hide under
# the feed-forward's weight stream on a second stream. Two limits say how long that pays:
# rows of the step (beyond them the linear layers are no longer pure weight streams; two branches
# against one at 48 rows: 4.19 against 4.49 ms a step, at 64 rows: 4.44 against 4.25), and the bytes of
# keys and values that one attention layer reads in the step: once they are tens of megabytes the
# attention competes with the weight stream instead of hiding under it (34 MB: 3.43 against 3.85 ms;
# 42 MB: 4.49 against 4.24). Heads wider than 64 need the decode kernel's large page ring, which keeps
# the stream's blocks off the SMs earlier (17 MB: 5.39 against 5.55 ms; 34 MB: 7.80 against 5.80).
WEIGHT_STREAM_MAX_ROWS = 48
DECODE_BESIDE_MAX_KV_BYTES = 40 << 20
DECODE_BESIDE_MAX_KV_BYTES_WIDE_HEADS = 24 << 20


def decode_attention_fits_beside(kv_bytes: int, head_dim: int) -> bool:
    """May a decode attention that reads ``kv_bytes`` of keys and values run beside a weight stream?"""
    return kv_bytes <= (DECODE_BESIDE_MAX_KV_BYTES if head_dim <= 64 else DECODE_BESIDE_MAX_KV_BYTES_WIDE_HEADS)


TC_LINEAR_MAX_ROWS = 128   # ptb_tc_linear_max_rows()
TC_LINEAR_K_MULTIPLE = 8   # ptb_tc_linear_k_multiple()


def tc_linear_takes(rows: int, k: int) -> bool:
    return 0 < rows <= TC_LINEAR_MAX_ROWS and k % TC_LINEAR_K_MULTIPLE == 0


def tc_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
              add: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """act(x @ w.T + bias) + add for up to 128 rows of bfloat16 x on the tcgen05 tensor cores: the
    weights stream once through shared memory (TMA), the sums stay in tensor memory, and bias,
    activation and the sum with ``add`` happen in the float32 epilogue. Result bfloat16 or float32."""
    _need_cuda(x, w, bias, add)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (add is not None and add.dtype != torch.bfloat16):
        raise KernelError("tc_linear takes bfloat16 x, w and add")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (add is not None and tuple(add.shape) != (m, n)):
        raise KernelError(f"tc_linear: shapes x {list(x.shape)}, w {list(w.shape)} do not fit")
    if not x.is_contiguous() or not w.is_contiguous() or (add is not None and not add.is_contiguous()):
        raise KernelError("tc_linear takes contiguous tensors")
    dev = x.device
    y = torch.empty((m, n), dtype=out_dtype, device=dev)
    ybf, yf = (y, None) if out_dtype == torch.bfloat16 else (None, y)
    _check(lib().ptb_tc_linear(_ptr(x), _ptr(w), _ptr(bias), _ptr(add), _ptr(ybf), _ptr(yf), m, n, k,
                               ACTIVATIONS[act], sm_count(dev), _ptr(error_flag(dev)), _stream(x)), "tc_linear")
    return y


def matmul_nt(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
              add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Library matrix product x @ w.T (+ add) for the bfloat16 path (cuBLAS through torch), where the
    reference's engine uses the same library. float32 inputs are refused: the float32 path has
    its own kernel (linear_f32)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("matmul_nt is the bfloat16 library product; float32 goes through linear_f32")
    _need_cuda(x, w)
    if add is not None:
        # the library's own epilogue adds in float32 and rounds once (beta = 1)
        if out_dtype not in (None, torch.bfloat16) or add.dtype != torch.bfloat16 or tuple(add.shape) != (x.shape[0], w.shape[0]):
            raise KernelError("matmul_nt adds a bfloat16 tensor of the result's shape to a bfloat16 result")
        return torch.addmm(add, x, w.t())
    if out_dtype is None or out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# ------------------------------------------------------------------------------------------------
# A float32 residual stream beside bfloat16 matrices
def norm_stream(x: torch.Tensor, gain: torch.Tensor, bias: Optional[torch.Tensor], eps: float, kind: str,
                out_dtype: torch.dtype, addend: Optional[torch.Tensor] = None):
    """Norm of float32 rows ``x`` (or of ``x + addend``, addend float32 or bfloat16) written in ``out_dtype``.
    Returns ``y``, or ``(sum, y)`` with the float32 sum when ``addend`` is given."""
    _need_cuda(x, gain, bias, addend)
    if x.dtype != torch.float32:
        raise KernelError("norm_stream takes a float32 stream")
    n, width = x.shape
    y = torch.empty((n, width), dtype=out_dtype, device=x.device)
    total = torch.empty_like(x) if addend is not None else None
    _check(lib().ptb_norm_stream(_ptr(x), 0 if addend is None else _dtype_code(addend), _ptr(addend), _ptr(total),
                                 _ptr(gain), _ptr(bias), _dtype_code(y), _ptr(y), n, width, ctypes.c_float(eps),
                                 NORM_KINDS[kind], _stream(x)), "norm_stream")
    return y if addend is None else (total, y)


def add_stream(x: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """x + a in float32: ``x`` is the float32 stream, ``a`` a branch's result in float32 or bfloat16."""
    _need_cuda(x, a)
    if x.dtype != torch.float32 or x.shape != a.shape:
        raise KernelError("add_stream takes a float32 stream and an addend of its shape")
    out = torch.empty_like(x)
    _check(lib().ptb_add_stream(_ptr(x), _dtype_code(a), _ptr(a), _ptr(out), ctypes.c_longlong(x.numel()), _stream(x)),
           "add_stream")
    return out


# ------------------------------------------------------------------------------------------------
# Latent attention
LATENT_ROWS = 16   # ptb_latent_rows(): (token, head) rows of a tile


def latent_store(src: torch.Tensor, norm_w: torch.Tensor, eps: float, pool: torch.Tensor, batch: StepBatchC, rope,
                 rank: int, rot_dim: int, interleaved: bool = True) -> None:
    """Rows ``src`` [tokens, rank + rot_dim] (a view whose rows may be wider apart) of the latent
    down-projection become cache rows: the first ``rank`` RMS-normed with ``norm_w``, the rest rotated by
    the tokens' positions (``rope`` = (cos, sin) [tokens, pairs])."""
    _need_cuda(norm_w, pool)
    if src.stride(1) != 1 or src.shape[1] != rank + rot_dim or pool.shape[-1] != rank + rot_dim or pool.dtype != src.dtype:
        raise KernelError("latent_store: the rows or the pool do not fit rank + rot_dim")
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    _check(lib().ptb_latent_store(_dtype_code(src), _ptr(src), ctypes.c_longlong(src.stride(0)), _ptr(norm_w),
                                  ctypes.c_float(eps), _ptr(pool), ctypes.byref(batch), _ptr(cos), _ptr(sin), pairs,
                                  1 if interleaved else 0, rank, rot_dim, _stream(pool)), "latent_store")


def latent_attention_mma_supports(rank: int, rot_dim: int) -> bool:
    return bool(lib().ptb_latent_attention_mma_supports(int(rank), int(rot_dim)))


def latent_attention(q_abs: torch.Tensor, q: torch.Tensor, q_rot_off: int, pool: torch.Tensor, batch: StepBatchC,
                     tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, tile_tokens: int, rope, rank: int,
                     rot_dim: int, scale: float, interleaved: bool = True, n_splits: int = 1,
                     tensor_cores: Optional[bool] = None) -> torch.Tensor:
    """Causal attention in latent space. ``q_abs`` [tokens, heads, rank] float32 (queries with the key
    up-projection folded in), ``q`` [tokens, heads, q_dim] whose entries from ``q_rot_off`` on are the part
    to rotate, ``pool`` the cache entry's rows [pages, 1, 64, rank + rot_dim]. A tile holds ``tile_tokens``
    tokens x 16 / tile_tokens heads; ``n_splits`` blocks share a tile's key pages. bfloat16 with ``rank`` a
    multiple of 64 and ``rot_dim`` of 16 runs on the tensor cores (``tensor_cores=False``: the general kernel). Returns
    [tokens, heads, rank] in the model dtype: per head, the softmax-weighted sum of the cached latents."""
    _need_cuda(q_abs, q, pool, tile_seq, tile_q0)
    n, heads, q_dim = q.shape
    if q_abs.dtype != torch.float32 or tuple(q_abs.shape) != (n, heads, rank) or pool.dtype != q.dtype:
        raise KernelError("latent_attention: q_abs must be float32 [tokens, heads, rank] and the pool of q's dtype")
    if pool.shape[-1] != rank + rot_dim or q_rot_off + rot_dim > q_dim:
        raise KernelError("latent_attention: sizes do not fit")
    if tensor_cores is None:
        tensor_cores = q.dtype == torch.bfloat16 and latent_attention_mma_supports(rank, rot_dim)
    heads_per_block = max(1, LATENT_ROWS // tile_tokens)
    if tensor_cores and n_splits == 1 and tile_tokens * heads_per_block == LATENT_ROWS:
        # the tensor-core kernel takes up to four groups of 16 rows on one staged page: more heads a block
        heads_per_block *= 4 if heads >= 4 * heads_per_block else (2 if heads >= 2 * heads_per_block else 1)
    out = torch.empty((n, heads, rank), dtype=q.dtype, device=q.device)
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    part = None
    if n_splits > 1:
        need = int(lib().ptb_latent_part_floats(n_tiles, heads, heads_per_block, n_splits, rank))
        part = torch.empty(need, dtype=torch.float32, device=q.device)
    if tensor_cores:
        _check(lib().ptb_latent_attention_mma(_ptr(q_abs), _ptr(q), q_dim, q_rot_off, _ptr(pool), _ptr(part), _ptr(out),
                                              ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(cos),
                                              _ptr(sin), pairs, 1 if interleaved else 0, heads, rank, rot_dim, tile_tokens,
                                              heads_per_block, ctypes.c_float(scale), n_splits, _stream(q)),
               "latent_attention_mma")
    else:
        _check(lib().ptb_latent_attention(_dtype_code(q), _ptr(q_abs), _ptr(q), q_dim, q_rot_off, _ptr(pool), _ptr(part),
                                          _ptr(out), ctypes.byref(batch), _ptr(tile_seq), _ptr(tile_q0), n_tiles, _ptr(cos),
                                          _ptr(sin), pairs, 1 if interleaved else 0, heads, rank, rot_dim, tile_tokens,
                                          heads_per_block, ctypes.c_float(scale), n_splits, _stream(q)), "latent_attention")
    if n_splits > 1:
        global launches
        launches += 1
    return out


def latent_unfolded_attention(q: torch.Tensor, pool: torch.Tensor, k_tmp: torch.Tensor, v_tmp: torch.Tensor,
                              w_ukv: torch.Tensor, gate: torch.Tensor, batch: StepBatchC, ctx_seq: torch.Tensor,
                              ctx_pos: torch.Tensor, n_ctx: int, mtile_seq: torch.Tensor, mtile_q0: torch.Tensor,
                              n_mma_tiles: int, rope, dim: int, rot_dim: int, vdim: int, rank: int, scale: float,
                              interleaved: bool = True) -> torch.Tensor:
    """Latent attention of prompts through the tcgen05 prompt kernel (bfloat16): the ``n_ctx`` cached rows
    (``ctx_seq``, ``ctx_pos``: sequence and position of each) of the step's sequences are unfolded with
    ``w_ukv`` = [W_uk; W_uv] into per-head keys and values in the scratch pools ``k_tmp`` / ``v_tmp``
    ([pages, heads, 64, hd], zero outside what is written here), the queries are laid out to match, and
    ``attention_tc`` runs on them. Returns the heads' outputs times sigmoid(gate): [tokens, heads * vdim]."""
    _need_cuda(q, pool, k_tmp, v_tmp, w_ukv, ctx_seq, ctx_pos)
    n, heads, dq = q.shape
    hd = k_tmp.shape[-1]
    if q.dtype != torch.bfloat16 or dq != dim + rot_dim or tuple(w_ukv.shape) != (heads * (dim + vdim), rank):
        raise KernelError("latent_unfolded_attention: sizes or dtypes do not fit")
    cos, sin = rope if rope is not None else (None, None)
    pairs = 0 if cos is None else cos.shape[1]
    stream = _stream(q)
    c_rows = torch.empty((n_ctx, rank), dtype=q.dtype, device=q.device)
    kr_rows = torch.empty((n_ctx, max(rot_dim, 1)), dtype=q.dtype, device=q.device)
    _check(lib().ptb_latent_gather(_ptr(pool), ctypes.byref(batch), _ptr(ctx_seq), _ptr(ctx_pos), n_ctx, _ptr(c_rows),
                                   _ptr(kr_rows), rank, rot_dim, stream), "latent_gather")
    kv = matmul_nt(c_rows, w_ukv)
    _check(lib().ptb_latent_unfold(_ptr(kv), _ptr(kr_rows), ctypes.byref(batch), _ptr(ctx_seq), _ptr(ctx_pos), n_ctx,
                                   _ptr(k_tmp), _ptr(v_tmp), heads, dim, rot_dim, vdim, hd, stream), "latent_unfold")
    q_tc = torch.empty((n, heads, hd), dtype=q.dtype, device=q.device)
    _check(lib().ptb_latent_q_unfold(_ptr(q), _ptr(cos), _ptr(sin), pairs, 1 if interleaved else 0, _ptr(q_tc), n, heads,
                                     dim, rot_dim, hd, stream), "latent_q_unfold")
    o = attention_tc(q_tc, k_tmp, v_tmp, batch, mtile_seq, mtile_q0, n_mma_tiles, heads, scale)
    out = torch.empty((n, heads * vdim), dtype=q.dtype, device=q.device)
    _check(lib().ptb_gate_heads(_ptr(o), _ptr(gate), ctypes.c_longlong(gate.stride(0)), _ptr(out), n, heads, vdim, hd,
                                stream), "gate_heads")
    return out


# ------------------------------------------------------------------------------------------------
# Block-diagonal linear layers and the gated linear recurrence
BLOCK_LINEAR_LIBRARY_ROWS = 256   # rows from which block_linear's product is the library's batched one (bfloat16)


def block_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
                 out_dtype: Optional[torch.dtype] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t, g] = act(w[g] @ x[t, g] + bias[g]) [* sigmoid(gate[t, g])]: ``x`` [tokens, groups, K] (any
    strides with unit stride along K), ``w`` [groups, N, K], ``bias`` [groups, N] float32, ``gate``
    [tokens, groups * N] (rows may be wider apart). ``act``: "none" or "sigmoid". Returns
    [tokens, groups, N] in ``out_dtype`` (float32, or the input's dtype)."""
    _need_cuda(w, bias)
    m, g, k = x.shape
    n = w.shape[1]
    if x.stride(2) != 1 or tuple(w.shape) != (g, n, k) or w.dtype != x.dtype:
        raise KernelError("block_linear: shapes or dtypes do not fit")
    if gate is not None and (gate.stride(1) != 1 or tuple(gate.shape) != (m, g * n) or gate.dtype != x.dtype):
        raise KernelError("block_linear: the gate does not fit")
    out_dtype = out_dtype or x.dtype
    y = torch.empty((m, g, n), dtype=out_dtype, device=x.device)
    if x.dtype == torch.bfloat16 and m >= BLOCK_LINEAR_LIBRARY_ROWS:
        # many rows in bfloat16: the library's batched product (as the plain linear layers use the library's
        # product for prompts), float32 out where the result is wanted in float32, then the epilogue
        if out_dtype == torch.float32:
            z = torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32)
        else:
            z = torch.bmm(x.transpose(0, 1), w.transpose(1, 2))
        _check(lib().ptb_block_epilogue(_dtype_code(z), _dtype_code(y), _ptr(z), _ptr(bias), _ptr(gate),
                                        ctypes.c_longlong(0 if gate is None else gate.stride(0)), _ptr(y), m, g, n,
                                        {"none": 0, "sigmoid": 1}[act], _stream(x)), "block_epilogue")
        return y
    _check(lib().ptb_block_linear(_dtype_code(x), _dtype_code(y), _ptr(x), ctypes.c_longlong(x.stride(0)),
                                  ctypes.c_longlong(x.stride(1)), _ptr(w), _ptr(bias), _ptr(y), _ptr(gate),
                                  ctypes.c_longlong(0 if gate is None else gate.stride(0)), m, g, n, k,
                                  {"none": 0, "sigmoid": 1}[act], _stream(x)), "block_linear")
    return y


def rglru_conv(proj: torch.Tensor, by: torch.Tensor, bx: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor,
               state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC):
    """From ``proj`` [tokens, 2 R] (gate branch | recurrent branch, before their biases): the gate branch's
    gelu_tanh and the recurrent branch's causal convolution over each sequence, earlier inputs from
    ``state`` (rows by cache slot: [S | last taps - 1 inputs]). Returns (y_act, u), [tokens, R] each."""
    _need_cuda(proj, by, bx, conv_w, conv_b, slots)
    n, two_r = proj.shape
    r = two_r // 2
    taps = conv_w.shape[1]
    if state.stride(1) != 1 or state.shape[1] != r * taps or state.dtype != torch.float32:
        raise KernelError("rglru_conv: the state rows must hold R * taps float32 values")
    y_act = torch.empty((n, r), dtype=proj.dtype, device=proj.device)
    u = torch.empty_like(y_act)
    _check(lib().ptb_rglru_conv(_dtype_code(proj), _ptr(proj), _ptr(by), _ptr(bx), _ptr(conv_w), _ptr(conv_b),
                                _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(slots), ctypes.byref(batch),
                                _ptr(y_act), _ptr(u), r, taps, _stream(proj)), "rglru_conv")
    return y_act, u


def rglru_scan(gates: torch.Tensor, u: torch.Tensor, y_act: torch.Tensor, lam: torch.Tensor, proj: torch.Tensor,
               bx: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC, blocks: int, taps: int,
               decay: float) -> torch.Tensor:
    """The recurrence over each sequence's new tokens from and into ``state``; ``gates``
    [tokens, blocks, 2 * R / blocks] float32 (recurrence gate | input gate, after their sigmoid).
    Returns (S * y_act) [tokens, R] in the model dtype."""
    _need_cuda(gates, u, y_act, lam, proj, bx, slots)
    n, r = u.shape
    if gates.dtype != torch.float32 or gates.numel() != n * 2 * r or state.stride(1) != 1 or state.shape[1] != r * taps:
        raise KernelError("rglru_scan: gates or state do not fit")
    out = torch.empty_like(u)
    _check(lib().ptb_rglru_scan(_dtype_code(u), _ptr(gates), _ptr(u), _ptr(y_act), _ptr(lam), _ptr(proj), _ptr(bx),
                                _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(slots), ctypes.byref(batch),
                                _ptr(out), r, blocks, taps, ctypes.c_float(decay), _stream(u)), "rglru_scan")
    return out


def rglru_scan_chunks(gates: torch.Tensor, u: torch.Tensor, y_act: torch.Tensor, lam: torch.Tensor, proj: torch.Tensor,
                      bx: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC, blocks: int, taps: int,
                      decay: float, chunk_seq: torch.Tensor, chunk_q0: torch.Tensor, seq_chunk0: torch.Tensor,
                      n_chunks: int, chunk_len: int) -> torch.Tensor:
    """``rglru_scan`` for long prompts: the sequences are cut into chunks of ``chunk_len`` tokens
    (``chunk_seq``, ``chunk_q0``: sequence and first token of each; ``seq_chunk0``: a sequence's first chunk)
    that run side by side and are joined in order (three passes)."""
    _need_cuda(gates, u, y_act, lam, proj, bx, slots, chunk_seq, chunk_q0, seq_chunk0)
    n, r = u.shape
    if gates.dtype != torch.float32 or gates.numel() != n * 2 * r or state.stride(1) != 1 or state.shape[1] != r * taps:
        raise KernelError("rglru_scan_chunks: gates or state do not fit")
    out = torch.empty_like(u)
    work = torch.empty(3 * n_chunks * r, dtype=torch.float32, device=u.device)
    _check(lib().ptb_rglru_scan_chunks(_dtype_code(u), _ptr(gates), _ptr(u), _ptr(y_act), _ptr(lam), _ptr(proj), _ptr(bx),
                                       _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(slots), ctypes.byref(batch),
                                       _ptr(chunk_seq), _ptr(chunk_q0), _ptr(seq_chunk0), n_chunks, chunk_len, _ptr(work),
                                       _ptr(out), r, blocks, taps, ctypes.c_float(decay), _stream(u)), "rglru_scan_chunks")
    global launches
    launches += 2
    return out


# ------------------------------------------------------------------------------------------------
# Routed experts
EXPERT_TILE_ROWS = (16, 64)   # rows of a tile of the grouped products: few pairs, many pairs
EXPERT_MMA_TILE_ROWS = (64, 128)   # rows of a tile of the tensor-core kernel


ROUTE_SCORES = {"softmax": 0, "sigmoid": 1}


def route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], n_groups: int, keep: int, top: int,
          scale: float, score: str = "softmax", extra: int = 0, group_top: int = 1, normalize: bool = False):
    """Router of a mixture of experts, float32: scores = softmax over all outputs (or a sigmoid per output),
    choice by score + correction (None: no correction) among the ``keep`` best of ``n_groups`` groups,
    weights = score * scale. Returns (ids int32 [tokens, top], weights float32 [tokens, top]).

    ``group_top`` 2: a group is scored by the sum of its two largest choice scores instead of its largest.
    ``normalize``: weights = score / (sum of the chosen scores + 1e-20) * scale. ``extra``: the last ``extra`` rows of
    ``w_router`` are no router outputs; their logits are formed with the others (same input, same float32 sums) and the
    call returns (ids, weights, logits float32 [tokens, outputs + extra])."""
    _need_cuda(h, w_router, correction)
    n_tokens, width = h.shape
    n = w_router.shape[0] - int(extra)
    if (w_router.dtype != torch.float32 or (correction is not None and correction.dtype != torch.float32)
            or w_router.shape[1] != width):
        raise KernelError("route: the router's matrix and correction are float32 [outputs, width] and [outputs]")
    ids = torch.empty((n_tokens, top), dtype=torch.int32, device=h.device)
    gates = torch.empty((n_tokens, top), dtype=torch.float32, device=h.device)
    logits = torch.empty((n_tokens, n + int(extra)), dtype=torch.float32, device=h.device)
    _check(lib().ptb_route_grouped(_dtype_code(h), _ptr(h), _ptr(w_router), _ptr(correction), _ptr(logits), _ptr(ids),
                                   _ptr(gates), n_tokens, width, n, n_groups, keep, top, ctypes.c_float(scale),
                                   ROUTE_SCORES[score], int(extra), int(group_top), 1 if normalize else 0, _stream(h)),
           "route")
    global launches
    launches += 1       # the logits and the choice are two kernels
    return (ids, gates, logits) if extra else (ids, gates)


def routed_experts(h: torch.Tensor, ids: torch.Tensor, gates: torch.Tensor, w_gate_up: torch.Tensor,
                   w_down: torch.Tensor, base: Optional[torch.Tensor] = None, mma_tile_rows: int = 0,
                   plain_act: Optional[str] = None, shared: Optional[torch.Tensor] = None,
                   shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """base + sum over a token's choices of weight * expert(h): experts ``w_gate_up`` [E, 2 F, width]
    (gate rows, then up rows) and ``w_down`` [E, width, F] compute down(silu(gate h) * (up h)); an id >= E
    is an identity expert. Pairs are sorted by expert on the device and run as tiles of grouped
    products. Returns [tokens, width] in ``base``'s dtype (float32 without a base).

    With ``plain_act`` (an activation's name) the experts have no gate and take their weight on the input:
    ``w_gate_up`` is [E, F, width] and the result is base + sum of down(act(up (weight * h))).

    ``shared`` (float32 [tokens, width]): the result of an expert that every token uses, added in the same kernel, times
    sigmoid(``shared_gate``) where that is given (float32 [tokens, 1], a view whose rows may lie wider apart)."""
    _need_cuda(h, ids, gates, w_gate_up, w_down, base, shared)
    if shared is not None and (shared.dtype != torch.float32 or shared.shape != h.shape):
        raise KernelError("routed_experts: the shared expert's rows are float32 [tokens, width]")
    if shared_gate is not None and (shared is None or shared_gate.dtype != torch.float32 or shared_gate.shape[0] != h.shape[0]):
        raise KernelError("routed_experts: the shared expert's gate is one float32 logit per token")
    n_tokens, width = h.shape
    top = ids.shape[1]
    n_experts, two_f, _ = w_gate_up.shape
    f = two_f // 2 if plain_act is None else two_f
    first, act = (0, 0) if plain_act is None else (2, ACTIVATIONS[plain_act])
    scale = None if plain_act is None else gates
    pairs = n_tokens * top
    # bfloat16 with row sizes in whole 16-byte words: the tensor-core kernel (tiles of 64 rows); else float32 FMAs
    mma = h.dtype == torch.bfloat16 and width % 8 == 0 and f % 8 == 0
    if mma:
        # tiles of 64 rows; 128 are built and tested too, but with about 200 rows an expert they were slower
        # (3.8 against 3.3 ms for four layers of 12,288 pairs over 64 experts): half-empty last tiles, fewer blocks an SM
        tile_rows = mma_tile_rows or EXPERT_MMA_TILE_ROWS[0]
        if tile_rows not in EXPERT_MMA_TILE_ROWS:
            raise KernelError(f"routed_experts: tiles of {EXPERT_MMA_TILE_ROWS} rows, got {tile_rows}")
    else:
        tile_rows = EXPERT_TILE_ROWS[0] if pairs <= 8 * n_experts else EXPERT_TILE_ROWS[1]
    max_tiles = pairs // tile_rows + min(pairs, n_experts)
    L = lib()
    plan = torch.empty(int(L.ptb_expert_plan_words(pairs, max_tiles)), dtype=torch.int32, device=h.device)
    stream = _stream(h)
    _check(L.ptb_expert_plan(_ptr(ids), _ptr(plan), pairs, n_experts, tile_rows, max_tiles, stream), "expert_plan")
    code = _dtype_code(h)
    a = torch.empty((pairs, f), dtype=h.dtype, device=h.device)
    y = torch.empty((pairs, width), dtype=torch.float32, device=h.device)
    if mma:
        _check(L.ptb_expert_linear_mma(first, _ptr(h), _ptr(w_gate_up), _ptr(a), _ptr(plan), pairs, max_tiles, top, f, width,
                                       tile_rows, _ptr(scale), act, stream), "expert_linear_mma (gate, up)")
        _check(L.ptb_expert_linear_mma(1, _ptr(a), _ptr(w_down), _ptr(y), _ptr(plan), pairs, max_tiles, top, width, f,
                                       tile_rows, None, 0, stream), "expert_linear_mma (down)")
    else:
        _check(L.ptb_expert_linear(code, first, _ptr(h), _ptr(w_gate_up), _ptr(a), _ptr(plan), pairs, max_tiles, top, f, width,
                                   tile_rows, _ptr(scale), act, stream), "expert_linear (gate, up)")
        _check(L.ptb_expert_linear(code, 1, _ptr(a), _ptr(w_down), _ptr(y), _ptr(plan), pairs, max_tiles, top, width, f,
                                   tile_rows, None, 0, stream), "expert_linear (down)")
    if base is not None and (base.shape != h.shape or base.dtype not in (torch.float32, h.dtype)):
        raise KernelError("routed_experts: base must have the input's shape, in float32 or the input's dtype")
    out = torch.empty((n_tokens, width), dtype=torch.float32 if base is None else base.dtype, device=h.device)
    row_of_pair = plan[1 + 3 * max_tiles:1 + 3 * max_tiles + pairs]
    _check(L.ptb_expert_combine_shared(code, _dtype_code(out), _ptr(base), _ptr(h), _ptr(y), _ptr(ids),
                                       _ptr(gates if plain_act is None else None),
                                       _ptr(row_of_pair), _ptr(out), n_tokens, width, top, _ptr(shared), _ptr(shared_gate),
                                       0 if shared_gate is None else shared_gate.stride(0), stream), "expert_combine")
    return out


# ------------------------------------------------------------------------------------------------
# Linear attention with a fixed decay per head; norms and gates around mixers; the clamped gated unit
LINEAR_ATTENTION_CHUNK = 64   # ptb_linear_attention_chunk_tokens()


def linear_attention_chunks_supports(dim: int, v_dim: int) -> bool:
    return bool(lib().ptb_linear_attention_chunks_supports(dim, v_dim))


def linear_attention_mma_takes(proj: torch.Tensor, dim: int, v_dim: int) -> bool:
    """Do the tensor-core passes of the chunked form take this projection (bfloat16, sizes of 64 or 128, rows and the
    q, k, v parts at whole 16-byte words)?"""
    return (proj.dtype == torch.bfloat16 and bool(lib().ptb_linear_attention_mma_supports(dim, v_dim))
            and proj.data_ptr() % 16 == 0 and proj.stride(0) % 8 == 0)


def linear_attention(proj: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC, decay: torch.Tensor,
                     heads: int, dim: int, v_dim: int, act: str = "silu", chunks=None, single_tokens: bool = False) -> torch.Tensor:
    """Per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over the step's tokens, continuing and leaving
    each sequence's S [heads, dim, v_dim] in ``state`` [slots, heads * dim * v_dim] (float32; rows may lie wider
    apart). ``proj`` [tokens, >= 2 heads dim + heads v_dim] holds q, k, v side by side (rows may lie wider apart);
    ``act`` "silu" is applied to all three as they are read. ``chunks``: (chunk_seq, chunk_q0, seq_chunk0, n_chunks)
    for the chunked form (prompts), None for the token-by-token form; ``single_tokens``: every sequence of the step
    brings one token (the state is then updated where it lies). Returns float32 [tokens, heads * v_dim]."""
    _need_cuda(decay, slots)
    n = proj.shape[0]
    if state.dtype != torch.float32 or state.shape[1] != heads * dim * v_dim or state.stride(1) != 1:
        raise KernelError("linear_attention: the state is float32 [slots, heads * dim * v_dim]")
    _check_rows(proj, proj.shape, proj.dtype, "linear_attention: proj")
    if act not in ("none", "silu") or decay.dtype != torch.float32 or decay.numel() != heads:
        raise KernelError("linear_attention: act is 'none' or 'silu'; decay is float32 [heads]")
    out = torch.empty((n, heads * v_dim), dtype=torch.float32, device=proj.device)
    code, a = _dtype_code(proj), 1 if act == "silu" else 0
    if single_tokens:
        _check(lib().ptb_linear_attention_token(code, _ptr(proj), proj.stride(0), _ptr(state), state.stride(0), _ptr(slots),
                                                ctypes.byref(batch), _ptr(decay), _ptr(out), heads, dim, v_dim, a,
                                                _stream(proj)), "linear_attention_token")
        return out
    if chunks is None:
        _check(lib().ptb_linear_attention_scan(code, _ptr(proj), proj.stride(0), _ptr(state), state.stride(0), _ptr(slots),
                                               ctypes.byref(batch), _ptr(decay), _ptr(out), heads, dim, v_dim, a,
                                               _stream(proj)), "linear_attention_scan")
        return out
    chunk_seq, chunk_q0, seq_chunk0, n_chunks = chunks
    sums = torch.empty((n_chunks, heads, dim, v_dim), dtype=torch.float32, device=proj.device)
    global launches
    if linear_attention_mma_takes(proj, dim, v_dim):
        # bfloat16 with keys and values of 64 or 128: passes 1 and 3 on the tensor cores, pass 2 as it is
        L, stream, args = lib(), _stream(proj), (ctypes.byref(batch), _ptr(chunk_seq), _ptr(chunk_q0), n_chunks, _ptr(decay))
        _check(L.ptb_linear_attention_chunks_mma(0, _ptr(proj), proj.stride(0), *args, _ptr(sums), None, heads, dim, v_dim, a,
                                                 stream), "linear_attention_chunks_mma (sums)")
        _check(L.ptb_linear_attention_chunk_join(_ptr(sums), _ptr(state), state.stride(0), _ptr(slots), ctypes.byref(batch),
                                                 _ptr(seq_chunk0), _ptr(decay), heads, dim, v_dim, stream),
               "linear_attention_chunk_join")
        _check(L.ptb_linear_attention_chunks_mma(1, _ptr(proj), proj.stride(0), *args, _ptr(sums), _ptr(out), heads, dim, v_dim,
                                                 a, stream), "linear_attention_chunks_mma (outputs)")
        return out
    _check(lib().ptb_linear_attention_chunks(code, _ptr(proj), proj.stride(0), _ptr(state), state.stride(0), _ptr(slots),
                                             ctypes.byref(batch), _ptr(chunk_seq), _ptr(chunk_q0), _ptr(seq_chunk0),
                                             n_chunks, _ptr(decay), _ptr(sums), _ptr(out), heads, dim, v_dim, a,
                                             _stream(proj)), "linear_attention_chunks")
    launches += 2       # three kernels
    return out


def norm_gate(x: torch.Tensor, gain: torch.Tensor, gate: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
              out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of float32 rows ``x`` times ``gain`` times sigmoid(``gate``) times ``out_scale``, in ``out_dtype``.
    ``gate`` and ``out`` [rows, width] are of ``out_dtype``; their rows may lie wider apart."""
    _need_cuda(x, gain)
    n, width = x.shape
    if x.dtype != torch.float32:
        raise KernelError("norm_gate takes float32 rows")
    if out is None:
        out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    _check_rows(out, (n, width), out_dtype, "norm_gate: out")
    if gate is not None:
        _check_rows(gate, (n, width), out_dtype, "norm_gate: gate")
    _check(lib().ptb_norm_gate(_ptr(x), _ptr(gain), _dtype_code(out), _ptr(gate), 0 if gate is None else gate.stride(0),
                               _dtype_code(out), _ptr(out), out.stride(0), n, width, ctypes.c_float(eps),
                               ctypes.c_float(out_scale), _stream(x)), "norm_gate")
    return out


def qk_norm_store(proj: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, batch: StepBatchC,
                  q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int,
                  v_dim: int, eps: float, write_cache: bool = True) -> torch.Tensor:
    """``proj`` [tokens, >= (heads + kv_heads) dim + kv_heads v_dim] holds q, k, v side by side (rows may lie wider
    apart). Queries and keys are RMS-normed per head with the gains [dim] (None: as they are); keys and values go
    into the paged pools at the tokens' positions. Returns q [tokens, heads, dim]."""
    _need_cuda(k_pool, v_pool, q_gain, k_gain)
    _check_rows(proj, proj.shape, proj.dtype, "qk_norm_store: proj")
    q = torch.empty((proj.shape[0], heads, dim), dtype=proj.dtype, device=proj.device)
    _check(lib().ptb_qk_norm_store(_dtype_code(proj), _ptr(proj), proj.stride(0), _ptr(q), _ptr(k_pool), _ptr(v_pool),
                                   ctypes.byref(batch), _ptr(q_gain), _ptr(k_gain), heads, kv_heads, dim, v_dim,
                                   ctypes.c_float(eps), 1 if write_cache else 0, _stream(proj)), "qk_norm_store")
    return q


def post_norm_add(x: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float, mult: float,
                  gain_next: Optional[torch.Tensor] = None, eps_next: float = 0.0,
                  next_dtype: Optional[torch.dtype] = None):
    """The float32 stream ``x`` plus ``mult`` times the RMS norm (gain ``gain``) of a branch's result ``y``
    (float32 or bfloat16). With ``gain_next`` also the RMS norm of the new stream in ``next_dtype``:
    returns ``out`` or ``(out, next)``."""
    _need_cuda(x, y, gain, gain_next)
    if x.dtype != torch.float32 or x.shape != y.shape:
        raise KernelError("post_norm_add takes a float32 stream and a branch result of its shape")
    n, width = x.shape
    out = torch.empty_like(x)
    nxt = torch.empty((n, width), dtype=next_dtype, device=x.device) if gain_next is not None else None
    _check(lib().ptb_post_norm_add(_ptr(x), _dtype_code(y), _ptr(y), _ptr(gain), ctypes.c_float(eps), ctypes.c_float(mult),
                                   _ptr(out), _ptr(gain_next), ctypes.c_float(eps_next),
                                   0 if nxt is None else _dtype_code(nxt), _ptr(nxt), n, width, _stream(x)),
           "post_norm_add")
    return out if nxt is None else (out, nxt)


def embed_sum(ids: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, positions: torch.Tensor,
              status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 rows table[ids] + positions[pos]: token embeddings plus a learned vector per position."""
    _need_cuda(ids, pos, table, positions)
    if table.dtype != positions.dtype or table.shape[1] != positions.shape[1]:
        raise KernelError("embed_sum: the two tables have one dtype and one width")
    n, width = ids.numel(), table.shape[1]
    out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    _check(lib().ptb_embed_sum(_dtype_code(table), _ptr(ids), _ptr(pos), _ptr(table), _ptr(positions), _ptr(out), n, width,
                               table.shape[0], positions.shape[0], _ptr(status), _stream(table)), "embed_sum")
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _need_cuda(x)
    if x.dtype != torch.float32:
        raise KernelError("softcap_ takes float32 values")
    _check(lib().ptb_softcap(_ptr(x), ctypes.c_float(cap), ctypes.c_longlong(x.numel()), _stream(x)), "softcap")
    return x


def glu_clamp(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """[rows, 2 F] (gate columns, then up columns) -> [rows, F]: g = min(gate, limit), u = clamp(up, -limit, limit),
    g * sigmoid(alpha g) * (u + 1)."""
    _need_cuda(gate_up)
    rows, two_f = gate_up.shape
    out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().ptb_glu_clamp(_dtype_code(gate_up), _ptr(gate_up), _ptr(out), rows, two_f // 2, ctypes.c_float(limit),
                               ctypes.c_float(alpha), _stream(gate_up)), "glu_clamp")
    return out


def glu_act(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    """[rows, 2 F] (gate columns, then up columns) -> [rows, F]: act(gate) * up, with ``act`` a name of ACTIVATIONS."""
    _need_cuda(gate_up)
    rows, two_f = gate_up.shape
    out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().ptb_glu_act(_dtype_code(gate_up), _ptr(gate_up), _ptr(out), rows, two_f // 2, ACTIVATIONS[act],
                             _stream(gate_up)), "glu_act")
    return out


# ------------------------------------------------------------------------------------------------
# The Dynamic Tanh norm with the short convolution on a mixer's input; the matrix memory with exponential gates
DYT_MAX_TAPS = 8


def dyt(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
        conv: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
        batch: Optional[StepBatchC] = None, single_tokens: bool = False, pending: Optional[torch.Tensor] = None,
        pending_bias: Optional[torch.Tensor] = None):
    """h = tanh(alpha x) * weight + bias, elementwise in float32 (``alpha``: one float32 on the device), written in
    ``out_dtype``. With ``conv`` (float32 [width, taps]) the result is h_t + sum_j conv[:, j] h_(t - taps + 1 + j) over
    each sequence's tokens; the last ``taps - 1`` rows of h per sequence are read from and left in ``state``
    [slots, >= (taps - 1) width] (float32; rows may lie wider apart). With ``pending`` (float32 [n, width], beside a
    float32 ``x``; ``pending_bias`` float32 [width] or None) the rows are x + (pending + pending_bias): the sum is
    formed on the way and returned too, as (result, sum)."""
    _need_cuda(x, alpha, weight, bias, conv, slots, pending, pending_bias)
    n, width = x.shape
    total = None
    if pending is not None:
        if x.dtype != torch.float32 or pending.dtype != torch.float32 or tuple(pending.shape) != (n, width) \
                or not x.is_contiguous() or not pending.is_contiguous():
            raise KernelError("dyt: a pending addend is float32 [n, width] beside a float32 x, both contiguous")
        if pending_bias is not None and (pending_bias.dtype != torch.float32 or pending_bias.numel() != width):
            raise KernelError("dyt: the pending addend's bias is float32 [width]")
        total = torch.empty_like(x)
    elif pending_bias is not None:
        raise KernelError("dyt: a bias of the pending addend without the addend")
    if alpha.dtype != torch.float32 or alpha.numel() != 1 or weight.dtype != torch.float32 or weight.numel() != width:
        raise KernelError("dyt: alpha is one float32, the weight float32 [width]")
    y = torch.empty((n, width), dtype=out_dtype, device=x.device)
    taps = 0
    if conv is not None:
        taps = conv.shape[1]
        if conv.dtype != torch.float32 or conv.shape[0] != width or not (1 <= taps <= DYT_MAX_TAPS) or batch is None:
            raise KernelError(f"dyt: the convolution is float32 [width, 1..{DYT_MAX_TAPS} taps] and needs the step's batch")
        if taps > 1 and (state is None or state.dtype != torch.float32 or state.shape[1] < (taps - 1) * width
                         or state.stride(1) != 1):
            raise KernelError("dyt: the convolution's state is float32 [slots, >= (taps - 1) * width]")
    _check(lib().ptb_dyt(_dtype_code(x), _ptr(x), _ptr(alpha), _ptr(weight), _ptr(bias), _dtype_code(y), _ptr(y), n, width,
                         _ptr(conv), _ptr(state if taps > 1 else None), 0 if state is None or taps <= 1 else state.stride(0),
                         _ptr(slots), ctypes.byref(batch) if batch is not None else None, taps, 1 if single_tokens else 0,
                         _ptr(pending), _ptr(pending_bias), _ptr(total), _stream(x)), "dyt")
    return y if pending is None else (y, total)


MLSTM_MAX_DIM = 256   # ptb_mlstm_max_dim()


def mlstm_state_floats(heads: int, dim: int, v_dim: int) -> int:
    """float32 values of one sequence's state: S, and a copy of n and m for every stretch of 32 value columns."""
    return heads * (dim * v_dim + ((v_dim + 31) // 32) * (dim + 1))


MLSTM_CHUNK = 64   # ptb_mlstm_chunk_tokens()


def mlstm_chunks_takes(proj: torch.Tensor, dim: int, v_dim: int) -> bool:
    """Does the chunked form of the matrix memory take this projection (bfloat16, sizes of 64 or 128, rows and the q, k, v
    parts at whole 16-byte words)?"""
    return (proj.dtype == torch.bfloat16 and bool(lib().ptb_mlstm_chunks_supports(dim, v_dim))
            and proj.data_ptr() % 16 == 0 and proj.stride(0) % 8 == 0 and (2 * dim) % 8 == 0)


def mlstm(proj: torch.Tensor, gates: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
          state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC, heads: int, dim: int, v_dim: int,
          q_scale: float, chunks=None) -> torch.Tensor:
    """The matrix memory with exponential gates over the step's tokens, continuing and leaving each sequence's state.
    ``proj`` [tokens, >= 2 heads dim + heads v_dim] holds q, k, v side by side (rows may lie wider apart); ``gates``
    float32 [tokens, 2 heads] holds the input and forget gates' projections and is overwritten with the gates'
    logarithms ``cap tanh((g + b) / cap)`` and ``logsigmoid`` of the same; ``state`` [slots, >= mlstm_state_floats]
    float32. ``chunks``: (chunk_seq, chunk_q0, seq_chunk0, n_chunks) for the chunked form on the tensor cores (prompts;
    ``mlstm_chunks_takes`` says whether it takes the projection), None for the token-by-token form. Returns float32
    [tokens, heads * v_dim]: S^T q / (max(|n . q|, exp(-m)) + 1e-6)."""
    _need_cuda(gates, bias_i, bias_f, slots)
    _check_rows(proj, proj.shape, proj.dtype, "mlstm: proj")
    n = proj.shape[0]
    if gates.dtype != torch.float32 or tuple(gates.shape) != (n, 2 * heads):
        raise KernelError("mlstm: the gates are float32 [tokens, 2 * heads]")
    if state.dtype != torch.float32 or state.shape[1] < mlstm_state_floats(heads, dim, v_dim) or state.stride(1) != 1:
        raise KernelError("mlstm: the state is float32 [slots, >= mlstm_state_floats(heads, dim, v_dim)]")
    _check(lib().ptb_mlstm_gates(_ptr(gates), _ptr(bias_i), _ptr(bias_f), n, heads, ctypes.c_float(cap), _stream(gates)),
           "mlstm_gates")
    out = torch.empty((n, heads * v_dim), dtype=torch.float32, device=proj.device)
    if chunks is not None:
        if not mlstm_chunks_takes(proj, dim, v_dim):
            raise KernelError("mlstm: the chunked form takes bfloat16 projections with keys and values of 64 or 128 entries")
        chunk_seq, chunk_q0, seq_chunk0, n_chunks = chunks
        scratch = torch.empty(int(lib().ptb_mlstm_chunks_scratch_floats(n_chunks, heads, dim, v_dim)), dtype=torch.float32,
                              device=proj.device)
        _check(lib().ptb_mlstm_chunks(_ptr(proj), proj.stride(0), _ptr(gates), _ptr(state), state.stride(0), _ptr(slots),
                                      ctypes.byref(batch), _ptr(chunk_seq), _ptr(chunk_q0), _ptr(seq_chunk0), n_chunks,
                                      _ptr(scratch), _ptr(out), heads, dim, v_dim, ctypes.c_float(q_scale), _stream(proj)),
               "mlstm_chunks")
        global launches
        launches += 2       # three kernels
        return out
    _check(lib().ptb_mlstm_scan(_dtype_code(proj), _ptr(proj), proj.stride(0), _ptr(gates), _ptr(state), state.stride(0),
                                _ptr(slots), ctypes.byref(batch), _ptr(out), heads, dim, v_dim, ctypes.c_float(q_scale),
                                _stream(proj)), "mlstm_scan")
    return out


def head_norm_gate(x: torch.Tensor, gain: torch.Tensor, gate: Optional[torch.Tensor], heads: int, eps: float,
                   out_dtype: torch.dtype, gate_act: str = "sigmoid") -> torch.Tensor:
    """Every head's stretch of the float32 rows ``x`` [tokens, heads * v_dim] divided by its root mean square, times
    ``gain`` [heads * v_dim] times sigmoid(``gate``) (of ``out_dtype``; rows may lie wider apart), in ``out_dtype``.
    ``gate_act`` "silu": times gate * sigmoid(gate) instead."""
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"head_norm_gate: the gate's activation is 'sigmoid' or 'silu', got {gate_act!r}")
    _need_cuda(x, gain)
    n, width = x.shape
    if x.dtype != torch.float32 or width % heads or gain.dtype != torch.float32 or gain.numel() != width:
        raise KernelError("head_norm_gate takes float32 rows [tokens, heads * v_dim] and a float32 gain of that width")
    out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    if gate is not None:
        _check_rows(gate, (n, width), out_dtype, "head_norm_gate: gate")
    _check(lib().ptb_head_norm_gate_act(_ptr(x), _ptr(gain), _dtype_code(out), _ptr(gate),
                                        0 if gate is None else gate.stride(0), _ptr(out), out.stride(0), n, heads,
                                        width // heads, ctypes.c_float(eps), 1 if gate_act == "silu" else 0, _stream(x)),
           "head_norm_gate")
    return out


# ------------------------------------------------------------------------------------------------
# Gated linear attention: a decay per token and key channel
GLA_MAX_DIM = 256   # ptb_gla_max_dim()
GLA_CHUNK = 64      # ptb_gla_chunk_tokens()


def gla_decay_(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> torch.Tensor:
    """In place on float32 rows [tokens, width]: z <- logsigmoid(z + bias) / tau, the logarithm of the decay
    sigmoid(z + bias) ** (1 / tau). ``bias`` float32 [width] or None."""
    _need_cuda(z, bias)
    if z.dtype != torch.float32 or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != z.shape[1])):
        raise KernelError("gla_decay_ takes float32 rows and a float32 bias of their width")
    _check(lib().ptb_gla_decay(_ptr(z), _ptr(bias), z.shape[0], z.shape[1], ctypes.c_float(tau), _stream(z)), "gla_decay")
    return z


def gla(proj: torch.Tensor, log_decay: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, batch: StepBatchC, heads: int,
        dim: int, v_dim: int, q_scale: float, chunks=None) -> torch.Tensor:
    """Per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t * q_scale) over the step's tokens, continuing and
    leaving each sequence's S [heads, dim, v_dim] in ``state`` [slots, heads * dim * v_dim] (float32; rows may lie wider
    apart). ``proj`` [tokens, >= 2 heads dim + heads v_dim] holds q, k, v side by side (rows may lie wider apart);
    ``log_decay`` float32 [tokens, heads * dim] the logarithms of the decays a_t. ``chunks``: (chunk_seq, chunk_q0,
    seq_chunk0, n_chunks) for the chunked form (prompts), None to walk every sequence token by token. Returns float32
    [tokens, heads * v_dim]."""
    _need_cuda(log_decay, slots)
    n = proj.shape[0]
    if state.dtype != torch.float32 or state.shape[1] != heads * dim * v_dim or state.stride(1) != 1:
        raise KernelError("gla: the state is float32 [slots, heads * dim * v_dim]")
    if log_decay.dtype != torch.float32 or tuple(log_decay.shape) != (n, heads * dim):
        raise KernelError("gla: the decays' logarithms are float32 [tokens, heads * dim]")
    _check_rows(proj, proj.shape, proj.dtype, "gla: proj")
    out = torch.empty((n, heads * v_dim), dtype=torch.float32, device=proj.device)
    if chunks is None:
        _check(lib().ptb_gla_walk(_dtype_code(proj), _ptr(proj), proj.stride(0), _ptr(log_decay), _ptr(state), state.stride(0),
                                  _ptr(slots), ctypes.byref(batch), _ptr(out), heads, dim, v_dim, ctypes.c_float(q_scale),
                                  _stream(proj)), "gla_walk")
        return out
    chunk_seq, chunk_q0, seq_chunk0, n_chunks = chunks
    sums = torch.empty((n_chunks, heads, dim, v_dim), dtype=torch.float32, device=proj.device)
    decays = torch.empty((n_chunks, heads, dim), dtype=torch.float32, device=proj.device)
    _check(lib().ptb_gla_chunks(_dtype_code(proj), _ptr(proj), proj.stride(0), _ptr(log_decay), _ptr(state), state.stride(0),
                                _ptr(slots), ctypes.byref(batch), _ptr(chunk_seq), _ptr(chunk_q0), _ptr(seq_chunk0), n_chunks,
                                _ptr(sums), _ptr(decays), _ptr(out), heads, dim, v_dim, ctypes.c_float(q_scale),
                                _stream(proj)), "gla_chunks")
    global launches
    launches += 2       # three kernels
    return out
