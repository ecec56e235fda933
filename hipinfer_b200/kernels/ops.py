"""The operations the parts are made of, each a call into the compiled sm_100a kernels on the
current CUDA stream. Tensors are torch tensors used as typed device buffers (the reference's
binding does the same, scripts/hipinfer.py:105-190); no torch operator computes anything here.

Element types are `torch.float32` and `torch.bfloat16`. Which kernel runs is chosen from the
element types and the sizes alone (never from what else is in the batch in a way that would
change a row's arithmetic beyond rounding): the tensor-core kernels of the `fast` library for
bfloat16 operands when they take the sizes, the plain 32-bit kernels of `core` otherwise.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_p, _i, _l, _f = C.c_void_p, C.c_int, C.c_long, C.c_float

_SIGS = {
    "core": {
        "hb_embed": [_p, _i, _p, _p, _i, _i, _p],
        "hb_rmsnorm": [_p, _p, _i, _p, _i, _p, _i, _i, _f, _p],
        "hb_gemm_simt": [_p, _i, _l, _p, _i, _l, _p, _i, _l, _i, _i, _i, _i, _p],
        "hb_swiglu": [_p, _i, _l, _p, _i, _l, _i, _i, _i, _p],
        "hb_rope_table": [_p, _p, _i, _i, C.c_double, _p],
        "hb_rope_kv": [_p, _i, _l, _p, _p, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
        "hb_attn_rows": [_p, _i, _p, _p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p],
        "hb_attn_merge": [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p],
        "hb_sample": [_p, _l, _i, _i, _p, _p, _p, _p, _p, _p],
        "hb_convert": [_p, _i, _p, _i, _l, _p],
        "hb_feed_tokens": [_p, _p, _p, _i, _p],
        "hb_embed_pos": [_p, _p, _i, _p, _p, _p, _i, _i, _f, _p],
        "hb_layernorm": [_p, _p, _p, _i, _p, _i, _p, _i, _i, _f, _p],
        "hb_gated_act": [_p, _i, _l, _p, _i, _l, _i, _i, _i, _i, _p],
        "hb_rope_norm_store": [_p, _l, _i, _i, _i, _p, _p, _p, _i, _i, _i, _i, _f, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i,
                               _f, _p],
        "hb_polynorm": [_p, _l, _p, _i, _l, _i, _i, _f, _f, _f, _f, _f, _p],
        "hb_scale_add": [_p, _p, _l, _p, _i, _i, _i, _p],
        "hb_bias_act": [_p, _l, _p, _i, _p, _i, _l, _i, _i, _i, _p],
        "hb_qkv_bias_store": [_p, _l, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
        "hb_gemm_simt_scaled": [_p, _i, _l, _p, _i, _l, _p, _l, _i, _i, _i, _p, _p],
    },
    "seqmix": {
        "hb_attn_masked": [_p, _i, _l, _p, _l, _p, _l, _i, _p, _i, _p, _p, _p, _p, _l, _i, _i, _p, _i, _l, _i, _i, _i, _i, _i,
                           _i, _i, _i, _i, _i, _f, _p, _i, _p, _l, _p, _i, _p],
        "hb_latent_prepare": [_p, _l, _i, _i, _i, _p, _p, _i, _p, _p, _p, _i, _f, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p],
        "hb_heads_linear": [_p, _l, _l, _p, _i, _p, _i, _l, _l, _i, _i, _i, _i, _p, _l, _i, _i, _i, _p, _p, _p, _p, _i, _i, _i, _p],
        "hb_gather_rows": [_p, _i, _p, _p, _i, _i, _i, _p],
        "hb_attn_masked_flash_supported": [_i, _i],
        "hb_attn_masked_heads_supported": [_i, _i, _i, _i, _i],
        "hb_attn_masked_heads": [_p, _l, _p, _l, _l, _l, _p, _l, _l, _l, _i, _p, _i, _p, _p, _p, _p, _l, _i, _i, _p, _i, _l, _i, _i,
                                 _i, _i, _i, _i, _i, _i, _i, _i, _f, _p, _i, _p, _l, _i, _p],
        "hb_attn_masked_flash": [_p, _l, _p, _l, _l, _l, _p, _l, _l, _l, _p, _i, _p, _p, _p, _i, _i, _i, _i, _p, _p, _l, _i, _i, _p,
                                 _i, _l, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p],
        "hb_gla": [_p, _l, _i, _i, _i, _i, _p, _l, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _f, _p],
    },
    "hybrid": {
        "hb_streams_norm": [_p, _p, _i, _p, _p, _i, _p, _i, _i, _i, _f, _p],
        "hb_streams_update": [_p, _p, _p, _p, _f, _i, _i, _i, _p],
        "hb_streams_update_norm": [_p, _p, _p, _p, _f, _p, _p, _i, _p, _i, _i, _i, _i, _f, _p],
        "hb_streams_expand": [_p, _p, _i, _i, _i, _p],
        "hb_glu_bias": [_p, _l, _p, _i, _p, _i, _l, _i, _i, _i, _i, _f, _f, _p],
        "hb_scale_bias_rows": [_p, _l, _p, _i, _f, _i, _i, _p],
        "hb_ssd_conv": [_p, _l, _i, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p],
        "hb_ssd_scan": [_p, _l, _p, _l, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p],
        "hb_ssd_gate_norm": [_p, _p, _l, _p, _i, _p, _i, _i, _i, _i, _f, _p],
        "hb_selective_scan": [_p, _l, _p, _l, _p, _l, _p, _l, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _l, _i, _i, _i, _i, _i, _p, _p,
                              _p],
        "hb_split_rounded": [_p, _l, _p, _p, _i, _i, _p],
        "hb_residual_norm": [_p, _p, _p, _p, _p, _p, _i, _f, _f, _f, _p, _f, _p, _i, _i, _i, _p],
        "hb_moe_route": [_p, _i, _l, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p],
        "hb_moe_gate_up_rows": [_p, _i, _l, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _p],
        "hb_moe_down_rows": [_p, _i, _p, _i, _p, _p, _l, _i, _i, _i, _i, _p],
        "hb_moe_sort": [_p, _p, _p, _p, _i, _i, _p],
        "hb_moe_grouped": [_p, _i, _l, _p, _i, _p, _i, _p, _p, _i, _i, _i, _p],
        "hb_moe_gather": [_p, _i, _l, _p, _p, _i, _i, _i, _p],
        "hb_moe_act": [_p, _p, _p, _p, _i, _i, _i, _i, _p],
        "hb_moe_combine": [_p, _p, _p, _l, _i, _i, _i, _p],
    },
    "mixers": {
        "hb_delta_rule": [_p, _l, _i, _i, _i, _i, _i, _p, _l, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _f, _f,
                          _i, _p],
        "hb_attn_window": [_p, _i, _p, _p, _i, _p, _i, _p, _p, _p, _l, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f,
                           _f, _i, _p, _i, _i, _p, _l, _p, _i, _p],
        "hb_attn_window_flash": [_p, _p, _p, _p, _i, _p, _p, _p, _p, _l, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f,
                                 _f, _f, _i, _p],
        "hb_attn_window_flash_supported": [_i, _i, _i, _i, _i],
        "hb_attn_window_rows_mma_supported": [_i, _i, _i, _i, _i],
        "hb_attn_window_rows_mma": [_p, _p, _p, _p, _i, _p, _p, _p, _l, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f, _f,
                                    _p, _i, _p, _l, _p, _i, _p],
    },
}
_fn_cache = {}


class KernelError(RuntimeError):
    pass


def _fn(lib_name: str, name: str):
    key = (lib_name, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = library.load(lib_name)
        f = getattr(lib, name)
        f.argtypes = _SIGS[lib_name][name]
        f.restype = C.c_int
        _fn_cache[key] = f
    return f


_NO_LAUNCH = {"hb_attn_rows_workspace"}


def _call(lib_name: str, name: str, *args):
    library.launches[0] += 1
    r = _fn(lib_name, name)(*args)
    if r != 0:
        raise KernelError(library.load(lib_name).hb_last_error().decode())


def _stream() -> int:
    return library.current_stream()


def check_device_status() -> None:
    """To be called where the host has just waited for the device: raises `fast.KernelTimeout` if a kernel
    gave up on one of its bounded waits since the last call (its output is not valid), and clears the word.
    It reads one word of pinned host memory. The reference's counterpart: HI_CHECK after its calls
    (src/hip_compat.h:95-97) and the -1 of its entry points (src/api.cu:1827-1839)."""
    from . import fast

    fast.check_status()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU implementation")


def _rows_contiguous(t: torch.Tensor, what: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")


# ------------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[i] = table[tokens[i]] into the float32 residual stream."""
    _need_cuda(table, tokens, out)
    T, H = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and tokens.dtype == torch.int32
    assert table.is_contiguous() and table.shape[1] == H and tokens.numel() == T
    _call("core", "hb_embed", table.data_ptr(), _dt(table), tokens.data_ptr(), out.data_ptr(), T, H, _stream())
    return out


def embedding_scaled(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
                     position_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = table[tokens[i]] * scale (+ position_table[positions[i]]) into the float32 residual stream."""
    _need_cuda(table, tokens, out, position_table, positions)
    T, H = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and tokens.dtype == torch.int32
    assert table.is_contiguous() and table.shape[1] == H and tokens.numel() == T
    if position_table is not None:
        assert position_table.dtype == table.dtype and position_table.is_contiguous() and position_table.shape[1] == H
        assert positions is not None and positions.dtype == torch.int32 and positions.numel() == T
    _call("core", "hb_embed_pos", table.data_ptr(), _ptr(position_table), _dt(table), tokens.data_ptr(), _ptr(positions),
          out.data_ptr(), T, H, float(scale), _stream())
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = weight * (x[r] - mean) / sqrt(var + eps) (+ bias), r = rows[i] or i; x float32 [*, H]."""
    _need_cuda(x, weight, out, rows, bias)
    if bias is not None:
        assert bias.numel() == weight.numel() and bias.dtype == weight.dtype and bias.is_contiguous()
    M, H = out.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.shape[1] == H
    assert weight.numel() == H and weight.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == M
    else:
        assert x.shape[0] == M
    _call("core", "hb_layernorm", x.data_ptr(), weight.data_ptr(), _ptr(bias), _dt(weight), out.data_ptr(), _dt(out), _ptr(rows),
          M, H, float(eps), _stream())
    return out


def polynorm(z: torch.Tensor, coef, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3] row by row, N(t) = t / rms(t); z float32."""
    _need_cuda(z, out)
    _rows_contiguous(z, "polynorm in")
    _rows_contiguous(out, "polynorm out")
    assert z.dtype == torch.float32 and z.shape == out.shape and len(coef) == 4
    M, I = out.shape
    _call("core", "hb_polynorm", z.data_ptr(), z.stride(0), out.data_ptr(), _dt(out), out.stride(0), M, I,
          float(coef[0]), float(coef[1]), float(coef[2]), float(coef[3]), float(eps), _stream())
    return out


def scale_add(x: torch.Tensor, y: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x[m, n] += scale[n] * y[m, n]; x, y float32."""
    _need_cuda(x, y, scale)
    _rows_contiguous(y, "scale_add y")
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and x.shape == y.shape
    assert scale.numel() == x.shape[1] and scale.is_contiguous()
    _call("core", "hb_scale_add", x.data_ptr(), y.data_ptr(), y.stride(0), scale.data_ptr(), _dt(scale), x.shape[0],
          x.shape[1], _stream())
    return x


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, act: str = "none") -> torch.Tensor:
    """out = act(x + bias) for float32 rows x (a view of some columns is fine); act "none" or "tanh"."""
    _need_cuda(x, bias, out)
    _rows_contiguous(x, "bias_act in")
    _rows_contiguous(out, "bias_act out")
    assert x.dtype == torch.float32 and x.shape == out.shape
    M, n = x.shape
    _call("core", "hb_bias_act", x.data_ptr(), x.stride(0), _ptr(bias), _dt(bias) if bias is not None else 0,
          out.data_ptr(), _dt(out), out.stride(0), M, n, {"none": 0, "tanh": 1}[act], _stream())
    return out


def qkv_bias_store(qkv: torch.Tensor, bq, bk, bv, slot_map: Optional[torch.Tensor], q_out: torch.Tensor,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_q: int, kv_heads: int,
                   k_width: int, v_width: int, page_size: int) -> torch.Tensor:
    """Rows [q | k | v] of a float32 projection (+ biases): q to q_out [T, n_q], k and v to their page slots (planes
    [page, kv_heads, page_size, width]); no position encoding. slot_map None: the rows hold q alone."""
    _need_cuda(qkv, bq, bk, bv, slot_map, q_out, k_cache, v_cache)
    _rows_contiguous(qkv, "qkv_bias_store in")
    T = qkv.shape[0]
    assert qkv.dtype == torch.float32 and q_out.is_contiguous() and q_out.shape == (T, n_q)
    bias_dt = _dt(next((b for b in (bq, bk, bv) if b is not None), q_out))
    if slot_map is not None:
        assert qkv.shape[1] == n_q + kv_heads * (k_width + v_width)
        assert k_cache.dtype == v_cache.dtype == q_out.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    else:
        assert qkv.shape[1] == n_q
    _call("core", "hb_qkv_bias_store", qkv.data_ptr(), qkv.stride(0), _ptr(bq), _ptr(bk), _ptr(bv), bias_dt, _ptr(slot_map),
          q_out.data_ptr(), _ptr(k_cache) if slot_map is not None else None, _ptr(v_cache) if slot_map is not None else None,
          _dt(q_out), T, n_q, kv_heads, k_width, v_width, page_size, _stream())
    return q_out


def delta_rule(proj: torch.Tensor, offsets, w_raw: torch.Tensor, w_bias, a_bias, norm_weight, state: torch.Tensor, batch,
               out: torch.Tensor, heads: int, dim: int, decay_scale: float, unit_eps: float, eps: float,
               force_any: bool = False) -> torch.Tensor:
    """The generalized delta rule over the step's rows, request by request, from and into each request's state slot
    (csrc/delta_rule.cu). proj float32 [T, *] holds r, k, v, the removal rate's and the gate's pre-activations at the
    column `offsets` (r, k, v, a, g); w_raw float32 [T, heads * dim] the decay's; state float32 [slots, heads, dim, dim]."""
    _need_cuda(proj, w_raw, w_bias, a_bias, norm_weight, state, out)
    _rows_contiguous(proj, "delta_rule proj")
    _rows_contiguous(w_raw, "delta_rule w_raw")
    assert proj.dtype == w_raw.dtype == state.dtype == torch.float32 and state.is_contiguous() and out.is_contiguous()
    assert state.shape[1:] == (heads, dim, dim) and out.shape == (proj.shape[0], heads * dim)
    assert w_bias.dtype == a_bias.dtype == norm_weight.dtype
    r, k, v, a, g = (int(o) for o in offsets)
    _call("mixers", "hb_delta_rule", proj.data_ptr(), proj.stride(0), r, k, v, a, g, w_raw.data_ptr(), w_raw.stride(0),
          w_bias.data_ptr(), a_bias.data_ptr(), norm_weight.data_ptr(), _dt(w_bias), state.data_ptr(),
          batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(), batch.req_state_slot.data_ptr(), out.data_ptr(),
          _dt(out), batch.n_requests, heads, dim, float(decay_scale), float(unit_eps), float(eps), 1 if force_any else 0,
          _stream())
    return out


WINDOW_FLASH_MIN_ROWS = 16     # requests that bring at least this many rows go to the flash kernel of attention_window


def attention_window(q, k_cache, v_cache, batch, group: int, out, n_heads: int, n_kv_heads: int, dim: int, vdim: int,
                     maps: int, page_size: int, window: int, keep_first: int, scale: float, lam: float = 0.0,
                     post: float = 1.0, eps: float = 0.0, norm: bool = False, gate: Optional[torch.Tensor] = None,
                     gate_offset: int = 0, force_rows: bool = False, force_plain: bool = False,
                     force_simt: bool = False) -> torch.Tensor:
    """Attention of the step's rows over their requests' pages with a window that keeps the first tokens, `maps` score
    maps per head (2: out = a0 - lam * a1), keys `dim` and values `vdim` wide, the head's result optionally divided by
    its root mean square and times `post`, and times sigmoid(gate[:, gate_offset + ...]) (float32) where a gate is given
    (csrc/attention_window.cu)."""
    _need_cuda(q, k_cache, v_cache, out, gate)
    T = q.shape[0]
    bt = batch.block_tables[group]
    assert q.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype == v_cache.dtype
    assert q.shape[1] == n_heads * maps * dim and out.shape == (T, n_heads * vdim)
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape[-1] == maps * dim and v_cache.shape[-1] == vdim
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == T
    gate_ld = gate.stride(0) if gate is not None else 0
    # requests that bring WINDOW_FLASH_MIN_ROWS rows or more go to the tensor-core kernel (bfloat16, two maps, the sizes it
    # takes), the other rows of the step to the row kernel; a decode-only step is the row kernel alone
    from . import fast

    flash = (maps == 2 and norm and q.dtype == torch.bfloat16 and not fast.PLAIN_ONLY and not force_rows
             and getattr(batch, "max_q_len", 0) >= WINDOW_FLASH_MIN_ROWS
             and _fn("mixers", "hb_attn_window_flash_supported")(n_heads, n_kv_heads, dim, vdim, maps) == 1
             and (gate is None or (gate_ld % 2 == 0 and gate_offset % 2 == 0)))
    if flash:
        _call("mixers", "hb_attn_window_flash", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(), bt.stride(0),
              batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(), batch.req_ctx_len.data_ptr(), _ptr(gate), gate_ld,
              int(gate_offset), out.data_ptr(), batch.n_requests, batch.max_q_len, n_heads, n_kv_heads, dim, vdim, page_size,
              int(window), int(keep_first), float(scale), float(lam), float(post), float(eps), WINDOW_FLASH_MIN_ROWS, _stream())
        if min(batch.h_q_len) >= WINDOW_FLASH_MIN_ROWS:
            return out
    # rows with many keys are split over several blocks, which meet in a workspace (bfloat16 rows kernels only)
    lib = library.load("mixers")
    lib.hb_attn_window_workspace.restype = C.c_long
    lib.hb_attn_window_rows_mma_workspace.restype = C.c_long
    max_pos = int(getattr(batch, "max_pos", 0)) or int(bt.shape[1]) * page_size - 1
    q_len_ptr = batch.req_q_len.data_ptr() if flash else None
    if (maps == 2 and norm and q.dtype == torch.bfloat16 and not fast.PLAIN_ONLY and not force_plain and not force_simt
            and _fn("mixers", "hb_attn_window_rows_mma_supported")(n_heads, n_kv_heads, dim, vdim, maps) == 1):
        # the heads of a kv head as the rows of a warp MMA tile
        n_ws = lib.hb_attn_window_rows_mma_workspace(T, n_heads, n_kv_heads, vdim, int(window), int(keep_first), max_pos)
        ws = torch.empty(n_ws, dtype=torch.float32, device=q.device) if n_ws else None
        arrived = fast._decode_counters(q.device, T * n_kv_heads) if n_ws else None
        _call("mixers", "hb_attn_window_rows_mma", q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), bt.data_ptr(),
              bt.stride(0), batch.row_request.data_ptr(), batch.positions.data_ptr(), _ptr(gate), gate_ld, int(gate_offset),
              out.data_ptr(), T, n_heads, n_kv_heads, dim, vdim, page_size, int(window), int(keep_first), float(scale),
              float(lam), float(post), float(eps), q_len_ptr, WINDOW_FLASH_MIN_ROWS, _ptr(ws), n_ws, _ptr(arrived), max_pos,
              _stream())
        return out
    n_ws = 0 if (q.dtype != torch.bfloat16 or force_plain) else lib.hb_attn_window_workspace(
        T, n_heads, n_kv_heads, vdim, maps, int(window), int(keep_first), max_pos)
    ws = torch.empty(n_ws, dtype=torch.float32, device=q.device) if n_ws else None
    arrived = fast._decode_counters(q.device, T * n_kv_heads) if n_ws else None
    _call("mixers", "hb_attn_window", q.data_ptr(), _dt(q), k_cache.data_ptr(), v_cache.data_ptr(), _dt(k_cache),
          bt.data_ptr(), bt.stride(0), batch.row_request.data_ptr(), batch.positions.data_ptr(), _ptr(gate), gate_ld,
          int(gate_offset), out.data_ptr(), T, n_heads, n_kv_heads, dim, vdim, maps, page_size, int(window), int(keep_first),
          float(scale), float(lam), float(post), float(eps), 1 if norm else 0,
          batch.req_q_len.data_ptr() if flash else None, WINDOW_FLASH_MIN_ROWS, 1 if force_plain else 0, _ptr(ws), n_ws,
          _ptr(arrived), max_pos, _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, pending: Optional["Pending"] = None) -> torch.Tensor:
    """out[i] = weight * x[rows[i] or i] / rms; x float32 [*, H], out [M, H] float32 or bfloat16.
    pending: a sum that has yet to be added into x; it is added first (in the same kernel where that applies)."""
    _need_cuda(x, weight, out, rows)
    M, H = out.shape
    if pending is not None:
        from . import fast

        if pending.out is x and pending.accumulate and fast.add_rmsnorm_slices_ok(x, pending.slices, weight, out):
            return fast.add_rmsnorm_slices(x, pending.slices, weight, eps, out, rows)
        pending.finish()
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and x.shape[1] == H
    assert weight.numel() == H and weight.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == M
    else:
        assert x.shape[0] == M
    _call("core", "hb_rmsnorm", x.data_ptr(), weight.data_ptr(), _dt(weight), out.data_ptr(), _dt(out), _ptr(rows),
          M, H, float(eps), _stream())
    return out


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T with the plain 32-bit kernel: a [M, K], w [N, K], out [M, N]."""
    _need_cuda(a, w, out)
    _rows_contiguous(a, "gemm a")
    _rows_contiguous(w, "gemm w")
    _rows_contiguous(out, "gemm out")
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N), (a.shape, w.shape, out.shape)
    _call("core", "hb_gemm_simt", a.data_ptr(), _dt(a), a.stride(0), w.data_ptr(), _dt(w), w.stride(0),
          out.data_ptr(), _dt(out), out.stride(0), M, N, K, 1 if accumulate else 0, _stream())
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, group: int) -> torch.Tensor:
    """out[m, i] = silu(g) * u for a gate/up matrix [M, 2I] interleaved in groups of `group` columns."""
    _need_cuda(gate_up, out)
    _rows_contiguous(gate_up, "swiglu in")
    _rows_contiguous(out, "swiglu out")
    M, I = out.shape
    assert gate_up.shape == (M, 2 * I)
    _call("core", "hb_swiglu", gate_up.data_ptr(), _dt(gate_up), gate_up.stride(0), out.data_ptr(), _dt(out),
          out.stride(0), M, I, group, _stream())
    return out


def rope_table(inv_freq: torch.Tensor, n_pos: int, magnitude: float = 1.0) -> torch.Tensor:
    """(cos, sin) float32 [n_pos, len(inv_freq), 2] of angle = float32(p) * inv_freq[i], both times `magnitude`."""
    _need_cuda(inv_freq)
    assert inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
    half = inv_freq.numel()
    table = torch.empty(n_pos, half, 2, dtype=torch.float32, device=inv_freq.device)
    _call("core", "hb_rope_table", inv_freq.data_ptr(), table.data_ptr(), n_pos, half, float(magnitude), _stream())
    return table


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_map: Optional[torch.Tensor], table: torch.Tensor,
                  q_out: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_heads: int,
                  n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                  pending: Optional["Pending"] = None) -> torch.Tensor:
    """Rotate q and k of qkv [T, (Hq + 2 Hkv) D]; q to q_out [T, Hq D]; k, v to their page slots
    (cache layout [page, Hkv, page_size, D]); slot_map None: no cache write. pending: qkv is not
    written yet, its K slices are added here (in the same kernel where that applies)."""
    _need_cuda(qkv, positions, slot_map, table, q_out, k_cache, v_cache)
    if pending is not None:
        from . import fast

        if (pending.out is qkv and not pending.accumulate and rotary_dim == head_dim and head_dim % 8 == 0
                and q_out.dtype == torch.bfloat16 and q_out.is_contiguous()
                and (slot_map is None or (k_cache.dtype == torch.bfloat16 and k_cache.is_contiguous() and v_cache.is_contiguous()))):
            return fast.rope_kv_slices(pending.slices, positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                                       n_kv_heads, head_dim, page_size)
        pending.finish()
    _rows_contiguous(qkv, "rope qkv")
    T = qkv.shape[0]
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert q_out.is_contiguous() and q_out.numel() == T * n_heads * head_dim
    assert table.shape[1] * 2 == rotary_dim and int(positions.numel()) == T
    if slot_map is not None:
        assert k_cache is not None and v_cache is not None and k_cache.dtype == q_out.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
    _call("core", "hb_rope_kv", qkv.data_ptr(), _dt(qkv), qkv.stride(0), positions.data_ptr(), _ptr(slot_map),
          table.data_ptr(), q_out.data_ptr(), _dt(q_out), _ptr(k_cache), _ptr(v_cache), _dt(q_out), T, n_heads,
          n_kv_heads, head_dim, rotary_dim, page_size, _stream())
    return q_out


def linear_rope_kv_write(a: torch.Tensor, w: "Weight", positions: torch.Tensor, slot_map: Optional[torch.Tensor],
                         table: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                         v_cache: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                         page_size: int) -> bool:
    """rope_kv_write of a @ w.T in one kernel, where one takes these sizes; False: nothing was done
    (the caller projects, then rotates). The results are the same bits either way."""
    from . import fast

    if not a.is_cuda:
        return False
    return fast.linear_rope_kv(a, w, positions, slot_map, table, q_out, k_cache, v_cache, n_heads, n_kv_heads, head_dim,
                               rotary_dim, page_size)


ATTN_CHUNK = 256  # keys per split of the plain attention kernel: absolute positions, so batch-independent


def attention_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                   row_request: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_heads: int,
                   n_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, max_pos: int,
                   chunk: int = ATTN_CHUNK) -> torch.Tensor:
    """Causal attention of every row over its request's pages with the plain kernel.
    q, out [T, Hq D]; block_table [R, pages] int32; row_request, positions [T] int32;
    max_pos: the largest position among the rows (sizes the grid and the workspace)."""
    _need_cuda(q, k_cache, v_cache, block_table, row_request, positions, out)
    T = q.shape[0]
    assert q.is_contiguous() and out.is_contiguous() and out.dtype == q.dtype == k_cache.dtype
    assert block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.dtype == torch.int32
    lib = library.load("core")
    lib.hb_attn_rows_workspace.restype = C.c_long
    lib.hb_attn_rows_workspace.argtypes = [_i, _i, _i, _i, _i]
    n_ws = lib.hb_attn_rows_workspace(T, n_heads, head_dim, int(max_pos), chunk)
    ws = torch.empty(n_ws, dtype=torch.float32, device=q.device) if n_ws else None
    _call("core", "hb_attn_rows", q.data_ptr(), _dt(q), k_cache.data_ptr(), v_cache.data_ptr(), _dt(k_cache),
          block_table.data_ptr(), block_table.stride(0), row_request.data_ptr(), positions.data_ptr(),
          out.data_ptr(), _ptr(ws), T, n_heads, n_kv_heads, head_dim, page_size, int(window), float(scale), chunk,
          int(max_pos), _stream())
    return out


def attention_workspace(T: int, n_heads: int, head_dim: int, max_pos: int, chunk: int, device):
    """The partials buffer for rows whose keys span several chunks (None when none does)."""
    lib = library.load("core")
    lib.hb_attn_rows_workspace.restype = C.c_long
    lib.hb_attn_rows_workspace.argtypes = [_i, _i, _i, _i, _i]
    n_ws = lib.hb_attn_rows_workspace(T, n_heads, head_dim, int(max_pos), chunk)
    return torch.empty(n_ws, dtype=torch.float32, device=device) if n_ws else None


def attention_merge(ws, positions, out, n_heads, head_dim, window, max_pos, chunk, row_request=None, q_len=None,
                    row_limit=0):
    """Finish rows whose keys span several chunks; rows of requests with row_limit rows or more are left alone."""
    if ws is None:
        return out
    _call("core", "hb_attn_merge", ws.data_ptr(), positions.data_ptr(), out.data_ptr(), _dt(out), out.shape[0], n_heads,
          head_dim, int(window), chunk, int(max_pos), _ptr(row_request), _ptr(q_len), int(row_limit), _stream())
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
           position: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: arg max (temperature 0 or None) or a
    temperature draw keyed by (seed, position) of the row."""
    _need_cuda(logits, temperature, seed, position)
    _rows_contiguous(logits, "sample logits")
    assert logits.dtype == torch.float32
    R, V = logits.shape
    if out is None:
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
    if temperature is not None:
        assert temperature.dtype == torch.float32 and temperature.numel() == R
        assert seed is not None and seed.dtype in (torch.int32, torch.uint32) and seed.numel() == R
        assert position is not None and position.dtype == torch.int32 and position.numel() == R
    n = library.load("core").hb_sample_slices(V)
    ws = _sample_workspace(logits.device, R) if n > 1 else None
    _call("core", "hb_sample", logits.data_ptr(), logits.stride(0), R, V, _ptr(temperature), _ptr(seed),
          _ptr(position), out.data_ptr(), _ptr(ws), _stream())
    return out


_sample_ws = {}
_sample_ws_retired = []


def _sample_workspace(device, rows):
    """Zeroed words in which the slices of a large vocabulary meet (12 bytes a row: the kernel leaves them zero); one
    buffer per device, shared by all calls (they run one after the other on the step's stream)."""
    ws = _sample_ws.get(device)
    if ws is None or ws.numel() < 3 * rows:
        if ws is not None:
            _sample_ws_retired.append(ws)       # a captured CUDA graph may still hold the old address
        ws = _sample_ws[device] = torch.zeros(3 * max(rows, 256), dtype=torch.int32, device=device)
    return ws


def feed_tokens(tokens: torch.Tensor, src: torch.Tensor, token_map: torch.Tensor) -> torch.Tensor:
    """tokens[i] = src[token_map[i]] where token_map[i] >= 0 (all int32 on the device)."""
    _need_cuda(tokens, src, token_map)
    assert tokens.dtype == src.dtype == token_map.dtype == torch.int32 and token_map.numel() == tokens.numel()
    _call("core", "hb_feed_tokens", tokens.data_ptr(), src.data_ptr(), token_map.data_ptr(), tokens.numel(), _stream())
    return tokens


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A copy of a contiguous tensor in another element type (float32 <-> bfloat16)."""
    _need_cuda(src)
    src = src.contiguous()
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _call("core", "hb_convert", src.data_ptr(), _dt(src), out.data_ptr(), _dt(out), src.numel(), _stream())
    return out


# ------------------------------------------------------------------------------------------
# Operations with a choice of kernel
# ------------------------------------------------------------------------------------------
class Weight:
    """A weight matrix [N, K] (K contiguous, row n produces output n, as the reference stores
    them, src/api.cu:81-83) with whatever a kernel prepared for it (tensor maps and the like)."""

    __slots__ = ("t", "prepared")

    def __init__(self, t: torch.Tensor):
        assert t.dim() == 2 and t.is_contiguous()
        self.t = t
        self.prepared = {}

    @property
    def nbytes(self) -> int:
        return self.t.numel() * self.t.element_size()

    @property
    def shape(self):
        return self.t.shape


def linear(a: torch.Tensor, w: Weight, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out (+)= a @ w.T. bfloat16 operands go to the tensor-core kernels when those take the
    sizes; everything else to the plain 32-bit kernel."""
    from . import fast

    if fast.linear(a, w, out, accumulate):
        return out
    return gemm_plain(a, w.t, out, accumulate)


def linear_into_stream(a: torch.Tensor, w: Weight, x: torch.Tensor) -> torch.Tensor:
    """x += a @ w.T into the float32 residual stream: for a few bfloat16 rows one kernel that owns whole-K stripes of the
    output (nothing left to add across blocks), else the product `linear` chooses."""
    if a.is_cuda and a.dtype == torch.bfloat16 and linear_add_rows(a, w, x):
        return x
    return linear(a, w, x, accumulate=True)


def linear_rows32(a: torch.Tensor, w: Weight, out: torch.Tensor) -> torch.Tensor:
    """out = a @ w.T as 32-bit rows for a 32-bit consumer. For a few bfloat16 rows the whole-K rows kernel adds into the
    zeroed rows (one kernel behind a memset instead of a split-K product and the reduction of its slices); else `linear`."""
    if a.is_cuda and a.dtype == torch.bfloat16 and out.dtype == torch.float32 and out.is_contiguous() and a.shape[0] <= 8:
        out.zero_()
        if linear_add_rows(a, w, out):
            return out
    return linear(a, w, out)


def linear_scaled_add(a: torch.Tensor, w: Weight, x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x[m, n] += scale[n] * (a @ w.T)[m, n]: an output projection times the layer's scale vector, added into the float32
    residual stream. One kernel with the plain product; the tensor-core product leaves its float32 result to a small
    kernel that scales and adds."""
    from . import fast

    M, N = a.shape[0], w.shape[0]
    if fast._tc_ok(a, w.t):
        y = torch.empty(M, N, dtype=torch.float32, device=a.device)
        fast.linear(a, w, y, False)
        return scale_add(x, y, scale)
    _need_cuda(a, x, scale)
    _rows_contiguous(a, "gemm a")
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (M, N) and scale.numel() == N
    if scale.dtype != w.t.dtype:
        y = torch.empty(M, N, dtype=torch.float32, device=a.device)
        gemm_plain(a, w.t, y)
        return scale_add(x, y, scale)
    _call("core", "hb_gemm_simt_scaled", a.data_ptr(), _dt(a), a.stride(0), w.t.data_ptr(), _dt(w.t), w.t.stride(0),
          x.data_ptr(), x.stride(0), M, N, a.shape[1], scale.data_ptr(), _stream())
    return x


def linear_swiglu(a: torch.Tensor, w_gate_up: Weight, act_out: torch.Tensor, group: int) -> torch.Tensor:
    """act_out = swiglu(a @ w_gate_up.T) for a gate/up matrix interleaved in groups of `group` rows."""
    from . import fast

    if fast.linear_swiglu(a, w_gate_up, act_out, group):
        return act_out
    gu = torch.empty(a.shape[0], w_gate_up.shape[0], dtype=torch.float32, device=a.device)
    gemm_plain(a, w_gate_up.t, gu)
    return swiglu(gu, act_out, group)


class LazyNorm:
    """The RMSNorm of residual rows that has not been computed yet: (x fp32 [T, H], weight, eps). A part that can
    fold the norm into its own first kernel (a few rows: the product's prologue) takes it as it is; any other
    calls materialize(), which runs the norm kernel. A part says that it understands one with `takes_lazy_norm`."""
    __slots__ = ("x", "weight", "eps", "dtype", "feed")

    def __init__(self, x, weight, eps, dtype, feed=None):
        self.x, self.weight, self.eps, self.dtype = x, weight, eps, dtype
        self.feed = feed       # a filled fast.NormFeed of this norm, left by the product that wrote x (or None)

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    def materialize(self) -> torch.Tensor:
        out = torch.empty(self.x.shape, dtype=self.dtype, device=self.x.device)
        return rmsnorm(self.x, self.weight, self.eps, out)


def lazy_norm_applies(x: torch.Tensor, weight: torch.Tensor, dtype) -> bool:
    """Whether a consumer could fold this norm into its product: a few bf16-path rows on the device."""
    from . import fast

    return (x.is_cuda and dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.float32
            and x.shape[0] <= fast.ROWS_MAX and not fast.PLAIN_ONLY)


def norm_linear_rope_kv_write(xn: "LazyNorm", w: "Weight", positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                              n_kv_heads, head_dim, rotary_dim, page_size) -> bool:
    """rope_kv_write of RMSNorm(x) @ w.T in one kernel for a few rows; False: nothing was done."""
    from . import fast

    if xn.feed is not None and fast.rows_scaled_qkv_rope(xn.feed, xn.x.shape[0], w.t, positions, slot_map, table, q_out, k_cache,
                                                         v_cache, n_heads, n_kv_heads, head_dim, rotary_dim, page_size):
        return True
    return fast.rows_norm_qkv_rope(xn.x, xn.weight, xn.eps, w.t, positions, slot_map, table, q_out, k_cache, v_cache, n_heads,
                                   n_kv_heads, head_dim, rotary_dim, page_size)


def norm_linear_swiglu(xn: "LazyNorm", w_gate_up: "Weight", act_out: torch.Tensor, group: int) -> bool:
    """act_out = swiglu(RMSNorm(x) @ w_gate_up.T) in one kernel for a few rows; False: nothing was done."""
    from . import fast

    if xn.feed is not None and fast.rows_scaled_swiglu(xn.feed, xn.x.shape[0], w_gate_up.t, act_out, group):
        return True
    return fast.rows_norm_swiglu(xn.x, xn.weight, xn.eps, w_gate_up.t, act_out, group)


def linear_add_rows(a: torch.Tensor, w: "Weight", out: torch.Tensor, norm_feed=None) -> bool:
    """out += a @ w.T finished in one kernel for a few rows (whole-K stripes, nothing left to add); False: nothing was done.
    norm_feed (a fast.NormFeed of the norm that reads `out` next, or None): the kernel prepares that norm on its way."""
    from . import fast

    return a.is_cuda and a.shape[0] <= fast.ROWS_MAX and fast.rows_add(a, w.t, out, norm_feed)


def make_norm_feed(weight: torch.Tensor, eps: float, rows: int):
    """A NormFeed for the norm (weight, eps) over `rows` residual rows, where the rows kernels apply; else None."""
    from . import fast

    return fast.NormFeed(weight, eps, rows) if fast.norm_feed_applies(weight, rows) else None


class Pending:
    """A product whose K slices have yet to be added: into `out` (accumulate) or as `out` itself.
    The kernel that reads the result next can add them on its way (rmsnorm and rope_kv_write take
    `pending`); anything else calls finish() first. It must be consumed before the next small
    product runs: the slices lie in scratch memory those products share."""
    __slots__ = ("slices", "out", "accumulate")

    def __init__(self, slices, out, accumulate):
        self.slices, self.out, self.accumulate = slices, out, accumulate

    def finish(self):
        from . import fast

        fast.finish_slices(self.slices, self.out, fast.EPI_ADD_F32 if self.accumulate else fast.EPI_F32)
        return self.out


def linear_deferred(a: torch.Tensor, w: Weight, out: torch.Tensor, accumulate: bool = False) -> Optional[Pending]:
    """out (+)= a @ w.T, with the last step (adding the K slices of a small product) left to the
    consumer where that applies: then a Pending comes back and `out` is not yet written. None: out is done."""
    from . import fast

    if out.dtype == torch.float32 and a.is_cuda:
        sl = fast.linear_slices(a, w)
        if sl is not None:
            return Pending(sl, out, accumulate)
    linear(a, w, out, accumulate)
    return None


def attention(q, k_cache, v_cache, batch, group: int, out, n_heads, n_kv_heads, head_dim, page_size, window, scale):
    """Attention of the step's rows over their requests' pages of cache group `group`."""
    from . import fast

    if fast.attention(q, k_cache, v_cache, batch, group, out, n_heads, n_kv_heads, head_dim, page_size, window, scale):
        return out
    return attention_rows(q, k_cache, v_cache, batch.block_tables[group], batch.row_request, batch.positions, out,
                          n_heads, n_kv_heads, head_dim, page_size, window, scale, batch.max_pos)


# ------------------------------------------------------------------------------------------
# Operations of gated feed-forwards, of attention with a mask, a sink and a gate chosen by parameters, of latent
# attention and of gated linear attention (csrc/core.cu, attention_masked.cu, latent.cu, gla.cu)
# ------------------------------------------------------------------------------------------
GATE_ACTS = {"silu": 0, "gelu_tanh": 1}


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, group: int, act: str = "silu") -> torch.Tensor:
    """out[m, i] = act(g) * u for a gate/up matrix [M, 2I] interleaved in groups of `group` columns; act "silu" or
    "gelu_tanh" (0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))))."""
    _need_cuda(gate_up, out)
    _rows_contiguous(gate_up, "gated_act in")
    _rows_contiguous(out, "gated_act out")
    M, I = out.shape
    assert gate_up.shape == (M, 2 * I)
    _call("core", "hb_gated_act", gate_up.data_ptr(), _dt(gate_up), gate_up.stride(0), out.data_ptr(), _dt(out),
          out.stride(0), M, I, group, GATE_ACTS[act], _stream())
    return out


def linear_gated(a: torch.Tensor, w_gate_up: "Weight", act_out: torch.Tensor, group: int, act: str) -> bool:
    """act_out = act(gate) * up of a @ w_gate_up.T as one kernel (the activation in the product's epilogue) where one
    takes these sizes; False: nothing was done (the caller runs the product, then gated_act)."""
    from . import fast

    return a.is_cuda and fast.linear_gated(a, w_gate_up, act_out, group, act)


_rope_tables = {}


def rope_frequencies(dims: int, base: float, scaling=None):
    """(frequencies float64 [dims / 2], magnitude): f_i = base^(-2i / dims), rescaled by `scaling` (a mapping or None):

    kind "wavelength_bands" (factor, low, high, original): with the wavelength l = 2 pi / f, f stays where l < original /
        high, becomes f / factor where l > original / low, and between the two is (1 - s) f / factor + s f with
        s = (original / l - low) / (high - low); magnitude 1.
    kind "yarn" (factor, original, fast, slow): with d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)),
        0), hi = min(ceil(d(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
        r_i f_i / factor + (1 - r_i) f_i, and cos and sin are both multiplied by the magnitude 0.1 ln(factor) + 1."""
    import math

    i = torch.arange(0, dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    kind = scaling.get("kind")
    if kind == "wavelength_bands":
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * math.pi / f
        s = (orig / wl - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        return torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, mid)), 1.0
    if kind == "yarn":
        factor, orig, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
        d_of = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(float(base)))
        lo, hi = max(math.floor(d_of(fast)), 0), min(math.ceil(d_of(slow)), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0
    raise KernelError(f"rotary scaling of kind {kind!r} is not known (known: 'wavelength_bands', 'yarn')")


def shared_rope_table(dims: int, base: float, n_pos: int, device, scaling=None) -> torch.Tensor:
    """(cos, sin) float32 [n_pos, dims / 2, 2] of the angles p * f_i, f_i = base^(-2i / dims) rescaled by `scaling` (see
    rope_frequencies; the magnitude is in the table): one table per (dims, base, scaling, n_pos, device), shared by every
    part that asks (the frequencies are computed in float64 and rounded to float32)."""
    skey = tuple(sorted((k, v) for k, v in scaling.items())) if scaling else None
    key = (int(dims), float(base), skey, int(n_pos), str(device))
    t = _rope_tables.get(key)
    if t is None:
        f, mag = rope_frequencies(int(dims), float(base), scaling)
        t = _rope_tables[key] = rope_table(f.to(torch.float32).to(device), n_pos, mag)
    return t


PAIRINGS = {"half": 0, "interleaved": 1}


def rope_norm_store(proj: torch.Tensor, offsets, positions: torch.Tensor, slot_map: Optional[torch.Tensor],
                    table: torch.Tensor, rot: int, pairing: str, unit_norm: bool, eps: float, q_out: torch.Tensor,
                    k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], n_heads: int, n_kv_heads: int,
                    dim: int, vdim: int, page_size: int, rot_off: int = 0, row_norm=None, row_norm_eps: float = 0.0) -> torch.Tensor:
    """From a float32 projection result whose rows hold q, k, v at the column `offsets` (q, k, v): q and k rotated on
    the `rot` dimensions from `rot_off` on (pairing "half": (i, i + rot/2); "interleaved": (2i, 2i + 1)) and, with unit_norm,
    divided by their root mean square over `dim`; q to q_out [T, n_heads * dim], k and v (vdim wide, raw) to their page
    slots. slot_map None: q alone. row_norm (wq [n_heads * dim], wk [n_kv_heads * dim]): before the rotation the whole
    q row and the whole k row are divided by their root mean square (row_norm_eps inside the root) and multiplied by the
    weights, column by column."""
    _need_cuda(proj, positions, slot_map, table, q_out, k_cache, v_cache)
    _rows_contiguous(proj, "rope_norm_store in")
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and q_out.is_contiguous() and q_out.shape == (T, n_heads * dim)
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] * 2 == rot
    if slot_map is not None:
        assert k_cache.dtype == v_cache.dtype == q_out.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[-1] == dim and v_cache.shape[-1] == vdim
    q_off, k_off, v_off = (int(o) for o in offsets)
    wq_pre, wk_pre = row_norm if row_norm is not None else (None, None)
    if wq_pre is not None:
        _need_cuda(wq_pre, wk_pre)
        assert wq_pre.dtype == wk_pre.dtype and wq_pre.numel() == n_heads * dim and wk_pre.numel() == n_kv_heads * dim
    _call("core", "hb_rope_norm_store", proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, positions.data_ptr(),
          _ptr(slot_map), table.data_ptr(), int(rot), int(rot_off), PAIRINGS[pairing], 1 if unit_norm else 0, float(eps), q_out.data_ptr(),
          _ptr(k_cache) if slot_map is not None else None, _ptr(v_cache) if slot_map is not None else None, _dt(q_out), T,
          n_heads, n_kv_heads, dim, vdim, page_size, _ptr(wq_pre), _ptr(wk_pre), _dt(wq_pre) if wq_pre is not None else 0,
          float(row_norm_eps), _stream())
    return q_out


MASKS = {"causal": 0, "window": 1, "chunk": 2}
MASKED_FLASH_MIN_ROWS = 16


def attention_masked(q, k_cache, v_cache, batch, group: int, out, n_heads: int, n_kv_heads: int, dim: int, vdim: int,
                     page_size: int, scale: float, mask: str = "causal", window: int = 0, keep_first: int = 0, chunk: int = 0,
                     sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_offset: int = 0,
                     gate_per_head: bool = False, force_rows: bool = False, row_limit: int = 0,
                     force_plain: bool = False) -> torch.Tensor:
    """Attention of the step's rows over their requests' pages (csrc/attention_masked.cu; requests that bring many rows:
    csrc/attention_masked_flash.cu). With row_limit, rows of requests that bring that many rows or more are left alone (the
    caller has another path for them). Keys `dim` and values `vdim`
    wide, each plane [page, kv head, page_size, width] with a width of its own (v_cache may be the key plane itself:
    the values are then its first `vdim` columns). mask "causal", "window" (the last `window` keys and the first
    `keep_first`) or "chunk" (the keys of the row's own chunk of `chunk` positions). sink: float32 [n_heads], joins the
    softmax's denominator as exp(sink). gate: float32 [T, *], sigmoid(gate[:, gate_offset + ...]) multiplies the result,
    one number per element or, with gate_per_head, one per head. out may be float32 beside bfloat16 q."""
    _need_cuda(q, k_cache, v_cache, out, gate, sink)
    T = q.shape[0]
    bt = batch.block_tables[group]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == k_cache.dtype == v_cache.dtype
    assert q.shape[1] == n_heads * dim and out.shape == (T, n_heads * vdim)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[-1] >= dim and v_cache.shape[-1] >= vdim
    assert k_cache.shape[1] == n_kv_heads
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.numel() == n_heads and sink.is_contiguous()
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == T
    lib = library.load("seqmix")
    lib.hb_attn_masked_workspace.restype = C.c_long
    lib.hb_attn_masked_workspace.argtypes = [_i] * 10
    lib.hb_attn_masked_counters.argtypes = [_i] * 5
    max_pos = int(getattr(batch, "max_pos", 0)) or int(bt.shape[1]) * page_size - 1
    m = MASKS[mask]
    # requests that bring MASKED_FLASH_MIN_ROWS rows or more go to the tensor-core kernel (bfloat16, the sizes it takes),
    # the other rows of the step to the row kernel; a decode-only step is the row kernel alone
    from . import fast

    kw, vw = k_cache.shape[-1], v_cache.shape[-1]
    flash = (q.dtype == torch.bfloat16 and not fast.PLAIN_ONLY and not force_rows and not force_plain and v_cache is not k_cache
             and getattr(batch, "max_q_len", 0) >= MASKED_FLASH_MIN_ROWS and masked_flash_supported(dim, vdim)
             and kw % 8 == 0 and vw % 8 == 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)
    if flash:
        _call("seqmix", "hb_attn_masked_flash", q.data_ptr(), q.stride(0), k_cache.data_ptr(), n_kv_heads * page_size * kw,
              page_size * kw, kw, v_cache.data_ptr(), n_kv_heads * page_size * vw, page_size * vw, vw, bt.data_ptr(), bt.stride(0),
              batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(), batch.req_ctx_len.data_ptr(), 0, batch.n_requests,
              batch.max_q_len, MASKED_FLASH_MIN_ROWS, _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0,
              int(gate_offset), (2 if gate_per_head else 1) if gate is not None else 0, out.data_ptr(), _dt(out), out.stride(0),
              n_heads, n_kv_heads, dim, vdim, page_size, m, int(window), int(keep_first), int(chunk), float(scale), _stream())
        if min(batch.h_q_len) >= MASKED_FLASH_MIN_ROWS:
            return out
    limit = int(row_limit) or (MASKED_FLASH_MIN_ROWS if flash else 0)
    alias = v_cache is k_cache
    if (q.dtype == torch.bfloat16 and not fast.PLAIN_ONLY and not force_plain and kw % 8 == 0 and vw % 8 == 0
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and _fn("seqmix", "hb_attn_masked_heads_supported")(n_heads, n_kv_heads, dim, vdim, 1 if alias else 0) == 1):
        # the heads of a kv head as the rows of warp MMA tiles: a key tile is read once for all of them
        lib.hb_attn_masked_heads_workspace.restype = C.c_long
        lib.hb_attn_masked_heads_workspace.argtypes = [_i] * 9
        n_ws = lib.hb_attn_masked_heads_workspace(T, n_heads, n_kv_heads, vdim, m, int(window), int(keep_first), int(chunk), max_pos)
        ws = torch.empty(n_ws, dtype=torch.float32, device=q.device) if n_ws else None
        _call("seqmix", "hb_attn_masked_heads", q.data_ptr(), q.stride(0), k_cache.data_ptr(), n_kv_heads * page_size * kw,
              page_size * kw, kw, v_cache.data_ptr(), n_kv_heads * page_size * vw, page_size * vw, vw, 1 if alias else 0,
              bt.data_ptr(), bt.stride(0), batch.row_request.data_ptr(), batch.positions.data_ptr(), _ptr(sink), _ptr(gate),
              gate.stride(0) if gate is not None else 0, int(gate_offset), (2 if gate_per_head else 1) if gate is not None else 0,
              out.data_ptr(), _dt(out), out.stride(0), T, n_heads, n_kv_heads, dim, vdim, page_size, m, int(window),
              int(keep_first), int(chunk), float(scale), batch.req_q_len.data_ptr() if limit else None, limit, _ptr(ws), n_ws,
              max_pos, _stream())
        return out
    n_ws = lib.hb_attn_masked_workspace(T, n_heads, n_kv_heads, dim, vdim, m, int(window), int(keep_first), int(chunk), max_pos)
    ws = arrived = None
    if n_ws:
        from . import fast

        ws = torch.empty(n_ws, dtype=torch.float32, device=q.device)
        arrived = fast._decode_counters(q.device, lib.hb_attn_masked_counters(T, n_heads, n_kv_heads, dim, vdim))
    _call("seqmix", "hb_attn_masked", q.data_ptr(), _dt(q), q.stride(0), k_cache.data_ptr(), k_cache.shape[-1],
          v_cache.data_ptr(), v_cache.shape[-1], _dt(k_cache), bt.data_ptr(), bt.stride(0), batch.row_request.data_ptr(),
          batch.positions.data_ptr(), _ptr(sink), _ptr(gate), gate.stride(0) if gate is not None else 0, int(gate_offset),
          (2 if gate_per_head else 1) if gate is not None else 0, out.data_ptr(), _dt(out), out.stride(0), T, n_heads,
          n_kv_heads, dim, vdim, page_size, m, int(window), int(keep_first), int(chunk), float(scale),
          batch.req_q_len.data_ptr() if limit else None, limit, _ptr(ws), n_ws, _ptr(arrived), max_pos, _stream())
    return out


def latent_prepare(proj: torch.Tensor, offsets, wq: torch.Tensor, wc: torch.Tensor, positions, slot_map, table, rot: int,
                   eps: float, cq_out: torch.Tensor, cache: Optional[torch.Tensor], q_rank: int, kv_rank: int, rot_dim: int,
                   page_size: int, pairing: str = "interleaved") -> torch.Tensor:
    """From a float32 projection result with the raw query latent, the raw key/value latent and the raw rotated key part
    at the column `offsets`: the query latent / rms * wq to cq_out [T, q_rank]; the key/value latent / rms * wc and the
    rotated key part (pairing "interleaved": pairs (2i, 2i + 1); "half": (i, i + rot / 2)) to the token's row of `cache`
    [page, 1, page_size, kv_rank + rot_dim]."""
    _need_cuda(proj, wq, wc, positions, slot_map, table, cq_out, cache)
    _rows_contiguous(proj, "latent_prepare in")
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and cq_out.is_contiguous() and cq_out.shape == (T, q_rank)
    assert wc.numel() == kv_rank and ((wq is None and q_rank == 0) or (wq.dtype == wc.dtype and wq.numel() == q_rank))
    if slot_map is not None:
        assert cache.is_contiguous() and cache.dtype == cq_out.dtype and cache.shape[1] == 1 and cache.shape[-1] == kv_rank + rot_dim
    a, b, c = (int(o) for o in offsets)
    _call("seqmix", "hb_latent_prepare", proj.data_ptr(), proj.stride(0), a, b, c, _ptr(wq), wc.data_ptr(), _dt(wc),
          positions.data_ptr(), _ptr(slot_map), table.data_ptr(), int(rot), float(eps), cq_out.data_ptr(),
          _ptr(cache) if slot_map is not None else None, _dt(cq_out), T, q_rank, kv_rank, rot_dim, page_size, PAIRINGS[pairing],
          _stream())
    return cq_out


def heads_linear(a: torch.Tensor, a_head: int, wt: torch.Tensor, out: torch.Tensor, o_head: int, gate=None,
                 gate_offset: int = 0, tail: int = 0, rot: int = 0, positions=None, table=None, batch=None,
                 row_limit: int = 0, pairing: str = "interleaved", gate_per_head: bool = False) -> torch.Tensor:
    """out[t, h * o_head + n] = sum_k a[t, h * a_head + k] wt[h, k, n] for every head h (a float32, 32-bit sums),
    optionally times sigmoid(gate[t, gate_offset + h * N + n]) (gate_per_head: of gate[t, gate_offset + h]); with `tail`,
    the tail columns behind a head's K inputs are rotated on their first `rot` (pairs (2i, 2i + 1), or (i, i + rot / 2)
    with pairing "half") by the row's position and copied behind its N outputs. With
    `batch` and `row_limit`, rows of requests that bring row_limit rows or more are left alone (another path has them)."""
    _need_cuda(a, wt, out, gate, positions, table)
    _rows_contiguous(a, "heads_linear a")
    _rows_contiguous(out, "heads_linear out")
    H, K, N = wt.shape
    T = a.shape[0]
    assert a.dtype == torch.float32 and wt.is_contiguous() and out.shape[0] == T
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1
    _call("seqmix", "hb_heads_linear", a.data_ptr(), a.stride(0), int(a_head), wt.data_ptr(), _dt(wt), out.data_ptr(),
          _dt(out), out.stride(0), int(o_head), T, H, K, N, _ptr(gate), gate.stride(0) if gate is not None else 0,
          int(gate_offset), int(tail), int(rot), _ptr(positions), _ptr(table),
          batch.row_request.data_ptr() if row_limit else None, batch.req_q_len.data_ptr() if row_limit else None, int(row_limit),
          PAIRINGS[pairing], 1 if gate_per_head else 0, _stream())
    return out


def gather_rows(plane: torch.Tensor, table: torch.Tensor, dst: torch.Tensor, n: int, page_size: int) -> torch.Tensor:
    """dst[t] = the cache row of position t, t < n, of a plane with one head [page, 1, page_size, W] through one request's
    block table (int32 on the device)."""
    _need_cuda(plane, table, dst)
    assert plane.is_contiguous() and dst.is_contiguous() and plane.shape[1] == 1 and dst.shape == (n, plane.shape[-1])
    assert plane.dtype == dst.dtype and table.dtype == torch.int32 and table.stride(-1) == 1
    _call("seqmix", "hb_gather_rows", plane.data_ptr(), _dt(plane), table.data_ptr(), dst.data_ptr(), int(n), plane.shape[-1],
          page_size, _stream())
    return dst


def fast_kernels_on() -> bool:
    """False when the plain kernels are asked for everywhere (HIPINFER_B200_PLAIN=1)."""
    from . import fast

    return not fast.PLAIN_ONLY


_identity_tables = {}


def _identity_table(device, n: int) -> torch.Tensor:
    t = _identity_tables.get(device)
    if t is None or t.numel() < n:
        t = _identity_tables[device] = torch.arange(max(n, 4096), dtype=torch.int32, device=device)
    return t


def masked_flash_supported(dim: int, vdim: int) -> bool:
    return _fn("seqmix", "hb_attn_masked_flash_supported")(int(dim), int(vdim)) == 1


def attention_flash_tokens(q, keys, values, batch, request: int, out, n_heads: int, n_kv_heads: int, dim: int, vdim: int,
                           scale: float, gate=None, gate_offset: int = 0, gate_per_head: bool = False, window: int = 0,
                           first_pos: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the rows of ONE request of the batch (index `request`) over keys and values made for its
    context in token-major buffers: keys [n, >= n_kv_heads * dim] and values [n, >= n_kv_heads * vdim] (views of wider
    rows are fine), row t the token at position first_pos + t. With `window` a row at position i sees the keys j with
    0 <= i - j < window (first_pos must not lie behind the first key that the request's first row sees). sink: float32
    [n_heads], joins the softmax's denominator as exp(sink). bfloat16; the tensor-core kernel of
    csrc/attention_masked_flash.cu."""
    _need_cuda(q, keys, values, out, gate, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads and sink.is_contiguous())
    n = keys.shape[0]
    assert q.dtype == keys.dtype == values.dtype == torch.bfloat16 and keys.stride(1) == values.stride(1) == 1
    _call("seqmix", "hb_attn_masked_flash", q.data_ptr(), q.stride(0), keys.data_ptr(), keys.stride(0), dim, 0, values.data_ptr(),
          values.stride(0), vdim, 0, _identity_table(q.device, n).data_ptr() - 4 * int(first_pos), 0, batch.req_q_start.data_ptr(),
          batch.req_q_len.data_ptr(), batch.req_ctx_len.data_ptr(), int(request), 1, int(batch.h_q_len[request]), 1, _ptr(sink),
          _ptr(gate), gate.stride(0) if gate is not None else 0, int(gate_offset), (2 if gate_per_head else 1) if gate is not None else 0,
          out.data_ptr(), _dt(out), out.stride(0), n_heads, n_kv_heads, dim, vdim, 1, 1 if window else 0, int(window), 0, 0,
          float(scale), _stream())
    return out


def gla(proj: torch.Tensor, offsets, z: torch.Tensor, a_bias, norm_weight, state: torch.Tensor, batch, out: torch.Tensor,
        heads: int, dim: int, vdim: int, tau: float, eps: float) -> torch.Tensor:
    """Gated linear attention over the step's rows, request by request, from and into each request's state slot
    (csrc/gla.cu). proj float32 [T, *] holds q, k, v and the gate's pre-activation at the column `offsets` (q, k, v, g);
    z float32 [T, heads * dim] the decay's pre-activation without its bias; state float32 [slots, heads, dim, vdim]."""
    _need_cuda(proj, z, a_bias, norm_weight, state, out)
    _rows_contiguous(proj, "gla proj")
    _rows_contiguous(z, "gla z")
    assert proj.dtype == z.dtype == state.dtype == torch.float32 and state.is_contiguous() and out.is_contiguous()
    assert state.shape[1:] == (heads, dim, vdim) and out.shape == (proj.shape[0], heads * vdim)
    assert a_bias.dtype == norm_weight.dtype and a_bias.numel() == heads * dim and norm_weight.numel() == vdim
    q, k, v, g = (int(o) for o in offsets)
    _call("seqmix", "hb_gla", proj.data_ptr(), proj.stride(0), q, k, v, g, z.data_ptr(), z.stride(0), a_bias.data_ptr(),
          norm_weight.data_ptr(), _dt(a_bias), state.data_ptr(), batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(),
          batch.req_state_slot.data_ptr(), out.data_ptr(), _dt(out), batch.n_requests, heads, dim, vdim, float(tau),
          float(eps), _stream())
    return out


# ------------------------------------------------------------------------------------------
# The `hybrid` library: residual streams with learned mixing, the state-space recurrence with a scalar decay per head,
# routed feed-forward layers, a gated activation with biases and limits
# ------------------------------------------------------------------------------------------
def streams_norm(x: torch.Tensor, read: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                 streams: int, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rms norm of u = sum_s read[s] x_s (read None: the plain sum) times weight, for the residual rows x float32
    [T, streams * W]; with `rows` (int32 on the device) of those rows only."""
    _need_cuda(x, read, weight, out, rows)
    W = weight.numel()
    n = x.shape[0] if rows is None else rows.numel()
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == streams * W and out.is_contiguous()
    assert out.shape == (n, W) and (read is None or (read.dtype == torch.float32 and read.numel() == streams))
    _call("hybrid", "hb_streams_norm", x.data_ptr(), _ptr(rows), n, _ptr(read), weight.data_ptr(), _dt(weight), out.data_ptr(),
          _dt(out), int(streams), W, float(eps), _stream())
    return out


def streams_update(x: torch.Tensor, y: torch.Tensor, write: Optional[torch.Tensor], mix: Optional[torch.Tensor], mult: float,
                   streams: int, next_read: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None,
                   eps: float = 0.0, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x_t <- sum_s mix[s, t] x_s + mult * write[t] * y for all streams t at once (write None: ones; mix None: the
    identity), x float32 [T, streams * W], y float32 [T, W]. With next_weight (and `out`): also the norm of the sublayer
    that reads x next, out = rms norm of sum_s next_read[s] x_s times next_weight, in the same pass over the row."""
    _need_cuda(x, y, write, mix, next_read, next_weight, out)
    T, W = y.shape
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and x.shape == (T, streams * W)
    for c, n in ((write, streams), (mix, streams * streams), (next_read, streams)):
        assert c is None or (c.dtype == torch.float32 and c.is_contiguous() and c.numel() == n)
    if next_weight is None:
        _call("hybrid", "hb_streams_update", x.data_ptr(), y.data_ptr(), _ptr(write), _ptr(mix), float(mult), T, int(streams), W,
              _stream())
        return None
    assert out.is_contiguous() and out.shape == (T, W) and next_weight.numel() == W
    _call("hybrid", "hb_streams_update_norm", x.data_ptr(), y.data_ptr(), _ptr(write), _ptr(mix), float(mult), _ptr(next_read),
          next_weight.data_ptr(), _dt(next_weight), out.data_ptr(), _dt(out), T, int(streams), W, float(eps), _stream())
    return out


def streams_expand(x: torch.Tensor, xs: torch.Tensor, streams: int) -> torch.Tensor:
    """xs [T, streams * W] = `streams` copies of every row of x [T, W] (float32)."""
    _need_cuda(x, xs)
    T, W = x.shape
    assert x.dtype == xs.dtype == torch.float32 and x.is_contiguous() and xs.is_contiguous() and xs.shape == (T, streams * W)
    _call("hybrid", "hb_streams_expand", x.data_ptr(), xs.data_ptr(), T, int(streams), W, _stream())
    return xs


GLU_KINDS = {"silu": 0, "gelu_tanh": 1, "clamped_sigmoid": 2}


def glu_bias(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, group: int, kind: str,
             limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """out[m, i] = the gated activation of a float32 gate/up matrix [M, 2I] interleaved in groups of `group` columns,
    after adding `bias` [2I] (same order). kind "silu" / "gelu_tanh": act(g) * u; "clamped_sigmoid": g' = min(g, limit),
    u' = clamp(u, -limit, limit), out = g' sigmoid(alpha g') (u' + 1)."""
    _need_cuda(gate_up, bias, out)
    _rows_contiguous(gate_up, "glu_bias in")
    _rows_contiguous(out, "glu_bias out")
    M, I = out.shape
    assert gate_up.dtype == torch.float32 and gate_up.shape == (M, 2 * I) and (bias is None or bias.numel() == 2 * I)
    _call("hybrid", "hb_glu_bias", gate_up.data_ptr(), gate_up.stride(0), _ptr(bias), _dt(bias) if bias is not None else 0,
          out.data_ptr(), _dt(out), out.stride(0), M, I, int(group), GLU_KINDS[kind], float(limit), float(alpha), _stream())
    return out


def scale_bias_rows(x: torch.Tensor, scale: float = 1.0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[m, n] = x[m, n] * scale + bias[n] in place on float32 rows (bias None: the scale alone)."""
    _need_cuda(x, bias)
    _rows_contiguous(x, "scale_bias_rows")
    assert x.dtype == torch.float32 and (bias is None or bias.numel() == x.shape[1])
    _call("hybrid", "hb_scale_bias_rows", x.data_ptr(), x.stride(0), _ptr(bias), _dt(bias) if bias is not None else 0,
          float(scale), x.shape[0], x.shape[1], _stream())
    return x


def ssd_conv(proj: torch.Tensor, offset: int, weight: torch.Tensor, bias: torch.Tensor, carried: torch.Tensor, batch,
             out: torch.Tensor) -> torch.Tensor:
    """out [T, C] = silu(causal convolution over each request's tokens + bias) of the C columns of the float32 rows `proj`
    from `offset` on; weight [C, K] (its last column multiplies the current token), zeros before a sequence. carried
    float32 [slots, K - 1, C] holds each request's last K - 1 raw inputs between steps and is brought up to date."""
    _need_cuda(proj, weight, bias, carried, out)
    _rows_contiguous(proj, "ssd_conv in")
    C, K = weight.shape
    assert proj.dtype == out.dtype == carried.dtype == torch.float32 and out.is_contiguous() and out.shape == (proj.shape[0], C)
    assert weight.is_contiguous() and weight.dtype == bias.dtype and bias.numel() == C and carried.is_contiguous()
    assert carried.shape[1:] == (K - 1, C)
    _call("hybrid", "hb_ssd_conv", proj.data_ptr(), proj.stride(0), int(offset), weight.data_ptr(), bias.data_ptr(), _dt(weight),
          carried.data_ptr() if carried.numel() else None, batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(),
          batch.req_state_slot.data_ptr(), out.data_ptr(), batch.n_requests, batch.max_q_len, C, K, _stream())
    return out


SSD_PIECE_TOKENS = 64    # tokens a piece of the state-space recurrence (ssd_scan); 0: always one walk a request


def ssd_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, batch, y: torch.Tensor, heads: int, vdim: int, n_state: int, groups: int) -> torch.Tensor:
    """The state-space recurrence with a scalar decay per head over the step's rows, request by request, from and into
    each request's state slot (csrc/ssd.cu). xbc float32 [T, heads * vdim | groups * n_state | groups * n_state] (x, B, C
    after the convolution), dt float32 [T, heads] raw (a view of wider rows is fine), state float32
    [slots, heads, n_state, vdim], y float32 [T, heads * vdim].

    A step whose longest portion has at least three times SSD_PIECE_TOKENS rows runs in pieces of that many tokens (every
    piece from a zero state, the pieces' starting states one after another, every piece again for y), so that a long
    prompt fills the GPU instead of one block a head; the results differ from the walk in one go by rounding only."""
    _need_cuda(xbc, dt, dt_bias, a_log, d_skip, state, y)
    _rows_contiguous(xbc, "ssd_scan xbc")
    _rows_contiguous(dt, "ssd_scan dt")
    T = xbc.shape[0]
    assert xbc.dtype == dt.dtype == state.dtype == y.dtype == torch.float32 and state.is_contiguous() and y.is_contiguous()
    assert xbc.shape[1] == heads * vdim + 2 * groups * n_state and dt.shape == (T, heads) and y.shape == (T, heads * vdim)
    assert state.shape[1:] == (heads, n_state, vdim) and dt_bias.dtype == a_log.dtype == d_skip.dtype
    assert dt_bias.numel() == a_log.numel() == d_skip.numel() == heads
    L, pieces, piece_state, piece_decay = int(SSD_PIECE_TOKENS), 0, None, None
    if L > 0 and batch.max_q_len >= 3 * L:
        pieces = -(-batch.max_q_len // L)
        room = T // L + batch.n_requests               # all requests' pieces: every request ends with at most one short piece
        piece_state = torch.empty(room, heads, n_state, vdim, dtype=torch.float32, device=xbc.device)
        piece_decay = torch.empty(room, heads, dtype=torch.float32, device=xbc.device)
    _call("hybrid", "hb_ssd_scan", xbc.data_ptr(), xbc.stride(0), dt.data_ptr(), dt.stride(0), dt_bias.data_ptr(),
          a_log.data_ptr(), d_skip.data_ptr(), _dt(dt_bias), state.data_ptr(), batch.req_q_start.data_ptr(),
          batch.req_q_len.data_ptr(), batch.req_state_slot.data_ptr(), y.data_ptr(), batch.n_requests, heads, vdim, n_state,
          groups, L, pieces, piece_state.data_ptr() if pieces else None, piece_decay.data_ptr() if pieces else None, _stream())
    return y


def ssd_gate_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    """out = (y * silu(z)) with each of the row's `parts` equal parts divided by its own root mean square (eps inside the
    root), times weight; y float32 [T, inner], z float32 [T, inner] (a view of wider rows is fine)."""
    _need_cuda(y, z, weight, out)
    _rows_contiguous(z, "ssd_gate_norm z")
    T, inner = y.shape
    assert y.dtype == z.dtype == torch.float32 and y.is_contiguous() and out.is_contiguous() and out.shape == (T, inner)
    assert weight.numel() == inner and z.shape == (T, inner)
    _call("hybrid", "hb_ssd_gate_norm", y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), _dt(weight), out.data_ptr(),
          _dt(out), T, inner, int(parts), float(eps), _stream())
    return out


SEL_PIECE_TOKENS = 64    # tokens a piece of the selective recurrence (selective_scan); 0: always one walk a request


def selective_scan(x: torch.Tensor, dt: torch.Tensor, bc: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor,
                   a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor, batch, out: torch.Tensor) -> torch.Tensor:
    """The selective recurrence with a decay per (channel, state) pair over the step's rows, request by request, from and
    into each request's state slot (csrc/selective_scan.cu). x, dt, z float32 [T, inner] (views of wider rows are fine):
    the convolved input, the step-size product without its bias, the gate's pre-activation; bc float32 [T, 2N]: B then C;
    dt_bias [inner], a_log [inner, N], d_skip [inner]; state float32 [slots, inner, N]. out [T, inner] = (sum_n S C + D x)
    silu(z), rounded once.

    A step whose longest portion has at least three times SEL_PIECE_TOKENS rows runs in pieces of that many tokens (every
    piece from a zero state, the pieces' starting states one after another, every piece again for the results), so that a
    long prompt fills the GPU; the results differ from the walk in one go by rounding only."""
    _need_cuda(x, dt, bc, z, dt_bias, a_log, d_skip, state, out)
    for t, what in ((x, "x"), (dt, "dt"), (bc, "bc"), (z, "z"), (out, "out")):
        _rows_contiguous(t, "selective_scan " + what)
    T, inner = x.shape
    N = a_log.shape[1]
    assert x.dtype == dt.dtype == bc.dtype == z.dtype == state.dtype == torch.float32 and state.is_contiguous()
    assert dt.shape == z.shape == out.shape == (T, inner) and bc.shape == (T, 2 * N) and state.shape[1:] == (inner, N)
    assert a_log.is_contiguous() and a_log.shape[0] == inner and dt_bias.numel() == d_skip.numel() == inner
    assert dt_bias.dtype == a_log.dtype == d_skip.dtype
    L, pieces, piece_state, piece_dt = int(SEL_PIECE_TOKENS), 0, None, None
    if L > 0 and batch.max_q_len >= 3 * L:
        pieces = -(-batch.max_q_len // L)
        room = T // L + batch.n_requests               # all requests' pieces: every request ends with at most one short piece
        piece_state = torch.empty(room, inner, N, dtype=torch.float32, device=x.device)
        piece_dt = torch.empty(room, inner, dtype=torch.float32, device=x.device)
    _call("hybrid", "hb_selective_scan", x.data_ptr(), x.stride(0), dt.data_ptr(), dt.stride(0), bc.data_ptr(), bc.stride(0),
          z.data_ptr(), z.stride(0), dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), _dt(a_log), state.data_ptr(),
          batch.req_q_start.data_ptr(), batch.req_q_len.data_ptr(), batch.req_state_slot.data_ptr(), out.data_ptr(), _dt(out),
          out.stride(0), batch.n_requests, inner, N, L, pieces, _ptr(piece_state), _ptr(piece_dt), _stream())
    return out


def linear_split32(a: torch.Tensor, w: "Weight", out: torch.Tensor) -> torch.Tensor:
    """out = a @ w.T for float32 rows a (a view of wider rows is fine) and float32 out. Where the weight is bfloat16 and
    the tensor-core product takes the sizes, a goes in as the sum of two bfloat16 matrices (round(a) and round(a - round(a)))
    through two products added in 32-bit: 16 bits of a's mantissa at tensor-core speed. Else the plain 32-bit product."""
    from . import fast

    _need_cuda(a, out)
    _rows_contiguous(a, "linear_split32 a")
    M, K = a.shape
    if (a.dtype == torch.float32 and w.t.dtype == torch.bfloat16 and out.dtype == torch.float32 and M > 64 and K % 8 == 0
            and not fast.PLAIN_ONLY):
        hi = torch.empty(M, K, dtype=torch.bfloat16, device=a.device)
        lo = torch.empty(M, K, dtype=torch.bfloat16, device=a.device)
        _call("hybrid", "hb_split_rounded", a.data_ptr(), a.stride(0), hi.data_ptr(), lo.data_ptr(), M, K, _stream())
        if fast.linear(hi, w, out, False) and fast.linear(lo, w, out, True):
            return out
    return linear(a, w, out)


class NormedPair:
    """Two side-by-side results that have yet to be joined: mix * (a / rms(a) * wa + b / rms(b) * wb), a and b float32
    [T, W], the weights [W], eps inside the roots. `residual_norm` joins them on its way over the row."""
    __slots__ = ("a", "b", "wa", "wb", "mix", "eps")

    def __init__(self, a, b, wa, wb, mix, eps):
        self.a, self.b, self.wa, self.wb, self.mix, self.eps = a, b, wa, wb, float(mix), float(eps)


def residual_norm(x: torch.Tensor, y: Optional[torch.Tensor] = None, pair: Optional[NormedPair] = None, alpha: float = 1.0,
                  weight: Optional[torch.Tensor] = None, eps: float = 0.0, rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The residual rows x float32 [T, W] after a sublayer, in place and in one pass: v = alpha * x + y + the joined `pair`
    (either may be absent); with `weight` (float32 [W]) x <- v / rms(v) * weight, the norm AFTER the sum, else x <- v.
    rounded: a tensor [T, W] of the compute element type that receives a copy of the new x."""
    _need_cuda(x, y, weight, rounded)
    T, W = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    assert y is None or (y.dtype == torch.float32 and y.is_contiguous() and y.shape == (T, W))
    assert weight is None or (weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == W)
    assert rounded is None or (rounded.is_contiguous() and rounded.shape == (T, W))
    a = b = wa = wb = None
    mix = pe = 0.0
    if pair is not None:
        a, b, wa, wb, mix, pe = pair.a, pair.b, pair.wa, pair.wb, pair.mix, pair.eps
        _need_cuda(a, b, wa, wb)
        assert a.dtype == b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous() and a.shape == b.shape == (T, W)
        assert wa.dtype == wb.dtype and wa.numel() == wb.numel() == W and wa.is_contiguous() and wb.is_contiguous()
    _call("hybrid", "hb_residual_norm", x.data_ptr(), _ptr(y), _ptr(a), _ptr(b), _ptr(wa), _ptr(wb),
          _dt(wa) if wa is not None else 0, float(mix), float(pe), float(alpha), _ptr(weight), float(eps), _ptr(rounded),
          _dt(rounded) if rounded is not None else 0, T, W, _stream())
    return x


MOE_SCORES = {"sigmoid": 0, "softmax_chosen": 1}


def moe_route(xn: torch.Tensor, router: torch.Tensor, top: int, bias: Optional[torch.Tensor] = None, score: str = "sigmoid"):
    """(expert int32 [T, top], weight float32 [T, top]): the `top` experts with the largest z = router @ row (+ bias), 32-bit
    sums; the largest first, ties to the lower index. score "sigmoid": the weights are sigmoid(z) of the chosen ones;
    "softmax_chosen": the softmax over the chosen logits alone."""
    _need_cuda(xn, router, bias)
    assert bias is None or (bias.dtype == router.dtype and bias.numel() == router.shape[0] and bias.is_contiguous())
    _rows_contiguous(xn, "moe_route in")
    T, (E, W) = xn.shape[0], router.shape
    assert router.is_contiguous() and xn.shape[1] == W
    expert = torch.empty(T, top, dtype=torch.int32, device=xn.device)
    weight = torch.empty(T, top, dtype=torch.float32, device=xn.device)
    _call("hybrid", "hb_moe_route", xn.data_ptr(), _dt(xn), xn.stride(0), router.data_ptr(), _ptr(bias), _dt(router),
          expert.data_ptr(), weight.data_ptr(), T, W, E, int(top), MOE_SCORES[score], _stream())
    return expert, weight


def moe_rows(xn: torch.Tensor, wgu: torch.Tensor, wdown: torch.Tensor, expert: torch.Tensor, score: torch.Tensor,
             y: torch.Tensor, at_output: bool = False) -> torch.Tensor:
    """y += sum over a row's chosen experts of Wd_e (silu(s Wg_e h) * (s Wu_e h)), row by row with nothing sorted and
    nothing on the host. wgu [E, 2F, W] (gate rows, then up rows), wdown [E, W, F], y float32 [T, W]. at_output: the
    weight multiplies the expert's result instead of its input, Wd_e (s silu(Wg_e h) * (Wu_e h))."""
    _need_cuda(xn, wgu, wdown, expert, score, y)
    _rows_contiguous(xn, "moe_rows in")
    _rows_contiguous(y, "moe_rows out")
    T, top = expert.shape
    E, F2, W = wgu.shape
    F = F2 // 2
    assert wgu.is_contiguous() and wdown.is_contiguous() and wdown.shape == (E, W, F) and y.dtype == torch.float32
    act = torch.empty(T * top, F, dtype=xn.dtype, device=xn.device)
    _call("hybrid", "hb_moe_gate_up_rows", xn.data_ptr(), _dt(xn), xn.stride(0), wgu.data_ptr(), _dt(wgu), expert.data_ptr(),
          score.data_ptr(), act.data_ptr(), T, W, F, top, 1 if at_output else 0, _stream())
    _call("hybrid", "hb_moe_down_rows", act.data_ptr(), _dt(act), wdown.data_ptr(), _dt(wdown), expert.data_ptr(), y.data_ptr(),
          y.stride(0), T, W, F, top, _stream())
    return y


def moe_sort(expert: torch.Tensor, n_experts: int):
    """The (row, choice) pairs sorted by expert: offsets int32 [E + 1] (first sorted row of each expert), pos int32 [pairs]
    (the sorted row of a pair), src int32 [pairs] (the pair of a sorted row)."""
    pairs = expert.numel()
    dev = expert.device
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(pairs, dtype=torch.int32, device=dev)
    src = torch.empty(pairs, dtype=torch.int32, device=dev)
    _call("hybrid", "hb_moe_sort", expert.data_ptr(), offsets.data_ptr(), pos.data_ptr(), src.data_ptr(), pairs, int(n_experts),
          _stream())
    return offsets, pos, src


def moe_grouped(a: torch.Tensor, src: Optional[torch.Tensor], top: int, w: torch.Tensor, offsets: torch.Tensor,
                out: torch.Tensor) -> torch.Tensor:
    """out[r] = w[e] a[row(r)] for the sorted rows r of every expert e (offsets[e] <= r < offsets[e + 1]); row(r) is
    src[r] // top where src is given (the step's input rows), else r. w [E, Nout, K]; out float32 [sorted rows, Nout].
    An expert's weights are read once for all of its rows; nothing is read by the host."""
    _need_cuda(a, w, offsets, out)
    _rows_contiguous(a, "moe_grouped in")
    E, Nout, K = w.shape
    assert w.is_contiguous() and a.shape[1] == K and out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == Nout
    assert offsets.numel() == E + 1 and offsets.dtype == torch.int32 and (src is None or src.dtype == torch.int32)
    _call("hybrid", "hb_moe_grouped", a.data_ptr(), _dt(a), a.stride(0), _ptr(src), int(top), w.data_ptr(), _dt(w),
          offsets.data_ptr(), out.data_ptr(), E, Nout, K, _stream())
    return out


def moe_gather(xn: torch.Tensor, src: torch.Tensor, top: int) -> torch.Tensor:
    """The input rows in sorted order: out[r] = xn[src[r] // top]."""
    _rows_contiguous(xn, "moe_gather in")
    out = torch.empty(src.numel(), xn.shape[1], dtype=xn.dtype, device=xn.device)
    _call("hybrid", "hb_moe_gather", xn.data_ptr(), _dt(xn), xn.stride(0), src.data_ptr(), out.data_ptr(), src.numel(),
          xn.shape[1], int(top), _stream())
    return out


def moe_act(gu: torch.Tensor, src: torch.Tensor, score: torch.Tensor, out: torch.Tensor, at_output: bool = False) -> torch.Tensor:
    """out[r] = silu(s g) * (s u) of the sorted rows' float32 [g | u], s the score of the row's pair; with at_output
    s silu(g) * u (the weight of the expert's result, brought in before the linear down product)."""
    pairs, F = out.shape
    assert gu.dtype == torch.float32 and gu.is_contiguous() and gu.shape == (pairs, 2 * F) and out.is_contiguous()
    _call("hybrid", "hb_moe_act", gu.data_ptr(), src.data_ptr(), score.data_ptr(), out.data_ptr(), _dt(out), pairs, F,
          1 if at_output else 0, _stream())
    return out


def moe_combine(ys: torch.Tensor, pos: torch.Tensor, y: torch.Tensor, top: int) -> torch.Tensor:
    """y[t] += the sorted results of row t's choices, added in the order of the choices."""
    _rows_contiguous(y, "moe_combine out")
    T, W = y.shape
    assert ys.dtype == y.dtype == torch.float32 and ys.is_contiguous() and ys.shape == (T * top, W)
    _call("hybrid", "hb_moe_combine", ys.data_ptr(), pos.data_ptr(), y.data_ptr(), y.stride(0), T, W, int(top), _stream())
    return y
