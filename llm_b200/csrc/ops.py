"""Python faces of the kernels: each takes torch tensors on the GPU, checks what
the kernel assumes, and calls the C entry point on the current stream.  There is
no other implementation behind them: without the library, or with a tensor that is
not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load, load_tensor

_F32, _BF16 = 0, 1


class KernelError(RuntimeError):
    pass


class PartialSum:
    """The result of a split-K product that has not been summed yet: float32
    [splits, rows, cols] in the shared scratch buffer.  The kernels that take one sum it on
    the fly, in the order of the splits.  It lives in one buffer per device and is valid only
    until the next product runs: consume it first."""

    def __init__(self, buf: torch.Tensor, splits: int, rows: int, cols: int, dtype: torch.dtype):
        self.buf, self.splits, self.rows, self.cols, self.dtype = buf, splits, rows, cols, dtype

    @property
    def split_stride(self) -> int:
        return self.rows * self.cols


def _split_args(x):
    """(direct pointer, partials pointer, splits, split stride) of a tensor, a PartialSum or None."""
    if isinstance(x, PartialSum):
        return c_void_p(0), c_void_p(x.buf.data_ptr()), c_int(x.splits), c_longlong(x.split_stride)
    return _ptr(x), c_void_p(0), c_int(0), c_longlong(0)


def settle(x, out: torch.Tensor, rows: int) -> torch.Tensor:
    """x itself if it is a tensor; the sum of a PartialSum's splits, written to out[:rows] (contiguous), otherwise."""
    if not isinstance(x, PartialSum):
        return x
    assert out.is_contiguous() and out.shape[-1] == x.cols and x.rows == rows
    _check_t(load_tensor().llmk_reduce_partials(_ptr(out), c_void_p(x.buf.data_ptr()), c_longlong(rows * x.cols), c_int(x.splits),
                                                c_int(_kind(out.dtype)), _stream()))
    return out


def _kind(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(t, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


_STREAM = None


def set_stream(handle) -> None:
    """Fix the CUDA stream that the kernels launch on (a raw handle), or None to go back to
    asking torch for its current stream at every launch, which costs several microseconds."""
    global _STREAM
    _STREAM = handle


def _stream():
    if _STREAM is not None:
        return c_void_p(_STREAM)
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches issued through this module so far (graph replays included)."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, tensor: bool = False) -> None:
    """Count a launch; raise with the text of the library that reported an error."""
    global _LAUNCHES
    _LAUNCHES += 1
    if code != 0:
        msg = (load_tensor() if tensor else load()).llmk_last_error().decode("utf-8", "replace")
        raise KernelError(f"kernel call failed ({code}): {msg}")


def _check_t(code: int) -> None:
    _check(code, tensor=True)


def _rows_contig(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with unit stride in its last dimension")


def embedding(resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, n_tokens: int,
              status: torch.Tensor, scale: float = 1.0) -> None:
    """resid[:n_tokens] (float32) = table[ids] * scale; an id outside the table sets status[0]."""
    assert resid.dtype == torch.float32 and ids.dtype == torch.int32 and status.dtype == torch.int32
    assert resid.is_contiguous() and table.is_contiguous()
    vocab, hidden = table.shape
    _check(load().llmk_embedding_scaled(_ptr(resid), _ptr(table), _ptr(ids), c_int(n_tokens), c_int(hidden),
                                        c_int(vocab), c_int(_kind(table.dtype)), _ptr(status), c_float(scale), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta, gamma: torch.Tensor, out, rows: int, eps: float) -> None:
    """resid[:rows] += delta (a tensor or a PartialSum, if given); out[:rows] = rmsnorm(resid) * gamma
    (if out given)."""
    assert resid.dtype == torch.float32 and gamma.dtype == torch.float32 and resid.is_contiguous()
    hidden = resid.shape[-1]
    ref = out if out is not None else delta
    if ref is None:
        return
    if isinstance(delta, PartialSum):
        assert delta.cols == hidden and delta.rows == rows
    elif delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == hidden
    if out is not None:
        assert out.is_contiguous() and out.shape[-1] == hidden
        if delta is not None:
            assert delta.dtype == out.dtype
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_add_rmsnorm(_ptr(resid), d, parts, splits, stride, _ptr(gamma), _ptr(out), c_int(rows),
                                   c_int(hidden), c_float(eps), c_int(_kind(ref.dtype)), _stream()))


def add_dyt(resid: torch.Tensor, delta, w: torch.Tensor, b: torch.Tensor, alpha: float, out, rows: int) -> None:
    """resid[:rows] += delta (a tensor or a PartialSum, if given); out[:rows] = tanh(alpha * resid) * w + b
    (if out given): Dynamic Tanh, a norm without statistics."""
    assert resid.dtype == torch.float32 and w.dtype == torch.float32 and b.dtype == torch.float32
    assert resid.is_contiguous() and w.is_contiguous() and b.is_contiguous()
    hidden = resid.shape[-1]
    ref = out if out is not None else delta
    if ref is None:
        return
    if isinstance(delta, PartialSum):
        assert delta.cols == hidden and delta.rows == rows
    elif delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == hidden
    if out is not None:
        assert out.is_contiguous() and out.shape[-1] == hidden
        if delta is not None:
            assert delta.dtype == out.dtype
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_add_dyt(_ptr(resid), d, parts, splits, stride, _ptr(w), _ptr(b), c_float(alpha), _ptr(out),
                               c_int(rows), c_int(hidden), c_int(_kind(ref.dtype)), _stream()))


def add_layernorm(resid: torch.Tensor, delta, post, mult: float, pre, out, rows: int, eps: float) -> None:
    """LayerNorm (a weight, no bias, float32 statistics) on both sides of the residual sum:
    resid[:rows] += mult * ln(delta; post) where delta (a tensor or a PartialSum) is given (post None: mult * delta);
    out[:rows] = ln(resid; pre) where out is given."""
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    hidden = resid.shape[-1]
    ref = out if out is not None else delta
    if ref is None:
        return
    for w in (post, pre):
        assert w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == hidden)
    if isinstance(delta, PartialSum):
        assert delta.cols == hidden and delta.rows == rows
    elif delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == hidden
    if out is not None:
        assert pre is not None and out.is_contiguous() and out.shape[-1] == hidden
        assert delta is None or delta.dtype == out.dtype
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_add_layernorm(_ptr(resid), d, parts, splits, stride, _ptr(post), c_float(mult), _ptr(pre), _ptr(out),
                                     c_int(rows), c_int(hidden), c_float(eps), c_int(_kind(ref.dtype)), _stream()))


def softcap(x: torch.Tensor, rows: int, cap: float) -> None:
    """x[:rows] = cap * tanh(x / cap), float32 in place."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(load().llmk_softcap(_ptr(x), c_longlong(rows * x.shape[-1]), c_float(cap), _stream()))


def concat_embedding(out: torch.Tensor, resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, n_tokens: int) -> None:
    """out[t] = [resid[t] rounded to out's dtype ; table[ids[t]]], width 2 * hidden."""
    vocab, hidden = table.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[-1] == hidden and ids.dtype == torch.int32
    assert out.is_contiguous() and out.shape[-1] == 2 * hidden and out.dtype == table.dtype and table.is_contiguous()
    _check(load().llmk_concat_embedding(_ptr(out), _ptr(resid), _ptr(table), _ptr(ids), c_int(n_tokens), c_int(hidden),
                                        c_int(vocab), c_int(_kind(out.dtype)), _stream()))


def head_rmsnorm_gate(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, gate, rows: int, heads: int, eps: float) -> None:
    """out[t, h] = x[t, h] / sqrt(mean(x[t, h]^2) + eps) * w * silu(gate[t, h]) per head of x float32 [rows, heads * n];
    w float32 [n] is shared by the heads; gate (the dtype of out, rows may be strided) or None."""
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[-1] == x.shape[-1]
    n = x.shape[-1] // heads
    assert n * heads == x.shape[-1] and w.dtype == torch.float32 and w.numel() == n
    if gate is not None:
        _rows_contig(gate, "gate")
        assert gate.dtype == out.dtype and gate.shape[1] == x.shape[-1]
    _check(load().llmk_head_rmsnorm_gate(_ptr(out), _ptr(x), _ptr(w), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0),
                                         c_int(rows), c_int(heads), c_int(n), c_float(eps), c_int(_kind(out.dtype)), _stream()))


def rope_pairs_kv_write(qkv, freqs, positions: torch.Tensor, slot_map, k_pages, v_pages, n_tokens: int, n_heads: int,
                        n_kv: int, dim: int, vdim: int, q_out=None) -> torch.Tensor:
    """Rotate the neighbouring pairs (2i, 2i+1), i < len(freqs), of every q and k head by position * freqs[i] and store
    k and v at slot_map in the pages (n_kv 0: queries only).  qkv is a tensor [T, >= n_heads*dim + n_kv*(dim+vdim)]
    (q is then rotated in place unless q_out is given) or a PartialSum (q_out required).  Returns the rotated q."""
    assert positions.dtype == torch.int32
    width = n_heads * dim + n_kv * (dim + vdim)
    if isinstance(qkv, PartialSum):
        assert q_out is not None and qkv.cols >= width
        src_stride = qkv.cols
    else:
        _rows_contig(qkv, "qkv")
        assert qkv.shape[1] >= width
        src_stride = qkv.stride(0)
        if q_out is None:
            q_out = qkv
    _rows_contig(q_out, "q_out")
    assert q_out.dtype == qkv.dtype
    page = 1
    if n_kv:
        assert slot_map.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert k_pages.shape[1] == n_kv and k_pages.shape[3] == dim and v_pages.shape[3] == vdim
        page = k_pages.shape[2]
    pairs = 0 if freqs is None else freqs.numel()
    assert freqs is None or (freqs.dtype == torch.float32 and freqs.is_contiguous())
    d, parts, splits, stride = _split_args(qkv)
    _check(load().llmk_rope_pairs_kv_write(d, parts, splits, stride, c_longlong(src_stride), _ptr(q_out), c_longlong(q_out.stride(0)),
                                           _ptr(freqs), c_int(pairs), _ptr(positions), _ptr(slot_map), _ptr(k_pages), _ptr(v_pages),
                                           c_int(n_tokens), c_int(n_heads), c_int(n_kv), c_int(dim), c_int(vdim), c_int(page),
                                           c_int(_kind(qkv.dtype)), _stream()))
    return q_out


def gla_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias, tau: float,
             q_scale: float, state: torch.Tensor, state_slots: torch.Tensor, cu_tokens: torch.Tensor, n_entries: int,
             n_tokens: int = 0, seg_len: int = 0, seg_state=None, seg_decay=None) -> None:
    """The gated-linear-attention recurrence over every entry's tokens (see recurrent.cu): q, k [T, heads*dim] and
    v [T, heads*vdim] are column ranges of one projection (equal row strides), z float32 [T, heads*dim] the decay's
    pre-activation (+ z_bias), state float32 [slots, heads, dim, vdim] read and written at state_slots[entry],
    out float32 [T, heads*vdim].  seg_len > 0: entries run as segments of that many tokens side by side, in two passes;
    n_tokens is the step's token count and seg_state / seg_decay are float32 scratch for n_tokens // seg_len + n_entries
    segments ([.., heads, dim, vdim] and [.., heads, dim]); z is then overwritten with the decays."""
    heads, dim, vdim = state.shape[1], state.shape[2], state.shape[3]
    if seg_len:
        segs = n_tokens // seg_len + n_entries
        assert seg_state.dtype == seg_decay.dtype == torch.float32 and seg_state.is_contiguous() and seg_decay.is_contiguous()
        assert seg_state.numel() >= segs * heads * dim * vdim and seg_decay.numel() >= segs * heads * dim
    for t in (q, k, v, z, out):
        _rows_contig(t, "gla operand")
    assert q.stride(0) == k.stride(0) == v.stride(0) and q.dtype == k.dtype == v.dtype
    assert q.shape[1] == k.shape[1] == z.shape[1] == heads * dim and v.shape[1] == out.shape[1] == heads * vdim
    assert z.dtype == out.dtype == state.dtype == torch.float32 and state.is_contiguous()
    assert state_slots.dtype == cu_tokens.dtype == torch.int32
    assert z_bias is None or (z_bias.dtype == torch.float32 and z_bias.numel() == heads * dim)
    _check(load().llmk_gla_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), _ptr(z),
                                c_longlong(z.stride(0)), _ptr(z_bias), c_float(tau), c_float(q_scale), _ptr(state), _ptr(state_slots),
                                _ptr(cu_tokens), c_int(n_entries), c_int(heads), c_int(dim), c_int(vdim), c_int(_kind(q.dtype)),
                                _stream(), c_int(n_tokens), c_int(seg_len), _ptr(seg_state), _ptr(seg_decay)))
    if seg_len:
        count_launches(3)


ACTIVATIONS = {"relu2": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "tanh": 4}
EPILOGUE_ACTIVATIONS = ("relu2", "gelu", "gelu_tanh", "silu")      # those the product kernels apply in their epilogues


def act_rows(out: torch.Tensor, x, rows: int, kind: str) -> None:
    """out[:rows] = act(x[:rows]) element by element in float32; x a tensor or a PartialSum.
    kind: "relu2" (the square of relu), "gelu" (erf), "gelu_tanh", "silu"."""
    cols = out.shape[-1]
    assert out.is_contiguous() and out.dtype == x.dtype
    if isinstance(x, PartialSum):
        assert x.cols == cols and x.rows == rows
    else:
        assert x.is_contiguous() and x.shape[-1] == cols
    d, parts, splits, stride = _split_args(x)
    _check(load().llmk_act_rows(_ptr(out), d, parts, splits, stride, c_longlong(rows * cols), c_int(ACTIVATIONS[kind]),
                                c_int(_kind(out.dtype)), _stream()))


HEADS_ON_TENSOR_CORES = True


def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, heads: int, gate=None) -> None:
    """Per-head products in one launch: out[:, h*N:(h+1)*N] = a[:, h*K:(h+1)*K] @ w[h].T for w [heads, N, K];
    with a gate [rows, >= heads] (a view with unit column stride) head h of a row is multiplied by
    sigmoid(gate[row, h]).  Float32 accumulation on the CUDA cores in a fixed k order."""
    _rows_contig(a, "a"); _rows_contig(out, "out")
    assert w.dim() == 3 and w.is_contiguous() and w.shape[0] == heads and a.dtype == w.dtype == out.dtype
    n, k = w.shape[1], w.shape[2]
    assert a.shape[1] == heads * k and out.shape[1] == heads * n
    if gate is not None:
        _rows_contig(gate, "gate")
        assert gate.dtype == a.dtype and gate.shape[1] >= heads
    if (HEADS_ON_TENSOR_CORES and a.dtype == torch.bfloat16 and rows >= NORMAL_MODE_FROM_ROWS and k % 8 == 0
            and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        # enough rows to fill an MMA's 128: one launch of the tcgen05 kernel, a product per head along the grid's z
        _check_t(load_tensor().llmk_gemm_tc_grouped(
            _ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k), c_longlong(a.stride(0)), c_longlong(k),
            c_longlong(out.stride(0)), c_int(_BF16), c_int(1), c_int(heads), c_int(k), c_longlong(n), c_void_p(0), c_void_p(0),
            c_int(-1), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0), c_int(0), _stream()))
        return
    _check(load().llmk_gemm_simt_batched(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                                         c_longlong(a.stride(0)), c_longlong(k), c_longlong(out.stride(0)), c_int(heads),
                                         c_longlong(k), c_longlong(n * k), c_longlong(n), _ptr(gate),
                                         c_longlong(gate.stride(0) if gate is not None else 0), c_int(_kind(a.dtype)), _stream()))


def latent_norm_store(x: torch.Tensor, gain: torch.Tensor, eps: float, slot_map: torch.Tensor, pages: torch.Tensor,
                      n_tokens: int) -> None:
    """pages[slot_map[t]] = x[t] / sqrt(mean(x[t]^2) + eps) * gain for the first rank = len(gain) columns of x;
    pages [pages, 1, page_size, width] with width >= rank (the rest of a row is written as zeros)."""
    _rows_contig(x, "x")
    rank, width = gain.numel(), pages.shape[3]
    assert pages.is_contiguous() and pages.shape[1] == 1 and pages.dtype == x.dtype and x.shape[1] >= rank and width >= rank
    assert gain.dtype == torch.float32 and slot_map.dtype == torch.int32
    _check(load().llmk_latent_norm_store(_ptr(x), c_longlong(x.stride(0)), _ptr(gain), c_float(eps), _ptr(slot_map),
                                         _ptr(pages), c_int(n_tokens), c_int(rank), c_int(width), c_int(_kind(x.dtype)), _stream()))


# ---- hyper-connections (hyper.cu) -------------------------------------------------------

def hc_embedding(resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, n_tokens: int, streams: int,
                 status: torch.Tensor) -> None:
    """resid[:n_tokens] (float32 [.., streams * hidden]): every stream of a token = table[ids]; an id outside the table
    sets status[0]."""
    vocab, hidden = table.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[-1] == streams * hidden
    assert ids.dtype == torch.int32 and status.dtype == torch.int32 and table.is_contiguous()
    _check(load().llmk_hc_embedding(_ptr(resid), _ptr(table), _ptr(ids), c_int(n_tokens), c_int(hidden), c_int(vocab),
                                    c_int(streams), c_int(_kind(table.dtype)), _ptr(status), _stream()))


def hc_norm(resid: torch.Tensor, y, write_mix, write_out, read_in, gain, out, rows: int, hidden: int, streams: int,
            eps: float, dtype: torch.dtype) -> None:
    """The streams of resid[:rows] (float32 [.., streams * hidden]) first take the pending write, if y is given (a tensor
    or a PartialSum [rows, hidden]): x_t <- sum_s write_mix[s, t] x_s + write_out[t] y; then, if out is given,
    out[:rows] = rms(sum_s read_in[s] x_s) * gain (gain one float32 number).  All weights float32 on the device."""
    assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape[-1] == streams * hidden
    for t, n in ((write_mix, streams * streams), (write_out, streams), (read_in, streams), (gain, 1)):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n)
    if isinstance(y, PartialSum):
        assert y.cols == hidden and y.rows == rows
    elif y is not None:
        assert y.is_contiguous() and y.shape[-1] == hidden and y.dtype == dtype
    if out is not None:
        assert out.is_contiguous() and out.shape[-1] == hidden and out.dtype == dtype
    if y is None and out is None:
        return
    d, parts, splits, stride = _split_args(y)
    _check(load().llmk_hc_norm(_ptr(resid), d, parts, splits, stride, _ptr(write_mix if y is not None else None),
                               _ptr(write_out if y is not None else None), _ptr(read_in), _ptr(gain), _ptr(out), c_int(rows),
                               c_int(hidden), c_int(streams), c_float(eps), c_int(_kind(dtype)), _stream()))


def hc_gather_sum(out: torch.Tensor, resid: torch.Tensor, rows: torch.Tensor, n_rows: int, streams: int) -> None:
    """out[r] = the sum over the streams of resid[rows[r]], float32."""
    hidden = out.shape[-1]
    assert out.dtype == resid.dtype == torch.float32 and rows.dtype == torch.int32 and resid.shape[-1] == streams * hidden
    _check(load().llmk_hc_gather_sum(_ptr(out), _ptr(resid), _ptr(rows), c_int(n_rows), c_int(hidden), c_int(streams), _stream()))


def scalar_rmsnorm_rows(out: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, n_rows: int, eps: float) -> None:
    """out[:n_rows] = x / sqrt(mean(x^2) + eps) * gain for float32 rows x and one float32 number gain."""
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[-1] == x.shape[-1]
    assert gain.dtype == torch.float32 and gain.numel() == 1
    _check(load().llmk_scalar_rmsnorm_rows(_ptr(out), _ptr(x), _ptr(gain), c_int(n_rows), c_int(x.shape[-1]), c_float(eps),
                                           c_int(_kind(out.dtype)), _stream()))


def diff_combine(out: torch.Tensor, a: torch.Tensor, gate, rows: int, heads: int, per_group: int, lam: float, post: float,
                 eps: float) -> None:
    """Two attention maps per head combined: a [rows, 2 * heads * V] holds the maps' outputs ordered [kv group][map][head
    within the group]; out[t, h] = rms_unit(a1 - lam * a2) * post * sigmoid(gate[t, h]) (gate in out's dtype, rows may be
    strided, or None), heads in their own order."""
    _rows_contig(a, "a")
    vdim = out.shape[-1] // heads
    assert out.is_contiguous() and out.dtype == a.dtype and a.shape[1] == 2 * heads * vdim and heads % per_group == 0
    if gate is not None:
        _rows_contig(gate, "gate")
        assert gate.dtype == out.dtype and gate.shape[1] == heads * vdim
    _check(load().llmk_diff_combine(_ptr(out), _ptr(a), c_longlong(a.stride(0)), _ptr(gate),
                                    c_longlong(gate.stride(0) if gate is not None else 0), c_int(rows), c_int(heads),
                                    c_int(per_group), c_int(vdim), c_float(lam), c_float(post), c_float(eps),
                                    c_int(_kind(out.dtype)), _stream()))


def scaled_sum(out: torch.Tensor, a, b, sa: float, sb: float, rows: int) -> None:
    """out[:rows] = sa * a + sb * b; a and b tensors or PartialSums [rows, width]."""
    width = out.shape[-1]
    assert out.is_contiguous()
    for t in (a, b):
        if isinstance(t, PartialSum):
            assert t.cols == width and t.rows == rows
        else:
            assert t.is_contiguous() and t.shape[-1] == width and t.dtype == out.dtype
    da, pa, sa_, sta = _split_args(a)
    db, pb, sb_, stb = _split_args(b)
    _check(load().llmk_scaled_sum(_ptr(out), da, pa, sa_, sta, db, pb, sb_, stb, c_float(sa), c_float(sb), c_int(rows),
                                  c_int(width), c_int(_kind(out.dtype)), _stream()))


def head_norm_kv_write(qkv, q_gain, k_gain, eps: float, slot_map, k_pages, v_pages, n_tokens: int, n_q: int, n_k: int, n_v: int,
                       dim: int, vdim: int, q_out=None) -> torch.Tensor:
    """A row of n_q query heads and n_k key heads of dim, then n_v value heads of vdim (a tensor or a PartialSum): every q
    and k head is RMS-normed on its own with one shared weight (q_gain, k_gain float32 [dim]; None: not normed); q goes to
    q_out (the source itself for a tensor unless given), k and v to slot_map in pages of n_k and n_v heads.  Returns q."""
    width = (n_q + n_k) * dim + n_v * vdim
    if isinstance(qkv, PartialSum):
        assert q_out is not None and qkv.cols >= width
        src_stride = qkv.cols
    else:
        _rows_contig(qkv, "qkv")
        assert qkv.shape[1] >= width
        src_stride = qkv.stride(0)
        if q_out is None:
            q_out = qkv
    _rows_contig(q_out, "q_out")
    assert q_out.dtype == qkv.dtype and slot_map.dtype == torch.int32
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype == qkv.dtype
    assert k_pages.shape[1] == n_k and k_pages.shape[3] == dim and v_pages.shape[1] == n_v and v_pages.shape[3] == vdim
    for t in (q_gain, k_gain):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == dim)
    d, parts, splits, stride = _split_args(qkv)
    _check(load().llmk_head_norm_kv_write(d, parts, splits, stride, c_longlong(src_stride), _ptr(q_out), c_longlong(q_out.stride(0)),
                                          _ptr(q_gain), _ptr(k_gain), c_float(eps), _ptr(slot_map), _ptr(k_pages), _ptr(v_pages),
                                          c_int(n_tokens), c_int(n_q), c_int(n_k), c_int(n_v), c_int(dim), c_int(vdim),
                                          c_int(k_pages.shape[2]), c_int(_kind(qkv.dtype)), _stream()))
    return q_out


# ---- short convolution (short_conv.cu) ----------------------------------------------------

def short_conv(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, bias, state: torch.Tensor, ctx, residual: bool = False,
               silu: bool = False) -> None:
    """out[t] = conv(x)_t (+ x_t if residual; silu of it if asked) over every entry's tokens, the entry's last taps - 1
    inputs before this step read from, and afterwards kept in, state [slots, >= (taps - 1) * channels] float32 (rows may be
    strided: a column range of a wider state).  w float32 [taps, channels] (a row per tap, the oldest input's first); bias
    float32 [channels] or None."""
    _rows_contig(out, "out"); _rows_contig(x, "x"); _rows_contig(state, "state")
    taps, channels = w.shape
    assert x.shape[1] == out.shape[1] == channels and x.dtype == out.dtype
    assert w.dtype == torch.float32 and w.is_contiguous() and state.dtype == torch.float32
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == channels)
    assert state.shape[1] >= (taps - 1) * channels
    _check(load().llmk_short_conv(_ptr(out), c_longlong(out.stride(0)), _ptr(x), c_longlong(x.stride(0)), _ptr(w), _ptr(bias),
                                  _ptr(state), c_longlong(state.stride(0)), _ptr(ctx.state_slots), _ptr(ctx.token_entry),
                                  _ptr(ctx.cu_tokens), c_int(ctx.n_tokens), c_int(ctx.n_entries), c_int(channels), c_int(taps),
                                  c_int(int(residual)), c_int(int(silu)), c_int(_kind(x.dtype)), _stream()))
    if taps > 1 and ctx.n_tokens != ctx.n_entries:
        count_launches(1)            # the state's update is a launch of its own unless every entry brings one token


# ---- recurrences with a diagonal decay (scan.cu) ------------------------------------------

def token_shift(out: torch.Tensor, h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, ctx) -> None:
    """out[t, m*W:(m+1)*W] = h_t + (h_(t-1) - h_t) * mu[m] for every mix m; the row before an entry's first token is
    state[slot] (float32 [slots, >= W], zero at admission; the recurrence kernel that follows renews it)."""
    _rows_contig(out, "out"); _rows_contig(h, "h"); _rows_contig(state, "state")
    mixes, width = mu.shape
    assert h.shape[1] == width and out.shape[1] == mixes * width and out.dtype == h.dtype
    assert mu.dtype == state.dtype == torch.float32 and mu.is_contiguous() and state.shape[1] >= width
    _check(load().llmk_token_shift(_ptr(out), c_longlong(out.stride(0)), _ptr(h), c_longlong(h.stride(0)), _ptr(mu), _ptr(state),
                                   c_longlong(state.stride(0)), _ptr(ctx.state_slots), _ptr(ctx.token_entry), _ptr(ctx.cu_tokens),
                                   c_int(ctx.n_tokens), c_int(width), c_int(mixes), c_int(_kind(h.dtype)), _stream()))


def _segment_scratch(ctx, seg_len: int, seg_state, seg_decay, state_numel: int, decay_numel: int):
    if not seg_len:
        return c_void_p(0), c_void_p(0)
    segs = ctx.n_tokens // seg_len + ctx.n_entries
    assert seg_state.dtype == seg_decay.dtype == torch.float32 and seg_state.is_contiguous() and seg_decay.is_contiguous()
    assert seg_state.numel() >= segs * state_numel and seg_decay.numel() >= segs * decay_numel
    return _ptr(seg_state), _ptr(seg_decay)


def wkv_scan(out: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: torch.Tensor,
             bonus: torch.Tensor, state: torch.Tensor, ctx, shift_src=None, shift_state=None, seg_len: int = 0,
             seg_state=None, seg_decay=None) -> None:
    """o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t; S_t = diag(exp(-exp(z_t + z_bias))) S_(t-1) + k_t v_t^T per head (scan.cu).
    r, k, v [T, heads*dim]: column ranges of one projection; z float32 [T, heads*dim]; bonus float32 [heads, dim];
    state float32 [slots, >= heads*dim*dim]; out float32 [T, heads*dim].  shift_src [T, W] / shift_state [slots, >= W]:
    the last row of every entry is kept there for the next step's token shift.  seg_len > 0: entries run as segments of that
    many tokens side by side in two passes; seg_state / seg_decay are float32 scratch for n_tokens // seg_len + n_entries
    segments of heads*dim*dim and heads*dim numbers."""
    for t in (out, r, k, v, z, state):
        _rows_contig(t, "wkv operand")
    heads, dim = bonus.shape
    assert r.stride(0) == k.stride(0) == v.stride(0) and r.dtype == k.dtype == v.dtype
    assert r.shape[1] == k.shape[1] == v.shape[1] == z.shape[1] == out.shape[1] == heads * dim
    assert z.dtype == out.dtype == state.dtype == bonus.dtype == z_bias.dtype == torch.float32
    assert bonus.is_contiguous() and z_bias.numel() == heads * dim and state.shape[1] >= heads * dim * dim
    width = 0
    if shift_src is not None:
        _rows_contig(shift_src, "shift_src"); _rows_contig(shift_state, "shift_state")
        width = shift_src.shape[1]
        assert shift_src.dtype == r.dtype and shift_state.dtype == torch.float32 and shift_state.shape[1] >= width
    _check(load().llmk_wkv_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(r), _ptr(k), _ptr(v), c_longlong(r.stride(0)), _ptr(z),
                                c_longlong(z.stride(0)), _ptr(z_bias), _ptr(bonus), _ptr(state), c_longlong(state.stride(0)),
                                _ptr(ctx.state_slots), _ptr(ctx.cu_tokens), c_int(ctx.n_entries), c_int(heads), c_int(dim),
                                _ptr(shift_src), c_longlong(shift_src.stride(0) if shift_src is not None else 0), _ptr(shift_state),
                                c_longlong(shift_state.stride(0) if shift_state is not None else 0), c_int(width),
                                c_int(_kind(r.dtype)), _stream(), c_int(ctx.n_tokens), c_int(seg_len),
                                *_segment_scratch(ctx, seg_len, seg_state, seg_decay, heads * dim * dim, heads * dim)))
    if seg_len:
        count_launches(2)


def ssd_scan(out: torch.Tensor, x: torch.Tensor, b: torch.Tensor, c: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor,
             a_log: torch.Tensor, skip: torch.Tensor, state: torch.Tensor, ctx, heads: int, groups: int, dim: int, vdim: int,
             seg_len: int = 0, seg_state=None, seg_decay=None) -> None:
    """S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + skip x_t per head, dt_t = softplus(dt + dt_bias),
    a_t = exp(-exp(a_log) dt_t) (scan.cu).  x [T, heads*vdim], b and c [T, groups*dim] (one row stride), dt [T, heads];
    dt_bias, a_log, skip float32 [heads]; state float32 [slots, >= heads*dim*vdim]; out float32 [T, heads*vdim]."""
    for t in (out, x, b, c, dt, state):
        _rows_contig(t, "ssd operand")
    assert b.stride(0) == c.stride(0) and x.dtype == b.dtype == c.dtype == dt.dtype
    assert x.shape[1] == out.shape[1] == heads * vdim and b.shape[1] == c.shape[1] == groups * dim and dt.shape[1] == heads
    assert out.dtype == state.dtype == torch.float32 and state.shape[1] >= heads * dim * vdim
    for t in (dt_bias, a_log, skip):
        assert t.dtype == torch.float32 and t.numel() == heads
    _check(load().llmk_ssd_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(x), c_longlong(x.stride(0)), _ptr(b), _ptr(c),
                                c_longlong(b.stride(0)), _ptr(dt), c_longlong(dt.stride(0)), _ptr(dt_bias), _ptr(a_log), _ptr(skip),
                                _ptr(state), c_longlong(state.stride(0)), _ptr(ctx.state_slots), _ptr(ctx.cu_tokens),
                                c_int(ctx.n_entries), c_int(heads), c_int(groups), c_int(dim), c_int(vdim), c_int(_kind(x.dtype)),
                                _stream(), c_int(ctx.n_tokens), c_int(seg_len),
                                *_segment_scratch(ctx, seg_len, seg_state, seg_decay, heads * dim * vdim, heads * dim)))
    if seg_len:
        count_launches(2)


def gate_scan(out: torch.Tensor, q: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias, lower: torch.Tensor,
              state: torch.Tensor, ctx, heads: int, dim: int, vdim: int, seg_len: int = 0, seg_state=None, seg_decay=None) -> None:
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T silu(q_t), f_t = lower + (1 - lower) sigmoid(z_t + z_bias)
    per head (scan.cu).  q [T, heads*dim], v [T, heads*vdim] in the compute dtype; z float32 [T, heads*dim]; z_bias, lower
    float32 [heads*dim]; state float32 [slots, >= heads*dim*vdim]; out float32 [T, heads*vdim].  Segments as in wkv_scan."""
    for t in (out, q, v, z, state):
        _rows_contig(t, "gate_scan operand")
    assert q.dtype == v.dtype and q.shape[1] == z.shape[1] == heads * dim and v.shape[1] == out.shape[1] == heads * vdim
    assert z.dtype == out.dtype == state.dtype == lower.dtype == torch.float32 and lower.numel() == heads * dim
    assert z_bias is None or (z_bias.dtype == torch.float32 and z_bias.numel() == heads * dim)
    assert state.shape[1] >= heads * dim * vdim
    _check(load().llmk_gate_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(v),
                                 c_longlong(v.stride(0)), _ptr(z), c_longlong(z.stride(0)), _ptr(z_bias), _ptr(lower), _ptr(state),
                                 c_longlong(state.stride(0)), _ptr(ctx.state_slots), _ptr(ctx.cu_tokens), c_int(ctx.n_entries),
                                 c_int(heads), c_int(dim), c_int(vdim), c_int(_kind(q.dtype)), _stream(), c_int(ctx.n_tokens),
                                 c_int(seg_len), *_segment_scratch(ctx, seg_len, seg_state, seg_decay, heads * dim * vdim, heads * dim)))
    if seg_len:
        count_launches(2)


def delta_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b: torch.Tensor, a: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, ctx, heads: int, qk_heads: int, dim: int,
               vdim: int, q_scale: float, norm_eps: float = 1e-6) -> None:
    """The gated delta rule (delta.cu): S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head, with q and k
    made unit vectors per head (q also times q_scale), beta = sigmoid(b), g = exp(-exp(a_log) softplus(a + dt_bias)).
    q, k [T, qk_heads*dim] (equal row strides), v [T, heads*vdim], b, a [T, heads] (equal row strides), all in the compute
    dtype; a_log, dt_bias float32 [heads]; state float32 [slots, >= heads*dim*vdim]; out float32 [T, heads*vdim]."""
    for t in (out, q, k, v, b, a, state):
        _rows_contig(t, "delta_scan operand")
    assert q.stride(0) == k.stride(0) and b.stride(0) == a.stride(0) and q.dtype == k.dtype == v.dtype == b.dtype == a.dtype
    assert q.shape[1] == k.shape[1] == qk_heads * dim and v.shape[1] == out.shape[1] == heads * vdim
    assert b.shape[1] == a.shape[1] == heads and out.dtype == state.dtype == torch.float32 and state.shape[1] >= heads * dim * vdim
    for t in (a_log, dt_bias):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads
    _check(load().llmk_delta_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(q), _ptr(k), c_longlong(q.stride(0)), _ptr(v),
                                  c_longlong(v.stride(0)), _ptr(b), _ptr(a), c_longlong(b.stride(0)), _ptr(a_log), _ptr(dt_bias),
                                  _ptr(state), c_longlong(state.stride(0)), _ptr(ctx.state_slots), _ptr(ctx.cu_tokens),
                                  c_int(ctx.n_entries), c_int(heads), c_int(qk_heads), c_int(dim), c_int(vdim), c_float(q_scale),
                                  c_float(norm_eps), c_int(_kind(q.dtype)), _stream()))


DELTA_CHUNK = 32       # tokens that the chunk-wise delta rule solves together (delta.cu)


def delta_chunk_scratch(n_chunks: int, heads: int, dim: int, vdim: int):
    """Float32 element counts of the chunk-wise delta rule's five scratch buffers for n_chunks chunks."""
    c = DELTA_CHUNK
    return [n_chunks * heads * n for n in (dim * 2 * c, c * dim, c * vdim, c * c, 1)]


def delta_chunk_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b: torch.Tensor, a: torch.Tensor,
                     a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, ctx, heads: int, qk_heads: int, dim: int,
                     vdim: int, q_scale: float, norm_eps: float, scratch) -> None:
    """delta_scan for a step with prompt portions: the rule chunk by chunk (32 tokens solved together, chunks chained through
    the state; see delta.cu).  scratch: five flat float32 tensors of at least delta_chunk_scratch(ctx.n_tokens // 32 +
    ctx.n_entries, ...) elements."""
    for t in (out, q, k, v, b, a, state):
        _rows_contig(t, "delta_chunk_scan operand")
    assert q.stride(0) == k.stride(0) and b.stride(0) == a.stride(0) and q.dtype == k.dtype == v.dtype == b.dtype == a.dtype
    assert q.shape[1] == k.shape[1] == qk_heads * dim and v.shape[1] == out.shape[1] == heads * vdim
    assert b.shape[1] == a.shape[1] == heads and out.dtype == state.dtype == torch.float32 and state.shape[1] >= heads * dim * vdim
    T = ctx.n_tokens
    for t, numel in zip(scratch, delta_chunk_scratch(T // DELTA_CHUNK + ctx.n_entries, heads, dim, vdim)):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= numel
    _check(load().llmk_delta_chunk_scan(_ptr(out), c_longlong(out.stride(0)), _ptr(q), _ptr(k), c_longlong(q.stride(0)), _ptr(v),
                                        c_longlong(v.stride(0)), _ptr(b), _ptr(a), c_longlong(b.stride(0)), _ptr(a_log),
                                        _ptr(dt_bias), _ptr(state), c_longlong(state.stride(0)), _ptr(ctx.state_slots),
                                        _ptr(ctx.cu_tokens), c_int(ctx.n_entries), c_int(T), c_int(heads), c_int(qk_heads),
                                        c_int(dim), c_int(vdim), c_float(q_scale), c_float(norm_eps), *[_ptr(t) for t in scratch],
                                        c_int(_kind(q.dtype)), _stream()))
    count_launches(1)


def group_rmsnorm_gate(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, rows: int, groups: int,
                       eps: float, gate_first: bool = False) -> None:
    """Per group of channels g: out = rms(x_g) * w_g * silu(gate_g), or with gate_first rms(x_g * silu(gate_g)) * w_g.
    x float32 [rows, groups * n] contiguous; w float32 [groups * n]; gate in out's dtype, rows may be strided."""
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape[-1] == x.shape[-1]
    n = x.shape[-1] // groups
    assert n * groups == x.shape[-1] and w.dtype == torch.float32 and w.numel() == x.shape[-1]
    _rows_contig(gate, "gate")
    assert gate.dtype == out.dtype and gate.shape[1] == x.shape[-1]
    _check(load().llmk_group_rmsnorm_gate(_ptr(out), _ptr(x), _ptr(w), _ptr(gate), c_longlong(gate.stride(0)), c_int(rows),
                                          c_int(groups), c_int(n), c_float(eps), c_int(int(gate_first)), c_int(_kind(out.dtype)),
                                          _stream()))


def pair_norm_mean(out: torch.Tensor, a, b, wa: torch.Tensor, wb: torch.Tensor, rows: int, eps: float) -> None:
    """out[:rows] = (rms(a) * wa + rms(b) * wb) / 2 row by row; a and b tensors or PartialSums [rows, width]."""
    width = out.shape[-1]
    assert out.is_contiguous() and wa.dtype == wb.dtype == torch.float32 and wa.numel() == wb.numel() == width
    for t in (a, b):
        if isinstance(t, PartialSum):
            assert t.cols == width and t.rows == rows
        else:
            assert t.is_contiguous() and t.shape[-1] == width and t.dtype == out.dtype
    da, pa, sa, sta = _split_args(a)
    db, pb, sb, stb = _split_args(b)
    _check(load().llmk_pair_norm_mean(_ptr(out), da, pa, sa, sta, db, pb, sb, stb, _ptr(wa), _ptr(wb), c_int(rows), c_int(width),
                                      c_float(eps), c_int(_kind(out.dtype)), _stream()))


def clamped_glu(out: torch.Tensor, gate_up, bias, rows: int, limit: float, alpha: float) -> None:
    """out[:rows, :I] = g * sigmoid(alpha g) * (u + 1), g = min(gate + b, limit), u = clamp(up + b, -limit, limit), for
    gate_up = [gate | up] (a tensor or a PartialSum [rows, 2 I]) and bias float32 [2 I] or None."""
    inter = out.shape[-1]
    assert out.is_contiguous() and out.dtype == gate_up.dtype
    if isinstance(gate_up, PartialSum):
        assert gate_up.cols == 2 * inter and gate_up.rows == rows
    else:
        assert gate_up.shape[-1] == 2 * inter and gate_up.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inter)
    d, parts, splits, stride = _split_args(gate_up)
    _check(load().llmk_clamped_glu(_ptr(out), d, parts, splits, stride, _ptr(bias), c_int(rows), c_int(inter), c_float(limit),
                                   c_float(alpha), c_int(_kind(out.dtype)), _stream()))


def latent_rope_norm_store(x: torch.Tensor, q_gain, q_rank: int, cq_out, gain: torch.Tensor, rot: int, freqs, positions,
                           eps: float, slot_map, pages, n_tokens: int) -> None:
    """x float32 [T, q_rank + rank + rot]: cq_out[t] = rms(x[:q_rank]) * q_gain (if q_rank), and the token's cache row
    pages[slot_map[t]] = [the rot last numbers with pairs (2i, 2i+1), i < len(freqs), turned by position * freqs[i] |
    rms(the rank numbers between) * gain | zeros]; pages None: no row is written."""
    _rows_contig(x, "x")
    rank = gain.numel()
    assert x.dtype == torch.float32 and x.shape[1] >= q_rank + rank + rot and gain.dtype == torch.float32
    pairs = 0 if freqs is None else freqs.numel()
    assert freqs is None or (freqs.dtype == torch.float32 and freqs.is_contiguous())
    kind = None
    if q_rank:
        _rows_contig(cq_out, "cq_out")
        assert q_gain.dtype == torch.float32 and q_gain.numel() == q_rank and cq_out.shape[1] >= q_rank
        kind = cq_out.dtype
    width = 0
    if pages is not None:
        assert pages.is_contiguous() and pages.shape[1] == 1 and slot_map.dtype == torch.int32
        assert kind is None or kind == pages.dtype
        kind, width = pages.dtype, pages.shape[3]
    _check(load().llmk_latent_rope_norm_store(_ptr(x), c_longlong(x.stride(0)), _ptr(q_gain), c_int(q_rank), _ptr(cq_out),
                                              c_longlong(cq_out.stride(0) if cq_out is not None else 0), _ptr(gain), c_int(rank),
                                              c_int(rot), _ptr(freqs), c_int(pairs), _ptr(positions), c_float(eps), _ptr(slot_map),
                                              _ptr(pages), c_int(n_tokens), c_int(width), c_int(_kind(kind)), _stream()))


def norm_rope_kv_write(qkv, q_gain, k_gain, eps: float, freqs, halves: bool, positions: torch.Tensor, slot_map, k_pages, v_pages,
                       n_tokens: int, n_heads: int, n_kv: int, dim: int, vdim: int, q_out=None) -> torch.Tensor:
    """As rope_pairs_kv_write, with the RMS norm of the token's whole q projection (weights q_gain, float32
    [n_heads * dim]) and whole k projection (k_gain [n_kv * dim]) first, either None for none, and the choice of pairs:
    halves turns channel i against channel i + len(freqs), else 2i against 2i + 1.  Returns the tensor that holds q."""
    assert positions.dtype == torch.int32
    width = n_heads * dim + n_kv * (dim + vdim)
    if isinstance(qkv, PartialSum):
        assert q_out is not None and qkv.cols >= width
        src_stride = qkv.cols
    else:
        _rows_contig(qkv, "qkv")
        assert qkv.shape[1] >= width
        src_stride = qkv.stride(0)
        if q_out is None:
            q_out = qkv
    _rows_contig(q_out, "q_out")
    assert q_out.dtype == qkv.dtype
    page = 1
    if n_kv:
        assert slot_map.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert k_pages.shape[1] == n_kv and k_pages.shape[3] == dim and v_pages.shape[3] == vdim
        page = k_pages.shape[2]
    pairs = 0 if freqs is None else freqs.numel()
    for t, n in ((q_gain, n_heads * dim), (k_gain, n_kv * dim), (freqs, pairs)):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n)
    d, parts, splits, stride = _split_args(qkv)
    _check(load().llmk_norm_rope_kv_write(d, parts, splits, stride, c_longlong(src_stride), _ptr(q_out), c_longlong(q_out.stride(0)),
                                          _ptr(q_gain), _ptr(k_gain), c_float(eps), _ptr(freqs), c_int(pairs), c_int(int(halves)),
                                          _ptr(positions), _ptr(slot_map), _ptr(k_pages), _ptr(v_pages), c_int(n_tokens),
                                          c_int(n_heads), c_int(n_kv), c_int(dim), c_int(vdim), c_int(page), c_int(_kind(qkv.dtype)),
                                          _stream()))
    return q_out


@functools.lru_cache(maxsize=None)
def moe_tile() -> int:
    """Slots per tile of the grouped products."""
    return int(load().llmk_moe_tile())


GROUPED_PERSISTENT = os.environ.get("LLM_B200_GROUPED_PERSISTENT", "1") != "0"      # see moe_gemm_tc
MOE_TC_TILE = 128       # slots per tile of the tensor-core grouped products (the MMA's 128 rows)


def moe_max_tiles(n_pairs: int, experts: int, tile: int = 0) -> int:
    """Tiles that the grouped list of n_pairs (token, choice) pairs can take at most."""
    return _ceil_div(n_pairs, tile or moe_tile()) + min(experts, n_pairs)


def moe_route(h: torch.Tensor, w: torch.Tensor, bias, logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
              n_tokens: int, top: int, over_all: bool = False, sigmoid_groups=None) -> None:
    """Router (over_all: the weights are the chosen experts' shares of the softmax over all experts, not
    renormalised): logits = h @ w.T with float32 accumulation (the tensor-core product in bfloat16 where it takes the
    shape, the CUDA-core product otherwise) into `logits` (float32 [>= n_tokens, experts]); plus bias, the `top`
    largest per token (ids, falling) and the softmax over those alone (weights)."""
    _rows_contig(h, "h")
    experts = w.shape[0]
    assert w.is_contiguous() and w.dtype == h.dtype and w.shape[1] == h.shape[1]
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.shape[1] == experts and logits.shape[0] >= n_tokens
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32 and ids.is_contiguous() and weights.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == experts)
    if gemm_fast_available(h, w, logits, n_tokens):
        z = gemm_fast(h, w, logits, n_tokens, allow_partial=True)
    else:
        gemm_simt(h, w, logits, n_tokens)
        z = logits
    d, parts, splits, stride = _split_args(z)
    if sigmoid_groups is not None:
        # (groups, keep): sigmoid scores, `bias` is the correction that enters the choice only; see routed.cu
        groups, keep = sigmoid_groups
        _check(load().llmk_moe_topk_sigmoid(d, parts, splits, stride, _ptr(bias), _ptr(ids), _ptr(weights), c_int(n_tokens),
                                            c_int(experts), c_int(top), c_int(groups), c_int(keep), _stream()))
        return
    _check(load().llmk_moe_topk(d, parts, splits, stride, _ptr(bias), _ptr(ids), _ptr(weights), c_int(n_tokens),
                                c_int(experts), c_int(top), c_int(int(over_all)), _stream()))


def moe_group(ids: torch.Tensor, n_pairs: int, experts: int, meta: torch.Tensor, tile_expert: torch.Tensor,
              slot_src: torch.Tensor, pair_slot: torch.Tensor, max_tiles: int, tile: int = 0) -> None:
    """Sort the pairs by expert into tiles of `tile` slots (see routed.cu); all int32 on the device."""
    tile = tile or moe_tile()
    for t in (ids, meta, tile_expert, slot_src, pair_slot):
        assert t.dtype == torch.int32 and t.is_contiguous()
    assert tile_expert.numel() >= max_tiles and slot_src.numel() >= max_tiles * tile and pair_slot.numel() >= n_pairs
    _check(load().llmk_moe_group(_ptr(ids), c_int(n_pairs), c_int(experts), _ptr(meta), _ptr(tile_expert), _ptr(slot_src),
                                 _ptr(pair_slot), c_int(max_tiles), c_int(tile), _stream()))


def moe_gather(out: torch.Tensor, x: torch.Tensor, slot_src, meta, div: int, tile: int, max_tiles: int) -> None:
    """out[slot] = x[pair of the slot // div] for the slots of the tiles in use, zeros in padding slots."""
    _rows_contig(x, "x")
    assert out.is_contiguous() and out.dtype == x.dtype and out.shape[1] == x.shape[1] and out.shape[0] >= max_tiles * tile
    _check(load().llmk_moe_gather(_ptr(out), _ptr(x), c_longlong(x.stride(0)), _ptr(slot_src), _ptr(meta), c_int(div),
                                  c_int(x.shape[1]), c_int(tile), c_int(max_tiles), c_int(_kind(x.dtype)), _stream()))


def moe_gemm_tc_available(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core grouped product takes these operands (bfloat16, rows of 16-byte multiples)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[2] % 8 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_gemm_tc(a: torch.Tensor, tile_expert, meta, w: torch.Tensor, out: torch.Tensor, max_tiles: int, act=None) -> None:
    """out[slot] = act(a[slot] @ w[expert of the slot's tile].T) on the tensor cores: a [slots, K] in slot order
    (tiles of 128 slots), w [experts, N, K], out bfloat16 or float32 [slots, N].  act "silu_gate": an expert's N rows
    are N/2 gate rows followed by N/2 up rows and out [slots, N/2] bfloat16 = silu(gate) * up, made in the epilogue."""
    _rows_contig(a, "a"); _rows_contig(out, "out")
    gated = act == "silu_gate"
    assert w.dim() == 3 and w.is_contiguous() and a.shape[1] == w.shape[2] and out.shape[1] == (w.shape[1] // 2 if gated else w.shape[1])
    assert not gated or (out.dtype == torch.bfloat16 and w.shape[1] % 2 == 0)
    rows = max_tiles * MOE_TC_TILE
    assert a.shape[0] >= rows and out.shape[0] >= rows
    _check_t(load_tensor().llmk_gemm_tc_grouped(
        _ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(w.shape[1]), c_int(w.shape[2]), c_longlong(a.stride(0)),
        c_longlong(w.shape[2]), c_longlong(out.stride(0)), c_int(_kind(out.dtype)), c_int(2), c_int(w.shape[0]), c_int(0),
        c_longlong(0), _ptr(tile_expert), _ptr(meta), c_int(4 if gated else ACTIVATIONS[act] if act else -1), c_void_p(0), c_longlong(0),
        c_int(int(GROUPED_PERSISTENT)), _stream()))


def moe_gemm(a: torch.Tensor, gather_div: int, slot_src, tile_expert, meta, w: torch.Tensor, out: torch.Tensor,
             max_tiles: int, act=None) -> None:
    """out[slot] = act(a[row of slot] @ w[expert of the slot's tile].T) for w [experts, N, K]; gather_div > 0:
    the row is the slot's pair // gather_div (its token), 0: the slot itself."""
    _rows_contig(a, "a"); _rows_contig(out, "out")
    assert w.dim() == 3 and w.is_contiguous() and w.dtype == a.dtype and a.shape[1] == w.shape[2] and out.shape[1] == w.shape[1]
    assert out.shape[0] >= max_tiles * moe_tile()
    _check(load().llmk_moe_gemm(_ptr(a), c_longlong(a.stride(0)), c_int(gather_div), _ptr(slot_src), _ptr(tile_expert),
                                _ptr(meta), _ptr(w), c_longlong(w.shape[2]), c_longlong(w.shape[1] * w.shape[2]), _ptr(out),
                                c_longlong(out.stride(0)), c_int(w.shape[1]), c_int(w.shape[2]), c_int(max_tiles),
                                c_int(ACTIVATIONS[act] if act else -1), c_int(_kind(a.dtype)), c_int(_kind(out.dtype)), _stream()))


def moe_combine(out: torch.Tensor, y: torch.Tensor, pair_slot, weights, shared, n_tokens: int, top: int) -> None:
    """out[t] = shared[t] (a tensor, a PartialSum or None) + sum_j weights[t, j] * y[pair_slot[t, j]]."""
    assert out.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous() and y.shape[1] == out.shape[1]
    d, parts, splits, stride = _split_args(shared)
    _check(load().llmk_moe_combine(_ptr(out), _ptr(y), _ptr(pair_slot), _ptr(weights), d, parts, splits, stride,
                                   c_int(n_tokens), c_int(top), c_int(out.shape[1]), c_int(_kind(out.dtype)), _stream()))


def gather_rows(out: torch.Tensor, resid: torch.Tensor, delta, rows: torch.Tensor, n_rows: int) -> None:
    """out[r] = resid[rows[r]] (+ delta[rows[r]], a tensor or a PartialSum), float32."""
    assert out.dtype == torch.float32 and resid.dtype == torch.float32 and rows.dtype == torch.int32
    kind = _kind(delta.dtype) if delta is not None else _F32
    d, parts, splits, stride = _split_args(delta)
    _check(load().llmk_gather_rows(_ptr(out), _ptr(resid), d, parts, splits, stride, _ptr(rows), c_int(n_rows),
                                   c_int(resid.shape[-1]), c_int(kind), _stream()))


def cast_rows(out: torch.Tensor, rows_f32: torch.Tensor, n_rows: int) -> None:
    """out[:n_rows] = rows_f32[:n_rows] rounded to out's dtype (float32 or bfloat16)."""
    assert rows_f32.dtype == torch.float32 and out.is_contiguous() and rows_f32.is_contiguous()
    assert out.shape[-1] == rows_f32.shape[-1]
    _check(load().llmk_cast_rows(_ptr(out), _ptr(rows_f32), c_longlong(n_rows * out.shape[-1]), c_int(_kind(out.dtype)),
                                 _stream()))


def add_bias(x: torch.Tensor, bias: torch.Tensor, rows: int) -> None:
    """x[:rows] += bias (float32 [cols]), in place."""
    _rows_contig(x, "x")
    assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == x.shape[1]
    _check(load().llmk_add_bias(_ptr(x), c_longlong(x.stride(0)), _ptr(bias), c_int(rows), c_int(x.shape[1]),
                                c_int(_kind(x.dtype)), _stream()))


GLU_ACTIVATIONS = {"silu": 0, "relu": 1}


def silu_mul(out: torch.Tensor, gate_up, rows: int, act: str = "silu") -> None:
    """out[:rows, :I] = act(gate_up[:, :I]) * gate_up[:, I:] with act silu or relu; gate_up a tensor or a PartialSum."""
    inter = out.shape[-1]
    assert out.is_contiguous() and out.dtype == gate_up.dtype
    if isinstance(gate_up, PartialSum):
        assert gate_up.cols == 2 * inter and gate_up.rows == rows
    else:
        assert gate_up.shape[-1] == 2 * inter and gate_up.is_contiguous()
    d, parts, splits, stride = _split_args(gate_up)
    _check(load().llmk_glu_mul(_ptr(out), d, parts, splits, stride, c_int(rows), c_int(inter),
                               c_int(_kind(out.dtype)), c_int(GLU_ACTIVATIONS[act]), _stream()))


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> None:
    """out[:rows] = a[:rows] @ w.T with float32 accumulation on the CUDA cores."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n and a.dtype == w.dtype
    _check(load().llmk_gemm_simt(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                                 c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                 c_int(_kind(a.dtype)), c_int(_kind(out.dtype)), _stream()))


def rope_kv_write(qkv, cos, sin, positions: torch.Tensor, slot_map: torch.Tensor,
                  k_pages, v_pages, n_tokens: int, n_heads: int, n_kv: int,
                  head_dim: int, q_out=None) -> torch.Tensor:
    """Rotate q and k by the tables, store k and v at slot_map in the pages.  qkv is a tensor
    [T, >= (n_heads + 2 n_kv) head_dim] (q is then rotated in place unless q_out is given) or a
    PartialSum of that shape (q_out is then required).  Returns the tensor that holds rotated q."""
    assert positions.dtype == torch.int32 and slot_map.dtype == torch.int32
    if isinstance(qkv, PartialSum):
        assert q_out is not None and qkv.cols >= (n_heads + 2 * n_kv) * head_dim
        src_stride = qkv.cols
    else:
        _rows_contig(qkv, "qkv")
        assert qkv.shape[1] >= (n_heads + 2 * n_kv) * head_dim
        src_stride = qkv.stride(0)
        if q_out is None:
            q_out = qkv
    _rows_contig(q_out, "q_out")
    assert q_out.dtype == qkv.dtype
    if n_kv:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert k_pages.shape[3] == head_dim and k_pages.shape[1] == n_kv
    page = k_pages.shape[2] if k_pages is not None else 1
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32
        assert cos.shape[1] == head_dim // 2 and cos.is_contiguous() and sin.is_contiguous()
    d, parts, splits, stride = _split_args(qkv)
    _check(load().llmk_rope_kv_write(d, parts, splits, stride, c_longlong(src_stride), _ptr(q_out),
                                     c_longlong(q_out.stride(0)), _ptr(cos), _ptr(sin),
                                     _ptr(positions), _ptr(slot_map), _ptr(k_pages), _ptr(v_pages),
                                     c_int(n_tokens), c_int(n_heads), c_int(n_kv), c_int(head_dim),
                                     c_int(page), c_int(_kind(qkv.dtype)), _stream()))
    return q_out


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, token_entry: torch.Tensor, positions: torch.Tensor,
                            n_tokens: int, n_heads: int, n_kv: int, head_dim: int, window: int,
                            scale: float, value_dim: int = 0, softcap: float = 0.0, sink: bool = False,
                            keep_first: int = 0, sink_values=None, chunk: int = 0, sigmoid_bias=None, dist_bias=None,
                            v_share: int = 1) -> None:
    """out[t, h*VS:(h+1)*VS] = causal (windowed) attention of q[t, h] over its request's pages.  value_dim: size of a
    value row where it differs from the keys' (0 = the same); softcap > 0: scores pass cap * tanh(s / cap); sink: the
    softmax's denominator gets one more term of score 0, or of score sink_values[h] (float32 [heads], not scaled);
    keep_first: with a window, the request's first keys stay visible; chunk > 0: instead of a window, a query sees the
    keys at or before it with the same floor(position / chunk); sigmoid_bias (float32 [heads]): the weight of a visible
    key is sigmoid(score + bias[h]) and nothing is normalised.  dist_bias (r1, r2), float32 [heads] each:
    r1[h] * ln(1 + r2[h] * distance) is taken off the capped score.  v_share > 1: v_pages holds n_kv / v_share heads and
    v_share neighbouring key heads read one of them."""
    r1, r2 = dist_bias if dist_bias is not None else (None, None)
    for t in (sink_values, sigmoid_bias, r1, r2):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
    assert v_share >= 1 and k_pages.shape[1] == n_kv and v_pages.shape[1] * v_share == n_kv
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert token_entry.dtype == torch.int32 and positions.dtype == torch.int32
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and q.dtype == k_pages.dtype == out.dtype
    _check(load().llmk_paged_attention_generic_ex(
        _ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(token_entry), _ptr(positions), c_int(n_tokens),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(value_dim or head_dim), c_int(k_pages.shape[2]), c_int(window or 0),
        c_int(keep_first or 0), c_float(scale), c_float(softcap or 0.0), c_int(int(bool(sink))), c_int(_kind(q.dtype)), _stream(),
        _ptr(sink_values), c_int(chunk or 0), _ptr(sigmoid_bias), _ptr(r1), _ptr(r2), c_int(v_share)))


def feed_tokens(token_ids: torch.Tensor, sampled: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, n: int) -> None:
    """token_ids[dst[i]] = sampled[src[i]] for i < n, all int32 on the device."""
    assert token_ids.dtype == sampled.dtype == dst.dtype == src.dtype == torch.int32
    _check(load().llmk_feed_tokens(_ptr(token_ids), _ptr(sampled), _ptr(dst), _ptr(src), c_int(n), _stream()))


def sample_rows(out: torch.Tensor, logits: torch.Tensor, rows: int, temperature=None, uniform=None) -> None:
    """out[r] = argmax of logits[r] (ties to the lowest id) where temperature[r] <= 0 or no
    temperatures are given, else the inverse-CDF draw of softmax(logits[r] / temperature[r])
    at uniform[r]."""
    _rows_contig(logits, "logits")
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and uniform is not None and uniform.dtype == torch.float32
    _check(load().llmk_sample_rows(_ptr(out), _ptr(logits), c_longlong(logits.stride(0)), c_int(rows),
                                   c_int(logits.shape[1]), _ptr(temperature), _ptr(uniform), _stream()))


_ATTN_PARTIALS = {}
_ATTN_PARTIALS_RETIRED = []      # outgrown buffers stay alive: captured graphs may still hold their addresses


def _attn_partials(device, n_floats: int) -> torch.Tensor:
    """Scratch of the decode attention; zeroed, because its first words are arrival counters
    that the kernel expects to be zero and leaves zero."""
    buf = _ATTN_PARTIALS.get(device)
    if buf is None or buf.numel() < n_floats:
        if buf is not None:
            _ATTN_PARTIALS_RETIRED.append(buf)
        buf = torch.zeros(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        _ATTN_PARTIALS[device] = buf
    return buf


def decode_splits(n_entries: int, n_kv: int, max_keys: int, sms: int = 0) -> int:
    """How many ranges the keys of one request are cut into.  Up to 2,048 keys: ranges of about
    128 keys (one tile of 32 per warp of a CTA) while the batch is small and the kernel bound by
    latency, fewer and longer ones as (requests x kv heads) grows, so that about 256 CTAs run; at
    most 16, and clusters of 7 or 8 CTAs measured slower than 6 longer ranges.  Beyond that the
    kernel is bound by bytes: as many ranges of at least 256 keys as fill the SMs with two CTAs
    each in one wave, at most 64.  sms: the device's SM count, if the caller has it."""
    pairs = max(1, n_entries * n_kv)
    if max_keys > 2048:
        return max(1, min(64, (2 * (sms or sm_count())) // pairs, max_keys // 256))
    s = max(1, min(16, _ceil_div(max_keys, 128), 256 // pairs))
    return 6 if s in (7, 8) else s


def paged_attention_decode(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, kv_lens: torch.Tensor, n_entries: int, n_heads: int,
                           n_kv: int, head_dim: int, window: int, scale: float, splits=None, max_keys: int = 0,
                           softcap: float = 0.0, sink: bool = False, keep_first: int = 0, sink_values=None, dist_bias=None,
                           v_share: int = 1) -> None:
    """One query token per entry (row e of q), attending to its request's kv_lens[e] keys.
    max_keys: an upper bound of kv_lens, if the host knows one below the table's width.
    softcap, sink, keep_first, dist_bias, v_share: as in paged_attention_generic (the CUDA-core kernel takes them)."""
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert kv_lens.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert q.dtype == k_pages.dtype == out.dtype
    page = k_pages.shape[2]
    if splits is None:
        splits = decode_splits(n_entries, n_kv, max_keys or block_table.shape[1] * page)
    buf = _attn_partials(q.device, _decode_scratch_floats(n_entries, n_heads, head_dim, splits))
    args = (_ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
            _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_lens), c_int(n_entries), c_int(n_heads),
            c_int(n_kv), c_int(head_dim), c_int(page), c_int(window or 0), c_float(scale), c_int(splits),
            c_void_p(buf.data_ptr()), c_int(_kind(q.dtype)))
    # bfloat16 with a head size of 64 or 128 and pages of a power of two: the query heads of a
    # group as rows of warp-level MMAs (tensor-core library); everything else on the CUDA cores
    assert sink_values is None or (sink_values.dtype == torch.float32 and sink_values.numel() == n_heads)
    r1, r2 = dist_bias if dist_bias is not None else (None, None)
    for t in (r1, r2):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
    assert v_share >= 1 and k_pages.shape[1] == n_kv and v_pages.shape[1] * v_share == n_kv
    extended = bool(softcap or sink or keep_first or dist_bias is not None or v_share > 1)
    if (not extended and q.dtype == torch.bfloat16 and head_dim in (64, 128) and page & (page - 1) == 0
            and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0):
        _check_t(load_tensor().llmk_paged_attention_decode_mma(*args, c_int(max_keys), _stream()))
    else:
        _check(load().llmk_paged_attention_decode_ex(*args, _stream(), c_float(softcap or 0.0), c_int(int(bool(sink))),
                                                     c_int(keep_first or 0), _ptr(sink_values), _ptr(r1), _ptr(r2), c_int(v_share)))


def _decode_scratch_floats(n_entries: int, n_heads: int, head_dim: int, splits: int) -> int:
    lib = load()
    lib.llmk_paged_attention_decode_scratch.restype = c_longlong
    return int(lib.llmk_paged_attention_decode_scratch(c_int(n_entries), c_int(n_heads), c_int(head_dim), c_int(splits)))


def decode_attention_fused_supported(qkv, cos, sin, head_dim: int, page_size: int = 16) -> bool:
    """Whether one kernel can rotate, store and attend for a decode step: bfloat16, head size 64
    or 128, pages of a power of two, rows that start on 16-byte boundaries."""
    if qkv.dtype != torch.bfloat16 or page_size & (page_size - 1):
        return False
    d, parts, _, stride = _split_args(qkv)
    src_stride = qkv.cols if isinstance(qkv, PartialSum) else qkv.stride(0)
    return bool(load_tensor().llmk_decode_attention_fused_supported(d, parts, stride, c_longlong(src_stride), _ptr(cos),
                                                             _ptr(sin), c_int(head_dim), c_int(_BF16)))


def decode_attention_fused(out: torch.Tensor, qkv, cos, sin, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, kv_lens: torch.Tensor, n_entries: int, n_heads: int,
                           n_kv: int, head_dim: int, window: int, scale: float, write_kv: bool = True,
                           splits=None, max_keys: int = 0) -> None:
    """One new token per entry: row e of qkv (a tensor or a PartialSum) holds its q, k and v
    heads (q alone if not write_kv).  q and k are rotated at position kv_lens[e] - 1, k and v are
    stored there in the entry's pages, and the token attends to its request's kv_lens[e] keys."""
    _rows_contig(out, "out")
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert kv_lens.dtype == torch.int32 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert qkv.dtype == k_pages.dtype == out.dtype == torch.bfloat16
    page = k_pages.shape[2]
    if splits is None:
        splits = decode_splits(n_entries, n_kv, max_keys or block_table.shape[1] * page)
    lib = load_tensor()
    buf = _attn_partials(out.device, _decode_scratch_floats(n_entries, n_heads, head_dim, splits))
    d, parts, qkv_splits, stride = _split_args(qkv)
    src_stride = qkv.cols if isinstance(qkv, PartialSum) else qkv.stride(0)
    if isinstance(qkv, PartialSum):
        assert qkv.rows == n_entries
    _check_t(lib.llmk_decode_attention_fused(
        _ptr(out), c_longlong(out.stride(0)), d, parts, qkv_splits, stride, c_longlong(src_stride), _ptr(cos),
        _ptr(sin), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), c_int(block_table.shape[1]), _ptr(kv_lens),
        c_int(n_entries), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page), c_int(window or 0),
        c_float(scale), c_int(splits), c_int(int(write_kv)), c_void_p(buf.data_ptr()), c_int(max_keys), _stream()))


def attention_tc_supported(dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention takes these sizes (bfloat16, head size 64 or 128, pages
    of 16 to 128 tokens, at most 128 query heads per kv head)."""
    if dtype != torch.bfloat16:
        return False
    return bool(load_tensor().llmk_attention_tc_supported(c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(page_size)))


def attention_tc(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 block_table: torch.Tensor, cu_tokens: torch.Tensor, kv_lens: torch.Tensor, n_tokens: int,
                 n_entries: int, n_heads: int, n_kv: int, head_dim: int, window: int, scale: float,
                 softcap: float = 0.0, sink: bool = False, keep_first: int = 0, sink_values=None, chunk: int = 0,
                 sigmoid_bias=None, dist_bias=None, v_share: int = 1) -> None:
    """Flash attention on the tensor cores for entries of any length: rows of entry e are
    cu_tokens[e] .. cu_tokens[e+1], its keys (new tokens included) number kv_lens[e].
    softcap, sink, keep_first, sink_values, chunk, sigmoid_bias, dist_bias, v_share: as in paged_attention_generic."""
    r1, r2 = dist_bias if dist_bias is not None else (None, None)
    assert v_share >= 1 and k_pages.shape[1] == n_kv and v_pages.shape[1] * v_share == n_kv
    for t in (sink_values, sigmoid_bias, r1, r2):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n_heads)
    assert sink_values is None or sigmoid_bias is None
    _rows_contig(out, "out"); _rows_contig(q, "q")
    assert q.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert block_table.dim() == 2 and block_table.is_contiguous() and block_table.dtype == torch.int32
    assert cu_tokens.dtype == torch.int32 and kv_lens.dtype == torch.int32
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    _check_t(load_tensor().llmk_attention_tc_ex(
        _ptr(out), c_longlong(out.stride(0)), _ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
        c_int(k_pages.shape[0]), _ptr(block_table), c_int(block_table.shape[1]), _ptr(cu_tokens), _ptr(kv_lens),
        c_int(n_tokens), c_int(n_entries), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_int(k_pages.shape[2]),
        c_int(window or 0), c_float(scale), _stream(), c_float(softcap or 0.0), c_int(int(bool(sink))),
        c_int(keep_first or 0), _ptr(sigmoid_bias if sigmoid_bias is not None else sink_values), c_int(chunk or 0),
        c_int(int(sigmoid_bias is not None)), _ptr(r1), _ptr(r2), c_int(v_share)))


def attention_tc_take_error() -> int:
    """The code the tensor-core attention left when one of its bounded waits gave up (0 = none)."""
    return int(load_tensor().llmk_attention_tc_take_error())


ATTENTION_FAST_OPTIONS = True      # False: the distance bias and shared values always run on the general kernel


def paged_attention(out, qkv, k_pages, v_pages, group, ctx, n_heads: int, n_kv: int, head_dim: int,
                    window: int, scale: float, value_dim: int = 0, softcap: float = 0.0, sink: bool = False,
                    keep_first: int = 0, sink_values=None, chunk: int = 0, sigmoid_bias=None, dist_bias=None,
                    v_share: int = 1) -> None:
    """Attention of the step's tokens over their requests' pages; q is the first
    n_heads * head_dim columns of qkv.  Chooses the kernel for the batch: in bfloat16 the
    split-key decode kernel when every entry brings one token and the tcgen05 kernel otherwise,
    where it takes the sizes; the general kernel for float32 and for all other sizes (head sizes
    off the 16-grid among them).  value_dim, softcap, sink, keep_first: see paged_attention_generic, the kernel
    that takes them in every combination.  sink_values (a learned score per head for the sink), chunk and sigmoid_bias (a
    chunked mask, sigmoid weights): the tcgen05 kernel for steps with prompt portions where it takes the sizes; else the
    split-key decode kernel (sink_values) or the general kernel, whose one warp per (token, head) walks at most one chunk.
    dist_bias (a bias that grows with the logarithm of the distance) and v_share (several key heads over one value head):
    in bfloat16 with values as wide as keys the split-key decode kernel for single tokens and the tcgen05 kernel for steps
    with prompt portions, where they take the sizes; the general kernel otherwise."""
    if dist_bias is not None or v_share > 1:
        same = not value_dim or value_dim == head_dim
        if ATTENTION_FAST_OPTIONS and same and qkv.dtype == torch.bfloat16 and ctx.decode_only and head_dim % 16 == 0 and head_dim <= 256:
            max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
            if window:
                max_keys = min(max_keys, window + keep_first)
            splits = max(1, min(16, 2 * decode_splits(ctx.n_entries, n_kv, max_keys), _ceil_div(max_keys, 32)))
            paged_attention_decode(out, qkv, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries, n_heads, n_kv,
                                   head_dim, window, scale, splits=splits, max_keys=max_keys, softcap=softcap,
                                   sink=sink or sink_values is not None, keep_first=keep_first, sink_values=sink_values,
                                   dist_bias=dist_bias, v_share=v_share)
            return
        if (ATTENTION_FAST_OPTIONS and same and not ctx.decode_only and qkv.stride(0) % 8 == 0
                and attention_tc_supported(qkv.dtype, n_heads, n_kv, head_dim, k_pages.shape[2])):
            attention_tc(out, qkv, k_pages, v_pages, group.block_table, ctx.cu_tokens, ctx.kv_lens, ctx.n_tokens, ctx.n_entries,
                         n_heads, n_kv, head_dim, window, scale, softcap=softcap, sink=sink or sink_values is not None,
                         keep_first=keep_first, sink_values=sink_values, dist_bias=dist_bias, v_share=v_share)
            return
        paged_attention_generic(out, qkv, k_pages, v_pages, group.block_table, ctx.token_entry, ctx.positions,
                                ctx.n_tokens, n_heads, n_kv, head_dim, window, scale, value_dim=value_dim,
                                softcap=softcap, sink=sink or sink_values is not None, keep_first=keep_first,
                                sink_values=sink_values, dist_bias=dist_bias, v_share=v_share)
        return
    if chunk or sigmoid_bias is not None:
        if (not ctx.decode_only and not softcap and (not value_dim or value_dim == head_dim) and qkv.stride(0) % 8 == 0
                and attention_tc_supported(qkv.dtype, n_heads, n_kv, head_dim, k_pages.shape[2])):
            attention_tc(out, qkv, k_pages, v_pages, group.block_table, ctx.cu_tokens, ctx.kv_lens, ctx.n_tokens,
                         ctx.n_entries, n_heads, n_kv, head_dim, 0 if chunk else window, scale, chunk=chunk,
                         sigmoid_bias=sigmoid_bias)
            return
        paged_attention_generic(out, qkv, k_pages, v_pages, group.block_table, ctx.token_entry, ctx.positions,
                                ctx.n_tokens, n_heads, n_kv, head_dim, 0 if chunk else window, scale, value_dim=value_dim,
                                softcap=softcap, chunk=chunk, sigmoid_bias=sigmoid_bias)
        return
    if sink_values is not None:
        sink = True
    extended = bool((value_dim and value_dim != head_dim) or softcap or sink or keep_first)
    if (extended and ctx.decode_only and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and (not value_dim or value_dim == head_dim)):
        # single tokens: the split-key kernel (CUDA cores) takes the soft cap, the sink and the kept keys
        max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
        if window:
            max_keys = min(max_keys, window + keep_first)
        # twice the ranges that the tensor-core decode kernel gets: a round of this kernel (32 keys) takes longer than a
        # tile of that one.  Measured at head size 128, 584 keys: batch 8, 43 -> 32 us a launch; batch 64, a step 2.16 -> 1.70 ms
        splits = max(1, min(16, 2 * decode_splits(ctx.n_entries, n_kv, max_keys), _ceil_div(max_keys, 32)))
        paged_attention_decode(out, qkv, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries,
                               n_heads, n_kv, head_dim, window, scale, splits=splits, max_keys=max_keys,
                               softcap=softcap, sink=sink, keep_first=keep_first, sink_values=sink_values)
        return
    if (extended and (not value_dim or value_dim == head_dim) and qkv.stride(0) % 8 == 0
            and attention_tc_supported(qkv.dtype, n_heads, n_kv, head_dim, k_pages.shape[2])):
        attention_tc(out, qkv, k_pages, v_pages, group.block_table, ctx.cu_tokens, ctx.kv_lens, ctx.n_tokens,
                     ctx.n_entries, n_heads, n_kv, head_dim, window, scale, softcap=softcap, sink=sink, keep_first=keep_first,
                     sink_values=sink_values)
        return
    if extended:
        paged_attention_generic(out, qkv, k_pages, v_pages, group.block_table, ctx.token_entry, ctx.positions,
                                ctx.n_tokens, n_heads, n_kv, head_dim, window, scale, value_dim=value_dim,
                                softcap=softcap, sink=sink, keep_first=keep_first, sink_values=sink_values)
        return
    if ctx.decode_only and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256:
        max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
        if window:
            max_keys = min(max_keys, window)
        paged_attention_decode(out, qkv, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries,
                               n_heads, n_kv, head_dim, window, scale,
                               splits=decode_splits(ctx.n_entries, n_kv, max_keys), max_keys=max_keys)
        return
    if attention_tc_supported(qkv.dtype, n_heads, n_kv, head_dim, k_pages.shape[2]) and qkv.stride(0) % 8 == 0:
        attention_tc(out, qkv, k_pages, v_pages, group.block_table, ctx.cu_tokens, ctx.kv_lens, ctx.n_tokens,
                     ctx.n_entries, n_heads, n_kv, head_dim, window, scale)
        return
    paged_attention_generic(out, qkv, k_pages, v_pages, group.block_table, ctx.token_entry, ctx.positions,
                            ctx.n_tokens, n_heads, n_kv, head_dim, window, scale)


FUSE_DECODE_ATTENTION = True


def rope_store_attend(out, qkv, cos, sin, k_pages, v_pages, group, ctx, n_heads: int, n_kv: int, head_dim: int,
                      window: int, scale: float, write_kv: bool, q_rot) -> None:
    """The three steps between the QKV product and the output projection: rotate q and k by the
    tables, store k and v in the pages (if write_kv), attend.  qkv is a tensor or a PartialSum;
    q_rot() gives a buffer for rotated queries when they cannot stay where they are.  A decode
    step in bfloat16 with a head size of 64 or 128 runs as one kernel, everything else as the
    rotate-and-store kernel followed by the attention kernel that fits the batch."""
    if (FUSE_DECODE_ATTENTION and ctx.decode_only and ctx.n_tokens == ctx.n_entries
            and decode_attention_fused_supported(qkv, cos, sin, head_dim, k_pages.shape[2])):
        max_keys = min(ctx.kv_bucket or 1 << 30, group.block_table.shape[1] * k_pages.shape[2])
        if window:
            max_keys = min(max_keys, window)
        decode_attention_fused(out, qkv, cos, sin, k_pages, v_pages, group.block_table, ctx.kv_lens, ctx.n_entries,
                               n_heads, n_kv, head_dim, window, scale, write_kv=write_kv,
                               splits=decode_splits(ctx.n_entries, n_kv, max_keys), max_keys=max_keys)
        return
    q = rope_kv_write(qkv, cos, sin, ctx.positions, group.slot_map, k_pages, v_pages, ctx.n_tokens, n_heads,
                      n_kv if write_kv else 0, head_dim, q_out=q_rot() if isinstance(qkv, PartialSum) else None)
    paged_attention(out, q, k_pages, v_pages, group, ctx, n_heads, n_kv, head_dim, window, scale)


# ---- tensor-core product ------------------------------------------------------------

_PARTIALS = {}      # device -> float32 scratch for split-K partial sums
_PARTIAL_BYTES = 64 << 20


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@functools.lru_cache(maxsize=None)
def sm_count() -> int:
    """Streaming multiprocessors of the current device (the planners size grids and rounds by it)."""
    return max(1, int(load().llmk_device_sm_count()))


PERSISTENT_GEMM = True
PAIR_GEMM = True


def plan_gemm(M: int, N: int, K: int, fused_reduce: bool = False, cta_limit: int = 0):
    """cta_limit > 0 (swapped mode only): at most so many CTAs, for a product that should leave
    SMs to the kernel after it."""
    return _plan_gemm(M, N, K, fused_reduce, PERSISTENT_GEMM, PAIR_GEMM, sm_count(), cta_limit)


@functools.lru_cache(maxsize=4096)
def _plan_gemm(M: int, N: int, K: int, fused_reduce: bool, persistent: bool, pair: bool = False, _SMS: int = 148,
               cta_limit: int = 0):
    """(swap, tile, splits, k-blocks per split, mode) for the tensor-core product; mode 0 = one
    CTA per tile, 1 = the splits of a tile sum on chip in a cluster, 2 = persistent CTAs, 3 =
    persistent pairs of CTAs on tiles of 256 rows.

    Up to 128 rows the weights take the 128-row side of the MMA and the rows become its N
    (16 to 128); above that the rows take the 128-row side and the tile is 128 or 256 weight
    rows wide.  K (in blocks of 64) is split over CTAs when there are too few tiles to keep
    all SMs streaming; where the shape allows it the splits of a tile form a cluster and sum
    their results in shared memory, else they write float32 partial results for a later sum.
    The estimate, in microseconds, for more than 128 rows: a fixed cost plus waves of tiles times
    k-blocks times a k-block's time, fitted to timings of the products of the 1.1B and 7B shapes
    at 129 to 4,096 rows; plus the sum of the partial results where K is split."""
    kb = _ceil_div(K, 64)
    if M < NORMAL_MODE_FROM_ROWS:
        return _plan_swapped(M, N, kb, fused_reduce, _SMS, cta_limit)
    if M <= 128:
        return _plan_few_rows(M, N, kb, fused_reduce, _SMS, cta_limit)
    best = None
    for tile in (256, 224, 192, 160, 128):
        tiles = _ceil_div(M, 128) * _ceil_div(N, tile)
        # us per k-block of one CTA: bound by the bytes that it brings into shared memory
        t_kb = (128 + tile) * 128 / 114e3
        for s in range(1, min(kb, 32) + 1):
            per = _ceil_div(kb, s)
            if _ceil_div(kb, per) != s:
                continue
            if s > 1 and s * M * N * 4 > _PARTIAL_BYTES:
                break
            mode = 0
            waves = _ceil_div(tiles * s, _SMS)
            cost = waves * (per * t_kb + 0.8) + 7.2
            if persistent and s == 1 and tiles > _SMS:
                # more than one wave of tiles: one CTA per SM walks over them and drains one
                # accumulator while the next tile's products run
                mode = 2
                cost = waves * per * t_kb + 12.3
            if s > 1:
                traffic = (2 * s + 1) * M * N * 4 / 3.3e6             # partials written and read back, us
                cost += traffic + (0.8 if fused_reduce else 3.3)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, False, tile, s, per, mode)
        if pair:
            # pairs of CTAs on tiles of 256 rows bring a third fewer bytes into shared memory per
            # product: a k-block takes what its MMAs take (with the gaps measured) or, on narrow
            # tiles, the latency of the ring
            t_kb = max(0.31 + 0.0004 * (tile - 128), 1.43 * 256 * tile * 64 * 2 / 2 / 15.2e6)
            waves = _ceil_div(_ceil_div(M, 256) * _ceil_div(N, tile), _SMS // 2)
            cost = waves * kb * t_kb + 8.6
            if cost < best[0] - 1e-9:
                best = (cost, False, tile, 1, kb, 3)
    return best[1:]


# From this many rows on (up to 128) the rows take the 128-row side of the MMA like a prompt's, one
# CTA per tile of 128 weight rows with the SM and a ring of 192 KB to itself, instead of the
# swapped mode's two CTAs per SM with rings half that size.  Measured on the four products of the
# 1.1B shape with the kernel that sums the partial results behind them (us, swapped -> normal):
# 32 rows 9.2 -> 8.5, 7.5 -> 6.7, 15.0 -> 10.6, 9.5 -> 10.2; 64 rows 11.4 -> 9.8, 9.3 -> 7.7, 17.9 ->
# 11.1, 11.6 -> 11.0; 128 rows 15.2 -> 10.7, 13.2 -> 9.1, 27.5 -> 11.8, 16.1 -> 12.6; at 16 rows and
# fewer the swapped mode is ahead (7.9 against 8.2, 8.0 against 10.0).  Whole decode steps: 24 requests
# 1.066 -> 1.055 ms, 31 requests 1.099 -> 1.087 ms, 64 requests 1.31 -> 1.20 ms; 17 requests the same.
NORMAL_MODE_FROM_ROWS = 24


def _plan_few_rows(M: int, N: int, kb: int, fused_reduce: bool, _SMS: int, cta_limit: int = 0):
    """The normal mode for 32 to 128 rows: tiles of 128 or 256 weight rows, one per CTA, K split
    over CTAs while there are too few tiles to draw the memory's bandwidth.  The estimate, in
    microseconds: a CTA's ring holds 192 KB in flight against a latency of about 1.5 us, of which
    the weights are a half (tiles of 128) or two thirds (of 256); the CTAs of a round share the
    measured 6.5 TB/s; a round costs a microsecond beside its bytes, the launch 1.6; partial
    results are written and read back where K is split.  Checked against timings of the products
    of the 1.1B, 7B and 8B shapes at 32, 64 and 128 rows."""
    best = None
    for tile in (128, 256):
        tiles = _ceil_div(N, tile)
        per_cta = 0.128e6 * tile / (128 + tile)                   # bytes of weights per microsecond that one CTA can draw
        for s in range(1, min(kb, 16) + 1):
            per = _ceil_div(kb, s)
            if _ceil_div(kb, per) != s:
                continue
            if s > 1 and (s * M * N * 4 > _PARTIAL_BYTES or (cta_limit and tiles * s > cta_limit)):
                break
            cta_bytes, left, cost = tile * per * 128, tiles * s, 1.6
            while left > 0:
                r = min(left, _SMS)
                cost += cta_bytes * r / min(6.5e6, r * per_cta) + 1.0
                left -= r
            if s > 1:
                cost += 2 * s * M * N * 4 / 7e6 + (0.5 * _ceil_div(s, 4) if fused_reduce else 3.0)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, False, tile, s, per, 0)
    return best[1:]


_SWAPPED_STAGES = {16: 6, 32: 5, 64: 4, 128: 3}      # as stages_for() in gemm_tc.cu


def _plan_swapped(M: int, N: int, kb: int, fused_reduce: bool, _SMS: int, cta_limit: int = 0):
    """The swapped mode (up to 128 rows): a stream of weights.  Two CTAs share an SM, so up to 296
    run at a time.  A CTA alone is bound by what its ring keeps in flight (stages x stage bytes per
    memory latency of about 2 us), the CTAs of one SM by its way to L2, all CTAs together by HBM;
    the constants were fitted to timings of the five products of the 1.1B shape at 16, 32, 64 and
    128 rows (the plans picked this way are within 1 % of the best measured ones in sum).  On-chip sums through a cluster measured
    slower at decode sizes than partial results plus a summing consumer (a cluster needs all its
    CTAs scheduled at once, which takes away the early start of the next product's weight loads);
    they stay an option of gemm_fast."""
    tile = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = _ceil_div(N, 128)
    stage_bytes = (128 + tile) * 128
    t_mma = 128 * tile * 64 * 2 / 15.2e6
    best = None
    for s in range(1, min(kb, 32) + 1):
        per = _ceil_div(kb, s)
        if _ceil_div(kb, per) != s:
            continue
        if s > 1 and s * M * N * 4 > _PARTIAL_BYTES:
            break
        n_cta = tiles * s
        if cta_limit and s > 1 and n_cta > cta_limit:
            break
        rounds = _ceil_div(n_cta, 2 * _SMS)
        conc = n_cta if rounds == 1 else 2 * _SMS
        per_sm = min(2, _ceil_div(n_cta, _SMS))           # CTAs on the fullest SM: they share its tensor pipe and its way to L2
        t_kb = max(t_mma * per_sm, 2.3 / _SWAPPED_STAGES[tile], stage_bytes * conc / 8.0e6, stage_bytes * per_sm / 80e3)
        cost = rounds * per * t_kb + 1.8
        if s > 1:
            cost += s * M * N * 4 / 7e6                   # partial results written
            # and summed: by their consumer (four splits' loads in flight at a time, so every
            # further four splits cost it another trip to L2), or by a kernel of their own
            cost += 0.5 * _ceil_div(s, 4) + s * M * N * 4 / 7e6 if fused_reduce else 3.0
        if best is None or cost < best[0] - 1e-9:
            best = (cost, True, tile, s, per, 0)
    return best[1:]


def _partials(device) -> torch.Tensor:
    buf = _PARTIALS.get(device)
    if buf is None:
        buf = torch.empty(_PARTIAL_BYTES // 4, dtype=torch.float32, device=device)
        _PARTIALS[device] = buf
    return buf


def gemm_fast_available(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """Whether the tcgen05 product takes this problem (bfloat16, rows of 16-byte multiples)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    # the conditions of llmk_gemm_tc_supported, checked here: this runs before every product of a
    # step that is not replayed from a graph, and a call into the library costs microseconds
    n, k = w.shape
    return (rows > 0 and n > 0 and k > 0 and k % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and a.is_cuda and w.is_cuda)


def gemm_fast(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, plan=None, allow_partial: bool = False,
              cta_limit: int = 0):
    """out[:rows] = a[:rows] @ w.T on the tensor cores (bfloat16 in, float32 accumulation).
    Returns out; or, with allow_partial and a split-K plan, a PartialSum that the caller hands to
    a kernel that sums it (out is then not written).  cta_limit: see plan_gemm."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n
    plan = plan or plan_gemm(rows, n, k, fused_reduce=allow_partial, cta_limit=cta_limit)
    swap, tile, splits, per = plan[:4]
    cluster = int(plan[4]) if len(plan) > 4 else 0
    lib = load_tensor()
    if splits == 1 or cluster:
        _check_t(lib.llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                                c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                c_int(_kind(out.dtype)), c_int(int(swap)), c_int(tile), c_int(splits), c_int(per),
                                c_int(int(cluster)), c_int(0), _stream()))
        return out
    part = _partials(a.device)
    _check_t(lib.llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(part), c_int(rows), c_int(n), c_int(k),
                            c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(n), c_int(_F32),
                            c_int(int(swap)), c_int(tile), c_int(splits), c_int(per), c_int(0), c_int(0), _stream()))
    if allow_partial:
        return PartialSum(part, splits, rows, n, out.dtype)
    assert out.is_contiguous()
    _check_t(lib.llmk_reduce_partials(_ptr(out), _ptr(part), c_longlong(rows * n), c_int(splits),
                                    c_int(_kind(out.dtype)), _stream()))
    return out


def gemm_swiglu_available(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """Whether gemm_swiglu takes this problem: bfloat16 throughout, more rows than the swapped
    mode serves (there K is split over CTAs and the activation kernel sums the splits), an even
    number of weight rows."""
    return (rows > 128 and out.dtype == torch.bfloat16 and w.shape[0] % 16 == 0
            and gemm_fast_available(a, w, out, rows))


def gemm_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, act: str = "silu") -> None:
    """out[:rows] = silu(a @ gate.T) * (a @ up.T) for w = [gate; up] stacked along its rows
    ([2I, K]), out [rows, I] bfloat16.  One persistent tensor-core kernel: each tile multiplies by
    128 gate rows and their 128 up rows and applies the activation in its epilogue, so the
    product never reaches memory.  act "relu": relu(gate) * up (the kernel on pairs of CTAs only)."""
    assert act == "silu" or (act == "relu" and PAIR_GEMM)
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n // 2 and n % 2 == 0
    if not gemm_swiglu_available(a, w, out, rows):
        raise KernelError(f"gemm_swiglu does not take {rows} rows of {a.dtype} -> {out.dtype}")
    _check_t(load_tensor().llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                               c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                               c_int(_BF16), c_int(0), c_int(256), c_int(1), c_int(_ceil_div(k, 64)),
                               c_int(3 if PAIR_GEMM else 2), c_int(-1 if act == "relu" else 1), _stream()))


def gemm_act_available(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int) -> bool:
    """Whether gemm_act takes this problem: bfloat16 throughout and more rows than the few-row modes serve
    (there K is split over CTAs and the activation kernel sums the splits)."""
    return PAIR_GEMM and rows > 128 and out.dtype == torch.bfloat16 and gemm_fast_available(a, w, out, rows)


def gemm_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, rows: int, act: str) -> None:
    """out[:rows] = act(a[:rows] @ w.T) with the activation applied to the float32 accumulator in the epilogue of
    the pair kernel, so the product itself never reaches memory."""
    _rows_contig(a, "a"); _rows_contig(w, "w"); _rows_contig(out, "out")
    n, k = w.shape
    assert a.shape[1] == k and out.shape[1] == n
    if not gemm_act_available(a, w, out, rows):
        raise KernelError(f"gemm_act does not take {rows} rows of {a.dtype} -> {out.dtype}")
    tile = 256 if n % 256 == 0 or n % 256 > 128 or n < 128 else 128
    tile = min(tile, _ceil_div(n, 32) * 32)
    _check_t(load_tensor().llmk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(rows), c_int(n), c_int(k),
                               c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                               c_int(_BF16), c_int(0), c_int(tile), c_int(1), c_int(_ceil_div(k, 64)),
                               c_int(3), c_int(2 + ACTIVATIONS[act]), _stream()))


FUSE_PROMPT_ROPE = True


def _qkv_rope_tile(rows: int, n: int, k: int, head_dim: int) -> int:
    """The tile width (whole heads, up to 256 columns) with the fewest rounds of pair tiles, by
    the pair kernel's terms of plan_gemm."""
    best = None
    _SMS = sm_count()
    for tile in range(head_dim, 257, head_dim):
        t_kb = max(0.31 + 0.0004 * (tile - 128), 1.43 * 256 * tile * 64 * 2 / 2 / 15.2e6)
        cost = _ceil_div(_ceil_div(rows, 256) * _ceil_div(n, tile), _SMS // 2) * t_kb
        if best is None or cost < best[0] - 1e-9:
            best = (cost, tile)
    return best[1]


def qkv_rope_store(x: torch.Tensor, w: torch.Tensor, q_out, rows: int, cos, sin, positions: torch.Tensor,
                   slot_map: torch.Tensor, k_pages, v_pages, n_heads: int, n_kv: int, head_dim: int):
    """The QKV projection of a prompt portion with rotation and cache store in its epilogue:
    x[:rows] @ w.T for w = [q heads; k heads; v heads] (n_kv of each; 0: query heads only), the
    query and key heads rotated by the tables at positions[t], queries written to q_out() [rows,
    n_heads * head_dim], keys and values to place slot_map[t] of the pages.  Returns the tensor
    of the queries; or None, having done nothing, where the kernel does not apply (float32, up to
    128 rows, whose product splits K instead, a head size other than 64 or 128): the caller then
    runs the product and rope_kv_write."""
    if (not FUSE_PROMPT_ROPE or not PAIR_GEMM or rows <= 128 or x.dtype != torch.bfloat16
            or w.dtype != torch.bfloat16 or head_dim not in (64, 128)):
        return None
    n, k = w.shape
    if n != (n_heads + 2 * n_kv) * head_dim:
        return None
    if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[1] != head_dim // 2
                            or not cos.is_contiguous() or not sin.is_contiguous()):
        return None
    if n_kv and not (k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == torch.bfloat16
                     and k_pages.shape[1] == n_kv and k_pages.shape[3] == head_dim):
        return None
    lib = load_tensor()
    q = q_out()
    _rows_contig(x, "x"); _rows_contig(w, "w"); _rows_contig(q, "q_out")
    assert q.dtype == torch.bfloat16 and positions.dtype == torch.int32 and slot_map.dtype == torch.int32
    args = (_ptr(x), _ptr(w), c_int(rows), c_int(n), c_int(k), c_longlong(x.stride(0)), c_longlong(w.stride(0)))
    if not lib.llmk_gemm_tc_qkv_rope_supported(*args, _ptr(q), c_longlong(q.stride(0)), _ptr(cos), _ptr(sin),
                                               _ptr(k_pages) if n_kv else c_void_p(0),
                                               _ptr(v_pages) if n_kv else c_void_p(0), c_int(n_heads), c_int(n_kv),
                                               c_int(head_dim)):
        return None
    _check_t(lib.llmk_gemm_tc_qkv_rope(_ptr(x), _ptr(w), _ptr(q), c_int(rows), c_int(n), c_int(k),
                                       c_longlong(x.stride(0)), c_longlong(w.stride(0)), c_longlong(q.stride(0)),
                                       c_int(_qkv_rope_tile(rows, n, k, head_dim)), _ptr(cos), _ptr(sin),
                                       _ptr(positions), _ptr(slot_map), _ptr(k_pages) if n_kv else c_void_p(0),
                                       _ptr(v_pages) if n_kv else c_void_p(0), c_int(n_heads), c_int(n_kv),
                                       c_int(head_dim), c_int(k_pages.shape[2] if n_kv else 1), _stream()))
    return q


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch between the kernels of a step (on by default); set in both
    kernel libraries."""
    load().llmk_set_pdl(c_int(int(on)))
    load_tensor().llmk_set_pdl(c_int(int(on)))


def set_error_block(block) -> None:
    """Point the tensor-core kernels' error words at `block` (int32 [4] on the device: word 1 is
    the product's, word 2 the attention's), or back at the library's own words with None."""
    if block is not None:
        assert block.dtype == torch.int32 and block.numel() >= 4 and block.is_contiguous()
    load_tensor().llmk_set_error_block(_ptr(block))


_WAIT_NAMES = {1: "TMA producer", 2: "MMA issuer", 0: "epilogue"}
_ATTN_WAITS = {11: "the query tile", 12: "a key/value tile", 13: "the scores", 14: "the probabilities",
               15: "the output product", 16: "tile alignment"}


def describe_wait(word: int, code: int) -> str:
    """What a code in an error word (1: tensor-core product, 2: tensor-core attention) stands for."""
    if word == 1:
        kernel = {0: "one-tile", 1: "persistent", 2: "pair"}.get((code - 1) // 3, "unknown")
        return f"the tensor-core product ({kernel} kernel): its {_WAIT_NAMES[code % 3]} gave up a bounded wait (code {code})"
    if word == 2:
        return f"the tensor-core attention gave up a bounded wait for {_ATTN_WAITS.get(code, 'code ' + str(code))} (code {code})"
    return f"error word {word}: code {code}"


def gemm_tc_take_error() -> int:
    """The code a tensor-core kernel left when one of its bounded waits gave up (0 = none)."""
    return int(load_tensor().llmk_gemm_tc_take_error())
