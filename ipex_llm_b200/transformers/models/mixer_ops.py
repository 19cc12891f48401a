"""Host side of the mixer kernels (ggml/model/mixers_cpp.py -> libb200mixers.so): argument checks, output allocation, one
native call each.  Every function takes CUDA tensors; the shapes are those of include/b200_mixers.h.

Conventions: ``x`` is the 32-bit residual stream [N, W] (N = batch * new tokens); projections are [B, S, P] tensors of the
model's dtype whose columns hold several quantities side by side (``off_*`` = first column of one); ``slot0`` numbers the
first new token's slot and ``pad`` [B] int32 is the rows' left padding."""
import torch

from ipex_llm_b200.ggml.model import mixers_cpp as native
from ipex_llm_b200.utils.common import invalidInputError


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


def embed_rows(table, ids):
    """fp32 [N, W] rows of the embedding table"""
    table, ids = _c(table), _c(ids.to(torch.int64))
    x = torch.empty(ids.numel(), table.shape[1], dtype=torch.float32, device=table.device)
    native.call("mixers_embed_rows", native.dtype_code(table.dtype), native.ptr(table), native.ptr(ids), ids.numel(), table.shape[1],
                native.ptr(x), native.stream(x.device))
    return x


def dyt_residual_norm(x, pending, add, pre, out_dtype):
    """x += DyT_post(y) for ``pending`` = (y, post norm module); x += add; returns DyT_pre(x) in ``out_dtype`` (None without
    ``pre``).  One launch; x is updated in place."""
    invalidInputError(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "the residual stream is a contiguous fp32 [N, W]")
    n, w = x.shape
    y, post = pending if pending is not None else (None, None)
    if y is not None:
        y = _c(y)
        invalidInputError(y.shape == x.shape and y.dtype == out_dtype, "sublayer output must match the residual's shape and the model's dtype")
    out = torch.empty(n, w, dtype=out_dtype, device=x.device) if pre is not None else None
    for mod in (post, pre):
        if mod is not None:
            invalidInputError(mod.weight.dtype == out_dtype, "normalisation parameters must have the model's dtype")
    native.call("mixers_dyt_residual_norm", native.dtype_code(out_dtype), native.ptr(x), n, w, native.ptr(y),
                native.ptr(post.weight) if post is not None else None, native.ptr(post.bias) if post is not None else None,
                native.ptr(post.alpha) if post is not None else None, native.ptr(_c(add)) if add is not None else None,
                native.ptr(pre.weight) if pre is not None else None, native.ptr(pre.bias) if pre is not None else None,
                native.ptr(pre.alpha) if pre is not None else None, native.ptr(out), native.stream(x.device))
    return out


def window_qk_prepare(proj, off_q, off_k, off_v, heads, kv_heads, dim, vdim, q_w, k_w, eps, inv_freq, rot_dims, k_store, v_store,
                      cap, held, shift, pad, dyn=None, q=None):
    """norm + rotary of the new tokens' queries and keys, cache write of keys and values; returns q fp32 [B, S, heads, dim]"""
    B, S, P = proj.shape
    invalidInputError(proj.is_contiguous() and k_store.is_contiguous() and v_store.is_contiguous() and k_store.shape[2] == cap
                      and v_store.shape[2] == cap
                      and k_store.dtype == proj.dtype and v_store.dtype == proj.dtype and inv_freq.dtype == torch.float64,
                      "window_qk_prepare: unexpected layout")
    if q is None:
        q = torch.empty(B, S, heads, dim, dtype=torch.float32, device=proj.device)
    native.call("mixers_window_qk_prepare", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, off_q, off_k, off_v, heads, kv_heads,
                dim, vdim, native.ptr(q_w), native.ptr(k_w), float(eps), native.ptr(inv_freq), rot_dims, native.ptr(q), native.ptr(k_store),
                native.ptr(v_store), cap, held, shift, native.ptr(pad), native.ptr(dyn), native.stream(proj.device))
    return q


def sigmoid_window_attention(q, k_store, v_store, cap, held, shift, pad, window, scale, head_bias, out, out_col, out_scale, dyn=None):
    """out[:, out_col : out_col + heads * vdim] = out_scale * attention of the new tokens (see the header)"""
    B, S, heads, dim = q.shape
    kv_heads, vdim = k_store.shape[1], v_store.shape[3]
    invalidInputError(out.is_contiguous() and out.shape[0] == B * S and out.dtype == k_store.dtype and k_store.is_contiguous()
                      and v_store.is_contiguous() and k_store.shape[2] == cap and v_store.shape[2] == cap,
                      "sigmoid_window_attention: unexpected layout")
    native.call("mixers_sigmoid_window_attention", native.dtype_code(out.dtype), native.ptr(q), native.ptr(k_store), native.ptr(v_store), B, S,
                heads, kv_heads, dim, vdim, cap, held, shift, native.ptr(pad), int(window), float(scale), native.ptr(head_bias), native.ptr(out),
                out.shape[1], out_col, float(out_scale), native.ptr(dyn), native.stream(out.device))


def short_conv_silu(proj, off, channels, weight, tail, tail_next, slot0, pad):
    """silu(short causal convolution) of ``channels`` columns of proj from column ``off``; writes the next tail"""
    B, S, P = proj.shape
    taps = weight.shape[1]
    invalidInputError(proj.is_contiguous() and weight.is_contiguous() and tail.is_contiguous() and tail_next.is_contiguous()
                      and weight.shape[0] == channels and tail.shape == (B, max(taps - 1, 1), channels), "short_conv_silu: unexpected layout")
    y = torch.empty(B, S, channels, dtype=proj.dtype, device=proj.device)
    native.call("mixers_short_conv_silu", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, off, channels, taps, native.ptr(weight),
                native.ptr(tail), native.ptr(tail_next), slot0, native.ptr(pad), native.ptr(y), native.stream(proj.device))
    return y


def short_conv(proj, off, channels, weight, bias, tail, tail_next, slot0, pad, silu=True, add_input=False):
    """short causal convolution of ``channels`` columns of proj from column ``off`` with an optional bias per channel, silu on
    the result (``silu``) and / or the token's own input added to it (``add_input``); writes the next tail"""
    B, S, P = proj.shape
    taps = weight.shape[1]
    invalidInputError(proj.is_contiguous() and weight.is_contiguous() and tail.is_contiguous() and tail_next.is_contiguous()
                      and weight.shape[0] == channels and tail.shape == (B, max(taps - 1, 1), channels)
                      and (bias is None or (bias.numel() == channels and bias.is_contiguous())), "short_conv: unexpected layout")
    y = torch.empty(B, S, channels, dtype=proj.dtype, device=proj.device)
    native.call("mixers_short_conv", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, off, channels, taps, native.ptr(weight),
                native.ptr(bias), int(bool(silu)) | (int(bool(add_input)) << 1), native.ptr(tail), native.ptr(tail_next), int(slot0),
                native.ptr(pad), native.ptr(y), native.stream(proj.device))
    return y


def channel_delta_rule(conv, kv_heads, heads, dim, vdim, proj, off_b, z, A_log, dt_bias, state, slot0, pad):
    """the delta rule with a decay per key channel over the new tokens (conv: q | k | v after the short convolutions; beta from
    column off_b of proj; z [B, S, heads * dim] decay logits, dt_bias [heads * dim], A_log [heads]); state fp32
    [B, heads, dim, vdim] in place; returns o fp32 [B, S, heads, vdim]"""
    B, S, C = conv.shape
    invalidInputError(C == 2 * kv_heads * dim + heads * vdim and conv.is_contiguous() and proj.is_contiguous() and z.is_contiguous()
                      and z.numel() == B * S * heads * dim and z.dtype == conv.dtype and dt_bias.numel() == heads * dim
                      and dt_bias.is_contiguous() and A_log.numel() == heads
                      and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (B, heads, dim, vdim),
                      "channel_delta_rule: unexpected layout")
    o = torch.empty(B, S, heads, vdim, dtype=torch.float32, device=conv.device)
    native.call("mixers_channel_delta_rule", native.dtype_code(conv.dtype), native.ptr(conv), B, S, kv_heads, heads, dim, vdim, native.ptr(proj),
                proj.shape[-1], off_b, native.ptr(z), native.ptr(A_log), native.ptr(dt_bias), native.ptr(state), int(slot0), native.ptr(pad),
                native.ptr(o), native.stream(conv.device))
    return o


def state_space_scan(conv, groups, heads, n_state, vdim, proj, off_dt, A_log, dt_bias, skip, state, slot0, pad):
    """the state-space recurrence over the new tokens (conv: x | B | C after the short convolution; the step-size logits from
    column off_dt of proj); state fp32 [B, heads, n_state, vdim] in place; returns y fp32 [B, S, heads, vdim]"""
    B, S, C = conv.shape
    invalidInputError(C == heads * vdim + 2 * groups * n_state and conv.is_contiguous() and proj.is_contiguous()
                      and A_log.numel() == heads and dt_bias.numel() == heads and skip.numel() == heads
                      and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (B, heads, n_state, vdim),
                      "state_space_scan: unexpected layout")
    o = torch.empty(B, S, heads, vdim, dtype=torch.float32, device=conv.device)
    native.call("mixers_state_space_scan", native.dtype_code(conv.dtype), native.ptr(conv), B, S, groups, heads, n_state, vdim, native.ptr(proj),
                proj.shape[-1], off_dt, native.ptr(A_log), native.ptr(dt_bias), native.ptr(skip), native.ptr(state), int(slot0),
                native.ptr(pad), native.ptr(o), native.stream(conv.device))
    return o


def gated_delta_rule(conv, kv_heads, heads, dim, vdim, proj, off_b, off_a, A_log, dt_bias, state, slot0, pad):
    """the delta-rule recurrence over the new tokens; state fp32 [B, heads, dim, vdim] in place; returns o fp32 [B, S, heads, vdim]"""
    B, S, C = conv.shape
    invalidInputError(C == 2 * kv_heads * dim + heads * vdim and conv.is_contiguous() and proj.is_contiguous()
                      and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (B, heads, dim, vdim),
                      "gated_delta_rule: unexpected layout")
    o = torch.empty(B, S, heads, vdim, dtype=torch.float32, device=conv.device)
    native.call("mixers_gated_delta_rule", native.dtype_code(conv.dtype), native.ptr(conv), B, S, kv_heads, heads, dim, vdim, native.ptr(proj),
                proj.shape[-1], off_b, off_a, native.ptr(A_log), native.ptr(dt_bias), native.ptr(state), slot0, native.ptr(pad), native.ptr(o),
                native.stream(conv.device))
    return o


def gated_linear_attention(proj, heads, dim, vdim, z, tau, state, slot0, pad):
    """gated linear attention over the new tokens (q | k | v in the first columns of proj, decay logits z)"""
    B, S, P = proj.shape
    invalidInputError(proj.is_contiguous() and z.is_contiguous() and z.shape == (B, S, heads * dim) and z.dtype == proj.dtype
                      and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (B, heads, dim, vdim),
                      "gated_linear_attention: unexpected layout")
    o = torch.empty(B, S, heads, vdim, dtype=torch.float32, device=proj.device)
    native.call("mixers_gated_linear_attention", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, heads, dim, vdim, native.ptr(z),
                float(tau), native.ptr(state), slot0, native.ptr(pad), native.ptr(o), native.stream(proj.device))
    return o


def gated_rms_norm(o, gate, off_g, weight, eps, out, out_col, out_scale, sigmoid=False, gate_first=False):
    """out[:, out_col:...] = out_scale * rms_norm(o per head) * weight * silu(gate columns from off_g); ``weight`` [vdim] serves
    every head, [heads * vdim] gives each head its own.  ``sigmoid``: the gate is sigmoid(.) instead of silu(.); ``gate_first``:
    the gate multiplies before the norm (the root mean square is that of the gated values)"""
    heads, vdim = o.shape[-2], o.shape[-1]
    n = o.numel() // (heads * vdim)
    invalidInputError(o.is_contiguous() and o.dtype == torch.float32 and gate.is_contiguous() and out.is_contiguous() and out.shape[0] == n
                      and gate.dtype == out.dtype and weight.numel() in (vdim, heads * vdim), "gated_rms_norm: unexpected layout")
    native.call("mixers_gated_rms_norm", native.dtype_code(out.dtype), native.ptr(o), n, heads, vdim, native.ptr(gate), gate.shape[-1], off_g,
                native.ptr(weight), vdim if weight.numel() == heads * vdim and heads > 1 else 0, float(eps), native.ptr(out), out.shape[1], out_col,
                float(out_scale), int(bool(sigmoid)) | (int(bool(gate_first)) << 1), native.stream(out.device))


def token_shift_mix(h, mu, tail, tail_next, slot0, pad):
    """[n_mix, B * S, C]: h + (previous h - h) * mu[m] for every mixing vector; ``tail`` [B, 1, C] holds the token before the
    call's first one, ``tail_next`` receives the call's last one"""
    B, S, C = h.shape
    invalidInputError(h.is_contiguous() and mu.is_contiguous() and mu.shape[1] == C and mu.dtype == h.dtype and tail.shape == (B, 1, C)
                      and tail.dtype == h.dtype and tail.is_contiguous() and tail_next.is_contiguous(), "token_shift_mix: unexpected layout")
    out = torch.empty(mu.shape[0], B * S, C, dtype=h.dtype, device=h.device)
    native.call("mixers_token_shift_mix", native.dtype_code(h.dtype), native.ptr(h), B, S, C, native.ptr(mu), mu.shape[0], native.ptr(tail),
                native.ptr(tail_next), int(slot0), native.ptr(pad), native.ptr(out), native.stream(h.device))
    return out


def wkv(r, k, v, B, S, heads, dim, z, w0, u, state, slot0, pad):
    """the RWKV-style recurrence over the new tokens; r, k, v [B * S, heads * dim] views with one row stride (parts of one
    buffer), z [B * S, heads * dim] decay logits; state fp32 [B, heads, dim, dim] in place; returns o fp32 [B, S, heads, dim]"""
    ld = r.stride(0)
    invalidInputError(k.stride(0) == ld and v.stride(0) == ld and r.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
                      and r.dtype == k.dtype == v.dtype == z.dtype and z.is_contiguous() and z.shape == (B * S, heads * dim)
                      and w0.numel() == heads * dim and u.numel() == heads * dim and w0.is_contiguous() and u.is_contiguous()
                      and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (B, heads, dim, dim),
                      "wkv: unexpected layout")
    o = torch.empty(B, S, heads, dim, dtype=torch.float32, device=r.device)
    native.call("mixers_wkv", native.dtype_code(r.dtype), native.ptr(r), native.ptr(k), native.ptr(v), B, S, ld, heads, dim, native.ptr(z),
                native.ptr(w0), native.ptr(u), native.ptr(state), int(slot0), native.ptr(pad), native.ptr(o), native.stream(r.device))
    return o


def layer_norm_residual(x, y_a, y_b, weight, eps, out_dtype, want_out=True):
    """x += y_a + y_b in place (x fp32 [N, W]; y_a in the model's dtype, y_b fp32, either may be None); returns the layer norm
    (weight only) of the new x in ``out_dtype``, or None without ``want_out``"""
    n, w = x.shape
    invalidInputError(x.dtype == torch.float32 and x.is_contiguous() and (y_a is None or (y_a.shape == x.shape and y_a.dtype == out_dtype and y_a.is_contiguous()))
                      and (y_b is None or (y_b.shape == x.shape and y_b.dtype == torch.float32 and y_b.is_contiguous())),
                      "layer_norm_residual: x a contiguous fp32 [N, W], y_a the model's dtype, y_b fp32")
    out = torch.empty(n, w, dtype=out_dtype, device=x.device) if want_out else None
    native.call("mixers_layer_norm_residual", native.dtype_code(out_dtype), native.ptr(x), n, w, native.ptr(y_a), native.ptr(y_b),
                native.ptr(weight) if want_out else None, float(eps), native.ptr(out), native.stream(x.device))
    return out


def wide_qkv_prepare(proj, off_q, off_k, off_v, heads, kv_heads, dim, vdim, q_w, k_w, eps, v_other, blend, k_store, v_store, cap, held, shift,
                     pad, dyn=None):
    """RMS norm over the whole query and the whole key projection of every new token, values blended with ``v_other`` (a
    [B * S, kv_heads * vdim] view with unit column stride, or None), cache write of keys and values; returns q [B * S, heads * dim]"""
    B, S, P = proj.shape
    invalidInputError(proj.is_contiguous() and k_store.is_contiguous() and v_store.is_contiguous() and k_store.shape[2] == cap
                      and v_store.shape[2] == cap and k_store.dtype == proj.dtype and v_store.dtype == proj.dtype
                      and (v_other is None or (v_other.stride(1) == 1 and v_other.shape == (B * S, kv_heads * vdim) and v_other.dtype == proj.dtype)),
                      "wide_qkv_prepare: unexpected layout")
    q = torch.empty(B * S, heads * dim, dtype=proj.dtype, device=proj.device)
    native.call("mixers_wide_qkv_prepare", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, off_q, off_k, off_v, heads, kv_heads, dim, vdim,
                native.ptr(q_w), native.ptr(k_w), float(eps), native.ptr(v_other), v_other.stride(0) if v_other is not None else 0,
                native.ptr(blend) if v_other is not None else None, native.ptr(q), native.ptr(k_store), native.ptr(v_store), cap, int(held), int(shift),
                native.ptr(pad), native.ptr(dyn), native.stream(proj.device))
    return q


def sigmoid_gate(o, gate, off_g, per_gate):
    """o[n, c] *= sigmoid(gate[n, off_g + c // per_gate]) in place (o [N, C] contiguous, gate [N, P] contiguous)"""
    invalidInputError(o.is_contiguous() and gate.is_contiguous() and o.dim() == 2 and gate.shape[0] == o.shape[0] and gate.dtype == o.dtype,
                      "sigmoid_gate: unexpected layout")
    native.call("mixers_sigmoid_gate", native.dtype_code(o.dtype), native.ptr(o), o.shape[0], o.shape[1], native.ptr(gate), gate.shape[-1],
                int(off_g), int(per_gate), native.stream(o.device))
    return o


def rms_pair_sum(a, b, w_a, w_b, eps, scale):
    """fp32 [N, W] = scale * (a / rms(a) * w_a + b / rms(b) * w_b)"""
    a, b = _c(a), _c(b)
    invalidInputError(a.shape == b.shape and a.dtype == b.dtype == w_a.dtype == w_b.dtype and w_a.numel() == a.shape[1] == w_b.numel(),
                      "rms_pair_sum: unexpected layout")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    native.call("mixers_rms_pair_sum", native.dtype_code(a.dtype), native.ptr(a), native.ptr(b), native.ptr(w_a), native.ptr(w_b), float(eps),
                float(scale), a.shape[0], a.shape[1], native.ptr(out), native.stream(a.device))
    return out


def sum_residual_norms(x, ys, out_dtype, eps, pre_gain=None, stack=None, index=0, coef=None, gain1=None, gain2=None):
    """x += sum(ys) in place (x fp32 [N, W]; ``ys``: up to two tensors of the model's dtype and two fp32 ones); ``pre_gain``: x is
    first divided by its root mean square and multiplied by this scalar; with ``stack`` [streams, N, W] the new x is kept as
    stream ``index`` and, with ``coef`` [index + 1], replaced by the coefficient-weighted sum of streams 0..index.  Returns
    (x / rms(x) * gain1, x / rms(x) * gain2) in ``out_dtype`` (None where no gain is given)."""
    n, w = x.shape
    invalidInputError(x.dtype == torch.float32 and x.is_contiguous(), "sum_residual_norms: x is a contiguous fp32 [N, W]")
    ys = [y for y in ys if y is not None]
    if out_dtype == torch.float32:                           # a 32-bit model: every addend fits either pair of slots
        floats, typed = ys[:2], ys[2:]
    else:
        typed, floats = [y for y in ys if y.dtype == out_dtype], [y for y in ys if y.dtype == torch.float32]
    invalidInputError(len(typed) <= 2 and len(floats) <= 2 and len(typed) + len(floats) == len(ys)
                      and all(y.shape == x.shape and y.is_contiguous() for y in typed + floats),
                      "sum_residual_norms: addends are contiguous [N, W] tensors of the model's dtype or fp32")
    invalidInputError(stack is None or (stack.dtype == torch.float32 and stack.is_contiguous() and stack.shape[1:] == x.shape and index < stack.shape[0]),
                      "sum_residual_norms: the kept streams are a contiguous fp32 [streams, N, W]")
    invalidInputError(coef is None or (stack is not None and coef.numel() == index + 1), "sum_residual_norms: one coefficient per kept stream")
    typed, floats = typed + [None, None], floats + [None, None]
    h1 = torch.empty(n, w, dtype=out_dtype, device=x.device) if gain1 is not None else None
    h2 = torch.empty(n, w, dtype=out_dtype, device=x.device) if gain2 is not None else None
    native.call("mixers_sum_residual_norms", native.dtype_code(out_dtype), native.ptr(x), n, w, native.ptr(typed[0]), native.ptr(typed[1]),
                native.ptr(floats[0]), native.ptr(floats[1]), native.ptr(pre_gain), float(eps), native.ptr(stack), n * w, int(index),
                native.ptr(coef), native.ptr(gain1), native.ptr(gain2), native.ptr(h1), native.ptr(h2), native.stream(x.device))
    return h1, h2


def gelu_erf(z):
    z = _c(z)
    out = torch.empty_like(z)
    if z.numel():
        native.call("mixers_gelu_erf", native.dtype_code(z.dtype), native.ptr(z), z.numel(), native.ptr(out), native.stream(z.device))
    return out


def rope_qk_prepare(proj, off_q, off_k, off_v, heads, kv_heads, q_dim, k_dim, vdim, q_rot_off, k_rot_off, rot_dims, inv_freq, amp, k_store,
                    k_strides, v_store, v_strides, held, shift, pad, eps=0.0, k_norm_w=None, k_norm_cols=0, dyn=None):
    """rotary positions on the new tokens' queries and keys (columns of proj [B, S, P]) and the cache write of keys and values;
    ``k_strides`` / ``v_strides``: (batch, position, head) strides of the caches in elements; ``inv_freq`` float64 [rot_dims / 2],
    ``amp`` multiplies cosine and sine; ``k_norm_w``: the first ``k_norm_cols`` channels of every key head are RMS-normalised with
    this weight.  Returns q [B * S, heads * q_dim]"""
    B, S, P = proj.shape
    invalidInputError(proj.is_contiguous() and k_store.dtype == proj.dtype and (v_store is None or v_store.dtype == proj.dtype)
                      and (rot_dims == 0 or (inv_freq.dtype == torch.float64 and inv_freq.numel() == rot_dims // 2 and inv_freq.is_contiguous())),
                      "rope_qk_prepare: unexpected layout")
    q = torch.empty(B * S, heads * q_dim, dtype=proj.dtype, device=proj.device)
    vs = v_strides if v_store is not None else (0, 0, 0)
    native.call("mixers_rope_qk_prepare", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, int(off_q), int(off_k), int(off_v), heads, kv_heads,
                q_dim, k_dim, vdim if v_store is not None else 0, int(q_rot_off), int(k_rot_off), int(rot_dims), native.ptr(inv_freq) if rot_dims else None,
                float(amp), native.ptr(k_norm_w), int(k_norm_cols), float(eps), native.ptr(q), native.ptr(k_store), *[int(v) for v in k_strides],
                native.ptr(v_store), *[int(v) for v in vs], int(held), int(shift), native.ptr(pad), native.ptr(dyn), native.stream(proj.device))
    return q


def poly_norm(z, coef, eps):
    z = _c(z)
    out = torch.empty_like(z)
    native.call("mixers_poly_norm", native.dtype_code(z.dtype), native.ptr(z), z.numel() // z.shape[-1], z.shape[-1], native.ptr(coef),
                float(eps), native.ptr(out), native.stream(z.device))
    return out


def soft_cap(x, cap):
    x = _c(x)
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    native.call("mixers_soft_cap", native.dtype_code(x.dtype), native.ptr(x), x.numel(), float(cap) if cap else 0.0, native.ptr(out),
                native.stream(x.device))
    return out


# ------------------------------------------------------------------ output-normalised residual stream, latent attention, routed experts
def embed_pair(table, scale, pair, buckets, mul_prev, mul_cur, ids, prev, slot0, pad, out_dtype, x_copy=None):
    """fp32 x [N, W] = table[id] * scale + pair[row]; also returns x in ``out_dtype``.  ids [B, S] int64, prev [B] int64 (the token
    before each row's first new one); ``x_copy``: a second fp32 [N, W] destination (the first of the kept streams)."""
    B, S = ids.shape
    ids = _c(ids)
    w = table.shape[1]
    invalidInputError(table.is_contiguous() and (pair is None or (pair.is_contiguous() and pair.shape[1] == w and pair.shape[0] > buckets)),
                      "embed_pair: unexpected layout")
    x = torch.empty(B * S, w, dtype=torch.float32, device=table.device)
    h = torch.empty(B * S, w, dtype=out_dtype, device=table.device)
    native.call("mixers_embed_pair", native.dtype_code(table.dtype), native.ptr(table), float(scale), native.ptr(pair), int(buckets), int(mul_prev),
                int(mul_cur), native.ptr(ids), native.ptr(prev), B, S, w, int(slot0), native.ptr(pad), native.ptr(x), native.ptr(x_copy),
                native.ptr(h), native.stream(x.device))
    return x, h


def rms_residual(x, y, gain, vec, eps, out_dtype, stack=None, index=0, coef=None, want_h=True):
    """x += y / rms(y) * gain * vec in place (x fp32 [N, W]); with ``stack`` [streams, N, W] the new x is kept as stream ``index``
    and, with ``coef`` [index + 1], replaced by the coefficient-weighted sum of streams 0..index.  Returns x in ``out_dtype``."""
    n, w = x.shape
    y = _c(y)
    invalidInputError(x.dtype == torch.float32 and x.is_contiguous() and y.shape == x.shape and y.dtype in (out_dtype, torch.float32),
                      "rms_residual: x is a contiguous fp32 [N, W], y the model's dtype or fp32")
    invalidInputError(stack is None or (stack.dtype == torch.float32 and stack.is_contiguous() and stack.shape[1:] == x.shape and index < stack.shape[0]),
                      "rms_residual: the kept streams are a contiguous fp32 [streams, N, W]")
    invalidInputError(coef is None or (stack is not None and coef.numel() == index + 1), "rms_residual: one coefficient per kept stream")
    h = torch.empty(n, w, dtype=out_dtype, device=x.device) if want_h else None
    native.call("mixers_rms_residual", native.dtype_code(out_dtype), native.ptr(x), n, w, native.ptr(y), int(y.dtype == torch.float32 and out_dtype != torch.float32),
                native.ptr(gain), native.ptr(vec), float(eps), native.ptr(stack), n * w, int(index), native.ptr(coef), native.ptr(h),
                native.stream(x.device))
    return h


def rms_norm_rows(x, gain, vec, eps, out_dtype):
    x = _c(x)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    native.call("mixers_rms_norm_rows", native.dtype_code(out_dtype), native.ptr(x), x.numel() // x.shape[-1], x.shape[-1], native.ptr(gain),
                native.ptr(vec), float(eps), native.ptr(out), native.stream(x.device))
    return out


def xielu(z, pq):
    z = _c(z)
    out = torch.empty_like(z)
    native.call("mixers_xielu", native.dtype_code(z.dtype), native.ptr(z), z.numel(), native.ptr(pq), native.ptr(out), native.stream(z.device))
    return out


def silu_mul(gate_up, cols):
    """silu(first ``cols`` columns) * the next ``cols`` columns"""
    gate_up = _c(gate_up)
    n = gate_up.numel() // gate_up.shape[-1]
    out = torch.empty(n, cols, dtype=gate_up.dtype, device=gate_up.device)
    if n:
        native.call("mixers_silu_mul", native.dtype_code(gate_up.dtype), native.ptr(gate_up), n, gate_up.shape[-1], 0, cols, cols, native.ptr(out),
                    native.stream(out.device))
    return out


def gelu_table_mul(g, table, col0, ids):
    """gelu_tanh(g [N, C]) * table[ids, col0 : col0 + C]"""
    g, ids = _c(g), _c(ids)
    out = torch.empty_like(g)
    native.call("mixers_gelu_table_mul", native.dtype_code(g.dtype), native.ptr(g), g.shape[0], g.shape[1], native.ptr(table), table.shape[1], int(col0),
                native.ptr(ids), native.ptr(out), native.stream(g.device))
    return out


def latent_prepare(proj, off_q, q_rank, q_w, off_c, kv_rank, c_w, eps, store, held, shift, pad, dyn=None):
    """the normalised query latent [B * S, q_rank]; the normalised key/value latent goes into ``store`` [B, cap, kv_rank]"""
    B, S, P = proj.shape
    invalidInputError(proj.is_contiguous() and store.is_contiguous() and store.dtype == proj.dtype and store.shape[0] == B
                      and store.shape[2] == kv_rank, "latent_prepare: unexpected layout")
    cq = torch.empty(B * S, q_rank, dtype=proj.dtype, device=proj.device)
    native.call("mixers_latent_prepare", native.dtype_code(proj.dtype), native.ptr(proj), B, S, P, off_q, q_rank, native.ptr(q_w), off_c, kv_rank,
                native.ptr(c_w), float(eps), native.ptr(cq), native.ptr(store), store.shape[1], int(held), int(shift), native.ptr(pad), native.ptr(dyn),
                native.stream(proj.device))
    return cq


def softmax_attention(q, k, v, B, S, heads, held, shift, pad, window, scale, out=None, out_col=0, dyn=None, tensor_cores=True, softcap=0.0,
                      sink=None, chunk=0):
    """q [B * S, heads * dim], or [B * S, heads, dim] with any token and head strides; k [B, L, kv_heads, dim], v [B, L, kv_heads,
    vdim] views (any strides with a unit last one); returns out [B * S, heads * vdim] in q's dtype.  ``softcap`` > 0 caps the
    scaled scores (cap * tanh(score / cap)); ``sink`` [heads]: a per-head term exp(sink) in the softmax's denominator;
    ``chunk`` > 0: a query sees only the earlier positions of its own chunk of that many positions"""
    kv_heads, dim, vdim = k.shape[2], k.shape[3], v.shape[3]
    q_hs = q.stride(1) if q.dim() == 3 else dim
    invalidInputError(q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and q.numel() == B * S * heads * dim and k.dtype == q.dtype
                      and v.dtype == q.dtype and v.shape[2] == kv_heads and (dyn is not None or (k.shape[1] >= held + S and v.shape[1] >= held + S)),
                      "softmax_attention: unexpected layout")
    invalidInputError(sink is None or (sink.numel() == heads and sink.dtype == q.dtype and sink.is_contiguous()), "softmax_attention: one sink per head")
    if out is None:
        out = torch.empty(B * S, heads * vdim, dtype=q.dtype, device=q.device)
    need = native.lib().mixers_softmax_attention_workspace(native.dtype_code(q.dtype), B, S, heads, kv_heads, dim, vdim) if tensor_cores else 0
    ws = torch.empty(need, dtype=torch.float32, device=q.device) if need else None
    native.call("mixers_softmax_attention", native.dtype_code(q.dtype), native.ptr(q), q.stride(0), q_hs, native.ptr(k), k.stride(0), k.stride(1),
                k.stride(2), native.ptr(v), v.stride(0), v.stride(1), v.stride(2), B, S, heads, kv_heads, dim, vdim, int(held), int(shift),
                native.ptr(pad), int(window), int(chunk), float(scale), float(softcap or 0.0), native.ptr(sink), native.ptr(out), out.stride(0), int(out_col),
                native.ptr(dyn), int(bool(tensor_cores)),
                native.ptr(ws), native.stream(q.device))
    return out


def grouped_router(h, router, correction, groups, keep, top):
    """(chosen outputs int32 [N, top], their softmax scores fp32 [N, top])"""
    h = _c(h)
    n, w = h.shape
    invalidInputError(router.is_contiguous() and router.shape[1] == w and router.dtype == h.dtype and correction.dtype == h.dtype
                      and correction.numel() == router.shape[0], "grouped_router: unexpected layout")
    idx = torch.empty(n, top, dtype=torch.int32, device=h.device)
    wgt = torch.empty(n, top, dtype=torch.float32, device=h.device)
    native.call("mixers_grouped_router", native.dtype_code(h.dtype), native.ptr(h), n, w, native.ptr(router), native.ptr(correction), router.shape[0],
                int(groups), int(keep), int(top), native.ptr(idx), native.ptr(wgt), native.stream(h.device))
    return idx, wgt


def scored_router(h, router, correction, groups, keep, top, sigmoid=True, group_top=2, renorm=True, scale=1.0, gate_row=None):
    """(chosen outputs int32 [N, top], weights fp32 [N, top], gate fp32 [N] or None).  Scores: a sigmoid per output (or the
    softmax over all); groups ranked by the sum of their ``group_top`` best choice scores; weights = the winners' scores, over
    their sum if ``renorm``, times ``scale``; ``gate_row`` [1, W]: gate = sigmoid(gate_row . h) for an expert every token runs"""
    h = _c(h)
    n, w = h.shape
    invalidInputError(router.is_contiguous() and router.shape[1] == w and router.dtype == h.dtype
                      and (correction is None or (correction.dtype == h.dtype and correction.numel() == router.shape[0])) and (gate_row is None or (gate_row.numel() == w and gate_row.dtype == h.dtype
                                                                                           and gate_row.is_contiguous())),
                      "scored_router: unexpected layout")
    idx = torch.empty(n, top, dtype=torch.int32, device=h.device)
    wgt = torch.empty(n, top, dtype=torch.float32, device=h.device)
    gate = torch.empty(n, dtype=torch.float32, device=h.device) if gate_row is not None else None
    native.call("mixers_scored_router", native.dtype_code(h.dtype), native.ptr(h), n, w, native.ptr(router), native.ptr(correction), router.shape[0],
                int(groups), int(keep), int(top), int(bool(sigmoid)), int(group_top), int(bool(renorm)), float(scale), native.ptr(gate_row),
                native.ptr(gate), native.ptr(idx), native.ptr(wgt), native.stream(h.device))
    return idx, wgt, gate


def clamped_glu(gate_up, cols, limit):
    """g' sigmoid(1.702 g') (u' + 1): g' = the first ``cols`` columns capped at ``limit``, u' = the next ``cols`` clamped to +-limit"""
    gate_up = _c(gate_up)
    n = gate_up.numel() // gate_up.shape[-1]
    out = torch.empty(n, cols, dtype=gate_up.dtype, device=gate_up.device)
    if n:
        native.call("mixers_clamped_glu", native.dtype_code(gate_up.dtype), native.ptr(gate_up), n, gate_up.shape[-1], 0, cols, cols, float(limit),
                    native.ptr(out), native.stream(out.device))
    return out


def moe_small(h, idx, wgt, gate_up_table, down_table, ff, n_experts, n_out, shared_out, ffs=None, always_on=False, always_w=None, clamped=False,
              limit=0.0, limit_always=0.0, ungated_gelu=False, weight_input=False):
    """fp32 [N, W]: the chosen experts of a few tokens through tables of the experts' weight addresses.  ``ffs``: int32 sizes per
    table entry (``ff`` = the largest); ``always_on``: table entry ``n_experts`` is an expert every token runs, with weight
    ``always_w`` [N] (None: 1); ``clamped``: the experts' activation is the clamped form with ``limit`` (``limit_always`` for the
    always-on expert) instead of silu(g) u; ``ungated_gelu``: the experts have no gate, their first matrix is [ff, width] and
    the activation the exact gelu; ``weight_input``: a chosen expert's weight multiplies its input instead of its output"""
    h = _c(h)
    n, w = h.shape
    top = idx.shape[1]
    act = torch.empty(max(n * (top + int(always_on)) * ff, 1), dtype=h.dtype, device=h.device)
    y = torch.empty(n, w, dtype=torch.float32, device=h.device)
    native.call("mixers_moe_small", native.dtype_code(h.dtype), native.ptr(h), n, w, int(ff), top, int(n_experts), int(n_out), native.ptr(idx),
                native.ptr(wgt), native.ptr(gate_up_table), native.ptr(down_table), native.ptr(ffs), int(bool(always_on)), native.ptr(always_w),
                2 if ungated_gelu else int(bool(clamped)), int(bool(weight_input)), float(limit), float(limit_always), native.ptr(shared_out), native.ptr(act), native.ptr(y), native.stream(h.device))
    return y


def moe_sort(idx, n_keys):
    """(counts int32 [n_keys], pos int32 [N, top], token_of int64 [N * top]): the (token, choice) pairs sorted by chosen output"""
    idx = _c(idx)
    n, top = idx.shape
    counts = torch.empty(n_keys, dtype=torch.int32, device=idx.device)
    pos = torch.empty(n, top, dtype=torch.int32, device=idx.device)
    token_of = torch.empty(n * top, dtype=torch.int64, device=idx.device)
    native.call("mixers_moe_sort", native.ptr(idx), n * top, top, int(n_keys), native.ptr(counts), native.ptr(pos), native.ptr(token_of),
                native.stream(idx.device))
    return counts, pos, token_of


def moe_scatter_scaled(h, pos, idx, wgt, n_experts, n_rows):
    """[n_rows, W] in h's dtype: row pos[n, k] = h[n] * wgt[n, k] for every choice of an expert (the experts' sorted, weighted inputs)"""
    h = _c(h)
    n, top = idx.shape
    rows = torch.empty(max(n_rows, 1), h.shape[1], dtype=h.dtype, device=h.device)
    native.call("mixers_moe_scatter_scaled", native.dtype_code(h.dtype), native.ptr(h), native.ptr(pos), native.ptr(idx), native.ptr(wgt), n * top, top,
                h.shape[1], int(n_experts), native.ptr(rows), native.stream(h.device))
    return rows


def moe_combine(rows, pos, idx, wgt, h, shared_out, n_experts, n_out, shared_w=None):
    """fp32 [N, W]: weighted sum of the experts' outputs ``rows`` (row pos[n, k] belongs to token n's k-th choice) + shared_out
    (times ``shared_w`` [N] when given); ``wgt`` None: every weight is 1"""
    h = _c(h)
    n, w = h.shape
    y = torch.empty(n, w, dtype=torch.float32, device=h.device)
    native.call("mixers_moe_combine", native.dtype_code(h.dtype), native.ptr(rows), native.ptr(pos), native.ptr(idx), native.ptr(wgt), native.ptr(h),
                native.ptr(shared_out), native.ptr(shared_w), n, w, idx.shape[1], int(n_experts), int(n_out), native.ptr(y), native.stream(h.device))
    return y
