"""Plain statements of the Nikedra design's mechanisms (PyTorch, any dtype; the tests use float64), one function each, and a
whole-model forward that recomputes every position from the full token list.  Nothing here is shared with the package:
weights come in as a dict of tensors under the checkpoint's names, the configuration as the parsed config.json.

The design: every layer normalises the stream twice with one scalar gain each (the mixer's and the feed-forward's input), adds
a short causal convolution over time to the mixer's input, runs mixer and feed-forward side by side on the same stream and adds
both; what a layer hands on is a learned combination of the embedding output and every layer's result so far.  Mixers: a delta
rule whose state decays per key channel ("channel_delta"), latent attention with one rotated key part shared by all heads under
a sliding window ("latent_attention"), and chunked grouped attention with scaled rotary frequencies next to a state-space
recurrence ("parallel").  Feed-forwards: a clamped gated one with biases, or sigmoid-routed experts whose weight scales the
expert's INPUT.
"""
import math

import torch


# ------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_taps(h, w, bias=None):
    """h [T, C], w [C, taps] (last column multiplies the current token), zeros before the first token"""
    T, C = h.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=h.dtype), h], dim=0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    return out if bias is None else out + bias


# ------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot, dtype=torch.float64):
    """(frequency per pair [dims / 2], amplitude) of a 'rot' block: base^(-2i / dims), optionally rescaled by a ramp between a
    fast and a slow number of turns within the original length; the amplitude multiplies cos and sin"""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=dtype)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=dtype)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """x [T, heads, D]: the first rot.dims channels of every head are rotated, channel i with channel i + dims / 2"""
    dims = int(rot["dims"])
    half = dims // 2
    f, amp = rotary_frequencies(rot, x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]                       # [T, half]
    cos, sin = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------ masks
def window_mask(T, size):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T, size):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def masked_softmax_attention(q, k, v, scale, mask):
    """q [T, H, D], k [T, H, D], v [T, H, Dv] (already one key/value head per query head), mask [T, T] True = visible"""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


# ------------------------------------------------------------------ mixers
def latent_attention_mixer(h, W, m, eps):
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W["q"].T).view(T, H, D + Dr)
    dkv = h @ W["dkv"].T
    c = unit_rms(dkv[:, :R], eps) * W["dkv.norm"]
    rot = dict(m["rot"], dims=Dr)
    k_rot = rotate_half(dkv[:, R:].view(T, 1, Dr), pos, rot)
    q_rot = rotate_half(q[..., D:], pos, rot)
    k = torch.cat([(c @ W["uk"].T).view(T, H, D), k_rot.expand(T, H, Dr)], dim=-1)
    qq = torch.cat([q[..., :D], q_rot], dim=-1)
    v = (c @ W["uv"].T).view(T, H, Dv)
    o = masked_softmax_attention(qq, k, v, m["scale"], window_mask(T, int(m["mask"]["size"]))).reshape(T, H * Dv)
    return (o * torch.sigmoid(h @ W["g"].T)) @ W["o"].T


def channel_decay(h, W, H, D):
    """per head and key channel, in (0, 1)"""
    T = h.shape[0]
    dt = softplus((h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]).view(T, H, D)
    return torch.exp(-torch.exp(W["A_log"]).view(1, H, 1) * dt)


def channel_delta_scan(q, k, v, g, beta):
    """q, k, g [T, H, D]; v [T, H, Dv]; beta [T, H].  State S [H, D, Dv] from zero:
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q"""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t].unsqueeze(-1) * S
        u = beta[t].unsqueeze(-1) * (v[t] - torch.einsum("hij,hi->hj", S, k[t]))
        S = S + k[t].unsqueeze(-1) * u.unsqueeze(-2)
        out.append(torch.einsum("hij,hi->hj", S, q[t]))
    return torch.stack(out)


def channel_delta_mixer(h, W, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = silu(causal_taps(h @ W["q"].T, W["q.conv"])).view(T, G, D)
    k = silu(causal_taps(h @ W["k"].T, W["k.conv"])).view(T, G, D)
    v = silu(causal_taps(h @ W["v"].T, W["v.conv"])).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W["b"].T)
    o = channel_delta_scan(q, k, v, channel_decay(h, W, H, D), beta)
    o = unit_rms(o, eps) * W["norm"] * torch.sigmoid((h @ W["g1"].T) @ W["g2"].T).view(T, H, Dv)
    return o.reshape(T, H * Dv) @ W["o"].T


def chunked_attention_branch(h, W, m):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate_half((h @ W["q"].T).view(T, H, D), pos, m["rot"])
    k = rotate_half((h @ W["k"].T).view(T, G, D), pos, m["rot"]).repeat_interleave(H // G, dim=1)
    v = (h @ W["v"].T).view(T, G, Dv).repeat_interleave(H // G, dim=1)
    o = masked_softmax_attention(q, k, v, m["scale"], chunk_mask(T, int(m["mask"]["size"])))
    o = o * torch.sigmoid(h @ W["g"].T).unsqueeze(-1)                        # one gate per head
    return o.reshape(T, H * Dv) @ W["o"].T


def state_space_scan(x, Bm, Cm, dt, A, Dskip):
    """x [T, H, P]; Bm, Cm [T, H, N]; dt [T, H]; A (positive) and Dskip [H].  S [H, N, P] from zero:
    S <- exp(-A dt) S + dt B x^T;  y = S^T C + Dskip x"""
    T, H, P = x.shape
    S = torch.zeros(H, Bm.shape[-1], P, dtype=x.dtype)
    out = []
    for t in range(T):
        S = torch.exp(-A * dt[t]).view(H, 1, 1) * S + dt[t].view(H, 1, 1) * Bm[t].unsqueeze(-1) * x[t].unsqueeze(-2)
        out.append(torch.einsum("hnp,hn->hp", S, Cm[t]) + Dskip.view(H, 1) * x[t])
    return torch.stack(out)


def state_space_branch(h, W, m, eps):
    T = h.shape[0]
    H, P, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    proj = h @ W["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_taps(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
    Cm = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + W["dt_bias"])
    y = state_space_scan(x, Bm, Cm, dt, torch.exp(W["A_log"]), W["D"]).reshape(T, inner)
    y = y * silu(z)
    y = unit_rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def parallel_mixer(h, W, m, eps):
    left = chunked_attention_branch(h, sub(W, "left."), m["left"])
    right = state_space_branch(h, sub(W, "right."), m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * W["left.out"] + unit_rms(right, eps) * W["right.out"])


# ------------------------------------------------------------------ feed-forwards
def clamped_dense(h, W, m):
    limit = float(m["limit"])
    g = torch.clamp(h @ W["gate"].T + W["gate.b"], max=limit)
    u = torch.clamp(h @ W["up"].T + W["up.b"], -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T + W["down.b"]


def route(h, router, top):
    """(chosen experts [T, top], their sigmoid scores [T, top]): the largest scores, lowest index first among equals"""
    s = torch.sigmoid(h @ router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def route_margins(h, router, top):
    """how far each token's last chosen score is above the best one left out (inf when all are chosen)"""
    s = torch.sort(torch.sigmoid(h @ router.T), dim=-1, descending=True).values
    if s.shape[1] <= top:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    return s[:, top - 1] - s[:, top]


def input_weighted_experts(h, W, m):
    E, top = int(m["router"]["experts"]), int(m["router"]["top"])
    idx, wgt = route(h, W["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] = out[t] + gelu_erf((wgt[t, j] * h[t]) @ W[f"e{e}.up"].T) @ W[f"e{e}.down"].T
    return out


# ------------------------------------------------------------------ the model
def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


MIXERS = {"latent_attention": latent_attention_mixer, "channel_delta": channel_delta_mixer, "parallel": parallel_mixer}


def forward(cfg, weights, tokens, collect=None, margins=None):
    """logits [T, vocab] of one sequence; ``collect``: a list that receives what every layer hands on (behind the depth
    average); ``margins``: a list that receives every routed layer's route_margins"""
    eps = float(cfg["norm"]["eps"])
    taps = int(cfg["canon"]["taps"])
    x = unit_rms(weights["embed"][torch.as_tensor(tokens)], eps) * weights["embed.norm"]
    streams = [x]
    for i, lc in enumerate(cfg["layers"]):
        W = sub(weights, f"l{i}.")
        h = unit_rms(x, eps) * W["norm1"]
        assert W["canon1"].shape[1] == taps
        h = h + causal_taps(h, W["canon1"])
        y = MIXERS[lc["type"]](h, sub(W, "mix."), lc["mixer"], eps)
        mlp = lc.get("mlp")
        if mlp is not None:
            h2 = unit_rms(x, eps) * W["norm2"]
            if mlp["kind"] == "dense":
                y = y + clamped_dense(h2, sub(W, "mlp."), mlp)
            else:
                if margins is not None:
                    margins.append(route_margins(h2, W["mlp.router"], int(mlp["router"]["top"])))
                y = y + input_weighted_experts(h2, sub(W, "mlp."), mlp)
        x = x + y
        streams.append(x)
        x = sum(W["dwa"][j] * streams[j] for j in range(i + 2))
        if collect is not None:
            collect.append(x.clone())
    x = unit_rms(x, eps) * weights["final.norm"]
    return (x @ weights["head"].T) * float(cfg["logit_scale"])


def greedy(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens


# ------------------------------------------------------------------ pieces the kernel tests address directly
def visible_attention(q, k, v, scale, held=0, first=0, window=0, chunk=0, origin=None):
    """q [S, H, D]: new tokens that sit at indices held .. held + S - 1 of k [L, G, D] / v [L, G, Dv]; indices below ``first`` do
    not exist (padding); ``origin``: the index that holds position 0 (``first`` unless earlier positions have left the storage,
    then negative).  ``window`` > 0: a query sees itself and the window - 1 positions before it; ``chunk`` > 0: only the earlier
    positions of its own chunk of positions.  Returns [S, H, Dv] (zeros where no query exists)."""
    S, H, D = q.shape
    per = H // k.shape[1]
    origin = first if origin is None else origin
    out = torch.zeros(S, H, v.shape[2], dtype=q.dtype)
    for t in range(S):
        c = held + t
        if c < first:
            continue
        lo = first
        if window:
            lo = max(lo, c - window + 1)
        if chunk:
            lo = max(lo, origin + ((c - origin) // chunk) * chunk)
        for hd in range(H):
            s = (k[lo:c + 1, hd // per] @ q[t, hd]) * scale
            out[t, hd] = torch.softmax(s, dim=0) @ v[lo:c + 1, hd // per]
    return out


# ------------------------------------------------------------------ random models
LATENT = dict(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=12, window=9, base=100.0, scale=0.3)
DELTA = dict(heads=4, kv_heads=2, dim=12, vdim=10, conv=4)
LEFT = dict(heads=6, kv_heads=2, dim=12, vdim=10, rot_dims=8, base=50.0, chunk=7, scale=0.25, factor=4.0, original=16, fast=4.0, slow=1.0)
RIGHT = dict(heads=4, vdim=6, state=10, groups=2, norm_groups=2, conv=2)
DENSE = dict(ff=24, limit=0.7)
MOE = dict(experts=5, top=2, ff=12)


def random_config(width=40, vocab=61, taps=3, order=("latent_attention", "channel_delta", "parallel", "channel_delta"),
                  mlps=("dense", "moe", None, "moe"), latent=None, delta=None, left=None, right=None, dense=None, moe=None, eps=1e-5,
                  logit_scale=0.5):
    """``order``: the layers' mixers; ``mlps``: per layer "dense", "moe" or None; the dicts override the sizes above"""
    la, de, le, ri, dn, mo = (dict(base, **(over or {})) for base, over in ((LATENT, latent), (DELTA, delta), (LEFT, left), (RIGHT, right),
                                                                             (DENSE, dense), (MOE, moe)))
    layers = []
    for kind, ff in zip(order, mlps):
        if kind == "latent_attention":
            mixer = {"heads": la["heads"], "dim": la["dim"], "rot_dim": la["rot_dim"], "vdim": la["vdim"], "kv_rank": la["kv_rank"],
                     "scale": la["scale"], "mask": {"size": la["window"]}, "rot": {"base": la["base"], "dims": la["rot_dim"]}}
        elif kind == "channel_delta":
            mixer = {k: de[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
        else:
            rot = {"base": le["base"], "dims": le["rot_dims"]}
            if le["factor"]:
                rot["scaling"] = {k: le[k] for k in ("factor", "original", "fast", "slow")}
            mixer = {"left": {"heads": le["heads"], "kv_heads": le["kv_heads"], "dim": le["dim"], "vdim": le["vdim"], "scale": le["scale"],
                              "mask": {"size": le["chunk"]}, "rot": rot},
                     "right": {k: ri[k] for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")}}
        mlp = None
        if ff == "dense":
            mlp = {"kind": "dense", "ff": dn["ff"], "limit": dn["limit"]}
        elif ff == "moe":
            mlp = {"kind": "moe", "expert": {"ff": mo["ff"]}, "router": {"experts": mo["experts"], "top": mo["top"]}}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Nikedra", "vocab": vocab, "width": width, "canon": {"taps": taps}, "norm": {"eps": eps}, "layers": layers,
            "logit_scale": logit_scale}


def random_weights(cfg, seed, ranks=(5, 3), dtype=torch.bfloat16):
    """weights under the checkpoint's names; ``ranks``: the inner sizes of a channel_delta layer's decay and gate projections"""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    taps = cfg["canon"]["taps"]

    def mat(o, i, s=1.0):
        return torch.randn(o, i, generator=g) * (s / math.sqrt(i))

    def vec(n, mean=1.0, s=0.2):
        return mean + torch.randn(n, generator=g) * s

    def gain():
        return torch.rand((), generator=g) * 1.0 + 0.6

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g), "embed.norm": gain(), "final.norm": gain(), "head": mat(cfg["vocab"], W)}
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = gain()
        w[p + "canon1"] = torch.randn(W, taps, generator=g) * 0.4
        dwa = torch.randn(i + 2, generator=g) * 0.3
        dwa[-1] += 1.0                                                      # mostly the layer's own result, some of every earlier stream
        w[p + "dwa"] = dwa
        x = p + "mix."
        if lc["type"] == "latent_attention":
            H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[x + "q"], w[x + "dkv"], w[x + "g"] = mat(H * (D + Dr), W, 2.0), mat(R + Dr, W, 2.0), mat(H * Dv, W)
            w[x + "dkv.norm"] = vec(R, 1.0, 0.4)
            w[x + "uk"], w[x + "uv"], w[x + "o"] = mat(H * D, R, 2.0), mat(H * Dv, R), mat(W, H * Dv)
        elif lc["type"] == "channel_delta":
            H, G, D, Dv, T = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            w[x + "q"], w[x + "k"], w[x + "v"], w[x + "b"] = mat(G * D, W, 2.0), mat(G * D, W, 2.0), mat(H * Dv, W, 2.0), mat(H, W, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[x + n + ".conv"] = torch.randn(c, T, generator=g) * 0.6
            w[x + "a1"], w[x + "a2"] = mat(ranks[0], W), mat(H * D, ranks[0], 2.0)
            w[x + "g1"], w[x + "g2"] = mat(ranks[1], W), mat(H * Dv, ranks[1], 2.0)
            w[x + "A_log"], w[x + "dt_bias"] = torch.randn(H, generator=g) * 0.7 - 0.5, torch.randn(H * D, generator=g) - 1.0
            w[x + "norm"], w[x + "o"] = vec(Dv), mat(W, H * Dv)
        else:
            l, r = m["left"], m["right"]
            H, G, D, Dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            w[x + "left.q"], w[x + "left.k"], w[x + "left.v"] = mat(H * D, W, 2.0), mat(G * D, W, 2.0), mat(G * Dv, W)
            w[x + "left.g"], w[x + "left.o"], w[x + "left.out"] = mat(H, W, 2.0), mat(W, H * Dv), vec(W)
            Hs, P, N, Gs, T = r["heads"], r["vdim"], r["state"], r["groups"], r["conv"]
            inner, C = Hs * P, Hs * P + 2 * Gs * N
            w[x + "right.in"] = mat(2 * inner + 2 * Gs * N + Hs, W, 1.5)
            w[x + "right.conv"], w[x + "right.conv.b"] = torch.randn(C, T, generator=g) * 0.6, torch.randn(C, generator=g) * 0.3
            w[x + "right.dt_bias"], w[x + "right.A_log"] = torch.randn(Hs, generator=g) - 0.5, torch.randn(Hs, generator=g) * 0.7 - 0.5
            w[x + "right.D"], w[x + "right.norm"] = vec(Hs, 0.5, 0.5), vec(inner)
            w[x + "right.o"], w[x + "right.out"] = mat(W, inner), vec(W)
        ff = lc.get("mlp")
        if ff is not None:
            w[p + "norm2"] = gain()
            y = p + "mlp."
            if ff["kind"] == "dense":
                F = ff["ff"]
                w[y + "gate"], w[y + "up"], w[y + "down"] = mat(F, W, 2.0), mat(F, W, 2.0), mat(W, F)
                w[y + "gate.b"], w[y + "up.b"], w[y + "down.b"] = (torch.randn(n, generator=g) * 0.3 for n in (F, F, W))
            else:
                E, F = ff["router"]["experts"], ff["expert"]["ff"]
                for e in range(E):
                    w[y + f"e{e}.up"], w[y + f"e{e}.down"] = mat(F, W, 2.0), mat(W, F)
                w[y + "router"] = mat(E, W, 3.0)
    return {k: v.to(dtype) for k, v in w.items()}
