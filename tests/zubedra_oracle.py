"""Plain statements of the Zubedra design's mechanisms (PyTorch, any dtype; the tests use float64), one function each, and a
whole-model forward that recomputes every position from the full token list.  Nothing here is shared with the package:
weights come in as a dict of tensors under the checkpoint's names, the configuration as the parsed config.json.

The design: a parallel layer (one layer norm feeds the mixer and the feed-forward, both are added to the stream at once) whose
mixer is either an RWKV-style recurrence ("wkv": token shift, per-channel decay from a low-rank projection, a bonus for the
current token) or position-free softmax attention (norm over the whole query / key projection, capped scores, a sink in the
denominator, values blended with those of the first blending layer); the feed-forward is a mixture of experts with sigmoid
scores, grouped choice, clamped gated experts and a gated shared expert.
"""
import math

import torch


# ------------------------------------------------------------------ norms
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, eps):
    """mean removed, divided by the standard deviation (variance = mean squared deviation), times w; no bias"""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


# ------------------------------------------------------------------ wkv mixer
def shifted(h):
    """row t holds h[t - 1]; zeros in front of the first token"""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu"""
    return h + (shifted(h) - h) * mu


def wkv_decay(xw, w1, w2, w0):
    """per head and key channel, in (0, 1): exp(-exp(w0 + W2 tanh(W1 xw)))"""
    return torch.exp(-torch.exp(torch.tanh(xw @ w1.T) @ w2.T + w0))


def wkv_scan(r, k, v, w, u):
    """r, k, v, w [T, H, D]; u [H, D].  State A [H, D(key), D(value)] starts at zero:
    out_t = (A + diag(u) k_t v_t^T)^T r_t;  A <- diag(w_t) A + k_t v_t^T"""
    T, H, D = r.shape
    A = torch.zeros(H, D, D, dtype=r.dtype)
    out = []
    for t in range(T):
        kv = k[t].unsqueeze(-1) * v[t].unsqueeze(-2)                         # [H, D, D]
        out.append(torch.einsum("hij,hi->hj", A + u.unsqueeze(-1) * kv, r[t]))
        A = w[t].unsqueeze(-1) * A + kv
    return torch.stack(out)


def wkv_mixer(h, W, m, eps):
    """h [T, width] of one sequence; W: the mixer's tensors by short name"""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    mix = {s: token_shift(h, W["mu." + s]) for s in "rkvgw"}
    r = (mix["r"] @ W["r"].T).view(T, H, D)
    k = (mix["k"] @ W["k"].T).view(T, H, D)
    v = (mix["v"] @ W["v"].T).view(T, H, D)
    g = mix["g"] @ W["g"].T
    gate = g * torch.sigmoid(g)
    w = wkv_decay(mix["w"], W["w1"], W["w2"], W["w0"]).view(T, H, D)
    o = unit_rms(wkv_scan(r, k, v, w, W["u"]), eps).reshape(T, H * D)
    return (o * W["norm"] * gate) @ W["o"].T


# ------------------------------------------------------------------ attention mixer
def capped(s, cap):
    return cap * torch.tanh(s / cap)


def sink_softmax(s, sink):
    """softmax over the last axis of s [..., H, T, T'] whose denominator also holds exp(sink) per head"""
    big = torch.maximum(s.max(-1, keepdim=True).values, sink.view(-1, 1, 1))
    e = torch.exp(s - big)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink.view(-1, 1, 1) - big))


def attention_values(h, W, m, v_first):
    """the layer's values [T, G * vdim]: its own projection, blended with the first blending layer's when there is one"""
    v = h @ W["v"].T
    if m.get("v_mix") and v_first is not None:
        lam = W["vmix"]
        v = (1 - lam) * v + lam * v_first
    return v


def attention_mixer(h, W, m, eps, v_first):
    """returns (output [T, width], the values this layer used)"""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (unit_rms(h @ W["q"].T, eps) * W["q.norm"]).view(T, H, D)
    k = (unit_rms(h @ W["k"].T, eps) * W["k.norm"]).view(T, G, D)
    v = attention_values(h, W, m, v_first)
    vh = v.view(T, G, Dv)
    per = H // G
    kk, vv = k.repeat_interleave(per, dim=1), vh.repeat_interleave(per, dim=1)
    s = capped(torch.einsum("ihd,jhd->hij", q, kk) * m["scale"], m["softcap"])
    s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
    p = sink_softmax(s, W["sink"])
    o = torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * Dv)
    return o @ W["o"].T, v


# ------------------------------------------------------------------ feed-forward
def clamped_expert(h, gate, up, down, limit):
    g = (h @ gate.T).clamp(max=limit)
    u = (h @ up.T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T


def route(h, router, correction, r):
    """(chosen [T, top], weights [T, top]): sigmoid scores; the choice adds the correction; groups of neighbours are ranked by
    the sum of their two best choice scores and only the kept groups' experts can win; weights are the winners' plain scores
    over their sum, times the router's scale"""
    n = router.shape[0]
    s = torch.sigmoid(h @ router.T)
    choice = s + correction
    grp = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(grp["count"]), int(grp["keep"])
    per = n // count
    idx_rows, w_rows = [], []
    for t in range(h.shape[0]):
        c = choice[t]
        gs = [sum(sorted(c[g * per:(g + 1) * per].tolist(), reverse=True)[:2]) for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-gs[g], g))[:keep]
        allowed = [e for g in kept for e in range(g * per, (g + 1) * per)]
        win = sorted(allowed, key=lambda e: (-float(c[e]), e))[:int(r["top"])]
        sw = s[t][torch.tensor(win)]
        idx_rows.append(win)
        w_rows.append(sw / (sw.sum() + 1e-20) * r["scale"])
    return torch.tensor(idx_rows), torch.stack(w_rows)


def route_margins(h, router, correction, r):
    """[T]: how far each token's choice is from another one -- the smallest gap between a kept and a dropped group's score and
    between the last winner's and the best loser's choice score (inf where there is no alternative)"""
    n = router.shape[0]
    choice = torch.sigmoid(h @ router.T) + correction
    grp = r.get("groups") or {"count": 1, "keep": 1}
    count, keep, top = int(grp["count"]), int(grp["keep"]), int(r["top"])
    per = n // count
    out = []
    for t in range(h.shape[0]):
        c = choice[t].tolist()
        gs = sorted(((sum(sorted(c[g * per:(g + 1) * per], reverse=True)[:2]), g) for g in range(count)), key=lambda p: (-p[0], p[1]))
        gap = gs[keep - 1][0] - gs[keep][0] if keep < count else float("inf")
        allowed = sorted((c[e] for _, g in gs[:keep] for e in range(g * per, (g + 1) * per)), reverse=True)
        if top < len(allowed):
            gap = min(gap, allowed[top - 1] - allowed[top])
        out.append(gap)
    return torch.tensor(out, dtype=torch.float64)


def moe(h, W, m):
    """W: the feed-forward's tensors by short name (router, correction, e<i>.gate/up/down, shared.*)"""
    idx, wgt = route(h, W["router"], W["correction"], m["router"])
    lim = m["expert"]["limit"]
    y = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t].tolist()):
            y[t] += wgt[t, j] * clamped_expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], lim)[0]
    if m.get("shared"):
        sg = torch.sigmoid(h @ W["shared.sg"].T)                             # [T, 1]
        y = y + sg * clamped_expert(h, W["shared.gate"], W["shared.up"], W["shared.down"], m["shared"]["limit"])
    return y


# ------------------------------------------------------------------ the model
def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def first_blending_layer(cfg):
    for i, lc in enumerate(cfg["layers"]):
        if lc["type"] == "attention" and lc["mixer"].get("v_mix"):
            return i
    return None


def forward(cfg, weights, tokens, collect=None, margins=None):
    """logits [T, vocab] of one sequence; ``collect`` (a list) receives the stream after every layer, ``margins`` (a list) every
    routed layer's ``route_margins``"""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][torch.tensor(tokens, dtype=torch.int64)] * cfg["embedding"]["scale"]
    first, v_first = first_blending_layer(cfg), None
    for i, lc in enumerate(cfg["layers"]):
        h = layer_norm(x, weights[f"l{i}.norm1"], eps)
        W = sub(weights, f"l{i}.mix.")
        if lc["type"] == "wkv":
            y = wkv_mixer(h, W, lc["mixer"], eps)
        elif lc["type"] == "attention":
            y, v = attention_mixer(h, W, lc["mixer"], eps, None if i == first else v_first)
            if i == first:
                v_first = v
        else:
            raise ValueError(lc["type"])
        if lc.get("mlp") is not None:
            y = y + moe(h, sub(weights, f"l{i}.mlp."), lc["mlp"])
            if margins is not None:
                margins.append(route_margins(h, weights[f"l{i}.mlp.router"], weights[f"l{i}.mlp.correction"], lc["mlp"]["router"]))
        x = x + y
        if collect is not None:
            collect.append(x.clone())
    return layer_norm(x, weights["final.norm"], eps) @ weights["head"].T * cfg["logit_scale"]


# ------------------------------------------------------------------ random models for the tests
def random_config(width=48, vocab=61, kinds=("attention", "wkv", "attention", "wkv"), heads=6, kv_heads=3, dim=8, vdim=12, scale=0.3,
                  softcap=5.0, v_mix=(True, True), wkv_heads=3, wkv_dim=16, experts=6, groups=(3, 2), top=2, expert_ff=20, limit=1.5,
                  router_scale=1.7, shared_ff=12, shared_limit=0.9, mlp=None, emb_scale=2.5, logit_scale=0.5, eps=1e-5):
    """``v_mix``: one flag per attention layer; ``mlp``: one flag per layer (None: every layer has a feed-forward)"""
    layers, a = [], 0
    for i, kind in enumerate(kinds):
        if kind == "attention":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "v_mix": bool(v_mix[a])}
            a += 1
        else:
            mixer = {"heads": wkv_heads, "dim": wkv_dim}
        ff = None
        if mlp is None or mlp[i]:
            ff = {"kind": "moe", "expert": {"ff": expert_ff, "limit": limit},
                  "router": {"experts": experts, "top": top, "scale": router_scale}}
            if groups:
                ff["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
            if shared_ff:
                ff["shared"] = {"ff": shared_ff, "limit": shared_limit}
        layers.append({"type": kind, "mixer": mixer, "mlp": ff})
    return {"architecture": "Zubedra", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "layers": layers,
            "norm": {"eps": eps}, "logit_scale": logit_scale}


def random_weights(cfg, seed, rank=5, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, s=1.0):
        return torch.randn(o, i, generator=g) * (s / math.sqrt(i))

    def vec(n, mean=1.0, s=0.2):
        return mean + torch.randn(n, generator=g) * s

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g) * 0.5, "final.norm": vec(W), "head": mat(cfg["vocab"], W)}
    for i, lc in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = vec(W)
        if lc["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * D, W, 2.0), mat(G * D, W, 2.0), mat(G * Dv, W)
            w[p + "mix.q.norm"], w[p + "mix.k.norm"] = vec(H * D, 1.5, 0.5), vec(G * D, 1.5, 0.5)
            w[p + "mix.vmix"] = torch.rand((), generator=g) * 0.6 + 0.2
            w[p + "mix.sink"] = torch.randn(H, generator=g) * 1.5
            w[p + "mix.o"] = mat(W, H * Dv)
        else:
            H, D = m["heads"], m["dim"]
            for s in "rkvgw":
                w[p + "mix.mu." + s] = torch.rand(W, generator=g)
            for s in "rkvg":
                w[p + "mix." + s] = mat(H * D, W)
            w[p + "mix.w1"], w[p + "mix.w2"] = mat(rank, W), mat(H * D, rank, 2.0)
            w[p + "mix.w0"] = torch.randn(H * D, generator=g) * 1.0 - 1.5
            w[p + "mix.u"] = torch.randn(H, D, generator=g) * 0.5
            w[p + "mix.norm"] = vec(H * D)
            w[p + "mix.o"] = mat(W, H * D)
        ff = lc.get("mlp")
        if ff is not None:
            E, F = ff["router"]["experts"], ff["expert"]["ff"]
            for e in range(E):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = mat(F, W, 2.0), mat(F, W, 2.0), mat(W, F)
            w[p + "mlp.router"] = mat(E, W, 3.0)
            w[p + "mlp.correction"] = torch.randn(E, generator=g) * 0.4 - 0.3
            if ff.get("shared"):
                Fs = ff["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(Fs, W, 2.0), mat(Fs, W, 2.0), mat(W, Fs)
                w[p + "mlp.shared.sg"] = mat(1, W, 2.0)
    return {k: v.to(dtype) for k, v in w.items()}


# ------------------------------------------------------------------ pieces the kernel tests address directly
def sink_attention(q, k, v, scale, cap, sink, held=0, first=0):
    """q [S, H, D]: new tokens that sit at indices held .. held + S - 1 of k [L, G, D] / v [L, G, Dv]; indices below ``first`` do
    not exist (padding).  cap 0 = no cap, sink None = no sink.  Returns [S, H, Dv] (zeros for queries that do not exist)."""
    S, H, D = q.shape
    per = H // k.shape[1]
    out = torch.zeros(S, H, v.shape[2], dtype=q.dtype)
    for t in range(S):
        c = held + t
        if c < first:
            continue
        for hd in range(H):
            s = (k[first:c + 1, hd // per] @ q[t, hd]) * scale
            if cap:
                s = capped(s, cap)
            big = s.max() if sink is None else torch.maximum(s.max(), sink[hd])
            e = torch.exp(s - big)
            den = e.sum() + (0 if sink is None else torch.exp(sink[hd] - big))
            out[t, hd] = (e / den) @ v[first:c + 1, hd // per]
    return out


def greedy(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens
