"""`python bench.py --arch zubedra`: the Zubedra design at layer sizes of a real model (random weights), beside a Serotar -- the
framework's closest model: softmax attention without positions, grouped routing, a shared expert, a 32-bit residual stream -- of
equal width, depth, head count and expert geometry: prefill and decode throughput through the public API, and every kernel of
the design timed alone against its roofline next to the like kernel of the Serotar / Zafepel paths at the same sizes.

Timing and rooflines as in bench_mixers.py: CUDA events on the launching stream, 3 warm-up runs, median of 7, a 256 MB buffer
rewritten between runs; algorithmic bytes / the measured copy bandwidth, or algorithmic flops / the measured bf16 GEMM burst
rate (MEASURED_PEAKS.json).  One JSON line on stdout.
"""
import json
import math
import os

from bench_mixers import NEW, PROMPT, ROOT, Timer, throughput

VOCAB, LAYERS = 32000, 8
# two sets of layer sizes: (width, heads, kv_heads, dim, vdim, wkv heads, wkv dim, decay rank, expert ff, shared ff)
SIZES = {"2048": (2048, 16, 4, 128, 128, 32, 64, 64, 2816, 2816), "4096": (4096, 32, 8, 128, 128, 64, 64, 128, 1408, 2816)}
EXPERTS, TOP, GROUPS, KEEP = 8, 2, 2, 1


def zubedra_config(size):
    W, H, G, D, Dv, RH, RD, _, EF, SF = SIZES[size]
    att = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": D ** -0.5, "softcap": 30.0, "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": EF, "limit": 7.0}, "shared": {"ff": SF, "limit": 7.0},
           "router": {"experts": EXPERTS, "top": TOP, "scale": 1.5, "groups": {"count": GROUPS, "keep": KEEP}}}
    layers = [{"type": "attention" if i % 2 == 0 else "wkv", "mixer": att if i % 2 == 0 else {"heads": RH, "dim": RD}, "mlp": moe} for i in range(LAYERS)]
    return {"architecture": "Zubedra", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
            "layers": layers, "wkv_ranks": {str(i): SIZES[size][7] for i in range(1, LAYERS, 2)}}


def _fill(model, dev, dtype, ones=("weight",), small=()):
    import torch
    gen = torch.Generator(device=dev).manual_seed(0)
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is None:
                continue
            t = torch.empty(p.shape, device=dev, dtype=torch.float32)
            if name in small:
                t.fill_(small[name])
            elif p.dim() >= 2:
                t.normal_(0.0, 1.0 / math.sqrt(p.shape[-1]), generator=gen)
            elif name in ones:
                t.fill_(1.0)
            else:
                t.normal_(0.0, 0.1, generator=gen)
            mod._parameters[name] = torch.nn.Parameter(t.to(dtype), requires_grad=False)


def build_zubedra(dev, dtype, size="2048"):
    import torch
    from ipex_llm_b200.transformers.convert import _optimize_pre, _optimize_post
    from ipex_llm_b200.transformers.models.zubedra import ZubedraConfig, ZubedraForCausalLM
    with torch.device("meta"):
        model = ZubedraForCausalLM(ZubedraConfig(**zubedra_config(size)))
    _fill(model, dev, dtype, small={"w0": -1.0, "mu": 0.5, "vmix": 0.3})
    return _optimize_post(_optimize_pre(model.eval()))


def build_serotar(dev, dtype, size="2048"):
    """the closest existing design at the same width, depth, heads and experts (latent ranks as in its own bench)"""
    import torch
    from ipex_llm_b200.transformers.convert import _optimize_pre, _optimize_post
    from ipex_llm_b200.transformers.models.serotar import SerotarConfig, SerotarForCausalLM
    W, H, _, D, Dv, _, _, _, EF, SF = SIZES[size]
    mixer = {"heads": H, "dim": D, "vdim": Dv, "q_rank": 768, "kv_rank": 512, "scale": D ** -0.5}
    moe = {"kind": "moe", "expert": {"ff": EF}, "shared": {"ff": SF},
           "router": {"experts": EXPERTS, "identity": 0, "top": TOP, "groups": {"count": GROUPS, "keep": KEEP}}}
    cfg = {"architecture": "Serotar", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": moe} for _ in range(LAYERS)]}
    with torch.device("meta"):
        model = SerotarForCausalLM(SerotarConfig(**cfg))
    _fill(model, dev, dtype, ones=("weight", "ls1", "ls2"))
    for layer in model.model.layers:
        layer.dwa.data.fill_(1.0 / layer.dwa.numel())
    return _optimize_post(_optimize_pre(model.eval()))


def kernel_table(dev, dtype, peaks, timer, size, model):
    """each kernel of the design alone at the layer's sizes (prefill: 1 x PROMPT tokens; decode: 8 rows, one token each, PROMPT
    cached), each followed by the like kernel of the closest designs at the same sizes"""
    import torch
    from ipex_llm_b200.transformers.models import experts, mixer_ops as ops
    W, H, G, D, Dv, RH, RD, RANK, EF, SF = SIZES[size]
    hbm, tc = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"])
    es = torch.empty((), dtype=dtype).element_size()
    rows = []

    def add(name, phase, ms, bytes_=None, flops=None, like_of=None):
        r = {"size": size, "kernel": name, "phase": phase, "us": ms * 1e3}
        if bytes_ is not None:
            r.update(gbs=bytes_ / ms / 1e6, frac_hbm=bytes_ / ms / 1e6 / hbm)
        if flops is not None:
            r.update(tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tc)
        if like_of:
            r["like_of"] = like_of
        rows.append(r)

    rnd = lambda *s: torch.randn(*s, device=dev).to(dtype)                                  # noqa: E731
    vec = lambda *s: (torch.rand(*s, device=dev) + 0.5).to(dtype)                            # noqa: E731
    moe = model.model.layers[0].mlp
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N, L = B * S, held + S
        pad = torch.zeros(B, dtype=torch.int32, device=dev)
        x, ya, yb, w = torch.randn(N, W, device=dev), rnd(N, W), torch.randn(N, W, device=dev), vec(W)
        add("layer_norm_residual", phase, timer(lambda: ops.layer_norm_residual(x, ya, yb, w, 1e-5, dtype)), N * W * (12 + 2 * es))
        add("rms_residual", phase, timer(lambda: ops.rms_residual(x, ya, w[:1], w, 1e-5, dtype)), N * W * (8 + 2 * es), like_of="layer_norm_residual")
        # attention: preparation and the attention itself
        P = H * D + G * D + G * Dv
        proj, qw, kw, lam = rnd(B, S, P), vec(H * D), vec(G * D), vec(1)[0]
        other = rnd(N, G * Dv)
        ks, vs = rnd(B, G, L, D), rnd(B, G, L, Dv)
        add("wide_qkv_prepare (norm, blend, cache write)", phase,
            timer(lambda: ops.wide_qkv_prepare(proj, 0, H * D, H * D + G * D, H, G, D, Dv, qw, kw, 1e-5, other, lam, ks, vs, L, held, 0, pad)),
            N * (2 * H * D + 2 * G * D + 3 * G * Dv) * es)
        lp, store, lqw, lcw = rnd(B, S, 768 + 512), rnd(B, L, 512), vec(768), vec(512)
        add("latent_prepare", phase, timer(lambda: ops.latent_prepare(lp, 0, 768, lqw, 768, 512, lcw, 1e-5, store, held, 0, pad)),
            N * (768 + 512) * 2 * es, like_of="wide_qkv_prepare")
        q, sink = rnd(N, H * D), rnd(H)
        kview, vview = ks.permute(0, 2, 1, 3), vs.permute(0, 2, 1, 3)
        att = dict(flops=2.0 * (D + Dv) * (S * (S + 1) / 2) * H * B) if S > 1 else dict(bytes_=B * G * L * (D + Dv) * es)
        add("softmax_attention (cap + sink)", phase,
            timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5, softcap=30.0, sink=sink)), **att)
        add("softmax_attention (plain)", phase, timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5)),
            like_of="softmax_attention (cap + sink)", **att)
        # wkv: token shift, recurrence, output norm
        h3, mu, tail = rnd(B, S, W), vec(5, W), rnd(B, 1, W)
        nxt = torch.empty_like(tail)
        add("token_shift_mix (5 mixes)", phase, timer(lambda: ops.token_shift_mix(h3, mu, tail, nxt, held, None)), N * W * 6 * es)
        C = 3 * W
        cw, ctail = vec(C, 4), rnd(B, 3, C)
        cproj, cnext = rnd(B, S, C), torch.empty_like(ctail)
        add("short_conv_silu (4 taps)", phase, timer(lambda: ops.short_conv_silu(cproj, 0, C, cw, ctail, cnext, held, None)), N * C * 2 * es,
            like_of="token_shift_mix")
        HD = RH * RD
        rkv, z = rnd(3, N, HD), rnd(N, HD)
        w0, u = rnd(HD) - 1.0, rnd(RH, RD)
        state = torch.zeros(B, RH, RD, RD, device=dev)
        rec_bytes = N * HD * (4 * es + 4) + 2 * B * RH * RD * RD * 4
        add("wkv recurrence", phase, timer(lambda: ops.wkv(rkv[0], rkv[1], rkv[2], B, S, RH, RD, z, w0, u, state, held, None)), rec_bytes)
        gproj, gz = rnd(B, S, 3 * HD), rnd(B, S, HD)
        add("gated_linear_attention", phase, timer(lambda: ops.gated_linear_attention(gproj, RH, RD, RD, gz, 16.0, state, held, None)), rec_bytes,
            like_of="wkv recurrence")
        o, gate, nw = torch.randn(N, RH, RD, device=dev), rnd(N, HD), vec(HD)
        out = torch.empty(N, HD, dtype=dtype, device=dev)
        add("gated_rms_norm (weight per head)", phase, timer(lambda: ops.gated_rms_norm(o, gate, 0, nw, 1e-5, out, 0, 1.0)), N * HD * (4 + 2 * es))
        add("gated_rms_norm (one weight)", phase, timer(lambda: ops.gated_rms_norm(o, gate, 0, nw[:RD].contiguous(), 1e-5, out, 0, 1.0)),
            N * HD * (4 + 2 * es), like_of="gated_rms_norm (weight per head)")
        # feed-forward
        h = rnd(N, W)
        add("scored_router (+ shared gate)", phase,
            timer(lambda: ops.scored_router(h, moe.router, moe.correction, GROUPS, KEEP, TOP, scale=1.5, gate_row=moe.shared_gate)),
            N * W * es + (EXPERTS + 1) * W * es)
        add("grouped_router", phase, timer(lambda: ops.grouped_router(h, moe.router, moe.correction, GROUPS, KEEP, TOP)),
            N * W * es + EXPERTS * W * es, like_of="scored_router")
        gu = rnd(N, 2 * EF)
        add("clamped_glu", phase, timer(lambda: ops.clamped_glu(gu, EF, 7.0)), N * EF * 3 * es)
        add("silu_mul", phase, timer(lambda: ops.silu_mul(gu, EF)), N * EF * 3 * es, like_of="clamped_glu")
        idx, wgt, sg = ops.scored_router(h, moe.router, moe.correction, GROUPS, KEEP, TOP, scale=1.5, gate_row=moe.shared_gate)
        if S == 1:
            tables = experts.address_tables(moe, dtype, dev)
            for n in (1, 8):
                distinct, pairs = int(idx[:n].unique().numel()), int(idx[:n].numel())
                traffic = (distinct * 3 * EF + 3 * SF) * W * es
                add(f"moe_small, clamped + gated shared ({n} rows, {pairs} expert calls on {distinct} experts)", phase,
                    timer(lambda: ops.moe_small(h[:n], idx[:n], wgt[:n], tables[0], tables[1], tables[3], EXPERTS, EXPERTS, None, ffs=tables[2],
                                                always_on=True, always_w=sg[:n], clamped=True, limit=7.0, limit_always=7.0)), bytes_=traffic)
                add(f"moe_small, silu + shared ({n} rows)", phase,
                    timer(lambda: ops.moe_small(h[:n], idx[:n], wgt[:n], tables[0], tables[1], tables[3], EXPERTS, EXPERTS, None, ffs=tables[2],
                                                always_on=True)), bytes_=traffic, like_of="moe_small, clamped + gated shared")
        else:
            rows_ = rnd(N * TOP, W)
            pos = torch.randperm(N * TOP, device=dev).to(torch.int32)
            add("moe_combine (gated shared)", phase, timer(lambda: ops.moe_combine(rows_, pos, idx, wgt, h, h, EXPERTS, EXPERTS, shared_w=sg)),
                N * W * (TOP * es + 2 * es + 4))
            add("moe_combine", phase, timer(lambda: ops.moe_combine(rows_, pos, idx, wgt, h, h, EXPERTS, EXPERTS)), N * W * (TOP * es + 2 * es + 4),
                like_of="moe_combine (gated shared)")
    return rows


def run(args):
    import torch
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dtype = torch.bfloat16
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        src = "MEASURED_PEAKS.json"
    except (OSError, ValueError):
        peaks, src = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"
    timer = Timer(dev)
    out = {"arch": "zubedra", "dtype": "bf16", "data": "synthetic (random weights)",
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": src},
           "config": {"sizes": {k: dict(zip(("width", "heads", "kv_heads", "dim", "vdim", "wkv_heads", "wkv_dim", "decay_rank", "expert_ff", "shared_ff"), v))
                                for k, v in SIZES.items()},
                      "layers": LAYERS, "layer_order": "attention, wkv, ...", "experts": EXPERTS, "top": TOP, "groups": [GROUPS, KEEP], "vocab": VOCAB,
                      "prompt": PROMPT, "new_tokens": NEW, "cache": "256 MB rewritten between timed runs"}}
    out["kernels"] = []
    for size in SIZES:
        model = build_zubedra(dev, dtype, size)
        out["zubedra_" + size] = [throughput(model, dev, timer, b) for b in (1, 8)]
        out["zubedra_recorded_step_failed"] = model.__dict__.get("_b200_state_graph_failed")
        out["kernels"] += kernel_table(dev, dtype, peaks, timer, size, model)
        model.__dict__.pop("_b200_state_graphs", None)
        del model
        torch.cuda.empty_cache()
        if not args.no_compare:
            other = build_serotar(dev, dtype, size)
            out["serotar_equal_size_" + size] = [throughput(other, dev, timer, b) for b in (1, 8)]
            other.__dict__.pop("_b200_state_graphs", None)
            del other
            torch.cuda.empty_cache()
    out["serotar_equal_size_note"] = "bf16, same width / layers / heads / experts / top / expert sizes; latent ranks 768 / 512"
    print(json.dumps(out))
