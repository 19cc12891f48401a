"""`python bench.py --arch nikedra`: the Nikedra design at layer sizes of a real model (random weights), beside a Serotar -- the
framework's closest model: latent attention, sigmoid-routed experts, a depth-weighted average over a 32-bit residual stream -- of
equal width, depth, head count and expert geometry: prefill and decode throughput through the public API, and every kernel of
the design timed alone against its roofline next to the like kernel of the Serotar / Zafepel / Zubedra paths at the same sizes.

Timing and rooflines as in bench_mixers.py: CUDA events on the launching stream, 3 warm-up runs, median of 7, a 256 MB buffer
rewritten between runs; algorithmic bytes / the measured copy bandwidth, or algorithmic flops / the measured bf16 GEMM burst
rate (MEASURED_PEAKS.json).  One JSON line on stdout.
"""
import json
import os

from bench_mixers import NEW, PROMPT, ROOT, Timer, throughput
from bench_zubedra import SIZES as SEROTAR_SIZES, _fill, build_serotar

VOCAB, LAYERS = 32000, 8
EXPERTS, TOP = 8, 2
ORDER = ("channel_delta", "latent_attention", "channel_delta", "parallel")
MLPS = ("moe", "moe", "dense", "moe")
# per size: width, heads, head size, latent rank, rotated part, window = chunk, state-space heads / head size / state, low ranks, expert ff, dense ff
SIZES = {"2048": dict(width=2048, heads=16, dim=128, kv_rank=512, rot=64, span=1024, s_heads=32, s_vdim=64, state=128, rank=64, expert_ff=2816, ff=5632),
         "4096": dict(width=4096, heads=32, dim=128, kv_rank=512, rot=64, span=1024, s_heads=64, s_vdim=64, state=128, rank=128, expert_ff=1408, ff=11264)}
TAPS, CONV = 4, 4


def nikedra_config(size):
    z = SIZES[size]
    H, D = z["heads"], z["dim"]
    delta = {"heads": H, "kv_heads": H // 2, "dim": D, "vdim": D, "conv": CONV}
    latent = {"heads": H, "dim": D, "rot_dim": z["rot"], "vdim": D, "kv_rank": z["kv_rank"], "scale": (D + z["rot"]) ** -0.5,
              "mask": {"size": z["span"]}, "rot": {"base": 10000.0, "dims": z["rot"]}}
    par = {"left": {"heads": H, "kv_heads": H // 4, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": z["span"]},
                    "rot": {"base": 500000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}},
           "right": {"heads": z["s_heads"], "vdim": z["s_vdim"], "state": z["state"], "groups": 2, "norm_groups": 2, "conv": CONV}}
    mixers = {"channel_delta": delta, "latent_attention": latent, "parallel": par}
    mlps = {"dense": {"kind": "dense", "ff": z["ff"], "limit": 7.0},
            "moe": {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": EXPERTS, "top": TOP}}}
    layers = [{"type": ORDER[i % 4], "mixer": mixers[ORDER[i % 4]], "mlp": mlps[MLPS[i % 4]]} for i in range(LAYERS)]
    return {"architecture": "Nikedra", "vocab": VOCAB, "width": z["width"], "canon": {"taps": TAPS}, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
            "layers": layers, "low_ranks": {str(i): [z["rank"], z["rank"]] for i in range(LAYERS) if ORDER[i % 4] == "channel_delta"}}


def build_nikedra(dev, dtype, size="2048"):
    import torch
    from ipex_llm_b200.transformers.convert import _optimize_pre, _optimize_post
    from ipex_llm_b200.transformers.models.nikedra import NikedraConfig, NikedraForCausalLM, LatentRopeAttention
    with torch.device("meta"):
        model = NikedraForCausalLM(NikedraConfig(**nikedra_config(size)))
    _fill(model, dev, dtype, small={"A_log": -1.0, "canon": 0.1, "conv_weight": 0.3})
    for mod in model.modules():
        if isinstance(mod, LatentRopeAttention):              # the expansion has the block form the loader gives it
            H, D, Dr, Dv, R = mod.heads, mod.dim, mod.rot_dim, mod.vdim, mod.kv_rank
            uk = torch.randn(H * D, R, device=dev, dtype=dtype) * R ** -0.5
            uv = torch.randn(H * Dv, R, device=dev, dtype=dtype) * R ** -0.5
            mod.expand.weight = torch.nn.Parameter(mod.expansion(uk.cpu(), uv.cpu()).to(dev), requires_grad=False)
    for layer in model.model.layers:
        layer.dwa.data.fill_(1.0 / layer.dwa.numel())
    return _optimize_post(_optimize_pre(model.eval()))


def kernel_table(dev, dtype, peaks, timer, size, model):
    """each kernel of the design alone at the layer's sizes (prefill: 1 x PROMPT tokens; decode: 8 rows, one token each, PROMPT
    cached), each followed by the like kernel of the closest designs at the same sizes"""
    import torch
    from ipex_llm_b200.transformers.models import experts, mixer_ops as ops
    from ipex_llm_b200.transformers.models.nikedra import rotary_frequencies
    z = SIZES[size]
    W, H, D, R, Dr, SPAN = z["width"], z["heads"], z["dim"], z["kv_rank"], z["rot"], z["span"]
    SH, SP, SN, RANK, EF = z["s_heads"], z["s_vdim"], z["state"], z["rank"], z["expert_ff"]
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
    moe = next(l.mlp for l in model.model.layers if hasattr(l.mlp, "router"))
    for phase, B, S, held in (("prefill", 1, PROMPT, 0), ("decode", 8, 1, PROMPT)):
        N, L = B * S, held + S
        pad = torch.zeros(B, dtype=torch.int32, device=dev)
        # the stream: sum, depth average over 5 kept streams, two norms
        x, ya, yb = torch.randn(N, W, device=dev), rnd(N, W), torch.randn(N, W, device=dev)
        stack, coef, gain, wa, wb = torch.randn(5, N, W, device=dev), vec(5), vec(1), vec(W), vec(W)
        add("sum_residual_norms (4 earlier streams, 2 norms)", phase,
            timer(lambda: ops.sum_residual_norms(x, [ya, yb], dtype, 1e-5, stack=stack, index=4, coef=coef, gain1=gain, gain2=gain)),
            N * W * (8 + es + 4 + 4 * 4 + 4 + 2 * es))
        add("rms_residual (4 earlier streams, 1 norm)", phase, timer(lambda: ops.rms_residual(x, ya, gain, wa, 1e-5, dtype, stack=stack, index=4, coef=coef)),
            N * W * (8 + es + 4 * 4 + 4 + es), like_of="sum_residual_norms")
        a, b = rnd(N, W), rnd(N, W)
        add("rms_pair_sum", phase, timer(lambda: ops.rms_pair_sum(a, b, wa, wb, 1e-5, 0.5)), N * W * (2 * es + 4))
        add("rms_norm_rows", phase, timer(lambda: ops.rms_norm_rows(x, gain, None, 1e-5, dtype)), N * W * (4 + es), like_of="rms_pair_sum")
        # convolutions: on the mixer's input (h + conv(h)) and inside the mixers (bias, silu)
        h3, cw, tail = rnd(B, S, W), vec(W, TAPS), rnd(B, TAPS - 1, W)
        nxt = torch.empty_like(tail)
        add("short_conv (input: h + conv(h))", phase, timer(lambda: ops.short_conv(h3, 0, W, cw, None, tail, nxt, held, None, silu=False, add_input=True)),
            N * W * 2 * es)
        C = SH * SP + 4 * SN                                                                 # x | B | C of two groups
        cproj, cw2, cb, ctail = rnd(B, S, C + 2 * SH * SP), vec(C, CONV), rnd(C), rnd(B, CONV - 1, C)
        cnext = torch.empty_like(ctail)
        add("short_conv (bias, silu)", phase, timer(lambda: ops.short_conv(cproj, SH * SP, C, cw2, cb, ctail, cnext, held, None, silu=True)), N * C * 2 * es)
        add("short_conv_silu", phase, timer(lambda: ops.short_conv_silu(cproj, SH * SP, C, cw2, ctail, cnext, held, None)), N * C * 2 * es,
            like_of="short_conv")
        # channel delta rule against the delta rule with one decay per head
        G = H // 2
        Cd = 2 * G * D + H * D
        conv, proj, zz = rnd(B, S, Cd), rnd(B, S, Cd + 2 * H), rnd(B, S, H * D)
        A_log, dtb_c, dtb_h = rnd(H) - 1.0, rnd(H * D), rnd(H)
        state = torch.zeros(B, H, D, D, device=dev)
        rec_bytes = N * (Cd * es + H * D * 4) + 2 * B * H * D * D * 4
        add("channel_delta_rule", phase, timer(lambda: ops.channel_delta_rule(conv, G, H, D, D, proj, Cd, zz, A_log, dtb_c, state, held, None)),
            rec_bytes + N * H * D * es, flops=6.0 * N * H * D * D)
        add("gated_delta_rule", phase, timer(lambda: ops.gated_delta_rule(conv, G, H, D, D, proj, Cd, Cd + H, A_log, dtb_h, state, held, None)),
            rec_bytes, flops=6.0 * N * H * D * D, like_of="channel_delta_rule")
        # state-space scan against gated linear attention (a decay row per token) at the same state size
        sproj, sstate = rnd(B, S, SH), torch.zeros(B, SH, SN, SP, device=dev)
        sconv, sa, sb, sd = rnd(B, S, C), rnd(SH), rnd(SH), vec(SH)
        ss_bytes = N * (C * es + SH * SP * 4) + 2 * B * SH * SN * SP * 4
        add("state_space_scan", phase, timer(lambda: ops.state_space_scan(sconv, 2, SH, SN, SP, sproj, 0, sa, sb, sd, sstate, held, None)),
            ss_bytes, flops=4.0 * N * SH * SN * SP)
        gproj, gz = rnd(B, S, SH * (2 * SN + SP)), rnd(B, S, SH * SN)
        add("gated_linear_attention", phase, timer(lambda: ops.gated_linear_attention(gproj, SH, SN, SP, gz, 16.0, sstate, held, None)),
            N * (SH * (3 * SN + SP) * es + SH * SP * 4) + 2 * B * SH * SN * SP * 4, flops=4.0 * N * SH * SN * SP, like_of="state_space_scan")
        # norms behind the recurrences
        o, gate, nw = torch.randn(N, H, D, device=dev), rnd(N, H * D), vec(H * D)
        out = torch.empty(N, H * D, dtype=dtype, device=dev)
        add("gated_rms_norm (sigmoid gate)", phase, timer(lambda: ops.gated_rms_norm(o, gate, 0, nw[:D].contiguous(), 1e-5, out, 0, 1.0, sigmoid=True)),
            N * H * D * (4 + 2 * es))
        add("gated_rms_norm (gate first, 2 parts)", phase,
            timer(lambda: ops.gated_rms_norm(o.view(N, 2, H * D // 2), gate, 0, nw, 1e-5, out, 0, 1.0, gate_first=True)), N * H * D * (4 + 2 * es))
        add("gated_rms_norm (silu gate)", phase, timer(lambda: ops.gated_rms_norm(o, gate, 0, nw[:D].contiguous(), 1e-5, out, 0, 1.0)),
            N * H * D * (4 + 2 * es), like_of="gated_rms_norm")
        og = rnd(N, H * D)
        add("sigmoid_gate (per head)", phase, timer(lambda: ops.sigmoid_gate(og, proj.view(N, -1), 0, D)), N * H * D * 2 * es)
        add("sigmoid_gate (per channel)", phase, timer(lambda: ops.sigmoid_gate(og, gate, 0, 1)), N * H * D * 3 * es)
        add("silu_mul", phase, timer(lambda: ops.silu_mul(gate, H * D // 2)), N * H * D // 2 * 3 * es, like_of="sigmoid_gate")
        # attention: preparation (rotary, cache write) and the attention itself
        G4 = H // 4
        P = H * D + 2 * G4 * D
        aproj = rnd(B, S, P)
        ks, vs = rnd(B, G4, L, D), rnd(B, G4, L, D)
        freq, amp = rotary_frequencies({"base": 500000.0, "dims": Dr, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}})
        inv = torch.tensor(freq, dtype=torch.float64, device=dev)
        add("rope_qk_prepare (grouped heads, rescaled frequencies)", phase,
            timer(lambda: ops.rope_qk_prepare(aproj, 0, H * D, H * D + G4 * D, H, G4, D, D, D, 0, 0, Dr, inv, amp, ks, (G4 * L * D, D, L * D), vs,
                                              (G4 * L * D, D, L * D), held, 0, pad)), N * (H * D * 2 + G4 * D * 4) * es)
        qw, kw = vec(D), vec(D)
        add("window_qk_prepare (norm + rotary, 32-bit queries)", phase,
            timer(lambda: ops.window_qk_prepare(aproj, 0, H * D, H * D + G4 * D, H, G4, D, D, qw, kw, 1e-5, inv, Dr, ks, vs, L, held, 0, pad)),
            N * (P * es + H * D * 4 + 2 * G4 * D * es), like_of="rope_qk_prepare (grouped heads)")
        Dq, Rk = D + Dr, R + Dr
        lproj, store, lw = rnd(B, S, H * Dq + Rk), rnd(B, L, Rk), vec(R)
        add("rope_qk_prepare (latent: norm, shared rotated part)", phase,
            timer(lambda: ops.rope_qk_prepare(lproj, 0, H * Dq, 0, H, 1, Dq, Rk, 0, D, R, Dr, inv, 1.0, store, (L * Rk, Rk, 0), None, None, held, 0, pad,
                                              eps=1e-5, k_norm_w=lw, k_norm_cols=R)), N * (H * Dq * 2 + Rk * 2) * es)
        sp, sstore, sqw, scw = rnd(B, S, 768 + 512), rnd(B, L, 512), vec(768), vec(512)
        add("latent_prepare", phase, timer(lambda: ops.latent_prepare(sp, 0, 768, sqw, 768, 512, scw, 1e-5, sstore, held, 0, pad)),
            N * (768 + 512) * 2 * es, like_of="rope_qk_prepare (latent)")
        q = rnd(N, H * D)
        kview, vview = ks.permute(0, 2, 1, 3), vs.permute(0, 2, 1, 3)
        if S > 1:
            full = dict(flops=2.0 * (D + D) * (S * (S + 1) / 2) * H * B)
            n_chunks, rest = divmod(S, SPAN)
            in_chunk = n_chunks * SPAN * (SPAN + 1) / 2 + rest * (rest + 1) / 2
            in_window = sum(min(SPAN, t + 1) for t in range(S))
            add("softmax_attention (chunks)", phase, timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5, chunk=SPAN)),
                flops=2.0 * (D + D) * in_chunk * H * B)
            add("softmax_attention (plain)", phase, timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5)),
                like_of="softmax_attention (chunks) / (window)", **full)
            ql, kx, vx = rnd(N, H * Dq), rnd(B, L, H, Dq), rnd(B, L, H, D)
            add("softmax_attention (window, keys and values expanded from the latent)", phase,
                timer(lambda: ops.softmax_attention(ql, kx, vx, B, S, H, held, 0, pad, SPAN, Dq ** -0.5)), flops=2.0 * (Dq + D) * in_window * H * B)
        else:
            seen = min(SPAN, L)
            add("softmax_attention (chunk, decode)", phase, timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5, chunk=SPAN)),
                bytes_=B * G4 * (L % SPAN or SPAN) * 2 * D * es)
            add("softmax_attention (plain, decode)", phase, timer(lambda: ops.softmax_attention(q, kview, vview, B, S, H, held, 0, pad, 0, D ** -0.5)),
                bytes_=B * G4 * L * 2 * D * es, like_of="softmax_attention (chunk, decode)")
            qa, rows_ = rnd(N, H, Rk), store.unsqueeze(2)
            add("softmax_attention (window, decode on the latent cache itself)", phase,
                timer(lambda: ops.softmax_attention(qa, rows_, rows_[..., :R], B, S, H, held, 0, pad, SPAN, Dq ** -0.5)), bytes_=B * seen * Rk * es)
            q5, rows5 = rnd(N, H, 512), sstore.unsqueeze(2)
            add("softmax_attention (decode on a latent cache of 512, no window)", phase,
                timer(lambda: ops.softmax_attention(q5, rows5, rows5, B, S, H, held, 0, pad, 0, Dq ** -0.5)), bytes_=B * L * 512 * es,
                like_of="softmax_attention (window, decode on the latent cache itself)")
        # feed-forwards
        h = rnd(N, W)
        add("scored_router (sigmoid scores kept)", phase,
            timer(lambda: ops.scored_router(h, moe.router, None, 1, 1, TOP, sigmoid=True, group_top=1, renorm=False, scale=1.0)), N * W * es + EXPERTS * W * es)
        corr = rnd(EXPERTS)
        add("scored_router (groups, renormalised)", phase, timer(lambda: ops.scored_router(h, moe.router, corr, 2, 1, TOP, scale=1.5)),
            N * W * es + EXPERTS * W * es, like_of="scored_router")
        gu = rnd(N, 2 * EF)
        add("clamped_glu", phase, timer(lambda: ops.clamped_glu(gu, EF, 7.0)), N * EF * 3 * es)
        up = rnd(N, EF)
        add("gelu_erf", phase, timer(lambda: ops.gelu_erf(up)), N * EF * 2 * es)
        add("silu_mul", phase, timer(lambda: ops.silu_mul(gu, EF)), N * EF * 3 * es, like_of="clamped_glu / gelu_erf")
        idx, wgt, _ = ops.scored_router(h, moe.router, None, 1, 1, TOP, sigmoid=True, group_top=1, renorm=False, scale=1.0)
        if S == 1:
            tables = experts.address_tables(moe, dtype, dev)
            for n in (1, 8):
                distinct, pairs = int(idx[:n].unique().numel()), int(idx[:n].numel())
                add(f"moe_small, ungated gelu, weighted input ({n} rows, {pairs} expert calls on {distinct} experts)", phase,
                    timer(lambda: ops.moe_small(h[:n], idx[:n], wgt[:n], tables[0], tables[1], tables[3], EXPERTS, EXPERTS, None, ffs=tables[2],
                                                ungated_gelu=True, weight_input=True)), bytes_=distinct * 2 * EF * W * es)
        else:
            n_rows = N * TOP
            pos = torch.randperm(n_rows, device=dev).to(torch.int32).view(N, TOP)
            rows_ = rnd(n_rows, W)
            add("moe_scatter_scaled (weighted inputs in sorted order)", phase, timer(lambda: ops.moe_scatter_scaled(h, pos, idx, wgt, EXPERTS, n_rows)),
                N * W * (es + TOP * es))
            add("moe_combine (unweighted sum)", phase, timer(lambda: ops.moe_combine(rows_, pos, idx, None, h, None, EXPERTS, EXPERTS)),
                N * W * (TOP * es + 4))
            add("moe_combine (weighted sum)", phase, timer(lambda: ops.moe_combine(rows_, pos, idx, wgt, h, None, EXPERTS, EXPERTS)),
                N * W * (TOP * es + 4), like_of="moe_combine (unweighted sum) / moe_scatter_scaled")
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
    out = {"arch": "nikedra", "dtype": "bf16", "data": "synthetic (random weights)",
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": src},
           "config": {"sizes": SIZES, "layers": LAYERS, "layer_order": list(ORDER), "feed_forwards": list(MLPS), "experts": EXPERTS, "top": TOP,
                      "input_taps": TAPS, "mixer_taps": CONV, "vocab": VOCAB, "prompt": PROMPT, "new_tokens": NEW,
                      "cache": "256 MB rewritten between timed runs"}}
    out["kernels"] = []
    sizes = [s for s in SIZES if not getattr(args, "sizes", None) or s in args.sizes.split(",")]
    for size in sizes:
        model = build_nikedra(dev, dtype, size)
        out["nikedra_" + size] = [throughput(model, dev, timer, b) for b in (1, 8)]
        out["nikedra_recorded_step_failed"] = model.__dict__.get("_b200_state_graph_failed")
        out["kernels"] += kernel_table(dev, dtype, peaks, timer, size, model)
        model.__dict__.pop("_b200_state_graphs", None)
        del model
        torch.cuda.empty_cache()
        if not args.no_compare and size in SEROTAR_SIZES:
            other = build_serotar(dev, dtype, size)
            out["serotar_equal_size_" + size] = [throughput(other, dev, timer, b) for b in (1, 8)]
            other.__dict__.pop("_b200_state_graphs", None)
            del other
            torch.cuda.empty_cache()
    out["serotar_equal_size_note"] = "bf16, same width / layers / heads / experts / top / expert sizes (plus a shared expert); latent ranks 768 / 512"
    print(json.dumps(out))
