"""The Zubedra design in the framework against the plain statements of tests/zubedra_oracle.py (float64).

CPU tests cover what needs no kernel: the configuration reader, the checkpoint's name map and the merged projections, the
registry, the state cache's bookkeeping for a layer that keeps a matrix state and the previous token's input, the oracle's router
against a brute-force statement.  GPU tests run the kernels (there is no CPU path): every mechanism alone on odd sizes (layer norm
fused with the residual update, token shift, the recurrence in its few-token and its pipelined form with carried state, the
whole-projection query / key norm with value blending, capped scores and sinks in all three attention kernels, the router with
negative choice scores and groups decided by their second-best member, the clamped experts on both paths), whole prompts against
token-by-token decoding and against portions down to two tokens, unequal batches against each request alone, rows leaving a
batch, storage that grows past its first block, long decoding, greedy generation through ``generate()`` and the step's cache
used again by other requests.
"""
import json
import math
import os

import pytest
import torch

import zubedra_oracle as O

F64 = torch.float64


# ------------------------------------------------------------------ helpers
def save_checkpoint(cfg, weights, folder):
    """config.json + model.safetensors (8-byte header length, JSON header, raw data)"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32"}
    header, blobs, off = {}, [], 0
    for k, v in weights.items():
        raw = v.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        header[k] = {"dtype": names[v.dtype], "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    h = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(len(h).to_bytes(8, "little"))
        f.write(h)
        for b in blobs:
            f.write(b)


def load_framework(folder, dtype, device=None, **kw):
    from ipex_llm_b200.transformers import AutoModelForCausalLM
    model = AutoModelForCausalLM.from_pretrained(str(folder), torch_dtype=dtype, **kw)
    return model.to(device) if device is not None else model


def position_errors(got, want):
    """per position: rms over the vocabulary of the difference (mean removed) over the rms of the wanted logits"""
    d = got.to(F64).cpu() - want.to(F64)
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.to(F64).pow(2).mean().sqrt()


def assert_close(got, want, dtype, clear=None):
    """a 32-bit model must agree everywhere; a 16-bit one may flip a routing choice that is a close call in a few places
    (``clear``: the positions whose own choices are no close calls -- only those are held to the worst-case bound)"""
    e = position_errors(got, want).reshape(-1)
    if dtype == torch.float32:
        assert e.max() < 3e-5, e.max()
    else:
        assert torch.isfinite(got).all()
        worst = e.max() if clear is None else e[clear].max()
        assert e.median() < 0.03 and e.quantile(0.9) < 0.15 and worst < 0.6, (e.median(), e.quantile(0.9), worst)


def clear_choices(margins, gap=0.02):
    """[T] bool: no routed layer's choice at the position is closer than ``gap`` to another one"""
    return torch.stack(margins).min(0).values > gap


CONFIGS = {
    # nothing coincides: six query heads on three key/value heads, dim != vdim, head sizes that are no multiples of 8, two attention
    # layers that blend values, six experts in three groups of which two are kept, a shared expert with its own size and limit
    "odd": dict(),
    # everything optional absent, 1 or equal: one head everywhere, no groups, one expert per token, no shared expert, no blending,
    # scales of 1, a layer without feed-forward, the recurrence first
    "plain": dict(width=32, vocab=40, kinds=("wkv", "attention", "wkv"), heads=1, kv_heads=1, dim=16, vdim=16, scale=0.25, softcap=50.0,
                  v_mix=(False,), wkv_heads=1, wkv_dim=8, experts=4, groups=None, top=1, expert_ff=8, limit=7.0, router_scale=1.0, shared_ff=0,
                  mlp=(True, False, True), emb_scale=1.0, logit_scale=1.0),
    # head sizes that tile into 16s (the tensor-core attention of a 16-bit model); three attention layers of which the FIRST does not
    # blend: the second one's values are what the third blends in; all experts in one kept group of two
    "tile": dict(width=64, vocab=83, kinds=("attention", "attention", "wkv", "attention"), heads=4, kv_heads=2, dim=32, vdim=16, scale=0.18,
                 softcap=8.0, v_mix=(False, True, True), wkv_heads=2, wkv_dim=64, experts=8, groups=(2, 1), top=4, expert_ff=24, shared_ff=8),
    # a query projection wider than one pass of the norm kernel holds in registers (20 heads x 64), as many key/value heads as
    # query heads in no layer, one key/value head, sixteen experts in four groups of which two are kept, three per token, a wide
    # recurrent head, attention only behind the recurrences
    "wide": dict(width=72, vocab=300, kinds=("wkv", "wkv", "attention", "attention"), heads=20, kv_heads=1, dim=64, vdim=40, scale=0.05,
                 softcap=30.0, v_mix=(True, True), wkv_heads=1, wkv_dim=136, experts=16, groups=(4, 2), top=3, expert_ff=8, shared_ff=40,
                 mlp=(False, True, True, True), emb_scale=1.3, logit_scale=0.1),
}


def make(name, seed=0):
    cfg = O.random_config(**CONFIGS[name])
    return cfg, O.random_weights(cfg, seed + 1, rank=3 if name == "plain" else 5)


def w64(w):
    return {k: v.to(F64) for k, v in w.items()}


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


# ================================================================== CPU: configuration, loader, cache bookkeeping
def test_loader_maps_every_tensor_and_merges(tmp_path):
    from ipex_llm_b200.transformers.models.utils import read_safetensors
    cfg, w = make("odd")
    save_checkpoint(cfg, w, tmp_path)
    back = read_safetensors(os.path.join(tmp_path, "model.safetensors"))
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    model = load_framework(tmp_path, torch.bfloat16)
    assert type(model).__name__ == "ZubedraForCausalLM" and model.config.model_type == "zubedra"
    assert model.config.wkv_ranks == {"1": 5, "3": 5} and model.config.first_blending_layer() == 0
    at = model.model.layers[0].mixer
    assert at.in_proj.weight.shape == (6 * 8 + 3 * 8 + 3 * 12, cfg["width"]) and not hasattr(at, "q_proj")
    assert torch.equal(at.in_proj.weight[:48], w["l0.mix.q"]) and torch.equal(at.in_proj.weight[72:], w["l0.mix.v"])
    assert at.q_norm.weight.shape == (48,) and at.k_norm.weight.shape == (24,) and at.sink.shape == (6,) and at.vmix.shape == ()
    rec = model.model.layers[1].mixer
    assert rec.mu.shape == (5, cfg["width"]) and torch.equal(rec.mu[3], w["l1.mix.mu.g"]) and torch.equal(rec.mu[4], w["l1.mix.mu.w"])
    assert rec.w1_proj.weight.shape == (5, cfg["width"]) and rec.w2_proj.weight.shape == (48, 5) and rec.u.shape == (3, 16)
    assert rec.rkvg.shape == (4, 48, cfg["width"]) and not hasattr(rec, "r_proj")
    assert torch.equal(rec.rkvg[0], w["l1.mix.r"]) and torch.equal(rec.rkvg[3], w["l1.mix.g"])
    moe = model.model.layers[1].mlp
    assert (moe.n_experts, moe.groups, moe.keep, moe.top, moe.scale, moe.limit) == (6, 3, 2, 2, 1.7, 1.5)
    assert torch.equal(moe.experts[4].gate_up.weight, torch.cat([w["l1.mlp.e4.gate"], w["l1.mlp.e4.up"]]))
    assert torch.equal(moe.shared.down.weight, w["l1.mlp.shared.down"]) and moe.shared.limit == 0.9 and moe.shared_gate.shape == (1, cfg["width"])
    # what the configuration does not have does not exist in the model either
    cfg2, w2 = make("plain")
    save_checkpoint(cfg2, w2, tmp_path / "plain")
    plain = load_framework(tmp_path / "plain", torch.float32)
    assert plain.model.layers[1].mlp is None and plain.model.layers[0].mlp.shared is None and plain.model.layers[0].mlp.groups == 1
    assert plain.config.first_blending_layer() is None and plain.config.wkv_ranks == {"0": 3, "2": 3}
    # a layer that blends nothing may come without a blending weight
    del w2["l1.mix.vmix"]
    save_checkpoint(cfg2, w2, tmp_path / "noblend")
    assert load_framework(tmp_path / "noblend", torch.float32).model.layers[1].mixer.vmix.item() == 0.0
    # a tensor of the wrong shape is refused, by name
    bad = dict(w)
    bad["l1.mlp.correction"] = torch.zeros(4, dtype=torch.bfloat16)
    save_checkpoint(cfg, bad, tmp_path / "bad")
    with pytest.raises(RuntimeError, match="correction"):
        load_framework(tmp_path / "bad", torch.bfloat16)


def test_registry_picks_the_design(tmp_path):
    from ipex_llm_b200.transformers.model import native_architecture
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Zubedra"}))
    assert native_architecture(tmp_path).endswith("models.zubedra")


def test_state_cache_bookkeeping():
    """a wkv layer keeps a matrix state and the previous token's input; an attention layer a store that is never trimmed"""
    from ipex_llm_b200.transformers import kv
    cache = kv.DynamicStateCache()
    cache.start(torch.tensor([[0, 1, 1], [1, 1, 1], [0, 0, 1]]), 3, 3, torch.device("cpu"))
    rec = cache.run_state(1).rec
    tail, nxt = rec.tails(3, 2, 4, torch.float32, torch.device("cpu"))
    assert tail.shape == (3, 1, 4) and tail.abs().sum() == 0 and cache.run_state(1).kv is None
    tail.copy_(torch.arange(3.0)[:, None, None].expand(3, 1, 4))
    m = rec.matrix(3, 2, 5, 5, torch.device("cpu"))
    m += torch.arange(3.0)[:, None, None, None]
    att = cache.run_state(0, window=0).kv
    assert isinstance(att, kv.WindowKVLayer) and att.window == 0
    k, v, held = att.slots(torch.empty(3, 2, 0, 4), torch.empty(3, 2, 0, 6), 3)
    assert held == 0 and k.shape[:2] == (3, 2) and k.shape[2] == att.capacity() >= 3 and v.shape[3] == 6
    k[:, :, :3] = torch.arange(3.0)[:, None, None, None]
    att.commit(3)
    cache.advance(3)
    for _ in range(40):                                                      # no window: nothing is ever dropped
        att.slots(torch.empty(3, 2, 0, 4), torch.empty(3, 2, 0, 6), 50)
        att.commit(50)
        cache.advance(50)
    assert att.get_seq_length() == 2003 and att.dropped == 0 and att.keys[1, 0, 0, 0] == 1
    cache.batch_select_indices([2, 0])
    assert cache.pad.tolist() == [2, 1] and rec.tail[:, 0, 0].tolist() == [2.0, 0.0] and rec.state[:, 0, 0, 0].tolist() == [2.0, 0.0]
    assert att.keys[:, 0, 0, 0].tolist() == [2.0, 0.0]
    address = rec.state.data_ptr()
    cache.restart()
    assert cache.seen == 0 and rec.state.abs().sum() == 0 and rec.tail.abs().sum() == 0 and rec.state.data_ptr() == address
    assert att.get_seq_length() == 0


def test_oracle_router_against_brute_force():
    g = torch.Generator().manual_seed(5)
    h, router = torch.randn(60, 12, generator=g, dtype=F64), torch.randn(12, 12, generator=g, dtype=F64)
    corr = torch.randn(12, generator=g, dtype=F64) * 0.3 - 2.0              # all choice scores negative
    r = {"experts": 12, "top": 3, "scale": 2.5, "groups": {"count": 4, "keep": 2}}
    chosen, weights = O.route(h, router, corr, r)
    second_decides = 0
    for t in range(60):
        s = torch.sigmoid(router @ h[t])
        c = (s + corr).tolist()
        pair_sum = lambda k: sum(sorted(c[3 * k:3 * k + 3])[-2:])
        gs = sorted(range(4), key=lambda k: -pair_sum(k))[:2]
        second_decides += set(gs) != set(sorted(range(4), key=lambda k: -max(c[3 * k:3 * k + 3]))[:2])
        allowed = [e for e in range(12) if e // 3 in gs]
        want = sorted(allowed, key=lambda e: -c[e])[:3]
        assert sorted(chosen[t].tolist()) == sorted(want)
        assert torch.allclose(weights[t], s[chosen[t]] / s[chosen[t]].sum() * 2.5)
    assert second_decides > 3                                               # ranking groups by their best member alone would differ


# ================================================================== GPU: each mechanism alone
@pytest.fixture(scope="module")
def mixers(cuda_device):
    from ipex_llm_b200.transformers.models import mixer_ops
    return mixer_ops


def _rand(shape, gen, dtype, device, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype).to(device)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,n", [(45, 5), (1024, 3), (1100, 4), (200, 300), (8200, 2), (1100, 100)])
def test_layer_norm_with_residual_update(mixers, cuda_device, dtype, width, n):
    """rows held in registers (few rows: up to 8192 wide, by blocks of 128 to 1024 threads) and the plain loop; both addends, one of them, none"""
    g = torch.Generator().manual_seed(width)
    eps = 1e-3
    x0 = torch.randn(n, width, generator=g) * 2 + 0.7
    ya, yb = _rand((n, width), g, dtype, cuda_device), _rand((n, width), g, torch.float32, cuda_device)
    w = _rand((width,), g, dtype, cuda_device) + 1.0
    tol = 2e-5 if dtype == torch.float32 else 0.05
    for a, b in ((ya, yb), (ya, None), (None, yb), (None, None)):
        x = x0.clone().to(cuda_device)
        h = mixers.layer_norm_residual(x, a, b, w, eps, dtype)
        new = x0.to(F64) + (0 if a is None else a.cpu().to(F64)) + (0 if b is None else b.cpu().to(F64))
        assert (x.cpu().to(F64) - new).abs().max() < 1e-5
        assert (h.cpu().to(F64) - O.layer_norm(new, w.cpu().to(F64), eps)).abs().max() < tol
    x = x0.clone().to(cuda_device)
    assert mixers.layer_norm_residual(x, ya, yb, None, eps, dtype, want_out=False) is None
    assert (x.cpu().to(F64) - (x0.to(F64) + ya.cpu().to(F64) + yb.cpu().to(F64))).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_in_portions_with_padding(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(3)
    B, T, C = 3, 9, 300
    pads = [0, 5, 8]
    h = _rand((B, T, C), g, dtype, cuda_device)
    mu = torch.rand(5, C, generator=g).to(dtype).to(cuda_device)
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    tail = torch.zeros(B, 1, C, dtype=dtype, device=cuda_device)
    nxt = torch.empty_like(tail)
    out, at = [], 0
    for n in (4, 1, 3, 1):                                                  # portions; the single tokens shift the tail in place
        part = h[:, at:at + n].contiguous()
        out.append(mixers.token_shift_mix(part, mu, tail, tail if n == 1 else nxt, at, pad if at == 0 else (pad if at < 8 else None)).view(5, B, n, C))
        if n > 1:
            tail.copy_(nxt)
        at += n
    got = torch.cat(out, dim=2).cpu().to(F64)
    tol = 1e-6 if dtype == torch.float32 else 0.02
    for b, p in enumerate(pads):
        hb = h[b, p:].cpu().to(F64)
        for m in range(5):
            assert (got[m, b, p:] - O.token_shift(hb, mu[m].cpu().to(F64))).abs().max() < tol
        assert got[:, b, :p].abs().sum() == 0
    assert torch.equal(tail[:, 0], h[:, -1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,sizes", [(3, 16, (70, 1, 5)), (2, 40, (1, 1, 33, 2)), (1, 136, (20, 3)), (2, 64, (129,)), (1, 8, (4, 4)), (40, 64, (36, 20))])
def test_wkv_recurrence_with_carried_state(mixers, cuda_device, dtype, H, D, sizes):
    """the few-token and the pipelined kernel, the state carried from call to call, a row whose first tokens are padding; the last
    case has more blocks than the GPU has SMs (the build of the kernel that shares an SM between two blocks)"""
    g = torch.Generator().manual_seed(H * D)
    B, T = 2, sum(sizes)
    pads = [0, min(3, sizes[0] - 1)]
    r, k, v = (_rand((B, T, H * D), g, dtype, cuda_device) for _ in range(3))
    z = _rand((B, T, H * D), g, dtype, cuda_device)
    w0, u = (_rand((H * D,), g, dtype, cuda_device) - 1.0), _rand((H, D), g, dtype, cuda_device, 0.5)
    state = torch.zeros(B, H, D, D, dtype=torch.float32, device=cuda_device)
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    out, at = [], 0
    for n in sizes:
        buf = torch.stack([t[:, at:at + n].reshape(B * n, H * D) for t in (r, k, v)]).contiguous()      # three tensors that follow one another
        o = mixers.wkv(buf[0], buf[1], buf[2], B, n, H, D, z[:, at:at + n].reshape(B * n, H * D).contiguous(), w0, u, state, at, pad if at == 0 else None)
        out.append(o)
        at += n
    got = torch.cat(out, dim=1).cpu().to(F64)
    tol = 2e-4 if dtype == torch.float32 else 2e-3                          # inputs are exact in both; the state is 32-bit
    for b, p in enumerate(pads):
        f = lambda t: t[b, p:].cpu().to(F64).view(T - p, H, D)
        w = torch.exp(-torch.exp(f(z) + w0.cpu().to(F64).view(H, D)))
        want = O.wkv_scan(f(r), f(k), f(v), w, u.cpu().to(F64))
        assert ((got[b, p:] - want).abs() / (1 + want.abs())).max() < tol
        assert got[b, :p].abs().sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_weight_per_head(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(9)
    n, H, D = 7, 3, 20
    o = torch.randn(n, H, D, generator=g).to(cuda_device)
    gate = _rand((n, H * D + 4), g, dtype, cuda_device)
    w = _rand((H * D,), g, dtype, cuda_device) + 1.0
    out = torch.empty(n, H * D, dtype=dtype, device=cuda_device)
    mixers.gated_rms_norm(o, gate, 4, w, 1e-3, out, 0, 1.0)
    gt = gate[:, 4:].cpu().to(F64)
    want = O.unit_rms(o.cpu().to(F64), 1e-3).reshape(n, H * D) * w.cpu().to(F64) * gt * torch.sigmoid(gt)
    assert (out.cpu().to(F64) - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.05)
    shared = torch.empty_like(out)
    mixers.gated_rms_norm(o, gate, 4, w[:D].contiguous(), 1e-3, shared, 0, 1.0)           # one vector for every head still works
    want = O.unit_rms(o.cpu().to(F64), 1e-3).reshape(n, H * D) * w[:D].cpu().to(F64).repeat(H) * gt * torch.sigmoid(gt)
    assert (shared.cpu().to(F64) - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.05)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv", [(6, 3, 8, 12), (20, 1, 64, 40), (1, 1, 5, 3), (3, 1, 3000, 8)])
def test_whole_projection_norm_blend_and_cache_write(mixers, cuda_device, dtype, H, G, D, Dv):
    g = torch.Generator().manual_seed(H)
    B, S, held, cap, eps = 2, 3, 4, 9, 1e-4
    off_k, off_v = 2 + H * D, 2 + H * D + G * D + 1
    proj = _rand((B, S, off_v + G * Dv + 3), g, dtype, cuda_device, 2.0)
    other = _rand((B * S, G * Dv + 5), g, dtype, cuda_device)[:, 5:]
    qw, kw = _rand((H * D,), g, dtype, cuda_device) + 1, _rand((G * D,), g, dtype, cuda_device) + 1
    lam = torch.tensor(0.3).to(dtype).to(cuda_device)
    pad = torch.tensor([0, 6], dtype=torch.int32, device=cuda_device)       # row 1: slots 4, 5 are padding, slot 6 is its first token
    p = proj.cpu().to(F64)
    tol = 1e-5 if dtype == torch.float32 else 0.04
    want_q = O.unit_rms(p[..., 2:2 + H * D], eps) * qw.cpu().to(F64)
    want_k = O.unit_rms(p[..., off_k:off_k + G * D], eps) * kw.cpu().to(F64)
    for v_other in (None, other):
        ks = torch.full((B, G, cap, D), 9.0, dtype=dtype, device=cuda_device)
        vs = torch.full((B, G, cap, Dv), 9.0, dtype=dtype, device=cuda_device)
        q = mixers.wide_qkv_prepare(proj, 2, off_k, off_v, H, G, D, Dv, qw, kw, eps, v_other, lam, ks, vs, cap, held, 0, pad)
        want_v = p[..., off_v:off_v + G * Dv]
        if v_other is not None:
            l64 = lam.cpu().to(F64)
            want_v = (1 - l64) * want_v + l64 * other.cpu().to(F64).view(B, S, -1)
        assert (q.view(B, S, -1)[0].cpu().to(F64) - want_q[0]).abs().max() < tol
        got_k = ks[:, :, held:held + S].permute(0, 2, 1, 3).reshape(B, S, -1).cpu().to(F64)
        got_v = vs[:, :, held:held + S].permute(0, 2, 1, 3).reshape(B, S, -1).cpu().to(F64)
        assert (got_k[0] - want_k[0]).abs().max() < tol and (got_v[0] - want_v[0]).abs().max() < tol
        assert got_k[1, :2].abs().max() == 0 and got_v[1, :2].abs().max() == 0              # padding
        assert (got_k[1, 2] - want_k[1, 2]).abs().max() < tol and (got_v[1, 2] - want_v[1, 2]).abs().max() < tol
        assert (ks[:, :, :held] == 9).all() and (ks[:, :, held + S:] == 9).all() and (vs[:, :, :held] == 9).all()


def _attention_case(g, B, S, held, H, G, D, Dv, dtype, device, extra=3):
    L = held + S
    q = _rand((B * S, H * D), g, dtype, device)
    kfull, vfull = _rand((B, L + extra, G, D + 8), g, dtype, device), _rand((B, L + extra, G, Dv + 16), g, dtype, device)
    return q, kfull[..., 8:], vfull[..., :Dv]


def _attention_want(q, k, v, B, S, held, H, scale, cap, sink, pads):
    D = k.shape[3]
    s64 = None if sink is None else sink.cpu().to(F64)
    return torch.stack([O.sink_attention(q.view(B, S, H, D)[b].cpu().to(F64), k[b].cpu().to(F64), v[b].cpu().to(F64), scale, cap, s64, held,
                                         pads[b]).reshape(S, -1) for b in range(B)]).reshape(B * S, -1)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,held,H,G,D,Dv,tc", [
    (torch.float32, 5, 0, 6, 2, 5, 7, False), (torch.float32, 1, 300, 4, 1, 24, 40, False), (torch.bfloat16, 1, 517, 3, 1, 64, 64, False),
    (torch.bfloat16, 40, 30, 4, 2, 32, 16, True), (torch.float16, 150, 0, 3, 1, 64, 48, True), (torch.bfloat16, 33, 200, 6, 2, 64, 48, True),
    (torch.bfloat16, 1, 700, 8, 2, 64, 128, True), (torch.bfloat16, 3, 130, 4, 1, 32, 256, True)])
def test_capped_scores_and_sinks_in_every_attention_kernel(mixers, cuda_device, dtype, S, held, H, G, D, Dv, tc):
    """the general kernel, the prompt kernel on the tensor cores (S >= 16) and the kernel that splits the keys of shared heads over
    blocks (few tokens, vdim 128 / 256): cap and sink together, each alone, neither"""
    g = torch.Generator().manual_seed(S * 100 + held)
    B = 2
    q, k, v = _attention_case(g, B, S, held, H, G, D, Dv, dtype, cuda_device)
    pads = [0, min(held + S - 1, 3)]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    sink = (torch.randn(H, generator=g) + math.log(held + S) + 1.0).to(dtype).to(cuda_device)      # about the weight of all keys together
    scale = 3.0 / D ** 0.5                                                  # scores of a few units: a cap of 2 bends most of them
    for cap, sk in ((2.0, sink), (0.0, sink), (2.0, None), (0.0, None)):
        got = mixers.softmax_attention(q, k, v, B, S, H, held, 0, pad, 0, scale, tensor_cores=tc, softcap=cap, sink=sk)
        want = _attention_want(q, k, v, B, S, held, H, scale, cap, sk, pads)
        assert (got.cpu().to(F64) - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.02), (cap, sk is None)
    # cap and sink matter here: leaving either out moves the result by far more than the tolerance
    full = _attention_want(q, k, v, B, S, held, H, scale, 2.0, sink, pads)
    assert (full - _attention_want(q, k, v, B, S, held, H, scale, 0.0, sink, pads)).abs().max() > 0.1 * full.abs().max()
    assert (full - _attention_want(q, k, v, B, S, held, H, scale, 2.0, None, pads)).abs().max() > 0.1 * full.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S", [(torch.float32, 1), (torch.float32, 40), (torch.bfloat16, 1), (torch.bfloat16, 40)])
def test_one_outstanding_key_or_the_sink_decides(mixers, cuda_device, dtype, S):
    """a key whose score dwarfs all others: the output is its value when it is visible and must not show it otherwise -- far back
    among hundreds, at the borders of the kernels' key tiles, in front of a row's first token, in the future.  Under a cap the
    same key only outweighs the others by e^cap; a sink far above every score takes all the weight and the output is zero."""
    g = torch.Generator().manual_seed(11)
    H, D, Dv, L = 2, 16, 16, 700
    held = L - S
    base_k, base_v = torch.randn(1, L + 8, 1, D, generator=g) * 0.1, torch.randn(1, L + 8, 1, Dv, generator=g)
    q = torch.randn(S, H * D, generator=g) * 0.1
    spike = torch.zeros(D)
    spike[3] = 40.0
    q = q + spike.repeat(H)[None] * 0.05                                   # q . spike key = 80 + noise

    def run(at, first=0, tc=False, cap=0.0, sink=None):
        k = base_k.clone()
        k[0, at, 0] = spike
        sk = None if sink is None else torch.tensor(sink).to(dtype).to(cuda_device)
        out = mixers.softmax_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device), base_v.to(dtype).to(cuda_device), 1, S, H, held, 0,
                                       torch.tensor([first], dtype=torch.int32, device=cuda_device), 0, 1.0, tensor_cores=tc, softcap=cap, sink=sk)
        return out.float().cpu().view(S, H, Dv)

    last = S - 1                                                            # the last query sits at storage index L - 1
    for tc in ([False, True] if (dtype != torch.float32 and S >= 16) else [False]):
        for at in (0, 1, 31, 32, 63, 64, 255, 256, 257, L - 2, L - 1):      # visible to the last query wherever it is
            assert (run(at, tc=tc, sink=[1.0, -2.0])[last] - base_v[0, at, 0]).abs().max() < 0.02, at
        assert (run(4, first=5, tc=tc)[last] - base_v[0, 4, 0]).abs().max() > 0.3             # in front of the row's first token
        assert (run(5, first=5, tc=tc)[last] - base_v[0, 5, 0]).abs().max() < 0.02            # the row's first token itself
        assert (run(L, tc=tc)[last] - base_v[0, L, 0]).abs().max() > 0.3                      # the future
        if S > 1:
            out = run(held + 20, tc=tc)
            assert (out[20] - base_v[0, held + 20, 0]).abs().max() < 0.02 and (out[19] - base_v[0, held + 20, 0]).abs().max() > 0.3
        # capped at 3 the key's weight is e^3 against ~700 weights near 1: the mean of the values dominates
        assert (run(300, tc=tc, cap=3.0)[last] - base_v[0, 300, 0]).abs().max() > 0.3
        # a sink of 200 against a best score of 80: all the weight is the sink's; head 1 has a harmless sink and still shows the key
        out = run(300, tc=tc, sink=[200.0, -200.0])[last]
        assert out[0].abs().max() < 1e-6 and (out[1] - base_v[0, 300, 0]).abs().max() < 0.02
        # a sink level with the key's score: half the weight each
        half = run(300, tc=tc, sink=[float(q[last, 3].to(dtype)) * 40.0, -200.0])[last, 0]
        assert (half - 0.5 * base_v[0, 300, 0]).abs().max() < 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_out,groups,keep,top,shift,w", [(9, 3, 2, 3, 0.0, 37), (12, 4, 2, 3, -3.0, 37), (8, 1, 1, 8, 0.0, 40), (10, 10, 3, 3, 0.0, 37),
                                                             (64, 8, 4, 6, -1.0, 37), (5, 1, 1, 1, 0.0, 37), (6, 3, 1, 2, 0.0, 37), (18, 2, 1, 2, -0.5, 88),
                                                             (8, 2, 1, 2, 0.0, 1100), (3, 1, 1, 2, 0.0, 4104), (40, 4, 2, 4, -0.5, 2048)])
def test_scored_router(mixers, cuda_device, dtype, n_out, groups, keep, top, shift, w):
    """the last three widths cut every row of the product into 2, 8 and 1 pieces (pieces of 552 + 548, of 520 with a short last one)"""
    g = torch.Generator().manual_seed(n_out)
    n = 50
    h, router = _rand((n, w), g, dtype, cuda_device), _rand((n_out, w), g, dtype, cuda_device, 2.4 / w ** 0.5)
    corr = (_rand((n_out,), g, dtype, cuda_device, 0.2) + shift).to(dtype)  # shift < 0: every choice score is negative
    gate_row = _rand((1, w), g, dtype, cuda_device, 2.4 / w ** 0.5)
    idx, wgt, gate = mixers.scored_router(h, router, corr, groups, keep, top, scale=1.7, gate_row=gate_row)
    r = {"top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    chosen, weights = O.route(h.cpu().to(F64), router.cpu().to(F64), corr.cpu().to(F64), r)
    assert torch.equal(idx.cpu().to(torch.int64).sort(1).values, chosen.sort(1).values)
    got = torch.zeros(n, n_out, dtype=F64).scatter_(1, idx.cpu().to(torch.int64), wgt.cpu().to(F64))
    want = torch.zeros(n, n_out, dtype=F64).scatter_(1, chosen, weights)
    assert (got - want).abs().max() < 1e-5                                  # the router is 32-bit whatever the dtype
    assert (gate.cpu().to(F64) - torch.sigmoid(h.cpu().to(F64) @ gate_row.cpu().to(F64).T)[:, 0]).abs().max() < 1e-5
    assert mixers.scored_router(h, router, corr, groups, keep, top)[2] is None
    # many tokens take smaller blocks: the same pieces added in the same order, so the same logits bit for bit
    many = torch.cat([h, h])
    idx2, wgt2, gate2 = mixers.scored_router(many, router, corr, groups, keep, top, scale=1.7, gate_row=gate_row)
    assert torch.equal(idx2[:n], idx) and torch.equal(wgt2[n:], wgt) and torch.equal(gate2[:n], gate)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_activation(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(6)
    gu = _rand((7, 26), g, dtype, cuda_device, 2.0)
    a, b = gu.cpu().to(F64)[:, :13].clamp(max=1.2), gu.cpu().to(F64)[:, 13:].clamp(-1.2, 1.2)
    want = a * torch.sigmoid(1.702 * a) * (b + 1)
    assert (gu[:, :13] > 1.2).any() and (gu[:, 13:] < -1.2).any() and (gu[:, :13] < -1.2).any()      # the gate has no lower limit
    assert ((mixers.clamped_glu(gu, 13, 1.2).cpu().to(F64) - want).abs() / (1 + want.abs())).max() < (1e-5 if dtype == torch.float32 else 0.03)


# ================================================================== GPU: the model
def build(tmp_path, name, dtype, device, seed=0, **kw):
    cfg, w = make(name, seed)
    folder = tmp_path / f"{name}{seed}"
    save_checkpoint(cfg, w, folder)
    return cfg, w64(w), load_framework(folder, dtype, device, **kw)


@torch.no_grad()
def run_portions(model, tokens, sizes, device):
    """one request fed in portions (the last size repeats); returns logits [T, V]"""
    ids = torch.tensor([tokens], device=device)
    cache, out, at, i = None, [], 0, 0
    while at < len(tokens):
        n = sizes[min(i, len(sizes) - 1)]
        o = model(input_ids=ids[:, at:at + n], past_key_values=cache, use_cache=True)
        cache = o.past_key_values
        out.append(o.logits[0])
        at, i = at + n, i + 1
    return torch.cat(out)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_decode_and_portions_against_the_oracle(tmp_path, cuda_device, name, dtype):
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    tokens = tokens_for(cfg, 75, 3)
    collect, margins = [], []
    want = O.forward(cfg, w, tokens, collect, margins)
    clear = clear_choices(margins)
    assert clear.sum() > 30
    model.collect_residual = []
    whole = run_portions(model, tokens, [len(tokens)], cuda_device)
    if dtype == torch.float32:                                              # the stream after every layer, too
        for got, ref in zip(model.collect_residual, collect):
            assert (got[0].cpu().to(F64) - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max())
    model.collect_residual = None
    assert_close(whole, want, dtype, clear)
    assert_close(run_portions(model, tokens, [40, 1], cuda_device), want, dtype, clear)            # a prompt, then token by token
    assert_close(run_portions(model, tokens, [1], cuda_device), want, dtype, clear)                # from the first token on
    for sizes in ([2], [3, 17, 2, 30], [20, 20, 19, 16], [1, 1, 40, 2]):
        assert_close(run_portions(model, tokens, sizes, cuda_device), want, dtype, clear)
    if dtype != torch.float32:                                              # the general attention kernel under a 16-bit model
        model.attention_tensor_cores = False
        assert_close(run_portions(model, tokens, [len(tokens)], cuda_device), want, dtype, clear)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,layer", [("odd", 1), ("wide", 2), ("plain", 0)])
def test_experts_few_tokens_and_many_tokens_agree(tmp_path, cuda_device, dtype, name, layer):
    """the host-free path (address tables) and the sorted path compute the same layer; both match the plain statement"""
    from ipex_llm_b200.transformers.models import experts
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    mlp, spec = model.model.layers[layer].mlp, cfg["layers"][layer]["mlp"]
    g = torch.Generator().manual_seed(8)
    h = _rand((20, cfg["width"]), g, dtype, cuda_device, 1.5)
    want = O.moe(h.cpu().to(F64), O.sub(w, f"l{layer}.mlp."), spec)
    few = model._experts(mlp, h, False)
    old, experts.MOE_SMALL_TOKENS = experts.MOE_SMALL_TOKENS, 0
    try:
        many = model._experts(mlp, h, False)
    finally:
        experts.MOE_SMALL_TOKENS = old
    tol = 3e-5 if dtype == torch.float32 else 0.08
    assert few.dtype == torch.float32 and (few.cpu().to(F64) - want).abs().max() < tol and (many.cpu().to(F64) - want).abs().max() < tol
    assert (few - many).abs().max() < (1e-5 if dtype == torch.float32 else 0.04)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "tile"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_matches_each_request_alone(tmp_path, cuda_device, name, dtype):
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    lens, extra = [1, 23, 50, 7], 6
    seqs = [tokens_for(cfg, n + extra, 20 + n) for n in lens]
    want = [O.forward(cfg, w, s) for s in seqs]
    width = max(lens)
    ids = torch.zeros(4, width, dtype=torch.int64)
    mask = torch.zeros(4, width, dtype=torch.int64)
    for b, (s, n) in enumerate(zip(seqs, lens)):
        ids[b, width - n:] = torch.tensor(s[:n])
        mask[b, width - n:] = 1
    with torch.no_grad():
        o = model(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), use_cache=True)
        cache = o.past_key_values
        for b, n in enumerate(lens):
            assert_close(o.logits[b, width - n:], want[b][:n], dtype)
        rows = [0, 1, 2, 3]
        for step in range(extra):
            if step == 2:                                                   # two requests end: their rows leave the batch
                cache.batch_select_indices(torch.tensor([3, 1]))
                rows = [3, 1]
            nxt = torch.tensor([[seqs[b][lens[b] + step]] for b in rows], device=cuda_device)
            o = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            for r, b in enumerate(rows):
                assert_close(o.logits[r], want[b][lens[b] + step:lens[b] + step + 1], dtype)


@pytest.mark.gpu
def test_long_decoding_through_growing_storage(tmp_path, cuda_device):
    """300 tokens one by one from a 5-token prompt: the key/value store outgrows its first block and moves, the recurrent state
    is carried 300 times"""
    cfg, w, model = build(tmp_path, "tile", torch.float32, cuda_device)
    tokens = tokens_for(cfg, 305, 9)
    want = O.forward(cfg, w, tokens)
    got = run_portions(model, tokens, [5, 1], cuda_device)
    assert_close(got, want, torch.float32)


@pytest.mark.gpu
def test_a_far_token_and_the_first_token_reach_the_last_logits(tmp_path, cuda_device):
    """changing one early token of a long prompt must change the last position's logits exactly as the plain statement says, in
    a prompt and when the tail is decoded token by token (attention sees it as a far key, the recurrence as old state)"""
    cfg, w, model = build(tmp_path, "odd", torch.float32, cuda_device)
    tokens = tokens_for(cfg, 260, 13)
    for at in (0, 1, 37):
        other = list(tokens)
        other[at] = (other[at] + 1) % cfg["vocab"]
        want_a, want_b = O.forward(cfg, w, tokens)[-1:], O.forward(cfg, w, other)[-1:]
        assert position_errors(want_a, want_b).max() > 1e-3                 # the early token matters
        for sizes in ([260], [200, 1]):
            assert position_errors(run_portions(model, other, sizes, cuda_device)[-1:], want_b).max() < 3e-5


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "plain"])
def test_greedy_generate_matches_the_oracle(tmp_path, cuda_device, name):
    cfg, w, model = build(tmp_path, name, torch.float32, cuda_device)
    prompt = tokens_for(cfg, 9, 4)
    want = O.greedy(cfg, w, prompt, 12)
    ids = torch.tensor([prompt], device=cuda_device)
    got = model.generate(ids, max_new_tokens=12, do_sample=False)
    assert model.__dict__.get("_b200_state_graph_failed") is None and model.__dict__.get("_b200_state_graphs")     # the recorded step ran
    assert got[0].tolist() == want
    # the step's cache serves other requests afterwards: a batch of two with padding, then the first request again
    other = tokens_for(cfg, 4, 5)
    want2 = O.greedy(cfg, w, other, 7)
    batch = torch.tensor([prompt, [0] * 5 + other], device=cuda_device)
    mask = torch.tensor([[1] * 9, [0] * 5 + [1] * 4], device=cuda_device)
    got2 = model.generate(batch, attention_mask=mask, max_new_tokens=7, do_sample=False)
    assert got2[0].tolist() == want[:16] and got2[1, 5:].tolist() == want2
    assert model.generate(ids, max_new_tokens=12, do_sample=False)[0].tolist() == want
    # sampling goes through transformers' loop on the same forward
    torch.manual_seed(0)
    sampled = model.generate(ids, max_new_tokens=5, do_sample=True, top_k=3)
    assert sampled.shape == (1, 14) and sampled[0, :9].tolist() == prompt


@pytest.mark.gpu
def test_recorded_step_of_a_16_bit_model_equals_the_eager_loop(tmp_path, cuda_device, monkeypatch):
    """a bf16 model whose decoding attention is the kernel that splits the keys of shared heads over blocks (8 heads on 2, values
    of 128): the replayed step reads the cache length from the device and must produce the tokens of the loop that passes it
    from the host; the recurrence's state and tail are updated in place by both"""
    cfg = O.random_config(width=64, vocab=70, kinds=("attention", "wkv", "attention"), heads=8, kv_heads=2, dim=16, vdim=128, scale=0.25, softcap=10.0,
                          wkv_heads=2, wkv_dim=32, experts=4, groups=(2, 1), top=2, expert_ff=16, shared_ff=16)
    w = O.random_weights(cfg, 5)
    save_checkpoint(cfg, w, tmp_path / "m")
    model = load_framework(tmp_path / "m", torch.bfloat16, cuda_device)
    from ipex_llm_b200.ggml.model import mixers_cpp
    assert mixers_cpp.lib().mixers_softmax_attention_workspace(mixers_cpp.dtype_code(torch.bfloat16), 2, 1, 8, 2, 16, 128) > 0
    prompts = torch.tensor([tokens_for(cfg, 70, 1), [0] * 30 + tokens_for(cfg, 40, 2)], device=cuda_device)
    mask = torch.tensor([[1] * 70, [0] * 30 + [1] * 40], device=cuda_device)
    replayed = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert model.__dict__.get("_b200_state_graph_failed") is None and model.__dict__.get("_b200_state_graphs")
    monkeypatch.setenv("IPEX_LLM_B200_DECODE_GRAPH", "0")
    eager = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert torch.equal(replayed, eager)
    # and both follow the plain statement as far as a 16-bit model can: the first new token of each row
    for b, n in ((0, 70), (1, 40)):
        want = O.forward(cfg, w64(w), prompts[b, 70 - n:].tolist())[-1]
        top2 = want.topk(2).values
        if top2[0] - top2[1] > 0.5:
            assert int(replayed[b, 70]) == int(want.argmax())
    # the same model against the oracle position by position, decoding through the split-key kernel
    tokens = tokens_for(cfg, 60, 7)
    margins = []
    want = O.forward(cfg, w64(w), tokens, None, margins)
    assert_close(run_portions(model, tokens, [30, 1], cuda_device), want, torch.bfloat16, clear_choices(margins))


@pytest.mark.gpu
def test_low_bit_conversion_runs_the_same_model(tmp_path, cuda_device, native_lib):
    """the projections are ordinary linears to the converter: a sym_int4 model answers close to the 16-bit one; its experts (no
    longer plain matrices) take the sorted path also for one token, the narrow decay projection stays a plain matrix"""
    from ipex_llm_b200.transformers.low_bit_linear import LowBitLinear
    from ipex_llm_b200.transformers.models import experts
    cfg = O.random_config(width=128, vocab=90, kinds=("attention", "wkv", "attention"), heads=2, kv_heads=1, dim=32, vdim=32, wkv_heads=2, wkv_dim=32,
                          experts=4, groups=None, top=2, expert_ff=64, shared_ff=64)
    w = O.random_weights(cfg, 3)
    save_checkpoint(cfg, w, tmp_path / "m")
    ref = load_framework(tmp_path / "m", torch.bfloat16, cuda_device)
    low = load_framework(tmp_path / "m", torch.bfloat16, None, load_in_low_bit="sym_int4").to(cuda_device)
    assert isinstance(low.model.layers[0].mixer.in_proj, LowBitLinear) and isinstance(low.model.layers[0].mlp.experts[0].down, LowBitLinear)
    assert isinstance(low.model.layers[1].mixer.r_proj, LowBitLinear) and type(low.model.layers[1].mixer.w2_proj) is torch.nn.Linear
    assert experts.address_tables(low.model.layers[0].mlp, torch.bfloat16, cuda_device) is None
    tokens = tokens_for(cfg, 30, 1)
    a = run_portions(ref, tokens, [30], cuda_device)
    b = run_portions(low, tokens, [25, 1], cuda_device)
    assert torch.isfinite(b).all() and position_errors(b, a.cpu().to(F64)).quantile(0.8) < 0.5
