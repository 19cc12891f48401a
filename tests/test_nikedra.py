"""The Nikedra design in the framework against the plain statements of tests/nikedra_oracle.py (float64).

CPU tests cover what needs no kernel: the configuration reader, the checkpoint's name map, the merged projections and the
expansion matrix of the latent attention, the registry, the rotary frequencies with their rescaling, the state cache's
bookkeeping for a layer with two convolution tails, and the oracle's masks against brute force.  GPU tests run the kernels (there
is no CPU path): every mechanism alone on odd sizes (the sum of mixer and feed-forward with the depth average and both scalar
norms, the input convolution in portions, both recurrences in their few-token and pipelined forms with carried state, the
rotary preparation with rescaled frequencies and the latent's norm, windows and chunks in all three attention kernels with one
outstanding key at every edge, the gates, the pair of width norms, the sigmoid router, input-weighted experts on both paths, the
clamped feed-forward with biases), then the model: whole prompts against token-by-token decoding and portions down to two
tokens, unequal batches against each request alone, rows leaving a batch, storage that grows and is used again, long decoding
across many windows and chunks, greedy generation through ``generate()`` and the trace runner's command line.
"""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import nikedra_oracle as O

F64 = torch.float64
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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


def clear_choices(margins, n, gap=0.02):
    """[T] bool: no routed layer's choice at the position is closer than ``gap`` to another one"""
    return torch.stack(margins).min(0).values > gap if margins else torch.ones(n, dtype=torch.bool)


CONFIGS = {
    # nothing coincides: fewer key than query heads everywhere, dim != vdim, head sizes that are no multiples of 8, a rotated part
    # smaller than the head, two groups of state-space heads normalised in two parts, two experts per token, a limit below 1, a
    # layer without feed-forward, windows and chunks of a few tokens so that every prompt crosses many edges
    "odd": dict(),
    # everything 1 or equal or absent: one head everywhere, one group, one expert per token, one convolution tap on the mixer's
    # input, rotary on the whole head without rescaling, a limit of 1, logits unscaled, window and chunk of one token's reach
    # more than the prompt in one layer and of a single token in another
    "plain": dict(width=32, vocab=40, taps=1, order=("parallel", "latent_attention", "channel_delta", "latent_attention"),
                  mlps=("moe", None, "dense", "dense"), latent=dict(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=8, window=1, scale=1.0),
                  delta=dict(heads=1, kv_heads=1, dim=8, vdim=8, conv=2), left=dict(heads=1, kv_heads=1, dim=8, vdim=8, rot_dims=8, chunk=500, factor=0),
                  right=dict(heads=1, vdim=8, state=8, groups=1, norm_groups=1, conv=1), dense=dict(ff=16, limit=1.0), moe=dict(experts=3, top=1, ff=8),
                  logit_scale=1.0),
    # head sizes that tile into 16s (the tensor-core attention of a 16-bit model); a window and a chunk that are no multiples of the
    # kernels' key tiles; every expert chosen by every token
    "tile": dict(width=64, vocab=83, taps=2, order=("parallel", "latent_attention", "parallel", "channel_delta"), mlps=("moe", "dense", "moe", None),
                 latent=dict(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=48, window=40, scale=0.15),
                 delta=dict(heads=4, kv_heads=1, dim=32, vdim=64, conv=3), left=dict(heads=4, kv_heads=2, dim=32, vdim=16, rot_dims=16, chunk=24, scale=0.2),
                 right=dict(heads=4, vdim=32, state=64, groups=4, norm_groups=4, conv=4), dense=dict(ff=40, limit=2.5), moe=dict(experts=3, top=3, ff=24)),
    # a latent of 128 numbers under eight heads (decoding takes the kernel that splits the keys of a shared head over blocks),
    # a window and a chunk longer than a key tile, a recurrent head wider than a warp, many small experts
    "wide": dict(width=72, vocab=300, taps=4, order=("channel_delta", "latent_attention", "parallel"), mlps=("moe", "moe", "dense"),
                 latent=dict(heads=8, dim=64, rot_dim=32, vdim=48, kv_rank=128, window=70, scale=0.1, base=10000.0),
                 delta=dict(heads=2, kv_heads=2, dim=136, vdim=24, conv=2), left=dict(heads=8, kv_heads=1, dim=64, vdim=128, rot_dims=32, chunk=90, scale=0.12,
                                                                                      factor=16.0, original=64, fast=8.0, slow=2.0, base=1000.0),
                 right=dict(heads=3, vdim=40, state=16, groups=3, norm_groups=1, conv=3), dense=dict(ff=100, limit=1.3), moe=dict(experts=16, top=4, ff=8),
                 logit_scale=0.1),
    # head sizes of a served model on a narrow stream: heads of 128, a latent of 512 + 64 rotated (decoding reads cache rows of 576 as
    # keys and their first 512 numbers as values in the split-key kernel), a state of 128 x 64
    "full": dict(width=128, vocab=97, taps=4, order=("latent_attention", "channel_delta", "parallel"), mlps=("moe", "dense", "moe"),
                 latent=dict(heads=4, dim=128, rot_dim=64, vdim=128, kv_rank=512, window=50, scale=0.07, base=10000.0),
                 delta=dict(heads=4, kv_heads=2, dim=128, vdim=128, conv=4), left=dict(heads=8, kv_heads=2, dim=128, vdim=128, rot_dims=64, chunk=32, scale=0.09,
                                                                                      factor=8.0, original=64, fast=16.0, slow=1.0, base=500000.0),
                 right=dict(heads=4, vdim=64, state=128, groups=2, norm_groups=2, conv=4), dense=dict(ff=256, limit=7.0), moe=dict(experts=3, top=2, ff=64)),
    # sizes that are multiples of nothing: rows that start off every vector boundary, five heads, three norm parts of five channels,
    # a window of three and a chunk of two tokens, every expert for every token, both low ranks of one
    "awkward": dict(width=52, vocab=37, taps=2, order=("parallel", "channel_delta", "latent_attention"), mlps=("moe", "dense", "moe"),
                    latent=dict(heads=5, dim=6, rot_dim=2, vdim=3, kv_rank=7, window=3, scale=0.5), delta=dict(heads=3, kv_heads=3, dim=5, vdim=9, conv=3),
                    left=dict(heads=3, kv_heads=1, dim=6, vdim=5, rot_dims=2, chunk=2, scale=0.4), right=dict(heads=5, vdim=3, state=7, groups=5, norm_groups=3, conv=2),
                    dense=dict(ff=25, limit=0.4), moe=dict(experts=2, top=2, ff=11), logit_scale=2.0),
}


def make(name, seed=0):
    cfg = O.random_config(**CONFIGS[name])
    return cfg, O.random_weights(cfg, seed + 1, ranks={"plain": (3, 1), "awkward": (1, 1)}.get(name, (5, 3)))


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
    assert type(model).__name__ == "NikedraForCausalLM" and model.config.model_type == "nikedra"
    assert model.config.low_ranks == {"1": [5, 3], "3": [5, 3]} and model.config.canon_taps == 3
    W = cfg["width"]
    layers = model.model.layers
    assert [l.kind for l in layers] == ["latent_attention", "channel_delta", "parallel", "channel_delta"]
    assert all(l.norm1.weight.shape == () and l.canon.shape == (W, 3) and l.dwa.shape == (i + 2,) for i, l in enumerate(layers))
    assert layers[2].mlp is None and not hasattr(layers[2], "norm2") and layers[0].norm2.weight.shape == ()
    la = layers[0].mixer                                                    # 3 heads of 10 + 6, latent 12 + 6 rotated, gate 3 x 14
    assert la.in_proj.weight.shape == (3 * 16 + 18 + 42, W) and not hasattr(la, "q_proj") and (la.window, la.rotary.dims) == (9, 6)
    assert torch.equal(la.in_proj.weight[:48], w["l0.mix.q"]) and torch.equal(la.in_proj.weight[48:66], w["l0.mix.dkv"])
    ex = la.expand.weight
    assert ex.shape == (3 * 16 + 3 * 14, 18)
    assert torch.equal(ex[16:26, :12], w["l0.mix.uk"][10:20]) and torch.equal(ex[26:32, 12:], torch.eye(6, dtype=ex.dtype)) and ex[16:26, 12:].abs().sum() == 0
    assert torch.equal(ex[48:, :12], w["l0.mix.uv"]) and ex[48:, 12:].abs().sum() == 0
    cd = layers[1].mixer                                                    # q, k: 2 x 12; v: 4 x 10; beta 4; ranks 5 and 3
    assert cd.in_proj.weight.shape == (24 + 24 + 40 + 4 + 5 + 3, W) and cd.conv_weight.shape == (88, 4) and cd.dt_bias.shape == (48,)
    assert torch.equal(cd.conv_weight[24:48], w["l1.mix.k.conv"]) and torch.equal(cd.in_proj.weight[92:97], w["l1.mix.a1"])
    assert cd.a2_proj.weight.shape == (48, 5) and cd.g2_proj.weight.shape == (40, 3) and cd.norm.weight.shape == (10,)
    pm = layers[2].mixer                                                    # left 72 + 24 + 20 + 6; right 2 x 24 + 2 x 20 + 4
    assert pm.in_proj.weight.shape == (122 + 92, W) and not hasattr(pm.left, "q_proj") and not hasattr(pm.right, "in_proj")
    assert torch.equal(pm.in_proj.weight[116:122], w["l2.mix.left.g"]) and torch.equal(pm.in_proj.weight[122:], w["l2.mix.right.in"])
    assert (pm.left.chunk, pm.left.rotary.dims, pm.right.conv_channels, pm.right.norm_groups) == (7, 8, 64, 2)
    assert pm.left.rotary.amp == pytest.approx(0.1 * math.log(4.0) + 1.0) and la.rotary.amp == 1.0
    dense, moe = layers[0].mlp, layers[1].mlp
    assert dense.limit == 0.7 and torch.equal(dense.gate_up.weight, torch.cat([w["l0.mlp.gate"], w["l0.mlp.up"]]))
    assert torch.equal(dense.gate_up.bias, torch.cat([w["l0.mlp.gate.b"], w["l0.mlp.up.b"]])) and torch.equal(dense.down.bias, w["l0.mlp.down.b"])
    assert (moe.n_experts, moe.top) == (5, 2) and torch.equal(moe.experts[4].up.weight, w["l1.mlp.e4.up"]) and moe.router.shape == (5, W)
    # a missing tensor and a tensor of the wrong shape are refused, by name
    for name, bad in (("l2.mix.right.conv.b", None), ("l1.mix.dt_bias", torch.zeros(4, dtype=torch.bfloat16))):
        broken = dict(w)
        if bad is None:
            del broken[name]
        else:
            broken[name] = bad
        save_checkpoint(cfg, broken, tmp_path / "bad")
        with pytest.raises(RuntimeError, match=name.split(".")[-1]):
            load_framework(tmp_path / "bad", torch.bfloat16)


def test_registry_picks_the_design(tmp_path):
    from ipex_llm_b200.transformers.model import native_architecture
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nikedra"}))
    assert native_architecture(tmp_path).endswith("models.nikedra")


def test_rotary_frequencies_between_the_bands():
    """pairs that turn often within the original length keep their frequency, slow ones are divided by the factor, the ones
    between are blended by their index; the framework's table against the plain statement, and both against hand values"""
    from ipex_llm_b200.transformers.models.nikedra import rotary_frequencies
    rot = {"base": 1000.0, "dims": 32, "scaling": {"factor": 16.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    freq, amp = rotary_frequencies(rot)
    want, want_amp = O.rotary_frequencies(rot)
    assert torch.allclose(torch.tensor(freq, dtype=F64), want, rtol=1e-14) and amp == pytest.approx(want_amp)
    plain = [1000.0 ** (-2.0 * i / 32) for i in range(16)]
    lo = math.floor(32 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(1000.0)))         # 0
    hi = math.ceil(32 * math.log(64 / (2 * math.pi * 2.0)) / (2 * math.log(1000.0)))          # 4
    assert (lo, hi) == (0, 4) and freq[0] == plain[0] and freq[2] == pytest.approx(plain[2] * (0.5 / 16 + 0.5))
    assert all(freq[i] == pytest.approx(plain[i] / 16) for i in range(4, 16))
    # without a scaling block the frequencies are the plain ones and the amplitude is 1
    assert rotary_frequencies({"base": 1000.0, "dims": 32}) == (plain, 1.0)


def test_oracle_masks_against_brute_force():
    for T, size in ((11, 1), (11, 4), (11, 11), (11, 30)):
        win, chk = O.window_mask(T, size), O.chunk_mask(T, size)
        for i in range(T):
            for j in range(T):
                assert bool(win[i, j]) == (0 <= i - j < size) and bool(chk[i, j]) == (j <= i and i // size == j // size)


def test_state_cache_keeps_two_tails_per_layer():
    """the input convolution's tail and the mixer's own, the matrix state, and a latent store or key/value store beside them"""
    from ipex_llm_b200.transformers import kv
    cache = kv.DynamicStateCache()
    cache.start(torch.tensor([[0, 1, 1], [1, 1, 1], [0, 0, 1]]), 3, 3, torch.device("cpu"))
    st = cache.run_state(0, latent=True)
    assert isinstance(st.kv, kv.LatentKVLayer) and isinstance(cache.run_state(1, window=0).kv, kv.WindowKVLayer) and cache.run_state(2).kv is None
    a, a_next = st.rec.tails(3, 4, 5, torch.float32, torch.device("cpu"), key="input")
    b, _ = st.rec.tails(3, 2, 7, torch.float32, torch.device("cpu"), key="mixer")
    assert a.shape == (3, 3, 5) and b.shape == (3, 1, 7) and a.data_ptr() != a_next.data_ptr()
    assert st.rec.tails(3, 4, 5, torch.float32, torch.device("cpu"), key="input")[0].data_ptr() == a.data_ptr()
    a += torch.arange(3.0)[:, None, None]
    b += 10 * torch.arange(3.0)[:, None, None]
    store, held = st.kv.slots(3, 6, 3, torch.float32, torch.device("cpu"))
    store[:, :3] = torch.arange(3.0)[:, None, None]
    st.kv.commit(3)
    cache.advance(3)
    cache.batch_select_indices([2, 0])
    a2, b2 = st.rec.tails(2, 4, 5, torch.float32, torch.device("cpu"), key="input")[0], st.rec.tails(2, 2, 7, torch.float32, torch.device("cpu"), key="mixer")[0]
    assert a2[:, 0, 0].tolist() == [2.0, 0.0] and b2[:, 0, 0].tolist() == [20.0, 0.0] and cache.pad.tolist() == [2, 1]
    assert st.kv.held()[:, 0, 0].tolist() == [2.0, 0.0] and st.kv.get_seq_length() == 3
    address = a2.data_ptr()
    cache.restart()
    assert cache.seen == 0 and a2.abs().sum() == 0 and b2.abs().sum() == 0 and st.kv.get_seq_length() == 0
    assert st.rec.tails(2, 4, 5, torch.float32, torch.device("cpu"), key="input")[0].data_ptr() == address


# ================================================================== GPU: each mechanism alone
@pytest.fixture(scope="module")
def mixers(cuda_device):
    from ipex_llm_b200.transformers.models import mixer_ops
    return mixer_ops


def _rand(shape, gen, dtype, device, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype).to(device)


def _c64(t):
    return t.cpu().to(F64)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,n", [(45, 5), (1100, 3), (352, 1500), (8200, 2), (2000, 70)])
def test_sum_two_norms_and_depth_average(mixers, cuda_device, dtype, width, n):
    """x + mixer + feed-forward, kept as a stream, replaced by the weighted sum of all streams so far, normalised twice with one
    number each -- rows in registers and the plain loop, with both addends, one, none; and the embedding's own norm in front"""
    g = torch.Generator().manual_seed(width)
    eps = 1e-3
    tol = 3e-5 if dtype == torch.float32 else 0.05
    streams = 4
    stack0 = torch.randn(streams, n, width, generator=g)
    x0 = torch.randn(n, width, generator=g) * 2 + 0.5
    ya, yb = _rand((n, width), g, dtype, cuda_device), _rand((n, width), g, torch.float32, cuda_device)
    coef = _rand((streams,), g, dtype, cuda_device) * 0.5
    g1, g2 = (torch.rand((), generator=g) + 0.5).to(dtype).to(cuda_device), (torch.rand((), generator=g) + 0.5).to(dtype).to(cuda_device)
    for ys in ([ya, yb], [ya, None], [None, yb], []):
        x, stack = x0.clone().to(cuda_device), stack0.clone().to(cuda_device)
        h1, h2 = mixers.sum_residual_norms(x, ys, dtype, eps, stack=stack, index=3, coef=coef, gain1=g1, gain2=g2)
        new = x0.to(F64) + sum(_c64(y) for y in ys if y is not None)
        assert (_c64(stack[3]) - new).abs().max() < 1e-5 and torch.equal(stack[:3].cpu(), stack0[:3])
        mixed = sum(_c64(coef)[j] * stack0[j].to(F64) for j in range(3)) + _c64(coef)[3] * new
        assert (_c64(x) - mixed).abs().max() < 1e-4
        assert (_c64(h1) - O.unit_rms(mixed, eps) * _c64(g1)).abs().max() < tol and (_c64(h2) - O.unit_rms(mixed, eps) * _c64(g2)).abs().max() < tol
    # the first stream: the embedding, normalised with its own number, is what is kept; no second norm asked for
    x, stack = x0.clone().to(cuda_device), torch.zeros(2, n, width, device=cuda_device)
    h1, h2 = mixers.sum_residual_norms(x, [], dtype, eps, pre_gain=g2, stack=stack, index=0, gain1=g1, gain2=None)
    emb = O.unit_rms(x0.to(F64), eps) * _c64(g2)
    assert h2 is None and (_c64(x) - emb).abs().max() < 1e-5 and (_c64(stack[0]) - emb).abs().max() < 1e-5
    assert (_c64(h1) - O.unit_rms(emb, eps) * _c64(g1)).abs().max() < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,bias,silu,add", [(4, False, False, True), (3, True, True, False), (1, False, False, True), (2, True, True, False),
                                                (1, True, True, False)])
def test_short_convolution_in_portions_with_padding(mixers, cuda_device, dtype, taps, bias, silu, add):
    """h + conv(h) on the mixer's input and silu(conv(.) + bias) inside a mixer: the tail carried from portion to portion (single
    tokens shift it in place), rows that start with padding, columns taken out of the middle of a wider projection"""
    g = torch.Generator().manual_seed(taps)
    B, T, C, off = 3, 12, 300, 5
    pads = [0, 3, 4]                                                        # padding only ever fills part of the first call
    proj = _rand((B, T, C + 9), g, dtype, cuda_device)
    w = _rand((C, taps), g, dtype, cuda_device, 0.6)
    bs = _rand((C,), g, dtype, cuda_device, 0.3) if bias else None
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    tail = torch.zeros(B, max(taps - 1, 1), C, dtype=dtype, device=cuda_device)
    nxt = torch.empty_like(tail)
    out, at = [], 0
    for n in (5, 1, 2, 1, 3):
        part = proj[:, at:at + n].contiguous()
        out.append(mixers.short_conv(part, off, C, w, bs, tail, tail if n == 1 else nxt, at, pad if at == 0 else None, silu=silu, add_input=add))
        if n > 1:
            tail.copy_(nxt)
        at += n
    got = _c64(torch.cat(out, dim=1))
    tol = 1e-5 if dtype == torch.float32 else 0.03
    for b, p in enumerate(pads):
        hb = _c64(proj[b, p:, off:off + C])
        want = O.causal_taps(hb, _c64(w), None if bs is None else _c64(bs))
        want = O.silu(want) if silu else want
        want = want + hb if add else want
        assert (got[b, p:] - want).abs().max() < tol
        assert got[b, :p].abs().sum() == 0
    if taps > 1:
        assert torch.equal(tail[0], proj[0, T - (taps - 1):, off:off + C])


REC_CASES = [(4, 2, 12, 10, (70, 1, 5)), (2, 2, 136, 24, (20, 3)), (4, 1, 32, 64, (1, 1, 33, 2)), (1, 1, 8, 8, (4, 4)), (3, 3, 48, 32, (129,)),
             (40, 8, 64, 64, (36, 20))]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,sizes", REC_CASES)
def test_channel_delta_rule_with_carried_state(mixers, cuda_device, dtype, H, G, D, Dv, sizes):
    """the few-token and the pipelined kernel, the state carried from call to call, a row whose first tokens are padding, fewer
    key heads than value heads; the last case has more blocks than the GPU has SMs"""
    g = torch.Generator().manual_seed(H * D + Dv)
    B, T = 2, sum(sizes)
    pads = [0, min(3, sizes[0] - 1)]
    C, off_b = 2 * G * D + H * Dv, 3
    conv = _rand((B, T, C), g, dtype, cuda_device)
    proj = _rand((B, T, off_b + H + 2), g, dtype, cuda_device, 1.5)
    z = _rand((B, T, H * D), g, dtype, cuda_device)
    A_log, dt_bias = _rand((H,), g, dtype, cuda_device, 0.7) - 0.5, _rand((H * D,), g, dtype, cuda_device) - 1.0
    state = torch.zeros(B, H, D, Dv, dtype=torch.float32, device=cuda_device)
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    out, at = [], 0
    for n in sizes:
        out.append(mixers.channel_delta_rule(conv[:, at:at + n].contiguous(), G, H, D, Dv, proj[:, at:at + n].contiguous(), off_b,
                                             z[:, at:at + n].contiguous(), A_log, dt_bias, state, at, pad if at == 0 else None))
        at += n
    got = _c64(torch.cat(out, dim=1))
    tol = 2e-4 if dtype == torch.float32 else 2e-3                          # inputs are exact in both; the state is 32-bit
    rep = H // G
    for b, p in enumerate(pads):
        n = T - p
        c = _c64(conv[b, p:])
        q, k, v = c[:, :G * D].view(n, G, D), c[:, G * D:2 * G * D].view(n, G, D), c[:, 2 * G * D:].view(n, H, Dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-torch.exp(_c64(A_log)).view(1, H, 1) * O.softplus(_c64(z[b, p:]) + _c64(dt_bias)).view(n, H, D))
        beta = torch.sigmoid(_c64(proj[b, p:, off_b:off_b + H]))
        want = O.channel_delta_scan(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, decay, beta)
        assert ((got[b, p:] - want).abs() / (1 + want.abs())).max() < tol
        assert got[b, :p].abs().sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,N,P,sizes", REC_CASES)
def test_state_space_scan_with_carried_state(mixers, cuda_device, dtype, H, G, N, P, sizes):
    g = torch.Generator().manual_seed(H * N + P + 1)
    B, T = 2, sum(sizes)
    pads = [0, min(3, sizes[0] - 1)]
    C, off_dt = H * P + 2 * G * N, 4
    conv = _rand((B, T, C), g, dtype, cuda_device)
    proj = _rand((B, T, off_dt + H + 1), g, dtype, cuda_device, 1.5)
    A_log, dt_bias, skip = _rand((H,), g, dtype, cuda_device, 0.7) - 0.5, _rand((H,), g, dtype, cuda_device) - 0.5, _rand((H,), g, dtype, cuda_device) + 0.5
    state = torch.zeros(B, H, N, P, dtype=torch.float32, device=cuda_device)
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    out, at = [], 0
    for n in sizes:
        out.append(mixers.state_space_scan(conv[:, at:at + n].contiguous(), G, H, N, P, proj[:, at:at + n].contiguous(), off_dt, A_log, dt_bias, skip,
                                           state, at, pad if at == 0 else None))
        at += n
    got = _c64(torch.cat(out, dim=1))
    tol = 2e-4 if dtype == torch.float32 else 2e-3
    rep = H // G
    for b, p in enumerate(pads):
        n = T - p
        c = _c64(conv[b, p:])
        x = c[:, :H * P].view(n, H, P)
        Bm, Cm = c[:, H * P:H * P + G * N].view(n, G, N).repeat_interleave(rep, 1), c[:, H * P + G * N:].view(n, G, N).repeat_interleave(rep, 1)
        dt = O.softplus(_c64(proj[b, p:, off_dt:off_dt + H]) + _c64(dt_bias))
        want = O.state_space_scan(x, Bm, Cm, dt, torch.exp(_c64(A_log)), _c64(skip))
        assert ((got[b, p:] - want).abs() / (1 + want.abs())).max() < tol
        assert got[b, :p].abs().sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norms_with_their_gates(mixers, cuda_device, dtype):
    """the delta rule's read-out: norm per head, one weight vector for all heads, a sigmoid gate behind it; the state-space
    branch: silu gate FIRST, then the norm in equal parts with a weight per channel"""
    g = torch.Generator().manual_seed(9)
    n, H, D, eps = 7, 3, 20, 1e-3
    o = torch.randn(n, H, D, generator=g).to(cuda_device) * 3
    gate = _rand((n, H * D + 4), g, dtype, cuda_device)
    w = _rand((H * D,), g, dtype, cuda_device) + 1.0
    tol = 1e-5 if dtype == torch.float32 else 0.05
    gt = _c64(gate[:, 4:])
    out = torch.empty(n, H * D, dtype=dtype, device=cuda_device)
    mixers.gated_rms_norm(o, gate, 4, w[:D].contiguous(), eps, out, 0, 1.0, sigmoid=True)
    want = O.unit_rms(_c64(o), eps).reshape(n, H * D) * _c64(w[:D]).repeat(H) * torch.sigmoid(gt)
    assert (_c64(out) - want).abs().max() < tol
    for parts in (1, 2, 5):                                                 # the whole inner width as one part, or several
        view = o.view(n, parts, H * D // parts)
        mixers.gated_rms_norm(view, gate, 4, w, eps, out, 0, 1.0, gate_first=True)
        gated = _c64(o).reshape(n, H * D) * gt * torch.sigmoid(gt)
        want = O.unit_rms(gated.view(n, parts, -1), eps).reshape(n, H * D) * _c64(w)
        assert (_c64(out) - want).abs().max() < tol, parts
    late = O.unit_rms(_c64(o).reshape(n, 5, H * D // 5), eps).reshape(n, H * D) * _c64(w) * gt * torch.sigmoid(gt)
    assert (late - want).abs().max() > 0.1                                  # gating behind the norm would be another function
    # heads wider than a warp handles well take a block each: the same function
    H, D = 3, 400
    o = torch.randn(n, H, D, generator=g).to(cuda_device) * 3
    gate, w = _rand((n, H * D + 4), g, dtype, cuda_device), _rand((H * D,), g, dtype, cuda_device) + 1.0
    gt = _c64(gate[:, 4:])
    out = torch.empty(n, H * D + 2, dtype=dtype, device=cuda_device)
    mixers.gated_rms_norm(o, gate, 4, w[:D].contiguous(), eps, out, 2, 1.0, sigmoid=True)
    assert (_c64(out[:, 2:]) - O.unit_rms(_c64(o), eps).reshape(n, H * D) * _c64(w[:D]).repeat(H) * torch.sigmoid(gt)).abs().max() < tol
    for parts in (1, 2):
        mixers.gated_rms_norm(o.view(n, parts, H * D // parts), gate, 4, w, eps, out, 2, 0.5, gate_first=True)
        gated = _c64(o).reshape(n, H * D) * gt * torch.sigmoid(gt)
        assert (_c64(out[:, 2:]) - 0.5 * O.unit_rms(gated.view(n, parts, -1), eps).reshape(n, H * D) * _c64(w)).abs().max() < tol, parts


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("held,shift", [(0, 0), (6, 4000)])
def test_rotary_preparation_and_cache_write(mixers, cuda_device, dtype, held, shift):
    """grouped heads whose first channels rotate with rescaled frequencies (keys and values into a [B, G, capacity, D] store), and
    the latent form: queries rotate their LAST channels, the one key row per token is [normalised latent | rotated part]; far
    positions keep their angle (formed in double precision), padding slots hold zeros"""
    from ipex_llm_b200.transformers.models.nikedra import rotary_frequencies
    g = torch.Generator().manual_seed(held + 1)
    B, S, cap = 2, 5, 16
    pads = [0, 2]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    tol = 2e-5 if dtype == torch.float32 else 0.04

    def positions(b):
        return torch.arange(S) + held + shift - pads[b]

    # grouped heads
    H, G, D, Dv = 6, 2, 12, 10
    rot = {"base": 50.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    freq, amp = rotary_frequencies(rot)
    inv = torch.tensor(freq, dtype=F64, device=cuda_device)
    off_k, off_v = H * D + 1, H * D + 1 + G * D + 2
    proj = _rand((B, S, off_v + G * Dv + 3), g, dtype, cuda_device)
    ks, vs = torch.full((B, G, cap, D), 9.0, dtype=dtype, device=cuda_device), torch.full((B, G, cap, Dv), 9.0, dtype=dtype, device=cuda_device)
    q = mixers.rope_qk_prepare(proj, 0, off_k, off_v, H, G, D, D, Dv, 0, 0, 8, inv, amp, ks, (G * cap * D, D, cap * D), vs, (G * cap * Dv, Dv, cap * Dv),
                               held, shift, pad)
    for b in range(B):
        first = max(pads[b] - held - shift, 0)
        p64 = _c64(proj[b])
        want_q = O.rotate_half(p64[:, :H * D].view(S, H, D), positions(b), rot)
        want_k = O.rotate_half(p64[:, off_k:off_k + G * D].view(S, G, D), positions(b), rot)
        assert (_c64(q.view(B, S, H, D)[b, first:]) - want_q[first:]).abs().max() < tol
        assert (_c64(ks[b, :, held + first:held + S]).transpose(0, 1) - want_k[first:]).abs().max() < tol
        assert (_c64(vs[b, :, held + first:held + S]).transpose(0, 1) - p64[first:, off_v:off_v + G * Dv].view(S - first, G, Dv)).abs().max() < tol
        assert ks[b, :, held:held + first].abs().sum() == 0 and vs[b, :, held:held + first].abs().sum() == 0
        assert (ks[b, :, :held] == 9).all() and (ks[b, :, held + S:] == 9).all() and (vs[b, :, held + S:] == 9).all()
    assert (O.rotate_half(p64[:, :H * D].view(S, H, D), positions(1), dict(rot, scaling=None)) - want_q).abs().max() > 0.1    # the rescaling matters
    # latent form
    H, D, Dr, R, eps = 3, 10, 6, 12, 1e-3
    rot = {"base": 100.0, "dims": Dr}
    freq, amp = rotary_frequencies(rot)
    inv = torch.tensor(freq, dtype=F64, device=cuda_device)
    off_c = H * (D + Dr)
    proj = _rand((B, S, off_c + R + Dr + 7), g, dtype, cuda_device)
    nw = _rand((R,), g, dtype, cuda_device, 0.4) + 1.0
    store = torch.full((B, cap, R + Dr), 9.0, dtype=dtype, device=cuda_device)
    q = mixers.rope_qk_prepare(proj, 0, off_c, 0, H, 1, D + Dr, R + Dr, 0, D, R, Dr, inv, amp, store, (cap * (R + Dr), R + Dr, 0), None, None, held, shift, pad,
                               eps=eps, k_norm_w=nw, k_norm_cols=R)
    for b in range(B):
        first = max(pads[b] - held - shift, 0)
        p64 = _c64(proj[b])
        qh = p64[:, :off_c].view(S, H, D + Dr)
        want_q = torch.cat([qh[..., :D], O.rotate_half(qh[..., D:], positions(b), rot)], dim=-1)
        want_c = O.unit_rms(p64[:, off_c:off_c + R], eps) * _c64(nw)
        want_r = O.rotate_half(p64[:, off_c + R:off_c + R + Dr].view(S, 1, Dr), positions(b), rot)[:, 0]
        assert (_c64(q.view(B, S, H, D + Dr)[b, first:]) - want_q[first:]).abs().max() < tol
        assert (_c64(store[b, held + first:held + S]) - torch.cat([want_c, want_r], dim=-1)[first:]).abs().max() < tol
        assert store[b, held:held + first].abs().sum() == 0 and (store[b, :held] == 9).all() and (store[b, held + S:] == 9).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,held,H,G,D,Dv,tc", [
    (torch.float32, 5, 0, 6, 2, 5, 7, False), (torch.float32, 1, 300, 4, 1, 24, 40, False), (torch.float32, 70, 90, 3, 3, 18, 12, False),
    (torch.bfloat16, 1, 517, 3, 1, 64, 64, False), (torch.bfloat16, 40, 30, 4, 2, 32, 16, True), (torch.float16, 150, 0, 3, 1, 64, 48, True),
    (torch.bfloat16, 33, 200, 6, 2, 64, 48, True), (torch.bfloat16, 1, 700, 8, 2, 64, 128, True), (torch.bfloat16, 3, 130, 4, 1, 32, 256, True),
    (torch.bfloat16, 16, 301, 8, 1, 112, 128, True)])
def test_windows_and_chunks_in_every_attention_kernel(mixers, cuda_device, dtype, S, held, H, G, D, Dv, tc):
    """the general kernel, the prompt kernel on the tensor cores (S >= 16) and the kernel that splits the keys of shared heads over
    blocks (few tokens, vdim 128 / 256): no limit, windows and chunks from one position to more than everything held, a row that
    starts with padding, storage whose first index is not position 0"""
    g = torch.Generator().manual_seed(S * 100 + held)
    B, L = 2, held + S
    q = _rand((B * S, H * D), g, dtype, cuda_device)
    k, v = _rand((B, L + 3, G, D + 8), g, dtype, cuda_device)[..., 8:], _rand((B, L + 3, G, Dv + 16), g, dtype, cuda_device)[..., :Dv]
    scale = 2.0 / D ** 0.5
    tol = 2e-5 if dtype == torch.float32 else 0.02
    for shift, pads in ((0, [0, min(L - 1, 3)]), (11, [0, 0]), (11, [0, 13])):
        pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
        for window, chunk in ((0, 0), (1, 0), (2, 0), (37, 0), (64, 0), (L + 50, 0), (0, 1), (0, 5), (0, 29), (0, 64), (0, 118), (0, L + 50)):
            got = mixers.softmax_attention(q, k, v, B, S, H, held, shift, pad, window, scale, tensor_cores=tc, chunk=chunk)
            for b in range(B):
                want = O.visible_attention(_c64(q.view(B, S, H, D)[b]), _c64(k[b]), _c64(v[b]), scale, held, max(pads[b] - shift, 0), window, chunk,
                                           origin=pads[b] - shift)
                assert (_c64(got.view(B, S, H, Dv)[b]) - want).abs().max() < tol, (shift, pads, window, chunk, b)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,tc", [(torch.float32, 1, False), (torch.bfloat16, 1, True), (torch.bfloat16, 9, True), (torch.bfloat16, 30, True)])
def test_values_that_are_the_first_channels_of_the_key_rows(mixers, cuda_device, dtype, S, tc):
    """one cache row per position, shared by eight heads: the whole row is the key, its first 128 numbers are the value (the
    decoding form of the latent attention) -- in the general kernel, the split-key kernel and the prompt kernel"""
    g = torch.Generator().manual_seed(S)
    B, H, D, Dv, held = 2, 8, 144, 128, 300
    L = held + S
    q = _rand((B * S, H, D), g, dtype, cuda_device)
    rows = _rand((B, L + 5, 1, D), g, dtype, cuda_device)
    pads = [0, 7]
    pad = torch.tensor(pads, dtype=torch.int32, device=cuda_device)
    if tc and S <= 16:
        from ipex_llm_b200.ggml.model import mixers_cpp
        assert mixers_cpp.lib().mixers_softmax_attention_workspace(mixers_cpp.dtype_code(dtype), B, S, H, 1, D, Dv) > 0
    for window in (0, 70, 301):
        got = mixers.softmax_attention(q, rows, rows[..., :Dv], B, S, H, held, 0, pad, window, 0.1, tensor_cores=tc)
        for b in range(B):
            want = O.visible_attention(_c64(q.view(B, S, H, D)[b]), _c64(rows[b]), _c64(rows[b, ..., :Dv]), 0.1, held, pads[b], window)
            assert (_c64(got.view(B, S, H, Dv)[b]) - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.02), (window, b)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,tc", [(torch.float32, 1, False), (torch.float32, 40, False), (torch.bfloat16, 1, False), (torch.bfloat16, 40, False),
                                        (torch.bfloat16, 40, True), (torch.bfloat16, 1, True), (torch.bfloat16, 9, True)])
def test_one_outstanding_key_at_every_edge(mixers, cuda_device, dtype, S, tc):
    """a key whose score dwarfs all others: the output is its value when it is visible and must not show it otherwise -- far back
    among hundreds, at the borders of the kernels' key tiles, just inside and just outside a window or a chunk, for the last of
    the new tokens and for one in their middle, in front of a row's first token, in the future"""
    g = torch.Generator().manual_seed(11)
    H, D, Dv, L = 4, 16, 128, 700
    held = L - S
    base_k, base_v = torch.randn(1, L + 8, 1, D, generator=g) * 0.1, torch.randn(1, L + 8, 1, Dv, generator=g)
    spike = torch.zeros(D)
    spike[3] = 40.0
    q = (torch.randn(S, H * D, generator=g) * 0.1 + spike.repeat(H)[None] * 0.05).to(dtype).to(cuda_device)      # q . spike key = 80 + noise
    v_dev = base_v.to(dtype).to(cuda_device)
    if tc and S <= 16:
        from ipex_llm_b200.ggml.model import mixers_cpp
        assert mixers_cpp.lib().mixers_softmax_attention_workspace(mixers_cpp.dtype_code(dtype), 1, S, H, 1, D, Dv) > 0       # the split-key kernel

    def shows(at, query=S - 1, window=0, chunk=0, first=0, shift=0):
        """``first``: the row's padding (storage index of its first token); ``shift``: positions that have left the storage"""
        k = base_k.clone()
        k[0, at, 0] = spike
        out = mixers.softmax_attention(q, k.to(dtype).to(cuda_device), v_dev, 1, S, H, held, shift, torch.tensor([first], dtype=torch.int32,
                                       device=cuda_device), window, 1.0, tensor_cores=tc, chunk=chunk)
        d = (out.float().cpu().view(S, H, Dv)[query] - base_v[0, at, 0]).abs().max()
        assert d < 0.03 or d > 0.3, d
        return bool(d < 0.03)

    last = L - 1
    for at in (0, 1, 31, 32, 63, 64, 255, 256, 257, last - 1, last):
        assert shows(at), at                                                # without a limit every earlier key is visible
    assert not shows(L) and not shows(4, first=5) and shows(5, first=5)    # the future; in front of the row's first token; that token itself
    for w in (1, 2, 16, 64, 65, 130, 300, 699, 700, 5000):
        assert shows(max(last - w + 1, 0), window=w), w                     # the oldest key the window keeps
        if last - w >= 0:
            assert not shows(last - w, window=w), w                         # the next older one
            assert not shows(last - w, window=w, shift=7) and shows(last - w + 1, window=w, shift=7)
    for c in (1, 2, 7, 64, 118, 233, 350, 699, 700, 5000):
        for first, shift in ((0, 0), (5, 0), (0, 9)):
            start = ((last + shift - first) // c) * c - shift + first       # the storage index at which the last query's chunk starts
            assert shows(max(start, first), chunk=c, first=first, shift=shift), (c, first, shift)
            if start - 1 >= first:
                assert not shows(start - 1, chunk=c, first=first, shift=shift), (c, first, shift)
        assert not shows(L, chunk=c)                                        # a later position of the same chunk
    if S > 21:                                                              # a query in the middle of a prompt
        i = held + 20
        for w in (1, 2, 17, 64, 300):
            assert shows(i - w + 1, query=20, window=w) and not shows(i - w + 1, query=21, window=w)
            assert not shows(i - w, query=20, window=w) and not shows(i + 1, query=20, window=w)
        for c in (3, 64, 100):
            start = (i // c) * c
            assert shows(start, query=20, chunk=c) and not shows(start - 1, query=20, chunk=c)
            nxt = start + c                                                 # the first position of the next chunk
            if nxt - held < S:
                assert shows(nxt, query=nxt - held, chunk=c) and not shows(nxt - 1, query=nxt - held, chunk=c)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates_and_the_pair_of_width_norms(mixers, cuda_device, dtype):
    g = torch.Generator().manual_seed(2)
    n, H, Dv, eps = 9, 5, 14, 1e-3
    tol = 1e-5 if dtype == torch.float32 else 0.04
    o = _rand((n, H * Dv), g, dtype, cuda_device)
    gate = _rand((n, 3 + H * Dv + 2), g, dtype, cuda_device, 2.0)
    per_head = mixers.sigmoid_gate(o.clone(), gate, 3, Dv)                  # one number per head
    want = _c64(o).view(n, H, Dv) * torch.sigmoid(_c64(gate[:, 3:3 + H])).unsqueeze(-1)
    assert (_c64(per_head) - want.reshape(n, -1)).abs().max() < tol
    per_channel = mixers.sigmoid_gate(o.clone(), gate, 3, 1)                # one number per channel
    assert (_c64(per_channel) - _c64(o) * torch.sigmoid(_c64(gate[:, 3:3 + H * Dv]))).abs().max() < tol
    for width in (45, 1100, 4100):
        a, b = _rand((n, width), g, dtype, cuda_device, 3.0), _rand((n, width), g, dtype, cuda_device, 0.2)
        wa, wb = _rand((width,), g, dtype, cuda_device) + 1.0, _rand((width,), g, dtype, cuda_device) + 1.0
        got = mixers.rms_pair_sum(a, b, wa, wb, eps, 0.5)
        want = 0.5 * (O.unit_rms(_c64(a), eps) * _c64(wa) + O.unit_rms(_c64(b), eps) * _c64(wb))
        assert got.dtype == torch.float32 and (_c64(got) - want).abs().max() < tol
    z = _rand((7, 33), g, dtype, cuda_device, 2.0)
    assert (_c64(mixers.gelu_erf(z)) - O.gelu_erf(_c64(z))).abs().max() < tol
    assert (O.gelu_erf(_c64(z)) - O.gelu_tanh(_c64(z))).abs().max() > 1e-4   # the tanh form is another function


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,w", [(5, 2, 37), (12, 1, 40), (3, 3, 37), (16, 4, 1100), (64, 6, 88)])
def test_sigmoid_router_keeps_the_scores(mixers, cuda_device, dtype, experts, top, w):
    """the winners' own sigmoid scores are the weights: no sum to divide by, no scale"""
    g = torch.Generator().manual_seed(experts)
    n = 50
    h, router = _rand((n, w), g, dtype, cuda_device), _rand((experts, w), g, dtype, cuda_device, 2.4 / w ** 0.5)
    idx, wgt, _ = mixers.scored_router(h, router, None, 1, 1, top, sigmoid=True, group_top=1, renorm=False, scale=1.0)
    chosen, weights = O.route(_c64(h), _c64(router), top)
    assert torch.equal(idx.cpu().to(torch.int64).sort(1).values, chosen.sort(1).values)
    got = torch.zeros(n, experts, dtype=F64).scatter_(1, idx.cpu().to(torch.int64), _c64(wgt))
    want = torch.zeros(n, experts, dtype=F64).scatter_(1, chosen, weights)
    assert (got - want).abs().max() < 1e-5                                  # the router is 32-bit whatever the dtype
    if top > 1:
        assert (want.sum(1) - 1).abs().max() > 0.05                         # renormalised weights would differ


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_feed_forward_with_biases(tmp_path, cuda_device, dtype):
    cfg, w, model = build(tmp_path, "odd", dtype, cuda_device)
    g = torch.Generator().manual_seed(6)
    h = _rand((11, cfg["width"]), g, dtype, cuda_device, 2.0)
    spec = cfg["layers"][0]["mlp"]
    W = O.sub(w, "l0.mlp.")
    pre = _c64(h) @ W["gate"].T + W["gate.b"]
    assert (pre > spec["limit"]).any() and (pre < -spec["limit"]).any()     # the gate is capped from above only; both happen here
    want = O.clamped_dense(_c64(h), W, spec)
    got = model.model.layers[0].mlp(h)
    assert ((_c64(got) - want).abs() / (1 + want.abs())).max() < (1e-5 if dtype == torch.float32 else 0.05)
    assert (O.clamped_dense(_c64(h), W, dict(spec, limit=1.0)) - want).abs().max() > 0.05


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
    tokens = tokens_for(cfg, 200 if name == "wide" else 75, 3)
    collect, margins = [], []
    want = O.forward(cfg, w, tokens, collect, margins)
    clear = clear_choices(margins, len(tokens))
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
@pytest.mark.parametrize("name,layer", [("odd", 1), ("wide", 0), ("plain", 0), ("tile", 2)])
def test_experts_few_tokens_and_many_tokens_agree(tmp_path, cuda_device, dtype, name, layer):
    """the host-free path (address tables) and the sorted path compute the same layer; both match the plain statement: the
    score multiplies what goes INTO the expert, so it passes through the gelu"""
    from ipex_llm_b200.transformers.models import experts
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    mlp, spec = model.model.layers[layer].mlp, cfg["layers"][layer]["mlp"]
    g = torch.Generator().manual_seed(8)
    h = _rand((20, cfg["width"]), g, dtype, cuda_device, 1.5)
    W = O.sub(w, f"l{layer}.mlp.")
    want = O.input_weighted_experts(_c64(h), W, spec)
    few = model._experts(mlp, h, False)
    old, experts.MOE_SMALL_TOKENS = experts.MOE_SMALL_TOKENS, 0
    try:
        many = model._experts(mlp, h, False)
    finally:
        experts.MOE_SMALL_TOKENS = old
    tol = 3e-5 if dtype == torch.float32 else 0.08
    assert few.dtype == torch.float32 and (_c64(few) - want).abs().max() < tol and (_c64(many) - want).abs().max() < tol
    assert (few - many).abs().max() < (1e-5 if dtype == torch.float32 else 0.04)
    # weighting the OUTPUT instead is another function
    idx, wgt = O.route(_c64(h), W["router"], spec["router"]["top"])
    outside = torch.stack([sum(wgt[t, j] * (O.gelu_erf(_c64(h)[t] @ W[f"e{int(idx[t, j])}.up"].T) @ W[f"e{int(idx[t, j])}.down"].T)
                               for j in range(idx.shape[1])) for t in range(20)])
    assert (outside - want).abs().max() > 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["odd", "tile", "plain"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_batch_matches_each_request_alone(tmp_path, cuda_device, name, dtype):
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    lens, extra = [1, 23, 50, 7], 12
    seqs = [tokens_for(cfg, n + extra, 20 + n) for n in lens]
    want, clear = [], []
    for s in seqs:
        margins = []
        want.append(O.forward(cfg, w, s, None, margins))
        clear.append(clear_choices(margins, len(s)))
    width = max(lens)
    ids = torch.zeros(4, width, dtype=torch.int64)
    mask = torch.zeros(4, width, dtype=torch.int64)
    for b, (s, n) in enumerate(zip(seqs, lens)):
        ids[b, width - n:] = torch.tensor(s[:n])
        mask[b, width - n:] = 1
    with torch.no_grad():
        o = model(input_ids=ids.to(cuda_device), attention_mask=mask.to(cuda_device), use_cache=True)
        cache = o.past_key_values
        got = [[o.logits[b, width - n:]] for b, n in enumerate(lens)]
        rows = [0, 1, 2, 3]
        for step in range(extra):
            if step == 2:                                                   # two requests end: their rows leave the batch
                cache.batch_select_indices(torch.tensor([3, 1]))
                rows = [3, 1]
            nxt = torch.tensor([[seqs[b][lens[b] + step]] for b in rows], device=cuda_device)
            o = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            for r, b in enumerate(rows):
                got[b].append(o.logits[r])
    for b in range(4):
        g = torch.cat(got[b])
        assert_close(g, want[b][:g.shape[0]], dtype, clear[b][:g.shape[0]])


@pytest.mark.gpu
def test_long_decoding_across_many_windows_and_chunks(tmp_path, cuda_device):
    """300 tokens one by one from a 5-token prompt: the stores outgrow their first block and move, the window passes over decoded
    tokens seven times and a dozen chunks begin while decoding, the recurrent states and both tails are carried 300 times"""
    cfg, w, model = build(tmp_path, "tile", torch.float32, cuda_device)
    tokens = tokens_for(cfg, 305, 9)
    want = O.forward(cfg, w, tokens)
    got = run_portions(model, tokens, [5, 1], cuda_device)
    assert_close(got, want, torch.float32)
    # the same request in portions whose edges fall inside, on and next to the edges of windows (40) and chunks (24)
    for sizes in ([24, 16, 8, 47, 1, 1, 23, 25, 80], [39, 1, 41, 100], [48, 2]):
        assert_close(run_portions(model, tokens, sizes, cuda_device), want, torch.float32)


@pytest.mark.gpu
def test_a_far_token_and_the_first_token_reach_the_last_logits(tmp_path, cuda_device):
    """changing one early token of a long prompt must change the last position's logits exactly as the plain statement says, in
    a prompt and when the tail is decoded token by token (the recurrences carry it as old state; no window or chunk of this
    configuration reaches that far)"""
    cfg, w = make("odd")
    for k in w:
        if k.endswith("A_log"):
            w[k] = w[k] - 6.0                                               # states that hardly decay
    save_checkpoint(cfg, w, tmp_path / "slow")
    w, model = w64(w), load_framework(tmp_path / "slow", torch.float32, cuda_device)
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
    """a bf16 model whose latent attention decodes through the kernel that splits the keys of a shared head over blocks (8 heads
    on one cache row whose first 128 numbers are the values): the replayed step reads the cache length from the device and must produce the tokens of the
    loop that passes it from the host; states and tails are updated in place by both; the window passes over decoded tokens"""
    cfg, w, model = build(tmp_path, "wide", torch.bfloat16, cuda_device)
    from ipex_llm_b200.ggml.model import mixers_cpp
    assert mixers_cpp.lib().mixers_softmax_attention_workspace(mixers_cpp.dtype_code(torch.bfloat16), 2, 1, 8, 1, 160, 128) > 0
    prompts = torch.tensor([tokens_for(cfg, 70, 1), [0] * 30 + tokens_for(cfg, 40, 2)], device=cuda_device)
    mask = torch.tensor([[1] * 70, [0] * 30 + [1] * 40], device=cuda_device)
    replayed = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert model.__dict__.get("_b200_state_graph_failed") is None and model.__dict__.get("_b200_state_graphs")
    monkeypatch.setenv("IPEX_LLM_B200_DECODE_GRAPH", "0")
    eager = model.generate(prompts, attention_mask=mask, max_new_tokens=80, do_sample=False)
    assert torch.equal(replayed, eager)
    # and both follow the plain statement as far as a 16-bit model can: the first new token of each row
    for b, n in ((0, 70), (1, 40)):
        want = O.forward(cfg, w, prompts[b, 70 - n:].tolist())[-1]
        top2 = want.topk(2).values
        if top2[0] - top2[1] > 0.5 * cfg["logit_scale"]:
            assert int(replayed[b, 70]) == int(want.argmax())


@pytest.mark.gpu
def test_low_bit_conversion_runs_the_same_model(tmp_path, cuda_device, native_lib):
    """the projections are ordinary linears to the converter: a sym_int4 model answers close to the 16-bit one; its experts (no
    longer plain matrices) take the sorted path also for one token"""
    from ipex_llm_b200.transformers.low_bit_linear import LowBitLinear
    from ipex_llm_b200.transformers.models import experts
    cfg = O.random_config(width=128, vocab=90, taps=3, order=("channel_delta", "latent_attention", "parallel"), mlps=("moe", "dense", "moe"),
                          latent=dict(heads=2, dim=32, rot_dim=32, vdim=32, kv_rank=64, window=20), delta=dict(heads=2, kv_heads=1, dim=32, vdim=64),
                          left=dict(heads=2, kv_heads=1, dim=32, vdim=32, rot_dims=32, chunk=16), right=dict(heads=2, vdim=32, state=32, groups=1),
                          dense=dict(ff=64), moe=dict(experts=4, top=2, ff=64))
    w = O.random_weights(cfg, 3, ranks=(64, 64))
    save_checkpoint(cfg, w, tmp_path / "m")
    ref = load_framework(tmp_path / "m", torch.bfloat16, cuda_device)
    low = load_framework(tmp_path / "m", torch.bfloat16, None, load_in_low_bit="sym_int4").to(cuda_device)
    assert isinstance(low.model.layers[0].mixer.in_proj, LowBitLinear) and isinstance(low.model.layers[0].mlp.experts[0].down, LowBitLinear)
    assert isinstance(low.model.layers[1].mlp.gate_up, LowBitLinear) and isinstance(low.model.layers[2].mixer.right.o_proj, LowBitLinear)
    assert experts.address_tables(low.model.layers[0].mlp, torch.bfloat16, cuda_device) is None
    tokens = tokens_for(cfg, 30, 1)
    a = run_portions(ref, tokens, [30], cuda_device)
    b = run_portions(low, tokens, [25, 1], cuda_device)
    assert torch.isfinite(b).all() and position_errors(b, a.cpu().to(F64)).quantile(0.8) < 0.5


@pytest.mark.gpu
def test_trace_runner_replays_batches_and_gives_rows_back(tmp_path, cuda_device):
    """the command line a user replays a trace with: requests of unequal length start together and are decoded together, one ends
    early, a second batch starts afterwards (its rows take the place the first batch gave back); float32, against the plain
    statement position by position"""
    cfg, w = make("odd")
    save_checkpoint(cfg, w, tmp_path / "m")
    seqs = {"a": tokens_for(cfg, 31, 1), "b": tokens_for(cfg, 12, 2), "c": tokens_for(cfg, 20, 3), "d": tokens_for(cfg, 9, 4)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": seqs["a"][:25], "want": [0, 24]}, {"id": "b", "tokens": seqs["b"][:6], "want": [5]}], "end": []}]
    for i in range(6):                                                      # b ends behind step 4, a goes on alone
        want = [] if i == 2 else [0]
        entries = [{"id": "a", "tokens": [seqs["a"][25 + i]], "want": want}, {"id": "b", "tokens": [seqs["b"][6 + i]], "want": want}]
        steps.append({"step": 1 + i, "entries": entries[:2 if i < 4 else 1], "end": ["b"] if i == 3 else []})   # step 3 wants nothing: no file
    steps.append({"step": 7, "entries": [{"id": "c", "tokens": seqs["c"], "want": [19]}, {"id": "d", "tokens": seqs["d"], "want": [0, 8]}], "end": ["a", "c", "d"]})
    out = tmp_path / "out"
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(8)]
    full = {k: O.forward(cfg, w64(w), s) for k, s in seqs.items()}
    V = cfg["vocab"]

    def rows(step):
        return torch.frombuffer(bytearray((out / f"{step}.f32").read_bytes()), dtype=torch.float32).view(-1, V)

    assert not (out / "3.f32").exists()
    assert_close(rows(0), torch.stack([full["a"][0], full["a"][24], full["b"][5]]), torch.float32)
    for i in (0, 1, 3, 4, 5):
        assert_close(rows(1 + i), torch.stack([full["a"][25 + i], full["b"][6 + i]][:2 if i < 4 else 1]), torch.float32)
    assert_close(rows(7), torch.stack([full["c"][19], full["d"][0], full["d"][8]]), torch.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype", [("tile", torch.bfloat16), ("odd", torch.float32), ("wide", torch.bfloat16)])
def test_feed_forward_beside_the_mixer_changes_nothing(tmp_path, cuda_device, name, dtype):
    """long prompts run every layer's feed-forward on a second stream while the mixer runs on the first: the same kernels on the
    same numbers, so the logits are the same bit for bit, call after call (storage that one stream frees is not handed to the
    other too early), and decoding continues from the state such a prompt left"""
    from ipex_llm_b200.transformers.models import nikedra
    cfg, w, model = build(tmp_path, name, dtype, cuda_device)
    ids = torch.tensor([tokens_for(cfg, 130, s) for s in (1, 2, 3)], device=cuda_device)
    assert ids.numel() >= nikedra.OVERLAP_MIN_TOKENS
    with torch.no_grad():
        model.overlap_feed_forward = False
        want = model(input_ids=ids, use_cache=True)
        want_next = model(input_ids=ids[:, :1], past_key_values=want.past_key_values, use_cache=True).logits
        model.overlap_feed_forward = True
        for _ in range(4):
            got = model(input_ids=ids, use_cache=True)
            assert model._side_stream is not None and torch.equal(got.logits, want.logits)
        assert torch.equal(model(input_ids=ids[:, :1], past_key_values=got.past_key_values, use_cache=True).logits, want_next)
