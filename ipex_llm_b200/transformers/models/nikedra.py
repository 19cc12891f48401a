"""Nikedra: a decoder-only design whose layers run their mixer and their feed-forward side by side on the same stream,

    x <- x + mixer(conv(norm1(x))) + ff(norm2(x)),

with RMS norms that have ONE number as their weight, a short causal convolution over time added to what the mixer reads
(h + conv(h); its last inputs are part of a sequence's state), and a **depth-weighted average**: what a layer hands on is a
learned combination of the embedding output and every layer's result so far.  A layer's mixer is one of

* ``channel_delta``: a gated delta rule whose matrix state decays per key channel (decay from a low-rank projection), behind short
  causal convolutions, with unit-norm q / k, a per-head RMS norm of the read-out and a low-rank sigmoid gate;
* ``latent_attention``: softmax attention under a sliding window whose keys and values are expanded per head from one
  normalised latent per position, plus one rotated key part that all heads share -- latent and rotated part are all the cache
  keeps --, with a sigmoid gate per output channel;
* ``parallel``: grouped softmax attention confined to chunks of positions, rotary frequencies rescaled between a fast and a slow
  band, a sigmoid gate per head -- next to a state-space recurrence (scalar decay per head, gate before the grouped norm); each
  branch's output is RMS-normalised over the width and the two are averaged;

and its feed-forward is dense (clamped gated activation, biases) or a **mixture of experts** with sigmoid scores whose weight
multiplies the chosen expert's INPUT (experts without a gate, exact gelu).

No library ships this model.  The module tree, the configuration reader and the checkpoint's name map live here; the state in
``transformers/kv.py`` (``DynamicStateCache``: latent cache, key/value store, matrix states, convolution tails), the kernels in
``csrc/mixers`` behind ``ggml/model/mixers_cpp.py``.  The projections are ``nn.Linear`` modules, so the low-bit conversion treats
them like any other model's.  The residual stream and the kept streams, every norm, the router, rotary angles, attention scores
and weights and everything inside the recurrences are 32-bit whatever the model's dtype.
"""
import json
import math
import os
from typing import Optional

import torch
from torch import nn
from transformers import GenerationMixin, PreTrainedConfig, PreTrainedModel
from transformers.modeling_outputs import CausalLMOutputWithPast

from ipex_llm_b200.transformers.kv import DynamicStateCache
from ipex_llm_b200.transformers.models import experts, mixer_ops as ops
from ipex_llm_b200.transformers.models.common import merge_linear
from ipex_llm_b200.transformers.models.utils import read_safetensors
from ipex_llm_b200.utils.common import invalidInputError

ABSORB_MAX_TOKENS = 16        # up to this many new tokens per row attend to the latent cache itself (no key / value expansion)
OVERLAP_MIN_TOKENS = 256      # from this many new tokens on, a layer's feed-forward runs on a second stream beside its mixer
YARN_AMP_SLOPE = 0.1          # cosine and sine of rescaled frequencies are multiplied by slope * ln(factor) + 1


class NikedraConfig(PreTrainedConfig):
    """config.json of the design: ``vocab``, ``width``, ``layers`` (per layer: ``type``, ``mixer`` sizes and constants, ``mlp`` or
    null), ``norm.eps``, ``canon.taps``, ``logit_scale``.  ``low_ranks`` (per channel_delta layer: the ranks of its decay and gate
    projections) is not a key of the design's config.json: the loader reads it off the checkpoint's shapes, and it is kept so
    that a saved model can be rebuilt from its configuration alone."""
    model_type = "nikedra"

    def __init__(self, vocab=256, width=64, layers=None, norm=None, canon=None, logit_scale=1.0, architecture="Nikedra", low_ranks=None,
                 **kwargs):
        self.vocab, self.width = int(vocab), int(width)
        self.layers = layers or []
        self.norm = norm or {"eps": 1e-5}
        self.canon = canon or {"taps": 1}
        self.logit_scale = float(logit_scale)
        self.architecture = architecture
        self.low_ranks = {str(k): [int(v[0]), int(v[1])] for k, v in (low_ranks or {}).items()}
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)
        self.vocab_size, self.hidden_size, self.num_hidden_layers = self.vocab, self.width, len(self.layers)
        self.use_cache = True

    @property
    def norm_eps(self):
        return float(self.norm["eps"])

    @property
    def canon_taps(self):
        return int(self.canon["taps"])


def rotary_frequencies(rot):
    """(frequency of every rotated pair as a list of floats, amplitude) of a ``rot`` block: base^(-2i / dims); with ``scaling``
    (factor, original, fast, slow) a pair whose wavelength makes fewer than ``slow`` turns within ``original`` positions is slowed
    down by ``factor``, one that makes more than ``fast`` turns is kept, the pairs between are blended linearly by their index,
    and cosine and sine are multiplied by 0.1 ln(factor) + 1"""
    dims, base = int(rot["dims"]), float(rot["base"])
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return freq, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_with_turns(turns):                              # the (fractional) pair index whose wavelength makes this many turns
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_with_turns(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_with_turns(float(sc["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, YARN_AMP_SLOPE * math.log(factor) + 1.0


class _Rotary:
    """frequencies of a ``rot`` block in double precision on the device they are needed on (not a buffer: ``model.to(dtype)`` must
    not round them; the kernel forms the angles in double precision too)"""

    def __init__(self, rot):
        self.dims = int(rot["dims"])
        invalidInputError(self.dims % 2 == 0, "rotary dims must be even")
        self.freq, self.amp = rotary_frequencies(rot)
        self._on = {}

    def inv_freq(self, device):
        t = self._on.get(device)
        if t is None:
            t = self._on[device] = torch.tensor(self.freq or [0.0], dtype=torch.float64).to(device)
        return t


class _Weight(nn.Module):
    """a lone parameter under the name ``<module>.weight``: a norm's vector of weights, or (shape ()) its single gain"""

    def __init__(self, *shape):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(tuple(shape)))


class ChannelDeltaMixer(nn.Module):
    """``q_proj`` .. ``g1_proj`` (everything that reads the mixer's input) become one ``in_proj`` when ``merge_projections`` has run"""
    PARTS = ("q_proj", "k_proj", "v_proj", "b_proj", "a1_proj", "g1_proj")

    def __init__(self, width, m, ranks):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim, self.taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
        invalidInputError(self.kv_heads >= 1 and self.heads % self.kv_heads == 0, "heads must be a multiple of kv_heads")
        qk, v = self.kv_heads * self.dim, self.heads * self.vdim
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(width, qk, bias=False), nn.Linear(width, qk, bias=False), nn.Linear(width, v, bias=False)
        self.b_proj = nn.Linear(width, self.heads, bias=False)
        self.a1_proj, self.a2_proj = nn.Linear(width, ranks[0], bias=False), nn.Linear(ranks[0], self.heads * self.dim, bias=False)
        self.g1_proj, self.g2_proj = nn.Linear(width, ranks[1], bias=False), nn.Linear(ranks[1], v, bias=False)
        self.conv_weight = nn.Parameter(torch.zeros(2 * qk + v, self.taps))          # q | k | v channels
        self.A_log, self.dt_bias = nn.Parameter(torch.zeros(self.heads)), nn.Parameter(torch.zeros(self.heads * self.dim))
        self.norm = _Weight(self.vdim)
        self.o_proj = nn.Linear(v, width, bias=False)


class LatentRopeAttention(nn.Module):
    """``q_proj`` / ``dkv`` / ``g_proj`` become one ``in_proj`` when ``merge_projections`` has run.  A cache row is [latent | rotated
    key part]; ``expand`` [heads * (dim + rot_dim) + heads * vdim, kv_rank + rot_dim] turns such rows into every head's key
    [W_uk latent | rotated part] and value [W_uv latent]: per head the key rows are (W_uk_h 0; 0 I), the value rows (W_uv_h 0).
    A plain parameter, because the attention of few tokens multiplies by its per-head blocks (queries into the cache's space,
    the weighted cache rows back out) instead of expanding the cache."""

    def __init__(self, width, m):
        super().__init__()
        self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        self.scale, self.window = float(m["scale"]), int(m["mask"]["size"])
        self.rotary = _Rotary(dict(m["rot"], dims=self.rot_dim))
        qd = self.dim + self.rot_dim
        self.q_proj = nn.Linear(width, self.heads * qd, bias=False)
        self.dkv = nn.Linear(width, self.kv_rank + self.rot_dim, bias=False)
        self.g_proj = nn.Linear(width, self.heads * self.vdim, bias=False)
        self.dkv_norm = _Weight(self.kv_rank)
        self.expand = _Weight(self.heads * (qd + self.vdim), self.kv_rank + self.rot_dim)
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)

    def expansion(self, uk, uv):
        """``expand`` from the checkpoint's per-head key rows uk [heads * dim, kv_rank] and value rows uv [heads * vdim, kv_rank]"""
        H, D, Dr, Dv, R = self.heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        keys = torch.zeros(H, D + Dr, R + Dr, dtype=uk.dtype)
        keys[:, :D, :R] = uk.view(H, D, R)
        keys[:, D:, R:] = torch.eye(Dr, dtype=uk.dtype)
        values = torch.zeros(H * Dv, R + Dr, dtype=uk.dtype)
        values[:, :R] = uv
        return torch.cat([keys.view(H * (D + Dr), R + Dr), values], dim=0)


class ChunkedAttention(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        invalidInputError(self.kv_heads >= 1 and self.heads % self.kv_heads == 0, "heads must be a multiple of kv_heads")
        self.scale, self.chunk = float(m["scale"]), int(m["mask"]["size"])
        self.rotary = _Rotary(m["rot"])
        invalidInputError(self.rotary.dims <= self.dim, "rotary dims exceed the head size")
        self.q_proj = nn.Linear(width, self.heads * self.dim, bias=False)
        self.k_proj = nn.Linear(width, self.kv_heads * self.dim, bias=False)
        self.v_proj = nn.Linear(width, self.kv_heads * self.vdim, bias=False)
        self.g_proj = nn.Linear(width, self.heads, bias=False)
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)
        self.out = _Weight(width)


class StateSpaceMixer(nn.Module):
    """``in_proj``'s rows: z (inner) | x (inner) | B (groups * state) | C (groups * state) | dt (heads), inner = heads * vdim"""

    def __init__(self, width, m):
        super().__init__()
        self.heads, self.vdim, self.state, self.groups = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
        self.norm_groups, self.taps = int(m["norm_groups"]), int(m["conv"])
        self.inner = self.heads * self.vdim
        invalidInputError(self.groups >= 1 and self.heads % self.groups == 0 and self.norm_groups >= 1 and self.inner % self.norm_groups == 0,
                          "heads must be a multiple of groups, and the inner width of norm_groups")
        self.conv_channels = self.inner + 2 * self.groups * self.state
        self.in_proj = nn.Linear(width, 2 * self.inner + 2 * self.groups * self.state + self.heads, bias=False)
        self.conv_weight, self.conv_bias = nn.Parameter(torch.zeros(self.conv_channels, self.taps)), nn.Parameter(torch.zeros(self.conv_channels))
        self.dt_bias, self.A_log, self.D = (nn.Parameter(torch.zeros(self.heads)) for _ in range(3))
        self.norm = _Weight(self.inner)
        self.o_proj = nn.Linear(self.inner, width, bias=False)
        self.out = _Weight(width)


class ParallelMixer(nn.Module):
    """``left.{q,k,v,g}_proj`` and ``right.in_proj`` become one ``in_proj`` when ``merge_projections`` has run"""

    def __init__(self, width, m):
        super().__init__()
        self.left, self.right = ChunkedAttention(width, m["left"]), StateSpaceMixer(width, m["right"])


class ClampedMLP(nn.Module):
    """down(g' sigmoid(1.702 g') (u' + 1)) with biases, g' = min(gate h, limit), u' = clamp(up h, -limit, limit); gate and up are the
    two halves of ``gate_up``'s rows"""

    def __init__(self, width, m):
        super().__init__()
        self.ff, self.limit = int(m["ff"]), float(m["limit"])
        self.gate_up, self.down = nn.Linear(width, 2 * self.ff, bias=True), nn.Linear(self.ff, width, bias=True)

    def forward(self, h):
        return self.down(ops.clamped_glu(self.gate_up(h), self.ff, self.limit))


class UngatedExpert(nn.Module):
    """down(gelu(up h)) with the exact gelu, no biases"""

    def __init__(self, width, ff):
        super().__init__()
        self.ff = int(ff)
        self.up, self.down = nn.Linear(width, self.ff, bias=False), nn.Linear(self.ff, width, bias=False)


class InputWeightedExperts(nn.Module):
    """sigmoid scores, the ``top`` largest win, their scores (not renormalised) multiply the chosen experts' inputs"""

    def __init__(self, width, m):
        super().__init__()
        self.n_experts, self.top = int(m["router"]["experts"]), int(m["router"]["top"])
        invalidInputError(1 <= self.top <= self.n_experts, "a token takes between one and all experts")
        self.router = nn.Parameter(torch.zeros(self.n_experts, width))
        self.experts = nn.ModuleList([UngatedExpert(width, m["expert"]["ff"]) for _ in range(self.n_experts)])
        self.shared = None
        self._tables = None


MIXER_TYPES = ("channel_delta", "latent_attention", "parallel")


class NikedraLayer(nn.Module):
    def __init__(self, config: NikedraConfig, index):
        super().__init__()
        lc, w = config.layers[index], config.width
        self.kind = lc["type"]
        invalidInputError(self.kind in MIXER_TYPES, f"unknown layer type {self.kind}")
        self.norm1 = _Weight()
        self.canon = nn.Parameter(torch.zeros(w, config.canon_taps))
        if self.kind == "channel_delta":
            self.mixer = ChannelDeltaMixer(w, lc["mixer"], config.low_ranks.get(str(index), [1, 1]))
        elif self.kind == "latent_attention":
            self.mixer = LatentRopeAttention(w, lc["mixer"])
        else:
            self.mixer = ParallelMixer(w, lc["mixer"])
        self.mlp = None
        m = lc.get("mlp")
        if m is not None:
            kind = m.get("kind", "dense")
            invalidInputError(kind in ("dense", "moe"), f"unknown feed-forward kind {kind}")
            self.mlp = ClampedMLP(w, m) if kind == "dense" else InputWeightedExperts(w, m)
            self.norm2 = _Weight()
        self.dwa = nn.Parameter(torch.ones(index + 2))


def merge_projections(module: nn.Module):
    """every projection that reads a mixer's input becomes one ``in_proj`` (one product per mixer and token)"""
    if isinstance(module, ChannelDeltaMixer) and not hasattr(module, "in_proj"):
        module.in_proj = merge_linear([getattr(module, n) for n in module.PARTS])
        for n in module.PARTS:
            delattr(module, n)
    elif isinstance(module, LatentRopeAttention) and not hasattr(module, "in_proj"):
        module.in_proj = merge_linear([module.q_proj, module.dkv, module.g_proj])
        del module.q_proj, module.dkv, module.g_proj
    elif isinstance(module, ParallelMixer) and not hasattr(module, "in_proj"):
        l, r = module.left, module.right
        module.in_proj = merge_linear([l.q_proj, l.k_proj, l.v_proj, l.g_proj, r.in_proj])
        del l.q_proj, l.k_proj, l.v_proj, l.g_proj, r.in_proj


class NikedraModel(nn.Module):
    def __init__(self, config: NikedraConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab, config.width)
        self.embed_norm = _Weight()
        self.layers = nn.ModuleList([NikedraLayer(config, i) for i in range(len(config.layers))])
        self.norm = _Weight()


class NikedraForCausalLM(PreTrainedModel, GenerationMixin):
    config_class = NikedraConfig
    base_model_prefix = "model"
    _no_split_modules = ["NikedraLayer"]
    _supports_attention_backend = False
    main_input_name = "input_ids"

    def __init__(self, config: NikedraConfig):
        super().__init__(config)
        self.model = NikedraModel(config)
        self.lm_head = nn.Linear(config.width, config.vocab, bias=False)
        self.collect_residual = None          # a list: gets the residual stream after every layer (debugging aid)
        self.attention_tensor_cores = True    # 16-bit models: prompts take the tensor-core attention kernel
        self.overlap_feed_forward = True      # prompts: mixer and feed-forward read the same stream, so they run side by side
        self._side_stream = None

    def _init_weights(self, module):
        pass

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    # ---- helpers
    def _plain_linears(self):
        """no projection was converted to a low-bit format (those products share one workspace per device, so two of them
        must not run on two streams at once)"""
        plain = self.__dict__.get("_b200_plain_linears")
        if plain is None:
            plain = self.__dict__["_b200_plain_linears"] = all(type(m) is nn.Linear for m in self.modules() if isinstance(m, nn.Linear) or
                                                               type(m).__name__ == "LowBitLinear")
        return plain

    @staticmethod
    def _conv(proj, off, channels, weight, bias, rec, key, B, S, cache, silu, add_input=False):
        """a short causal convolution over the new tokens and the state's tail (which keeps its address: a recorded step holds it)"""
        taps = weight.shape[1]
        tail, tail_next = rec.tails(B, taps, channels, proj.dtype, proj.device, key=key)
        pad = cache.pad if cache.seen == 0 else None                         # padding only ever precedes a row's first call
        y = ops.short_conv(proj, off, channels, weight, bias, tail, tail if S == 1 else tail_next, cache.seen, pad, silu=silu, add_input=add_input)
        if S > 1:
            tail.copy_(tail_next)
        return y

    # ---- mixers (h: the mixer's input in the model's dtype, [N, W]); each returns [N, W]
    def _channel_delta(self, mx, h, st, B, S, cache):
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        H, G, D, Dv = mx.heads, mx.kv_heads, mx.dim, mx.vdim
        proj = mx.in_proj(h)                                                 # q | k | v | beta | decay rank | gate rank
        P = proj.shape[1]
        C = 2 * G * D + H * Dv
        off_b = C
        off_a1 = off_b + H
        off_g1 = off_a1 + mx.a2_proj.in_features
        conv = self._conv(proj.view(B, S, P), 0, C, mx.conv_weight, None, st.rec, "mixer", B, S, cache, silu=True)
        z = mx.a2_proj(proj[:, off_a1:off_g1])                               # decay logits [N, H D]
        gate = mx.g2_proj(proj[:, off_g1:off_g1 + mx.g2_proj.in_features])   # [N, H Dv]
        state = st.rec.matrix(B, H, D, Dv, h.device)
        o = ops.channel_delta_rule(conv, G, H, D, Dv, proj.view(B, S, P), off_b, z, mx.A_log, mx.dt_bias, state, cache.seen,
                                   cache.pad if cache.seen == 0 else None)
        out = torch.empty(B * S, H * Dv, dtype=h.dtype, device=h.device)
        ops.gated_rms_norm(o, gate, 0, mx.norm.weight, self.config.norm_eps, out, 0, 1.0, sigmoid=True)
        return mx.o_proj(out)

    def _latent_attention(self, mx, h, st, B, S, cache):
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        H, D, Dr, Dv, R, N = mx.heads, mx.dim, mx.rot_dim, mx.vdim, mx.kv_rank, B * S
        Dq, Rk = D + Dr, R + Dr
        kv = st.kv
        proj = mx.in_proj(h)                                                 # q (head by head: unrotated | rotated) | latent | rotated key | gate
        P = proj.shape[1]
        off_c, off_g = H * Dq, H * Dq + Rk
        store, held = kv.slots(B, Rk, S, h.dtype, h.device)
        shift = cache.seen - held                                            # storage index + shift = slot number
        # a recorded decode step reads the length from the device (the value given here is the one at recording time)
        dyn = kv.length_dev if (cache.frozen and S == 1) else None
        cap = store.shape[1]
        q = ops.rope_qk_prepare(proj.view(B, S, P), 0, off_c, 0, H, 1, Dq, Rk, 0, D, R, Dr, mx.rotary.inv_freq(h.device), mx.rotary.amp,
                                store, (cap * Rk, Rk, 0), None, None, held, shift, cache.pad, eps=self.config.norm_eps,
                                k_norm_w=mx.dkv_norm.weight, k_norm_cols=R, dyn=dyn)
        kv.commit(S)
        w = mx.expand.weight
        if S <= ABSORB_MAX_TOKENS:
            # few new tokens: the query of head h moves into the cache rows' space (W_uk_h^T q | rotated q), the cache itself is
            # the key of one shared head, its latent part (the first R numbers of a row) the value, and W_uv_h maps the weighted
            # latents back
            wk, wv = w[:H * Dq].view(H, Dq, Rk), w[H * Dq:].view(H, Dv, Rk)[:, :, :R]
            qa = torch.matmul(q.view(N, H, Dq).transpose(0, 1), wk).transpose(0, 1)                  # [N, H, Rk], stored head by head
            rows = store.unsqueeze(2)                                        # [B, capacity, 1, Rk]
            o_rows = ops.softmax_attention(qa, rows, rows[..., :R], B, S, H, held, shift, cache.pad, mx.window, mx.scale, dyn=dyn)
            o = torch.matmul(o_rows.view(N, H, R).transpose(0, 1), wv.transpose(1, 2)).transpose(0, 1).reshape(N, H * Dv)
        else:
            # a prompt or a long portion: keys and values of the positions that some new token still sees, expanded from the cache
            first = max(held - (mx.window - 1), 0)
            total = held + S
            kvx = torch.nn.functional.linear(store[:, first:total], w)      # [B, total - first, H * (Dq + Dv)]
            k = kvx[..., :H * Dq].view(B, total - first, H, Dq)
            v = kvx[..., H * Dq:].view(B, total - first, H, Dv)
            o = ops.softmax_attention(q, k, v, B, S, H, held - first, shift + first, cache.pad, mx.window, mx.scale,
                                      tensor_cores=self.attention_tensor_cores)
        ops.sigmoid_gate(o, proj, off_g, 1)
        return mx.o_proj(o)

    def _parallel(self, mx, h, st, B, S, cache):
        """fp32 [N, W]"""
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        l, r = mx.left, mx.right
        H, G, D, Dv = l.heads, l.kv_heads, l.dim, l.vdim
        proj = mx.in_proj(h)                                                 # left q | k | v | gate | right z | x | B | C | dt
        P = proj.shape[1]
        proj3 = proj.view(B, S, P)
        eps = self.config.norm_eps
        off_k = H * D
        off_v = off_k + G * D
        off_g = off_v + G * Dv
        off_z = off_g + H
        off_x = off_z + r.inner
        off_dt = off_x + r.conv_channels
        # left: rotary, cache append, attention inside the chunk, a gate per head
        kv = st.kv
        like_k = torch.empty((B, G, 0, D), dtype=h.dtype, device=h.device)
        like_v = torch.empty((B, G, 0, Dv), dtype=h.dtype, device=h.device)
        k_store, v_store, held = kv.slots(like_k, like_v, S)
        shift = cache.seen - held
        dyn = kv.length_dev if (cache.frozen and S == 1) else None
        cap = kv.capacity()
        q = ops.rope_qk_prepare(proj3, 0, off_k, off_v, H, G, D, D, Dv, 0, 0, l.rotary.dims, l.rotary.inv_freq(h.device), l.rotary.amp,
                                k_store, (G * cap * D, D, cap * D), v_store, (G * cap * Dv, Dv, cap * Dv), held, shift, cache.pad, dyn=dyn)
        kv.commit(S)
        o = ops.softmax_attention(q, k_store.permute(0, 2, 1, 3), v_store.permute(0, 2, 1, 3), B, S, H, held, shift, cache.pad, 0, l.scale,
                                  dyn=dyn, tensor_cores=self.attention_tensor_cores, chunk=l.chunk)
        ops.sigmoid_gate(o, proj, off_g, Dv)
        left = l.o_proj(o)
        # right: convolution over x | B | C, the scan, the gate, the grouped norm
        conv = self._conv(proj3, off_x, r.conv_channels, r.conv_weight, r.conv_bias, st.rec, "mixer", B, S, cache, silu=True)
        state = st.rec.matrix(B, r.heads, r.state, r.vdim, h.device)
        y = ops.state_space_scan(conv, r.groups, r.heads, r.state, r.vdim, proj3, off_dt, r.A_log, r.dt_bias, r.D, state, cache.seen,
                                 cache.pad if cache.seen == 0 else None)
        out = torch.empty(B * S, r.inner, dtype=h.dtype, device=h.device)
        ops.gated_rms_norm(y.view(B * S, r.norm_groups, r.inner // r.norm_groups), proj, off_z, r.norm.weight, eps, out, 0, 1.0,
                           gate_first=True)
        right = r.o_proj(out)
        return ops.rms_pair_sum(left, right, l.out.weight, r.out.weight, eps, 0.5)

    def _experts(self, mlp, h, frozen_step):
        """fp32 [N, W]"""
        idx, wgt, _ = ops.scored_router(h, mlp.router, None, 1, 1, mlp.top, sigmoid=True, group_top=1, renorm=False, scale=1.0)
        N, E = h.shape[0], mlp.n_experts
        tables = experts.address_tables(mlp, h.dtype, h.device) if (N <= experts.MOE_SMALL_TOKENS or frozen_step) else None
        if tables is not None:
            up, down, ffs, ff_max, _ = tables
            return ops.moe_small(h, idx, wgt, up, down, ff_max, E, E, None, ffs=ffs, ungated_gelu=True, weight_input=True)
        return experts.sorted_experts(mlp, h, idx, wgt, E, lambda u, expert: ops.gelu_erf(u), weight_input=True)

    def forward(self, input_ids: Optional[torch.LongTensor] = None, attention_mask: Optional[torch.Tensor] = None,
                position_ids=None, past_key_values=None, inputs_embeds=None, use_cache: Optional[bool] = None,
                logits_to_keep=0, **kwargs):
        """``input_ids`` [B, S]: the next S tokens of every row.  On the first call of a batch ``attention_mask`` [B, S] gives
        the left padding; later calls continue from ``past_key_values`` (a ``DynamicStateCache``; any other or no cache
        starts a new one).  Positions follow from the padding, ``position_ids`` is not read.  ``logits_to_keep``: 0 = all
        positions, n = the last n, or a 1-D tensor of positions."""
        invalidInputError(input_ids is not None and inputs_embeds is None, "the model takes token ids")
        core, cfg = self.model, self.config
        B, S = input_ids.shape
        dev, dtype = core.embed_tokens.weight.device, core.embed_tokens.weight.dtype
        eps = cfg.norm_eps
        cache = past_key_values
        if not isinstance(cache, DynamicStateCache):
            invalidInputError(cache is None or cache.get_seq_length() == 0, "a filled cache of another class cannot be continued")
            cache = DynamicStateCache()
        if cache.seen == 0:                                                  # a batch's first call: the mask gives the padding
            cache.start(attention_mask, B, S, dev)
        invalidInputError(cache.pad.shape[0] == B, "batch size differs from the cache's")
        input_ids = input_ids.to(dev).contiguous()
        frozen_step = cache.frozen and S == 1
        n_layers = len(core.layers)
        # padding only occurs in a batch's first call; later calls (a replayed step among them, whose slot number is the one at
        # recording time) say so by passing no padding
        x, _ = ops.embed_pair(core.embed_tokens.weight, 1.0, None, 0, 0, 0, input_ids, None, cache.seen, cache.pad if cache.seen == 0 else None, dtype)
        stack = torch.empty(n_layers + 1, B * S, cfg.width, dtype=torch.float32, device=dev)       # the embedding output and every layer's result

        def gains(i):
            """the two norms that read the stream in front of layer i (none behind the last layer)"""
            if i >= n_layers:
                return None, None
            layer = core.layers[i]
            return layer.norm1.weight, (layer.norm2.weight if layer.mlp is not None else None)

        main = side = forked = None
        if (self.overlap_feed_forward and B * S >= OVERLAP_MIN_TOKENS and dev.type == "cuda" and not cache.frozen
                and not torch.cuda.is_current_stream_capturing() and self._plain_linears()):
            main = torch.cuda.current_stream(dev)
            if self._side_stream is None or self._side_stream.device != dev:
                self._side_stream = torch.cuda.Stream(dev)
            side = self._side_stream
        g1, g2 = gains(0)
        h1, h2 = ops.sum_residual_norms(x, [], dtype, eps, pre_gain=core.embed_norm.weight, stack=stack, index=0, gain1=g1, gain2=g2)
        for i, layer in enumerate(core.layers):
            if layer.kind == "latent_attention":
                st = cache.run_state(i, latent=True)
            else:
                st = cache.run_state(i, window=0 if layer.kind == "parallel" else None)
            if side is not None and layer.mlp is not None:
                forked = main.record_event()                                 # h2 is ready here; nothing of this layer's mixer is queued yet
            hm = self._conv(h1.view(B, S, -1), 0, cfg.width, layer.canon, None, st.rec, "input", B, S, cache, silu=False, add_input=True)
            hm = hm.view(B * S, -1)
            if layer.kind == "channel_delta":
                y_mix = self._channel_delta(layer.mixer, hm, st, B, S, cache)
            elif layer.kind == "latent_attention":
                y_mix = self._latent_attention(layer.mixer, hm, st, B, S, cache)
            else:
                y_mix = self._parallel(layer.mixer, hm, st, B, S, cache)
            y_ff = None
            if layer.mlp is not None and side is not None:
                # behind the mixer's launches in program order, but waiting only for what was on the main stream before them: the
                # recurrences walk their tokens on a fraction of the SMs, the feed-forward's matrix products take the rest
                side.wait_event(forked)
                with torch.cuda.stream(side):
                    y_ff = layer.mlp(h2) if isinstance(layer.mlp, ClampedMLP) else self._experts(layer.mlp, h2, frozen_step)
                y_ff.record_stream(main)
                main.wait_stream(side)
            elif layer.mlp is not None:
                y_ff = layer.mlp(h2) if isinstance(layer.mlp, ClampedMLP) else self._experts(layer.mlp, h2, frozen_step)
            g1, g2 = gains(i + 1)
            h1, h2 = ops.sum_residual_norms(x, [y_mix, y_ff], dtype, eps, stack=stack, index=i + 1, coef=layer.dwa, gain1=g1, gain2=g2)
            if self.collect_residual is not None:
                self.collect_residual.append(x.view(B, S, -1).clone())
        cache.advance(S)
        xs = x.view(B, S, -1)
        if not (isinstance(logits_to_keep, int) and logits_to_keep == 0):
            idx = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep.to(dev)
            xs = xs[:, idx, :].contiguous()
        hn = ops.rms_norm_rows(xs, core.norm.weight, None, eps, dtype)
        # every kept position as a row of its own ([rows, 1, W]): a converted lm_head keeps only the last position of a long
        # sequence axis (the reference's prefill shortcut), and which positions to keep is decided here, by logits_to_keep
        logits = self.lm_head(hn.reshape(-1, 1, hn.shape[-1])).to(torch.float32).view(B, xs.shape[1], -1)
        if cfg.logit_scale != 1.0:
            logits = logits * cfg.logit_scale
        return CausalLMOutputWithPast(logits=logits, past_key_values=cache)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs):
        """generate() hands over every token so far; the model takes those its cache has not seen"""
        seen = past_key_values.get_seq_length() if isinstance(past_key_values, DynamicStateCache) else 0
        return {"input_ids": input_ids[:, seen:], "attention_mask": attention_mask, "past_key_values": past_key_values,
                "use_cache": True, "logits_to_keep": 1}


# ------------------------------------------------------------------ checkpoint
def checkpoint_key_map(config: NikedraConfig):
    """the model's parameter names -> the checkpoint's tensor names: one name, or a list of them (concatenated by rows).  The
    latent attention's ``expand`` is not in the map: ``load_pretrained`` builds it from the key and value expansions."""
    m = {"model.embed_tokens.weight": "embed", "model.embed_norm.weight": "embed.norm", "lm_head.weight": "head", "model.norm.weight": "final.norm"}
    for i, lc in enumerate(config.layers):
        d, s = f"model.layers.{i}.", f"l{i}."
        m[d + "norm1.weight"], m[d + "canon"], m[d + "dwa"] = s + "norm1", s + "canon1", s + "dwa"
        dm, sm = d + "mixer.", s + "mix."
        if lc["type"] == "channel_delta":
            for n in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o"):
                m[dm + n + "_proj.weight"] = sm + n
            m[dm + "conv_weight"] = [sm + "q.conv", sm + "k.conv", sm + "v.conv"]
            m[dm + "A_log"], m[dm + "dt_bias"], m[dm + "norm.weight"] = sm + "A_log", sm + "dt_bias", sm + "norm"
        elif lc["type"] == "latent_attention":
            m[dm + "q_proj.weight"], m[dm + "dkv.weight"], m[dm + "g_proj.weight"], m[dm + "o_proj.weight"] = sm + "q", sm + "dkv", sm + "g", sm + "o"
            m[dm + "dkv_norm.weight"] = sm + "dkv.norm"
        else:
            for n in ("q", "k", "v", "g", "o"):
                m[dm + "left." + n + "_proj.weight"] = sm + "left." + n
            m[dm + "left.out.weight"], m[dm + "right.out.weight"] = sm + "left.out", sm + "right.out"
            dr, sr = dm + "right.", sm + "right."
            m[dr + "in_proj.weight"], m[dr + "o_proj.weight"] = sr + "in", sr + "o"
            m[dr + "conv_weight"], m[dr + "conv_bias"] = sr + "conv", sr + "conv.b"
            m[dr + "dt_bias"], m[dr + "A_log"], m[dr + "D"], m[dr + "norm.weight"] = sr + "dt_bias", sr + "A_log", sr + "D", sr + "norm"
        mlp = lc.get("mlp")
        if mlp is not None:
            m[d + "norm2.weight"] = s + "norm2"
            dp, sp = d + "mlp.", s + "mlp."
            if mlp.get("kind", "dense") == "dense":
                m[dp + "gate_up.weight"], m[dp + "gate_up.bias"] = [sp + "gate", sp + "up"], [sp + "gate.b", sp + "up.b"]
                m[dp + "down.weight"], m[dp + "down.bias"] = sp + "down", sp + "down.b"
            else:
                m[dp + "router"] = sp + "router"
                for e in range(int(mlp["router"]["experts"])):
                    m[dp + f"experts.{e}.up.weight"], m[dp + f"experts.{e}.down.weight"] = sp + f"e{e}.up", sp + f"e{e}.down"
    return m


def load_pretrained(model_dir, torch_dtype=None, device=None):
    """config.json + model.safetensors of the design -> a ``NikedraForCausalLM``.  Sizes that config.json does not state (the
    ranks of a channel_delta layer's decay and gate projections) come from the tensors' shapes."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    if "low_ranks" not in raw:
        raw["low_ranks"] = {str(i): [tensors[f"l{i}.mix.a1"].shape[0], tensors[f"l{i}.mix.g1"].shape[0]]
                            for i, lc in enumerate(raw.get("layers", []))
                            if lc["type"] == "channel_delta" and f"l{i}.mix.a1" in tensors and f"l{i}.mix.g1" in tensors}
    config = NikedraConfig(**raw)
    if torch_dtype in (None, "auto"):
        torch_dtype = tensors["embed"].dtype
    with torch.device("meta"):
        model = NikedraForCausalLM(config)
    state = {}
    for dst, src in checkpoint_key_map(config).items():
        names = [src] if isinstance(src, str) else list(src)
        missing = [s for s in names if s not in tensors]
        invalidInputError(not missing, f"the checkpoint has no tensor {missing}")
        t = tensors[src] if isinstance(src, str) else torch.cat([tensors[s] for s in src], dim=0)
        state[dst] = t.to(torch_dtype)
    for i, layer in enumerate(model.model.layers):
        if layer.kind == "latent_attention":
            uk, uv = f"l{i}.mix.uk", f"l{i}.mix.uv"
            invalidInputError(uk in tensors and uv in tensors, f"the checkpoint has no tensor {[n for n in (uk, uv) if n not in tensors]}")
            mx = layer.mixer
            invalidInputError(tuple(tensors[uk].shape) == (mx.heads * mx.dim, mx.kv_rank) and tuple(tensors[uv].shape) == (mx.heads * mx.vdim, mx.kv_rank),
                              f"l{i}: the key / value expansions do not have the sizes the configuration gives")
            state[f"model.layers.{i}.mixer.expand.weight"] = mx.expansion(tensors[uk].to(torch_dtype), tensors[uv].to(torch_dtype))
    for name, p in model.named_parameters():
        invalidInputError(name in state, f"no checkpoint tensor for parameter {name}")
        if tuple(state[name].shape) != tuple(p.shape) and [d for d in state[name].shape if d != 1] == [d for d in p.shape if d != 1]:
            state[name] = state[name].reshape(p.shape)                       # the same numbers with or without axes of length 1
        invalidInputError(tuple(state[name].shape) == tuple(p.shape),
                          f"{name}: checkpoint shape {tuple(state[name].shape)} but the configuration gives {tuple(p.shape)}")
    model.load_state_dict(state, strict=True, assign=True)
    model.eval()
    model.requires_grad_(False)
    model.config.dtype = torch_dtype
    if device is not None:
        model = model.to(device)
    return model


# the loaders that go through transformers' Auto classes (load_low_bit builds the architecture from a saved configuration)
def _register():
    from transformers import AutoConfig, AutoModelForCausalLM
    try:
        AutoConfig.register("nikedra", NikedraConfig)
        AutoModelForCausalLM.register(NikedraConfig, NikedraForCausalLM)
    except ValueError:                                                       # registered already
        pass


_register()
