"""Serotar: a decoder-only design built from

* an embedding of the token plus an embedding of the (previous token, token) pair, hashed into a table of buckets;
* **latent attention** without positions: queries through a normalised low-rank latent, keys and values expanded per head
  from ONE normalised latent per position -- the only thing the cache keeps (``LatentKVLayer``); causal softmax;
* feed-forwards that are dense (xIELU activation) or a **mixture of experts** (softmax router, a correction that only affects
  the choice, groups of experts of which the best few may be chosen from, identity experts, a shared expert);
* a residual stream that adds ``norm(sublayer(x)) * layer scale`` -- the sublayers read x itself, the RMS norm with a single
  gain sits on their OUTPUT --, a per-layer input that looks the token up in a side table, and a **depth-weighted average**:
  what a layer hands on is a learned combination of the embedding output and every layer's result so far.

No library ships this model.  The module tree, the configuration reader and the checkpoint's name map live here; the cache in
``transformers/kv.py`` (``DynamicStateCache`` with ``LatentKVLayer`` and the previous-token state), the kernels in
``csrc/mixers`` behind ``ggml/model/mixers_cpp.py``.  The projections are ``nn.Linear`` modules (one per expert and
projection), so the low-bit conversion treats them like any other model's.  The residual stream, every norm, the router, the
attention scores and weights are 32-bit whatever the model's dtype.
"""
import json
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
MOE_SMALL_TOKENS = experts.MOE_SMALL_TOKENS


class SerotarConfig(PreTrainedConfig):
    """config.json of the design: ``vocab``, ``width``, ``embedding`` (``scale``, optional ``bigram``: ``buckets``, ``mul_prev``,
    ``mul_cur``), ``layers`` (per layer: ``type``, ``mixer`` sizes, ``mlp`` or null), ``norm.eps``, ``token_side.dim`` (optional).
    ``layer_scale`` / ``depth_average`` are not keys of the design's config.json: the loader sets them from the tensors the
    checkpoint has, and they are kept so that a saved model can be rebuilt from its configuration alone."""
    model_type = "serotar"

    def __init__(self, vocab=256, width=64, embedding=None, layers=None, norm=None, token_side=None, architecture="Serotar",
                 layer_scale=True, depth_average=True, **kwargs):
        self.vocab, self.width = int(vocab), int(width)
        self.embedding = embedding or {"scale": 1.0}
        self.layers = layers or []
        self.norm = norm or {"eps": 1e-6}
        self.token_side = token_side
        self.architecture = architecture
        self.layer_scale, self.depth_average = bool(layer_scale), bool(depth_average)
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)
        self.vocab_size, self.hidden_size, self.num_hidden_layers = self.vocab, self.width, len(self.layers)
        self.use_cache = True

    @property
    def norm_eps(self):
        return float(self.norm["eps"])

    @property
    def bigram(self):
        return self.embedding.get("bigram") or None

    @property
    def side_dim(self):
        return int(self.token_side["dim"]) if self.token_side else 0


class _Weight(nn.Module):
    """a lone parameter under the name ``<module>.weight``: a norm's vector of weights, or (shape ()) its single gain"""

    def __init__(self, *shape):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(tuple(shape)))


class LatentAttention(nn.Module):
    """``dq`` / ``dkv`` become one ``in_proj`` when ``merge_projections`` has run.  ``expand``: the per-head key rows
    [heads * dim, kv_rank] followed by the value rows [heads * vdim, kv_rank]; a plain parameter, because the attention of few
    tokens multiplies by its per-head blocks (queries into the latent space, the weighted latent back out) instead of
    expanding the cache."""

    def __init__(self, width, m):
        super().__init__()
        self.heads, self.dim, self.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        self.q_rank, self.kv_rank, self.scale = int(m["q_rank"]), int(m["kv_rank"]), float(m["scale"])
        self.dq, self.dkv = nn.Linear(width, self.q_rank, bias=False), nn.Linear(width, self.kv_rank, bias=False)
        self.dq_norm, self.dkv_norm = _Weight(self.q_rank), _Weight(self.kv_rank)
        self.uq = nn.Linear(self.q_rank, self.heads * self.dim, bias=False)
        self.expand = _Weight(self.heads * (self.dim + self.vdim), self.kv_rank)
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)


class XieluMLP(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        self.up_proj, self.down_proj = nn.Linear(width, int(m["ff"]), bias=False), nn.Linear(int(m["ff"]), width, bias=False)
        self.act = nn.Parameter(torch.zeros(2))


class GatedExpert(nn.Module):
    """down(silu(gate h) * (up h)); gate and up are the two halves of ``gate_up``'s rows"""

    def __init__(self, width, ff):
        super().__init__()
        self.ff = int(ff)
        self.gate_up, self.down = nn.Linear(width, 2 * self.ff, bias=False), nn.Linear(self.ff, width, bias=False)

    def forward(self, h):
        return self.down(ops.silu_mul(self.gate_up(h), self.ff))


class RoutedExperts(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        r = m["router"]
        self.n_experts, self.n_identity, self.top = int(r["experts"]), int(r.get("identity", 0) or 0), int(r["top"])
        g = r.get("groups") or {"count": 1, "keep": 1}
        self.groups, self.keep = int(g["count"]), int(g["keep"])
        self.n_out = self.n_experts + self.n_identity
        invalidInputError(self.n_out % self.groups == 0 and 1 <= self.keep <= self.groups, "experts + identity experts must form equal groups")
        self.ff = int(m["expert"]["ff"])
        self.router, self.correction = nn.Parameter(torch.zeros(self.n_out, width)), nn.Parameter(torch.zeros(self.n_out))
        self.experts = nn.ModuleList([GatedExpert(width, self.ff) for _ in range(self.n_experts)])
        self.shared = GatedExpert(width, m["shared"]["ff"]) if m.get("shared") else None
        self._tables = None

    def address_tables(self, dtype, device):
        """see ``experts.address_tables``"""
        return experts.address_tables(self, dtype, device)


class TokenSide(nn.Module):
    def __init__(self, width, dim):
        super().__init__()
        self.gate, self.proj = nn.Linear(width, dim, bias=False), nn.Linear(dim, width, bias=False)
        self.norm = _Weight(width)


class SerotarLayer(nn.Module):
    def __init__(self, config: SerotarConfig, index):
        super().__init__()
        lc, w = config.layers[index], config.width
        invalidInputError(lc["type"] == "latent_attention", f"unknown layer type {lc['type']}")
        self.mixer = LatentAttention(w, lc["mixer"])
        self.norm1 = _Weight()
        self.ls1 = nn.Parameter(torch.ones(w)) if config.layer_scale else None
        self.mlp = None
        m = lc.get("mlp")
        if m is not None:
            kind = m.get("kind", "dense")
            invalidInputError(kind in ("dense", "moe"), f"unknown feed-forward kind {kind}")
            self.mlp = XieluMLP(w, m) if kind == "dense" else RoutedExperts(w, m)
            self.norm2 = _Weight()
            self.ls2 = nn.Parameter(torch.ones(w)) if config.layer_scale else None
        self.side = TokenSide(w, config.side_dim) if config.side_dim else None
        self.dwa = nn.Parameter(torch.ones(index + 2)) if config.depth_average else None


def merge_projections(module: nn.Module):
    """the two projections that read the mixer's input (query latent, key/value latent) become one ``in_proj``"""
    if isinstance(module, LatentAttention) and not hasattr(module, "in_proj"):
        module.in_proj = merge_linear([module.dq, module.dkv])
        del module.dq, module.dkv


class SerotarModel(nn.Module):
    def __init__(self, config: SerotarConfig):
        super().__init__()
        self.config = config
        w = config.width
        self.embed_tokens = nn.Embedding(config.vocab, w)
        self.pair_embed = nn.Embedding(int(config.bigram["buckets"]) + 1, w) if config.bigram else None
        self.side_embed = nn.Embedding(config.vocab, config.side_dim * len(config.layers)) if config.side_dim else None
        self.layers = nn.ModuleList([SerotarLayer(config, i) for i in range(len(config.layers))])
        self.norm = _Weight()


class SerotarForCausalLM(PreTrainedModel, GenerationMixin):
    config_class = SerotarConfig
    base_model_prefix = "model"
    _no_split_modules = ["SerotarLayer"]
    _supports_attention_backend = False
    main_input_name = "input_ids"

    def __init__(self, config: SerotarConfig):
        super().__init__(config)
        self.model = SerotarModel(config)
        self.lm_head = nn.Linear(config.width, config.vocab, bias=False)
        self.collect_residual = None          # a list: gets the residual stream after every layer (debugging aid)
        self.attention_tensor_cores = True    # 16-bit models: prompts take the tensor-core attention kernel

    def _init_weights(self, module):
        pass

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    # ---- sublayers (h: the stream in the model's dtype, [N, W])
    def _attention(self, mx, h, kv, B, S, cache):
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        H, D, Dv, R, N = mx.heads, mx.dim, mx.vdim, mx.kv_rank, B * S
        proj = mx.in_proj(h)
        store, held = kv.slots(B, R, S, h.dtype, h.device)
        # a recorded decode step reads the length from the device (the value given here is the one at recording time)
        dyn = kv.length_dev if (cache.frozen and S == 1) else None
        cq = ops.latent_prepare(proj.view(B, S, proj.shape[-1]), 0, mx.q_rank, mx.dq_norm.weight, mx.q_rank, R, mx.dkv_norm.weight,
                                self.config.norm_eps, store, held, 0, cache.pad, dyn)
        kv.commit(S)
        q = mx.uq(cq)                                                        # [N, H * D]
        w = mx.expand.weight
        if S <= ABSORB_MAX_TOKENS:
            # few new tokens: score = (W_uk^T q) . c and out = W_uv (sum p c): the cache itself is key and value of one shared head
            wk, wv = w[:H * D].view(H, D, R), w[H * D:].view(H, Dv, R)
            qa = torch.matmul(q.view(N, H, D).transpose(0, 1), wk).transpose(0, 1)                   # [N, H, R], stored head by head
            lat = store.unsqueeze(2)                                         # [B, capacity, 1, R]
            o_lat = ops.softmax_attention(qa, lat, lat, B, S, H, held, 0, cache.pad, 0, mx.scale, dyn=dyn)
            o = torch.matmul(o_lat.view(N, H, R).transpose(0, 1), wv.transpose(1, 2)).transpose(0, 1).reshape(N, H * Dv)
        else:
            # a prompt or a long portion: keys and values of every position so far, expanded from the latents
            total = held + S
            kvx = torch.nn.functional.linear(store[:, :total], w)           # [B, total, H * (D + Dv)]
            k = kvx[..., :H * D].view(B, total, H, D)
            v = kvx[..., H * D:].view(B, total, H, Dv)
            o = ops.softmax_attention(q, k, v, B, S, H, held, 0, cache.pad, 0, mx.scale, tensor_cores=self.attention_tensor_cores)
        return mx.o_proj(o)

    def _experts(self, mlp, h, frozen_step):
        idx, wgt = ops.grouped_router(h, mlp.router, mlp.correction, mlp.groups, mlp.keep, mlp.top)
        N, E = h.shape[0], mlp.n_experts
        tables = mlp.address_tables(h.dtype, h.device) if (N <= MOE_SMALL_TOKENS or frozen_step) else None
        if tables is not None:
            gate_up, down, ffs, ff_max, with_shared = tables
            shared = mlp.shared(h) if (mlp.shared is not None and not with_shared) else None
            return ops.moe_small(h, idx, wgt, gate_up, down, ff_max, E, mlp.n_out, shared, ffs=ffs, always_on=with_shared)
        shared = mlp.shared(h) if mlp.shared is not None else None
        return experts.sorted_experts(mlp, h, idx, wgt, mlp.n_out, lambda gu, expert: ops.silu_mul(gu, expert.ff), shared)

    def forward(self, input_ids: Optional[torch.LongTensor] = None, attention_mask: Optional[torch.Tensor] = None,
                position_ids=None, past_key_values=None, inputs_embeds=None, use_cache: Optional[bool] = None,
                logits_to_keep=0, **kwargs):
        """``input_ids`` [B, S]: the next S tokens of every row.  On the first call of a batch ``attention_mask`` [B, S] gives
        the left padding; later calls continue from ``past_key_values`` (a ``DynamicStateCache``; any other or no cache
        starts a new one).  ``logits_to_keep``: 0 = all positions, n = the last n, or a 1-D tensor of positions."""
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
        ids = input_ids.reshape(-1)
        frozen_step = cache.frozen and S == 1
        n_layers = len(core.layers)
        stack = torch.empty(n_layers + 1, B * S, cfg.width, dtype=torch.float32, device=dev) if cfg.depth_average else None
        bg = cfg.bigram
        prev = cache.previous_tokens(B, dev)
        # padding and first tokens only occur in a batch's first call; later calls (a replayed step among them, whose slot
        # number is the one at recording time) say so by passing no padding
        x, h = ops.embed_pair(core.embed_tokens.weight, cfg.embedding.get("scale", 1.0), core.pair_embed.weight if bg else None,
                              bg["buckets"] if bg else 0, bg["mul_prev"] if bg else 0, bg["mul_cur"] if bg else 0, input_ids, prev,
                              cache.seen, cache.pad if cache.seen == 0 else None, dtype, x_copy=stack[0] if stack is not None else None)
        prev.copy_(input_ids[:, -1])                                         # the pair of the next call's first token
        for i, layer in enumerate(core.layers):
            def add(y, gain, vec, last):
                """x += norm(y) * gain * vec; the layer's last addition also keeps the stream and takes the depth average"""
                if last and stack is not None:
                    return ops.rms_residual(x, y, gain, vec, eps, dtype, stack=stack, index=i + 1, coef=layer.dwa)
                return ops.rms_residual(x, y, gain, vec, eps, dtype)

            st = cache.run_state(i, latent=True)
            y = self._attention(layer.mixer, h, st.kv, B, S, cache)
            h = add(y, layer.norm1.weight, layer.ls1, layer.mlp is None and layer.side is None)
            if layer.mlp is not None:
                if isinstance(layer.mlp, XieluMLP):
                    y = layer.mlp.down_proj(ops.xielu(layer.mlp.up_proj(h), layer.mlp.act))
                else:
                    y = self._experts(layer.mlp, h, frozen_step)
                h = add(y, layer.norm2.weight, layer.ls2, layer.side is None)
            if layer.side is not None:
                g = ops.gelu_table_mul(layer.side.gate(h), core.side_embed.weight, i * cfg.side_dim, ids)
                h = add(layer.side.proj(g), None, layer.side.norm.weight, True)
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
        return CausalLMOutputWithPast(logits=logits, past_key_values=cache)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs):
        """generate() hands over every token so far; the model takes those its cache has not seen"""
        seen = past_key_values.get_seq_length() if isinstance(past_key_values, DynamicStateCache) else 0
        return {"input_ids": input_ids[:, seen:], "attention_mask": attention_mask, "past_key_values": past_key_values,
                "use_cache": True, "logits_to_keep": 1}


# ------------------------------------------------------------------ checkpoint
def checkpoint_key_map(config: SerotarConfig):
    """the model's parameter names -> the checkpoint's tensor names (or a list of them, concatenated by rows)"""
    m = {"model.embed_tokens.weight": "embed", "lm_head.weight": "head", "model.norm.weight": "final.norm"}
    if config.bigram:
        m["model.pair_embed.weight"] = "bigram"
    if config.side_dim:
        m["model.side_embed.weight"] = "side.embed"
    for i, lc in enumerate(config.layers):
        d, s = f"model.layers.{i}.", f"l{i}."
        m[d + "norm1.weight"] = s + "norm1"
        dm, sm = d + "mixer.", s + "mix."
        m[dm + "dq.weight"], m[dm + "dq_norm.weight"], m[dm + "uq.weight"] = sm + "dq", sm + "dq.norm", sm + "uq"
        m[dm + "dkv.weight"], m[dm + "dkv_norm.weight"] = sm + "dkv", sm + "dkv.norm"
        m[dm + "expand.weight"], m[dm + "o_proj.weight"] = [sm + "uk", sm + "uv"], sm + "o"
        if config.layer_scale:
            m[d + "ls1"] = s + "ls1"
        mlp = lc.get("mlp")
        if mlp is not None:
            m[d + "norm2.weight"] = s + "norm2"
            if config.layer_scale:
                m[d + "ls2"] = s + "ls2"
            dp, sp = d + "mlp.", s + "mlp."
            if mlp.get("kind", "dense") == "dense":
                m[dp + "up_proj.weight"], m[dp + "down_proj.weight"], m[dp + "act"] = sp + "up", sp + "down", sp + "act"
            else:
                m[dp + "router"], m[dp + "correction"] = sp + "router", sp + "correction"
                names = [(f"experts.{e}.", f"e{e}.") for e in range(int(mlp["router"]["experts"]))]
                if mlp.get("shared"):
                    names.append(("shared.", "shared."))
                for dn, sn in names:
                    m[dp + dn + "gate_up.weight"] = [sp + sn + "gate", sp + sn + "up"]
                    m[dp + dn + "down.weight"] = sp + sn + "down"
        if config.side_dim:
            m[d + "side.gate.weight"], m[d + "side.proj.weight"], m[d + "side.norm.weight"] = s + "side.gate", s + "side.proj", s + "side.norm"
        if config.depth_average:
            m[d + "dwa"] = s + "dwa"
    return m


def load_pretrained(model_dir, torch_dtype=None, device=None):
    """config.json + model.safetensors of the design -> a ``SerotarForCausalLM``.  Whether the layers have a layer scale and a
    depth average is read off the checkpoint's tensors (config.json has no key for either)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    raw.setdefault("layer_scale", "l0.ls1" in tensors)
    raw.setdefault("depth_average", "l0.dwa" in tensors)
    config = SerotarConfig(**raw)
    if torch_dtype in (None, "auto"):
        torch_dtype = tensors["embed"].dtype
    with torch.device("meta"):
        model = SerotarForCausalLM(config)
    state = {}
    for dst, src in checkpoint_key_map(config).items():
        missing = [s for s in ([src] if isinstance(src, str) else src) if s not in tensors]
        invalidInputError(not missing, f"the checkpoint has no tensor {missing}")
        t = tensors[src] if isinstance(src, str) else torch.cat([tensors[s] for s in src], dim=0)
        state[dst] = t.to(torch_dtype)
    for name, p in model.named_parameters():
        invalidInputError(name in state, f"no checkpoint tensor for parameter {name}")
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
        AutoConfig.register("serotar", SerotarConfig)
        AutoModelForCausalLM.register(SerotarConfig, SerotarForCausalLM)
    except ValueError:                                                       # registered already
        pass


_register()
