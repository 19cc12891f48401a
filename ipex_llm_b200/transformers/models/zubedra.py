"""Zubedra: a decoder-only design of **parallel layers** -- one layer norm (a weight, no bias) feeds the mixer AND the
feed-forward, and both results are added to the stream at once -- whose mixer is one of

* ``wkv``: an RWKV-style recurrence.  Five token-shifted copies of the input (h + (previous h - h) * mu) feed the receptance, key,
  value, gate and decay projections; the decay of every key channel is exp(-exp(low-rank(h) + w0)); a matrix state per head is
  read BEFORE the token's update, plus a bonus u for the token itself; the heads' outputs are divided by their root mean square,
  weighted, gated with silu and projected;
* ``attention``: softmax attention without positions.  Queries and keys are RMS-normalised over their WHOLE projection (all
  heads at once), scores are capped (cap * tanh(score / cap)), the softmax's denominator holds a learned sink per head, and a
  layer that blends values stores (1 - l) v + l v_first, v_first being the values of the first blending layer for the same
  token;

and whose feed-forward is a **mixture of experts**: sigmoid scores, a correction that only affects the choice, groups of
neighbouring experts ranked by their two best members, weights = the winners' scores over their sum times a scale, experts with
a clamped gated activation, and a shared expert under a sigmoid gate of its own.

No library ships this model.  The module tree, the configuration reader and the checkpoint's name map live here; the state in
``transformers/kv.py`` (``DynamicStateCache``: a key/value store per attention layer, a matrix state and the previous token's
input per wkv layer), the kernels in ``csrc/mixers`` behind ``ggml/model/mixers_cpp.py``.  The projections are ``nn.Linear``
modules, so the low-bit conversion treats them like any other model's.  The residual stream, every norm, the router, the
attention scores and weights and everything inside the recurrence are 32-bit whatever the model's dtype.
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

SHIFTS = ("r", "k", "v", "g", "w")     # the order of the token-shift vectors in ``WkvMixer.mu``
GROUP_TOP = 2                          # a group of experts is ranked by the sum of this many best members


class ZubedraConfig(PreTrainedConfig):
    """config.json of the design: ``vocab``, ``width``, ``embedding.scale``, ``layers`` (per layer: ``type``, ``mixer`` sizes and
    constants, ``mlp`` or null), ``norm.eps``, ``logit_scale``.  ``wkv_ranks`` (the rank of each wkv layer's decay projection) is
    not a key of the design's config.json: the loader reads it off the checkpoint's shapes, and it is kept so that a saved model
    can be rebuilt from its configuration alone."""
    model_type = "zubedra"

    def __init__(self, vocab=256, width=64, embedding=None, layers=None, norm=None, logit_scale=1.0, architecture="Zubedra",
                 wkv_ranks=None, **kwargs):
        self.vocab, self.width = int(vocab), int(width)
        self.embedding = embedding or {"scale": 1.0}
        self.layers = layers or []
        self.norm = norm or {"eps": 1e-5}
        self.logit_scale = float(logit_scale)
        self.architecture = architecture
        self.wkv_ranks = {str(k): int(v) for k, v in (wkv_ranks or {}).items()}
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)
        self.vocab_size, self.hidden_size, self.num_hidden_layers = self.vocab, self.width, len(self.layers)
        self.use_cache = True

    @property
    def norm_eps(self):
        return float(self.norm["eps"])

    def first_blending_layer(self):
        """index of the first attention layer that blends values (its own values are what the later ones blend in), or None"""
        for i, lc in enumerate(self.layers):
            if lc["type"] == "attention" and lc["mixer"].get("v_mix"):
                return i
        return None


class _Weight(nn.Module):
    """a lone vector under the name ``<module>.weight``"""

    def __init__(self, n):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))


class SinkAttention(nn.Module):
    """``q_proj`` / ``k_proj`` / ``v_proj`` become one ``in_proj`` when ``merge_projections`` has run"""

    def __init__(self, width, m):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        invalidInputError(self.kv_heads >= 1 and self.heads % self.kv_heads == 0, "heads must be a multiple of kv_heads")
        self.scale, self.softcap, self.blend = float(m["scale"]), float(m.get("softcap") or 0.0), bool(m.get("v_mix"))
        self.q_proj = nn.Linear(width, self.heads * self.dim, bias=False)
        self.k_proj = nn.Linear(width, self.kv_heads * self.dim, bias=False)
        self.v_proj = nn.Linear(width, self.kv_heads * self.vdim, bias=False)
        self.q_norm, self.k_norm = _Weight(self.heads * self.dim), _Weight(self.kv_heads * self.dim)
        self.vmix = nn.Parameter(torch.zeros(()))
        self.sink = nn.Parameter(torch.zeros(self.heads))
        self.o_proj = nn.Linear(self.heads * self.vdim, width, bias=False)


class WkvMixer(nn.Module):
    """``r_proj`` / ``k_proj`` / ``v_proj`` / ``g_proj`` become one ``rkvg`` [4, heads * dim, width] when ``merge_projections`` has
    run on a model that keeps plain matrices: they read four different inputs, so they merge into one BATCHED product"""

    def __init__(self, width, m, rank):
        super().__init__()
        self.heads, self.dim = int(m["heads"]), int(m["dim"])
        hd = self.heads * self.dim
        self.mu = nn.Parameter(torch.zeros(len(SHIFTS), width))
        self.r_proj, self.k_proj, self.v_proj, self.g_proj = (nn.Linear(width, hd, bias=False) for _ in range(4))
        self.w1_proj, self.w2_proj = nn.Linear(width, rank, bias=False), nn.Linear(rank, hd, bias=False)
        self.w0 = nn.Parameter(torch.zeros(hd))
        self.u = nn.Parameter(torch.zeros(self.heads, self.dim))
        self.norm = _Weight(hd)
        self.o_proj = nn.Linear(hd, width, bias=False)


class ClampedExpert(nn.Module):
    """down(g' sigmoid(1.702 g') (u' + 1)), g' = min(gate h, limit), u' = clamp(up h, -limit, limit); gate and up are the two
    halves of ``gate_up``'s rows"""

    def __init__(self, width, m):
        super().__init__()
        self.ff, self.limit = int(m["ff"]), float(m["limit"])
        self.gate_up, self.down = nn.Linear(width, 2 * self.ff, bias=False), nn.Linear(self.ff, width, bias=False)

    def forward(self, h):
        return self.down(ops.clamped_glu(self.gate_up(h), self.ff, self.limit))


class SigmoidRoutedExperts(nn.Module):
    def __init__(self, width, m):
        super().__init__()
        invalidInputError(m.get("kind", "moe") == "moe", f"unknown feed-forward kind {m.get('kind')}")
        r = m["router"]
        self.n_experts, self.top, self.scale = int(r["experts"]), int(r["top"]), float(r.get("scale", 1.0))
        g = r.get("groups") or {"count": 1, "keep": 1}
        self.groups, self.keep = int(g["count"]), int(g["keep"])
        invalidInputError(self.n_experts % self.groups == 0 and 1 <= self.keep <= self.groups, "the experts must form equal groups")
        invalidInputError(self.top <= self.keep * (self.n_experts // self.groups), "more experts per token than the kept groups hold")
        self.router, self.correction = nn.Parameter(torch.zeros(self.n_experts, width)), nn.Parameter(torch.zeros(self.n_experts))
        self.experts = nn.ModuleList([ClampedExpert(width, m["expert"]) for _ in range(self.n_experts)])
        self.limit = float(m["expert"]["limit"])
        self.shared = ClampedExpert(width, m["shared"]) if m.get("shared") else None
        self.shared_gate = nn.Parameter(torch.zeros(1, width)) if self.shared is not None else None
        self._tables = None


class ZubedraLayer(nn.Module):
    def __init__(self, config: ZubedraConfig, index):
        super().__init__()
        lc, w = config.layers[index], config.width
        self.kind = lc["type"]
        invalidInputError(self.kind in ("wkv", "attention"), f"unknown layer type {self.kind}")
        self.norm1 = _Weight(w)
        self.mixer = SinkAttention(w, lc["mixer"]) if self.kind == "attention" else WkvMixer(w, lc["mixer"], config.wkv_ranks.get(str(index), 1))
        self.mlp = SigmoidRoutedExperts(w, lc["mlp"]) if lc.get("mlp") is not None else None


def merge_projections(module: nn.Module, stack: bool = True):
    """the three projections that read an attention mixer's input become one ``in_proj``.  The four wide projections of a wkv mixer
    read four different token-shifted inputs; with ``stack`` (the linears stay plain matrices: no low-bit conversion follows) they
    become the parameter ``rkvg`` [4, heads * dim, width], one batched product instead of four"""
    if isinstance(module, SinkAttention) and not hasattr(module, "in_proj"):
        module.in_proj = merge_linear([module.q_proj, module.k_proj, module.v_proj])
        del module.q_proj, module.k_proj, module.v_proj
    elif isinstance(module, WkvMixer) and stack and not hasattr(module, "rkvg"):
        parts = [module.r_proj, module.k_proj, module.v_proj, module.g_proj]
        if all(type(p) is nn.Linear and p.bias is None for p in parts):
            module.rkvg = nn.Parameter(torch.stack([p.weight.data for p in parts]), requires_grad=False)
            del module.r_proj, module.k_proj, module.v_proj, module.g_proj


class ZubedraModel(nn.Module):
    def __init__(self, config: ZubedraConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab, config.width)
        self.layers = nn.ModuleList([ZubedraLayer(config, i) for i in range(len(config.layers))])
        self.norm = _Weight(config.width)


def _into(linear, x, out):
    """out[:] = linear(x): a plain matrix writes its product straight into ``out`` (a contiguous [N, rows] part of a buffer)"""
    if type(linear) is nn.Linear and linear.bias is None:
        torch.mm(x, linear.weight.t(), out=out)
    else:
        out.copy_(linear(x))


class ZubedraForCausalLM(PreTrainedModel, GenerationMixin):
    config_class = ZubedraConfig
    base_model_prefix = "model"
    _no_split_modules = ["ZubedraLayer"]
    _supports_attention_backend = False
    main_input_name = "input_ids"

    def __init__(self, config: ZubedraConfig):
        super().__init__(config)
        self.model = ZubedraModel(config)
        self.lm_head = nn.Linear(config.width, config.vocab, bias=False)
        self.collect_residual = None          # a list: gets the residual stream after every layer (debugging aid)
        self.attention_tensor_cores = True    # 16-bit models: prompts take the tensor-core attention kernel

    def _init_weights(self, module):
        pass

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    # ---- sublayers (h: the normalised stream in the model's dtype, [N, W])
    def _attention(self, mx, h, kv, B, S, cache, v_first):
        """returns (output [N, W], this layer's own value columns: a view of the projection)"""
        invalidInputError(hasattr(mx, "in_proj"), "the mixers' projections are merged at load time (merge_projections)")
        H, G, D, Dv = mx.heads, mx.kv_heads, mx.dim, mx.vdim
        proj = mx.in_proj(h)                                                 # [N, H D + G D + G Dv]
        off_k = H * D
        off_v = off_k + G * D
        like_k = torch.empty((B, G, 0, D), dtype=h.dtype, device=h.device)
        like_v = torch.empty((B, G, 0, Dv), dtype=h.dtype, device=h.device)
        k_store, v_store, held = kv.slots(like_k, like_v, S)
        shift = cache.seen - held                                            # storage index + shift = slot number
        # a recorded decode step reads the length from the device (the value given here is the one at recording time)
        dyn = kv.length_dev if (cache.frozen and S == 1) else None
        own_v = proj[:, off_v:off_v + G * Dv]
        if v_first is not None:
            invalidInputError(v_first.shape == own_v.shape, "layers that blend values must have values of one size")
        q = ops.wide_qkv_prepare(proj.view(B, S, proj.shape[-1]), 0, off_k, off_v, H, G, D, Dv, mx.q_norm.weight, mx.k_norm.weight,
                                 self.config.norm_eps, v_first, mx.vmix, k_store, v_store, kv.capacity(), held, shift, cache.pad, dyn)
        kv.commit(S)
        o = ops.softmax_attention(q, k_store.permute(0, 2, 1, 3), v_store.permute(0, 2, 1, 3), B, S, H, held, shift, cache.pad, 0, mx.scale,
                                  dyn=dyn, tensor_cores=self.attention_tensor_cores, softcap=mx.softcap, sink=mx.sink)
        return mx.o_proj(o), own_v

    def _wkv(self, mx, h, rec, B, S, cache):
        H, D, N = mx.heads, mx.dim, B * S
        hd = H * D
        tail, tail_next = rec.tails(B, 2, h.shape[-1], h.dtype, h.device)     # the previous token's input, [B, 1, W]
        pad = cache.pad if cache.seen == 0 else None                         # padding only ever precedes a row's first call
        mix = ops.token_shift_mix(h.view(B, S, -1), mx.mu, tail, tail if S == 1 else tail_next, cache.seen, pad)
        if S > 1:
            tail.copy_(tail_next)                                            # the tail keeps its address (a recorded step holds it)
        rkvg = torch.empty(4, N, hd, dtype=h.dtype, device=h.device)
        if hasattr(mx, "rkvg"):
            torch.bmm(mix[:4], mx.rkvg.transpose(1, 2), out=rkvg)
        else:
            for i, lin in enumerate((mx.r_proj, mx.k_proj, mx.v_proj, mx.g_proj)):
                _into(lin, mix[i], rkvg[i])
        z = mx.w2_proj(torch.tanh(mx.w1_proj(mix[4])))                       # decay logits [N, H D]
        state = rec.matrix(B, H, D, D, h.device)
        o = ops.wkv(rkvg[0], rkvg[1], rkvg[2], B, S, H, D, z, mx.w0, mx.u, state, cache.seen, pad)
        out = torch.empty(N, hd, dtype=h.dtype, device=h.device)
        ops.gated_rms_norm(o, rkvg[3], 0, mx.norm.weight, self.config.norm_eps, out, 0, 1.0)
        return mx.o_proj(out)

    def _experts(self, mlp, h, frozen_step):
        """fp32 [N, W]"""
        idx, wgt, gate = ops.scored_router(h, mlp.router, mlp.correction, mlp.groups, mlp.keep, mlp.top, sigmoid=True, group_top=GROUP_TOP,
                                           renorm=True, scale=mlp.scale, gate_row=mlp.shared_gate)
        N, E = h.shape[0], mlp.n_experts
        tables = experts.address_tables(mlp, h.dtype, h.device) if (N <= experts.MOE_SMALL_TOKENS or frozen_step) else None
        shared_out = None
        if mlp.shared is not None and (tables is None or not tables[4]):
            shared_out = mlp.shared(h)
        if tables is not None:
            gate_up, down, ffs, ff_max, with_shared = tables
            if shared_out is not None:                                       # a converted shared expert beside plain experts
                shared_out = (shared_out.to(torch.float32) * gate.unsqueeze(1)).to(h.dtype)
            return ops.moe_small(h, idx, wgt, gate_up, down, ff_max, E, E, shared_out, ffs=ffs, always_on=with_shared, always_w=gate,
                                 clamped=True, limit=mlp.limit, limit_always=mlp.shared.limit if mlp.shared is not None else 0.0)
        return experts.sorted_experts(mlp, h, idx, wgt, E, lambda gu, expert: ops.clamped_glu(gu, expert.ff, expert.limit), shared_out, gate)

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
        frozen_step = cache.frozen and S == 1
        # padding only occurs in a batch's first call; later calls (a replayed step among them, whose slot number is the one at
        # recording time) say so by passing no padding
        x, _ = ops.embed_pair(core.embed_tokens.weight, cfg.embedding.get("scale", 1.0), None, 0, 0, 0, input_ids, None, cache.seen,
                              cache.pad if cache.seen == 0 else None, dtype)
        first_blend, v_first = cfg.first_blending_layer(), None
        y_mix = y_ff = None                                                  # the last layer's results, not yet added to x
        for i, layer in enumerate(core.layers):
            h = ops.layer_norm_residual(x, y_mix, y_ff, layer.norm1.weight, eps, dtype)
            if layer.kind == "attention":
                blend = layer.mixer.blend and i != first_blend
                y_mix, own_v = self._attention(layer.mixer, h, cache.run_state(i, window=0).kv, B, S, cache, v_first if blend else None)
                if i == first_blend:
                    v_first = own_v
            else:
                y_mix = self._wkv(layer.mixer, h, cache.run_state(i).rec, B, S, cache)
            y_ff = self._experts(layer.mlp, h, frozen_step) if layer.mlp is not None else None
            if self.collect_residual is not None:
                ops.layer_norm_residual(x, y_mix, y_ff, None, eps, dtype, want_out=False)
                y_mix = y_ff = None
                self.collect_residual.append(x.view(B, S, -1).clone())
        cache.advance(S)
        if isinstance(logits_to_keep, int) and logits_to_keep == 0:
            hn = ops.layer_norm_residual(x, y_mix, y_ff, core.norm.weight, eps, dtype).view(B, S, -1)
        else:
            ops.layer_norm_residual(x, y_mix, y_ff, None, eps, dtype, want_out=False)
            idx = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep.to(dev)
            xk = x.view(B, S, -1)[:, idx, :].contiguous()
            hn = ops.layer_norm_residual(xk.view(-1, xk.shape[-1]), None, None, core.norm.weight, eps, dtype).view(B, xk.shape[1], -1)
        # every kept position as a row of its own ([rows, 1, W]): a converted lm_head keeps only the last position of a long
        # sequence axis (the reference's prefill shortcut), and which positions to keep is decided here, by logits_to_keep
        logits = self.lm_head(hn.reshape(-1, 1, hn.shape[-1])).to(torch.float32).view(B, hn.shape[1], -1)
        if cfg.logit_scale != 1.0:
            logits = logits * cfg.logit_scale
        return CausalLMOutputWithPast(logits=logits, past_key_values=cache)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, **kwargs):
        """generate() hands over every token so far; the model takes those its cache has not seen"""
        seen = past_key_values.get_seq_length() if isinstance(past_key_values, DynamicStateCache) else 0
        return {"input_ids": input_ids[:, seen:], "attention_mask": attention_mask, "past_key_values": past_key_values,
                "use_cache": True, "logits_to_keep": 1}


# ------------------------------------------------------------------ checkpoint
def checkpoint_key_map(config: ZubedraConfig):
    """the model's parameter names -> the checkpoint's tensor names: one name, a list of them (concatenated by rows), or a tuple
    (stacked as the rows of a matrix)"""
    m = {"model.embed_tokens.weight": "embed", "lm_head.weight": "head", "model.norm.weight": "final.norm"}
    for i, lc in enumerate(config.layers):
        d, s = f"model.layers.{i}.", f"l{i}."
        m[d + "norm1.weight"] = s + "norm1"
        dm, sm = d + "mixer.", s + "mix."
        if lc["type"] == "attention":
            for n in ("q", "k", "v", "o"):
                m[dm + n + "_proj.weight"] = sm + n
            m[dm + "q_norm.weight"], m[dm + "k_norm.weight"] = sm + "q.norm", sm + "k.norm"
            m[dm + "vmix"], m[dm + "sink"] = sm + "vmix", sm + "sink"
        else:
            m[dm + "mu"] = tuple(sm + "mu." + n for n in SHIFTS)
            for n in ("r", "k", "v", "g", "w1", "w2", "o"):
                m[dm + n + "_proj.weight"] = sm + n
            m[dm + "w0"], m[dm + "u"], m[dm + "norm.weight"] = sm + "w0", sm + "u", sm + "norm"
        mlp = lc.get("mlp")
        if mlp is not None:
            dp, sp = d + "mlp.", s + "mlp."
            m[dp + "router"], m[dp + "correction"] = sp + "router", sp + "correction"
            names = [(f"experts.{e}.", f"e{e}.") for e in range(int(mlp["router"]["experts"]))]
            if mlp.get("shared"):
                names.append(("shared.", "shared."))
                m[dp + "shared_gate"] = sp + "shared.sg"
            for dn, sn in names:
                m[dp + dn + "gate_up.weight"] = [sp + sn + "gate", sp + sn + "up"]
                m[dp + dn + "down.weight"] = sp + sn + "down"
    return m


def load_pretrained(model_dir, torch_dtype=None, device=None):
    """config.json + model.safetensors of the design -> a ``ZubedraForCausalLM``.  Sizes that config.json does not state (the
    rank of a wkv layer's decay projection) come from the tensors' shapes."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    if "wkv_ranks" not in raw:
        raw["wkv_ranks"] = {str(i): tensors[f"l{i}.mix.w1"].shape[0] for i, lc in enumerate(raw.get("layers", []))
                            if lc["type"] == "wkv" and f"l{i}.mix.w1" in tensors}
    config = ZubedraConfig(**raw)
    if torch_dtype in (None, "auto"):
        torch_dtype = tensors["embed"].dtype
    with torch.device("meta"):
        model = ZubedraForCausalLM(config)
    state = {}
    for dst, src in checkpoint_key_map(config).items():
        names = [src] if isinstance(src, str) else list(src)
        missing = [s for s in names if s not in tensors]
        if missing and dst.endswith(".vmix"):                                # a layer that blends nothing may come without its weight
            state[dst] = torch.zeros((), dtype=torch_dtype)
            continue
        invalidInputError(not missing, f"the checkpoint has no tensor {missing}")
        if isinstance(src, str):
            t = tensors[src]
        elif isinstance(src, tuple):
            t = torch.stack([tensors[s] for s in src], dim=0)
        else:
            t = torch.cat([tensors[s] for s in src], dim=0)
        state[dst] = t.to(torch_dtype)
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
        AutoConfig.register("zubedra", ZubedraConfig)
        AutoModelForCausalLM.register(ZubedraConfig, ZubedraForCausalLM)
    except ValueError:                                                       # registered already
        pass


_register()
