"""What the mixture-of-experts feed-forwards of this package's own designs share on the host: the device tables of the
experts' weight addresses (the path of a few tokens and of a recorded step, which runs no host code between router and result)
and the many-token path (the (token, choice) pairs sorted by expert on the device, one pair of matrix products per expert on
its rows, a weighted sum).  An expert is a module with ``gate_up`` [2 ff, width] (gate rows first) -- or, for an expert without a
gate, ``up`` [ff, width] --, ``down`` [width, ff] and ``ff``; the owner keeps ``experts`` (a ModuleList), ``shared`` (an expert
every token runs, or None) and a ``_tables`` slot.
"""
import torch
from torch import nn

from ipex_llm_b200.transformers.models import mixer_ops as ops

MOE_SMALL_TOKENS = 32         # up to this many tokens take the experts' host-free path


def first_matrix(expert):
    """the projection an expert applies to its input: gate and up rows together, or the up rows of an expert without a gate"""
    return expert.gate_up if hasattr(expert, "gate_up") else expert.up


def address_tables(mlp, dtype, device):
    """(gate_up addresses, down addresses, sizes, largest size, shared expert included?) as device arrays, or None when the
    experts are not plain matrices of ``dtype`` (converted to a low-bit format); rebuilt when the weights moved.  A shared
    expert that is a plain matrix too becomes the tables' last entry (the kernel runs it for every token)."""
    def plain(mods):
        return all(type(m) is nn.Linear and m.weight.dtype == dtype and m.weight.device == device and m.weight.is_contiguous() for m in mods)
    experts = list(mlp.experts)
    if not experts or not plain([m for e in experts for m in (first_matrix(e), e.down)]):
        return None
    with_shared = getattr(mlp, "shared", None) is not None and plain([first_matrix(mlp.shared), mlp.shared.down])
    if with_shared:
        experts.append(mlp.shared)
    key = (device, dtype, with_shared) + tuple(m.weight.data_ptr() for e in (experts[0], experts[-1]) for m in (first_matrix(e), e.down))
    if mlp._tables is None or mlp._tables[0] != key:
        def table(ws):
            return torch.tensor([w.weight.data_ptr() for w in ws], dtype=torch.int64, device=device)
        ffs = torch.tensor([e.ff for e in experts], dtype=torch.int32, device=device)
        mlp._tables = (key, table([first_matrix(e) for e in experts]), table([e.down for e in experts]), ffs, max(e.ff for e in experts), with_shared)
    return mlp._tables[1:]


def sorted_experts(mlp, h, idx, wgt, n_out, activation, shared_out=None, shared_w=None, weight_input=False):
    """fp32 [N, W] for many tokens: the pairs sorted by expert on the device (the counts are read on the host: the one
    synchronisation of the layer), then per expert ``down(activation(gate_up(rows), expert))`` straight into the sorted rows
    and the weighted sum.  Outputs numbered from len(experts) up to ``n_out`` are identity experts.  ``weight_input``: a
    choice's weight multiplies the expert's input rows (scattered into sorted order already weighted) instead of its output."""
    E = len(mlp.experts)
    counts, pos, token_of = ops.moe_sort(idx, n_out + 1)
    counts = counts[:E].tolist()
    rows = torch.empty(max(sum(counts), 1), h.shape[1], dtype=h.dtype, device=h.device)
    rows_in = ops.moe_scatter_scaled(h, pos, idx, wgt, E, sum(counts)) if weight_input else None
    off = 0
    for e, cnt in enumerate(counts):
        if cnt:
            expert = mlp.experts[e]
            x = rows_in[off:off + cnt] if weight_input else h.index_select(0, token_of[off:off + cnt])
            a = activation(first_matrix(expert)(x), expert)
            if type(expert.down) is nn.Linear:
                torch.mm(a, expert.down.weight.t(), out=rows[off:off + cnt])                 # straight into the sorted rows
            else:
                rows[off:off + cnt] = expert.down(a)
            off += cnt
    return ops.moe_combine(rows, pos, idx, None if weight_input else wgt, h, shared_out, E, n_out, shared_w=shared_w)
