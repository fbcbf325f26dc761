"""Mixture-of-experts feed-forward (Mixtral / DBRX style top-k routing).

Routing math follows the reference (`custom_modeling/flash_mixtral_modeling.py:449-459`): softmax over all experts,
keep the top k, renormalise the kept weights.  Expert weights are laid out expert-parallel: rank r holds experts
[r*E/ws, (r+1)*E/ws) in full (the reference shards every expert's FFN dimension across ranks instead,
`flash_mixtral_modeling.py:202-233`).  Hidden states are replicated after attention, so "dispatch" is a local
row selection and "combine" is the sum over ranks of the per-expert contributions.

On a GPU (bf16, experts as stacked tensors) the whole block runs on the device (`csrc/kernels/moe.cu`): routing kernel,
gather, a grouped tcgen05 GEMM over (expert, feature tile, token tile) work items for w1|w3, act * up, a second grouped GEMM
for w2 and the weighted combine.  Only the k experts of a token do work for it, every count stays on the device and every
launch has static shapes, so a decode step with experts is captured in a CUDA graph like a dense one.

Elsewhere (CPU, packed / quantised experts) two PyTorch shapes remain:
  * decode-sized batches: every local expert runs over all tokens and the routing weight (zero for unrouted tokens)
    scales its output;
  * prefill: tokens are gathered per expert, so each expert only computes the rows routed to it.
"""

from __future__ import annotations

import torch

DENSE_MAX_TOKENS = 256


def route(router_logits: torch.Tensor, k: int):
    """-> dense routing weights [T, E] (zero where an expert is not selected)."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    topv, topi = probs.topk(k, dim=-1)
    topv = topv / topv.sum(-1, keepdim=True)
    w = torch.zeros_like(probs)
    w.scatter_(1, topi, topv)
    return w


def moe_forward(model, x: torch.Tensor, lw, li: int, inp) -> torch.Tensor:
    c, ops = model.config, model.ops
    E = c.num_local_experts
    ws, rk = model.tp.world_size, model.tp.rank
    e_local = len(lw.experts_w13)             # a stacked tensor, or a list of packed (weight-only quantised) matrices
    e0 = rk * e_local if e_local < E else 0
    T = x.shape[0]
    if (x.is_cuda and x.dtype == torch.bfloat16 and isinstance(lw.experts_w13, torch.Tensor) and isinstance(lw.experts_w2, torch.Tensor)
            and lw.experts_w13.dtype == torch.bfloat16 and lw.experts_w13.shape[1] % 128 == 0 and lw.experts_w2.shape[1] % 128 == 0
            and model.hidden % 8 == 0 and c.intermediate_size % 8 == 0 and E <= 64 and c.num_experts_per_tok <= 8 and hasattr(ops, "moe_ffn")):
        out = ops.moe_ffn(x, lw.router_w.to(torch.bfloat16) if lw.router_w.dtype != torch.bfloat16 else lw.router_w, lw.experts_w13,
                          lw.experts_w2, c.num_experts_per_tok, e0, c.hidden_act)
        if ws > 1 and e_local < E:
            out = model.tp.all_reduce(out)
        return out
    # the router is tiny (E output features): plain matmul keeps it exact across ranks
    router_logits = x.float() @ lw.router_w.float().t()
    w = route(router_logits, c.num_experts_per_tok)
    out = torch.zeros(T, model.hidden, dtype=torch.float32, device=x.device)
    I = c.intermediate_size
    for j in range(e_local):
        e = e0 + j
        we = w[:, e]
        if T <= DENSE_MAX_TOKENS:
            gu = model._gemm(x, lw.experts_w13[j], None)
            a = ops.act_mul(gu, I, c.hidden_act, gated=True)
            dn = model._gemm(a, lw.experts_w2[j], None)
            out.addcmul_(dn.float(), we[:, None])
        else:
            idx = torch.nonzero(we > 0, as_tuple=False)[:, 0]
            if idx.numel() == 0:
                continue
            xe = x.index_select(0, idx).contiguous()
            gu = model._gemm(xe, lw.experts_w13[j], None)
            a = ops.act_mul(gu, I, c.hidden_act, gated=True)
            dn = model._gemm(a, lw.experts_w2[j], None)
            out.index_add_(0, idx, dn.float() * we.index_select(0, idx)[:, None])
    out = out.to(x.dtype)
    if ws > 1 and e_local < E:
        out = model.tp.all_reduce(out)
    return out
