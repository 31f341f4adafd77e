"""AdamW, gradient norm and parameter initialisation with the reference's signatures.

``adam_w_in_place`` / ``init_adam_w`` / ``grads_l2norm`` follow loss_and_optimizer_triton.py:362-416; the update of
every tensor is ONE fused kernel instead of ~17 elementwise launches, and it really is in place.
"""
from __future__ import annotations

import math
from typing import List

import torch

from . import _lib
from .gpt2 import GPT2Config, unflatten_like
from .operators import _ptr, _stream

INIT_SCALE = 2e-2  # model_torch_func.py:3


def init_transformer_gpt2(vocab_size, emb_dim, layers, num_heads, ffn_dim, seq_len, device="cuda", seed=None):
    """Parameter pytree with the reference's shapes, scales and draw order (model_torch_func.py:12-43): N(0, 0.02)
    weights, output projections of both sub-blocks scaled by 1/sqrt(2 L), zero biases, unit LayerNorm scales.
    Drawn on the CPU generator (optionally seeded) and moved to `device`, so a given seed yields the same values
    as the reference run with its DEVICE set to "cpu"."""
    if seed is not None:
        torch.manual_seed(seed)
    res = INIT_SCALE / math.sqrt(2 * layers)
    dh = emb_dim // num_heads
    rn = lambda *shape: torch.randn(shape)
    params = [[INIT_SCALE * rn(vocab_size, emb_dim), torch.zeros(vocab_size)], [INIT_SCALE * rn(seq_len, emb_dim)]]
    for _ in range(layers):
        params.append([
            torch.ones(emb_dim), torch.zeros(emb_dim),
            INIT_SCALE * rn(num_heads, 3, dh, emb_dim), res * rn(emb_dim, emb_dim),
            torch.ones(emb_dim), torch.zeros(emb_dim),
            INIT_SCALE * rn(ffn_dim, emb_dim), torch.zeros(ffn_dim),
            res * rn(emb_dim, ffn_dim), torch.zeros(emb_dim),
        ])
    params.append([torch.ones(emb_dim), torch.zeros(emb_dim)])
    return [[t.to(device) for t in grp] for grp in params]


def init_from_config(cfg: GPT2Config, device="cuda", seed=None):
    return init_transformer_gpt2(cfg.vocab, cfg.dim, cfg.layers, cfg.heads, cfg.ffn, cfg.seq, device=device, seed=seed)


def count_num_params(params) -> int:
    return sum(sum(p.numel() for p in grp) for grp in params)


def weight_decay_mask(params):
    """train_gpt2_triton.py:69-71: no decay for 1-D tensors that are all zero at initialisation."""
    return tuple(tuple(not (p.ndim == 1 and bool((p == 0).all())) for p in grp) for grp in params)


def init_adam_w(params):
    """(zero gradients, [first moments, second moments]) (loss_and_optimizer_triton.py:362-363)."""
    z = lambda: [[torch.zeros_like(p) for p in grp] for grp in params]
    return z(), [z(), z()]


def adam_w_in_place(params, grads, lr, betas, epsilon, moments, i, weight_decay=0.0, weight_decay_mask=None):
    """One AdamW step with t = i + 1 (loss_and_optimizer_triton.py:376-401). Updates params and moments in place
    and returns them. Tensors must be float32 CUDA tensors."""
    t = int(i) + 1
    lib = _lib.lib()
    for gi, grp in enumerate(params):
        for pi, p in enumerate(grp):
            g, m, v = grads[gi][pi], moments[0][gi][pi], moments[1][gi][pi]
            for x in (p, g, m, v):
                if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
                    raise RuntimeError("adam_w_in_place needs contiguous float32 CUDA tensors")
            wd = weight_decay if (weight_decay_mask is None or weight_decay_mask[gi][pi]) else 0.0
            n = p.numel()
            n4 = n - n % 4
            if n4:
                _lib.check(lib.ptj_adamw(_ptr(p), _ptr(g), _ptr(m), _ptr(v), 0, n4, 0, 0, 0, lr, betas[0], betas[1],
                                         epsilon, wd, t, 1.0, 0, 0.0, _stream()), "ptj_adamw")
            if n != n4:  # ragged tail (e.g. a bias of 50257 entries): pad to one vector
                tail = [torch.zeros(4, device=p.device) for _ in range(4)]
                views = [x.view(-1)[n4:] for x in (p, g, m, v)]
                for dst, src in zip(tail, views):
                    dst[: n - n4] = src
                _lib.check(lib.ptj_adamw(*[_ptr(x) for x in tail], 0, 4, 0, 0, 0, lr, betas[0], betas[1], epsilon, wd, t,
                                         1.0, 0, 0.0, _stream()), "ptj_adamw")
                for dst, src in zip((views[0], views[2], views[3]), (tail[0], tail[2], tail[3])):
                    dst.copy_(src[: n - n4])
    return params, moments


def sumsq(flat: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Sum of squares of a float32 vector as a device scalar (deterministic two-stage reduction)."""
    if out is None:
        out = torch.empty(1, device=flat.device, dtype=torch.float32)
    n = flat.numel()
    ns = _lib.lib().ptj_sumsq_scratch_floats(n)
    scratch = torch.empty(ns, device=flat.device, dtype=torch.float32)
    _lib.check(_lib.lib().ptj_sumsq(_ptr(flat), _ptr(out), _ptr(scratch), ns, n, _stream()), "ptj_sumsq")
    return out


def grads_l2norm(grads) -> float:
    """Global L2 norm of a gradient pytree (loss_and_optimizer_triton.py:411-416)."""
    total = 0.0
    for grp in grads:
        for g in grp:
            total += float(sumsq(g.contiguous().view(-1).float()).item())
    return math.sqrt(total)


def pytree_like(cfg: GPT2Config, flat: List[torch.Tensor]):
    return unflatten_like(flat, cfg)
