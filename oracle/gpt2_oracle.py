"""CPU oracle for the GPT-2 training hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on the CPU, the arithmetic of the reference's torch.func model
(model_torch_func.py), its loss (loss_and_optimizer_triton.py) and its hand-written per-operator backward formulas
(model_triton.py). It exists to CHECK the CUDA kernels; nothing in the product imports it. Only tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import it.

Pinning: tests/golden/make_golden.py runs the real reference (imported from its checkout, unmodified) on seeded
inputs and stores its outputs (make_golden_eval.py and make_golden_packed.py do the same for the evaluation callers
and for batches packed by the reference's collator); tests/test_oracle_golden.py checks every function here against
those fixtures.
Dropout randomness is the one thing that cannot be pinned to the reference (its masks come from triton.language.rand
/ torch.bernoulli, which never agreed with each other either): the oracle takes the 0/1 masks as INPUTS, so the
semantics "multiply by the mask, do not rescale" are checked exactly while the bit stream is this project's Philox
(oracle/philox.py).

All functions work in the dtype of their inputs (float32 like the reference, or float64 for a tighter yardstick).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch

MaskFn = Optional[Callable[[str, torch.Size], torch.Tensor]]


# ---- elementary operators ------------------------------------------------------------------------------------------
def log_softmax(x: torch.Tensor) -> torch.Tensor:
    """model_torch_func.py:48-50."""
    x = x - x.max(dim=-1, keepdim=True).values
    return x - torch.logsumexp(x, dim=-1, keepdim=True)


def log_softmax_bwd(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """VJP of log_softmax: dy - softmax(x) * sum(dy)  (model_triton.py:91-102)."""
    return dy - torch.softmax(x, dim=-1) * dy.sum(dim=-1, keepdim=True)


def gelu(x: torch.Tensor) -> torch.Tensor:
    """tanh-GELU, model_torch_func.py:60-62."""
    k = math.sqrt(2.0 / math.pi)
    return 0.5 * x * (1.0 + torch.tanh(k * (x + 0.044715 * x ** 3)))


def gelu_bwd(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """model_triton.py:262-271."""
    k = math.sqrt(2.0 / math.pi)
    t = torch.tanh(k * (x + 0.044715 * x ** 3))
    dt = (1.0 - t * t) * k * (1.0 + 3.0 * 0.044715 * x * x)
    return dy * (0.5 * (1.0 + t) + 0.5 * x * dt)


def layernorm(gamma: torch.Tensor, beta: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Unbiased standard deviation, no epsilon: model_torch_func.py:104-108."""
    mean = x.mean(dim=-1, keepdim=True)
    std = x.std(dim=-1, keepdim=True)  # torch default: divide by n - 1
    return (x - mean) / std * gamma + beta


def layernorm_bwd(dy: torch.Tensor, gamma: torch.Tensor, x: torch.Tensor):
    """(dx, dgamma, dbeta): model_triton.py:1773-1783 and :1652-1660."""
    n = x.shape[-1]
    mean = x.mean(dim=-1, keepdim=True)
    rstd = 1.0 / x.std(dim=-1, keepdim=True)
    xh = (x - mean) * rstd
    lead = tuple(range(x.dim() - 1))
    dgamma = (dy * xh).sum(dim=lead)
    dbeta = dy.sum(dim=lead)
    g = dy * gamma
    dx = (g - g.mean(dim=-1, keepdim=True) - xh * (g * xh).mean(dim=-1, keepdim=True) * (n / (n - 1.0))) * rstd
    return dx, dgamma, dbeta


def dropout(x: torch.Tensor, p: float, train: bool, mask: Optional[torch.Tensor]) -> torch.Tensor:
    """model_torch_func.py:98-102: training multiplies by a 0/1 mask WITHOUT rescaling; evaluation multiplies by 1-p."""
    if not train:
        return x * (1.0 - p)
    if mask is None:
        assert p == 0.0, "training-mode dropout with p > 0 needs an explicit mask"
        return x
    return x * mask.to(x.dtype)


def causal_attention(q, k, v, p: float = 0.0, train: bool = True, mask: Optional[torch.Tensor] = None,
                     attn_mask: Optional[torch.Tensor] = None):
    """q,k,v: [..., S, d]. softmax(masked(q k^T / sqrt(d)), fill -1e9) -> dropout on the probabilities -> @ v
    (model_torch_func.py:70-78). attn_mask: bool, broadcastable to [..., S, S], True = attend (the collator's
    causal x block-diagonal x padding mask, tokenized_dataset.py:110-131); None = causal. A row without any True
    gets -1e9 everywhere and therefore attends all keys uniformly, as in the reference.
    Returns (out, probabilities before dropout)."""
    S, d = q.shape[-2], q.shape[-1]
    s = q @ k.transpose(-2, -1) / math.sqrt(d)
    tri = torch.tril(torch.ones(S, S, dtype=torch.bool)) if attn_mask is None else attn_mask
    s = torch.where(tri, s, torch.full_like(s, -1e9))
    pr = torch.exp(log_softmax(s))
    return dropout(pr, p, train, mask) @ v, pr


def causal_attention_stats(q, k):
    """Row maximum of the scaled, masked scores and sum of exp(score - max): what the reference's flash kernel
    stores as acts0 / acts1 (model_triton.py:699-700)."""
    S, d = q.shape[-2], q.shape[-1]
    s = q @ k.transpose(-2, -1) / math.sqrt(d)
    tri = torch.tril(torch.ones(S, S, dtype=torch.bool))
    s = torch.where(tri, s, torch.full_like(s, float("-inf")))
    m = s.max(dim=-1).values
    return m, torch.exp(s - m.unsqueeze(-1)).sum(dim=-1)


def causal_attention_bwd(d_out, q, k, v, p: float = 0.0, train: bool = True, mask: Optional[torch.Tensor] = None,
                         attn_mask: Optional[torch.Tensor] = None):
    """(dq, dk, dv): model_triton.py:801-811 with :550-577."""
    d = q.shape[-1]
    _, pr = causal_attention(q, k, v, p, train, mask, attn_mask)
    prd = dropout(pr, p, train, mask)
    dv = prd.transpose(-2, -1) @ d_out
    dprd = d_out @ v.transpose(-2, -1)
    dpr = dropout(dprd, p, train, mask)
    ds = pr * (dpr - (dpr * pr).sum(dim=-1, keepdim=True))
    if attn_mask is not None:  # the fill value carries no gradient (model_triton.py:568): matters for rows without keys
        ds = torch.where(attn_mask, ds, torch.zeros_like(ds))
    dq = ds @ k / math.sqrt(d)
    dk = ds.transpose(-2, -1) @ q / math.sqrt(d)
    return dq, dk, dv


def avg_cross_entropy_loss(labels: torch.Tensor, logits: torch.Tensor):
    """(mean of -log_softmax[label] over labels != 0, count of labels != 0): loss_and_optimizer_triton.py:26-32."""
    lab = labels.reshape(-1).long()
    lg = logits.reshape(lab.numel(), -1)
    picked = log_softmax(lg)[torch.arange(lab.numel()), lab]
    valid = lab != 0
    return -(picked[valid]).mean() if valid.any() else picked.new_tensor(float("nan")), valid.sum()


def cross_entropy_fwd_bwd(labels: torch.Tensor, logits: torch.Tensor):
    """(loss, n_valid, dlogits) with dlogits = (softmax - onehot) / n_valid on rows with label != 0 and 0 elsewhere:
    loss_and_optimizer_triton.py:83-106."""
    lab = labels.reshape(-1).long()
    lg = logits.reshape(lab.numel(), -1)
    loss, n_valid = avg_cross_entropy_loss(labels, logits)
    g = torch.softmax(lg, dim=-1)
    g[torch.arange(lab.numel()), lab] -= 1.0
    g = g / n_valid.to(g.dtype)
    g[lab == 0] = 0.0
    return loss, n_valid, g.reshape(logits.shape)


def accuracy(labels: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """loss_and_optimizer_triton.py:199-200."""
    valid = labels != 0
    hit = labels.long() == logits.argmax(dim=-1)
    return hit[valid].to(logits.dtype).mean()


# ---- the model ---------------------------------------------------------------------------------------------------------
def forward_gpt2(params, ids: torch.Tensor, p: float = 0.0, train: bool = True, mask_fn: MaskFn = None,
                 attn_mask: Optional[torch.Tensor] = None):
    """Batched forward pass: [B, S] token ids -> [B, S, V] logits (model_torch_func.py:110-133, batched directly
    instead of through vmap). mask_fn(site, shape) supplies dropout masks; sites are "embed", "l{i}.attn",
    "l{i}.res1", "l{i}.res2". attn_mask: the batch's attention mask [B, S, S] bool (y_mask of the reference,
    shared by all heads), None = causal."""
    am = None if attn_mask is None else attn_mask.bool().unsqueeze(1)
    mk = (lambda site, shape: mask_fn(site, shape)) if (mask_fn is not None and train) else (lambda site, shape: None)
    w_emb, b_head = params[0]
    (w_pos,) = params[1]
    D = w_emb.shape[1]
    x = w_emb[ids.long()] * math.sqrt(D) + w_pos  # model_torch_func.py:54-55, 120-121
    x = dropout(x, p, train, mk("embed", x.shape))
    for i, lp in enumerate(params[2:-1]):
        g1, b1, w_qkv, w_o, g2, b2, w1, b1f, w2, b2f = lp
        H = w_qkv.shape[0]
        h = layernorm(g1, b1, x)
        # per-head projections: q_h = h W[h,0]^T etc. (model_torch_func.py:80-82)
        qkv = torch.einsum("bsd,hced->bhcse", h, w_qkv)  # [B, H, 3, S, dh]
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        a, _ = causal_attention(q, k, v, p, train, mk(f"l{i}.attn", (q.shape[0], H, q.shape[2], q.shape[2])), am)
        a = a.permute(0, 2, 1, 3).reshape(x.shape)  # concatenate heads along the feature axis (:88)
        a = a @ w_o.t()
        x = x + dropout(a, p, train, mk(f"l{i}.res1", x.shape))
        h = layernorm(g2, b2, x)
        f = gelu(h @ w1.t() + b1f) @ w2.t() + b2f
        x = x + dropout(f, p, train, mk(f"l{i}.res2", x.shape))
    gf, bf = params[-1]
    x = layernorm(gf, bf, x)
    return x @ w_emb.t() + b_head  # tied output projection with its own bias (:132)


def loss_and_grads(params, y: torch.Tensor, p: float = 0.0, train: bool = True, mask_fn: MaskFn = None,
                   attn_mask: Optional[torch.Tensor] = None):
    """(grads pytree, (loss, accuracy, valid fraction)) for y [B, S+1]: inputs y[:, :-1], labels y[:, 1:]
    (loss_and_optimizer_triton.py:221-235). Gradients come from autograd over the restated forward."""
    leaves = [[t.detach().clone().requires_grad_(True) for t in grp] for grp in params]
    logits = forward_gpt2(leaves, y[:, :-1], p, train, mask_fn, attn_mask)
    labels = y[:, 1:]
    loss, n_valid = avg_cross_entropy_loss(labels, logits)
    flat = [t for grp in leaves for t in grp]
    gflat = torch.autograd.grad(loss, flat, allow_unused=True)
    gflat = [g if g is not None else torch.zeros_like(t) for g, t in zip(gflat, flat)]
    it = iter(gflat)
    grads = [[next(it) for _ in grp] for grp in leaves]
    acc = accuracy(labels, logits.detach())
    return grads, (loss.detach(), acc, n_valid.to(loss.dtype) / labels.numel())


# ---- evaluation / inference callers ------------------------------------------------------------------------------------
def loss_eval(params, y: torch.Tensor, p: float):
    """(loss, accuracy, valid fraction) with every dropout site in eval mode, i.e. scaled by 1 - p
    (loss_and_optimizer_triton.py:221-232 with train=False)."""
    logits = forward_gpt2(params, y[:, :-1], p, False)
    labels = y[:, 1:]
    loss, n_valid = avg_cross_entropy_loss(labels, logits)
    return loss, accuracy(labels, logits), n_valid.to(loss.dtype) / labels.numel()


def log_probs(params, y: torch.Tensor, p: float) -> torch.Tensor:
    """[B]: sum over positions of log softmax(logits)[label] in eval mode; a padding label (0) adds +1 instead
    (the reference's torch.where(labels != 0, elem, 1), loss_and_optimizer_triton.py:293-311)."""
    logits = forward_gpt2(params, y[:, :-1], p, False)
    labels = y[:, 1:].long()
    lp = log_softmax(logits).gather(-1, labels.unsqueeze(-1)).squeeze(-1)
    return torch.where(labels != 0, lp, torch.ones_like(lp)).sum(dim=1)


def predict(params, batch: int, sample_len: int, start_tok: int, end_tok: int, p: float) -> torch.Tensor:
    """Greedy decoding, full forward per new token (loss_and_optimizer_triton.py:203-212): [batch, sample_len - 1].
    Positions where the running maximum of the ids equals end_tok, and ids equal to start_tok, become 0."""
    ys = torch.full((batch, sample_len), start_tok, dtype=torch.int64)
    for i in range(sample_len - 1):
        logits = forward_gpt2(params, ys, p, False)
        ys[:, i + 1] = torch.argmax(logits[:, i], dim=-1)
    ys = torch.where(torch.cummax(ys, dim=1)[0] != end_tok, ys, torch.zeros_like(ys))[:, 1:]
    return torch.where(ys != start_tok, ys, torch.zeros_like(ys))


# ---- optimizer ---------------------------------------------------------------------------------------------------------
def adam_w(params, grads, lr, betas, eps, moments, i, weight_decay=0.0, decay_mask=None):
    """One AdamW step with t = i + 1; returns new (params, [m, v]): loss_and_optimizer_triton.py:376-401."""
    t = i + 1
    b1, b2 = betas
    new_p, new_m, new_v = [], [], []
    for gi, grp in enumerate(params):
        pp, mm, vv = [], [], []
        for pi, prm in enumerate(grp):
            g = grads[gi][pi]
            m = moments[0][gi][pi] * b1 + (1 - b1) * g
            v = moments[1][gi][pi] * b2 + (1 - b2) * g * g
            mh, vh = m / (1 - b1 ** t), v / (1 - b2 ** t)
            wd = weight_decay if (decay_mask is None or decay_mask[gi][pi]) else 0.0
            pp.append(prm + (-lr * (mh / (torch.sqrt(vh) + eps) + wd * prm)))
            mm.append(m)
            vv.append(v)
        new_p.append(pp); new_m.append(mm); new_v.append(vv)
    return new_p, [new_m, new_v]


def grads_l2norm(grads) -> float:
    """loss_and_optimizer_triton.py:411-416."""
    return math.sqrt(sum(float((g.double() ** 2).sum()) for grp in grads for g in grp))


def clip_scale(norm: float, max_norm: float) -> float:
    """Standard global-norm clipping factor min(1, c / (norm + 1e-6)); the reference only logs the norm."""
    return min(1.0, max_norm / (norm + 1e-6))


def decay_mask(params):
    """train_gpt2_triton.py:69-71."""
    return [[not (t.dim() == 1 and bool((t == 0).all())) for t in grp] for grp in params]


def init_params(vocab, dim, layers, heads, ffn, seq, seed: int, dtype=torch.float32):
    """Same shapes / scales / draw order as model_torch_func.py:12-43, on the CPU generator."""
    torch.manual_seed(seed)
    s, res, dh = 2e-2, 2e-2 / math.sqrt(2 * layers), dim // heads
    prm = [[s * torch.randn(vocab, dim), torch.zeros(vocab)], [s * torch.randn(seq, dim)]]
    for _ in range(layers):
        prm.append([torch.ones(dim), torch.zeros(dim), s * torch.randn(heads, 3, dh, dim), res * torch.randn(dim, dim),
                    torch.ones(dim), torch.zeros(dim), s * torch.randn(ffn, dim), torch.zeros(ffn),
                    res * torch.randn(dim, ffn), torch.zeros(dim)])
    prm.append([torch.ones(dim), torch.zeros(dim)])
    return [[t.to(dtype) for t in grp] for grp in prm]
