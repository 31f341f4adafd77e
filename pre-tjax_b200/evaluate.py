"""Evaluation and inference callers of the GPT-2 path, on the same sm_100a kernels with ``train=False`` semantics.

Mirrors the callers the reference's train script uses between training steps:

* ``t_gpt2_forward``  – logits only (model_triton.py:2523-2527, the forward without saved activations)
* ``t_loss`` / ``loss_eval`` – ``(loss, (loss, accuracy, valid fraction))`` (loss_and_optimizer_triton.py:217-232)
* ``log_probs``       – per-sequence sum of label log-probabilities, HellaSwag-style scoring (:293-311)
* ``predict``         – greedy decoding that re-runs the whole forward for every new token (:203-212)

With ``train=False`` every dropout site multiplies by ``1 - DROPOUT_RATE`` (model_torch_func.py:98-102) instead of
drawing a mask. The quirks of the reference are kept because its outputs are the contract: ``log_probs`` adds **1**
for every padding label (``torch.where(y != 0, elem, 1)``, loss_and_optimizer_triton.py:306), and ``predict`` blanks a
position when the running maximum of the token ids equals ``end_tok`` (:209).
"""
from __future__ import annotations

from functools import partial

import torch

from . import operators as ops
from .gpt2 import Gpt2Step, Weights, _seeds_or_zero, config_from_params


def _forward_padded(params, ids, train, p_gen_aux, y_mask=None):
    """(logits [B*S, vocab_ld], cfg, step): the first cfg.vocab columns of a row are valid."""
    cfg = config_from_params(params, ops.DROPOUT_RATE)
    step = Gpt2Step(cfg, params[0][0].dtype)
    w = Weights.from_pytree(params, cfg, step.dtype)
    logits, _ = step.forward(w, ids.to(torch.int32).contiguous(), train, _seeds_or_zero(p_gen_aux, cfg),
                             row_kstart=ops._kstart_or_none(y_mask))
    return logits, cfg, step


def t_gpt2_forward(params, y, y_mask=None, y_indices=None, train=True, p_gen_aux=None):
    """logits [B, S, V] for token ids y [B, S]. y_mask [B,S,S] bool: the collator's causal x block-diagonal x padding
    mask (None = causal); y_indices are ignored, as in the reference."""
    logits, cfg, _ = _forward_padded(params, y, train, p_gen_aux, y_mask)
    B, S = y.shape
    return logits.view(B, S, -1)[:, :, :cfg.vocab]


def t_loss(params, y, y_mask=None, y_indices=None, train=True, p_gen_aux=None):
    """y [B, S+1]: inputs y[:, :-1], labels y[:, 1:]. Returns (loss, (loss, accuracy, fraction of labels != 0)),
    the shape ``_loss`` returns (loss_and_optimizer_triton.py:221-230); one fused kernel produces all three."""
    labels = y[:, 1:].contiguous()
    logits, cfg, _ = _forward_padded(params, y[:, :-1], train, p_gen_aux, y_mask)
    stats, _, _ = ops.cross_entropy(labels, logits, cols=cfg.vocab, want_grad=False)
    return stats[0], (stats[0], stats[1], stats[2])


loss_eval = partial(t_loss, train=False)


def log_probs(params, y, y_mask=None, y_indices=None):
    """float32[B]: for each sequence the sum over positions of log softmax(logits)[label], evaluated with
    ``train=False``; a padding label (id 0) contributes +1, as in the reference."""
    B = y.shape[0]
    labels = y[:, 1:].contiguous()
    logits, cfg, _ = _forward_padded(params, y[:, :-1], False, None, y_mask)
    _, _, _, row_loss = ops.cross_entropy(labels, logits, cols=cfg.vocab, want_grad=False, want_rows=True)
    elems = torch.where(labels.reshape(-1) != 0, -row_loss, torch.ones_like(row_loss))
    return elems.view(B, -1).sum(dim=1)


def predict(params, y_mask, y_indices, sample_len, start_tok, end_tok):
    """Greedy decoding of ``y_mask.shape[0]`` sequences (an int batch size is accepted too): int64[B, sample_len-1].
    Every step runs the full forward over the ``sample_len`` positions (the reference has no KV cache) and takes the
    arg-max of position ``step`` with the row arg-max kernel. ``sample_len`` must equal the model's sequence length
    because the positional table is added without slicing."""
    B = int(y_mask) if isinstance(y_mask, int) else y_mask.shape[0]
    device = params[0][0].device
    y_sample = torch.full((B, sample_len), start_tok, device=device, dtype=torch.int64)
    for step_i in range(sample_len - 1):
        logits, cfg, _ = _forward_padded(params, y_sample, False, None)
        rows = logits.view(B, sample_len, -1)[:, step_i]  # [B, vocab_ld], row stride sample_len * vocab_ld
        y_sample[:, step_i + 1] = ops.argmax_rows(rows, cols=cfg.vocab).to(torch.int64)
    # the END token and what follows become padding (the reference tests the running maximum of the ids)
    y_sample = torch.where(torch.cummax(y_sample, dim=1)[0] != end_tok, y_sample, torch.zeros_like(y_sample))
    y_sample = y_sample[:, 1:]
    return torch.where(y_sample != start_tok, y_sample, torch.zeros_like(y_sample))
