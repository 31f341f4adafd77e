"""Generates ``eval_callers.npz`` by RUNNING THE REFERENCE's evaluation / inference callers on the CPU.

Usage (only where a checkout of martin-kukla/pre-tjax is available):

    PTJ_REFERENCE_DIR=/path/to/pre-tjax python tests/golden/make_golden_eval.py

Inputs are the weights and token ids of ``tiny_model.npz`` (made by make_golden.py, which must run first). The
dropout rate is 0.1 so that the eval-time ``x * (1 - p)`` scaling shows in every output. Stored:

  loss, acc, frac      lot.loss(params, y, mask, idx, train=False)           (what loss_eval compiles)
  log_probs            lot.log_probs(params, y, mask, idx)                   (+1 per padding label, as the reference)
  predict              lot.predict(params', mask, idx, 16, start_tok, end_tok) greedy decode, full forward per token.
                       With the toy weights every position would repeat its input token (tied embedding), so this
                       case swaps in a large positional table and a small random head bias (stored as w_pos_pred,
                       b_head_pred), which makes the decoded ids differ from position to position.
  logits_eval          batched_forward_gpt2(params, y[:, :-1], mask, idx, False)
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from make_golden import causal_mask, load_reference, npy

OUT = Path(__file__).resolve().parent
DROPOUT = 0.1
START_TOK, END_TOK = 1, 63  # END is the largest id: the reference blanks positions where cummax(ids) == end_tok


def main():
    mtf, mt, lot = load_reference(DROPOUT)
    g = np.load(OUT / "tiny_model.npz")
    V, D, L, H, F, S, B = (int(v) for v in g["dims"])
    flat = [torch.from_numpy(g[f"p{i}"]) for i in range(2 + 1 + 10 * L + 2)]
    it = iter(flat)
    params = [[next(it), next(it)], [next(it)]] + [[next(it) for _ in range(10)] for _ in range(L)] + [[next(it), next(it)]]
    y = torch.from_numpy(g["y"])
    mask = causal_mask(B, S)
    idx = torch.arange(S).unsqueeze(0).expand(B, S).contiguous()
    with torch.no_grad():
        loss, (_, acc, frac) = lot.loss(params, y, mask, idx, False)
        lp = lot.log_probs(params, y, mask, idx)
        gen = torch.Generator().manual_seed(11)
        w_pos_pred = torch.randn(S, D, generator=gen) * 4.0
        b_head_pred = torch.randn(V, generator=gen) * 0.05
        params_pred = [[params[0][0], b_head_pred], [w_pos_pred]] + params[2:]
        pred = lot.predict(params_pred, mask, idx, S, START_TOK, END_TOK)
        logits = mtf.batched_forward_gpt2(params, y[:, :-1], mask, idx, False)
    d = {"loss": npy(loss), "acc": npy(acc), "frac": npy(frac), "log_probs": npy(lp), "predict": npy(pred),
         "logits_eval": npy(logits), "w_pos_pred": npy(w_pos_pred), "b_head_pred": npy(b_head_pred), "dropout": np.float32(DROPOUT), "start_tok": np.int64(START_TOK),
         "end_tok": np.int64(END_TOK)}
    np.savez_compressed(OUT / "eval_callers.npz", **d)
    print("eval_callers.npz", (OUT / "eval_callers.npz").stat().st_size, "bytes; loss", float(loss), "log_probs", lp.tolist())
    print("predict", pred.tolist())


if __name__ == "__main__":
    main()
