"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE ITSELF on seeded inputs.

Usage (only where a checkout of martin-kukla/pre-tjax is available):

    PTJ_REFERENCE_DIR=/path/to/pre-tjax python tests/golden/make_golden.py

The reference modules are imported unmodified (on the CPU: its init helpers read the module constant DEVICE at call
time, and its dropout rate is a module constant that is patched to the value a case needs). Inputs are stored next
to the outputs, so the tests never depend on a random-number generator reproducing the same stream.

Fixtures written:
  ops_small.npz     per-operator inputs/outputs of the reference's plain-torch operator definitions
  tiny_model.npz    full loss / accuracy / every gradient of a 2-layer toy model from torch.func.grad
  cfg1_summary.npz  the "tiny GPT-2" benchmark configuration (2 layers, d_model 128, 4 heads, FFN 512, seq 128,
                    vocab 1024, batch 4, ids uniform in [0,1024) seed 0, dropout 0): loss, accuracy, per-tensor
                    gradient norms / sums and a strided sample of every gradient (full tensors would be 2 MB)
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

REF = os.environ.get("PTJ_REFERENCE_DIR")  # a checkout of martin-kukla/pre-tjax
OUT = Path(__file__).resolve().parent
SAMPLE_STRIDE = 97


def load_reference(dropout_rate: float):
    if not REF:
        raise SystemExit("set PTJ_REFERENCE_DIR to a checkout of martin-kukla/pre-tjax")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import model_torch_func as mtf
    mtf.DEVICE = "cpu"
    mtf.DROPOUT_RATE = dropout_rate
    import model_triton as mt
    mt.DROPOUT_RATE = dropout_rate
    import loss_and_optimizer_triton as lot
    return mtf, mt, lot


def npy(t):
    return t.detach().cpu().numpy()


def flat_params(params):
    return [t for grp in params for t in grp]


def causal_mask(B, S):
    return torch.tril(torch.ones((S, S), dtype=torch.bool)).unsqueeze(0).expand(B, S, S).contiguous()


def make_ops(mtf, mt, lot):
    g = torch.Generator().manual_seed(1234)
    rn = lambda *s: torch.randn(*s, generator=g)
    d = {}
    # LayerNorm
    x, gamma, beta, dy = rn(2, 5, 24), 1 + 0.1 * rn(24), 0.1 * rn(24), rn(2, 5, 24)
    d.update(ln_x=x, ln_gamma=gamma, ln_beta=beta, ln_dy=dy, ln_y=mt.t_layernorm_fwd((gamma, beta), x),
             ln_dx=mt.t_layernorm_bkwd2_x(dy, (gamma, beta), x))
    dg, db = mt.t_layernorm_bkwd2_p(dy, (gamma, beta), x)
    d.update(ln_dgamma=dg, ln_dbeta=db)
    # GELU
    x, dy = 2 * rn(3, 40), rn(3, 40)
    d.update(gelu_x=x, gelu_dy=dy, gelu_y=mt.t_gelu_fwd(x), gelu_dx=mt.t_gelu_bkwd2(dy, x))
    # log-softmax
    x, dy = 3 * rn(4, 37), rn(4, 37)
    d.update(lsm_x=x, lsm_dy=dy, lsm_y=mt.t_log_softmax_fwd(x), lsm_dx=mt.t_log_softmax_bkwd2(dy, x))
    # cross entropy (label 0 = padding)
    logits = 2 * rn(2, 6, 50)
    labels = torch.randint(0, 50, (2, 6), generator=g, dtype=torch.int32)
    labels[0, 1] = 0
    labels[1, 4] = 0
    loss, nvalid, dlog = lot.t_avg_cross_entropy_loss_bkwd3(labels, logits)
    loss2, nvalid2 = lot.t_avg_cross_entropy_loss(labels, logits)
    d.update(ce_logits=logits, ce_labels=labels, ce_loss=loss, ce_nvalid=nvalid, ce_dlogits=dlog, ce_loss_fwd=loss2,
             ce_acc=lot.accuracy(labels, logits))
    # attention, dropout rate 0 in training mode
    qkv, d_o = rn(2, 2, 3, 16, 8), rn(2, 2, 16, 8)
    mask = causal_mask(2, 16)
    out, acts = mt.t_scaled_dot_prod_attn_fwd3(qkv, mask, True, 1)
    dq, dk, dv = mt.t_scaled_dot_prod_attn_bkwd3(d_o, acts, qkv, mask, True, 1)
    d.update(attn_qkv=qkv, attn_do=d_o, attn_out=out, attn_probs=acts[0], attn_dq=dq, attn_dk=dk, attn_dv=dv)
    # FFN block
    w1, b1, w2, b2, x = 0.2 * rn(48, 24), 0.1 * rn(48), 0.2 * rn(24, 48), 0.1 * rn(24), rn(5, 24)
    d.update(ffn_w1=w1, ffn_b1=b1, ffn_w2=w2, ffn_b2=b2, ffn_x=x, ffn_y=mt.t_tlayer_ffn_fwd((w1, b1, w2, b2), x, mt.t_gelu_fwd))
    # AdamW, two steps with a decay mask
    params = [[rn(6, 4), torch.zeros(6)], [torch.ones(4)]]
    grads1 = [[rn(6, 4), rn(6)], [rn(4)]]
    grads2 = [[rn(6, 4), rn(6)], [rn(4)]]
    mask_wd = [[True, False], [True]]
    moments = [[[torch.zeros_like(p) for p in grp] for grp in params] for _ in range(2)]
    p0 = [[p.clone() for p in grp] for grp in params]
    p1, moments = lot.adam_w_in_place([[p.clone() for p in grp] for grp in params], grads1, 3e-3, (0.9, 0.95), 1e-8,
                                      moments, 0, weight_decay=0.1, weight_decay_mask=mask_wd)
    p1c = [[p.clone() for p in grp] for grp in p1]
    p2, moments = lot.adam_w_in_place(p1, grads2, 3e-3, (0.9, 0.95), 1e-8, moments, 1, weight_decay=0.1,
                                      weight_decay_mask=mask_wd)
    for i, t in enumerate(flat_params(p0)): d[f"adam_p0_{i}"] = t
    for i, t in enumerate(flat_params(grads1)): d[f"adam_g1_{i}"] = t
    for i, t in enumerate(flat_params(grads2)): d[f"adam_g2_{i}"] = t
    for i, t in enumerate(flat_params(p1c)): d[f"adam_p1_{i}"] = t
    for i, t in enumerate(flat_params(p2)): d[f"adam_p2_{i}"] = t
    for i, t in enumerate(flat_params(moments[0])): d[f"adam_m2_{i}"] = t
    for i, t in enumerate(flat_params(moments[1])): d[f"adam_v2_{i}"] = t
    d["adam_gnorm1"] = torch.tensor(lot.grads_l2norm(grads1))
    return {k: npy(v) for k, v in d.items()}


def make_ops_eval_dropout():
    mtf, mt, lot = load_reference(0.1)
    g = torch.Generator().manual_seed(77)
    x = torch.randn(3, 10, generator=g)
    return {"drop_x": npy(x), "drop_eval_y": npy(mt.t_dropout_fwd(x, train=False)), "drop_rate": np.float32(0.1)}


def run_model(mtf, lot, V, D, L, H, F, S, B, seed, id_low, pad_at=()):
    torch.manual_seed(seed)
    params = mtf.init_transformer_gpt2(V, D, L, H, F, S)
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(id_low, V, (B, S + 1), generator=g, dtype=torch.int32)
    for b, s in pad_at:
        y[b, s] = 0
    mask = causal_mask(B, S)
    idx = torch.arange(S).unsqueeze(0).expand(B, S).contiguous()
    grads, (loss, acc, frac) = lot.uncompiled_grad_loss(params, y, mask, idx)
    return params, y, grads, loss, acc, frac


def main():
    mtf, mt, lot = load_reference(0.0)
    ops = make_ops(mtf, mt, lot)

    # 2-layer toy model, ids may be 0 (padding) so the masking rule is exercised
    params, y, grads, loss, acc, frac = run_model(mtf, lot, 64, 32, 2, 2, 64, 16, 2, seed=5, id_low=0,
                                                  pad_at=((0, 3), (1, 9), (1, 16)))
    tiny = {"y": npy(y), "loss": npy(loss), "acc": npy(acc), "frac": npy(frac),
            "dims": np.array([64, 32, 2, 2, 64, 16, 2])}
    for i, (p, g) in enumerate(zip(flat_params(params), flat_params(grads))):
        tiny[f"p{i}"], tiny[f"g{i}"] = npy(p), npy(g)
    # the reference's hand-written backward (plain torch generation) must agree with torch.func.grad
    g3, (l3, _, _) = lot.t_loss_bkwd3(params, y, causal_mask(2, 16), None, True, [1] * 7)
    worst = max(float((a - b).abs().max()) for a, b in zip(flat_params(grads), flat_params(g3)))
    assert worst < 1e-6, worst

    # benchmark configuration 1
    params, y, grads, loss, acc, frac = run_model(mtf, lot, 1024, 128, 2, 4, 512, 128, 4, seed=0, id_low=0)
    cfg1 = {"y": npy(y), "loss": npy(loss), "acc": npy(acc), "frac": npy(frac),
            "dims": np.array([1024, 128, 2, 4, 512, 128, 4]), "stride": np.array(SAMPLE_STRIDE)}
    for i, (p, g) in enumerate(zip(flat_params(params), flat_params(grads))):
        gd = g.double().reshape(-1)
        cfg1[f"g{i}_l2"] = np.float64(gd.norm())
        cfg1[f"g{i}_sum"] = np.float64(gd.sum())
        cfg1[f"g{i}_sample"] = npy(g.reshape(-1)[::SAMPLE_STRIDE])
        cfg1[f"p{i}_l2"] = np.float64(p.double().norm())  # lets the test confirm it rebuilt identical weights

    ops.update(make_ops_eval_dropout())
    np.savez_compressed(OUT / "ops_small.npz", **ops)
    np.savez_compressed(OUT / "tiny_model.npz", **tiny)
    np.savez_compressed(OUT / "cfg1_summary.npz", **cfg1)
    for f in ("ops_small.npz", "tiny_model.npz", "cfg1_summary.npz"):
        print(f, (OUT / f).stat().st_size, "bytes")
    print("tiny loss", float(tiny["loss"]), "cfg1 loss", float(cfg1["loss"]))


if __name__ == "__main__":
    main()
