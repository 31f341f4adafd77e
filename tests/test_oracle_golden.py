"""The CPU oracle against the outputs of the real reference (tests/golden/*.npz, made by make_golden.py)."""
import math

import numpy as np
import torch

from conftest import rel_err, tt
from oracle import gpt2_oracle as orc
from oracle import philox

TOL = 2e-6  # float32 restatement vs float32 reference: only summation-order noise is allowed


def close(a, b, tol=TOL):
    if a.numel() == 1 and b.numel() == 1:
        a, b = a.reshape(()), b.reshape(())
    assert a.shape == b.shape, (a.shape, b.shape)
    assert rel_err(a, b) < tol, rel_err(a, b)


def test_layernorm(ops_golden):
    g = ops_golden
    x, gamma, beta, dy = (tt(g[k]) for k in ("ln_x", "ln_gamma", "ln_beta", "ln_dy"))
    close(orc.layernorm(gamma, beta, x), tt(g["ln_y"]))
    dx, dg, db = orc.layernorm_bwd(dy, gamma, x)
    close(dx, tt(g["ln_dx"]))
    close(dg, tt(g["ln_dgamma"]))
    close(db, tt(g["ln_dbeta"]))


def test_gelu(ops_golden):
    g = ops_golden
    close(orc.gelu(tt(g["gelu_x"])), tt(g["gelu_y"]))
    close(orc.gelu_bwd(tt(g["gelu_dy"]), tt(g["gelu_x"])), tt(g["gelu_dx"]))


def test_log_softmax(ops_golden):
    g = ops_golden
    close(orc.log_softmax(tt(g["lsm_x"])), tt(g["lsm_y"]))
    close(orc.log_softmax_bwd(tt(g["lsm_dy"]), tt(g["lsm_x"])), tt(g["lsm_dx"]))


def test_cross_entropy(ops_golden):
    g = ops_golden
    labels, logits = tt(g["ce_labels"]), tt(g["ce_logits"])
    loss, n, dl = orc.cross_entropy_fwd_bwd(labels, logits)
    close(loss, tt(g["ce_loss"]))
    close(loss, tt(g["ce_loss_fwd"]))
    assert int(n) == int(g["ce_nvalid"]) == 10
    close(dl, tt(g["ce_dlogits"]))
    close(orc.accuracy(labels, logits), tt(g["ce_acc"]))
    # rows whose label is the padding id get exactly zero gradient
    assert float(dl[0, 1].abs().max()) == 0.0 and float(dl[1, 4].abs().max()) == 0.0


def test_attention(ops_golden):
    g = ops_golden
    qkv, d_o = tt(g["attn_qkv"]), tt(g["attn_do"])
    q, k, v = qkv.unbind(dim=2)
    out, probs = orc.causal_attention(q, k, v)
    close(out, tt(g["attn_out"]))
    close(probs, tt(g["attn_probs"]))
    dq, dk, dv = orc.causal_attention_bwd(d_o, q, k, v)
    close(dq, tt(g["attn_dq"]))
    close(dk, tt(g["attn_dk"]))
    close(dv, tt(g["attn_dv"]))
    m, l = orc.causal_attention_stats(q, k)
    lse = torch.logsumexp(torch.where(torch.tril(torch.ones(16, 16, dtype=torch.bool)),
                                      q @ k.transpose(-2, -1) / math.sqrt(8), torch.tensor(-1e9)), dim=-1)
    close(m + torch.log(l), lse)


def test_ffn_and_eval_dropout(ops_golden):
    g = ops_golden
    x = tt(g["ffn_x"])
    y = orc.gelu(x @ tt(g["ffn_w1"]).t() + tt(g["ffn_b1"])) @ tt(g["ffn_w2"]).t() + tt(g["ffn_b2"])
    close(y, tt(g["ffn_y"]))
    close(orc.dropout(tt(g["drop_x"]), float(g["drop_rate"]), False, None), tt(g["drop_eval_y"]))


def test_adamw(ops_golden):
    g = ops_golden
    tree = lambda pre: [[tt(g[f"{pre}_0"]), tt(g[f"{pre}_1"])], [tt(g[f"{pre}_2"])]]
    p0, g1, g2 = tree("adam_p0"), tree("adam_g1"), tree("adam_g2")
    mom = [[[torch.zeros_like(p) for p in grp] for grp in p0] for _ in range(2)]
    mask = [[True, False], [True]]
    p1, mom = orc.adam_w(p0, g1, 3e-3, (0.9, 0.95), 1e-8, mom, 0, 0.1, mask)
    for a, b in zip([t for grp in p1 for t in grp], [t for grp in tree("adam_p1") for t in grp]):
        close(a, b)
    p2, mom = orc.adam_w(p1, g2, 3e-3, (0.9, 0.95), 1e-8, mom, 1, 0.1, mask)
    for a, b in zip([t for grp in p2 for t in grp], [t for grp in tree("adam_p2") for t in grp]):
        close(a, b)
    for a, b in zip([t for grp in mom[0] for t in grp], [t for grp in tree("adam_m2") for t in grp]):
        close(a, b)
    for a, b in zip([t for grp in mom[1] for t in grp], [t for grp in tree("adam_v2") for t in grp]):
        close(a, b)
    assert abs(orc.grads_l2norm(g1) - float(g["adam_gnorm1"])) < 1e-5
    assert orc.decay_mask(p0) == mask


def _tree_from(g, dims):
    V, D, L, H, F, S, B = (int(v) for v in dims)
    n = 3 + 10 * L + 2
    flat = [tt(g[f"p{i}"]) for i in range(n)]
    it = iter(flat)
    tree = [[next(it), next(it)], [next(it)]] + [[next(it) for _ in range(10)] for _ in range(L)] + [[next(it), next(it)]]
    return tree, n


def test_tiny_model_full_gradients(tiny_golden):
    g = tiny_golden
    params, n = _tree_from(g, g["dims"])
    y = tt(g["y"])
    assert (y[:, 1:] == 0).any(), "fixture is meant to contain padding labels"
    grads, (loss, acc, frac) = orc.loss_and_grads(params, y)
    close(loss, tt(g["loss"]))
    close(acc, tt(g["acc"]))
    close(frac, tt(g["frac"]))
    for i, gr in enumerate(t for grp in grads for t in grp):
        close(gr, tt(g[f"g{i}"]), 2e-5)


def test_cfg1_benchmark_configuration(cfg1_golden):
    """BASELINE configuration 1: weights rebuilt from the seed must be the reference's, then loss and gradients match."""
    g = cfg1_golden
    V, D, L, H, F, S, B = (int(v) for v in g["dims"])
    params = orc.init_params(V, D, L, H, F, S, seed=0)
    flat = [t for grp in params for t in grp]
    for i, p in enumerate(flat):
        assert abs(float(p.double().norm()) - float(g[f"p{i}_l2"])) <= 1e-9 * max(1.0, float(g[f"p{i}_l2"]))
    y = tt(g["y"])
    grads, (loss, acc, frac) = orc.loss_and_grads(params, y)
    close(loss, tt(g["loss"]))
    close(acc, tt(g["acc"]))
    stride = int(g["stride"])
    for i, gr in enumerate(t for grp in grads for t in grp):
        ref_l2 = float(g[f"g{i}_l2"])
        assert abs(float(gr.double().norm()) - ref_l2) <= 2e-5 * max(ref_l2, 1e-12)
        close(gr.reshape(-1)[::stride], tt(g[f"g{i}_sample"]), 5e-5)


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 from the Random123 test suite (kat_vectors)."""
    kat = [
        ([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
        ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
        ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
         [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]),
    ]
    for ctr, key, want in kat:
        got = [int(x) for x in philox.philox4x32_10(ctr, key)]
        assert got == want


def test_mask_statistics():
    m = philox.keep_mask(seed=123456789, stream_id=0, n=1 << 20, p=0.1)
    assert abs(float(m.mean()) - 0.9) < 2e-3
    # neighbouring elements and different seeds are uncorrelated
    assert abs(float(np.corrcoef(m[:-1], m[1:])[0, 1])) < 5e-3
    m2 = philox.keep_mask(seed=123456790, stream_id=0, n=1 << 20, p=0.1)
    assert abs(float(np.corrcoef(m, m2)[0, 1])) < 5e-3
    assert philox.keep_mask(1, 0, 1000, 0.0).min() == 1.0


def _tiny_params(g):
    L = int(g["dims"][2])
    it = iter([tt(g[f"p{i}"]) for i in range(3 + 10 * L + 2)])
    return [[next(it), next(it)], [next(it)]] + [[next(it) for _ in range(10)] for _ in range(L)] + [[next(it), next(it)]]


def test_eval_callers(tiny_golden, eval_golden):
    """loss_eval / log_probs / predict restated on the CPU against the reference's own outputs (eval_callers.npz,
    made by make_golden_eval.py): dropout 0.1 in eval mode, padding labels present, greedy decoding over 16 positions."""
    g, e = tiny_golden, eval_golden
    params, y, p = _tiny_params(g), tt(g["y"]), float(e["dropout"])
    close(orc.forward_gpt2(params, y[:, :-1], p, False), tt(e["logits_eval"]))
    loss, acc, frac = orc.loss_eval(params, y, p)
    close(loss, tt(e["loss"]))
    close(acc, tt(e["acc"]))
    close(frac, tt(e["frac"]))
    assert int((y[:, 1:] == 0).sum()) > 0  # the +1-per-padding-label rule is exercised
    close(orc.log_probs(params, y, p), tt(e["log_probs"]))
    params_pred = [[params[0][0], tt(e["b_head_pred"])], [tt(e["w_pos_pred"])]] + params[2:]
    pred = orc.predict(params_pred, y.shape[0], int(g["dims"][5]), int(e["start_tok"]), int(e["end_tok"]), p)
    assert torch.equal(pred, tt(e["predict"]))
    assert len(set(pred[0].tolist())) > 5  # the decoded ids differ from position to position


def test_packed_batch_with_document_and_padding_masks(packed_golden):
    """Rows built by the reference's collator (several documents per row, padding tail): the oracle with the same
    dense mask reproduces the reference's loss, accuracy and every gradient, and its attention operator pair."""
    g = packed_golden
    params, n = _tree_from(g, g["dims"])
    y, mask = tt(g["y"]), tt(g["mask"])
    assert not mask[0, 6, 5] and mask[0, 6, 6] and not mask[0, 12].any(), "document boundary and padding rows expected"
    grads, (loss, acc, frac) = orc.loss_and_grads(params, y, attn_mask=mask)
    close(loss, tt(g["loss"]))
    close(acc, tt(g["acc"]))
    close(frac, tt(g["frac"]))
    for i, gr in enumerate(t for grp in grads for t in grp):
        close(gr, tt(g[f"g{i}"]), 2e-5)
    qkv, d_o = tt(g["attn_qkv"]), tt(g["attn_do"])
    am = mask.unsqueeze(1)
    out, _ = orc.causal_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], attn_mask=am)
    close(out, tt(g["attn_out"]))
    dq, dk, dv = orc.causal_attention_bwd(d_o, qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], attn_mask=am)
    close(dq, tt(g["attn_dq"]), 2e-5)
    close(dk, tt(g["attn_dk"]), 2e-5)
    close(dv, tt(g["attn_dv"]), 2e-5)
