"""Operator parity on the GPU: every launcher of the reference's Triton surface, called through the C ABI, against
the CPU oracle (and the reference's own outputs in tests/golden). Tolerances: float32 path 1e-4 relative, bf16 path
2e-2 relative (fp32 accumulate), as stated for this hot path."""
import math

import numpy as np
import pytest
import torch

from conftest import pkg, rel_err, tt
from oracle import gpt2_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def ops():
    o = pkg("operators")
    assert pkg("_lib").lib().ptj_device_check() == 0, "these tests need an sm_100 device"
    return o


def gpu(t, dtype=None):
    return t.to("cuda", dtype) if dtype is not None else t.to("cuda")


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return scale * torch.randn(*shape, generator=g)


def check(a, b, tol):
    assert tuple(a.shape) == tuple(b.shape), (a.shape, b.shape)
    e = rel_err(a.float(), b.float())
    assert e < tol, f"relative error {e:.3e} >= {tol}"


# ---- golden fixtures straight from the reference ---------------------------------------------------------------------
def test_golden_layernorm_gelu_softmax(ops, ops_golden):
    g = ops_golden
    x, gamma, beta, dy = (gpu(tt(g[k])) for k in ("ln_x", "ln_gamma", "ln_beta", "ln_dy"))
    check(ops.t_layernorm_fwd_t((gamma, beta), x), tt(g["ln_y"]), F32_TOL)
    check(ops.t_layernorm_bkwd2_x_t(dy, (gamma, beta), x), tt(g["ln_dx"]), F32_TOL)
    dg, db = ops.t_layernorm_bkwd2_p_t(dy, (gamma, beta), x)
    check(dg, tt(g["ln_dgamma"]), F32_TOL)
    check(db, tt(g["ln_dbeta"]), F32_TOL)
    check(ops.t_gelu_fwd_t(gpu(tt(g["gelu_x"]))), tt(g["gelu_y"]), F32_TOL)
    check(ops.t_gelu_bkwd2_t(gpu(tt(g["gelu_dy"])), gpu(tt(g["gelu_x"]))), tt(g["gelu_dx"]), F32_TOL)
    check(ops.t_log_softmax_fwd_t(gpu(tt(g["lsm_x"]))), tt(g["lsm_y"]), F32_TOL)
    check(ops.t_log_softmax_bkwd2_t(gpu(tt(g["lsm_dy"])), gpu(tt(g["lsm_x"]))), tt(g["lsm_dx"]), F32_TOL)


def test_golden_cross_entropy(ops, ops_golden):
    g = ops_golden
    labels, logits = gpu(tt(g["ce_labels"])), gpu(tt(g["ce_logits"]))
    loss, n, dl = ops.t_avg_cross_entropy_loss_bkwd3_t(labels, logits)
    check(loss.reshape(()), tt(g["ce_loss"]).reshape(()), F32_TOL)
    assert int(n) == int(g["ce_nvalid"])
    check(dl, tt(g["ce_dlogits"]), F32_TOL)
    assert float(dl[0, 1].abs().max()) == 0.0 and float(dl[1, 4].abs().max()) == 0.0
    loss2, n2 = ops.t_avg_cross_entropy_loss(labels, logits)
    check(loss2.reshape(()), tt(g["ce_loss_fwd"]).reshape(()), F32_TOL)
    check(ops.accuracy_from_logits(labels, logits).reshape(()), tt(g["ce_acc"]).reshape(()), 1e-6)


def test_golden_attention(ops, ops_golden):
    g = ops_golden
    ops.DROPOUT_RATE = 0.0
    try:
        qkv, d_o = gpu(tt(g["attn_qkv"])), gpu(tt(g["attn_do"]))
        out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv, None, True, 1)
        check(out, tt(g["attn_out"]), F32_TOL)
        dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o, acts, qkv, None, True, 1)
        check(dq, tt(g["attn_dq"]), F32_TOL)
        check(dk, tt(g["attn_dk"]), F32_TOL)
        check(dv, tt(g["attn_dv"]), F32_TOL)
        q, k, _ = tt(g["attn_qkv"]).unbind(dim=2)
        m, l = orc.causal_attention_stats(q, k)
        check(acts[0] + torch.log(acts[1]), m + torch.log(l), F32_TOL)  # logsumexp of the scaled scores
    finally:
        ops.DROPOUT_RATE = 0.1


def test_golden_ffn_dropout_adamw(ops, ops_golden):
    g = ops_golden
    prm = tuple(gpu(tt(g[k])) for k in ("ffn_w1", "ffn_b1", "ffn_w2", "ffn_b2"))
    check(ops.t_tlayer_ffn_fwd_t(prm, gpu(tt(g["ffn_x"]))), tt(g["ffn_y"]), F32_TOL)
    ops.DROPOUT_RATE = float(g["drop_rate"])
    check(ops.t_dropout_fwd_t(gpu(tt(g["drop_x"])), train=False), tt(g["drop_eval_y"]), 1e-6)
    opt = pkg("optimizer")
    tree = lambda pre: [[gpu(tt(g[f"{pre}_0"])), gpu(tt(g[f"{pre}_1"]))], [gpu(tt(g[f"{pre}_2"]))]]
    p, g1, g2 = tree("adam_p0"), tree("adam_g1"), tree("adam_g2")
    _, mom = opt.init_adam_w(p)
    mask = opt.weight_decay_mask(p)
    assert [list(m) for m in mask] == [[True, False], [True]]
    p, mom = opt.adam_w_in_place(p, g1, 3e-3, (0.9, 0.95), 1e-8, mom, 0, weight_decay=0.1, weight_decay_mask=mask)
    for i, t in enumerate(x for grp in p for x in grp):
        check(t, tt(g[f"adam_p1_{i}"]), 1e-6)
    p, mom = opt.adam_w_in_place(p, g2, 3e-3, (0.9, 0.95), 1e-8, mom, 1, weight_decay=0.1, weight_decay_mask=mask)
    for i, t in enumerate(x for grp in p for x in grp):
        check(t, tt(g[f"adam_p2_{i}"]), 1e-6)
    for i, t in enumerate(x for grp in mom[0] for x in grp):
        check(t, tt(g[f"adam_m2_{i}"]), 1e-6)
    for i, t in enumerate(x for grp in mom[1] for x in grp):
        check(t, tt(g[f"adam_v2_{i}"]), 1e-6)
    assert abs(opt.grads_l2norm(g1) - float(g["adam_gnorm1"])) < 1e-4


# ---- oracle comparisons over shapes and dtypes ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("rows,dim", [(1, 8), (7, 24), (64, 128), (300, 768), (33, 1024), (5, 1000), (3, 4100)])
def test_layernorm_shapes(ops, dtype, tol, rows, dim):
    x = rnd(rows, dim, seed=1).to(dtype)
    dy = rnd(rows, dim, seed=2).to(dtype)
    res = rnd(rows, dim, seed=5).to(dtype)
    gamma, beta = 1 + 0.2 * rnd(dim, seed=3), 0.2 * rnd(dim, seed=4)
    xf, dyf = x.float(), dy.float()
    check(ops.t_layernorm_fwd_t((gpu(gamma), gpu(beta)), gpu(x)), orc.layernorm(gamma, beta, xf), tol)
    dx, dg, db = ops.layernorm_bwd(gpu(dy), (gpu(gamma), None), gpu(x), dx_add=gpu(res))
    odx, odg, odb = orc.layernorm_bwd(dyf, gamma, xf)
    check(dx, odx + res.float(), tol)
    check(dg, odg, tol)
    check(db, odb, tol)
    # reproducible: no atomics anywhere
    dx2, dg2, db2 = ops.layernorm_bwd(gpu(dy), (gpu(gamma), None), gpu(x), dx_add=gpu(res))
    assert torch.equal(dg, dg2) and torch.equal(db, db2) and torch.equal(dx, dx2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("n", [1, 7, 1024, 100003])
def test_gelu_shapes(ops, dtype, tol, n):
    x, dy = rnd(n, seed=1, scale=2.0).to(dtype), rnd(n, seed=2).to(dtype)
    check(ops.t_gelu_fwd_t(gpu(x)), orc.gelu(x.float()), tol)
    check(ops.t_gelu_bkwd2_t(gpu(dy), gpu(x)), orc.gelu_bwd(dy.float(), x.float()), tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("rows,cols", [(3, 5), (16, 1024), (9, 50257), (4, 50304), (2, 70001)])
def test_log_softmax_shapes(ops, dtype, tol, rows, cols):
    x, dy = rnd(rows, cols, seed=1, scale=3.0).to(dtype), rnd(rows, cols, seed=2).to(dtype)
    check(ops.t_log_softmax_fwd_t(gpu(x)), orc.log_softmax(x.float()), tol)
    check(ops.t_log_softmax_bkwd2_t(gpu(dy), gpu(x)), orc.log_softmax_bwd(dy.float(), x.float()), tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
@pytest.mark.parametrize("rows,cols", [(6, 11), (64, 1024), (40, 50257)])
def test_cross_entropy_shapes(ops, dtype, tol, rows, cols):
    g = torch.Generator().manual_seed(3)
    logits = rnd(rows, cols, seed=1, scale=2.0).to(dtype)
    labels = torch.randint(0, cols, (rows,), generator=g, dtype=torch.int32)
    labels[::5] = 0
    loss, n, dl = ops.t_avg_cross_entropy_loss_bkwd3_t(gpu(labels), gpu(logits))
    ol, on, odl = orc.cross_entropy_fwd_bwd(labels, logits.float())
    check(loss.reshape(()), ol.reshape(()), tol)
    assert int(n) == int(on)
    check(dl, odl, tol)
    assert float(dl[0].abs().max()) == 0.0
    acc = ops.accuracy_from_logits(gpu(labels), gpu(logits))
    check(acc.reshape(()), orc.accuracy(labels, logits.float()).reshape(()), 1e-6)
    # in-place variant with a padded leading dimension, as the training step uses it
    ld = (cols + 127) // 128 * 128
    buf = torch.zeros(rows, ld, dtype=dtype)
    buf[:, :cols] = logits
    buf = gpu(buf)
    stats, nv, d2 = ops.cross_entropy(gpu(labels), buf, cols=cols, want_grad=True, in_place=True)
    assert d2.data_ptr() == buf.data_ptr()
    check(d2[:, :cols], odl, tol)
    check(stats[0].reshape(()), ol.reshape(()), tol)


def test_cross_entropy_label_outside_vocabulary_is_not_counted(ops):
    """An id beyond the vocabulary (or negative) contributes nothing and must not be counted either: the divisor is
    the number of rows that were actually summed."""
    rows, cols = 12, 40
    logits = rnd(rows, cols, seed=1, scale=2.0)
    labels = torch.randint(1, cols, (rows,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    labels[3], labels[7], labels[9] = cols, -5, 0
    loss, n, dl = ops.t_avg_cross_entropy_loss_bkwd3_t(gpu(labels), gpu(logits))
    clean = labels.clone()
    clean[3] = clean[7] = 0  # the oracle's only notion of "no contribution" is the padding id
    ol, on, odl = orc.cross_entropy_fwd_bwd(clean, logits)
    assert int(n) == int(on) == rows - 3
    check(loss.reshape(()), ol.reshape(()), F32_TOL)
    check(dl, odl, F32_TOL)


def test_cross_entropy_bf16_ties_tail_and_label_positions(ops):
    """The bf16 kernel for 16-byte aligned rows: a vocabulary that is not a multiple of the vector width (scalar tail),
    labels in the first vector, in the tail and in between, and rows whose maximum occurs twice (the first index
    wins, as in torch.argmax), against the oracle on the same bf16 values."""
    rows, cols, ld = 24, 1003, 1008
    x = rnd(rows, cols, seed=4, scale=2.0).bfloat16()
    labels = torch.randint(1, cols, (rows,), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    labels[0], labels[1], labels[2], labels[3] = 1, 7, cols - 1, cols - 3      # first vector / tail
    x[4, 100] = x[4, 900] = 9.0; labels[4] = 100                               # tie, label is the first maximum
    x[5, 100] = x[5, 900] = 9.0; labels[5] = 900                               # tie, label is the second one
    x[6, 1001] = 9.0; labels[6] = 1001                                         # the maximum sits in the scalar tail
    x[7, 3] = x[7, 1002] = 9.0; labels[7] = 1002
    labels[8] = 0
    buf = torch.zeros(rows, ld, dtype=torch.bfloat16)
    buf[:, :cols] = x
    buf = gpu(buf)
    stats, nv, d = ops.cross_entropy(gpu(labels), buf, cols=cols, want_grad=True, in_place=False)
    ol, on, odl = orc.cross_entropy_fwd_bwd(labels, x.float())
    check(stats[0].reshape(()), ol.reshape(()), 1e-4)
    check(d[:, :cols], odl, BF16_TOL)
    assert float(d[8, :cols].abs().max()) == 0.0 and float(d[:, cols:].abs().max()) == 0.0
    want_hits = (torch.argmax(x.float(), dim=1).to(torch.int32) == labels) & (labels != 0)
    assert abs(float(stats[1]) - float(want_hits.sum()) / int(on)) < 1e-6
    assert bool(want_hits[4]) and not bool(want_hits[5]) and bool(want_hits[6]) and not bool(want_hits[7])
    # forward only (no gradient buffer): same statistics
    stats2, _, none = ops.cross_entropy(gpu(labels), buf, cols=cols, want_grad=False)
    assert none is None and torch.equal(stats, stats2)


def test_cross_entropy_all_padding(ops):
    logits = gpu(rnd(4, 16, seed=1))
    labels = gpu(torch.zeros(4, dtype=torch.int32))
    loss, n, dl = ops.t_avg_cross_entropy_loss_bkwd3_t(labels, logits)
    assert int(n) == 0 and math.isnan(float(loss)) and float(dl.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dropout_mask_matches_host_philox(ops, dtype):
    n, p, seed = 10007, 0.1, 0x1234_5678_9ABC
    x = rnd(n, seed=1).to(dtype)
    ops.DROPOUT_RATE = p
    y = ops.t_dropout_fwd_t(gpu(x), True, seed).cpu().float()
    mask = torch.from_numpy(philox.keep_mask(seed, 0, n, p))
    assert torch.equal(y, x.float() * mask)  # exact: multiply by 0/1, never rescaled
    dy = rnd(n, seed=2).to(dtype)
    back = ops.t_dropout_bkwd2_t(gpu(dy), gpu(x), True, seed).cpu().float()
    assert torch.equal(back, dy.float() * mask)  # backward regenerates the very same mask
    ev = ops.t_dropout_fwd_t(gpu(x), False, None).cpu().float()
    check(ev, x.float() * (1 - p), 1e-2 if dtype == torch.bfloat16 else 1e-6)
    res = rnd(n, seed=3).to(dtype)
    fused = ops.dropout(gpu(x), True, seed, residual=gpu(res)).cpu().float()
    check(fused, res.float() + x.float() * mask, 1e-2 if dtype == torch.bfloat16 else 1e-6)


def test_dropout_statistics(ops):
    """Keep rate, independence between seeds and between neighbours (mask bits are not comparable to the reference's
    generators, so the distribution is what is checked)."""
    n = 1 << 22
    ops.DROPOUT_RATE = 0.1
    ones = torch.ones(n, device="cuda")
    a = ops.t_dropout_fwd_t(ones, True, 11)
    b = ops.t_dropout_fwd_t(ones, True, 12)
    assert abs(float(a.mean()) - 0.9) < 1e-3
    assert set(a.unique().tolist()) == {0.0, 1.0}
    both = float((a * b).mean())
    assert abs(both - 0.81) < 2e-3
    assert abs(float((a[:-1] * a[1:]).mean()) - 0.81) < 2e-3
    ops.DROPOUT_RATE = 0.0
    assert torch.equal(ops.t_dropout_fwd_t(ones, True, 11), ones)
    ops.DROPOUT_RATE = 0.1


@pytest.mark.parametrize("M,N,K", [(5, 7, 3), (64, 64, 64), (130, 70, 33), (256, 96, 200)])
def test_matmul_fp32_exact_path(ops, M, N, K):
    a, b = rnd(M, K, seed=1), rnd(K, N, seed=2)
    check(ops.t_matmul_t(gpu(a), gpu(b)), a.double() @ b.double(), F32_TOL)
    w, bias = rnd(N, K, seed=3), rnd(N, seed=4)
    check(ops.t_linear_fwd_t((gpu(w), gpu(bias)), gpu(a)), a.double() @ w.double().t() + bias.double(), F32_TOL)
    check(ops.t_linear_fwd_t((gpu(w), gpu(bias)), gpu(a), activation="gelu"),
          orc.gelu(a.double() @ w.double().t() + bias.double()), F32_TOL)


@pytest.mark.parametrize("B,H,S,D", [(1, 1, 1, 4), (2, 3, 17, 8), (2, 4, 128, 32), (1, 2, 200, 64), (1, 1, 96, 128)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_attention_exact_path(ops, B, H, S, D, dtype, tol, monkeypatch):
    """CUDA-core attention kernels (float32 always; bf16 at shapes the tensor-core kernels do not take)."""
    ops.DROPOUT_RATE = 0.0
    qkv = rnd(B, H, 3, S, D, seed=1).to(dtype)
    d_o = rnd(B, H, S, D, seed=2).to(dtype)
    q, k, v = qkv.float().unbind(dim=2)
    out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(gpu(qkv), None, True, 5)
    o_ref, _ = orc.causal_attention(q, k, v)
    check(out, o_ref, tol)
    m, l = orc.causal_attention_stats(q, k)
    check(acts[0] + torch.log(acts[1]), m + torch.log(l), tol)
    dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(gpu(d_o), acts, gpu(qkv), None, True, 5)
    # the backward differentiates the forward it ran: feed the oracle the output as rounded by the kernel
    rq, rk, rv = orc.causal_attention_bwd(d_o.float(), q, k, v)
    check(dq, rq, tol)
    check(dk, rk, tol)
    check(dv, rv, tol)
    ops.DROPOUT_RATE = 0.1


def test_attention_dropout_with_host_mask(ops):
    """Dropout on the probabilities (not rescaled), mask regenerated identically in backward."""
    B, H, S, D, p, seed = 2, 2, 40, 16, 0.25, 991
    ops.DROPOUT_RATE = p
    qkv, d_o = rnd(B, H, 3, S, D, seed=1), rnd(B, H, S, D, seed=2)
    q, k, v = qkv.unbind(dim=2)
    mask = torch.from_numpy(philox.keep_mask(seed, 0, B * H * S * S, p)).view(B, H, S, S)
    out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(gpu(qkv), None, True, seed)
    o_ref, _ = orc.causal_attention(q, k, v, p, True, mask)
    check(out, o_ref, F32_TOL)
    dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(gpu(d_o), acts, gpu(qkv), None, True, seed)
    rq, rk, rv = orc.causal_attention_bwd(d_o, q, k, v, p, True, mask)
    check(dq, rq, F32_TOL); check(dk, rk, F32_TOL); check(dv, rv, F32_TOL)
    out_e, _ = ops.t_scaled_dot_prod_attn_fwd3_t(gpu(qkv), None, False, None)
    check(out_e, orc.causal_attention(q, k, v, p, False, None)[0], F32_TOL)
    ops.DROPOUT_RATE = 0.1


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_embedding_forward_backward(ops, dtype, tol):
    B, S, D, V, p, seed = 3, 12, 16, 50, 0.2, 77
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, V, (B, S), generator=g, dtype=torch.int32)
    ids[0, :4] = 7  # repeated ids: the scatter must sum them
    w_emb, w_pos = rnd(V, D, seed=1).to(dtype), rnd(S, D, seed=2).to(dtype)
    mask = torch.from_numpy(philox.keep_mask(seed, 0, B * S * D, p)).view(B, S, D)
    y = ops.embed_fwd(gpu(ids), gpu(w_emb), gpu(w_pos), True, seed, p=p)
    ref = (w_emb.float()[ids.long()] * math.sqrt(D) + w_pos.float()) * mask
    check(y, ref, tol)
    dy = rnd(B, S, D, seed=3).to(dtype)
    d_emb = torch.full((V, D), 0.5, device="cuda")
    d_pos = torch.empty((S, D), device="cuda")
    ops.embed_bwd(gpu(dy), gpu(ids), d_emb, d_pos, accumulate=True, train=True, seed=seed, p=p)
    gm = dy.float() * mask
    ref_emb = torch.full((V, D), 0.5).index_add_(0, ids.reshape(-1).long(), gm.reshape(-1, D) * math.sqrt(D))
    check(d_emb, ref_emb, tol)
    check(d_pos, gm.sum(dim=0), tol)
    d_emb2 = torch.full((V, D), 9.0, device="cuda")
    ops.embed_bwd(gpu(dy), gpu(ids), d_emb2, d_pos, accumulate=False, train=True, seed=seed, p=p)
    check(d_emb2, ref_emb - 0.5, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)])
def test_embedding_backward_long_runs(ops, dtype, tol):
    """Tokens that occur more than 32 times in a batch are summed by a cluster of thread blocks (slices of the run
    meet through distributed shared memory): run lengths on both sides of that limit, of the 64-position chunk a block
    scans for run heads and of the 256-position batch,
    one run that starts at sorted position 0 and one that ends at the last position, dropout on, against a float64
    scatter; two calls agree bit for bit."""
    B, S, D, V, p, seed = 4, 1024, 64, 300, 0.1, 5
    g = torch.Generator().manual_seed(1)
    counts = {1: 1500, 5: 32, 6: 33, 9: 64, 11: 65, 17: 257, 21: 600, 299: 200}
    flat = [t for t, n in counts.items() for _ in range(n)]
    rest = B * S - len(flat)
    flat += torch.randint(30, 290, (rest,), generator=g).tolist()
    ids = torch.tensor(flat, dtype=torch.int32)[torch.randperm(B * S, generator=g)].view(B, S)
    dy = rnd(B, S, D, seed=3).to(dtype)
    mask = torch.from_numpy(philox.keep_mask(seed, 0, B * S * D, p)).view(B, S, D)
    gm = (dy.double() * mask).reshape(-1, D) * math.sqrt(D)
    ref = torch.zeros(V, D, dtype=torch.float64).index_add_(0, ids.reshape(-1).long(), gm)
    outs = []
    for _ in range(2):
        d_emb = torch.full((V, D), 7.0, device="cuda")
        d_pos = torch.empty((S, D), device="cuda")
        ops.embed_bwd(gpu(dy), gpu(ids), d_emb, d_pos, accumulate=False, train=True, seed=seed, p=p)
        outs.append((d_emb, d_pos))
    check(outs[0][0], ref.float(), tol)
    check(outs[0][1], (dy.double() * mask).sum(dim=0).float(), tol)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # evaluation mode scales instead of masking
    d_emb = torch.zeros((V, D), device="cuda")
    ops.embed_bwd(gpu(dy), gpu(ids), d_emb, torch.empty((S, D), device="cuda"), accumulate=True, train=False, seed=seed, p=p)
    ref_e = torch.zeros(V, D, dtype=torch.float64).index_add_(0, ids.reshape(-1).long(), dy.double().reshape(-1, D) * math.sqrt(D) * (1 - p))
    check(d_emb, ref_e.float(), tol)


@pytest.mark.parametrize("rows,cols", [(1, 1), (100, 7), (513, 300), (2048, 50257)])
def test_colsum_and_sumsq(ops, rows, cols):
    x = rnd(rows, cols, seed=1)
    check(ops.colsum(gpu(x)), x.double().sum(dim=0), F32_TOL)
    check(ops.colsum(gpu(x.bfloat16())), x.bfloat16().double().sum(dim=0), F32_TOL)
    opt = pkg("optimizer")
    s = opt.sumsq(gpu(x).view(-1))
    check(s.reshape(()), (x.double() ** 2).sum().reshape(()), F32_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [200, 512, 768, 1016, 1280, 1536, 1792, 2048])
@pytest.mark.parametrize("rows", [5, 1237])
def test_layernorm_backward_bf16_rows_over_several_warps(dim, rows):
    """The bf16 backward spreads a row over ceil(dim / 256) warps (the forward is checked on the same shapes): every warp count, rows that do not divide over
    the blocks and row groups, all outputs against the oracle, and the two reduced forms (parameter gradients only;
    dx without parameter gradients) bit for bit against the full call."""
    ops = pkg("operators")
    x, dy, res = (rnd(rows, dim, seed=s).bfloat16() for s in (1, 2, 5))
    x = (x.float() * 0.5 + 3.0).bfloat16()  # a mean well away from zero
    gamma = 1 + 0.2 * rnd(dim, seed=3)
    beta = 0.3 * rnd(dim, seed=4)
    check(ops.t_layernorm_fwd_t((gpu(gamma), gpu(beta)), gpu(x)), orc.layernorm(gamma, beta, x.float()), BF16_TOL)
    dx, dg, db = ops.layernorm_bwd(gpu(dy), (gpu(gamma), None), gpu(x), dx_add=gpu(res))
    odx, odg, odb = orc.layernorm_bwd(dy.float(), gamma, x.float())
    check(dx, odx + res.float(), BF16_TOL)
    check(dg, odg, 1e-3)  # float32 sums of exact products of the bf16 inputs
    check(db, odb, 1e-4)
    dg2, db2 = ops.t_layernorm_bkwd2_p_t(gpu(dy), (gpu(gamma), gpu(gamma)), gpu(x))
    assert torch.equal(dg, dg2) and torch.equal(db, db2)
    dx3 = ops.t_layernorm_bkwd2_x_t(gpu(dy), (gpu(gamma), gpu(gamma)), gpu(x))
    check(dx3, odx, BF16_TOL)
    dx4, dg4, db4, dropped = ops.layernorm_bwd(gpu(dy), (gpu(gamma), None), gpu(x), dx_add=gpu(res), dropped=(True, 77, 0.25, 3))
    assert torch.equal(dx4, dx) and torch.equal(dg4, dg) and torch.equal(db4, db)
    assert torch.equal(dropped, ops.dropout(dx, True, 77, stream_id=3, p=0.25))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm_backward_with_fused_dropout_output(dtype):
    """ptj_layernorm_bwd_dropout: dx, dgamma, dbeta equal the plain call bit for bit, and the extra output equals
    ptj_dropout applied to that dx (training mask and evaluation scaling)."""
    ops = pkg("operators")
    g = torch.Generator().manual_seed(3)
    rows, dim = 300, 768
    x = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    dy = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    add = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    gamma = (1 + 0.1 * torch.randn(dim, generator=g)).cuda()
    for train in (True, False):
        dx0, dg0, db0 = ops.layernorm_bwd(dy, (gamma, None), x, dx_add=add)
        dx1, dg1, db1, dxd = ops.layernorm_bwd(dy, (gamma, None), x, dx_add=add, dropped=(train, 41, 0.3, 2))
        assert torch.equal(dx0, dx1) and torch.equal(dg0, dg1) and torch.equal(db0, db1)
        ref = ops.dropout(dx0, train, 41, stream_id=2, p=0.3)
        assert torch.equal(dxd, ref)
        if train:
            kept = float((dxd != 0).float().mean())
            assert abs(kept - 0.7) < 0.01


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dim", [(torch.float32, 768), (torch.bfloat16, 768), (torch.bfloat16, 1024),
                                       (torch.float32, 64), (torch.bfloat16, 2048)])
def test_layernorm_backward_fused_column_sums_of_dropped_output(dtype, dim):
    """The optional third reduction of ptj_layernorm_bwd_dropout: column sums of the dropped output equal a float64
    sum of that output (it is the bias gradient of the linear layer feeding the branch); the other results do not
    change by a bit, and repeated calls give identical sums (fixed summation order)."""
    ops = pkg("operators")
    g = torch.Generator().manual_seed(5)
    rows = 1000
    x = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    dy = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    add = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    gamma = (1 + 0.1 * torch.randn(dim, generator=g)).cuda()
    for train in (True, False):
        dx0, dg0, db0, dxd0 = ops.layernorm_bwd(dy, (gamma, None), x, dx_add=add, dropped=(train, 9, 0.1, 1))
        cs = torch.full((dim,), 123.0, device="cuda")
        dx1, dg1, db1, dxd1 = ops.layernorm_bwd(dy, (gamma, None), x, dx_add=add, dropped=(train, 9, 0.1, 1),
                                                dropped_colsum_out=cs)
        assert torch.equal(dx0, dx1) and torch.equal(dg0, dg1) and torch.equal(db0, db1) and torch.equal(dxd0, dxd1)
        ref = dxd1.double().sum(dim=0)
        assert rel_err(cs, ref) < 1e-5
        cs2 = torch.empty_like(cs)
        ops.layernorm_bwd(dy, (gamma, None), x, dx_add=add, dropped=(train, 9, 0.1, 1), dropped_colsum_out=cs2)
        assert torch.equal(cs, cs2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (77, 64), (1000, 3072), (513, 1000)])
def test_gelu_backward_with_fused_column_sums(dtype, rows, cols):
    """ptj_gelu_bwd_colsum: the gradient equals ptj_gelu_bwd bit for bit (also in place), the column sums equal a float64
    sum of the stored gradient, and two calls give identical sums."""
    ops = pkg("operators")
    g = torch.Generator().manual_seed(rows + cols)
    dy = torch.randn(rows, cols, generator=g).to(dtype).cuda()
    x = (2 * torch.randn(rows, cols, generator=g)).to(dtype).cuda()
    ref = ops.t_gelu_bkwd2_t(dy, x)
    dx, cs = ops.gelu_bwd_colsum(dy, x)
    assert torch.equal(dx, ref)
    assert rel_err(cs, ref.double().sum(dim=0)) < 1e-5
    if dtype == torch.float32:
        assert rel_err(dx, orc.gelu_bwd(dy.double().cpu(), x.double().cpu())) < 1e-5
    dy2 = dy.clone()
    dx2, cs2 = ops.gelu_bwd_colsum(dy2, x, in_place=True)
    assert dx2.data_ptr() == dy2.data_ptr() and torch.equal(dx2, ref) and torch.equal(cs2, cs)
