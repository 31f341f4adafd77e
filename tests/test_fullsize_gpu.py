"""Full BASELINE sizes (T = 8 x 1024 tokens, d_model 768, FFN 3072, 12 heads x 64, vocab 50257), where running the CPU
oracle on everything would take too long: size-independent properties plus oracle checks on sampled rows / heads."""
import math

import pytest
import torch

from conftest import pkg, rel_err
from oracle import gpt2_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu

T, D, F, V, H, S, B = 8192, 768, 3072, 50257, 12, 1024, 8


def bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (scale * torch.randn(*shape, device="cuda", generator=g)).bfloat16()


def test_attention_config2_sampled_heads():
    """BASELINE configuration 2: B=8, H=12, S=1024, d_head=64, N(0,1) inputs; O, logsumexp, dQ, dK, dV of sampled
    (batch, head) pairs against the fp32 oracle, and bit-reproducibility of the whole result."""
    ops = pkg("operators")
    ops.DROPOUT_RATE = 0.0
    qkv, d_o = bf(B, H, 3, S, 64, seed=1), bf(B, H, S, 64, seed=2)
    out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv, None, True, 1)
    dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o, acts, qkv, None, True, 1)
    out2, acts2 = ops.t_scaled_dot_prod_attn_fwd3_t(qkv, None, True, 1)
    dq2, dk2, dv2 = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o, acts2, qkv, None, True, 1)
    assert torch.equal(out, out2) and torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert ops.last_kernel_fault() == 0
    for b, h in ((0, 0), (3, 7), (7, 11)):
        q, k, v = (qkv[b, h, c].float().cpu() for c in range(3))
        g = d_o[b, h].float().cpu()
        o_ref, _ = orc.causal_attention(q, k, v)
        m, l = orc.causal_attention_stats(q, k)
        assert rel_err(out[b, h], o_ref) < 2e-2
        assert rel_err(acts[0][b, h] + torch.log(acts[1][b, h]), m + torch.log(l)) < 1e-3
        rq, rk, rv = orc.causal_attention_bwd(g, q, k, v)
        assert rel_err(dq[b, h], rq) < 2e-2 and rel_err(dk[b, h], rk) < 2e-2 and rel_err(dv[b, h], rv) < 2e-2
    # causality: perturbing the last key/value row changes only the last query row
    qkv2 = qkv.clone()
    qkv2[:, :, 1:, S - 1] += 1.0
    out3, _ = ops.t_scaled_dot_prod_attn_fwd3_t(qkv2, None, True, 1)
    assert torch.equal(out3[:, :, : S - 1], out[:, :, : S - 1])
    ops.DROPOUT_RATE = 0.1


@pytest.mark.parametrize("name,N,K,a_k,b_k", [("qkv", 2304, 768, True, True), ("ffn2", 768, 3072, True, True),
                                              ("dgrad", 768, 2304, True, False), ("wgrad", 3072, 768, False, False)])
def test_gemm_config3_shapes_sampled_rows(name, N, K, a_k, b_k):
    """The block's GEMM shapes at T = 8192: sampled output rows against float64, and linearity in A."""
    ops = pkg("operators")
    M = T if name != "wgrad" else 3072
    if name == "wgrad":  # dW[3072, 768] = dY^T X with the 8192 tokens as the reduction dimension
        M, N, K = 3072, 768, T
    A, Bm = bf(M, K, seed=3), bf(N, K, seed=4, scale=0.05)
    a_dev = A if a_k else A.t().contiguous()
    b_dev = Bm if b_k else Bm.t().contiguous()
    kw = dict(a_kmajor=a_k, b_kmajor=b_k, M=M, N=N, K=K, out_dtype=torch.float32)
    c = ops.gemm(a_dev, b_dev, **kw)
    rows = torch.tensor([0, 1, 127, 128, M // 2 + 5, M - 1])
    ref = A[rows].double().cpu() @ Bm.double().cpu().t()
    assert rel_err(c[rows], ref) < 1e-3
    c2 = ops.gemm((2 * a_dev.float()).bfloat16(), b_dev, **kw)  # exact doubling in bf16
    assert torch.equal(c2, 2 * c)
    assert ops.last_kernel_fault() == 0


def test_lm_head_and_cross_entropy_full_vocab():
    """[8192, 768] x [50257, 768]^T + bias, then CE forward+backward in place over the padded logits buffer."""
    ops = pkg("operators")
    ld = (V + 127) // 128 * 128
    x, w = bf(T, D, seed=5), bf(V, D, seed=6, scale=0.02)
    bias = 0.01 * torch.randn(V, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
    labels = torch.randint(0, V, (T,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(8),
                           dtype=torch.int32)
    labels[::97] = 0  # some padding rows
    logits = torch.full((T, ld), 3.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm(x, w, bias=bias, out=logits, N=V, ldc=ld)
    assert float((logits[:, V:] - 3.0).abs().max()) == 0.0, "padding columns must stay untouched"
    rows = torch.tensor([0, 5, 97, 4096, T - 1])
    ref = x[rows].double().cpu() @ w.double().cpu().t() + bias.double().cpu()
    assert rel_err(logits[rows, :V], ref) < 2e-2
    kept = logits.clone()
    stats, n_valid, dlog = ops.cross_entropy(labels, logits, cols=V, want_grad=True, in_place=True)
    n = int((labels != 0).sum())
    assert int(n_valid) == n
    # every non-padding row of (softmax - onehot) / n sums to zero; padding rows are exactly zero
    sums = dlog[:, :V].float().sum(dim=1)
    assert float(sums.abs().max()) < 2e-3 / n * V ** 0.5 + 1e-5
    assert float(dlog[labels == 0][:, :V].abs().max()) == 0.0
    lab = labels[rows].cpu()
    _, _, g_ref = orc.cross_entropy_fwd_bwd(lab, kept[rows, :V].float().cpu())
    g_ref = g_ref * (int((lab != 0).sum()) / n)  # the oracle normalised by the sample's own count
    assert rel_err(dlog[rows, :V], g_ref) < 2e-2
    lse = torch.logsumexp(kept[:, :V].float(), dim=1)
    picked = kept[:, :V].float().gather(1, labels.long().unsqueeze(1)).squeeze(1)
    loss_ref = ((lse - picked) * (labels != 0)).sum() / n
    assert rel_err(stats[0], loss_ref) < 1e-3


def test_train_step_full_size_is_reproducible_and_learns():
    """GPT-2 small, micro-batch 8 x 1024, dropout 0.1: two trainers with the same seeds stay bit-identical, the loss
    falls, no kernel reports a fault."""
    ptj = pkg()
    cfg = ptj.PRESETS["gpt2-small"]
    g = torch.Generator().manual_seed(0)
    y = torch.randint(1, cfg.vocab, (8, cfg.seq + 1), generator=g, dtype=torch.int32)
    losses = []
    for _ in range(2):
        t = ptj.Trainer(cfg, ptj.TrainConfig.benchmark_recipe(seed=3), device="cuda")
        run = [float(t.step(y)[0]) for _ in range(4)]
        losses.append(run)
        final = t.p.clone()
        if len(losses) == 2:
            assert torch.equal(final, first_final)
        first_final = final
        del t
    assert losses[0] == losses[1]
    # at initialisation the tied, sqrt(D)-scaled embedding makes the model predict its INPUT token (self-logit about
    # D * 0.02^2 / 0.02 = 15), so the loss on random next tokens sits above ln(V) = 10.8
    assert math.log(cfg.vocab) < losses[0][0] < 16.0
    assert losses[0][-1] < losses[0][0] - 0.5              # the same batch is being memorised
    assert ptj.operators.last_kernel_fault() == 0


def test_full_size_model_loss_against_cpu_oracle():
    """All 12 layers at d_model 768 / vocab 50257 on one 1024-token sequence, dropout off: the bf16 GPU loss against
    the fp32 oracle forward on the same bf16-rounded weights."""
    ptj = pkg()
    cfg = ptj.gpt2.GPT2Config(vocab=50257, dim=768, layers=12, heads=12, ffn=3072, seq=1024, dropout=0.0)
    prm = orc.init_params(cfg.vocab, cfg.dim, cfg.layers, cfg.heads, cfg.ffn, cfg.seq, seed=1)
    prm_r = [[t.bfloat16().float() if t.dim() > 1 else t for t in grp] for grp in prm]
    y = torch.randint(1, cfg.vocab, (1, cfg.seq + 1), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    t = ptj.Trainer(cfg, ptj.TrainConfig.benchmark_recipe(seed=0), params=prm, device="cuda")
    stats = t.step(y)
    with torch.no_grad():
        logits = orc.forward_gpt2(prm_r, y[:, :-1])
        ref_loss, _ = orc.avg_cross_entropy_loss(y[:, 1:], logits)
        ref_acc = orc.accuracy(y[:, 1:], logits)
    assert rel_err(stats[0], ref_loss) < 2e-2
    assert abs(float(stats[1]) - float(ref_acc)) < 5e-3
    assert ptj.operators.last_kernel_fault() == 0
