"""Packed and padded batches: the attention mask of the reference's collator (causal x block-diagonal over the
documents packed into a row x padding, tokenized_dataset.py:110-131) reaches the kernels as one int32 per query row
(the first key it attends to) instead of a dense [B, N, N] tensor. Checked against the reference's own outputs on a
batch its collator built (tests/golden/packed_model.npz) and against the oracle run with the dense mask."""
import math

import pytest
import torch

from conftest import pkg, rel_err, tt
from oracle import gpt2_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu


def flat(tree):
    return [t for grp in tree for t in grp]


def collator_mask(doc_lengths, S):
    """What build_masks / create_packs produce for rows that pack documents of these lengths (padding after them)."""
    B = len(doc_lengths)
    mask = torch.zeros(B, S, S, dtype=torch.bool)
    for b, lens in enumerate(doc_lengths):
        pos = 0
        for n in lens:
            n = min(n, S - pos)
            mask[b, pos:pos + n, pos:pos + n] = torch.tril(torch.ones(n, n, dtype=torch.bool))
            pos += n
    return mask


def non_pad_rows(mask):
    return mask.any(dim=2)  # [B, S]


def test_row_kstart_forms_agree_and_bad_masks_are_refused():
    ops = pkg("operators")
    lens = [[6, 5], [4, 7, 9], [10], [16]]
    S = 16
    mask = collator_mask(lens, S)
    ks = ops.row_kstart_from_mask(mask.cuda())
    assert torch.equal(ks, ops.row_kstart_from_lengths(lens, S))
    assert ks[0, 7].item() == 6 and ks[0, 12].item() == 13 and ks[3].abs().sum().item() == 0
    assert ops._kstart_or_none(torch.tril(torch.ones(2, 8, 8, dtype=torch.bool)).cuda()) is None  # plain causal
    bad = mask.clone()
    bad[0, 4, 2] = False  # a hole inside a row's interval
    with pytest.raises(ValueError, match="interval"):
        ops.row_kstart_from_mask(bad.cuda())
    bad = mask.clone()
    bad[0, 2, 5] = True  # a key beyond the row's own position
    with pytest.raises(ValueError, match="interval"):
        ops.row_kstart_from_mask(bad.cuda())


def test_reference_packed_batch_fp32(packed_golden):
    """The reference's own loss, accuracy and gradients on a batch its collator packed, fp32 path."""
    g, ops, gpt2 = packed_golden, pkg("operators"), pkg("gpt2")
    ops.DROPOUT_RATE = 0.0
    try:
        L = int(g["dims"][2])
        it = iter([tt(g[f"p{i}"]) for i in range(3 + 10 * L + 2)])
        params = [[next(it), next(it)], [next(it)]] + [[next(it) for _ in range(10)] for _ in range(L)] + [[next(it), next(it)]]
        gp = [[t.cuda() for t in grp] for grp in params]
        y, mask = tt(g["y"]).cuda(), tt(g["mask"]).cuda()
        grads, (loss, acc, frac) = gpt2.t_loss_bkwd3_t(gp, y, mask, None, True, [1] * (1 + 3 * L))
        assert rel_err(loss, tt(g["loss"])) < 1e-4
        assert rel_err(acc, tt(g["acc"])) < 1e-6 and rel_err(frac, tt(g["frac"])) < 1e-6
        for i, gr in enumerate(flat(grads)):
            assert rel_err(gr, tt(g[f"g{i}"])) < 1e-4, f"gradient {i}"
        # ignoring the mask must give a different answer (documents would attend across their boundaries)
        grads_c, _ = gpt2.t_loss_bkwd3_t(gp, y, None, None, True, [1] * (1 + 3 * L))
        assert rel_err(grads_c[2][2], grads[2][2]) > 1e-2, "the first layer's QKV gradient must feel the mask"
        # the attention operator pair with the dense mask, non-padding rows (the reference attends all keys uniformly
        # on a row without keys; here such rows give zeros)
        qkv, d_o = tt(g["attn_qkv"]).cuda(), tt(g["attn_do"]).cuda()
        keep = non_pad_rows(tt(g["mask"]))[:, None, :, None]
        out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv, mask, True, 1)
        assert rel_err(out.cpu() * keep, tt(g["attn_out"]) * keep) < 1e-4
        assert float((out.cpu() * ~keep).abs().max()) == 0.0
    finally:
        ops.DROPOUT_RATE = 0.1


@pytest.mark.parametrize("dtype,d_head,S,lens", [
    (torch.float32, 16, 40, [[13, 20], [40], [7, 7, 7, 7]]),                 # CUDA-core kernels, ragged everything
    (torch.bfloat16, 64, 256, [[100, 60, 50], [256], [128, 128], [30]]),      # tensor-core kernels, two tiles
    (torch.bfloat16, 64, 512, [[200, 200, 112], [129, 300], [512], [384, 1, 64]]),  # four tiles, boundaries everywhere
])
@pytest.mark.parametrize("p", [0.0, 0.2])
def test_attention_with_document_masks(dtype, d_head, S, lens, p):
    """Forward and backward of one attention call against the oracle run with the dense collator mask and the same
    dropout mask; the upstream gradient of padding rows is zero, as it is inside the model (their labels are padding)."""
    ops = pkg("operators")
    ops.DROPOUT_RATE = p
    try:
        B, H = len(lens), 2
        g = torch.Generator().manual_seed(S + d_head)
        qkv = torch.randn(B, H, 3, S, d_head, generator=g).to(dtype)
        mask = collator_mask(lens, S)
        live = non_pad_rows(mask)[:, None, :, None]
        d_o = (torch.randn(B, H, S, d_head, generator=g) * live).to(dtype)
        seed = 4711
        out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv.cuda(), mask.cuda(), True, seed)
        dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o.cuda(), acts, qkv.cuda(), mask.cuda(), True, seed)
        torch.cuda.synchronize()
        assert ops.last_kernel_fault() == 0
        drop = None
        if p > 0:
            drop = torch.from_numpy(philox.keep_mask(seed, 0, B * H * S * S, p)).view(B, H, S, S)
        q, k, v = (qkv[:, :, c].float() for c in range(3))
        am = mask.unsqueeze(1)
        o_ref, _ = orc.causal_attention(q, k, v, p, True, drop, am)
        rq, rk, rv = orc.causal_attention_bwd(d_o.float(), q, k, v, p, True, drop, am)
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert rel_err(out.cpu().float() * live, o_ref * live) < tol
        assert float((out.cpu().float() * ~live).abs().max()) == 0.0, "rows without keys give zeros"
        for name, a, b in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
            assert torch.isfinite(a).all(), name
            assert rel_err(a, b) < tol, f"{name}: {rel_err(a, b):.3e}"
        # log-sum-exp of the live rows
        s = torch.where(am, q @ k.transpose(-2, -1) / math.sqrt(d_head), torch.full((), float("-inf")))
        lse_ref = torch.logsumexp(s, dim=-1)
        lse = (acts[0] + torch.log(acts[1])).cpu()
        lv = live[..., 0].expand_as(lse)
        assert rel_err(lse[lv], lse_ref[lv]) < (1e-4 if dtype == torch.float32 else 1e-3)
        if dtype == torch.bfloat16 and p > 0:  # keep flags handed in or drawn in the kernels: same bits
            o4 = torch.empty_like(out)
            qd = qkv.cuda()
            ks = ops.row_kstart_from_mask(mask.cuda())
            bits = ops.attn_keep_bits(qd[:, :, 0], qd[:, :, 1], qd[:, :, 2], o4, seed)
            assert bits is not None
            ops.attn_fwd(qd[:, :, 0], qd[:, :, 1], qd[:, :, 2], o4, True, seed, keep_bits=bits, row_kstart=ks)
            assert torch.equal(o4, out)
    finally:
        ops.DROPOUT_RATE = 0.1


def test_tile_skipping_over_long_rows_and_several_items_per_block():
    """S = 1024 (eight tiles per row) with documents that start on and off tile boundaries, one row that is a single
    document, a padding tail that covers whole tiles, and more (row, head, tile) items than the GPU has SMs, so that
    blocks walk several items and both kernels' skip tables have more than one entry. Forward and backward against
    the oracle run with the dense mask, keep flags handed in (p = 0.1) and none (p = 0)."""
    ops = pkg("operators")
    S, H, dh = 1024, 4, 64
    lens = [[128] * 8, [1024], [100, 156, 256, 300, 212], [640], [513, 511], [1, 127, 129, 255, 257, 255]]
    B = len(lens)
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(B, H, 3, S, dh, generator=g).bfloat16()
    mask = collator_mask(lens, S)
    live = non_pad_rows(mask)[:, None, :, None]
    d_o = (torch.randn(B, H, S, dh, generator=g) * live).bfloat16()
    q, k, v = (qkv[:, :, c].float() for c in range(3))
    am = mask.unsqueeze(1)
    for p, seed in ((0.0, 3), (0.1, 4)):
        ops.DROPOUT_RATE = p
        try:
            out, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv.cuda(), mask.cuda(), True, seed)
            dq, dk, dv = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o.cuda(), acts, qkv.cuda(), mask.cuda(), True, seed)
            torch.cuda.synchronize()
            assert ops.last_kernel_fault() == 0
            drop = torch.from_numpy(philox.keep_mask(seed, 0, B * H * S * S, p)).view(B, H, S, S) if p > 0 else None
            o_ref, _ = orc.causal_attention(q, k, v, p, True, drop, am)
            rq, rk, rv = orc.causal_attention_bwd(d_o.float(), q, k, v, p, True, drop, am)
            assert rel_err(out.cpu().float() * live, o_ref * live) < 2e-2
            assert float((out.cpu().float() * ~live).abs().max()) == 0.0
            for name, a, b in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
                assert torch.isfinite(a).all(), name
                assert rel_err(a, b) < 2e-2, f"{name} (p = {p}): {rel_err(a, b):.3e}"
            # a second call gives the same bits (tile streams and reductions are fixed)
            out2, acts2 = ops.t_scaled_dot_prod_attn_fwd3_t(qkv.cuda(), mask.cuda(), True, seed)
            dq2, dk2, dv2 = ops.t_scaled_dot_prod_attn_bkwd3_t(d_o.cuda(), acts2, qkv.cuda(), mask.cuda(), True, seed)
            assert torch.equal(out, out2) and torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
        finally:
            ops.DROPOUT_RATE = 0.1


def test_packed_batch_bf16_model_against_oracle():
    """A small model on the tensor-core path (d_head 64, S 256) with packed rows and a padding tail, dropout 0.1 at
    all four sites: loss and every gradient against the fp32 oracle run with the dense mask."""
    ops, gpt2 = pkg("operators"), pkg("gpt2")
    p = 0.1
    ops.DROPOUT_RATE = p
    try:
        V, D, L, H, F, S = 512, 128, 2, 2, 256, 256
        lens = [[100, 90], [256], [64, 64, 64, 40]]
        B = len(lens)
        prm = orc.init_params(V, D, L, H, F, S, seed=12)
        prm_r = [[t.bfloat16().float() if t.dim() > 1 else t for t in grp] for grp in prm]
        y = torch.randint(1, V, (B, S + 1), generator=torch.Generator().manual_seed(13), dtype=torch.int32)
        mask = collator_mask(lens, S)
        for b, ls in enumerate(lens):
            y[b, sum(ls):] = 0  # the padding tail (inputs and labels)
        seeds = [500 + 7 * i for i in range(1 + 3 * L)]

        def mask_fn(site, shape):
            if site == "embed":
                sd = seeds[0]
            else:
                l, kind = site.split(".")
                sd = seeds[1 + 3 * int(l[1:]) + {"attn": 0, "res1": 1, "res2": 2}[kind]]
            return torch.from_numpy(philox.keep_mask(sd, 0, math.prod(shape), p)).view(shape)

        gp = [[(t.bfloat16() if t.dim() > 1 else t).cuda() for t in grp] for grp in prm]
        grads, (loss, acc, frac) = gpt2.t_loss_bkwd3_t(gp, y.cuda(), mask.cuda(), None, True, seeds)
        torch.cuda.synchronize()
        assert ops.last_kernel_fault() == 0
        ref, (rloss, _, rfrac) = orc.loss_and_grads(prm_r, y, p=p, train=True, mask_fn=mask_fn, attn_mask=mask)
        assert rel_err(loss, rloss) < 2e-2 and abs(float(frac) - float(rfrac)) < 1e-6
        for i, (a, b) in enumerate(zip(flat(grads), flat(ref))):
            assert torch.isfinite(a).all()
            assert rel_err(a, b) < 2e-2, f"gradient {i}: {rel_err(a, b):.3e}"
        # the trainer takes the same information as document lengths
        tr = pkg("trainer")
        cfg = gpt2.GPT2Config(vocab=V, dim=D, layers=L, heads=H, ffn=F, seq=S, dropout=0.0)
        t = tr.Trainer(cfg, tr.TrainConfig(seed=1), params=prm, device="cuda")
        ks = ops.row_kstart_from_lengths(lens, S)
        stats = t.step(y, row_kstart=ks)
        ref0, (rloss0, _, _) = orc.loss_and_grads(prm_r, y, attn_mask=mask)
        assert rel_err(stats[0], rloss0) < 2e-2
    finally:
        ops.DROPOUT_RATE = 0.1
