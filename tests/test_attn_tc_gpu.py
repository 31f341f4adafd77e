"""tcgen05 flash attention (bf16, head size 64, sequence a multiple of 128) through the C ABI against the CPU oracle:
forward output, saved softmax statistics, dQ / dK / dV, dropout on the probabilities with the host-generated mask,
strided views of a fused projection buffer, and bit-reproducibility."""
import math

import pytest
import torch

from conftest import pkg, rel_err
from oracle import gpt2_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def ops():
    return pkg("operators")


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).bfloat16()


def run_case(ops, B, H, S, p, train, seed, fused_layout):
    D = 64
    ops.DROPOUT_RATE = p
    try:
        if fused_layout:  # [B*S, H*3*D] projection output, columns ordered (head, q/k/v, d): what the train step uses
            buf = rnd(B * S, H * 3 * D, seed=1).cuda()
            v5 = buf.view(B, S, H, 3, D)
            q, k, v = (v5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
            out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
            o4 = out.view(B, S, H, D).permute(0, 2, 1, 3)
            d_out = rnd(B * S, H * D, seed=2).cuda()
            do4 = d_out.view(B, S, H, D).permute(0, 2, 1, 3)
            dbuf = torch.empty_like(buf)
            d5 = dbuf.view(B, S, H, 3, D)
            dq, dk, dv = (d5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
        else:  # the reference's [B, H, 3, N, D] tensor
            qkv = rnd(B, H, 3, S, D, seed=1).cuda()
            q, k, v = qkv.unbind(dim=2)
            o4 = torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16)
            do4 = rnd(B, H, S, D, seed=2).cuda()
            dq, dk, dv = (torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        m, l = ops.attn_fwd(q, k, v, o4, train, seed)
        ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, train, seed)
        torch.cuda.synchronize()
        assert ops.last_kernel_fault() == 0, "a bounded wait inside a tensor-core kernel ran out"
        qf, kf, vf, gf = (t.float().cpu() for t in (q, k, v, do4))
        mask = None
        if train and p > 0:
            mask = torch.from_numpy(philox.keep_mask(seed, 0, B * H * S * S, p)).view(B, H, S, S)
        o_ref, _ = orc.causal_attention(qf, kf, vf, p, train, mask)
        assert rel_err(o4, o_ref) < TOL, f"O {rel_err(o4, o_ref):.3e}"
        rm, rl = orc.causal_attention_stats(qf, kf)
        assert rel_err(m + torch.log(l), rm + torch.log(rl)) < 1e-3
        rq, rk, rv = orc.causal_attention_bwd(gf, qf, kf, vf, p, train, mask)
        for name, a, b in (("dQ", dq, rq), ("dK", dk, rk), ("dV", dv, rv)):
            assert rel_err(a, b) < TOL, f"{name} {rel_err(a, b):.3e}"
        return o4.clone(), dq.clone(), dk.clone(), dv.clone()
    finally:
        ops.DROPOUT_RATE = 0.1


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 512), (2, 12, 1024)])
@pytest.mark.parametrize("fused_layout", [False, True])
def test_no_dropout(ops, B, H, S, fused_layout):
    run_case(ops, B, H, S, 0.0, True, 0, fused_layout)


@pytest.mark.parametrize("B,H,S", [(1, 2, 128), (2, 2, 384)])
def test_dropout_on_probabilities(ops, B, H, S):
    run_case(ops, B, H, S, 0.1, True, 0xABCDEF12345, True)
    run_case(ops, B, H, S, 0.1, False, 0, False)  # evaluation: probabilities scaled by 1 - p


def test_bit_reproducible(ops):
    a = run_case(ops, 2, 4, 512, 0.1, True, 77, True)
    b = run_case(ops, 2, 4, 512, 0.1, True, 77, True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_tensor_core_and_cuda_core_kernels_agree(ops, monkeypatch):
    """Same bf16 inputs through the tcgen05 kernels and through the exact-fp32 CUDA-core kernels (sequence 192 is not
    a multiple of 128, so slicing the same data to 192 rows routes to the other implementation)."""
    B, H, S, D = 1, 2, 256, 64
    qkv = rnd(B, H, 3, S, D, seed=5).cuda()
    ops.DROPOUT_RATE = 0.0
    out_tc, acts = ops.t_scaled_dot_prod_attn_fwd3_t(qkv, None, True, 1)
    out_cc, _ = ops.t_scaled_dot_prod_attn_fwd3_t(qkv[:, :, :, :192].contiguous(), None, True, 1)
    assert rel_err(out_tc[:, :, :192], out_cc) < TOL  # causal: the first 192 rows do not see the rest
    ops.DROPOUT_RATE = 0.1


def test_keep_bits_handed_over_match_the_in_kernel_mask():
    """ptj_attn_keep_bits draws the call's dropout flags once; forward and backward given those flags must return
    exactly what they return when they draw the mask themselves, and the flags must equal the oracle's mask stream."""
    ops = pkg("operators")
    B, H, S, D, p, seed = 2, 3, 384, 64, 0.25, 77
    ops.DROPOUT_RATE = p
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, H, 3, S, D, generator=g).bfloat16().cuda()
    q, k, v = qkv.unbind(dim=2)
    do4 = torch.randn(B, H, S, D, generator=g).bfloat16().cuda()
    res = []
    for use_bits in (False, True):
        o4 = torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16)
        dq, dk, dv = (torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        bits = ops.attn_keep_bits(q, k, v, o4, seed) if use_bits else None
        assert (bits is not None) == use_bits
        m, l = ops.attn_fwd(q, k, v, o4, True, seed, keep_bits=bits)
        ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, True, seed, keep_bits=bits)
        res.append((o4, m, l, dq, dk, dv, bits))
    torch.cuda.synchronize()
    assert ops.last_kernel_fault() == 0
    for a, b in zip(res[0][:6], res[1][:6]):
        assert torch.equal(a, b)
    # layout: uint4 per (batch*head, tile (qt, kt) in triangular order, row); word c = columns 32c..32c+31
    bits = res[1][6].cpu().numpy().view("uint32").reshape(B * H, 6, 128, 4)
    mask = philox.keep_mask(seed, 0, B * H * S * S, p).reshape(B * H, S, S)
    for bh, qt, kt, row, c in ((0, 0, 0, 5, 0), (3, 2, 1, 127, 3), (5, 1, 1, 64, 2), (2, 2, 0, 0, 1)):
        word = int(bits[bh, qt * (qt + 1) // 2 + kt, row, c])
        want = mask[bh, qt * 128 + row, kt * 128 + c * 32: kt * 128 + c * 32 + 32]
        got = [(word >> i) & 1 for i in range(32)]
        assert got == [int(x) for x in want]
    ops.DROPOUT_RATE = 0.1
