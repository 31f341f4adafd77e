"""tcgen05 GEMM through the C ABI against float64 products of the same bf16 inputs: every operand layout
(K-major / MN-major for A and B), ragged edges, both tile widths, split-K, and every epilogue."""
import math

import pytest
import torch

from conftest import pkg, rel_err
from oracle import gpt2_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu

TOL = 2e-2  # bf16 inputs, fp32 accumulate, bf16 or fp32 output


@pytest.fixture(scope="module")
def ops():
    return pkg("operators")


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).bfloat16()


def no_fault(ops):
    torch.cuda.synchronize()
    assert ops.last_kernel_fault() == 0, "a bounded wait inside the kernel ran out"


@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 512, 192), (200, 136, 72), (1024, 768, 768),
                                   (384, 2304, 768), (8, 8, 8)])
def test_layouts_and_edges(ops, a_k, b_k, M, N, K):
    A, B = rnd(M, K, seed=1), rnd(N, K, seed=2)  # logical A[M,K], B[N,K]
    ref = A.double() @ B.double().t()
    a_dev = (A if a_k else A.t().contiguous()).cuda()
    b_dev = (B if b_k else B.t().contiguous()).cuda()
    for out_dtype in (torch.bfloat16, torch.float32):
        c = ops.gemm(a_dev, b_dev, a_kmajor=a_k, b_kmajor=b_k, M=M, N=N, K=K, out_dtype=out_dtype)
        no_fault(ops)
        assert rel_err(c.float(), ref) < (TOL if out_dtype == torch.bfloat16 else 1e-3)


@pytest.mark.parametrize("split", [2, 3, 8])
def test_split_k_weight_gradient_shape(ops, split):
    """dW[N_out, N_in] = dY^T X with the token dimension as K: both operands MN-major, fp32 output, split-K."""
    T, N_out, N_in = 1024, 200, 136
    dY, X = rnd(T, N_out, seed=1), rnd(T, N_in, seed=2)
    ref = dY.double().t() @ X.double()
    out = torch.empty(N_out, N_in, device="cuda", dtype=torch.float32)
    ops.gemm(dY.cuda(), X.cuda(), a_kmajor=False, b_kmajor=False, M=N_out, N=N_in, K=T, out=out, split_k=split)
    no_fault(ops)
    assert rel_err(out, ref) < 1e-3
    out2 = torch.empty_like(out)
    ops.gemm(dY.cuda(), X.cuda(), a_kmajor=False, b_kmajor=False, M=N_out, N=N_in, K=T, out=out2, split_k=split)
    assert torch.equal(out, out2), "split-K must reduce in a fixed order"
    # accumulate onto existing contents
    lib = pkg("_lib")
    base = torch.full_like(out, 0.25)
    ops.gemm(dY.cuda(), X.cuda(), a_kmajor=False, b_kmajor=False, M=N_out, N=N_in, K=T, out=base, split_k=split,
             epilogue=lib.EPI_ACCUM)
    assert rel_err(base, ref + 0.25) < 1e-3


def test_epilogues(ops):
    lib = pkg("_lib")
    M, N, K = 256, 384, 128
    A, W = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.1)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(3))
    acc = A.double() @ W.double().t() + bias.double()
    a, w, b = A.cuda(), W.cuda(), bias.cuda()
    # bias only
    assert rel_err(ops.gemm(a, w, bias=b).float(), acc) < TOL
    # bias + GELU, pre-activation saved
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    act = ops.gemm(a, w, bias=b, epilogue=lib.EPI_GELU, aux_out=pre)
    assert rel_err(pre.float(), acc) < TOL
    assert rel_err(act.float(), orc.gelu(pre.float().cpu().double())) < TOL
    # GELU backward: acc * gelu'(saved pre-activation)
    pre_in = rnd(M, N, seed=4)
    out = ops.gemm(a, w, epilogue=lib.EPI_GELU_BWD, aux=pre_in.cuda())
    ref = orc.gelu_bwd(A.double() @ W.double().t(), pre_in.double())
    assert rel_err(out.float(), ref) < TOL
    # dropout + residual, mask from the host Philox on the logical [M, N] index space
    p, seed = 0.3, 4242
    resid = rnd(M, N, seed=5)
    mask = torch.from_numpy(philox.keep_mask(seed, 0, M * N, p)).view(M, N).double()
    out = ops.gemm(a, w, bias=b, epilogue=lib.EPI_DROPOUT_RESID, aux=resid.cuda(), dropout_args=(p, True, seed, 0))
    assert rel_err(out.float(), resid.double() + acc * mask) < TOL
    out = ops.gemm(a, w, bias=b, epilogue=lib.EPI_DROPOUT_RESID, aux=resid.cuda(), dropout_args=(p, False, seed, 0))
    assert rel_err(out.float(), resid.double() + acc * (1 - p)) < TOL
    no_fault(ops)


def test_padded_vocab_projection(ops):
    """LM-head pattern: N not a multiple of anything, leading dimension padded, and the matching input-gradient
    product whose reduction runs over the ragged dimension."""
    T, D, V = 256, 64, 1001
    ld = (V + 127) // 128 * 128
    X, W = rnd(T, D, seed=1), rnd(V, D, seed=2, scale=0.2)
    bias = torch.randn(V, generator=torch.Generator().manual_seed(3))
    logits = torch.full((T, ld), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.gemm(X.cuda(), W.cuda(), bias=bias.cuda(), out=logits, N=V, ldc=ld)
    ref = X.double() @ W.double().t() + bias.double()
    assert rel_err(logits[:, :V].float(), ref) < TOL
    assert float((logits[:, V:] - 7.0).abs().max()) == 0.0, "padding columns must not be written"
    dl = logits  # pretend gradient; padding columns hold junk that must not leak into the product
    dx = ops.gemm(dl, W.cuda(), a_kmajor=True, b_kmajor=False, M=T, N=D, K=V, lda=ld, ldb=D)
    assert rel_err(dx.float(), dl[:, :V].double().cpu() @ W.double()) < TOL
    dw = torch.empty(V, D, device="cuda", dtype=torch.float32)
    ops.gemm(dl, X.cuda(), a_kmajor=False, b_kmajor=False, M=V, N=D, K=T, lda=ld, ldb=D, out=dw)
    assert rel_err(dw, dl[:, :V].double().cpu().t() @ X.double()) < 1e-3
    no_fault(ops)


def test_rejects_bad_arguments(ops):
    a = rnd(64, 64).cuda()
    with pytest.raises(RuntimeError, match="aligned"):
        ops.gemm(a[:, 1:], a, M=64, N=64, K=56, lda=64)  # operand pointer not 16-byte aligned
    with pytest.raises(RuntimeError, match="shape"):
        ops.gemm(a, a, M=64, N=64, K=64, lda=8)  # leading dimension smaller than K


# ---- CTA-pair kernel (M, N >= 256 and K >= 2048 or N >= 8192) ---------------------------------------------------------
# The shapes below all route to the two-CTA kernel (256 x 256 tiles, tcgen05.mma.cta_group::2): exact multiples, a
# ragged M and N edge, and the long-K weight-gradient form.
PAIR_SHAPES = [(512, 768, 3072), (296, 520, 2048), (256, 256, 2048), (1024, 8200, 128)]


@pytest.mark.parametrize("a_k,b_k", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
def test_pair_kernel_layouts_and_edges(ops, a_k, b_k, M, N, K):
    A, B = rnd(M, K, seed=11), rnd(N, K, seed=12, scale=0.25)
    ref = A.double() @ B.double().t()
    a_dev = (A if a_k else A.t().contiguous()).cuda()
    b_dev = (B if b_k else B.t().contiguous()).cuda()
    for out_dtype in (torch.bfloat16, torch.float32):
        guard = torch.full((M + 1, N), 5.0, device="cuda", dtype=out_dtype)  # one row beyond the ragged M edge
        c = ops.gemm(a_dev, b_dev, a_kmajor=a_k, b_kmajor=b_k, M=M, N=N, K=K, out=guard[:M])
        no_fault(ops)
        assert rel_err(c.float(), ref) < (TOL if out_dtype == torch.bfloat16 else 1e-3)
        assert float((guard[M] - 5.0).abs().max()) == 0.0, "rows beyond M must not be written"


@pytest.mark.parametrize("M,N,K", [(512, 768, 3072), (296, 520, 2048)])
def test_pair_kernel_epilogues(ops, M, N, K):
    """Every epilogue of the two-CTA kernel, including the side input that arrives through tile loads (full blocks)
    and through plain loads (the ragged shape), against float64."""
    lib = pkg("_lib")
    A, W = rnd(M, K, seed=21), rnd(N, K, seed=22, scale=0.05)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(23))
    acc = A.double() @ W.double().t() + bias.double()
    a, w, b = A.cuda(), W.cuda(), bias.cuda()
    assert rel_err(ops.gemm(a, w, bias=b).float(), acc) < TOL
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    act = ops.gemm(a, w, bias=b, epilogue=lib.EPI_GELU, aux_out=pre)
    assert rel_err(pre.float(), acc) < TOL
    assert rel_err(act.float(), orc.gelu(pre.float().cpu().double())) < TOL
    for b_k in (True, False):  # forward form (x W^T) and input-gradient form (dy W) of the side-input epilogues
        w_dev = w if b_k else W.t().contiguous().cuda()
        pre_in = rnd(M, N, seed=24)
        out = ops.gemm(a, w_dev, b_kmajor=b_k, M=M, N=N, K=K, epilogue=lib.EPI_GELU_BWD, aux=pre_in.cuda())
        assert rel_err(out.float(), orc.gelu_bwd(A.double() @ W.double().t(), pre_in.double())) < TOL
        p, seed = 0.3, 777
        resid = rnd(M, N, seed=25)
        mask = torch.from_numpy(philox.keep_mask(seed, 0, M * N, p)).view(M, N).double()
        out = ops.gemm(a, w_dev, b_kmajor=b_k, M=M, N=N, K=K, bias=b, epilogue=lib.EPI_DROPOUT_RESID, aux=resid.cuda(),
                       dropout_args=(p, True, seed, 0))
        assert rel_err(out.float(), resid.double() + acc * mask) < TOL
        out = ops.gemm(a, w_dev, b_kmajor=b_k, M=M, N=N, K=K, bias=b, epilogue=lib.EPI_DROPOUT_RESID, aux=resid.cuda(),
                       dropout_args=(p, False, seed, 0))
        assert rel_err(out.float(), resid.double() + acc * (1 - p)) < TOL
    no_fault(ops)


@pytest.mark.parametrize("split", [1, 2, 3])
@pytest.mark.parametrize("N_out,N_in", [(768, 768), (520, 296)])
def test_pair_kernel_weight_gradient_split_k_accumulate(ops, split, N_out, N_in):
    """dW = dY^T X over 8192 tokens (both operands MN-major) on the two-CTA kernel: plain, split-K with the fixed-order
    reduction, and accumulation onto existing contents (the tied embedding gradient)."""
    lib = pkg("_lib")
    T = 8192
    dY, X = rnd(T, N_out, seed=31, scale=0.1), rnd(T, N_in, seed=32)
    ref = dY.double().t() @ X.double()
    kw = dict(a_kmajor=False, b_kmajor=False, M=N_out, N=N_in, K=T, split_k=split)
    out = torch.empty(N_out, N_in, device="cuda", dtype=torch.float32)
    ops.gemm(dY.cuda(), X.cuda(), out=out, **kw)
    no_fault(ops)
    assert rel_err(out, ref) < 1e-3
    again = torch.empty_like(out)
    ops.gemm(dY.cuda(), X.cuda(), out=again, **kw)
    assert torch.equal(out, again)
    base = torch.full_like(out, -0.5)
    ops.gemm(dY.cuda(), X.cuda(), out=base, epilogue=lib.EPI_ACCUM, **kw)
    assert rel_err(base, ref - 0.5) < 1e-3
    no_fault(ops)


@pytest.mark.parametrize("layout", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("shapes,K,splits", [
    (((3072, 768), (768, 3072)), 4096, (1, 1)),      # the two FFN weight gradients: 36 + 36 tiles, one round
    (((2304, 768), (768, 768)), 4096, (2, 2)),       # QKV + out-projection, K in two parts each
    (((520, 296), (264, 1032)), 2048, (1, 3)),       # ragged edges, different splits, second product accumulates
])
def test_two_products_in_one_launch_match_two_launches(ops, layout, shapes, K, splits):
    """ptj_gemm_grouped2 deals the tiles of two products to the thread-block pairs as one list: results must equal two
    separate launches with the same K split bit for bit, and the float64 product within tolerance."""
    lib = pkg("_lib")
    a_k, b_k = layout
    probs, refs, singles = [], [], []
    for i, ((M, N), s) in enumerate(zip(shapes, splits)):
        A, B = rnd(M, K, seed=41 + i, scale=0.1), rnd(N, K, seed=51 + i)
        a_dev = (A if a_k else A.t().contiguous()).cuda()
        b_dev = (B if b_k else B.t().contiguous()).cuda()
        acc = i == 1 and len(set(splits)) > 1
        out = torch.full((M, N), 0.25 if acc else float("nan"), device="cuda")
        one = out.clone()
        ops.gemm(a_dev, b_dev, a_kmajor=a_k, b_kmajor=b_k, M=M, N=N, K=K, out=one, split_k=s,
                 epilogue=lib.EPI_ACCUM if acc else lib.EPI_NONE)
        singles.append(one)
        refs.append(A.double() @ B.double().t() + (0.25 if acc else 0.0))
        probs.append(dict(a=a_dev, b=b_dev, out=out, lda=a_dev.stride(0), ldb=b_dev.stride(0), split_k=s, accumulate=acc))
    assert ops.gemm_grouped2(probs, K, a_kmajor=a_k, b_kmajor=b_k)
    no_fault(ops)
    for pr, one, ref in zip(probs, singles, refs):
        assert rel_err(pr["out"], ref) < 1e-3
        assert torch.equal(pr["out"], one), "grouped and separate launches walk K in the same order"


def test_grouped_launch_refuses_small_products(ops):
    """Products the thread-block-pair kernel does not take are refused as a pair (nothing is launched)."""
    a, b = rnd(128, 256, seed=1).cuda(), rnd(128, 256, seed=2).cuda()
    out = torch.zeros(128, 128, device="cuda")
    pr = dict(a=a, b=b, out=out, lda=256, ldb=256)
    assert ops.gemm_grouped2([dict(pr), dict(pr)], 256) is False
    assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("T,N,K", [(8192, 768, 3072), (8192, 768, 2304), (5000, 776, 2048)])
def test_input_gradient_with_the_last_round_of_tiles_split_over_k(T, N, K):
    """Gpt2Step._dgrad hands a product whose last round of 256 x 256 tiles is mostly empty to the two-product launch:
    head rows as they were, the remaining rows split over K. Head rows equal the plain launch bit for bit, the rest
    within rounding of it (another summation order), everything within tolerance of the float64 product."""
    gpt2, ops = pkg("gpt2"), pkg("operators")
    step = gpt2.Gpt2Step(gpt2.GPT2Config(vocab=512, dim=128, layers=1, heads=2, ffn=256, seq=128, dropout=0.0))
    dy, w = rnd(T, K, seed=61, scale=0.1), rnd(K, N, seed=62)  # dx = dy w, w read MN-major
    ref = dy.double() @ w.double()
    tail = gpt2.tail_split_for(T, N, K)  # (first split row, workspace floats) or None
    got = step._dgrad(dy.cuda(), w.cuda())
    no_fault(ops)
    plain = ops.gemm(dy.cuda(), w.cuda(), a_kmajor=True, b_kmajor=False, M=T, N=N, K=K)
    assert rel_err(got, ref) < TOL
    if tail is None:
        assert torch.equal(got, plain)
    else:
        head = tail[0]
        assert 0 < head < T
        assert torch.equal(got[:head], plain[:head])
        assert rel_err(got[head:], plain[head:]) < 1e-2
    step.tail_split = False
    assert torch.equal(step._dgrad(dy.cuda(), w.cuda()), plain)


@pytest.mark.parametrize("train", [True, False])
def test_dropout_residual_product_with_the_last_round_split_over_k(ops, train):
    """FFN-2 forward at GPT-2 small size (96 tiles of 256 x 256) with PTJ_SPLIT_TAIL: bias + dropout + residual of the
    split rows are applied by the finishing kernel with the mask of their position in the whole matrix. Head rows
    equal the unsplit launch bit for bit; everything matches the float64 product with the host mask."""
    lib = pkg("_lib")
    M, N, K, p_drop, seed = 8192, 768, 3072, 0.3, 99
    A, B = rnd(M, K, seed=71, scale=0.1), rnd(N, K, seed=72)
    bias, res = torch.randn(N, generator=torch.Generator().manual_seed(3)), rnd(M, N, seed=73)
    head = int(lib.lib().ptj_gemm_tail_split_rows(M, N, K))
    assert 0 < head < M
    kw = dict(bias=bias.cuda(), epilogue=lib.EPI_DROPOUT_RESID, aux=res.cuda(), dropout_args=(p_drop, train, seed, 2))
    plain = ops.gemm(A.cuda(), B.cuda(), **kw)
    got = ops.gemm(A.cuda(), B.cuda(), split_k=ops.SPLIT_TAIL, **kw)
    no_fault(ops)
    acc = A.double() @ B.double().t() + bias.double()
    if train:
        keep = torch.from_numpy(philox.keep_mask(seed, 2, M * N, p_drop)).view(M, N)
        ref = res.double() + acc * keep
    else:
        ref = res.double() + acc * (1 - p_drop)
    assert rel_err(got, ref) < TOL and rel_err(plain, ref) < TOL
    assert torch.equal(got[:head], plain[:head])
    assert rel_err(got[head:], plain[head:]) < 1e-2
    if train:  # the same elements are dropped (where the product is dropped the output IS the residual)
        assert torch.equal(got == res.cuda(), plain == res.cuda())
