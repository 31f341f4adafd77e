"""Evaluation / inference callers on the GPU (loss_eval, log_probs, predict, the row arg-max kernel) against the
reference's own outputs (tests/golden/eval_callers.npz) and the CPU oracle."""
import pytest
import torch

from conftest import pkg, rel_err, tt
from oracle import gpt2_oracle as orc
from test_model_gpu import BF16_TOL, F32_TOL, to_cuda, tree_from_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,ld", [(1, 1, 1), (7, 33, 40), (64, 1001, 1024), (16, 50257, 50264)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_argmax_rows(rows, cols, ld, dtype):
    ops = pkg("operators")
    g = torch.Generator().manual_seed(rows * 131 + cols)
    x = torch.randn(rows, ld, generator=g).to(dtype).cuda()
    x[:, cols:] = 100.0  # padding columns must not be looked at
    if cols > 8:
        x[0, 5] = x[0, 3] = 50.0  # a tie: the first index wins
    got = ops.argmax_rows(x, cols=cols)
    ref = torch.argmax(x[:, :cols].float().cpu(), dim=-1)
    assert got.dtype == torch.int32 and torch.equal(got.cpu().long(), ref)
    if cols > 8:
        assert int(got[0]) == 3


def test_argmax_rows_strided_rows():
    ops = pkg("operators")
    x = torch.randn(4, 6, 72, generator=torch.Generator().manual_seed(3)).cuda()
    got = ops.argmax_rows(x[:, 2], cols=65)  # rows 6 * 72 elements apart, as predict slices its logits
    assert torch.equal(got.cpu().long(), torch.argmax(x[:, 2, :65].cpu(), dim=-1))


def test_eval_callers_fp32_match_reference(tiny_golden, eval_golden):
    g, e, ops, ev = tiny_golden, eval_golden, pkg("operators"), pkg("evaluate")
    assert abs(ops.DROPOUT_RATE - float(e["dropout"])) < 1e-6
    params = to_cuda(tree_from_golden(g, g["dims"]))
    y = tt(g["y"]).cuda()
    logits = ev.t_gpt2_forward(params, y[:, :-1], None, None, False)
    assert rel_err(logits, tt(e["logits_eval"])) < F32_TOL
    loss, (loss2, acc, frac) = ev.loss_eval(params, y)
    assert rel_err(loss, tt(e["loss"])) < F32_TOL and float(loss) == float(loss2)
    assert rel_err(acc, tt(e["acc"])) < 1e-6 and rel_err(frac, tt(e["frac"])) < 1e-6
    lp = ev.log_probs(params, y)
    assert lp.shape == (y.shape[0],) and rel_err(lp, tt(e["log_probs"])) < F32_TOL
    # training-mode loss differs (masks instead of the 1 - p scale), so the flag really reaches the kernels
    loss_train, _ = ev.t_loss(params, y, None, None, True, [3] * 7)
    assert abs(float(loss_train) - float(loss)) > 1e-4


def test_predict_fp32_matches_reference(tiny_golden, eval_golden):
    g, e, ev = tiny_golden, eval_golden, pkg("evaluate")
    params = tree_from_golden(g, g["dims"])
    params = to_cuda([[params[0][0], tt(e["b_head_pred"])], [tt(e["w_pos_pred"])]] + params[2:])
    S, B = int(g["dims"][5]), int(g["dims"][6])
    pred = ev.predict(params, B, None, S, int(e["start_tok"]), int(e["end_tok"]))
    assert pred.shape == (B, S - 1) and pred.dtype == torch.int64
    assert torch.equal(pred.cpu(), tt(e["predict"]))


def test_eval_callers_bf16_against_oracle():
    """bf16 compute against the fp32 oracle at the bf16 tolerance, on a model big enough to use the tensor-core path."""
    ops, ev, opt = pkg("operators"), pkg("evaluate"), pkg("optimizer")
    V, D, L, H, F, S, B = 512, 128, 2, 2, 256, 128, 2
    params = orc.init_params(V, D, L, H, F, S, seed=9)
    y = torch.randint(0, V, (B, S + 1), generator=torch.Generator().manual_seed(9), dtype=torch.int32)
    p = ops.DROPOUT_RATE
    rounded = [[t.bfloat16().float() if t.dim() > 1 else t for t in grp] for grp in params]  # weights as the GPU sees them
    loss_ref, acc_ref, frac_ref = orc.loss_eval(rounded, y.long(), p)
    lp_ref = orc.log_probs(rounded, y.long(), p)
    dev = [[(t.bfloat16() if t.dim() > 1 else t).cuda() for t in grp] for grp in params]
    loss, (_, acc, frac) = ev.loss_eval(dev, y.cuda())
    assert rel_err(loss, loss_ref) < BF16_TOL and rel_err(frac, frac_ref) < 1e-6
    assert rel_err(ev.log_probs(dev, y.cuda()), lp_ref) < BF16_TOL
