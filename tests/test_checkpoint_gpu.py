"""Resuming a Trainer from a checkpoint in the reference's wire format continues the run bit for bit."""
import pytest
import torch

from conftest import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_trainer_resume_is_bit_exact(tmp_path, dtype):
    gpt2, tr, ck = pkg("gpt2"), pkg("trainer"), pkg("checkpoint")
    cfg = gpt2.GPT2Config(vocab=160, dim=64, layers=2, heads=2, ffn=128, seq=32, dropout=0.1)
    tc = tr.TrainConfig.benchmark_recipe(lr=1e-3, compute_dtype=dtype, seed=21)
    g = torch.Generator().manual_seed(8)
    batches = [torch.randint(0, 160, (2, 33), generator=g, dtype=torch.int32) for _ in range(5)]
    a = tr.Trainer(cfg, tc, device="cuda")
    for y in batches[:3]:
        a.step(y)
    path = ck.checkpoint_name(str(tmp_path), a)
    assert path.endswith("checkpoint_3.pkl")
    ck.save_trainer(path, a, ds_train_rows_read=6)
    b = tr.Trainer(cfg, tr.TrainConfig.benchmark_recipe(lr=1e-3, compute_dtype=dtype, seed=21), device="cuda")
    assert ck.load_trainer_state(b, path) == (3, 6) and b.t == 3
    for y in batches[3:]:
        sa, sb = a.step(y), b.step(y)
        assert torch.equal(sa, sb)  # same dropout seeds (derived from the step index), same weights, same moments
    assert torch.equal(a.p, b.p) and torch.equal(a.m, b.m) and torch.equal(a.v, b.v)
    # the file holds float32 CPU pytrees in the reference's layout
    i, rows, params, (m, v) = ck.load_checkpoint(path)
    assert [len(grp) for grp in params] == [2, 1, 10, 10, 2] and params[0][0].shape == (160, 64)
