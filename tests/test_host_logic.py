"""Host-side logic of the data-parallel trainer on the CPU: flat layout, buckets, weight-decay segments, seeds, and
the bucketed gradient allreduce across two gloo ranks (including its failure paths)."""
import math
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import pkg
from oracle import gpt2_oracle as orc


def cfg_small():
    return pkg("gpt2").GPT2Config(vocab=101, dim=16, layers=3, heads=2, ffn=32, seq=8, dropout=0.1)


def test_layout_covers_every_parameter_once():
    tr, cfg = pkg("trainer"), cfg_small()
    lay = tr.FlatLayout.build(cfg)
    assert sorted(lay.names) == sorted(n for n, _ in cfg.param_shapes())
    spans = sorted((lay.offsets[n], lay.offsets[n] + math.prod(lay.shapes[n])) for n in lay.names)
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 <= b0
    assert all(o % tr.ALIGN == 0 for o in lay.offsets.values()) and lay.total % tr.ALIGN == 0
    # backward order: head bias first, embedding (tied, finished by the scatter) last
    assert lay.names[0] == "b_head" and lay.names[-2:] == ["w_emb", "w_pos"]
    assert lay.names.index("l2.w2") < lay.names.index("l1.w2") < lay.names.index("l0.w2")
    assert cfg.num_params() == sum(math.prod(s) for s in lay.shapes.values())


def test_gpt2_small_parameter_count():
    g = pkg("gpt2")
    assert g.PRESETS["gpt2-small"].num_params() == 124_453_201
    assert g.PRESETS["gpt2-medium"].num_params() == 354_775_121
    assert g.PRESETS["tiny"].num_params() == 544_256


def test_buckets_are_contiguous_and_bounded():
    tr, cfg = pkg("trainer"), cfg_small()
    lay = tr.FlatLayout.build(cfg)
    buckets = tr.make_buckets(lay, 1500)
    assert buckets[0].start == 0 and buckets[-1].end == lay.total
    for a, b in zip(buckets, buckets[1:]):
        assert a.end == b.start
    assert [n for b in buckets for n in b.names] == lay.names
    for b in buckets:
        assert len(b.names) == 1 or b.end - b.start <= 1500
    assert len(tr.make_buckets(lay, 10 ** 9)) == 1


def test_decay_segments_follow_reference_rule():
    tr, g, cfg = pkg("trainer"), pkg("gpt2"), cfg_small()
    lay = tr.FlatLayout.build(cfg)
    starts, flags = lay.decay_segments()
    assert starts[0] == 0 and starts[-1] == lay.total and len(starts) == len(flags) + 1
    assert all(a < b for a, b in zip(starts, starts[1:])) and all(s % 4 == 0 for s in starts)
    for n in lay.names:
        seg = max(i for i, s in enumerate(starts[:-1]) if s <= lay.offsets[n])
        assert bool(flags[seg]) == g.is_decayed(n)
    # LayerNorm scales are decayed, shifts and biases are not (1-D tensors that start as zeros)
    assert g.is_decayed("l0.g1") and g.is_decayed("g_f") and g.is_decayed("l1.w_qkv")
    assert not g.is_decayed("l0.b1") and not g.is_decayed("b_head") and not g.is_decayed("l2.b2f")
    prm = pkg("optimizer").init_from_config(cfg, device="cpu", seed=0)
    mask = pkg("optimizer").weight_decay_mask(prm)
    flat_mask = [m for grp in mask for m in grp]
    assert flat_mask == [g.is_decayed(n) for n, _ in cfg.param_shapes()]


def test_init_matches_reference_scales():
    opt, cfg = pkg("optimizer"), pkg("gpt2").GPT2Config(vocab=500, dim=64, layers=4, heads=4, ffn=256, seq=32)
    prm = opt.init_from_config(cfg, device="cpu", seed=3)
    assert [len(g) for g in prm] == [2, 1, 10, 10, 10, 10, 2]
    assert abs(float(prm[0][0].std()) - 0.02) < 1e-3
    assert abs(float(prm[2][3].std()) - 0.02 / math.sqrt(8)) < 5e-4  # attention output projection
    assert abs(float(prm[2][8].std()) - 0.02 / math.sqrt(8)) < 5e-4  # second FFN matrix
    assert float(prm[2][0].min()) == 1.0 and float(prm[2][1].abs().max()) == 0.0
    assert tuple(prm[2][2].shape) == (4, 3, 16, 64)
    again = opt.init_from_config(cfg, device="cpu", seed=3)
    assert all(torch.equal(a, b) for ga, gb in zip(prm, again) for a, b in zip(ga, gb))


def test_step_seeds_are_distinct():
    tr = pkg("trainer")
    a = tr.step_seeds(0, 0, 0, 37)
    assert len(set(a)) == 37
    assert set(a).isdisjoint(tr.step_seeds(0, 1, 0, 37)) and set(a).isdisjoint(tr.step_seeds(0, 0, 1, 37))
    assert a == tr.step_seeds(0, 0, 0, 37)
    assert all(0 <= s < 2 ** 63 for s in a)  # bit 63 of a seed argument marks a device-resident seed


def test_split_k_heuristic():
    f = pkg("gpt2").split_k_for     # (M, N, K) of the weight-gradient product, K = tokens
    assert f(50257, 768, 8192) == 1      # LM-head weight gradient: plenty of tiles already
    assert f(768, 768, 8192) == 8        # 9 tiles of 256 x 256: needs a K split to fill the 74 thread-block pairs
    assert f(3072, 768, 8192) == 2       # 36 tiles: two parts make one round of 72 work items
    assert f(2304, 768, 8192) == 5
    assert f(128, 128, 128) == 1         # nothing to split


# ---- two gloo ranks -------------------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tr, cfg = pkg("trainer"), cfg_small()
        lay = tr.FlatLayout.build(cfg)
        g = torch.Generator().manual_seed(100 + rank)
        flat = torch.randn(lay.total, generator=g)
        mine = flat.clone()
        red = tr.GradReducer(flat, lay, bucket_mb=0.004, group=None)
        assert len(red.buckets) > 3
        if case == "sum":
            for names in ([n] for n in lay.names):  # gradients become ready one tensor at a time
                red.mark_ready(names)
            red.finish()
            other = torch.randn(lay.total, generator=torch.Generator().manual_seed(100 + (1 - rank)))
            ok = torch.allclose(flat, mine + other, atol=1e-6)
            red.reset()
            red.mark_ready(lay.names)
            red.finish()
            ret[rank] = bool(ok)
        elif case == "missing":
            red.mark_ready(lay.names[:-1])  # the last gradient never arrives: finish must refuse, not hang
            try:
                red.finish()
                ret[rank] = False
            except RuntimeError as e:
                ret[rank] = "never produced" in str(e)
        elif case == "twice":
            red.mark_ready([lay.names[0]])
            try:
                red.mark_ready([lay.names[0]] * 50)
                ret[rank] = False
            except RuntimeError as e:
                ret[rank] = "twice" in str(e)
    finally:
        dist.destroy_process_group()


def _leaver(rank, world, port, ret):
    """Both ranks run two steps; rank 1 then leaves between steps (nothing in flight). Rank 0 must learn of it on the
    host, before it launches the third step's collective, and within the watch's time limit."""
    import time
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tr, cfg = pkg("trainer"), cfg_small()
    lay = tr.FlatLayout.build(cfg)
    store = dist.distributed_c10d._get_default_store()
    watch = tr.PeerWatch(store, rank, world, timeout_s=1.5)
    flat = torch.ones(lay.total)
    red = tr.GradReducer(flat, lay, bucket_mb=0.004, wait_timeout_s=5.0)
    launched_after_loss = False
    try:
        for step in range(3):
            if rank == 1 and step == 2:
                ret[rank] = "left"
                return  # leaves between steps, without announcing step 2
            watch.announce(step)
            t0 = time.time()
            try:
                watch.check(step)
            except tr.PeerLost as e:
                ret[rank] = ("lost", step, time.time() - t0 < 10.0, "rank(s) [1]" in str(e), launched_after_loss)
                return
            red.reset()
            red.mark_ready(lay.names)
            launched_after_loss = launched_after_loss or step == 2
            red.finish()
        ret[rank] = "finished"
    finally:
        if rank == 1:
            time.sleep(3.0)  # keep the store's peer alive while rank 0 times out on the missing key
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_leaving_between_steps_is_noticed_on_the_host():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert ret.get(1) == "left"
    assert ret.get(0) == ("lost", 2, True, True, False), ret.get(0)


@pytest.mark.parametrize("case", ["sum", "missing", "twice"])
def test_bucketed_allreduce_two_ranks(case):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert ret.get(0) is True and ret.get(1) is True


def test_sharded_oracle_gradients_average_to_full_batch():
    """The data-parallel contract, stated on the CPU oracle: with no padding labels, the mean over ranks of the
    per-shard gradients equals the gradient of the concatenated batch."""
    from oracle import gpt2_oracle as orc
    prm = orc.init_params(64, 16, 1, 2, 32, 8, seed=1, dtype=torch.float64)
    g = torch.Generator().manual_seed(2)
    y = torch.randint(1, 64, (4, 9), generator=g)
    full, (loss, _, frac) = orc.loss_and_grads(prm, y)
    assert float(frac) == 1.0
    a, _ = orc.loss_and_grads(prm, y[:2])
    b, _ = orc.loss_and_grads(prm, y[2:])
    for fa, fb, ff in zip((t for grp in a for t in grp), (t for grp in b for t in grp), (t for grp in full for t in grp)):
        assert torch.allclose((fa + fb) / 2, ff, atol=1e-12)


def test_checkpoint_wire_format_round_trip(tmp_path):
    """The file is the reference's pickle tuple (i, ds_train_rows_read, params, [m, v]) (train_gpt2_triton.py:413-419):
    plain pickle.load, as the reference's resume code does (:277-280), must give that structure back."""
    import pickle
    ck = pkg("checkpoint")
    prm = orc.init_params(40, 16, 2, 2, 32, 8, seed=3)
    g = torch.Generator().manual_seed(4)
    m = [[torch.randn(t.shape, generator=g) for t in grp] for grp in prm]
    v = [[torch.rand(t.shape, generator=g) for t in grp] for grp in prm]
    path = tmp_path / "run" / "checkpoint_7.pkl"
    ck.save_checkpoint(str(path), 7, 1234, prm, [m, v])
    with open(path, "rb") as f:
        i, rows, p2, mom = pickle.load(f)
    assert (i, rows) == (7, 1234) and len(mom) == 2
    assert [len(grp) for grp in p2] == [2, 1, 10, 10, 2]
    for a, b in zip([t for grp in p2 for t in grp], [t for grp in prm for t in grp]):
        assert a.dtype == torch.float32 and a.device.type == "cpu" and torch.equal(a, b)
    i, rows, p3, (m3, v3) = ck.load_checkpoint(str(path))
    assert (i, rows) == (7, 1234)
    assert all(torch.equal(a, b) for ga, gb in zip(m3, m) for a, b in zip(ga, gb))
    assert all(torch.equal(a, b) for ga, gb in zip(v3, v) for a, b in zip(ga, gb))
    # a file written the way the reference writes it loads as well
    ref_style = tmp_path / "ref.pkl"
    with open(ref_style, "wb") as f:
        pickle.dump((3, 99, prm, [m, v]), f)
    assert ck.load_checkpoint(str(ref_style))[:2] == (3, 99)
    # structure errors are reported, not silently accepted
    with pytest.raises(ValueError):
        ck.save_checkpoint(str(tmp_path / "bad.pkl"), 0, 0, prm, [m[:-1], v])
    with open(tmp_path / "short.pkl", "wb") as f:
        pickle.dump((1, 2, prm), f)
    with pytest.raises(ValueError):
        ck.load_checkpoint(str(tmp_path / "short.pkl"))
    assert not list(tmp_path.glob("**/*.tmp.*"))


def test_checkpoint_step_index_follows_the_reference(tmp_path):
    """The reference counts a micro-step BEFORE it pickles (train_gpt2_triton.py:408-419): after N steps the file holds
    i = N, is named checkpoint_N.pkl, and the run that resumes it calls adam_w_in_place(..., i) next, i.e. AdamW step
    count N + 1 (:321). A trainer that loads such a file must stand at t = N completed steps, and a trainer that has
    completed N steps must write i = N."""
    import pickle
    from types import SimpleNamespace
    ck, gpt2, tr = pkg("checkpoint"), pkg("gpt2"), pkg("trainer")
    cfg = gpt2.GPT2Config(vocab=40, dim=16, layers=2, heads=2, ffn=32, seq=8, dropout=0.0)
    prm = orc.init_params(40, 16, 2, 2, 32, 8, seed=3)
    zeros = lambda: [[torch.zeros_like(t) for t in grp] for grp in prm]
    N = 5
    # the reference's loop, reduced to its counters
    i, rows, moments = 0, 0, [zeros(), zeros()]
    adamw_counts = []
    for _ in range(N):
        adamw_counts.append(i + 1)  # adam_w_in_place(params, grads, lr, betas, eps, moments, i, ...): t = i + 1
        i, rows = i + 1, rows + 4
    ref_file = tmp_path / f"checkpoint_{i}.pkl"
    with open(ref_file, "wb") as f:
        pickle.dump((i, rows, prm, moments), f)
    assert adamw_counts[-1] == N and i == N

    lay = tr.FlatLayout.build(cfg)
    flat = lambda: torch.zeros(lay.total)
    stand_in = SimpleNamespace(cfg=cfg, layout=lay, p=flat(), m=flat(), v=flat(), t=0, device=torch.device("cpu"),
                               _refresh_shadow=lambda: None)
    assert ck.load_trainer_state(stand_in, str(ref_file)) == (N, rows)
    assert stand_in.t == N  # Trainer.apply_update increments before use: the next AdamW step count is N + 1
    for (name, _), t in zip(cfg.param_shapes(), [t for grp in prm for t in grp]):
        assert torch.equal(lay.view(stand_in.p, name), t)
    # and the other direction: N completed steps are written as i = N under the reference's file name
    out = ck.checkpoint_name(str(tmp_path / "run"), stand_in)
    assert out.endswith(f"checkpoint_{N}.pkl")
    ck.save_trainer(out, stand_in, ds_train_rows_read=rows)
    with open(out, "rb") as f:
        i2, rows2, p2, _ = pickle.load(f)
    assert (i2, rows2) == (N, rows)
    assert all(torch.equal(a, b) for ga, gb in zip(p2, prm) for a, b in zip(ga, gb))
