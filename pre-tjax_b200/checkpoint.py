"""Checkpoints in the reference's own wire format, so that either side can resume the other's run.

The reference's train script pickles the tuple ``(i, ds_train_rows_read, params, moments)``
(train_gpt2_triton.py:413-419) and resumes with ``i, ds_train_rows_read, params, moments = pickle.load(f)``
(:277-280): ``i`` is the micro-step index, ``ds_train_rows_read`` the number of dataset rows consumed, ``params`` the
parameter pytree of model_torch_func.py:36-43 and ``moments = [m, v]`` two pytrees of the same shape
(``init_adam_w``, loss_and_optimizer_triton.py:362-363). Tensors are float32. Files written here hold CPU tensors (a
pickle of CUDA tensors can only be opened on a machine with a GPU); ``load_checkpoint`` moves them to the device asked
for. A ``Trainer`` keeps parameters and moments in flat buffers; ``trainer_state`` / ``load_trainer_state`` convert
between those and the pytrees. The reference increments ``i`` BEFORE it pickles (train_gpt2_triton.py:408-419): the
saved ``i`` is the number of completed micro-steps, which is also the index of the next one, and the next AdamW call
``adam_w_in_place(..., i)`` uses step count ``i + 1`` (:321). A trainer that has taken ``t`` steps is therefore saved
as ``i = t`` (file name ``checkpoint_{t}.pkl`` in the reference's scheme) and a loaded ``i`` becomes ``trainer.t = i``.
"""
from __future__ import annotations

import os
import pickle
from typing import Tuple

import torch

from .gpt2 import unflatten_like


def _map_tree(tree, fn):
    return [[fn(t) for t in grp] for grp in tree]


def check_same_structure(a, b, what: str):
    if len(a) != len(b) or any(len(x) != len(y) for x, y in zip(a, b)):
        raise ValueError(f"{what}: pytree structure differs")
    for gx, gy in zip(a, b):
        for tx, ty in zip(gx, gy):
            if tuple(tx.shape) != tuple(ty.shape):
                raise ValueError(f"{what}: tensor shape {tuple(tx.shape)} differs from {tuple(ty.shape)}")


def save_checkpoint(path: str, i: int, ds_train_rows_read: int, params, moments) -> None:
    """Pickle ``(i, ds_train_rows_read, params, moments)`` with float32 CPU tensors; written to a temporary file first
    and renamed, so an interrupted save never leaves a truncated checkpoint under the final name."""
    m, v = moments
    check_same_structure(params, m, "first moments")
    check_same_structure(params, v, "second moments")
    cpu = lambda t: t.detach().to("cpu", torch.float32).clone()
    state = (int(i), int(ds_train_rows_read), _map_tree(params, cpu), [_map_tree(m, cpu), _map_tree(v, cpu)])
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        pickle.dump(state, f)
    os.replace(tmp, path)


def load_checkpoint(path: str, device="cpu") -> Tuple[int, int, list, list]:
    """``(i, ds_train_rows_read, params, moments)`` with every tensor on ``device``; accepts files written by the
    reference as well (tuple of four, moments a pair of pytrees)."""
    with open(path, "rb") as f:
        state = pickle.load(f)
    if not isinstance(state, (tuple, list)) or len(state) != 4:
        raise ValueError("not a (i, ds_train_rows_read, params, moments) checkpoint")
    i, rows, params, moments = state
    if len(moments) != 2:
        raise ValueError("moments must be the pair [m, v]")
    check_same_structure(params, moments[0], "first moments")
    check_same_structure(params, moments[1], "second moments")
    dev = lambda t: t.to(device)
    return int(i), int(rows), _map_tree(params, dev), [_map_tree(moments[0], dev), _map_tree(moments[1], dev)]


def trainer_state(trainer):
    """(params, [m, v]) pytrees (views of the trainer's flat float32 buffers, no copy)."""
    cfg, lay = trainer.cfg, trainer.layout
    tree = lambda flat: unflatten_like([lay.view(flat, n) for n, _ in cfg.param_shapes()], cfg)
    return tree(trainer.p), [tree(trainer.m), tree(trainer.v)]


def save_trainer(path: str, trainer, ds_train_rows_read: int = 0) -> None:
    """The trainer has completed ``trainer.t`` micro-steps; like the reference, which counts the step before it
    pickles (train_gpt2_triton.py:408-419), the file stores ``i = trainer.t``."""
    params, moments = trainer_state(trainer)
    save_checkpoint(path, trainer.t, ds_train_rows_read, params, moments)


def checkpoint_name(run_dir: str, trainer) -> str:
    """The reference's file name for a checkpoint taken now: ``runs/<run>/checkpoint_<i>.pkl`` with the completed
    step count (train_gpt2_triton.py:415)."""
    return os.path.join(run_dir, f"checkpoint_{trainer.t}.pkl")


def load_trainer_state(trainer, path: str) -> Tuple[int, int]:
    """Copies a checkpoint's parameters and moments into the trainer's flat buffers, refreshes the bf16 weight shadow
    and sets the step counter to the ``i`` completed steps, so that the next update runs AdamW with step count
    ``i + 1`` and draws the dropout seeds of step index ``i``. Returns ``(i, ds_train_rows_read)``."""
    i, rows, params, moments = load_checkpoint(path, trainer.device)
    cur, (m, v) = trainer_state(trainer)
    check_same_structure(cur, params, "parameters")
    for dst_tree, src_tree in ((cur, params), (m, moments[0]), (v, moments[1])):
        for gd, gs in zip(dst_tree, src_tree):
            for d, s in zip(gd, gs):
                d.copy_(s.to(torch.float32))
    trainer.t = i
    trainer._refresh_shadow()
    return i, rows
