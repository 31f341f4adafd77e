"""B200 (sm_100a) implementation of pre-tjax's GPT-2 training hot path.

The directory name contains a hyphen, so import it with ``importlib.import_module("pre-tjax_b200")`` (the repository
root must be on ``sys.path``). Sub-modules:

* ``operators``  – the reference's launcher surface (``t_layernorm_fwd_t``, ``t_scaled_dot_prod_attn_fwd3_t`` …)
* ``gpt2``       – forward / hand-written backward composition (``t_loss_bkwd3_t`` …)
* ``optimizer``  – ``adam_w_in_place``, ``init_adam_w``, ``grads_l2norm``, parameter initialisation
* ``trainer``    – flat-buffer, data-parallel training step
* ``evaluate``   – ``loss_eval``, ``log_probs``, ``predict`` (eval-mode callers of the same kernels)
* ``build``      – compiles ``csrc/*.cu`` into ``libptj_b200.so``

Everything computes on the GPU through the C ABI in ``include/ptj_b200.h``; there is no CPU fallback.
"""
from . import _lib, evaluate, gpt2, operators, optimizer, trainer  # noqa: F401
from .gpt2 import GPT2Config, PRESETS, t_gpt2_bkwd3_p_t, t_gpt2_forward_with_acts_t, t_loss_bkwd3_t  # noqa: F401
from .optimizer import adam_w_in_place, grads_l2norm, init_adam_w, init_transformer_gpt2  # noqa: F401
from .trainer import TrainConfig, Trainer  # noqa: F401

__all__ = ["operators", "gpt2", "optimizer", "trainer", "GPT2Config", "PRESETS", "Trainer", "TrainConfig",
           "t_loss_bkwd3_t", "t_gpt2_forward_with_acts_t", "t_gpt2_bkwd3_p_t", "adam_w_in_place", "init_adam_w",
           "grads_l2norm", "init_transformer_gpt2"]
