"""GPT-2 forward + hand-written backward on the sm_100a kernels.

Mirrors the composition functions of the reference's Triton path — ``t_gpt2_forward_with_acts_t``
(model_triton.py:2535-2539), ``t_gpt2_bkwd3_p_t`` (:2583-2593) and ``t_loss_bkwd3_t``
(loss_and_optimizer_triton.py:279-289) — with the same parameter pytree (model_torch_func.py:36-43):

    [[W_emb(V,D), b_head(V)], [W_pos(S,D)],
     L x [g1, b1, W_qkv(H,3,dh,D), W_o(D,D), g2, b2, W1(F,D), b1f(F), W2(D,F), b2f(D)],
     [g_f, b_f]]

Differences in HOW (not in what is computed): the three head projections are ONE GEMM whose output columns are
ordered (head, q/k/v, d_head) so W_qkv keeps the reference layout; attention reads/writes strided views (no stack,
transpose or concat copies); bias, GELU, dropout and the residual add run in GEMM epilogues; the causal mask is
analytic; QKV and the FFN pre-activation are saved instead of recomputed in backward; the cross entropy overwrites
the logits with their gradient; nothing uses atomics, so results are bit-reproducible.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from . import _lib, operators as ops

LAYER_TENSORS = ("g1", "b1", "w_qkv", "w_o", "g2", "b2", "w1", "b1f", "w2", "b2f")
# which tensors take part in the tensor-core GEMMs and therefore live in the compute dtype
MATRIX_TENSORS = {"w_emb", "w_pos", "w_qkv", "w_o", "w1", "w2"}


@dataclass(frozen=True)
class GPT2Config:
    vocab: int
    dim: int
    layers: int
    heads: int
    ffn: int
    seq: int
    dropout: float = 0.1

    @property
    def d_head(self) -> int:
        return self.dim // self.heads

    def param_shapes(self):
        """[(name, shape)] in the order of the flattened reference pytree."""
        V, D, H, F, S = self.vocab, self.dim, self.heads, self.ffn, self.seq
        out = [("w_emb", (V, D)), ("b_head", (V,)), ("w_pos", (S, D))]
        for l in range(self.layers):
            out += [(f"l{l}.g1", (D,)), (f"l{l}.b1", (D,)), (f"l{l}.w_qkv", (H, 3, D // H, D)), (f"l{l}.w_o", (D, D)),
                    (f"l{l}.g2", (D,)), (f"l{l}.b2", (D,)), (f"l{l}.w1", (F, D)), (f"l{l}.b1f", (F,)),
                    (f"l{l}.w2", (D, F)), (f"l{l}.b2f", (D,))]
        out += [("g_f", (D,)), ("b_f", (D,))]
        return out

    def num_params(self) -> int:
        return sum(math.prod(s) for _, s in self.param_shapes())


PRESETS = {
    "tiny": GPT2Config(vocab=1024, dim=128, layers=2, heads=4, ffn=512, seq=128, dropout=0.0),
    "gpt2-small": GPT2Config(vocab=50257, dim=768, layers=12, heads=12, ffn=3072, seq=1024, dropout=0.1),
    "gpt2-medium": GPT2Config(vocab=50257, dim=1024, layers=24, heads=16, ffn=4096, seq=1024, dropout=0.1),
}


def base_name(name: str) -> str:
    return name.split(".")[-1]


def is_decayed(name: str) -> bool:
    """Weight-decay rule of the reference (train_gpt2_triton.py:69-71): everything except 1-D tensors that start as
    zeros, i.e. biases and LayerNorm shifts are exempt while LayerNorm scales (initialised to one) are decayed."""
    return base_name(name) not in ("b_head", "b1", "b2", "b1f", "b2f", "b_f")


def flatten_pytree(tree) -> List[torch.Tensor]:
    return [t for grp in tree for t in grp]


def unflatten_like(flat: Sequence[torch.Tensor], cfg: GPT2Config):
    """Regroup a flat list into the reference's [[2], [1], L x [10], [2]] nesting."""
    it = iter(flat)
    tree = [[next(it), next(it)], [next(it)]]
    for _ in range(cfg.layers):
        tree.append([next(it) for _ in range(10)])
    tree.append([next(it), next(it)])
    return tree


def config_from_params(params, dropout: float) -> GPT2Config:
    V, D = params[0][0].shape
    S = params[1][0].shape[0]
    L = len(params) - 3
    H = params[2][2].shape[0]
    F = params[2][6].shape[0]
    return GPT2Config(vocab=V, dim=D, layers=L, heads=H, ffn=F, seq=S, dropout=dropout)


class Weights:
    """Named views of the parameters: matrices in the compute dtype, vectors (LayerNorm, biases) in float32."""

    def __init__(self, cfg: GPT2Config, tensors: dict):
        self.cfg = cfg
        self.t = tensors

    def __getitem__(self, name):
        return self.t[name]

    @staticmethod
    def from_pytree(params, cfg: GPT2Config, compute_dtype: torch.dtype) -> "Weights":
        flat = flatten_pytree(params)
        names = [n for n, _ in cfg.param_shapes()]
        assert len(flat) == len(names), "parameter pytree does not match the configuration"
        t = {}
        for n, p in zip(names, flat):
            if not p.is_cuda:
                raise RuntimeError("parameters must live on a CUDA device: there is no CPU implementation")
            want = compute_dtype if base_name(n) in MATRIX_TENSORS else torch.float32
            p = p.contiguous()
            t[n] = p if p.dtype == want else p.to(want)
        return Weights(cfg, t)


def split_k_for(M: int, N: int, K: int) -> int:
    """K split of a weight-gradient GEMM (long K, small output): the number of equal parts of K that, dealt to the 74
    thread-block pairs of the 256 x 256-tile kernel, finishes first. Cost of S parts = rounds needed for tiles * S work
    items, each 1/S long, plus a charge per part for writing and re-reading its float32 partial output (measured on
    the GPT-2 small shapes at K = 8192: about 1.7 us per part of a 9.4 MB output against 55 us for a full-K tile; the
    sweep's optimum is 2 parts for the 3072 x 768 FFN matrices, 5 for the QKV matrix, 8 for 768 x 768)."""
    tiles = max(1, -(-M // 256) * -(-N // 256))
    k_blocks = max(1, K // 64)
    per_part = 0.0032 * (M * N * 4e-6) * (8192.0 / max(K, 1))
    best, best_cost = 1, float("inf")
    for s in range(1, 9):
        if s > max(1, k_blocks // 4):
            break
        cost = -(-tiles * s // 74) / s + per_part * s
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def tail_split_for(M: int, N: int, K: int):
    """(first row of the range that is split over K, floats of workspace) when ptj_gemm's PTJ_SPLIT_TAIL changes how a
    bf16 product of this shape runs (its last round of 256 x 256 tiles would leave most thread-block pairs idle: 96
    tiles on 74 pairs), else None."""
    lib = _lib.lib()
    n = lib.ptj_gemm_tail_split_floats(M, N, K)
    return (int(lib.ptj_gemm_tail_split_rows(M, N, K)), int(n)) if n else None


class Gpt2Step:
    """One forward + backward pass. Gradients are written into caller-provided float32 tensors (``grads[name]``),
    so a trainer can hand in views of one flat buffer and overlap their reduction with the rest of backward."""

    def __init__(self, cfg: GPT2Config, compute_dtype: torch.dtype = torch.bfloat16):
        self.cfg = cfg
        self.dtype = compute_dtype
        # logits rows are padded so that every row starts on a 16-byte boundary
        self.vocab_ld = (cfg.vocab + 127) // 128 * 128
        self._ws = None
        # FFN backward: gelu' inside the input-gradient GEMM's epilogue followed by a column-sum pass over its output
        # (measured 0.1 ms per GPT-2 small step faster), or, when set, a plain GEMM followed by ONE elementwise pass
        # that applies gelu' and sums the columns. Same results.
        self.split_gelu_bwd = False
        # the two FFN weight gradients of a layer in one launch, and the QKV + out-projection pair in another
        self.pair_wgrads = True
        # input gradients whose last round of tiles is mostly empty: that round's rows split over K, same launch
        self.tail_split = True
        self._ws2 = [None, None]

    # -- helpers --
    def _wgrad(self, dy2d, x2d, out, accumulate=False):
        """out[N_out, N_in] = dy^T x : both operands are read 'MN-major' (tokens are the reduction dimension)."""
        T = dy2d.shape[0]
        M, N = out.shape[0], x2d.shape[1]
        split = 1
        if dy2d.dtype == torch.bfloat16:
            split = split_k_for(M, N, T)
            need = split * M * N
            if split > 1 and (self._ws is None or self._ws.numel() < need):
                self._ws = torch.empty(need, device=out.device, dtype=torch.float32)
        ops.gemm(dy2d, x2d, a_kmajor=False, b_kmajor=False, M=M, N=N, K=T, lda=dy2d.stride(0), ldb=x2d.stride(0),
                 out=out.view(M, N), epilogue=_lib.EPI_ACCUM if accumulate else _lib.EPI_NONE, split_k=split,
                 workspace=self._ws)

    def _workspace(self, floats: int):
        if self._ws is None or self._ws.numel() < floats:
            self._ws = torch.empty(floats, device="cuda", dtype=torch.float32)
        return self._ws

    def _wgrad2(self, first, second):
        """Two weight gradients (dy, x, out) in ONE launch of the thread-block-pair kernel when both qualify: their
        tiles share the 74 pairs, so the two FFN matrices (36 tiles each at GPT-2 small) need no K split and no reduce
        launch, and the QKV + out-projection pair (27 + 9 tiles) is split in two parts instead of five and eight.
        Falls back to two launches."""
        (dy0, x0, out0), (dy1, x1, out1) = first, second
        T = dy0.shape[0]
        ok = dy0.dtype == torch.bfloat16 and dy1.shape[0] == T and self.pair_wgrads
        if ok:
            tiles = sum(-(-o.shape[0] // 256) * -(-x.shape[1] // 256) for o, x in ((out0, x0), (out1, x1)))
            out_mb = max(out0.shape[0] * x0.shape[1], out1.shape[0] * x1.shape[1]) * 4e-6
            k_blocks = max(1, T // 64)
            best, best_cost = 1, float("inf")
            for s_ in range(1, 9):  # the cost model of split_k_for, on the tiles of both products
                if s_ > max(1, k_blocks // 4):
                    break
                cost = -(-tiles * s_ // 74) / s_ + 0.0032 * out_mb * (8192.0 / max(T, 1)) * s_ * (s_ > 1)
                if cost < best_cost - 1e-9:
                    best, best_cost = s_, cost
            probs = []
            for i, (dy, x, out) in enumerate(((dy0, x0, out0), (dy1, x1, out1))):
                M, N = out.shape[0], x.shape[1]
                ws = None
                if best > 1:
                    ws = self._ws2[i]
                    if ws is None or ws.numel() < best * M * N:
                        ws = self._ws2[i] = torch.empty(best * M * N, device=out.device, dtype=torch.float32)
                probs.append(dict(a=dy, b=x, out=out.view(M, N), lda=dy.stride(0), ldb=x.stride(0), split_k=best,
                                  workspace=ws))
            ok = ops.gemm_grouped2(probs, T, a_kmajor=False, b_kmajor=False)
        if not ok:
            self._wgrad(dy0, x0, out0)
            self._wgrad(dy1, x1, out1)

    def _dgrad(self, dy2d, w2d, cols=None, **kw):
        """dx[T, N_in] = dy[T, N_out] w[N_out, N_in]: w is the 'MN-major' B operand."""
        T = dy2d.shape[0]
        K = w2d.shape[0] if cols is None else cols
        N = w2d.shape[1]
        # A very long K with a narrow output (the LM head: K = vocabulary, N = model width) leaves the 74 thread-block
        # pairs a bad last round (96 tiles of 256 x 256 at GPT-2 small); parts of K even it out. Measured at
        # [8192, 768, 50257]: 543 us unsplit, 478 / 467 / 496 us in 2 / 3 / 4 parts; the K = 2304 and 3072 products of a
        # layer only lose (32 -> 40 us, 48 -> 56 us), hence the lower bound on K.
        split = 1
        if dy2d.dtype == torch.bfloat16 and not kw:
            tail = tail_split_for(T, N, K) if self.tail_split else None
            if tail is not None:
                split = ops.SPLIT_TAIL  # the rows of the last, mostly empty round of tiles are split over K
                self._workspace(tail[1])
            elif K >= 16384:
                split = split_k_for(T, N, K)
                self._workspace(split * T * N)
        return ops.gemm(dy2d, w2d, a_kmajor=True, b_kmajor=False, M=T, N=N, K=K, lda=dy2d.stride(0),
                        ldb=w2d.stride(0), out_dtype=self.dtype, split_k=split, workspace=self._ws, **kw)

    # -- forward --
    def forward(self, w: Weights, ids_in: torch.Tensor, train: bool, seeds: Sequence[int], row_kstart=None):
        """Returns (logits [B*S, vocab_ld] (first `vocab` columns valid), saved activations).
        row_kstart: optional int32 [B, S], first key each position attends to (packed documents / padding, see
        operators.row_kstart_from_mask); None = plain causal attention."""
        cfg, p = self.cfg, self.cfg.dropout
        B, S = ids_in.shape
        assert S == cfg.seq, "the positional table is added without slicing: sequence length must equal cfg.seq"
        D, H, dh, T = cfg.dim, cfg.heads, cfg.d_head, B * S
        if not train:
            seeds = [0] * (1 + 3 * cfg.layers)
        x = ops.embed_fwd(ids_in, w["w_emb"], w["w_pos"], train, seeds[0], out_dtype=self.dtype, p=p).view(T, D)
        acts = {"layers": [], "row_kstart": row_kstart}
        for l in range(cfg.layers):
            s_attn, s_res1, s_res2 = seeds[1 + 3 * l: 4 + 3 * l]
            g = lambda n: w[f"l{l}.{n}"]
            a = {"x": x}
            a["ln1"] = ops.t_layernorm_fwd_t((g("g1"), g("b1")), x)
            a["qkv"] = ops.gemm(a["ln1"], g("w_qkv").view(3 * D, D))  # columns ordered (head, q/k/v, d_head)
            qkv5 = a["qkv"].view(B, S, H, 3, dh)
            q, k, v = (qkv5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
            a["attn"] = torch.empty((T, D), device=x.device, dtype=self.dtype)
            o4 = a["attn"].view(B, S, H, dh).permute(0, 2, 1, 3)
            # the layer's attention-dropout keep flags are drawn once and shared by the forward and backward kernels
            a["keep"] = ops.attn_keep_bits(q, k, v, o4, s_attn, p=p) if (train and p > 0.0) else None
            a["m"], a["l"] = ops.attn_fwd(q, k, v, o4, train, s_attn, p=p, keep_bits=a["keep"], row_kstart=row_kstart)
            a["x_mid"] = ops.gemm(a["attn"], g("w_o"), epilogue=_lib.EPI_DROPOUT_RESID, aux=x,
                                  dropout_args=(p, train, s_res1, 0))
            a["ln2"] = ops.t_layernorm_fwd_t((g("g2"), g("b2")), a["x_mid"])
            a["h_pre"] = torch.empty((T, cfg.ffn), device=x.device, dtype=self.dtype)
            a["h_act"] = ops.gemm(a["ln2"], g("w1"), bias=g("b1f"), epilogue=_lib.EPI_GELU, aux_out=a["h_pre"])
            tail = tail_split_for(T, D, cfg.ffn) if (self.tail_split and self.dtype == torch.bfloat16) else None
            x = ops.gemm(a["h_act"], g("w2"), bias=g("b2f"), epilogue=_lib.EPI_DROPOUT_RESID, aux=a["x_mid"],
                         dropout_args=(p, train, s_res2, 0), split_k=ops.SPLIT_TAIL if tail else 1,
                         workspace=self._workspace(tail[1]) if tail else None)
            acts["layers"].append(a)
        acts["x_last"] = x
        acts["x_f"] = ops.t_layernorm_fwd_t((w["g_f"], w["b_f"]), x)
        logits = torch.empty((T, self.vocab_ld), device=x.device, dtype=self.dtype)
        ops.gemm(acts["x_f"], w["w_emb"], bias=w["b_head"], out=logits, N=cfg.vocab, ldc=self.vocab_ld)
        return logits, acts

    # -- backward --
    def backward(self, w: Weights, grads: dict, dlogits: torch.Tensor, acts: dict, ids_in: torch.Tensor, train: bool,
                 seeds: Sequence[int], on_ready: Optional[Callable[[List[str]], None]] = None):
        """dlogits: [B*S, vocab_ld]. Fills grads[name] (float32) for every parameter; calls on_ready(names) as soon as
        the kernels producing those gradients have been enqueued."""
        cfg, p = self.cfg, self.cfg.dropout
        B, S = ids_in.shape
        D, H, dh, T, F, V = cfg.dim, cfg.heads, cfg.d_head, B * S, cfg.ffn, cfg.vocab
        if not train:
            seeds = [0] * (1 + 3 * cfg.layers)
        ready = on_ready or (lambda names: None)

        # LM head (tied to the embedding): bias, weight (the embedding scatter is added at the very end), input
        ops.colsum(dlogits, cols=V, out=grads["b_head"])
        self._head_wgrad(dlogits, acts["x_f"], grads["w_emb"])
        ready(["b_head"])
        d = self._dgrad(dlogits, w["w_emb"], cols=V)
        # every LayerNorm backward also writes dropout(dx) for the residual branch that consumes it next
        fuse = D % 8 == 0 and D <= (2048 if self.dtype == torch.bfloat16 else 1024)
        s_next = seeds[3 * cfg.layers] if cfg.layers > 0 else 0  # last layer's second residual dropout
        # ... and its column sums, which are the bias gradient of that branch's last linear layer (FFN-2)
        dx, dy = self._ln_bwd(d, w["g_f"], acts["x_last"], grads["g_f"], grads["b_f"],
                              dropped=(train, s_next, p) if (fuse and cfg.layers > 0) else None,
                              colsum_out=grads[f"l{cfg.layers - 1}.b2f"] if (fuse and cfg.layers > 0) else None)
        ready(["g_f", "b_f"])

        for l in reversed(range(cfg.layers)):
            s_attn, s_res1, s_res2 = seeds[1 + 3 * l: 4 + 3 * l]
            a = acts["layers"][l]
            g = lambda n: w[f"l{l}.{n}"]
            G = lambda n: grads[f"l{l}.{n}"]
            # x_next = x_mid + dropout(W2 gelu(W1 ln2(x_mid) + b1f) + b2f)
            if dy is None:
                dy = ops.dropout(dx, train, s_res2, p=p)
                ops.colsum(dy, out=G("b2f"))
            dy_ffn = dy
            if self.split_gelu_bwd and F % 8 == 0 and F <= 8192:
                # plain product, then one elementwise pass that applies gelu' in place and sums the columns (b1f)
                dh_pre, _ = ops.gelu_bwd_colsum(self._dgrad(dy, g("w2")), a["h_pre"], colsum_out=G("b1f"), in_place=True)
            else:
                dh_pre = self._dgrad(dy, g("w2"), epilogue=_lib.EPI_GELU_BWD, aux=a["h_pre"])
                ops.colsum(dh_pre, out=G("b1f"))
            self._wgrad2((dy_ffn, a["h_act"], G("w2")), (dh_pre, a["ln2"], G("w1")))
            d_ln2 = self._dgrad(dh_pre, g("w1"))
            dx, dy = self._ln_bwd(d_ln2, g("g2"), a["x_mid"], G("g2"), G("b2"), dx_add=dx,
                                  dropped=(train, s_res1, p) if fuse else None)
            ready([f"l{l}.{n}" for n in ("b2f", "w2", "b1f", "w1", "g2", "b2")])
            # x_mid = x + dropout(attn(ln1(x)) W_o^T)
            if dy is None:
                dy = ops.dropout(dx, train, s_res1, p=p)
            dy_attn = dy
            d_attn = self._dgrad(dy, g("w_o"))
            dqkv = torch.empty((T, 3 * D), device=dy.device, dtype=self.dtype)
            qkv5, dqkv5 = a["qkv"].view(B, S, H, 3, dh), dqkv.view(B, S, H, 3, dh)
            q, k, v = (qkv5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
            dq, dk, dv = (dqkv5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
            o4 = a["attn"].view(B, S, H, dh).permute(0, 2, 1, 3)
            do4 = d_attn.view(B, S, H, dh).permute(0, 2, 1, 3)
            ops.attn_bwd(do4, q, k, v, o4, a["m"], a["l"], dq, dk, dv, train, s_attn, p=p, keep_bits=a.get("keep"),
                         row_kstart=acts.get("row_kstart"))
            self._wgrad2((dqkv, a["ln1"], G("w_qkv").view(3 * D, D)), (dy_attn, a["attn"], G("w_o")))
            d_ln1 = self._dgrad(dqkv, g("w_qkv").view(3 * D, D))
            s_prev = seeds[3 * l] if l > 0 else 0  # the layer below's second residual dropout consumes this dx
            dx, dy = self._ln_bwd(d_ln1, g("g1"), a["x"], G("g1"), G("b1"), dx_add=dx,
                                  dropped=(train, s_prev, p) if (fuse and l > 0) else None,
                                  colsum_out=grads[f"l{l - 1}.b2f"] if (fuse and l > 0) else None)
            ready([f"l{l}.{n}" for n in ("w_o", "w_qkv", "g1", "b1")])

        # embedding + positions; the scatter accumulates onto the LM-head weight gradient (tied weights)
        ops.embed_bwd(dx, ids_in, grads["w_emb"], grads["w_pos"], accumulate=True, train=train, seed=seeds[0], p=p,
                      sorted_pos=acts.get("sorted_pos"))
        ready(["w_emb", "w_pos"])

    def _head_wgrad(self, dlogits, x_f, out):
        V = self.cfg.vocab
        T = dlogits.shape[0]
        ops.gemm(dlogits, x_f, a_kmajor=False, b_kmajor=False, M=V, N=x_f.shape[1], K=T, lda=dlogits.stride(0),
                 ldb=x_f.stride(0), out=out)

    def _ln_bwd(self, dy, gamma, x, dgamma_out, dbeta_out, dx_add=None, dropped=None, colsum_out=None):
        """Returns (dx, dropout(dx) or None); colsum_out receives the column sums of dropout(dx)."""
        res = ops.layernorm_bwd(dy, (gamma, None), x, want_dx=True, want_dp=True, dx_add=dx_add,
                                dgamma_out=dgamma_out, dbeta_out=dbeta_out, dropped=dropped,
                                dropped_colsum_out=colsum_out if dropped is not None else None)
        return res[0], (res[3] if dropped is not None else None)

    # -- loss + gradients --
    def loss_and_grads(self, w: Weights, grads: dict, y: torch.Tensor, train: bool, seeds: Sequence[int],
                       n_valid: Optional[torch.Tensor] = None, on_ready=None, sorted_pos=None, row_kstart=None):
        """y: [B, S+1] token ids; inputs y[:, :-1], labels y[:, 1:] (loss_and_optimizer_triton.py:280-281).
        Returns float32[3] = (mean loss over labels != 0, accuracy, fraction of labels != 0)."""
        ids_in = y[:, :-1].contiguous().to(torch.int32)
        labels = y[:, 1:].contiguous().to(torch.int32)
        logits, acts = self.forward(w, ids_in, train, seeds, row_kstart=row_kstart)
        if sorted_pos is not None:
            acts["sorted_pos"] = sorted_pos
        stats, _, dlogits = ops.cross_entropy(labels, logits, cols=self.cfg.vocab, want_grad=True, in_place=True,
                                              n_valid=n_valid)
        self.backward(w, grads, dlogits, acts, ids_in, train, seeds, on_ready)
        return stats


# ---- reference-shaped entry points ------------------------------------------------------------------------------------
def _seeds_or_zero(p_gen_aux, cfg):
    return list(p_gen_aux) if p_gen_aux is not None else [0] * (1 + 3 * cfg.layers)


def t_gpt2_forward_with_acts_t(params, y, y_mask=None, y_indices=None, train=True, p_gen_aux=None):
    """(logits [B,S,V], acts) (model_triton.py:2535-2539). y_mask [B,S,S] bool is the reference collator's mask
    (causal, optionally x block-diagonal over packed documents x padding; None = causal); y_indices are ignored, as in
    both of the reference's paths (the position table is added whole, :2339). The activations object is opaque: pass
    it to t_gpt2_bkwd3_p_t."""
    cfg = config_from_params(params, ops.DROPOUT_RATE)
    step = Gpt2Step(cfg, params[0][0].dtype)
    w = Weights.from_pytree(params, cfg, step.dtype)
    ids = y.to(torch.int32).contiguous()
    logits, acts = step.forward(w, ids, train, _seeds_or_zero(p_gen_aux, cfg), row_kstart=ops._kstart_or_none(y_mask))
    B, S = ids.shape
    acts["_step"], acts["_w"], acts["_logits_padded"] = step, w, logits
    return logits.view(B, S, -1)[:, :, :cfg.vocab], acts


def t_gpt2_bkwd3_p_t(dloss_dx, acts, params, y, y_mask=None, y_indices=None, train=True, p_gen_aux=None):
    """Gradient pytree from dloss/dlogits [B,S,V] (model_triton.py:2583-2593)."""
    step, w = acts["_step"], acts["_w"]
    cfg = step.cfg
    ids = y.to(torch.int32).contiguous()
    T = ids.numel()
    d = torch.zeros((T, step.vocab_ld), device=dloss_dx.device, dtype=step.dtype)
    d[:, :cfg.vocab] = dloss_dx.reshape(T, cfg.vocab)
    grads = {n: torch.empty(s, device=d.device, dtype=torch.float32) for n, s in cfg.param_shapes()}
    step.backward(w, grads, d, acts, ids, train, _seeds_or_zero(p_gen_aux, cfg))
    return unflatten_like([grads[n] for n, _ in cfg.param_shapes()], cfg)


def t_loss_bkwd3_t(params, y, y_mask=None, y_indices=None, train=True, p_gen_aux=None):
    """(grads pytree, (loss, accuracy, valid fraction)) for y[B, S+1] (loss_and_optimizer_triton.py:279-289)."""
    cfg = config_from_params(params, ops.DROPOUT_RATE)
    step = Gpt2Step(cfg, params[0][0].dtype)
    w = Weights.from_pytree(params, cfg, step.dtype)
    grads = {n: torch.empty(s, device=y.device, dtype=torch.float32) for n, s in cfg.param_shapes()}
    stats = step.loss_and_grads(w, grads, y, train, _seeds_or_zero(p_gen_aux, cfg),
                                row_kstart=ops._kstart_or_none(y_mask))
    return unflatten_like([grads[n] for n, _ in cfg.param_shapes()], cfg), (stats[0], stats[1], stats[2])
