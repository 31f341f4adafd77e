"""Data-parallel GPT-2 training step on flat buffers.

The reference trains on one GPU with gradient accumulation (train_gpt2_triton.py:261, 298-321); here every rank owns
one GPU and one micro-batch, and the only collective is a sum-allreduce of the gradients:

* parameters, gradients and both Adam moments live in four flat float32 buffers with identical layout, plus a bf16
  shadow of the parameters that the tensor-core GEMMs read;
* tensors are laid out in the order in which backward produces their gradients, so a bucket is a contiguous slice
  that the GEMM epilogues write directly (no pack / unpack copies) and that the fused AdamW reads directly;
* as soon as every gradient of a bucket has been enqueued, the bucket is all-reduced on a side stream while the
  compute stream carries on with the rest of backward;
* clipping uses the norm of the reduced buffer, so it is identical on every rank without another collective.

Loss normalisation under data parallelism: each rank divides by its OWN number of non-padding labels and the ranks'
gradients are averaged — the same "mean of per-micro-batch means" the reference's accumulation loop computes
(train_gpt2_triton.py:315-318). With ``global_token_norm=True`` the label count is all-reduced first and the result
equals the single-process gradient of the concatenated batch exactly.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .gpt2 import GPT2Config, Gpt2Step, MATRIX_TENSORS, Weights, base_name, is_decayed, unflatten_like

ALIGN = 64  # elements; every tensor starts on a 256-byte boundary of the flat buffers


def backward_order(cfg: GPT2Config) -> List[str]:
    """Parameter names in the order their gradients become final during backward."""
    names = ["b_head", "g_f", "b_f"]
    for l in reversed(range(cfg.layers)):
        names += [f"l{l}.{n}" for n in ("b2f", "w2", "b1f", "w1", "g2", "b2", "w_o", "w_qkv", "g1", "b1")]
    names += ["w_emb", "w_pos"]
    return names


@dataclass
class FlatLayout:
    """Offsets of every parameter inside the flat buffers."""
    names: List[str]
    shapes: Dict[str, Tuple[int, ...]]
    offsets: Dict[str, int]
    total: int

    @staticmethod
    def build(cfg: GPT2Config) -> "FlatLayout":
        shapes = dict(cfg.param_shapes())
        offsets, off = {}, 0
        names = backward_order(cfg)
        assert sorted(names) == sorted(shapes), "layout must cover every parameter exactly once"
        for n in names:
            offsets[n] = off
            off += (math.prod(shapes[n]) + ALIGN - 1) // ALIGN * ALIGN
        return FlatLayout(names, shapes, offsets, off)

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        n = math.prod(self.shapes[name])
        o = self.offsets[name]
        return flat[o:o + n].view(self.shapes[name])

    def views(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: self.view(flat, n) for n in self.names}

    def decay_segments(self) -> Tuple[List[int], List[int]]:
        """(segment starts incl. final end, decay flag per segment), consecutive equal flags merged."""
        starts, flags = [], []
        for n in self.names:
            f = 1 if is_decayed(n) else 0
            if not flags or flags[-1] != f:
                starts.append(self.offsets[n])
                flags.append(f)
        starts.append(self.total)
        return starts, flags


@dataclass
class Bucket:
    start: int
    end: int
    names: List[str]
    pending: int = 0
    work: object = None
    event: object = None


def make_buckets(layout: FlatLayout, bucket_elems: int) -> List[Bucket]:
    """Cut the flat gradient buffer into contiguous buckets at tensor boundaries, in backward order."""
    buckets, cur = [], None
    for n in layout.names:
        size = (math.prod(layout.shapes[n]) + ALIGN - 1) // ALIGN * ALIGN
        o = layout.offsets[n]
        if cur is None or (cur.end - cur.start) + size > bucket_elems and cur.names:
            cur = Bucket(o, o, [])
            buckets.append(cur)
        cur.names.append(n)
        cur.end = o + size
    return buckets


class PeerLost(RuntimeError):
    """A rank of the data-parallel group stopped reporting, or a collective did not finish within its time limit."""


class PeerWatch:
    """Host-side failure detection for the data-parallel group, through the process group's key-value store.

    Every rank publishes the index of the step it is about to run; before launching the step's first collective a
    rank checks that every peer has published that index too, waiting at most ``timeout_s``. A rank that raised,
    exited or never joined is therefore noticed on the host, between steps, with nothing in flight on the GPU: the
    survivors get a PeerLost instead of a collective that never returns. (The reference is a single process and has
    nothing of the kind; a crash there loses everything since the last pickle.)"""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "ptj/step"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def announce(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}/{step}", b"1")

    def check(self, step: int):
        import datetime
        keys = [f"{self.prefix}/{r}/{step}" for r in range(self.world) if r != self.rank]
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as e:  # the store raises its own timeout type
            missing = []
            for r, k in zip([r for r in range(self.world) if r != self.rank], keys):
                try:
                    self.store.wait([k], datetime.timedelta(milliseconds=1))
                except Exception:
                    missing.append(r)
            raise PeerLost(f"rank(s) {missing or '?'} did not reach step {step} within {self.timeout_s:.1f} s: "
                           f"not launching this step's collectives") from e
        if step >= 2:  # keep the store small
            try:
                self.store.delete_key(f"{self.prefix}/{self.rank}/{step - 2}")
            except Exception:
                pass


class GradReducer:
    """Bucketed sum-allreduce of a flat gradient buffer, overlapped with backward. Works with NCCL on CUDA tensors
    (side stream + events) and with gloo on CPU tensors (synchronous), which is how the host logic is tested."""

    def __init__(self, flat_grads: torch.Tensor, layout: FlatLayout, bucket_mb: float, group=None,
                 wait_timeout_s: Optional[float] = None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.flat = flat_grads
        self.buckets = make_buckets(layout, max(1, int(bucket_mb * (1 << 20) / 4)))
        self.owner = {n: i for i, b in enumerate(self.buckets) for n in b.names}
        self.cuda = flat_grads.is_cuda
        self.comm_stream = torch.cuda.Stream() if self.cuda else None
        self.launched: List[int] = []
        # host-side bound on waiting for a collective (None: the process group's own timeout is the only limit)
        self.wait_timeout_s = wait_timeout_s
        # (event before the wait, event after it) of recent steps, when exposure is being measured
        self.measure_exposed = False
        self.exposed_events: List[Tuple[object, object]] = []
        # when set, called with the bucket index instead of launching the all-reduce (graph recording, see Trainer)
        self.on_complete: Optional[Callable[[int], None]] = None
        self.reset()

    def reset(self):
        for b in self.buckets:
            b.pending = len(b.names)
            b.work = None
        self.launched = []

    def mark_ready(self, names: Sequence[str]):
        for n in names:
            b = self.buckets[self.owner[n]]
            b.pending -= 1
            if b.pending < 0:
                raise RuntimeError(f"gradient {n} reported ready twice in one step")
            if b.pending == 0:
                (self.on_complete or self._launch)(self.owner[n])

    def launch_bucket(self, idx: int):
        """All-reduce bucket idx now: its gradients are final as far as the current stream is concerned (used when the
        kernels come from recorded graph segments and nothing reports tensor by tensor)."""
        self.buckets[idx].pending = 0
        self._launch(idx)

    def _launch(self, idx: int):
        b = self.buckets[idx]
        view = self.flat[b.start:b.end]
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(ev)
            with torch.cuda.stream(self.comm_stream):
                b.work = self.dist.all_reduce(view, op=self.dist.ReduceOp.SUM, group=self.group, async_op=True)
        else:
            b.work = self.dist.all_reduce(view, op=self.dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.launched.append(idx)

    def finish(self):
        """Block the compute stream (not the host, on CUDA) until every bucket has been reduced."""
        missing = [b.names for b in self.buckets if b.pending != 0]
        if missing:
            raise RuntimeError(f"backward never produced the gradients of {missing[0]}: bucket cannot be reduced")
        ev0 = ev1 = None
        if self.cuda and self.measure_exposed and not torch.cuda.is_current_stream_capturing():
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        for idx in self.launched:
            w = self.buckets[idx].work
            if w is None:
                continue
            try:
                if self.cuda or self.wait_timeout_s is None:
                    w.wait()  # NCCL: makes the current stream wait for the collective; gloo: blocks the host
                else:
                    import datetime
                    if w.wait(datetime.timedelta(seconds=self.wait_timeout_s)) is False:
                        raise RuntimeError("timed out")
            except Exception as e:
                raise PeerLost(f"all-reduce of gradient bucket {idx} ({self.buckets[idx].names[0]} ...) failed: {e}") from e
            # (an asynchronous NCCL error - a peer died, a link fault - is raised by the process group's watchdog from
            # wait() or from the next call on the group, within the group's timeout; it lands in the except above)
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            if ev1 is not None:
                ev1.record()
                self.exposed_events.append((ev0, ev1))

    def exposed_ms(self) -> List[float]:
        """Per measured step, the time the compute stream spent waiting for gradient all-reduces that backward did not
        hide (synchronises the device; clears the record)."""
        torch.cuda.synchronize()
        out = [a.elapsed_time(b) for a, b in self.exposed_events]
        self.exposed_events = []
        return out


@dataclass
class TrainConfig:
    """Defaults are the reference train script's recipe (train_gpt2_triton.py:263-266, 305-310, 321): peak learning
    rate 2.5e-4, betas (0.9, 0.98), epsilon 1e-8, weight decay 0.01 and NO gradient clipping (the reference only logs
    the norm, :328), so a caller who takes the defaults trains with the dynamics of the run being replaced.
    ``benchmark_recipe`` gives the hyper-parameters of the throughput benchmark instead."""
    lr: float = 2.5e-4
    betas: Tuple[float, float] = (0.9, 0.98)
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip: Optional[float] = None
    bucket_mb: float = 48.0
    seed: int = 0
    global_token_norm: bool = False
    compute_dtype: torch.dtype = torch.bfloat16
    # Record forward + backward of a step once as a CUDA graph and replay it (plain causal batches): the host then
    # issues one graph launch instead of some 360 kernel launches per step. Dropout seeds live in device memory and are
    # rewritten before every replay, so the masks change from step to step exactly as without the graph.
    # With data parallelism the recording is cut into one graph per gradient bucket: the NCCL all-reduces are NOT
    # recorded (a recording that contained them left both ranks of a two-GPU run waiting on each other); they are
    # issued from the host between the graph launches, on their own stream, as in the unrecorded step.
    cuda_graph: bool = False

    @staticmethod
    def benchmark_recipe(**overrides) -> "TrainConfig":
        """AdamW lr 6e-4, betas (0.9, 0.95), weight decay 0.1, global-norm clip 1.0: the GPT-2 recipe the throughput
        benchmark is quoted on (not the reference's own, which has no clipping)."""
        kw = dict(lr=6e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip=1.0)
        kw.update(overrides)
        return TrainConfig(**kw)


def step_seeds(base_seed: int, step: int, rank: int, n: int) -> List[int]:
    """Dropout seeds of one step, derived on the host (the reference draws them on the GPU and reads them back with
    .item(), loss_and_optimizer_triton.py:319-325, which stalls the device every step). splitmix64 of
    (base, step, rank, site): distinct sites, steps and ranks get unrelated Philox keys."""
    out = []
    for site in range(n):
        z = (base_seed * 0x9E3779B97F4A7C15 + step * 0xBF58476D1CE4E5B9 + rank * 0x94D049BB133111EB + site + 1) & (2**64 - 1)
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2**64 - 1)
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2**64 - 1)
        out.append((z ^ (z >> 31)) & (2**63 - 1))  # 63 bits: bit 63 of a seed argument marks a device-resident seed
    return out


class Trainer:
    """fwd + bwd + gradient allreduce + clip + AdamW for one micro-batch per rank."""

    def __init__(self, cfg: GPT2Config, tc: TrainConfig = None, params=None, device="cuda", world: int = 1,
                 rank: int = 0, group=None, peer_watch: Optional[PeerWatch] = None):
        from .optimizer import init_from_config
        self.cfg, self.tc = cfg, tc or TrainConfig()
        self.world, self.rank = world, rank
        self.device = torch.device(device)
        self.layout = FlatLayout.build(cfg)
        n = self.layout.total
        z = lambda dt=torch.float32: torch.zeros(n, device=self.device, dtype=dt)
        self.p, self.g, self.m, self.v = z(), z(), z(), z()
        self.shadow = z(torch.bfloat16) if self.tc.compute_dtype == torch.bfloat16 else None
        if params is None:
            params = init_from_config(cfg, device="cpu", seed=self.tc.seed)
        flat_params = [t for grp in params for t in grp]
        for (name, _), t in zip(cfg.param_shapes(), flat_params):
            self.layout.view(self.p, name).copy_(t.to(self.device, torch.float32))
        self.pv, self.gv = self.layout.views(self.p), self.layout.views(self.g)
        self._refresh_shadow()
        starts, flags = self.layout.decay_segments()
        self.seg_start = torch.tensor(starts, device=self.device, dtype=torch.int64)
        self.seg_decay = torch.tensor(flags, device=self.device, dtype=torch.uint8)
        self.nseg = len(flags)
        self.engine = Gpt2Step(cfg, self.tc.compute_dtype)
        self.sumsq = torch.zeros(1, device=self.device, dtype=torch.float32)
        ns = _lib.lib().ptj_sumsq_scratch_floats(n)
        self.sumsq_scratch = torch.empty(ns, device=self.device, dtype=torch.float32)
        self.reducer = GradReducer(self.g, self.layout, self.tc.bucket_mb, group) if world > 1 else None
        self.peer_watch = peer_watch  # optional: checked on the host before each step's collectives
        self.t = 0
        self.ids_dev = None
        self.use_graph = (bool(self.tc.cuda_graph) and self.device.type == "cuda"
                          and not (world > 1 and self.tc.global_token_norm))
        self._graph = None           # (batch shape, [graph | bucket index, ...], static ids, static stats)
        self._seed_words = None      # int64[1 + 3 L] on the device: this step's dropout seeds, read by the kernels
        self._seed_host = None
        self.graph_launches = 0      # kernels recorded in the graph (one replay launches that many)
        self.graph_replays = 0

    # weights the kernels read: bf16 shadow for matrices, fp32 master for vectors
    def _refresh_shadow(self):
        if self.shadow is not None:
            _lib.check(_lib.lib().ptj_cast_f32_to_bf16(self.p.data_ptr(), self.shadow.data_ptr(), self.p.numel(),
                                                       torch.cuda.current_stream().cuda_stream), "ptj_cast_f32_to_bf16")
            sv = self.layout.views(self.shadow)
            self.w = Weights(self.cfg, {n: (sv[n] if base_name(n) in MATRIX_TENSORS else self.pv[n]) for n in self.layout.names})
        else:
            self.w = Weights(self.cfg, dict(self.pv))

    def params_pytree(self):
        return unflatten_like([self.pv[n] for n, _ in self.cfg.param_shapes()], self.cfg)

    def grads_pytree(self):
        return unflatten_like([self.gv[n] for n, _ in self.cfg.param_shapes()], self.cfg)

    def step(self, y: torch.Tensor, lr: Optional[float] = None, train: bool = True, row_kstart=None) -> torch.Tensor:
        """y: [B, S+1] int32 token ids (host, ideally pinned, or device). Returns float32[3] on the device:
        mean loss, accuracy, fraction of non-padding labels (of this rank's micro-batch).
        row_kstart: optional int32 [B, S] on the device for packed / padded batches (operators.row_kstart_from_lengths
        or row_kstart_from_mask): position i attends keys [row_kstart[b, i], i]; None = plain causal."""
        if self.use_graph and train and row_kstart is None and (self.world == 1 or self.t >= 2):
            return self._graph_step(y, lr)  # (data parallel: the first two steps run unrecorded and warm everything up)
        if not y.is_cuda:
            if self.ids_dev is None or self.ids_dev.shape != y.shape:
                self.ids_dev = torch.empty(y.shape, device=self.device, dtype=torch.int32)
            self.ids_dev.copy_(y, non_blocking=True)
            y = self.ids_dev
        seeds = step_seeds(self.tc.seed, self.t, self.rank, 1 + 3 * self.cfg.layers)
        sorted_pos = torch.sort(y[:, :-1].reshape(-1), stable=True).indices.to(torch.int32)
        n_valid = None
        if self.reducer is not None:
            if self.peer_watch is not None:  # every peer is alive and about to run this step: safe to communicate
                self.peer_watch.announce(self.t)
                self.peer_watch.check(self.t)
            self.reducer.reset()
            if self.tc.global_token_norm:
                lab = y[:, 1:]  # the kernel's predicate: not padding and inside the vocabulary
                n_valid = ((lab > 0) & (lab < self.cfg.vocab)).sum().to(torch.float32).reshape(1)
                self.reducer.dist.all_reduce(n_valid, group=self.reducer.group)
                n_valid = n_valid / self.world  # gradients are averaged over ranks afterwards
        on_ready = self.reducer.mark_ready if self.reducer is not None else None
        stats = self.engine.loss_and_grads(self.w, self.gv, y, train, seeds, n_valid=n_valid, on_ready=on_ready,
                                           sorted_pos=sorted_pos, row_kstart=row_kstart)
        if self.reducer is not None:
            self.reducer.finish()
        self.apply_update(lr if lr is not None else self.tc.lr)
        return stats

    def _graph_step(self, y: torch.Tensor, lr: Optional[float]) -> torch.Tensor:
        """The same step with forward + backward replayed from a CUDA graph. Per step the host copies the token ids
        and the step's dropout seeds into fixed device buffers, launches the graph, and runs clip + AdamW (whose
        step count and learning rate change every step) as ordinary launches."""
        from . import operators as ops
        n_seeds = 1 + 3 * self.cfg.layers
        if self._seed_words is None:
            self._seed_words = torch.zeros(n_seeds, device=self.device, dtype=torch.int64)
            self._seed_host = torch.zeros(n_seeds, dtype=torch.int64).pin_memory()
        self._seed_host.copy_(torch.tensor(step_seeds(self.tc.seed, self.t, self.rank, n_seeds), dtype=torch.int64))
        self._seed_words.copy_(self._seed_host, non_blocking=True)
        if self._graph is None or self._graph[0] != tuple(y.shape):
            ids = torch.empty(tuple(y.shape), device=self.device, dtype=torch.int32)
            ids.copy_(y, non_blocking=True)
            refs = [ops.seed_at(self._seed_words, i) for i in range(n_seeds)]

            def fwd_bwd(on_ready=None):
                sorted_pos = torch.sort(ids[:, :-1].reshape(-1), stable=True).indices.to(torch.int32)
                return self.engine.loss_and_grads(self.w, self.gv, ids, True, refs, sorted_pos=sorted_pos,
                                                  on_ready=on_ready)

            before = _lib.launch_count()
            if self.reducer is None:
                side = torch.cuda.Stream(self.device)
                side.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(side):  # warm-up: sizes the allocator's pools and every lazily initialised cache
                    for _ in range(2):
                        fwd_bwd()
                torch.cuda.current_stream(self.device).wait_stream(side)
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                before = _lib.launch_count()
                with torch.cuda.graph(graph):
                    stats = fwd_bwd()
                parts = [graph]
            else:
                parts, stats = self._record_segments(fwd_bwd)
            self.graph_launches = _lib.launch_count() - before
            self._graph = (tuple(y.shape), parts, ids, stats)
        _, parts, ids, stats = self._graph
        ids.copy_(y, non_blocking=True)
        if self.reducer is not None:
            if self.peer_watch is not None:
                self.peer_watch.announce(self.t)
                self.peer_watch.check(self.t)
            self.reducer.reset()
        for part in parts:
            if isinstance(part, int):
                self.reducer.launch_bucket(part)  # event on this stream -> NCCL stream -> all-reduce in place
            else:
                part.replay()
        if self.reducer is not None:
            self.reducer.finish()
        self.graph_replays += 1
        self.apply_update(lr if lr is not None else self.tc.lr)
        return stats

    def _record_segments(self, fwd_bwd):
        """Records forward + backward as a chain of CUDA graphs that ends one graph at every point where a gradient
        bucket becomes final, and returns [graph, bucket, graph, bucket, ...] in launch order. Nothing runs while
        recording and no collective is recorded; all graphs draw from one memory pool, so tensors made in one segment
        stay valid in the later ones, and they are always replayed in this order."""
        dev = self.device
        torch.cuda.synchronize(dev)
        pool = torch.cuda.graph_pool_handle()
        stream = torch.cuda.Stream(dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        parts: List[object] = []
        cur = [None]

        def begin():
            cur[0] = torch.cuda.CUDAGraph()
            cur[0].capture_begin(pool=pool, capture_error_mode="thread_local")

        def cut(bucket: int):
            cur[0].capture_end()
            parts.extend([cur[0], bucket])
            begin()

        self.reducer.reset()
        self.reducer.on_complete = cut
        try:
            with torch.cuda.stream(stream):
                begin()
                try:
                    stats = fwd_bwd(self.reducer.mark_ready)
                finally:
                    import warnings
                    with warnings.catch_warnings():  # nothing follows the last bucket: the final graph may be empty
                        warnings.filterwarnings("ignore", message="The CUDA Graph is empty")
                        cur[0].capture_end()
                parts.append(cur[0])
        finally:
            self.reducer.on_complete = None
        torch.cuda.current_stream(dev).wait_stream(stream)
        return parts, stats

    def apply_update(self, lr: float):
        """Clip by the global norm of the (reduced) gradient buffer and run the fused AdamW; t counts from 1."""
        lib, st = _lib.lib(), torch.cuda.current_stream().cuda_stream
        self.t += 1
        scale = 1.0 / self.world
        sumsq_ptr, max_norm = 0, 0.0
        if self.tc.clip is not None:
            _lib.check(lib.ptj_sumsq(self.g.data_ptr(), self.sumsq.data_ptr(), self.sumsq_scratch.data_ptr(),
                                     self.sumsq_scratch.numel(), self.g.numel(), st), "ptj_sumsq")
            sumsq_ptr, max_norm = self.sumsq.data_ptr(), float(self.tc.clip)
        _lib.check(
            lib.ptj_adamw(self.p.data_ptr(), self.g.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                          self.shadow.data_ptr() if self.shadow is not None else 0, self.p.numel(),
                          self.seg_start.data_ptr(), self.seg_decay.data_ptr(), self.nseg, lr, self.tc.betas[0],
                          self.tc.betas[1], self.tc.eps, self.tc.weight_decay, self.t, scale, sumsq_ptr, max_norm, st),
            "ptj_adamw")

    def grad_norm(self) -> float:
        """Pre-clip global gradient norm of the last step (host sync; for logging)."""
        return math.sqrt(float(self.sumsq.item())) / self.world

    def state_dict(self):
        return {"p": self.p.clone(), "m": self.m.clone(), "v": self.v.clone(), "t": self.t, "seed": self.tc.seed}

    def load_state_dict(self, sd):
        self.p.copy_(sd["p"]); self.m.copy_(sd["m"]); self.v.copy_(sd["v"])
        self.t = int(sd["t"])
        self._refresh_shadow()
