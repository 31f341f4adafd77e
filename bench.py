"""Benchmark of the GPT-2 training hot path (fwd + hand-written bwd + clip + AdamW) on 1..8 B200.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the reference algorithm on the host cores (CPU oracle port)

Prints ONE JSON line (rank 0). `value` = tokens/s of the whole job with the token ids already resident in HBM;
`e2e` = the same step driven from pinned host buffers with the host-to-device copy of the ids and the
device-to-host read of the loss inside the timed region. Workload: GPT-2 small (12 layers, d_model 768, 12 heads,
FFN 3072, seq 1024, vocab 50257, tied embeddings, dropout 0.1), bf16 compute with fp32 master weights and fp32
accumulation, AdamW lr 6e-4 betas (0.9, 0.95) wd 0.1, gradient clip 1.0, micro-batch 8 sequences per GPU of
Zipf(1.1) token ids (synthetic stand-in for the text corpus), data-parallel gradient allreduce over NCCL.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "GPT-2 113M train tokens/s"
UNIT = "tokens/s"
MICRO_BATCH = 8
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the tcgen05 GEMM at the shapes of the
# GPT-2 small step, from single-kernel ncu captures of pre-tjax_b200/kernel_bench.py cases (the summaries under
# profiles/ named here). `roofline.traffic` is the launch-weighted mean over the GEMM launches of the timed steps:
# a captured shape contributes its measured bytes, any other shape its algorithmic bytes (operands read once, output
# written once), and the line says how many launches were covered by a capture.
NCU_GEMM_TRAFFIC = {
    # (M, N, K, a_kmajor, b_kmajor): (bytes per launch, profiles/ file)
    (8192, 3072, 768, True, True): (67.7e6, "gemm_tc_kernel_ffn1_fwd_ffn2_dgrad_counters.md"),    # FFN-1 forward + GELU
    (8192, 3072, 768, True, False): (89.8e6, "gemm_tc_kernel_ffn1_fwd_ffn2_dgrad_counters.md"),   # dy W2 x gelu'
    (3072, 768, 8192, False, False): (68.1e6, "gemm_tc_pair_kernel_wgrad_dgrad_ffn1_counters.md"),  # FFN-1 weight gradient
    (8192, 768, 3072, True, False): (58.8e6, "gemm_tc_pair_kernel_wgrad_dgrad_ffn1_counters.md"),   # dh W1
    # the two FFN weight gradients in one launch
    ("grouped", 768, 3072, 3072, 768, 8192): (130.7e6, "gemm_tc_pair_kernel_wgrad_dgrad_ffn1_counters.md"),
}


def zipf_ids(vocab: int, shape, seed: int, a: float = 1.1) -> torch.Tensor:
    """Token ids with P(id = r) proportional to r^-a over r = 1..vocab-1 (id 0 is the padding id and never drawn)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.arange(1, vocab, dtype=torch.float64).pow(-a)
    cdf = torch.cumsum(w / w.sum(), 0)
    u = torch.rand(shape, generator=g, dtype=torch.float64)
    return (torch.searchsorted(cdf, u).clamp_(max=vocab - 2) + 1).to(torch.int32)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0])); mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def measured_peaks() -> tuple:
    """(bf16 TFLOP/s sustained, HBM GB/s, label) from MEASURED_PEAKS.json, else the stated fallback."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))), float(d["hbm_gbs"]), "measured"
    return 1400.0, 6650.0, "fallback"


# ---- CPU arm: the reference algorithm (oracle port) on the host cores -----------------------------------------------
def reference_checkout_step_rate(ref_dir: str, cfg, steps: int, warmup: int, seqs: int) -> dict:
    """The UNMODIFIED reference (a checkout of martin-kukla/pre-tjax at ref_dir) on the host cores: its torch.func
    gradient (uncompiled_grad_loss, loss_and_optimizer_triton.py:234) + adam_w_in_place (:376-401), float32, dropout
    rate 0 (a module constant of the reference), the reference's own parameter initialisation. The reference has no
    gradient clipping, so none is timed."""
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import model_torch_func as mtf
    mtf.DEVICE = "cpu"
    mtf.DROPOUT_RATE = 0.0
    import model_triton as mt
    mt.DROPOUT_RATE = 0.0
    import loss_and_optimizer_triton as lot
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    torch.manual_seed(0)
    prm = mtf.init_transformer_gpt2(cfg.vocab, cfg.dim, cfg.layers, cfg.heads, cfg.ffn, cfg.seq)
    mom = [[[torch.zeros_like(t) for t in grp] for grp in prm] for _ in range(2)]
    wd_mask = [[not (t.dim() == 1 and bool((t == 0).all())) for t in grp] for grp in prm]
    mask = torch.tril(torch.ones((cfg.seq, cfg.seq), dtype=torch.bool)).unsqueeze(0).expand(seqs, -1, -1).contiguous()
    idx = torch.arange(cfg.seq).unsqueeze(0).expand(seqs, -1).contiguous()
    times = []
    for i in range(warmup + steps):
        y = zipf_ids(cfg.vocab, (seqs, cfg.seq + 1), seed=1000 + i)
        t0 = time.perf_counter()
        grads, _ = lot.uncompiled_grad_loss(prm, y, mask, idx)
        prm, mom = lot.adam_w_in_place(prm, grads, 6e-4, (0.9, 0.95), 1e-8, mom, i, weight_decay=0.1,
                                       weight_decay_mask=wd_mask)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return {"value": seqs * cfg.seq / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference",
            "sample": f"{seqs} sequence(s) of {cfg.seq} tokens per step (micro-batch {MICRO_BATCH}), {steps} timed "
                      f"step(s) after {warmup} warm-up, the unmodified reference's torch.func path, float32, dropout off",
            "sec_per_step": sec}


def cpu_reference_step_rate(cfg, steps: int, warmup: int, seqs: int = 1) -> dict:
    """tokens/s of fwd + bwd + clip + AdamW in float32 on the CPU for `seqs` sequences per step: the unmodified
    reference when PTJ_REFERENCE_DIR names a checkout of it, else the oracle port of the same algorithm."""
    ref_dir = os.environ.get("PTJ_REFERENCE_DIR")
    if ref_dir and os.path.isfile(os.path.join(ref_dir, "model_torch_func.py")):
        return reference_checkout_step_rate(ref_dir, cfg, steps, warmup, seqs)
    from oracle import gpt2_oracle as orc
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    prm = orc.init_params(cfg.vocab, cfg.dim, cfg.layers, cfg.heads, cfg.ffn, cfg.seq, seed=0)
    mom = [[[torch.zeros_like(t) for t in grp] for grp in prm] for _ in range(2)]
    mask = orc.decay_mask(prm)
    times = []
    for i in range(warmup + steps):
        y = zipf_ids(cfg.vocab, (seqs, cfg.seq + 1), seed=1000 + i)
        t0 = time.perf_counter()
        grads, _ = orc.loss_and_grads(prm, y, p=0.0, train=True)
        s = orc.clip_scale(orc.grads_l2norm(grads), 1.0)
        prm, mom = orc.adam_w(prm, [[g * s for g in grp] for grp in grads], 6e-4, (0.9, 0.95), 1e-8, mom, i, 0.1, mask)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return {"value": seqs * cfg.seq / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{seqs} sequence(s) of {cfg.seq} tokens per step (micro-batch {MICRO_BATCH}), "
                      f"{steps} timed step(s) after {warmup} warm-up, float32, dropout off", "sec_per_step": sec}


def cpu_arm(cfg, steps: int, warmup: int) -> dict:
    """The CPU arm on the FULL micro-batch (what one GPU step processes); if the host cannot hold the float32
    activations of all sequences at once (about 30 GB for GPT-2 small x 8), on as many sequences as fit."""
    seqs = MICRO_BATCH
    while True:
        try:
            return cpu_reference_step_rate(cfg, steps, warmup, seqs=seqs)
        except (MemoryError, RuntimeError) as e:
            if seqs == 1 or "memory" not in str(e).lower() and not isinstance(e, MemoryError):
                raise
            seqs = max(1, seqs // 2)


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 2))
    warm = 1 if args.warmup > 0 else 0
    r = cpu_arm(cfg, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": r["sec_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args.gpus), "gpu_launches": 0,
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": ("the unmodified reference's torch.func path" if r["kind"] == "reference" else
                 "reference torch.func algorithm restated on the CPU (no checkout of the reference was named in "
                 "PTJ_REFERENCE_DIR)") + "; requested steps are capped so the CPU run stays within minutes",
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, n):
    name = {12: "gpt2-small", 24: "gpt2-medium"}.get(cfg.layers, "gpt2")
    note = " (the reference calls its V=35k/S=512 variant of this model 113M)" if cfg.layers == 12 else ""
    return {"workload": f"{name} {cfg.layers}L/d{cfg.dim}/{cfg.heads}H/FFN{cfg.ffn}/S{cfg.seq}/V{cfg.vocab}, "
                        f"{cfg.num_params():,} params{note}: full train step fwd+bwd+clip+AdamW, "
                        f"dropout {cfg.dropout}, Zipf(1.1) ids",
            "global_batch": MICRO_BATCH * n, "micro_batch_per_gpu": MICRO_BATCH, "seq_len": cfg.seq,
            "parallelism": f"dp{n}", "l2": "per-step working set (about 1.3 GB of weights+moments traffic and several "
                                           "GB of activations) far exceeds the 126 MB L2; no explicit flush"}


# ---- our arm --------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt2-small", choices=["gpt2-small", "gpt2-medium"])
    ap.add_argument("--micro-batch", type=int, default=None, help="sequences per GPU (default 8; 16 for gpt2-medium)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="issue every kernel of a step from the host instead of replaying CUDA graphs of forward + backward")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    ptj = importlib.import_module("pre-tjax_b200")
    cfg = ptj.PRESETS[args.model]
    global MICRO_BATCH
    MICRO_BATCH = args.micro_batch or (16 if args.model == "gpt2-medium" else 8)
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # (NCCL's own choice of thread blocks per collective is kept: capping it to 8 made the last, exposed all-reduce
        # 1.2 ms long on two GPUs, more than the persistent kernels gained from the SMs it freed)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    ops = ptj.operators
    tc = ptj.TrainConfig.benchmark_recipe(seed=0, cuda_graph=not args.no_graph)
    trainer = ptj.Trainer(cfg, tc, device=f"cuda:{local}", world=world, rank=rank)
    n_batches = 4
    host = [zipf_ids(cfg.vocab, (MICRO_BATCH, cfg.seq + 1), seed=17 + 1000 * rank + i).pin_memory() for i in range(n_batches)]
    dev = [h.cuda() for h in host]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = [0.0]

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        for i in range(steps):
            fn(i)
        host_ms[0] = (time.perf_counter() - t0) * 1e3 / steps  # time the host needs to enqueue one step
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    losses = []
    for i in range(args.warmup):
        losses.append(trainer.step(dev[i % n_batches]))
    # device-resident inputs; nothing but the step's own kernels on the stream
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0, replays0 = ptj._lib.launch_count(), trainer.graph_replays
    ms = timed(lambda i: losses.append(trainer.step(dev[i % n_batches])), args.steps)
    host_enqueue_ms = host_ms[0]
    # kernels of this library launched in the timed region: those issued one by one plus, per graph replay, the
    # kernels recorded in the graph
    launches = ptj._lib.launch_count() - launches0 + (trainer.graph_replays - replays0) * trainer.graph_launches
    exposed = None
    # the same steps once more with every GEMM launch bracketed by CUDA events (the roofline line). The events sit
    # between kernels of the stream, where they keep the next kernel's set-up from overlapping the previous
    # kernel's tail, so this pass is a little slower than the one above and is not the one reported as `value`.
    graph_mode, trainer.use_graph = trainer.use_graph, False  # events around single launches need ordinary launches
    trainer.step(dev[0])  # one untimed step with ordinary launches (their memory pools are not the graph's)
    if trainer.reducer is not None:
        trainer.reducer.measure_exposed = True
    ops.GEMM_PROFILE = []
    ms_prof = timed(lambda i: losses.append(trainer.step(dev[i % n_batches])), args.steps)
    gemm_events, ops.GEMM_PROFILE = ops.GEMM_PROFILE, None
    if trainer.reducer is not None:  # time the compute stream waited for all-reduces that backward did not hide
        trainer.reducer.measure_exposed = False
        ex = trainer.reducer.exposed_ms()
        exposed = sum(ex) / max(1, len(ex))
    trainer.use_graph = graph_mode
    clocks = sampler.stop() if rank == 0 else None
    # end to end: pinned host ids -> device, loss read back every step
    sink = []
    ms_e2e = timed(lambda i: sink.append(float(trainer.step(host[i % n_batches])[0].item())), args.steps)

    tokens_per_step = MICRO_BATCH * cfg.seq * world
    if rank == 0:
        peak_tf, peak_gbs, label = measured_peaks()
        gemm_ms = sum(e[0].elapsed_time(e[1]) for e in gemm_events)
        gemm_flop = sum(e[2] for e in gemm_events)
        traffic, covered = 0.0, 0
        for e in gemm_events:
            hit = NCU_GEMM_TRAFFIC.get(e[3])
            covered += hit is not None
            traffic += hit[0] if hit is not None else e[4]
        achieved = gemm_flop / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        line = {
            "metric": METRIC, "value": tokens_per_step * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(cfg, world), "clocks": clocks,
            "e2e": {"value": tokens_per_step * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": host[0].numel() * 4, "d2h_bytes_per_step": 4,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches), "host_enqueue_ms_per_step": host_enqueue_ms,
            "launch_mode": ("CUDA graph of forward + backward, clip + AdamW launched directly" if world == 1 else
                            "CUDA graphs of forward + backward, cut at every gradient bucket; all-reduces, clip + AdamW launched directly")
            if graph_mode else "every kernel launched from the host",
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05 GEMM, all launches of the timed steps)",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": (achieved / peak_tf) if achieved else None, "peak_source": f"of {label}",
                         "launches": len(gemm_events), "avg_launch_ms": gemm_ms / max(1, len(gemm_events)),
                         "gemm_share_of_step": gemm_ms / ms if ms > 0 else None,
                         "ms_per_step_with_events": ms_prof / args.steps,
                         "traffic": traffic / max(1, len(gemm_events)),
                         "traffic_source": f"{covered} of {len(gemm_events)} launches at shapes with an ncu capture "
                                           f"(profiles/), the rest at their algorithmic bytes"},
            "final_loss": float(losses[-1][0].item()),
        }
        if exposed is not None:
            line["allreduce_exposed_ms"] = exposed
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_arm(cfg, steps=1, warmup=1)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
