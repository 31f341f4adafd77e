"""Per-kernel micro-benchmarks at the GPT-2 small training shapes: achieved TFLOP/s or GB/s next to the measured peaks.

    python pre-tjax_b200/kernel_bench.py [--json out.json] [--tokens 8192] [--only gemm|attention|memory]
                                         [--case SUBSTRING] [--reps N] [--no-graph]

--case keeps only the cases whose name contains SUBSTRING and --no-graph launches directly instead of replaying a
CUDA graph: together they give a small, plain process to put under a profiler.

Each case is timed with CUDA events on the launching stream after warm-up, back to back without host
synchronisation. Memory-bound cases cycle through enough distinct copies of their operands that the bytes touched
between two uses of the same copy exceed twice the 126 MB L2, so every launch reads from HBM as it does inside a
training step. "Algorithmic" bytes / FLOPs are the ones a perfect implementation must move or compute (inputs read
once, outputs written once).
"""
from __future__ import annotations

import importlib
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


REPS = 20
USE_GRAPH = True
CASE = None


def time_us(fn, reps=None, warm=3, name=None):
    """Average device time of fn() in microseconds; fn may take the repetition index (to rotate operands).
    The repetitions are captured into one CUDA graph and replayed, so the host-side cost of a launch (tens of
    microseconds from Python) does not hide kernels that only take a few microseconds."""
    if CASE is not None and name is not None and CASE not in name:
        return None
    reps = reps or REPS
    import inspect
    takes_i = len(inspect.signature(fn).parameters) > 0
    call = (lambda i: fn(i)) if takes_i else (lambda i: fn())
    for i in range(warm):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if USE_GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                call(i)
        graph.replay()
        e0.record()
        graph.replay()
    else:
        e0.record()
        for i in range(reps):
            call(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def copies(make, nbytes_per_copy):
    """Enough independent copies of an operand set to defeat the L2 (at least 2 x 126 MB in rotation)."""
    n = max(2, -(-(2 * 126 << 20) // max(1, nbytes_per_copy)) + 1)
    return [make() for _ in range(min(n, 64))]


def main():
    args = sys.argv[1:]
    T = int(args[args.index("--tokens") + 1]) if "--tokens" in args else 8192
    out_json = args[args.index("--json") + 1] if "--json" in args else None
    only = args[args.index("--only") + 1] if "--only" in args else None
    global REPS, USE_GRAPH, CASE
    if "--reps" in args:
        REPS = int(args[args.index("--reps") + 1])
    USE_GRAPH = "--no-graph" not in args
    CASE = args[args.index("--case") + 1] if "--case" in args else None
    want = lambda section: only is None or only == section
    ptj = importlib.import_module("pre-tjax_b200")
    ops, lib = ptj.operators, ptj._lib
    dev = "cuda"
    D, F, V, H, S = 768, 3072, 50257, 12, 1024
    B = T // S
    Vp = (V + 127) // 128 * 128
    peak_tf, peak_gbs, label = peaks()
    bf = lambda *s: torch.randn(*s, device=dev).bfloat16()
    rows = []

    def add(name, us, flops=None, nbytes=None):
        if us is None:
            return
        r = {"kernel": name, "us": round(us, 2)}
        if flops is not None:
            r.update(tflops=round(flops / us / 1e6, 1), frac=round(flops / us / 1e6 / peak_tf, 3), bound="tensor")
        if nbytes is not None:
            r.update(gbs=round(nbytes / us / 1e3, 1), frac=round(nbytes / us / 1e3 / peak_gbs, 3), bound="hbm")
        rows.append(r)
        print(json.dumps(r), flush=True)

    def run(name, fn, flops=None, nbytes=None, reps=None):
        """Times one case unless --case names another one."""
        add(name, time_us(fn, reps=reps, name=name), flops, nbytes)

    # ---- GEMMs (bf16 in, fp32 accumulate) ----
    if want("gemm"):
        x_d, x_f = bf(T, D), bf(T, F)
        w_qkv, w_o, w1, w2, w_emb = bf(3 * D, D), bf(D, D), bf(F, D), bf(D, F), bf(V, D)
        b_f, b_d, b_v = (torch.randn(n, device=dev) for n in (F, D, V))
        y_qkv, y_d, y_f = bf(T, 3 * D), bf(T, D), bf(T, F)
        logits = torch.empty(T, Vp, device=dev, dtype=torch.bfloat16)
        drop = (0.1, True, 1234, 0)
        cases = [
            ("gemm fwd qkv        [T,768]x[2304,768]^T", lambda: ops.gemm(x_d, w_qkv), 2 * T * 3 * D * D),
            ("gemm fwd out-proj   +dropout+residual", lambda: ops.gemm(x_d, w_o, epilogue=lib.EPI_DROPOUT_RESID, aux=y_d, dropout_args=drop), 2 * T * D * D),
            ("gemm fwd ffn1       +bias+gelu (saves pre-act)", lambda: ops.gemm(x_d, w1, bias=b_f, epilogue=lib.EPI_GELU, aux_out=y_f), 2 * T * F * D),
            ("gemm fwd ffn2       +bias+dropout+residual", lambda: ops.gemm(x_f, w2, bias=b_d, epilogue=lib.EPI_DROPOUT_RESID, aux=y_d, dropout_args=drop), 2 * T * F * D),
            ("gemm fwd lm-head    [T,768]x[50257,768]^T +bias", lambda: ops.gemm(x_d, w_emb, bias=b_v, out=logits, N=V, ldc=Vp), 2 * T * V * D),
            ("gemm dgrad ffn2     dy W2, *gelu'(pre)", lambda: ops.gemm(y_d, w2, a_kmajor=True, b_kmajor=False, M=T, N=F, K=D, epilogue=lib.EPI_GELU_BWD, aux=y_f), 2 * T * F * D),
            ("gemm dgrad ffn1     dh W1 (last round of tiles split over K, as in the step)", lambda: step._dgrad(y_f, w1), 2 * T * F * D),
            ("gemm dgrad out-proj dy Wo", lambda: ops.gemm(y_d, w_o, a_kmajor=True, b_kmajor=False, M=T, N=D, K=D), 2 * T * D * D),
            ("gemm dgrad qkv      dqkv Wqkv (last round split over K)", lambda: step._dgrad(y_qkv, w_qkv), 2 * T * 3 * D * D),
            ("gemm dgrad lm-head  dlogits Wemb (last round split over K)", lambda: step._dgrad(logits, w_emb, cols=V), 2 * T * V * D),
        ]
        step = ptj.gpt2.Gpt2Step(ptj.PRESETS["gpt2-small"])
        g_w2, g_w1, g_wo, g_wqkv, g_emb = (torch.empty(*s, device=dev) for s in ((D, F), (F, D), (D, D), (3 * D, D), (V, D)))
        cases += [
            ("gemm wgrad ffn2     dy^T h   [768,3072] (+split-K reduce)", lambda: step._wgrad(y_d, x_f, g_w2), 2 * T * F * D),
            ("gemm wgrad ffn1     dh^T x   [3072,768] (+split-K reduce)", lambda: step._wgrad(y_f, x_d, g_w1), 2 * T * F * D),
            ("gemm wgrad out-proj dy^T a   [768,768] (+split-K reduce)", lambda: step._wgrad(y_d, x_d, g_wo), 2 * T * D * D),
            ("gemm wgrad qkv      dqkv^T x [2304,768] (+split-K reduce)", lambda: step._wgrad(y_qkv, x_d, g_wqkv), 2 * T * 3 * D * D),
            ("gemm wgrad ffn2 + ffn1 in one launch (no K split, no reduce)", lambda: step._wgrad2((y_d, x_f, g_w2), (y_f, x_d, g_w1)), 4 * T * F * D),
            ("gemm wgrad qkv + out-proj in one launch (K in two parts each)", lambda: step._wgrad2((y_qkv, x_d, g_wqkv), (y_d, x_d, g_wo)), 2 * T * 4 * D * D),
            ("gemm wgrad lm-head  dlogits^T x [50257,768]", lambda: step._head_wgrad(logits, x_d, g_emb), 2 * T * V * D),
        ]
        for name, fn, fl in cases:
            add(name, time_us(fn, name=name), flops=fl)
        del logits, w_emb, g_emb

    # ---- attention (causal, dropout 0.1 on the probabilities) ----
    if want("attention"):
        qkv = bf(T, 3 * D)
        v5 = qkv.view(B, S, H, 3, 64)
        q, k, v = (v5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
        o = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
        o4, do4 = o.view(B, S, H, 64).permute(0, 2, 1, 3), bf(T, D).view(B, S, H, 64).permute(0, 2, 1, 3)
        dqkv = torch.empty_like(qkv)
        d5 = dqkv.view(B, S, H, 3, 64)
        dq, dk, dv = (d5[:, :, :, c, :].permute(0, 2, 1, 3) for c in range(3))
        fl_attn = 4 * B * H * S * S * 64 / 2
        m, l = ops.attn_fwd(q, k, v, o4, True, 5, p=0.1)
        run("attention fwd  B*H=%d S=1024 d=64 dropout 0.1" % (B * H), lambda: ops.attn_fwd(q, k, v, o4, True, 5, p=0.1), flops=fl_attn)
        run("attention bwd  (dQ, dK, dV; recompute) dropout 0.1", lambda: ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, True, 5, p=0.1), flops=2.5 * fl_attn)
        bits = ops.attn_keep_bits(q, k, v, o4, 5, p=0.1)
        run("attention keep flags of one call (Philox, 16-bit lanes)", lambda: ops.attn_keep_bits(q, k, v, o4, 5, p=0.1, bits=bits))
        run("attention fwd  dropout 0.1, keep flags given", lambda: ops.attn_fwd(q, k, v, o4, True, 5, p=0.1, keep_bits=bits), flops=fl_attn)
        run("attention bwd  dropout 0.1, keep flags given", lambda: ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, True, 5, p=0.1, keep_bits=bits), flops=2.5 * fl_attn)
        # packed batch: every row holds eight documents of 128 tokens (tiles before a document's first key are skipped)
        ks_packed = ops.row_kstart_from_lengths([[128] * (S // 128)] * B, S)
        ks_one = ops.row_kstart_from_lengths([[S]] * B, S)
        run("attention fwd  packed, 8 documents of 128 per row, keep flags given", lambda: ops.attn_fwd(q, k, v, o4, True, 5, p=0.1, keep_bits=bits, row_kstart=ks_packed))
        run("attention bwd  packed, 8 documents of 128 per row, keep flags given", lambda: ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, True, 5, p=0.1, keep_bits=bits, row_kstart=ks_packed))
        run("attention fwd  one document per row through the packed path", lambda: ops.attn_fwd(q, k, v, o4, True, 5, p=0.1, keep_bits=bits, row_kstart=ks_one))
        run("attention fwd  no dropout", lambda: ops.attn_fwd(q, k, v, o4, True, 5, p=0.0), flops=fl_attn)
        run("attention bwd  no dropout", lambda: ops.attn_bwd(do4, q, k, v, o4, m, l, dq, dk, dv, True, 5, p=0.0), flops=2.5 * fl_attn)

    # ---- memory-bound operators (operands rotate through copies so that nothing is served from L2) ----
    if want("memory"):
        st = lambda: torch.cuda.current_stream().cuda_stream
        g, bta = torch.ones(D, device=dev), torch.zeros(D, device=dev)
        dg, db = torch.empty(D, device=dev), torch.empty(D, device=dev)
        xs = copies(lambda: (bf(T, D), bf(T, D), bf(T, D)), 3 * T * D * 2)
        n = len(xs)
        run("layernorm fwd [T,768] bf16", lambda i: ops.t_layernorm_fwd_t((g, bta), xs[i % n][0]), nbytes=2 * T * D * 2)
        run("layernorm bwd dx+dgamma+dbeta (+residual grad)", lambda i: ops.layernorm_bwd(xs[i % n][1], (g, None), xs[i % n][0], dx_add=xs[i % n][2], dgamma_out=dg, dbeta_out=db), nbytes=4 * T * D * 2)
        cs = torch.empty(D, device=dev)
        run("layernorm bwd ... + dropout(dx) as a second output", lambda i: ops.layernorm_bwd(xs[i % n][1], (g, None), xs[i % n][0], dx_add=xs[i % n][2], dgamma_out=dg, dbeta_out=db, dropped=(True, 7, 0.1)), nbytes=5 * T * D * 2)
        run("layernorm bwd ... + dropout(dx) + its column sums", lambda i: ops.layernorm_bwd(xs[i % n][1], (g, None), xs[i % n][0], dx_add=xs[i % n][2], dgamma_out=dg, dbeta_out=db, dropped=(True, 7, 0.1), dropped_colsum_out=cs), nbytes=5 * T * D * 2)
        run("colsum (bias grad) [T,768]", lambda i: ops.colsum(xs[i % n][0], out=cs), nbytes=T * D * 2)
        run("dropout [T,768] (mask regenerated)", lambda i: ops.dropout(xs[i % n][0], True, 7, p=0.1), nbytes=2 * T * D * 2)
        run("dropout + residual add [T,768]", lambda i: ops.dropout(xs[i % n][0], True, 7, residual=xs[i % n][1], p=0.1), nbytes=3 * T * D * 2)
        del xs
        fs = copies(lambda: (bf(T, F), bf(T, F)), 2 * T * F * 2)
        n = len(fs)
        run("gelu fwd [T,3072]", lambda i: ops.t_gelu_fwd_t(fs[i % n][0]), nbytes=2 * T * F * 2)
        run("gelu bwd [T,3072]", lambda i: ops.t_gelu_bkwd2_t(fs[i % n][1], fs[i % n][0]), nbytes=3 * T * F * 2)
        run("colsum (bias grad) [T,3072]", lambda i: ops.colsum(fs[i % n][0]), nbytes=T * F * 2)
        del fs
        lg, lg2 = bf(T, Vp), torch.empty(T, Vp, device=dev, dtype=torch.bfloat16)  # 824 MB each: far beyond L2
        labels = torch.randint(1, V, (T,), device=dev, dtype=torch.int32)
        r5 = max(3, REPS // 4)
        run("log-softmax fwd [T,50257] (ld 50304)", lambda: lib.check(lib.lib().ptj_log_softmax_fwd(lg.data_ptr(), lg2.data_ptr(), T, V, Vp, Vp, 1, st()), "lsm"), reps=r5, nbytes=2 * T * V * 2)
        run("log-softmax bwd [T,50257]", lambda: lib.check(lib.lib().ptj_log_softmax_bwd(lg.data_ptr(), lg.data_ptr(), lg2.data_ptr(), T, V, Vp, 1, st()), "lsm"), reps=r5, nbytes=3 * T * V * 2)
        run("colsum (lm-head bias grad) [T,50257]", lambda: ops.colsum(lg, cols=V), reps=r5, nbytes=T * V * 2)
        run("cross-entropy fwd+bwd in place [T,50257]", lambda: ops.cross_entropy(labels, lg2, cols=V, want_grad=True, in_place=True), reps=r5, nbytes=2 * T * V * 2)
        del lg, lg2
        n = 124_453_248
        p_, g_, m_, v_ = (torch.zeros(n, device=dev) for _ in range(4))
        sh = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        run("adamw fused (+bf16 shadow) 124M params", lambda: lib.check(lib.lib().ptj_adamw(p_.data_ptr(), g_.data_ptr(), m_.data_ptr(), v_.data_ptr(), sh.data_ptr(), n, 0, 0, 0, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, 0, 0.0, st()), "adamw"), reps=r5, nbytes=n * 30)
        run("grad sum of squares 124M", lambda: ptj.optimizer.sumsq(g_), reps=r5, nbytes=n * 4)
        del p_, g_, m_, v_, sh
        # embedding backward on Zipf(1.1) token ids (the most frequent token makes a run of several hundred rows)
        gz = torch.Generator().manual_seed(0)
        wz = torch.arange(1, V, dtype=torch.float64).pow(-1.1)
        ids = (torch.searchsorted(torch.cumsum(wz / wz.sum(), 0), torch.rand((B, S), generator=gz, dtype=torch.float64))
               .clamp_(max=V - 2) + 1).to(torch.int32).to(dev)
        spos = torch.sort(ids.reshape(-1), stable=True).indices.to(torch.int32)
        dwe, dwp, dy_e = torch.zeros(V, D, device=dev), torch.zeros(S, D, device=dev), bf(T, D)
        add("embedding backward (scatter by token run + positions), Zipf ids, dropout 0.1",
            time_us(lambda: ops.embed_bwd(dy_e, ids, dwe, dwp, True, True, 3, sorted_pos=spos, p=0.1), reps=r5),
            nbytes=T * D * 2 * 2)

    print(f"# peaks ({label}): {peak_tf} TFLOP/s bf16, {peak_gbs} GB/s", flush=True)
    if out_json:
        Path(out_json).write_text(json.dumps({"peaks": {"tflops": peak_tf, "gbs": peak_gbs, "source": label}, "rows": rows}, indent=1))


if __name__ == "__main__":
    main()
