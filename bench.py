"""Benchmark of the GLoRCQ real-quant decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config qwen15|mixtral|qwen3]

Workload (default, one GPU): greedy batch-1 decode of the whole Qwen1.5-MoE-A2.7B-shaped decoder after a
512-token prompt -- 24 layers of {4-bit g128 attention projections with a rank-64 correction, attention over
a static key/value cache, router, 60 experts top-4 (intermediate 1408) + shared expert (5632), every expert
projection 2-bit g128 with a rank-64 low-rank correction whose input-side factor U is shared by 128 clusters
of experts across layers}, final norm and the fp16 output projection over a vocabulary of 151936 with the
arg-max -- on seeded synthetic weights.  One step = one decoded token: GLoRCQGraphWrapper.replay (token id and
position into the static buffers, one CUDA-graph replay), the next token taken on the device.  The weights
(6.6 GB) are far larger than L2 and a token touches ~1.5 GB of them.

One JSON line on stdout:
  value     decoded tokens/s, device-timed with CUDA events: the median of R >= 25 windows of exactly K steps,
            each window bracketed by a barrier + synchronize and starting at the position after the prompt
  e2e       the same through the public API with the token id coming from pinned host memory and the next
            token id read back to the host, every step
  roofline  the dominant kernel (the grouped dequant-GEMV) timed alone, live, on 240 distinct
            expert-projection problems (1408 x 2048, 2-bit g128, rank 64; 240 MB, larger than L2):
            algorithmic bytes / CUDA-event time against the measured HBM peak
  moe_only  the 24 MoE blocks alone (no attention, no output projection), chained through their fused
            residual + norm, one CUDA graph per token
  cpu_baseline  the CPU restatement of the reference's own path (oracle/), timed on the host cores on a
            bounded sample (one layer's pieces and the output projection for one token, repeated)
`--impl reference` times that CPU path as the main line (rank 0 only).  N > 1: the routed experts are sharded
over the ranks (expert e on rank e % N), everything else is replicated, one token stream per rank.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "moe_decode_tok_s"
UNIT = "tok/s"


def model_config(name):
    from glorcq_b200 import synthetic
    if name == "qwen15":
        return dict(synthetic.QWEN15_MOE_A27B), "Qwen1.5-MoE-A2.7B", 512
    if name == "mixtral":
        return dict(synthetic.MIXTRAL_8X7B), "Mixtral-8x7B", 1024
    if name == "qwen3":
        return dict(synthetic.QWEN3_30B_A3B), "Qwen3-30B-A3B", 512
    raise ValueError(name)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return json.load(open(path))
        except Exception:
            pass
    return None


def measured_peak_gbs():
    p = _peaks()
    return (float(p["hbm_gbs"]), "measured") if p and "hbm_gbs" in p else (6650.0, "fallback")


def measured_peak_tflops():
    p = _peaks()
    return (float(p["bf16_tflops"]), "measured") if p and "bf16_tflops" in p else (1590.0, "fallback")


def profiled_traffic(name):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu summary committed under profiles/
    (a line `traffic_bytes_per_launch: <number>` in profiles/<name>); None when there is none."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        for ln in open(path):
            if ln.strip().startswith("traffic_bytes_per_launch:"):
                return float(ln.split(":", 1)[1].split()[0])
    except OSError:
        pass
    return None


# ---- clocks ---------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        sm, smax, reasons = [], 0, set()
        for ln in self.samples:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(int(float(f[0])))
                smax = max(smax, int(float(f[1])))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- CPU baseline (reference arm): the oracle's pieces of one decode token --------------------------
class CpuToken:
    """One decode token of the decoder through the CPU oracle (the reference's PyTorch path restated), as a
    bounded sample: ONE layer's pieces -- q/k/v/o projections (4-bit + rank-64 correction), attention of the new
    token over `context` cached positions, the MoE block -- and the output projection, each for one token.
    seconds per token = layers x layer + output projection."""

    def __init__(self, cfg, context):
        from oracle import glorcq_oracle as O
        from tests import cases
        self.O, self.cfg = O, cfg
        torch.set_num_threads(os.cpu_count() or 1)
        H = cfg["hidden_size"]
        nh = cfg["num_attention_heads"]
        nkv = cfg.get("num_key_value_heads") or nh
        hd = cfg.get("head_dim") or H // nh
        E = cfg.get("num_experts", cfg.get("num_local_experts", 0))
        I = cfg.get("moe_intermediate_size", cfg.get("intermediate_size"))
        self.nh, self.nkv, self.hd = nh, nkv, hd
        blk = cases.make_moe(2001, H, I, E, cfg["num_experts_per_tok"], I_shared=cfg.get("shared_expert_intermediate_size", 0),
                             rank=64, experts_per_cluster=4, norm_topk_prob=cfg.get("norm_topk_prob", "num_local_experts" in cfg))
        self.moe = cases.to_oracle_moe(blk)
        self.attn = [cases.to_oracle_linear(cases.make_linear(2100 + i, n, k, rank=64, bits=4))
                     for i, (n, k) in enumerate([(nh * hd, H), (nkv * hd, H), (nkv * hd, H), (H, nh * hd)])]
        g = torch.Generator().manual_seed(2200)
        self.k_cache = torch.randn(1, nkv, context, hd, generator=g).half()
        self.v_cache = torch.randn(1, nkv, context, hd, generator=g).half()
        self.lm_head = (torch.randn(cfg["vocab_size"], H, generator=g) * 0.02).half()
        self.x = cases.make_x(3001, 1, H).reshape(1, 1, H)

    @torch.no_grad()
    def layer(self):
        O, x = self.O, self.x
        q = O.linear_forward(self.attn[0], x).view(1, 1, self.nh, self.hd).transpose(1, 2)
        k = O.linear_forward(self.attn[1], x).view(1, 1, self.nkv, self.hd).transpose(1, 2)
        v = O.linear_forward(self.attn[2], x).view(1, 1, self.nkv, self.hd).transpose(1, 2)
        kk = torch.cat([self.k_cache, k], 2).repeat_interleave(self.nh // self.nkv, dim=1)
        vv = torch.cat([self.v_cache, v], 2).repeat_interleave(self.nh // self.nkv, dim=1)
        s = (q.float() @ kk.float().transpose(-1, -2)) / self.hd ** 0.5
        a = (torch.softmax(s, -1).half() @ vv).transpose(1, 2).reshape(1, 1, -1)
        y = x + O.linear_forward(self.attn[3], a)
        out, _ = O.moe_forward(self.moe, y)
        return out

    @torch.no_grad()
    def head(self):
        return self.x.reshape(1, -1) @ self.lm_head.T

    def seconds(self, sample_seconds, max_reps):
        def med(fn):
            fn()
            ts, t_start = [], time.perf_counter()
            while len(ts) < max_reps and (time.perf_counter() - t_start < sample_seconds or len(ts) < 3):
                t0 = time.perf_counter()
                fn()
                ts.append(time.perf_counter() - t0)
            ts.sort()
            return ts[len(ts) // 2], len(ts)
        tl, nl = med(self.layer)
        th, _ = med(self.head)
        return self.cfg["num_hidden_layers"] * tl + th, torch.get_num_threads(), nl


def workload_config(cfg, name, prompt, batch, layers):
    E = cfg.get("num_experts", cfg.get("num_local_experts", 0))
    return {"workload": f"{name}-shaped decoder, greedy decode after a {prompt}-token prompt, batch {batch} per token stream set: "
                        f"{layers} layers (hidden {cfg['hidden_size']}, {cfg['num_attention_heads']} heads, attention projections "
                        f"4-bit g128 + rank 64, {E} experts top-{cfg['num_experts_per_tok']} x "
                        f"{cfg.get('moe_intermediate_size', cfg.get('intermediate_size'))}"
                        + (f" + shared expert {cfg['shared_expert_intermediate_size']}" if cfg.get("shared_expert_intermediate_size") else "")
                        + f", experts 2-bit g128 + rank-64 correction with 128 cross-layer shared-U clusters), fp16 output projection "
                        f"over {cfg['vocab_size']} tokens with arg-max; CUDA-graph replay per token",
            "layers": layers, "prompt": prompt,
            "l2": "per-token weight reads (~1.5 GB, different experts every token) far exceed the 126 MB L2"}


def run_reference(args, rank):
    if rank != 0:
        return
    cfg, name, prompt = model_config(args.config)
    prompt = args.prompt or prompt
    cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
    cpu = CpuToken(cfg, prompt)
    cpu.seconds(2.0, 3)                               # warm-up sample
    per = []
    for _ in range(max(1, args.steps)):
        sec, threads, _ = cpu.seconds(6.0 / max(1, args.steps) + 0.5, 20)
        per.append(sec)
    per.sort()
    sec = per[len(per) // 2]
    value = 1.0 / sec
    sample = (f"one token: 1 of {cfg['num_hidden_layers']} layers (4 attention projections, attention over {prompt} cached "
              f"positions, MoE block) and the output projection, median of repeated CPU forwards; "
              f"tok/s = 1 / ({cfg['num_hidden_layers']} x layer + output projection)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(cfg, name, prompt, args.batch, cfg["num_hidden_layers"]),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------------------
def _c1_problems(dev, P, seed, fmt="q2"):
    from glorcq_b200.tiled import TiledWeight
    N, K, r = 1408, 2048, 64
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    keep, descs = [], []
    for _ in range(P):
        if fmt == "t2":       # 2-bit codebook codes, per-row norms, the reference's Lloyd-Max codebook shape
            tw = TiledWeight.from_turbo(torch.randint(0, 256, (N, K // 4), generator=g, device=dev, dtype=torch.uint8),
                                        (torch.rand(N, generator=g, device=dev) + 0.5).float(),
                                        torch.tensor([-1.51, -0.4528, 0.4528, 1.51], device=dev) / (K ** 0.5))
        else:
            bits = 4 if fmt == "q4" else 2
            tw = TiledWeight.from_gptq(torch.randint(0, 1 << bits, (N, K), generator=g, device=dev, dtype=torch.int32),
                                       (torch.randn(N, K // 128, generator=g, device=dev) * 0.02).abs().half(),
                                       torch.randint(0, 1 << bits, (N, K // 128), generator=g, device=dev).half(), bits, 128)
        tw.put_sv(0, (torch.randn(N, r, generator=g, device=dev) * 0.01).half())
        keep.append(tw)
        descs.append(tw.desc_bytes())
    table = torch.frombuffer(bytearray(b"".join(descs)), dtype=torch.uint8).to(dev)
    return keep, table, g


def gemv_roofline(dev, peak_gbs, peak_kind, P=240, iters=50, fmt="q2"):
    """The grouped dequant-GEMV alone: P distinct 1408x2048 rank-64 problems, one row each (2-bit g128 codes;
    `fmt` "q4" / "t2": 4-bit g128 / 2-bit codebook codes)."""
    import ctypes as C
    from glorcq_b200 import _lib
    N, K, r = 1408, 2048, 64
    L = _lib.lib()
    keep, table, g = _c1_problems(dev, P, 7, fmt)
    x = torch.randn(P, K, generator=g, device=dev).half()
    a = (torch.randn(P, r, generator=g, device=dev) * 0.1).half()
    y = torch.empty(P, N, dtype=torch.float16, device=dev)
    m = _lib.MMArgs()
    lib_fmt = {"q2": _lib.FMT_Q2, "q4": _lib.FMT_Q4, "t2": _lib.FMT_T2}[fmt]
    m.fmt, m.group_size, m.epilogue, m.n_problems, m.max_rows, m.rows_stride = lib_fmt, (0 if fmt == "t2" else 128), 0, P, 1, 1
    m.N, m.K, m.rank = N, K, r
    m.w_table = table.data_ptr()
    m.x, m.ldx, m.a0, m.lda, m.y, m.ldy = x.data_ptr(), K, a.data_ptr(), r, y.data_ptr(), N
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(5):
        _lib.check(L.glq_grouped_matmul(C.byref(m), st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        _lib.check(L.glq_grouped_matmul(C.byref(m), st))
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / iters * 1e-3
    # per problem: codes + (scale, zero) pairs + SV + x + a + y  (U is read by the separate x.U kernel)
    if fmt == "t2":       # codes + row norms + SV + x + a + y
        per = N * K // 4 + N * 4 + N * r * 2 + K * 2 + r * 2 + N * 2
    else:
        per = N * K * (4 if fmt == "q4" else 2) // 8 + N * (K // 128) * 4 + N * r * 2 + K * 2 + r * 2 + N * 2
    achieved = P * per / sec / 1e9
    # ncu captures at P = 240 (none for the 4-bit launch)
    t240 = profiled_traffic(f"gemv_stream_kernel_{fmt}_240x1408x2048.md") if fmt in ("q2", "t2") else None
    names = {"q2": ("stream_kernel<Q2,int8 path>", "2-bit g128"), "q4": ("stream_kernel<Q4,int8 path>", "4-bit g128"),
             "t2": ("stream_kernel<T2,int8 path>", "2-bit codebook")}[fmt]
    if os.environ.get("GLQ_NO_I8", "")[:1] == "1":      # the library's switch back to the fp16 path
        names = (names[0].replace("int8 path", "fp16 path"), names[1])
    return {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
            "traffic": None if t240 is None else t240 * P / 240.0,
            "kernel": f"{names[0]} (grouped dequant-GEMV)",
            "launch_us": sec * 1e6, "bytes_per_launch": P * per, "peak_kind": peak_kind,
            "problems": f"{P} x (1408x2048, {names[1]}, rank 64), 1 row each; {P * per / 1e6:.0f} MB > L2"}


def gemm_roofline(dev, P=8, rows=2048, iters=20):
    """The grouped dequant-GEMM (tcgen05 path) alone: P distinct 1408x2048 2-bit g128 rank-64 problems of
    `rows` activation rows each (a prefill-sized grouped launch), x.U given."""
    import ctypes as C
    from glorcq_b200 import _lib
    N, K, r = 1408, 2048, 64
    L = _lib.lib()
    keep, table, g = _c1_problems(dev, P, 11)
    x = torch.randn(P * rows, K, generator=g, device=dev).half()
    a = (torch.randn(P * rows, r, generator=g, device=dev) * 0.1).half()
    y = torch.empty(P * rows, N, dtype=torch.float16, device=dev)
    m = _lib.MMArgs()
    m.fmt, m.group_size, m.epilogue, m.n_problems, m.max_rows, m.rows_stride = _lib.FMT_Q2, 128, 0, P, rows, rows
    m.N, m.K, m.rank, m.total_rows = N, K, r, P * rows
    m.w_table = table.data_ptr()
    m.x, m.ldx, m.a0, m.lda, m.y, m.ldy = x.data_ptr(), K, a.data_ptr(), r, y.data_ptr(), N
    ws = torch.empty(L.glq_mm_workspace_bytes(C.byref(m)) + 256, dtype=torch.uint8, device=dev)
    m.workspace, m.workspace_bytes = (ws.data_ptr() + 255) // 256 * 256, ws.numel() - 256
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        _lib.check(L.glq_grouped_matmul(C.byref(m), st))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        _lib.check(L.glq_grouped_matmul(C.byref(m), st))
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / iters * 1e-3
    flops = P * rows * (2.0 * N * K + 2.0 * N * r)
    peak, kind = measured_peak_tflops()
    ach = flops / sec / 1e12
    return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
            "kernel": "grouped dequant-GEMM on tcgen05 (weights unpacked into tensor memory)", "launch_us": sec * 1e6,
            "flops_per_launch": flops, "peak_kind": kind,
            "problems": f"{P} x (1408x2048, 2-bit g128, rank 64), {rows} rows each"}


def lm_head_roofline(dev, peak_gbs, V=151936, H=2048, iters=30):
    """The output projection alone (fp16 V x H, one row, arg-max folded in)."""
    from glorcq_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    W = (torch.randn(V, H, generator=g, device=dev) * 0.02).half()
    x = torch.randn(1, H, generator=g, device=dev).half()
    logits = torch.empty(1, V, dtype=torch.float16, device=dev)
    best = torch.empty(1, dtype=torch.int64, device=dev)
    ws = torch.empty(L.glq_lm_head_workspace_bytes(), dtype=torch.uint8, device=dev)
    ctr = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def call():
        _lib.check(L.glq_lm_head(x.data_ptr(), H, W.data_ptr(), 1, V, H, logits.data_ptr(), V, best.data_ptr(),
                                 ws.data_ptr(), ws.numel(), ctr.data_ptr(), st))
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        call()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / iters * 1e-3
    nbytes = V * H * 2 + H * 2 + V * 2
    return {"bound": "hbm", "achieved": nbytes / sec / 1e9, "peak": peak_gbs, "unit": "GB/s",
            "frac": nbytes / sec / 1e9 / peak_gbs, "launch_us": sec * 1e6, "bytes_per_launch": nbytes,
            "kernel": "lm_head_kernel (fp16 GEMV + arg-max)", "problems": f"{V} x {H} fp16, 1 row; {nbytes / 1e6:.0f} MB > L2"}


def dropins_vs_reference(dev, P=240):
    """The drop-in GEMV entry points beside the reference's own CUDA kernels built for this GPU (oracle/_ref, when
    present): P distinct C1-shaped problems (one row each; the weights of all of them exceed L2), each arm
    captured as one CUDA graph of P calls and replayed; microseconds per call."""
    from oracle import build_ref
    import glorcq_b200.kernels as GK
    rt, rg = build_ref.load_module("ref_turbo_matmul_cuda"), build_ref.load_module("ref_gptq_matmul_cuda")
    if rt is None or rg is None:
        return {"unavailable": "oracle/_ref holds no build of the reference's kernels (python oracle/build_ref.py)"}
    N, K = 1408, 2048
    g = torch.Generator(device=dev)
    g.manual_seed(21)
    packed = torch.randint(0, 256, (P, N, K // 4), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
    norms = torch.rand(P, N, generator=g, device=dev) + 0.1
    cent = torch.sort(torch.randn(4, generator=g, device=dev))[0] * 0.05
    q8 = torch.randint(0, 4, (P, N, K), generator=g, device=dev, dtype=torch.int32).to(torch.int8)
    sc = (torch.randn(P, N, K // 128, generator=g, device=dev) * 0.02).abs().half()
    zr = torch.randint(0, 4, (P, N, K // 128), generator=g, device=dev).half()
    xh = torch.randn(1, K, generator=g, device=dev).half()
    xf = xh.float()
    empty = torch.empty(0, device=dev)

    def timed(fn):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for i in range(3):
                fn(i)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(P):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * P) * 1e3
    out = {"problems": f"{P} x (1408x2048), 1 row, distinct weights > L2, CUDA graph of {P} calls",
           "turbo_gemv_us": {"ours": timed(lambda i: GK.turbo_dequant_matmul(xh, packed[i], norms[i], cent)),
                             "reference": timed(lambda i: rt.turbo_dequant_matmul(xh, packed[i], norms[i], cent))},
           "gptq_gemv_us": {"ours": timed(lambda i: GK.gptq_dequant_matmul(xf, q8[i], sc[i], zr[i], 128, False, empty)),
                            "reference": timed(lambda i: rg.gptq_dequant_matmul(xf, q8[i], sc[i], zr[i], 128, False, empty))}}
    return out


def _stage(rank, what):
    if os.environ.get("GLQ_BENCH_VERBOSE"):
        print(f"[bench rank {rank}] {what}", file=sys.stderr, flush=True)


def token_bytes(cfg, layers, context, rank_=64):
    """Algorithmic bytes of one decoded token at batch 1: every layer's attention projections (4-bit g128 +
    rank-64 factors), the key/value cache of `context` positions, the MoE block, and the output projection."""
    from glorcq_b200 import synthetic
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or H // nh

    def lin4(N, K):
        return N * K // 2 + 2 * N * ((K + 127) // 128) * 2 + K * rank_ * 2 + N * rank_ * 2 + K * 2 + N * 2
    attn = lin4(nh * hd, H) + 2 * lin4(nkv * hd, H) + lin4(H, nh * hd) + 2 * nkv * hd * context * 2
    E = cfg.get("num_experts", cfg.get("num_local_experts", 0))
    I = cfg.get("moe_intermediate_size", cfg.get("intermediate_size"))
    moe = synthetic.block_bytes_per_token(H=H, I=I, top_k=cfg["num_experts_per_tok"],
                                          I_shared=cfg.get("shared_expert_intermediate_size", 0), rank=rank_, E=E)
    return layers * (attn + moe) + cfg["vocab_size"] * H * 2, layers * moe


def launches_per_token(model):
    """Kernel launches of this library inside one captured decode step, counted from the model's structure:
    per layer the attention side (x.U and product of the grouped q/k/v, attention, x.U and product of the output
    projection, residual + norm) and the MoE block (its own count), plus the output projection."""
    from glorcq_b200.moe_block import GraphCompatibleMoeBlock
    n = 1
    for att, mlp in zip(model.attn, model.mlp):
        n += (2 if att._qkv is not None else 6) + 1 + 2 + 1
        n += mlp.launches_per_call() if isinstance(mlp, GraphCompatibleMoeBlock) else 6
    return n


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from glorcq_b200 import _build, synthetic, tiled
    from glorcq_b200.graph_wrapper import GLoRCQGraphWrapper
    from glorcq_b200.parallel import PeerExchange
    _build.build()
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg, name, prompt = model_config(args.config)
    prompt = args.prompt or prompt
    layers = cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
    ep = world > 1 and not args.replicas
    # expert-parallel degree D: ranks [g*D, (g+1)*D) share one copy of the routed experts (expert e on the group's rank
    # e % D) and step the same D * batch token streams; world / D such groups run side by side on different streams.
    # Default: at most 4, so that a step of one stream per rank (4 tokens) stays inside the persistent block kernel.
    D = 1
    if ep:
        D = args.ep_degree or min(world, 4)
        if world % D != 0:
            raise SystemExit(f"--ep-degree {D} does not divide --gpus {world}")
    G = world // D
    gid, grank = rank // D, rank % D
    grp = None
    if ep and G > 1:
        groups = [dist.new_group(list(range(g * D, (g + 1) * D))) for g in range(G)]   # every rank creates every group
        grp = groups[gid]
    # weak scaling: `args.batch` token streams per rank; every rank of a group holds all of the group's streams
    # (attention, router and shared expert are replicated) and its share of the routed experts
    streams = args.batch * (D if ep and not args.strong else 1)
    K, W = max(1, args.steps), max(3, args.warmup)
    peer_ok = ep and args.exchange == "peer" and streams <= 16
    if peer_ok:
        ok = torch.ones(1, device=dev)
        try:
            PeerExchange.get(grp, dev, 16 * cfg["num_experts_per_tok"], cfg["hidden_size"])
        except Exception as exc:       # noqa: BLE001 - any failure here means "use NCCL"
            _stage(rank, f"peer exchange unavailable: {exc!r}")
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        peer_ok = float(ok) != 0
    model = synthetic.make_decoder(cfg, dev, seed=77, ep_rank=grank if ep else 0, ep_world=D if ep else 1, ep_group=grp,
                                   peer_exchange_max_tokens=16 if peer_ok else 0)
    _stage(rank, "model built")
    if world > 1:
        dist.barrier()          # the first step is a collective: the ranks start it together
    w = GLoRCQGraphWrapper(model, max_batch_size=streams, max_seq_len=prompt + K + W + 24)
    ids = torch.randint(0, cfg["vocab_size"], (streams, prompt), generator=torch.Generator().manual_seed(5 + gid)).to(dev)
    w.capture_graph()
    out, _ = w.generate(ids, max_new_tokens=8)           # the prompt's keys and values, and a first replay
    torch.cuda.synchronize()
    first = out[:, prompt:prompt + 1].contiguous()       # the token decoded from the prompt
    _stage(rank, "captured, prompt processed")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def next_token():
        return w.static_next if w.static_next is not None else torch.argmax(w.static_logits[:, -1, :], dim=-1, keepdim=True)

    def window(steps):
        tok = first
        for i in range(steps):
            w.replay(tok, prompt + i)
            tok = next_token()
        return tok

    window(W)
    if args.profile_window:
        # for `ncu --profile-from-start off`: one window of K steps between cudaProfilerStart / Stop, nothing else
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        window(K)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if rank == 0:
            print(json.dumps({"profile_window": {"steps": K, "launches_per_token": launches_per_token(model)}}), flush=True)
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-resident timing: R windows of exactly K steps ----
    R = max(25, int(math.ceil(0.6 / max(1e-4, K * 1.0e-3))))
    R = min(R, 400)
    times = []
    for _ in range(R):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        window(K)
        e1.record()
        barrier()
        times.append(e0.elapsed_time(e1))
    _stage(rank, "device timing done")
    # ---- end to end: token id from pinned host memory in, next token id back to the host, every step ----
    mine = grank if streams > 1 and ep else 0
    h_in = torch.empty(args.batch if ep else streams, 1, dtype=torch.int64).pin_memory()
    h_out = torch.empty_like(h_in).pin_memory()
    rows = slice(mine * args.batch, (mine + 1) * args.batch) if ep else slice(0, streams)
    own = torch.empty(h_in.shape, dtype=torch.int64, device=dev)
    all_ids = torch.empty(streams, 1, dtype=torch.int64, device=dev)

    def e2e_window(steps):
        h_in.copy_(first[rows].cpu())
        for i in range(steps):
            if ep and not args.strong:
                own.copy_(h_in, non_blocking=True)
                dist.all_gather_into_tensor(all_ids, own, group=grp)
                w.replay(all_ids, prompt + i)
            else:
                all_ids.copy_(h_in, non_blocking=True)
                w.replay(all_ids, prompt + i)
            h_out.copy_(next_token()[rows], non_blocking=True)
            torch.cuda.synchronize()
            h_in.copy_(h_out)
    e2e_window(3)
    e2e_times = []
    for _ in range(max(5, R // 3)):
        barrier()
        t0 = time.perf_counter()
        e2e_window(K)
        barrier()
        e2e_times.append((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop() if rank == 0 else None
    PeerExchange.check_all()

    t = torch.tensor([times, e2e_times + [0.0] * (len(times) - len(e2e_times))], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)       # every window: the slowest rank's time
    ms = float(t[0].median())
    e2e_ms = float(t[1][:len(e2e_times)].median())

    # ---- expert parallel: layer 0's block against an unsharded copy on the same inputs ----
    ep_check = None
    if ep and rank == 0:
        single = synthetic.make_decoder({**cfg, "num_hidden_layers": 1}, dev, seed=77).mlp[0]
        hx = torch.randn(1, streams, cfg["hidden_size"], device=dev, dtype=torch.float16,
                         generator=torch.Generator(device=dev).manual_seed(11))
        ref_y = single(hx)[0]
        del single
    if ep:
        hx = torch.randn(1, streams, cfg["hidden_size"], device=dev, dtype=torch.float16,
                         generator=torch.Generator(device=dev).manual_seed(11))
        barrier()
        with torch.no_grad():
            got = model.mlp[0](hx)[0]
        torch.cuda.synchronize()
        if rank == 0:
            ep_check = {"layer0_block_bit_equal_to_unsharded": bool(torch.equal(got, ref_y)), "tokens": streams}

    # ---- the MoE blocks alone ----
    moe_only = None
    if rank == 0 and world == 1 and not args.no_extras:
        moe_only = moe_blocks_alone(model, dev, cfg, layers)
    err = tiled.debug_error()
    if rank == 0:
        peak, kind = measured_peak_gbs()
        roof = gemv_roofline(dev, peak, kind)
        extras = {}
        if not args.no_extras:
            extras["roofline_t2"] = gemv_roofline(dev, peak, kind, fmt="t2")     # the same launch on 2-bit codebook codes
            extras["roofline_gemm"] = gemm_roofline(dev)
            extras["roofline_lm_head"] = lm_head_roofline(dev, peak, cfg["vocab_size"], cfg["hidden_size"])
            try:
                extras["dropins_vs_reference_kernels"] = dropins_vs_reference(dev)
            except Exception as exc:      # noqa: BLE001 - a side leg must not take the line down
                extras["dropins_vs_reference_kernels"] = {"unavailable": repr(exc)[:200]}
        cpu = None
        if world == 1:      # the CPU leg is timed at N = 1 only
            sec_tok, threads, reps = CpuToken(cfg, prompt).seconds(8.0, 100)
            cpu = {"value": 1.0 / sec_tok, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"one token: 1 of {layers} layers (4 attention projections, attention over {prompt} cached positions, "
                             f"MoE block) and the output projection through the CPU oracle, median of {reps} forwards; "
                             f"tok/s = 1 / ({layers} x layer + output projection)"}
        bytes_tok, bytes_moe = token_bytes(cfg, layers, prompt + K // 2)
        total_streams = streams * (G if ep else 1)
        value = total_streams * K / (ms * 1e-3)
        conf = workload_config(cfg, name, prompt, args.batch, layers)
        conf.update({"parallelism": "single GPU" if world == 1 else
                     (f"expert parallel ep{D}" + (f" x {G} groups of {D} GPUs (each group one copy of the routed experts)" if G > 1 else "")
                      + f": expert e on rank e % {D}" + (" of its group" if G > 1 else "") + "; attention, router, shared expert and output "
                      f"projection replicated; " + ("exchange kernel over peer memory (peer stores + flags)" if peer_ok else
                                                    "NCCL all-reduce of the per-entry outputs") + f" once per block; {streams} token stream(s) per step"
                      + (f" and group, {total_streams} in all" if G > 1 else "")
                      if ep else f"replicas x{world}"),
                     "batch": total_streams, "windows": R, "window_ms_min_median_max": [min(times), ms, max(times)],
                     "algorithmic_bytes_per_token": bytes_tok,
                     "token_hbm_frac_of_peak": bytes_tok * K / (ms * 1e-3) / 1e9 / peak})
        nl = launches_per_token(model)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
                "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
                "scaling": "strong" if ep and args.strong else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": conf,
                "e2e": {"value": total_streams * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 8 * h_in.numel(),
                        "d2h_bytes_per_step": 8 * h_out.numel()},
                "gpu_launches": K * nl, "launches_per_token": nl,
                "roofline": roof, **extras, "moe_only": moe_only,
                "cpu_baseline": cpu, "clocks": clocks, "kernel_self_check": err}
        if ep:
            line["exchange"] = {"kind": "peer" if peer_ok else "nccl", "waits_run_out": 0}
            line["ep_check"] = ep_check
        print(json.dumps(line), flush=True)
    if world > 1:
        # all ranks leave together (rank 0 was busy with the roofline legs); a teardown that does not return
        # must not keep the launcher waiting
        dist.barrier()
        del w
        torch.cuda.synchronize()
        sys.stdout.flush()
        tm = threading.Timer(20.0, os._exit, (0,))
        tm.daemon = True
        tm.start()
        dist.destroy_process_group()


def prefill_alone(dev, cfg, prompt, reps=5, profile=False):
    """The prompt pass of the whole decoder alone (batch 1, eager, as `generate` runs it): every quantized product
    goes through the tcgen05 dequant-GEMM, experts grouped by the device-side routing.  Tokens per second and the
    rate of the quantized products' arithmetic (2 flops per weight of every projection a token passes through)."""
    from glorcq_b200 import synthetic
    from glorcq_b200.graph_wrapper import GLoRCQGraphWrapper
    model = synthetic.make_decoder(cfg, dev, seed=77)
    w = GLoRCQGraphWrapper(model, max_batch_size=1, max_seq_len=prompt + 32)
    ids = torch.randint(0, cfg["vocab_size"], (1, prompt), generator=torch.Generator().manual_seed(5)).to(dev)
    w._set_moe_graph_mode(False)
    kw = {"logits_to_keep": 1} if w._keep_last_only else {}

    def run():
        w.static_cache.reset()
        return w.model(input_ids=ids, cache_position=torch.arange(prompt, device=dev), past_key_values=w.static_cache,
                       use_cache=True, return_dict=False, **kw)[0]
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    if profile:        # for `ncu --profile-from-start off`: one prompt pass between cudaProfilerStart / Stop
        torch.cuda.profiler.start()
        run()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = sorted(times)[len(times) // 2]
    H, k = cfg["hidden_size"], cfg["num_experts_per_tok"]
    I = cfg.get("moe_intermediate_size", cfg.get("intermediate_size"))
    Is = cfg.get("shared_expert_intermediate_size", 0) or 0
    nh = cfg["num_attention_heads"]
    nkv, hd = cfg.get("num_key_value_heads") or nh, cfg.get("head_dim") or H // nh
    per_tok = 2.0 * (H * hd * (2 * nh + 2 * nkv) + 3 * H * I * k + 3 * H * Is)
    layers = cfg["num_hidden_layers"]
    peak, kind = measured_peak_tflops()
    tf = per_tok * layers * prompt / (ms * 1e-3) / 1e12
    return {"prompt_tokens": prompt, "ms": ms, "tok_s": prompt / (ms * 1e-3), "quantized_products_tflops": tf,
            "frac_of_bf16_peak": tf / peak, "peak_kind": kind, "layers": layers,
            "note": "whole prompt pass incl. attention (glq_attn_prefill below 2048 tokens, the library call from there), "
                    "norms, routing and the output projection of the last token"}


def moe_blocks_alone(model, dev, cfg, layers, steps=100):
    """One token through the decoder's MoE blocks alone, each block's output feeding the next through the fused
    residual-free RMS norm, replayed from one CUDA graph: the part of a token the quantized expert path owns."""
    from glorcq_b200 import synthetic
    from glorcq_b200.moe_block import GraphCompatibleMoeBlock
    blocks = [m for m in model.mlp if isinstance(m, GraphCompatibleMoeBlock)]
    if not blocks:
        return None
    H = cfg["hidden_size"]
    gx = torch.Generator(device=dev)
    gx.manual_seed(4242)
    static_x = torch.randn(1, 1, H, device=dev, dtype=torch.float16, generator=gx)
    eps = torch.finfo(torch.float16).eps

    def token(x):
        for blk in blocks:
            _, _, x = blk(x, next_norm=(None, eps))
        return x
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s), torch.no_grad():
        for _ in range(2):
            token(static_x)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad():
        static_y = token(static_x)
    for _ in range(5):
        static_x.copy_(static_y)
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        static_x.copy_(static_y)
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    E = cfg.get("num_experts", cfg.get("num_local_experts", 0))
    I = cfg.get("moe_intermediate_size", cfg.get("intermediate_size"))
    nbytes = len(blocks) * synthetic.block_bytes_per_token(H=H, I=I, top_k=cfg["num_experts_per_tok"],
                                                           I_shared=cfg.get("shared_expert_intermediate_size", 0), rank=64, E=E)
    peak, _ = measured_peak_gbs()
    return {"value": 1e3 / ms, "unit": UNIT, "ms_per_token": ms, "us_per_block": ms * 1e3 / len(blocks), "blocks": len(blocks),
            "launches_per_block": blocks[0].launches_per_call(), "algorithmic_bytes_per_token": nbytes,
            "hbm_frac_of_peak": nbytes / (ms * 1e-3) / 1e9 / peak}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="qwen15", choices=["qwen15", "mixtral", "qwen3"],
                    help="decoder shape: Qwen1.5-MoE-A2.7B (default), Mixtral-8x7B or Qwen3-30B-A3B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--batch", type=int, default=1, help="token streams per rank")
    ap.add_argument("--prompt", type=int, default=0, help="prompt length (0: the configuration's)")
    ap.add_argument("--prefill-only", action="store_true",
                    help="time the prompt pass of the whole decoder alone (--prompt tokens, default 4096; batch 1)")
    ap.add_argument("--gemv-fmt", choices=["q2", "q4", "t2"], default="q2",
                    help="with --gemv-only: 2-bit g128 codes (default), 4-bit g128 codes or 2-bit codebook codes")
    ap.add_argument("--gemv-only", action="store_true",
                    help="time only the grouped dequant-GEMV roofline case (small enough for an ncu capture)")
    ap.add_argument("--gemm-only", action="store_true",
                    help="time only the grouped tcgen05 dequant-GEMM roofline case (small enough for an ncu capture)")
    ap.add_argument("--lm-head-only", action="store_true", help="time only the output projection kernel")
    ap.add_argument("--moe-only", action="store_true", help="time only the MoE blocks of the model (moe_only of the line)")
    ap.add_argument("--profile-window", action="store_true",
                    help="run one window of --steps tokens between cudaProfilerStart and cudaProfilerStop and exit "
                         "(for ncu --profile-from-start off)")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMM / lm_head roofline legs and moe_only")
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--problems", type=int, default=240)
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the per-block exchange, this library's peer-memory kernel or NCCL's all-reduce")
    ap.add_argument("--strong", action="store_true",
                    help="with --gpus N > 1: the same token streams for all ranks (strong scaling) instead of --batch per rank")
    ap.add_argument("--ep-degree", type=int, default=0,
                    help="with --gpus N > 1: GPUs that share one copy of the routed experts (N / degree groups run side by "
                         "side); default min(N, 4)")
    ap.add_argument("--replicas", action="store_true",
                    help="with --gpus N > 1: N independent copies of the model instead of expert parallelism")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.prefill_only:
        from glorcq_b200 import _build
        _build.build()
        dev = torch.device("cuda:0")
        torch.cuda.set_device(dev)
        cfg, name, prompt = model_config(args.config)
        cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
        print(json.dumps({"prefill": {"model": name, **prefill_alone(dev, cfg, args.prompt or 4096, reps=max(3, args.steps), profile=args.profile_window)}}),
              flush=True)
        return
    if args.gemv_only or args.gemm_only or args.lm_head_only or args.moe_only:
        from glorcq_b200 import _build, synthetic
        _build.build()
        dev = torch.device("cuda:0")
        peak, kind = measured_peak_gbs()
        if args.gemv_only:
            out = {"roofline": gemv_roofline(dev, peak, kind, P=args.problems, iters=max(1, args.steps), fmt=args.gemv_fmt)}
        elif args.gemm_only:
            P = args.problems if args.problems != 240 else 8
            out = {"roofline_gemm": gemm_roofline(dev, P=P, rows=args.rows, iters=max(1, args.steps))}
        elif args.lm_head_only:
            out = {"roofline_lm_head": lm_head_roofline(dev, peak, iters=max(1, args.steps))}
        else:
            cfg, name, prompt = model_config(args.config)
            cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
            torch.cuda.set_device(dev)
            model = synthetic.make_decoder(cfg, dev, seed=77)
            out = {"moe_only": moe_blocks_alone(model, dev, cfg, cfg["num_hidden_layers"], steps=max(1, args.steps))}
        print(json.dumps(out), flush=True)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
