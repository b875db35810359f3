"""Benchmark of the GLoRCQ real-quant decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Workload (one GPU): batch-1 decode through the MoE blocks of the Qwen1.5-MoE-A2.7B-shaped model --
24 layers of {router, 60 experts top-4 (intermediate 1408), shared expert (5632)}, every projection
2-bit g128 with a rank-64 low-rank correction whose input-side factor U is shared by clustered
experts across layers -- on seeded synthetic weights.  One step = one token through all layers, the
output of a block feeding the next, replayed from one CUDA graph.  The weights of the 24 layers
(5.7 GB) are far larger than L2, and every token touches ~0.67 GB of them.

One JSON line on stdout:
  value     tokens/s with the hidden state resident in HBM (device-timed with CUDA events)
  e2e       the same through the public API with pinned host buffers: h2d of the hidden state, graph
            replay, d2h of the block output, every step
  roofline  the dominant kernel (the grouped dequant-GEMV) timed alone, live, on 240 distinct
            expert-projection problems (1408 x 2048, 2-bit g128, rank 64; 240 MB, larger than L2):
            algorithmic bytes / CUDA-event time against the measured HBM peak
  cpu_baseline  the CPU restatement of the reference's own path (oracle/), timed on the host cores on
            a bounded sample (one layer, one token, repeated)
`--impl reference` times that CPU path as the main line (rank 0 only).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

CFG = dict(H=2048, I=1408, E=60, top_k=4, I_shared=5632, rank=64, experts_per_cluster=4)
METRIC = "moe_decode_tok_s"
UNIT = "tok/s"


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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


# ---- CPU baseline (reference arm) -----------------------------------------------------------------
def cpu_layer_seconds(sample_seconds=12.0, max_reps=200):
    """One layer, one token, through the CPU oracle (the reference's PyTorch path restated); returns
    (median seconds per layer-forward, threads, reps)."""
    from oracle import glorcq_oracle as O
    from tests import cases
    torch.set_num_threads(os.cpu_count() or 1)
    blk = cases.make_moe(2001, CFG["H"], CFG["I"], CFG["E"], CFG["top_k"], I_shared=CFG["I_shared"], rank=CFG["rank"],
                         experts_per_cluster=CFG["experts_per_cluster"])
    ob = cases.to_oracle_moe(blk)
    x = cases.make_x(3001, 1, CFG["H"]).reshape(1, 1, CFG["H"])
    with torch.no_grad():
        for _ in range(2):
            O.moe_forward(ob, x)
        ts, t_start = [], time.perf_counter()
        while len(ts) < max_reps and (time.perf_counter() - t_start < sample_seconds or len(ts) < 3):
            t0 = time.perf_counter()
            O.moe_forward(ob, x)
            ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2], torch.get_num_threads(), len(ts)


def run_reference(args, rank):
    if rank != 0:
        return
    layers = args.layers
    per = []
    sec, threads, reps = cpu_layer_seconds(sample_seconds=3.0, max_reps=5)      # warm-up sample
    for _ in range(max(1, args.steps)):
        sec, threads, reps = cpu_layer_seconds(sample_seconds=8.0 / max(1, args.steps) + 1.0, max_reps=50)
        per.append(sec)
    per.sort()
    sec = per[len(per) // 2]
    value = 1.0 / (sec * layers)
    sample = f"1 of {layers} layers, 1 token, median of repeated CPU forwards; tok/s = 1 / ({layers} x layer time)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * layers * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(layers),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(layers):
    return {"workload": f"Qwen1.5-MoE-A2.7B-shaped MoE decode, one token stream per GPU: {layers} MoE blocks (hidden 2048, 60 experts "
                        "top-4 x 1408, shared expert 5632), 2-bit g128 + rank-64 shared-U correction; attention "
                        "and lm_head not included", "layers": layers, "batch": 1,
            "l2": "weights (240 MB per layer) far exceed L2; each token reads other experts' weights of 24 distinct layers"}


# ---- GPU arm ----------------------------------------------------------------------------------------
def gemv_roofline(dev, peak_gbs, peak_kind, P=240, iters=50):
    """The grouped dequant-GEMV alone: P distinct 1408x2048 2-bit g128 rank-64 problems, one row each."""
    import ctypes as C
    from glorcq_b200 import _lib
    from glorcq_b200.tiled import TiledWeight
    N, K, r = 1408, 2048, 64
    L = _lib.lib()
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    keep, descs = [], []
    for _ in range(P):
        tw = TiledWeight.from_gptq(torch.randint(0, 4, (N, K), generator=g, device=dev, dtype=torch.int32),
                                   (torch.randn(N, K // 128, generator=g, device=dev) * 0.02).abs().half(),
                                   torch.randint(0, 4, (N, K // 128), generator=g, device=dev).half(), 2, 128)
        tw.put_sv(0, (torch.randn(N, r, generator=g, device=dev) * 0.01).half())
        keep.append(tw)
        descs.append(tw.desc_bytes())
    table = torch.frombuffer(bytearray(b"".join(descs)), dtype=torch.uint8).to(dev)
    x = torch.randn(P, K, generator=g, device=dev).half()
    a = (torch.randn(P, r, generator=g, device=dev) * 0.1).half()
    y = torch.empty(P, N, dtype=torch.float16, device=dev)
    m = _lib.MMArgs()
    m.fmt, m.group_size, m.epilogue, m.n_problems, m.max_rows, m.rows_stride = _lib.FMT_Q2, 128, 0, P, 1, 1
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
    per = N * K // 4 + N * (K // 128) * 4 + N * r * 2 + K * 2 + r * 2 + N * 2
    achieved = P * per / sec / 1e9
    # DRAM bytes of one launch of this case from the ncu capture summarised under profiles/
    # (dram__bytes_read.sum + dram__bytes_write.sum = 239.47 MB + 4.13 MB at P = 240); scaled by P otherwise
    traffic = 243.60e6 * P / 240.0
    return {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
            "traffic": traffic, "kernel": "stream_kernel<Q2,int8 path> (grouped dequant-GEMV)",
            "launch_us": sec * 1e6, "bytes_per_launch": P * per, "peak_kind": peak_kind,
            "problems": f"{P} x (1408x2048, 2-bit g128, rank 64), 1 row each; {P * per / 1e6:.0f} MB > L2"}


def _stage(rank, what):
    if os.environ.get("GLQ_BENCH_VERBOSE"):
        print(f"[bench rank {rank}] {what}", file=sys.stderr, flush=True)


def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def gemm_roofline(dev, P=8, rows=2048, iters=20):
    """The grouped dequant-GEMM (tcgen05 path) alone: P distinct 1408x2048 2-bit g128 rank-64 problems of
    `rows` activation rows each (a prefill-sized grouped launch), x.U given."""
    import ctypes as C
    from glorcq_b200 import _lib
    from glorcq_b200.tiled import TiledWeight
    N, K, r = 1408, 2048, 64
    L = _lib.lib()
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    keep, descs = [], []
    for _ in range(P):
        tw = TiledWeight.from_gptq(torch.randint(0, 4, (N, K), generator=g, device=dev, dtype=torch.int32),
                                   (torch.randn(N, K // 128, generator=g, device=dev) * 0.02).abs().half(),
                                   torch.randint(0, 4, (N, K // 128), generator=g, device=dev).half(), 2, 128)
        tw.put_sv(0, (torch.randn(N, r, generator=g, device=dev) * 0.01).half())
        keep.append(tw)
        descs.append(tw.desc_bytes())
    table = torch.frombuffer(bytearray(b"".join(descs)), dtype=torch.uint8).to(dev)
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
            "kernel": "tc_pack_b_kernel + tc_ts_kernel<Q2> (grouped dequant-GEMM, tcgen05, weights unpacked into TMEM)", "launch_us": sec * 1e6,
            "flops_per_launch": flops, "peak_kind": kind,
            "problems": f"{P} x (1408x2048, 2-bit g128, rank 64), {rows} rows each"}


def run_full_model(args):
    """BASELINE config 3: the whole Qwen1.5-MoE-A2.7B-shaped decoder (attention 4-bit g128, experts 2-bit
    rank 64 with 128 random cross-layer U clusters, fp16 lm_head), 512-token prefill then 256 greedy decode
    steps replayed from one CUDA graph.  Printed as its own JSON line (not the driver's metric line)."""
    from glorcq_b200 import _build, synthetic
    from glorcq_b200.graph_wrapper import GLoRCQGraphWrapper
    _build.build()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    cfg = dict(synthetic.QWEN15_MOE_A27B)
    cfg["num_hidden_layers"] = args.layers
    model = synthetic.make_decoder(cfg, dev, seed=77)
    w = GLoRCQGraphWrapper(model, max_batch_size=1, max_seq_len=1024)
    ids = torch.randint(0, cfg["vocab_size"], (1, args.prompt), generator=torch.Generator().manual_seed(5)).to(dev)
    w.capture_graph()
    w.generate(ids, max_new_tokens=8)                   # warm-up of prefill and replay
    out, seconds = w.generate(ids, max_new_tokens=args.new_tokens)
    line = {"full_model": {"workload": f"Qwen1.5-MoE-A2.7B-shaped decoder, {args.layers} layers, prompt {args.prompt}, "
                                       f"{args.new_tokens} greedy tokens, CUDA graph decode",
                           "decode_tok_s": (args.new_tokens - 1) / w.last_decode_seconds,
                           "prefill_tok_s": args.prompt / w.last_prefill_seconds,
                           "prefill_s": w.last_prefill_seconds, "decode_s": w.last_decode_seconds, "total_s": seconds,
                           "generated": int(out.shape[1] - ids.shape[1])}}
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from glorcq_b200 import _build, synthetic, tiled
    _build.build()
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    layers = args.layers
    pools = {}
    # N > 1: the experts of every block are sharded over the ranks (expert e on rank e % N); router and
    # shared expert are replicated; one all-reduce of the per-entry outputs per block (--replicas: N
    # independent copies of the whole model instead)
    ep = world > 1 and not args.replicas
    blocks = [synthetic.make_moe_block(1000 + l, dev, pools=pools, ep_rank=rank if ep else 0,
                                       ep_world=world if ep else 1, **CFG) for l in range(layers)]
    _stage(rank, "blocks built")
    H = CFG["H"]
    # the exchange: this library's kernel over peer-mapped memory (peer stores + flags), or NCCL's all-reduce
    # when asked for or when the symmetric allocation is not to be had on every rank
    peer = None
    if ep and args.exchange == "peer":
        from glorcq_b200 import parallel
        ok = torch.ones(1, device=dev)
        try:
            peer = parallel.PeerExchange.get(None, dev, 16 * CFG["top_k"], H)
        except Exception as exc:       # noqa: BLE001 - any failure here means "use NCCL"
            _stage(rank, f"peer exchange unavailable: {exc!r}")
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0:
            peer = None
        for blk in blocks:
            blk.peer_exchange_max_tokens = 16 if peer is not None else 0
    # weak scaling: one token stream per rank, so a step decodes `batch` = N tokens; every rank holds all
    # N hidden states (the replicated router and shared expert see them all) and its share of the experts
    batch = world if ep and not args.strong else 1
    gx = torch.Generator(device=dev)
    gx.manual_seed(4242)
    static_x = torch.randn(1, batch, H, device=dev, dtype=torch.float16, generator=gx)
    x0 = static_x.clone()
    mine = rank if batch > 1 else 0

    def token(x):
        # the decoder's RMS norm between blocks keeps every layer's input at unit scale; it runs inside the
        # block's combine kernel (same arithmetic as torch's rms_norm on the block output)
        eps = torch.finfo(torch.float16).eps
        for blk in blocks:
            _, _, x = blk(x, next_norm=(None, eps))
        return x

    # warm-up outside capture (builds workspaces), then capture one token
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s), torch.no_grad():
        for _ in range(2):
            token(static_x)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    if peer is not None:
        bad = torch.tensor([float(peer.error() != 0)], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if float(bad) != 0:            # a wait ran out during warm-up: do not time that
            _stage(rank, "peer exchange: a wait ran out in warm-up, using NCCL")
            peer = None
            for blk in blocks:
                blk.peer_exchange_max_tokens = 0
            with torch.no_grad():
                token(static_x)
            torch.cuda.synchronize()
    _stage(rank, "eager warm-up done")
    if args.no_graph:
        class _Eager:
            def replay(self):
                with torch.no_grad():
                    static_y.copy_(token(static_x))
        with torch.no_grad():
            static_y = token(static_x).clone()
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            static_y = token(static_x)
    _stage(rank, "captured")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    for _ in range(max(3, args.warmup)):
        static_x.copy_(static_y)
        graph.replay()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        static_x.copy_(static_y)     # next token's hidden state stays on the device
        graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    _stage(rank, f"device timing done: {ms:.2f} ms")
    # ---- end to end: pinned host in, host out, every step ----
    # every rank owns one token stream: its hidden state comes from its pinned host buffer, the ranks
    # exchange the rows (all-gather, N > 1), the graph runs, the rank's own output row goes back
    hx = torch.empty(1, H, dtype=torch.float16).pin_memory()
    hy = torch.empty(1, H, dtype=torch.float16).pin_memory()
    hx.copy_(x0[0, mine:mine + 1].cpu())
    own = torch.empty(1, H, dtype=torch.float16, device=dev)

    def e2e_step():
        if batch > 1:
            own.copy_(hx, non_blocking=True)
            dist.all_gather_into_tensor(static_x.view(batch, H), own)
        else:
            static_x.view(1, H).copy_(hx, non_blocking=True)
        graph.replay()
        hy.copy_(static_y.view(batch, H)[mine:mine + 1], non_blocking=True)
        torch.cuda.synchronize()
        hx.copy_(hy)
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    err = tiled.debug_error()
    if rank == 0:
        peak, kind = measured_peak_gbs()
        roof = gemv_roofline(dev, peak, kind)
        roof_gemm = gemm_roofline(dev)
        cpu = None
        if world == 1:      # the CPU leg is timed at N=1 only
            sec_layer, threads, reps = cpu_layer_seconds()
            cpu = {"value": 1.0 / (sec_layer * layers), "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"1 of {layers} layers, 1 token, median of {reps} CPU forwards of the oracle"}
        bytes_tok = synthetic.block_bytes_per_token(**{k: CFG[k] for k in ("H", "I", "top_k", "I_shared", "rank", "E")}) * layers
        streams = batch if ep else world      # token streams decoded at once
        value = streams * args.steps / (ms * 1e-3)
        cfg = workload_config(layers)
        cfg.update({"parallelism": "single GPU" if world == 1 else
                    (f"expert parallel ep{world}: expert e on rank e % {world}, router and shared expert replicated, "
                     + ("exchange kernel over peer memory (peer stores + flags)" if peer is not None else
                        "NCCL all-reduce of the per-entry outputs") + f" once per block; {batch} token stream(s) per step"
                     if ep else f"replicas x{world}"),
                    "batch": batch,
                    "algorithmic_bytes_per_token": bytes_tok,
                    "token_hbm_frac_of_peak": bytes_tok * args.steps / (ms * 1e-3) / 1e9 / peak})
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong" if ep and batch == 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": cfg,
                "e2e": {"value": streams * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": H * 2,
                        "d2h_bytes_per_step": H * 2},
                "gpu_launches": args.steps * layers * (11 if peer is not None else 10),
                "roofline": roof, "roofline_gemm": roof_gemm,
                "cpu_baseline": cpu,
                "clocks": clocks, "kernel_self_check": err}
        if ep:
            line["exchange"] = {"kind": "peer" if peer is not None else "nccl",
                                "waits_run_out": None if peer is None else int(peer.error() != 0)}
        print(json.dumps(line), flush=True)
    if world > 1:
        # all ranks leave together (rank 0 was busy with the roofline and CPU legs); a teardown that does
        # not return must not keep the launcher waiting
        dist.barrier()
        del graph
        torch.cuda.synchronize()
        sys.stdout.flush()
        t = threading.Timer(20.0, os._exit, (0,))
        t.daemon = True
        t.start()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--gemv-only", action="store_true",
                    help="time only the grouped dequant-GEMV roofline case (small enough for an ncu capture)")
    ap.add_argument("--full-model", action="store_true",
                    help="time the whole decoder (prefill + graph decode) instead of the MoE-block metric line")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--gemm-only", action="store_true",
                    help="time only the grouped tcgen05 dequant-GEMM roofline case (small enough for an ncu capture)")
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--problems", type=int, default=240)
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: the per-block exchange, this library's peer-memory kernel or NCCL's all-reduce")
    ap.add_argument("--strong", action="store_true",
                    help="with --gpus N > 1: one token stream for all ranks (strong scaling) instead of one per rank")
    ap.add_argument("--replicas", action="store_true",
                    help="with --gpus N > 1: N independent copies of the model instead of expert parallelism")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.gemv_only:
        from glorcq_b200 import _build
        _build.build()
        peak, kind = measured_peak_gbs()
        print(json.dumps({"roofline": gemv_roofline(torch.device("cuda:0"), peak, kind, P=args.problems,
                                                     iters=max(1, args.steps))}), flush=True)
        return
    if args.full_model:
        run_full_model(args)
        return
    if args.gemm_only:
        from glorcq_b200 import _build
        _build.build()
        P = args.problems if args.problems != 240 else 8
        print(json.dumps({"roofline_gemm": gemm_roofline(torch.device("cuda:0"), P=P, rows=args.rows,
                                                          iters=max(1, args.steps))}), flush=True)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
