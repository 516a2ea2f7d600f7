#!/usr/bin/env python
"""Benchmark of the tensor-parallel decoder-layer path.

    python bench.py --gpus N --steps K --warmup W            # this library, TP = N
    python bench.py --impl reference --gpus N --steps K ...  # CPU arm (oracle port of the reference path)

A step = one Llama-3-8B-shaped decoder layer (hidden 4096,
32 q / 8 kv heads, head_dim 128, intermediate 14336, bf16) over one Sarathi
mixed chunk of 512 tokens (448 prefill + 64 decode), tensor-parallel over N
GPUs, attention replaced by the stand-in attn_out = q (attention is outside
the path).  Inputs are seeded synthetic tensors (sarathi_serve_b200.synthetic).

`value`   : tokens/s of the device-resident layer (4 kernels per step at N > 1: qkv GEMM+rotary,
            o_proj GEMM+all-reduce+residual+RMSNorm, gate_up GEMM+SiLU*mul,
            down GEMM+all-reduce+residual+next RMSNorm; at N = 1, where nothing is exchanged, the two
            row-parallel GEMMs are each followed by the add+RMSNorm kernel: 6 kernels), all timed steps
            in one CUDA graph, CUDA-event timed, max over ranks.
`gpu_comparison`: the same step as the reference runs it on a GPU (cuBLAS GEMMs, separate rotary /
            SiLU*mul / add+RMSNorm kernels, NCCL all-reduce), same graph timing.
`e2e`     : tokens/s through the public layer API with HOST buffers: every step uploads its hidden states
            and positions from pinned host memory, runs LlamaDecoderLayer.forward (captured once per layer in a
            CUDA graph, graph_runner.LayerGraph) and brings its result back to pinned host memory, where the
            host waits for it.  graph_runner.HostPipeline keeps three steps in flight: the upload of step i+1
            and the download of step i-1 run on copy streams under the kernels of step i.  At N > 1 every rank
            moves its T/N token rows over PCIe and the full input is assembled over NVLink inside the graph
            (shard_host_io).
`roofline`: the dominant kernel (gate_up GEMM + SiLU*mul), timed alone with CUDA events.
Weights of several distinct layers are cycled so that each step's operands exceed the L2.
One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tp_decoder_layer_tokens_per_s"
UNIT = "tokens/s"
L2_BYTES = 126 << 20


# dram__bytes_read.sum + dram__bytes_write.sum of one gate_up launch at TP=1 (ncu --set full capture,
# summarised in profiles/gemm_gate_up_silu_tp1_ncu_full.md)
GATE_UP_TP1_DRAM_BYTES = 256.7e6


def workload_text(name: str, world: int) -> str:
    return (f"{name}: Llama-3-8B-shaped decoder layer (hidden 4096, 32q/8kv heads, head_dim 128, intermediate 14336), "
            f"512-token mixed chunk (448 prefill + 64 decode), TP={world}, attention stand-in attn_out=q")


NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool's B200s (nominal 900)


def layer_roofline(case, T: int, world: int, peak_tf: float, peak_hbm: float) -> dict:
    """Lower bound of one layer step per GPU: the slowest of dense FLOPs at the bf16 peak, bytes at the HBM
    copy bandwidth (each tensor crossing HBM once) and all-reduce bytes at the NVLink bandwidth
    (2 all-reduces x 2 (tp-1)/tp T H s per direction)."""
    H, I, hd = case.hidden_size, case.intermediate_size, case.head_dim
    nq, nkv, s = case.num_heads, case.num_kv_heads, 2
    flops = 2.0 * T * H * ((nq + 2 * nkv) * hd + nq * hd + 3 * I) / world
    hbm = s * H * ((nq + 2 * nkv) * hd + nq * hd + 3 * I) / world + s * T * (
        2 * H + (nq + 2 * nkv) * hd / world + nq * hd / world + 2 * I / world + 2 * H + 4 * H)
    nvl = 2 * 2.0 * (world - 1) / world * T * H * s
    t = {"compute_us": flops / (peak_tf * 1e12) * 1e6, "hbm_us": hbm / (peak_hbm * 1e9) * 1e6,
         "nvlink_us": nvl / (NVLINK_GBS * 1e9) * 1e6}
    t["t_roof_us"] = max(t.values())
    t["flops"], t["hbm_bytes"], t["nvlink_bytes_per_direction"] = flops, hbm, nvl
    return t


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="config2")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parts", action="store_true",
                    help="instead of the step benchmark: time every kernel of the path on its own (CUDA graphs) and "
                         "print one JSON line of per-kernel times with achieved TFLOP/s, HBM GB/s and NVLink GB/s")
    ap.add_argument("--kernel-pass", action="store_true",
                    help="with --parts: launch every kernel of the path twice, eagerly, at the workload's shapes and "
                         "exit -- the short program a profiler is pointed at (one GPU)")
    ap.add_argument("--tune-cache", default=None,
                    help="JSON file of tile configurations: read if present (no tuning launches), else written")
    ap.add_argument("--cpu-baseline-seconds", type=float, default=15.0)
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU arm
def cpu_layer_runner(case, threads: int):
    """Returns (fn, tokens): fn() runs the oracle port of the reference layer path once on the CPU."""
    import torch
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import synthetic as S
    torch.set_num_threads(threads)
    t = S.generate(case)
    params = [S.shard(t, 0, 1)]
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    x = t.x.to(case.dtype)

    def fn():
        with torch.inference_mode():
            return O.decoder_layer(params, x, t.positions, num_heads=case.num_heads, num_kv_heads=case.num_kv_heads,
                                   head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache)["out"]
    return fn, case.num_tokens


def time_cpu(case, budget_s: float, warmup: int = 1, max_iters: int = 50, min_iters: int = 2):
    threads = os.cpu_count() or 1
    fn, tokens = cpu_layer_runner(case, threads)
    for _ in range(warmup):
        fn()
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max_iters and (len(times) < min_iters or time.perf_counter() < t_end):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return tokens / med, threads, len(times), med


def bench_config(workload: str, world: int, tokens: int) -> dict:
    """The `config` object of the JSON line: the same in both arms."""
    return {"workload": workload_text(workload, world), "tokens_per_step": tokens, "parallelism": f"tp{world}"}


def run_reference_arm(a):
    """The reference's path on the host cores: the oracle port (torch CPU kernels, bf16, all host
    threads) of LlamaDecoderLayer over the same workload, every shard of the layer in one process;
    rank 0 only.  A step = one full pass of the workload (about 30 ms), so `--steps` / `--warmup` are
    taken as given."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from sarathi_serve_b200 import synthetic as S
    case = S.CASES[a.workload]
    threads = os.cpu_count() or 1
    fn, tokens = cpu_layer_runner(case, threads)
    steps, warm = max(1, a.steps), max(0, a.warmup)
    for _ in range(warm):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    v = tokens / dt
    line = {"metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": steps, "warmup": warm,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": bench_config(a.workload, a.gpus, tokens),
            "how": "oracle port of the reference layer path, one process on the host cores (the whole layer, all "
                   "shards)",
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{steps} full layer passes of the workload"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------- native arm
PARITY_TOL = 2e-2  # bf16: max|a - b| / max|ref| per tensor


def check_parity(case, t, world, rank, dev, step_resident, runner0, layers, max_over_ranks, pipelined_out=None) -> dict:
    import torch
    from oracle import tp_layer_oracle as O
    from sarathi_serve_b200 import synthetic as S
    T = case.num_tokens
    normed, resid = step_resident(0)
    normed, resid = normed.clone(), resid.clone()
    host_out = runner0.replay_host_io()
    torch.cuda.current_stream().synchronize()
    e2e_out = host_out.clone()
    shards = [S.shard(t, r, world) for r in range(world)]
    cache = O.cos_sin_cache(case.head_dim, case.head_dim, case.max_position, case.rope_theta, case.dtype)
    nxt_w = layers[1 % len(layers)].input_layernorm.weight.data.cpu()
    ref = O.decoder_layer(shards, t.x.to(case.dtype), t.positions, num_heads=case.num_heads,
                          num_kv_heads=case.num_kv_heads, head_dim=case.head_dim, eps=case.rms_norm_eps, cache=cache,
                          next_norm_weight=nxt_w)
    rpr = -(-T // world)
    lo, hi = rank * rpr, min(T, rank * rpr + rpr)
    err_out = O.rel_err(normed.cpu(), ref["out_normed"])
    err_res = float((resid[lo:hi].cpu().double() - ref["out"][lo:hi].double()).abs().max()) / float(ref["out"].double().abs().max())
    io_lo, io_hi = runner0.row_range
    err_e2e = float((e2e_out.double() - ref["out"][io_lo:io_hi].double()).abs().max()) / float(ref["out"].double().abs().max())
    p = {"max_rel_err_out": max_over_ranks(err_out), "max_rel_err_residual_rows": max_over_ranks(err_res),
         "max_rel_err_e2e": max_over_ranks(err_e2e), "tol": PARITY_TOL,
         "against": f"CPU oracle of the layer over all {world} shards; every rank checks its outputs, max over ranks"}
    keys = ["max_rel_err_out", "max_rel_err_residual_rows", "max_rel_err_e2e"]
    if pipelined_out is not None:
        # what the TIMED pipelined end-to-end steps left in the host buffer of the first layer's slot (three steps
        # in flight); the caller reports the pipelined figure only if this passes, the serial one otherwise
        err_pipe = float((pipelined_out.double() - ref["out"][io_lo:io_hi].double()).abs().max()) / float(ref["out"].double().abs().max())
        p["max_rel_err_e2e_pipelined"] = max_over_ranks(err_pipe)
    p["ok"] = all(p[k] <= PARITY_TOL for k in keys)
    return p


class QAttention:
    def forward(self, q, k, v, layer_cache_idx, softmax_scale=1.0, layer_id=None):
        return q


def run_native(a):
    import torch
    import torch.distributed as dist
    from sarathi_serve_b200 import dense_ops, parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    ps.initialize_model_parallel(world)

    case = S.CASES[a.workload]
    T, H = case.num_tokens, case.hidden_size
    es = 2
    comm = ps.get_tensor_model_parallel_comm(max(64 << 20, -(-T // world) * world * H * es))

    torch.set_default_dtype(case.dtype)
    t = S.generate(case)
    params = S.shard(t, rank, world)
    per_layer_bytes = sum(v.numel() for k, v in params.items() if "proj" in k) * es
    n_layers = max(1, -(-2 * L2_BYTES // per_layer_bytes))
    layers = []
    for i in range(n_layers):
        layer = LlamaDecoderLayer(case.hf_config(), layer_id=i)
        S.load_layer(layer, params)  # same values, distinct device buffers: what matters is distinct addresses
        layers.append(layer)
    attn = QAttention()
    x_dev = t.x.to(case.dtype).to(dev)
    pos_dev = t.positions.to(dev)
    with torch.inference_mode():
        normed0 = layers[0].input_layernorm(x_dev)

    def step_resident(i):
        layer = layers[i % n_layers]
        nxt = layers[(i + 1) % n_layers].input_layernorm
        # as in a stack of layers: normed hidden states + residual stream (kept sharded by rows) go to the next layer
        return layer.forward_carry(pos_dev, normed0, x_dev, 0, attn, nxt, shard_residual=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        tt = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    with torch.inference_mode():
        # ---- tile configurations for this shape (timed candidates; every rank adopts rank 0's choice)
        cache = a.tune_cache and f"{a.tune_cache}.tp{world}"
        if cache and os.path.exists(cache):
            dense_ops.load_tuned(cache)
        layers[0].tune(T)
        if cache and rank == 0 and not os.path.exists(cache):
            dense_ops.save_tuned(cache)
        barrier()
        # ---- device-resident value: K steps captured once in a CUDA graph, replayed for the timed region
        for i in range(a.warmup):
            step_resident(i)
        barrier()
        comm.check_status()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(a.steps):
                    step_resident(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()  # untimed: first replay of a fresh graph
        barrier()
        # Clocks are sampled under the same load: the sampler is started, the graph is replayed untimed
        # (every rank the same number of times) until nvidia-smi has had time to report, and the timed
        # replay of exactly `steps` steps follows without a gap.
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        lead_in = max(2, int(0.3 / max(1e-4, a.steps * 2.5e-4)))
        for _ in range(lead_in):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        for _ in range(2):  # keeps the load up while the last samples are taken; outside the timed region
            graph.replay()
        barrier()
        ms_resident = max_over_ranks(e0.elapsed_time(e1) / a.steps)
        clocks = sampler.stop() if rank == 0 else None
        comm.check_status()
        dense_ops.check_status(dev)

        # ---- end to end through the layer API with host buffers
        x_host = t.x.to(case.dtype).pin_memory()
        pos_host = t.positions.pin_memory()

        # the public call for a fixed batch shape: captured layers (LayerGraph) fed from pinned host buffers
        # through HostPipeline -- the upload of step i+1 and the download of step i-1 run on copy streams while
        # the kernels of step i do; every step's input crosses PCIe and every step's result is read on the host.
        #  At N > 1 the host buffers are sharded by token rows: each rank uploads T/N rows, the full input is
        #  assembled over NVLink by an all-gather inside the graph, and each rank downloads its T/N rows of the
        #  result -- the step's hidden states cross PCIe once per node, not once per rank.)
        from sarathi_serve_b200.graph_runner import HostPipeline, LayerGraph
        n_slots = max(3, n_layers)
        runners = [LayerGraph(layers[j % n_layers], T, attn, host_io=True, shard_host_io=world > 1, copies_in_graph=False)
                   for j in range(n_slots)]
        io_lo, io_hi = runners[0].row_range
        for r_ in runners:
            r_.host_positions.copy_(pos_host)
            r_.host_hidden_states.copy_(x_host[io_lo:io_hi])
        barrier()

        def time_e2e(step, finish):
            """ms per step of `step(i)`; `finish()` brings the last results to the host before the clock stops.
            Untimed lead-in: at least `warmup` steps and at least 0.3 s of them, so that the clocks have settled
            under this leg's duty cycle (the GPU idled while the graphs were built); the same count on every rank."""
            n_warm = max(10, a.warmup)
            t_w = time.perf_counter()
            for i in range(n_warm):
                step(i)
            per = max(1e-5, (time.perf_counter() - t_w) / n_warm)
            extra = int(max_over_ranks(max(0.0, 0.3 - n_warm * per) / per))
            for i in range(extra):
                step(i)
            finish()
            barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                step(i)
            finish()
            barrier()
            return max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps)

        e2e_steps = max(50, a.steps)

        # (1) one step at a time: upload, layer, download, host synchronisation
        def step_serial(i):
            runners[i % n_slots].replay_host_io()
            torch.cuda.current_stream().synchronize()

        ms_e2e_serial = time_e2e(step_serial, lambda: None)
        comm.check_status()

        # (2) three steps in flight.  This is the figure reported when the result it leaves in the host buffer
        # passes the parity check below on every rank; otherwise the serial figure stands.
        pipe = HostPipeline(runners)

        def step_pipelined(i):
            pipe.submit()
            if pipe.in_flight >= 3:
                pipe.collect()  # waits for the oldest step's result to be in host memory

        ms_e2e_pipelined, pipelined_out, pipeline_note = None, None, ""
        failed = 0
        try:
            ms_local = time_e2e(step_pipelined, pipe.drain)
            pipelined_out = runners[0].host_output.clone()
            comm.check_status()
        except RuntimeError as e:  # (a bounded wait that ran out, or a stream / graph error)
            failed, pipeline_note = 1, f"pipelined leg failed on rank {rank}: {str(e)[:200]}"
        if max_over_ranks(float(failed)) > 0:
            torch.cuda.synchronize()
            if world > 1:
                comm.reset()  # every rank: the contexts' call counters and flags are back in step
            pipelined_out = None
            pipeline_note = pipeline_note or "pipelined leg failed on another rank"
        else:
            ms_e2e_pipelined = ms_local

        # ---- parity of what was just timed, outside the timed regions: one resident step (normed output on
        # every rank, the rows of the new residual this rank owns) and one end-to-end step (host buffers in,
        # host buffer out) against the CPU oracle of the layer over all `world` shards
        parity = check_parity(case, t, world, rank, dev, step_resident, runners[0], layers, max_over_ranks, pipelined_out)
        if ms_e2e_pipelined is not None and parity.get("max_rel_err_e2e_pipelined", 1.0) <= PARITY_TOL:
            ms_e2e, e2e_mode = ms_e2e_pipelined, ("3 steps in flight: upload of step i+1 and download of step i-1 on copy "
                                                  "streams under the kernels of step i; the host waits for every step's result")
        else:
            ms_e2e, e2e_mode = ms_e2e_serial, ("one step at a time (upload, layer, download, host synchronisation)"
                                               + (": " + pipeline_note if pipeline_note else ": the pipelined leg's result "
                                                  "did not pass the parity check"))

        def graph_ms(fn, n, reps=5, lead_in=True):
            """Mean device time of one fn(i) call: n calls captured in a CUDA graph, replayed reps times;
            lead_in: about 0.3 s of the same load first (the power / clock state of a long run)."""
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                for i in range(3):
                    fn(i)
                barrier()
                g_ = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_, stream=st):
                    for i in range(n):
                        fn(i)
                k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                k0.record(st)
                g_.replay()
                k1.record(st)
                barrier()
                # same thermal / power state as the layer steps: about 0.3 s of load before the timed replays
                # (the same count on every rank: the replayed graphs may hold collectives)
                est_ms = max_over_ranks(k0.elapsed_time(k1))
                for _ in range(min(2000, max(1, int(300.0 / max(1e-3, est_ms)))) if lead_in else 0):
                    g_.replay()
                k0.record(st)
                for _ in range(reps):
                    g_.replay()
                k1.record(st)
                barrier()
            torch.cuda.current_stream().wait_stream(st)
            return max_over_ranks(k0.elapsed_time(k1) / (n * reps))

        # ---- dominant kernel alone: gate_up GEMM + SiLU*mul (weights cycled like in the layer steps)
        gu = [l.mlp.gate_up_proj for l in layers]
        # timed alone, without the lead-in: the figure that goes against the burst peak
        ms_kernel = graph_ms(lambda i: gu[i % n_layers].forward_silu_mul(normed0), 2 * n_layers, lead_in=False)

        # ---- the reference's GPU sequence on this box, for comparison: cuBLAS GEMMs (torch.matmul), the
        # separate rotary / SiLU*mul / add+RMSNorm kernels and an NCCL all-reduce after each row-parallel GEMM
        ref_ops = load_reference_ops()
        if ref_ops is not None:
            # the reference's own compiled kernels (its csrc built by its setup.py into baseline/_ref)
            layernorm_ops, activation_ops, pos_encoding_ops = ref_ops["layernorm_ops"], ref_ops["activation_ops"], ref_ops["pos_encoding_ops"]
        else:
            from sarathi_serve_b200 import activation_ops, layernorm_ops, pos_encoding_ops
        sa0 = layers[0].self_attn
        cache = sa0.rotary_emb.cos_sin_cache
        d_loc = case.intermediate_size // world

        def step_cublas(i):
            l = layers[i % n_layers]
            nxt = layers[(i + 1) % n_layers].input_layernorm
            qkv = torch.matmul(normed0, l.self_attn.qkv_proj.weight.t())
            q, k, v = qkv.split([sa0.q_size, sa0.kv_size, sa0.kv_size], dim=-1)
            pos_encoding_ops.rotary_embedding(pos_dev, q, k, sa0.head_dim, cache, True)
            o = torch.matmul(q, l.self_attn.o_proj.weight.t())
            if world > 1:
                dist.all_reduce(o)
            h = torch.empty_like(o)
            if ref_ops is not None:
                # as the reference's layer does it (models/llama.py:248-254): ATen add, then its rms_norm kernel
                r = x_dev + o
                layernorm_ops.rms_norm(h, r, l.post_attention_layernorm.weight.data, 1e-5)
            else:
                r = torch.empty_like(o)
                layernorm_ops.fused_add_rms_norm(h, r, o, x_dev, l.post_attention_layernorm.weight.data, 1e-5)
            gu_ = torch.matmul(h, l.mlp.gate_up_proj.weight.t())
            act = torch.empty(T, d_loc, dtype=gu_.dtype, device=dev)
            activation_ops.silu_and_mul(act, gu_)
            dn = torch.matmul(act, l.mlp.down_proj.weight.t())
            if world > 1:
                dist.all_reduce(dn)
            if ref_ops is not None:
                o2 = r + dn
                layernorm_ops.rms_norm(h, o2, nxt.weight.data, 1e-5)
            else:
                layernorm_ops.fused_add_rms_norm(h, o, dn, r, nxt.weight.data, 1e-5)
            return h

        try:
            ms_cublas = graph_ms(step_cublas, 2 * n_layers)
        except Exception as exc:  # the comparison is optional: say why it is missing
            ms_cublas = None
            cublas_err = f"{type(exc).__name__}: {exc}"

    peak_tf, peak_hbm, peak_src = peaks()
    d = case.intermediate_size // world
    flops = 2.0 * T * H * 2 * d
    achieved = flops / (ms_kernel * 1e-3) / 1e12
    line = None
    if rank == 0:
        value = T / (ms_resident * 1e-3)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": ms_resident, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": bench_config(a.workload, world, T),
                "l2": f"{n_layers} distinct weight sets ({n_layers * per_layer_bytes >> 20} MiB/GPU) cycled: "
                      "operands of consecutive steps exceed the 126 MB L2",
                "parity": parity,
                "pcie": pcie_probe(dev, T * H * es),
                "clocks": clocks,
                "e2e": {"value": T / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": (io_hi - io_lo) * H * es + T * 8, "d2h_bytes_per_step": (io_hi - io_lo) * H * es,
                        "io": (f"per rank: token rows [{io_lo}, {io_hi}) of the {T} x {H} hidden states up and down, all "
                               f"{T} positions up; whole job: {T * H * es} B up and down plus {world} x {T * 8} B of positions"
                               if world > 1 else "the full batch up and down"),
                        "pipeline": e2e_mode, "ms_per_step_serial": ms_e2e_serial,
                        "ms_per_step_pipelined": ms_e2e_pipelined},
                "gpu_launches": (4 if world > 1 else 6) * a.steps, "launch_mode": "one CUDA graph of all timed steps",
                "tile_cfgs": {k[0] + f"[{k[2]}x{k[3]}]": v for k, v in dense_ops._tuned.items()},
                "roofline": {"bound": "tensor", "kernel": "gemm_sm100_kernel<bf16, EPI_SILU_MUL> (gate_up + SiLU*mul)",
                             "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                             "peak_source": f"{peak_src} (burst bf16)", "ms_per_launch": ms_kernel,
                             # DRAM bytes per launch from the committed ncu capture of this kernel (TP=1 workload)
                             "traffic": GATE_UP_TP1_DRAM_BYTES if (world == 1 and a.workload == "config2") else None,
                             "algorithmic_bytes": 2 * d * H * es + T * H * es + T * d * es},
                "layer_roofline": dict(layer_roofline(case, T, world, peak_tf, peak_hbm),
                                       frac=layer_roofline(case, T, world, peak_tf, peak_hbm)["t_roof_us"] / (ms_resident * 1e3),
                                       peaks=f"{peak_src}: {peak_tf} TFLOP/s bf16 burst, {peak_hbm} GB/s HBM; NVLink "
                                             f"{NVLINK_GBS} GB/s per direction (measured peer copy)"),
                "gpu_comparison": ({"what": "the reference's GPU sequence on this box: cuBLAS GEMMs (torch.matmul, what its "
                                            "F.linear calls), " +
                                            ("the reference's own rotary / silu_and_mul / rms_norm kernels compiled from its csrc "
                                             f"({ref_ops['where']}) and ATen residual adds" if ref_ops is not None else
                                             "this library's rotary / SiLU*mul / add+RMSNorm kernels (the reference's "
                                             "compiled ops were not found under oracle/_ref or baseline/_ref)") +
                                            (" + NCCL all-reduce" if world > 1 else "") + ", one CUDA graph",
                                    "ms_per_step": ms_cublas,
                                    "value": T / (ms_cublas * 1e-3), "unit": UNIT} if ms_cublas else
                                   {"unavailable": cublas_err})}
        if not a.no_cpu_baseline:
            v, cores, iters, med = time_cpu(case, a.cpu_baseline_seconds)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"{iters} full layer passes of the same workload "
                                              f"(median {med * 1e3:.0f} ms each), oracle port, torch CPU bf16"}
        print(json.dumps(line), flush=True)
    barrier()
    ps.destroy_model_parallel()
    if world > 1:
        dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit(f"parity against the oracle failed: {parity}")


def load_reference_ops():
    """The reference's own compiled CUDA ops (layernorm_ops, activation_ops, pos_encoding_ops) for the GPU comparison
    arm: the reference's csrc compiled for sm_100 by oracle/build_ref.py into oracle/_ref (preferred), or the
    extensions of a pip install of the reference under baseline/_ref; loaded as extension modules without importing
    the reference's Python package.  None if neither is there or its kernels do not run on this GPU."""
    import glob
    import importlib.util
    import torch
    for base, pattern in ((os.path.join(ROOT, "oracle", "_ref"), "{}.so"),
                          (os.path.join(ROOT, "baseline", "_ref", "sarathi"), "{}.*.so")):
        mods = {}
        try:
            for name in ("layernorm_ops", "activation_ops", "pos_encoding_ops"):
                path = glob.glob(os.path.join(base, pattern.format(name)))
                if not path:
                    raise FileNotFoundError(name)
                spec = importlib.util.spec_from_file_location(name, path[0])
                m = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(m)
                mods[name] = m
            # one trial launch: a build for another architecture fails here, not inside a graph capture
            t = torch.ones(8, 64, device="cuda", dtype=torch.bfloat16)
            o = torch.empty_like(t)
            mods["layernorm_ops"].rms_norm(o, t, torch.ones(64, device="cuda", dtype=torch.bfloat16), 1e-5)
            torch.cuda.synchronize()
            mods["where"] = os.path.relpath(base, ROOT)
            return mods
        except Exception:
            continue
    return None


def pcie_probe(dev, nbytes: int) -> dict:
    """Pinned-host <-> device copy rates of this box for a buffer of the step's size (explains the gap between
    the device-resident and the end-to-end figure; other tenants of the host share the PCIe links)."""
    import torch
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = {}
    for name, fn in (("h2d", lambda: d.copy_(h, non_blocking=True)), ("d2h", lambda: h.copy_(d, non_blocking=True))):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100.0
        out[name + "_us"] = us
        out[name + "_gbs"] = nbytes / us / 1e3
    out["bytes"] = nbytes
    return out


def run_moe(a):
    """Mixtral-8x7B-shaped MoE block (hidden 4096, 8 experts, top-2, expert intermediate 14336, experts sharded
    along the intermediate dimension over N ranks) on a 1024-token chunk: router gate, routing, block
    alignment, the two grouped expert GEMMs and the sum over the k slots fused with the all-reduce.  The block is
    HBM-bound (every expert's shard is read once per step), so the roofline is bytes over the HBM copy rate.
    `--parts` adds the time of every kernel of the block on its own."""
    import torch
    import torch.distributed as dist
    from sarathi_serve_b200 import dense_ops, fused_moe as FM, moe_ops, parallel_state as ps, synthetic as S
    from sarathi_serve_b200.decoder_layer import MixtralMoE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    ps.initialize_model_parallel(world)
    case = S.MOE_CASES[a.workload]
    T, H, E, k, I = case.num_tokens, case.hidden_size, case.num_experts, case.top_k, case.intermediate_size
    es = 2
    d = I // world
    comm = ps.get_tensor_model_parallel_comm(max(64 << 20, -(-T // world) * world * H * es))
    shard = S.generate_moe(case, world=world, rank=rank)
    g = torch.Generator().manual_seed(5)
    gate_w = (torch.randn(E, H, generator=g) * 0.05).to(case.dtype)
    weight_bytes = E * 3 * H * d * es
    n_sets = max(1, -(-2 * L2_BYTES // weight_bytes))
    torch.set_default_dtype(case.dtype)
    blocks = []
    for _ in range(n_sets):
        m = MixtralMoE(E, k, H, I)
        sd = m.state_dict()
        with torch.no_grad():
            sd["gate.weight"].copy_(gate_w)
            sd["experts.w13_weight"].copy_(shard["w13"])
            sd["experts.w2_weight"].copy_(shard["w2"])
        blocks.append(m)
    x = shard["x"].to(dev)
    xs = [x.clone() for _ in range(n_sets)]  # the block overwrites its input

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        tt = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def graph_us(fn, n, reps=5):
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st), torch.inference_mode():
            for i in range(3):
                fn(i)
            barrier()
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=st):
                for i in range(n):
                    fn(i)
            g_.replay()
            barrier()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(st)
            for _ in range(reps):
                g_.replay()
            k1.record(st)
            barrier()
        torch.cuda.current_stream().wait_stream(st)
        return max_over_ranks(k0.elapsed_time(k1) / (n * reps) * 1e3)

    def step(i):
        j = i % n_sets
        xs[j].copy_(x)  # restores the input the previous use overwrote (4 MiB, part of neither figure's bytes)
        return blocks[j](xs[j])

    peak_tf, peak_hbm, peak_src = peaks()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    us_copy = graph_us(lambda i: xs[i % n_sets].copy_(x), max(a.steps, 4))
    us_step = graph_us(step, max(a.steps, 4)) - us_copy
    clocks = sampler.stop() if rank == 0 else None
    comm.check_status()
    dense_ops.check_status(dev)
    # parity of one step against the CPU oracle on a subset of tokens (the oracle of the full block takes minutes):
    # the block is token-wise apart from the expert sort, so the first 64 tokens alone give the same rows
    from oracle import tp_layer_oracle as O
    with torch.inference_mode():
        got = blocks[0](x.clone())[:64].cpu()
    shards_all = [S.generate_moe(case, world=world, rank=r) for r in range(world)] if world <= 2 or case.name != "config5" else None
    parity = None
    if shards_all is not None:
        ref = O.moe_layer(shard["x"][:64], gate_w, [s_["w13"] for s_ in shards_all], [s_["w2"] for s_ in shards_all], k)
        err = max_over_ranks(O.rel_err(got, ref))
        parity = {"max_rel_err_out": err, "tol": PARITY_TOL, "ok": err <= PARITY_TOL,
                  "against": "CPU oracle of the MoE block on the first 64 tokens"}
    flops = 2.0 * T * k * H * 3 * d
    hbm_bytes = weight_bytes + es * (T * H * 2 + T * k * (H + 2 * d) * 2)
    parts = None
    if a.parts:
        with torch.inference_mode():
            m0 = blocks[0]
            logits, _ = m0.gate(x)
            tw, ti = FM.fused_topk(x, logits, k, True)
            blk = FM.block_rows()
            parts = {}
            parts["router_gate_gemm"] = {"us": graph_us(lambda i: blocks[i % n_sets].gate(x), 8)}
            parts["topk_softmax"] = {"us": graph_us(lambda i: FM.fused_topk(x, logits, k, True), 8)}
            parts["moe_align_block_size"] = {"us": graph_us(lambda i: FM.moe_align_block_size(ti, blk, E), 8)}
            us_e = graph_us(lambda i: FM._expert_slots(x, blocks[i % n_sets].experts.w13_weight,
                                                       blocks[i % n_sets].experts.w2_weight, tw, ti, True), 2 * n_sets)
            parts["align+gather+gemm1+gemm2"] = {"us": us_e, "hbm_gbs": weight_bytes / us_e / 1e3,
                                                 "tflops": flops / us_e / 1e6}
    if rank == 0:
        line = {"metric": "tp_moe_block_tokens_per_s", "value": T / (us_step * 1e-6), "unit": UNIT, "n_gpus": world,
                "steps": a.steps, "warmup": a.warmup, "ms_per_step": us_step * 1e-3, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"{a.workload}: Mixtral-8x7B-shaped MoE block (hidden {H}, {E} experts, top-{k}, expert "
                                       f"intermediate {I}), {T}-token chunk, TP={world}", "tokens_per_step": T,
                           "parallelism": f"tp{world}"},
                "clocks": clocks, "parity": parity,
                "roofline": {"bound": "hbm", "kernel": "MoE block: grouped expert GEMMs (gemm_sm100_kernel, grouped mode)",
                             "achieved": hbm_bytes / us_step / 1e3, "peak": peak_hbm, "unit": "GB/s",
                             "frac": hbm_bytes / us_step / 1e3 / peak_hbm, "peak_source": peak_src, "traffic": None,
                             "algorithmic_bytes": hbm_bytes, "compute_us": flops / (peak_tf * 1e6),
                             "hbm_us": hbm_bytes / (peak_hbm * 1e3)},
                "parts": parts, "gpu_launches": 7 * a.steps}
        print(json.dumps(line), flush=True)
    barrier()
    ps.destroy_model_parallel()
    if world > 1:
        dist.destroy_process_group()


def kernel_pass(case, layers, x, pos, normed, q, h, resid, act, nw, comm, dev):
    """Two eager launches of every kernel of the path at the workload's shapes (nothing timed)."""
    import torch
    from sarathi_serve_b200 import (activation_ops, dense_ops, embedding_ops, fused_moe as FM, layernorm_ops, moe_ops,
                                    pos_encoding_ops, synthetic as S)
    T, H = x.shape
    nl = len(layers)
    sa = layers[0].self_attn
    d = act.shape[1]
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    gu = torch.randn(T, 2 * d, device=dev, dtype=torch.float32).to(x.dtype)
    ao = torch.empty(T, d, device=dev, dtype=x.dtype)
    qkv = torch.randn(T, sa.q_size + 2 * sa.kv_size, device=dev, dtype=torch.float32).to(x.dtype)
    qs, ks, _ = qkv.split([sa.q_size, sa.kv_size, sa.kv_size], dim=-1)
    mc = S.MOE_CASES["config5"]
    E, k, Tm, blk = mc.num_experts, mc.top_k, mc.num_tokens, FM.block_rows()
    logits = torch.randn(Tm, E, device=dev, dtype=torch.float32)
    tw = torch.empty(Tm, k, dtype=torch.float32, device=dev)
    ti = torch.empty(Tm, k, dtype=torch.int32, device=dev)
    xm = torch.randn(Tm, H, device=dev, dtype=torch.float32).to(x.dtype)
    dm = mc.intermediate_size // 8  # the per-rank expert shard of an 8-way split
    w13 = (torch.randn(E, 2 * dm, H, device=dev, dtype=torch.float32) * 0.02).to(x.dtype)
    w2 = (torch.randn(E, H, dm, device=dev, dtype=torch.float32) * 0.02).to(x.dtype)
    for i in range(2):
        l = layers[i % nl]
        layernorm_ops.rms_norm(o1, x, nw, 1e-5)
        layernorm_ops.fused_add_rms_norm(o1, o2, h, x, nw, 1e-5)
        activation_ops.silu_and_mul(ao, gu)
        pos_encoding_ops.rotary_embedding(pos, qs, ks, sa.head_dim, sa.rotary_emb.cos_sin_cache, True)
        l.self_attn.qkv_rotary(pos, normed)
        dense_ops.linear(q, l.self_attn.o_proj.weight)
        l.mlp.gate_up_proj.forward_silu_mul(h)
        dense_ops.linear(act, l.mlp.down_proj.weight, residual=resid)
        comm.rowpar_linear(q, l.self_attn.o_proj.weight, residual=x, norm_weight=nw, eps=1e-5)
        moe_ops.topk_softmax(tw, ti, None, logits, renormalize=True)
        FM.moe_align_block_size(ti, blk, E)
        out3 = FM._expert_slots(xm, w13, w2, tw, ti, True)
        FM.fused_experts(xm, w13, w2, tw, ti)
        torch.cuda.synchronize()
    comm.check_status()
    dense_ops.check_status(dev)
    print("kernel pass done", flush=True)


def run_parts(a):
    """Per-kernel device times of the path (each kernel alone, back-to-back launches in one CUDA graph with
    the weights of several layers cycled), with the achieved rate against the roofline that bounds it."""
    import torch
    import torch.distributed as dist
    from sarathi_serve_b200 import (activation_ops, dense_ops, layernorm_ops, moe_ops, parallel_state as ps,
                                    pos_encoding_ops, synthetic as S)
    from sarathi_serve_b200.decoder_layer import LlamaDecoderLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    ps.initialize_model_parallel(world)
    case = S.CASES[a.workload]
    T, H, es = case.num_tokens, case.hidden_size, 2
    comm = ps.get_tensor_model_parallel_comm(max(64 << 20, -(-T // world) * world * H * es))
    torch.set_default_dtype(case.dtype)
    t = S.generate(case)
    params = S.shard(t, rank, world)
    per_layer_bytes = sum(v.numel() for k, v in params.items() if "proj" in k) * es
    nl = max(2, -(-2 * L2_BYTES // per_layer_bytes))
    layers = []
    for i in range(nl):
        layer = LlamaDecoderLayer(case.hf_config(), layer_id=i)
        S.load_layer(layer, params)
        layers.append(layer)
    x = t.x.to(case.dtype).to(dev)
    pos = t.positions.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def graph_us(fn, n=None, reps=5):
        n = n or 2 * nl
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            for i in range(3):
                fn(i)
            barrier()
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=st):
                for i in range(n):
                    fn(i)
            g_.replay()
            barrier()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(st)
            for _ in range(reps):
                g_.replay()
            k1.record(st)
            barrier()
        torch.cuda.current_stream().wait_stream(st)
        v = torch.tensor([k0.elapsed_time(k1) / (n * reps) * 1e3], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    peak_tf, peak_hbm, peak_src = peaks()
    nq, nkv, hd, I = case.num_heads, case.num_kv_heads, case.head_dim, case.intermediate_size
    qkv_n, d = (nq + 2 * nkv) * hd // world, I // world
    out = {}

    def gemm_entry(name, us, flops, extra=None):
        e = {"us": us, "tflops": flops / us / 1e6, "frac_of_bf16_peak": flops / us / 1e6 / peak_tf}
        e.update(extra or {})
        out[name] = e

    def hbm_entry(name, us, nbytes):
        out[name] = {"us": us, "bytes": nbytes, "hbm_gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peak_hbm}

    with torch.inference_mode():
        cache = a.tune_cache and f"{a.tune_cache}.tp{world}"
        if cache and os.path.exists(cache):
            dense_ops.load_tuned(cache)
        layers[0].tune(T)
        if cache and rank == 0 and not os.path.exists(cache):
            dense_ops.save_tuned(cache)
        barrier()
        l0 = layers[0]
        sa = l0.self_attn
        normed = l0.input_layernorm(x)
        q, k, v = sa.qkv_rotary(pos, normed)
        nw = l0.post_attention_layernorm.weight.data
        h, resid = sa.o_proj.forward_fused(q, x, nw, 1e-5)
        h, resid = h.clone(), resid.clone()
        act = l0.mlp.gate_up_proj.forward_silu_mul(h)
        if a.kernel_pass:
            kernel_pass(case, layers, x, pos, normed, q, h, resid, act, nw, comm, dev)
            ps.destroy_model_parallel()
            if world > 1:
                dist.destroy_process_group()
            return
        ar_bytes = 2.0 * (world - 1) / world * T * H * es  # per direction, per GPU
        gemm_entry("qkv_gemm+rotary", graph_us(lambda i: layers[i % nl].self_attn.qkv_rotary(pos, normed)), 2.0 * T * H * qkv_n)
        # (as on the layer path: the new residual stays with the owner of each row -- resid_everywhere=False)
        us = graph_us(lambda i: layers[i % nl].self_attn.o_proj.forward_fused(q, x, nw, 1e-5, resid_everywhere=False))
        gemm_entry("o_proj_gemm+allreduce+add+rmsnorm", us, 2.0 * T * H * nq * hd / world,
                   {"nvlink_gbs_per_direction": ar_bytes / us / 1e3 if world > 1 else None})
        gemm_entry("gate_up_gemm+silu_mul", graph_us(lambda i: layers[i % nl].mlp.gate_up_proj.forward_silu_mul(h)), 2.0 * T * H * 2 * d)
        us = graph_us(lambda i: layers[i % nl].mlp.down_proj.forward_fused(act, resid, nw, 1e-5, resid_everywhere=False))
        gemm_entry("down_gemm+allreduce+add+rmsnorm", us, 2.0 * T * H * d,
                   {"nvlink_gbs_per_direction": ar_bytes / us / 1e3 if world > 1 else None})
        gemm_entry("o_proj_gemm_alone", graph_us(lambda i: dense_ops.linear(q, layers[i % nl].self_attn.o_proj.weight)), 2.0 * T * H * nq * hd / world)
        gemm_entry("down_gemm_alone", graph_us(lambda i: dense_ops.linear(act, layers[i % nl].mlp.down_proj.weight)), 2.0 * T * H * d)
        if world > 1:
            us = graph_us(lambda i: comm.all_reduce(h, residual=x, norm_weight=nw, eps=1e-5, resid_everywhere=False))
            out["allreduce+add+rmsnorm_alone"] = {"us": us, "nvlink_bytes_per_direction": ar_bytes,
                                                   "nvlink_gbs_per_direction": ar_bytes / us / 1e3,
                                                   "frac_of_nvlink": ar_bytes / us / 1e3 / NVLINK_GBS}
            buf = h.clone()
            us = graph_us(lambda i: dist.all_reduce(buf))
            out["nccl_allreduce_alone"] = {"us": us, "nvlink_gbs_per_direction": ar_bytes / us / 1e3}

            def ref_tail(xin, wt, res_in):
                y = torch.matmul(xin, wt.t())
                dist.all_reduce(y)
                r_, o_ = torch.empty_like(y), torch.empty_like(y)
                layernorm_ops.fused_add_rms_norm(o_, r_, y, res_in, nw, 1e-5)
                return o_
            out["cublas_o_proj+nccl+add_rmsnorm"] = {"us": graph_us(lambda i: ref_tail(q, layers[i % nl].self_attn.o_proj.weight, x))}
            out["cublas_down+nccl+add_rmsnorm"] = {"us": graph_us(lambda i: ref_tail(act, layers[i % nl].mlp.down_proj.weight, resid))}
        # the element-wise kernels on their own (HBM-bound); inputs of a few MB sit in L2, so they can read above the HBM figure
        o1, o2 = torch.empty_like(x), torch.empty_like(x)
        hbm_entry("rms_norm", graph_us(lambda i: layernorm_ops.rms_norm(o1, x, nw, 1e-5), n=8), (2 * T * H + H) * es)
        hbm_entry("fused_add_rms_norm", graph_us(lambda i: layernorm_ops.fused_add_rms_norm(o1, o2, h, x, nw, 1e-5), n=8), (4 * T * H + H) * es)
        gu = torch.randn(T, 2 * d, device=dev, dtype=torch.float32).to(case.dtype)
        ao = torch.empty(T, d, device=dev, dtype=case.dtype)
        hbm_entry("silu_and_mul", graph_us(lambda i: activation_ops.silu_and_mul(ao, gu), n=8), 3 * T * d * es)
        qkv = torch.randn(T, qkv_n, device=dev, dtype=torch.float32).to(case.dtype)
        qs, ks, _ = qkv.split([sa.q_size, sa.kv_size, sa.kv_size], dim=-1)
        cache = sa.rotary_emb.cos_sin_cache
        hbm_entry("rotary_embedding", graph_us(lambda i: pos_encoding_ops.rotary_embedding(pos, qs, ks, hd, cache, True), n=8),
                  2 * T * (sa.q_size + sa.kv_size) * es + 8 * T + T * hd * es)
        E, topk, Tm = 8, 2, 1024
        logits = torch.randn(Tm, E, device=dev, dtype=torch.float32)
        tw = torch.empty(Tm, topk, dtype=torch.float32, device=dev)
        ti = torch.empty(Tm, topk, dtype=torch.int32, device=dev)
        hbm_entry("topk_softmax", graph_us(lambda i: moe_ops.topk_softmax(tw, ti, None, logits, renormalize=True), n=8), Tm * E * 4 + Tm * topk * 12)
        blk = 64
        cap = Tm * topk + E * (blk - 1)
        sids = torch.empty(cap, dtype=torch.int32, device=dev)
        eids = torch.empty(-(-cap // blk), dtype=torch.int32, device=dev)
        npp = torch.empty(1, dtype=torch.int32, device=dev)
        moe_ops.topk_softmax(tw, ti, None, logits, renormalize=True)
        hbm_entry("moe_align_block_size", graph_us(lambda i: moe_ops.moe_align_block_size(ti, E, blk, sids, eids, npp), n=8),
                  4 * Tm * topk + 4 * (cap + cap // blk + 1))
    comm.check_status()
    if rank == 0:
        print(json.dumps({"parts": out, "n_gpus": world, "workload": workload_text(a.workload, world),
                          "peaks": {"bf16_tflops": peak_tf, "hbm_gbs": peak_hbm, "nvlink_gbs_per_direction": NVLINK_GBS,
                                    "source": peak_src},
                          "tile_cfgs": {k_[0] + f"[{k_[2]}x{k_[3]}]": v_ for k_, v_ in dense_ops._tuned.items()}}), flush=True)
    barrier()
    ps.destroy_model_parallel()
    if world > 1:
        dist.destroy_process_group()


def main():
    a = parse()
    if a.impl == "reference":
        run_reference_arm(a)
    elif a.workload in ("config5", "mini_moe"):
        run_moe(a)
    elif a.parts:
        run_parts(a)
    else:
        run_native(a)


if __name__ == "__main__":
    main()
