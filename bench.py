"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the W4A16 shape sweep over every Qwen3-1.7B projection.  One
step = one decode pass (batch M = 1) over the full random-init weight set: 28
layers x {q,k,v,o,gate,up,down}_proj + lm_head = 197 int4 linears, 887 MB of
packed weights, i.e. several times the 126 MB L2, so every weight byte of a step
comes from HBM.  The pass is one persistent launch (garnet_b200_w4a16_list_*);
its linears read fixed activation buffers, i.e. they do not wait for one
another.  `value` is algorithmic bytes / step time with activations resident in
HBM; `chained` repeats the pass with the data dependencies the shapes allow
(q/k/v <- previous down, o <- q, gate/up <- o, down <- gate, lm_head <- last down),
every dependent linear waiting on the device for its producer; `e2e` is the
same pass through the host-buffer entry point (pinned host x -> device, one
launch, device -> host y).  `sweep` holds the per-shape, per-batch (M in
1,4,16,64,256) numbers measured on rotating weight copies larger than twice the
L2.  With N > 1 the lm_head is sharded along N across the ranks and the logits
are all-gathered over NVLink; the decoder layers are replicated (the
configuration's definition), so scaling is strong.

--impl reference times the reference's own CPU operator (Q4Q8Linear compiled
from the reference sources when available, otherwise its restatement) on the
host cores for the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GROUP = 128
LAYERS = 28
PROJ = [("q_proj", 2048, 2048), ("k_proj", 2048, 1024), ("v_proj", 2048, 1024), ("o_proj", 2048, 2048),
        ("gate_proj", 2048, 6144), ("up_proj", 2048, 6144), ("down_proj", 6144, 2048)]
LM_HEAD = ("lm_head", 2048, 151936)
SWEEP_M = [1, 4, 8, 16, 64, 256]   # the configured sweep plus 8 rows (two 4-row MMA column blocks)
# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of a launch of
# w4a16_list_kernel, from the ncu capture summarised in the file named below (an
# eight-layer list, 208 MB of weights, captured instead of the full 890 MB pass to keep the
# replay short; traffic grows in proportion to the weights streamed)
TRAFFIC_RATIO = 1.017
TRAFFIC_SOURCE = "profiles/w4a16_list_kernel_8layers_m1.md"


def weight_bytes(k, n):
    return n * k // 2 + n * (k // GROUP) * 2


def algo_bytes(k, n, m):
    return weight_bytes(k, n) + m * k * 2 + m * n * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=float(d["hbm_gbs"]), tf=float(d["bf16_tflops"]), tf_sus=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ GPU arm

def make_linear(torch, gb, k, n, gen, shard=(0, 1)):
    nib = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device="cuda", generator=gen)
    sc = (torch.randn(n, k // GROUP, device="cuda", generator=gen).abs() * (0.02 / 7.0)).to(torch.bfloat16)
    lin = gb.W4A16Linear().prepare(nib, sc, n, k, GROUP, shard_rank=shard[0], shard_world=shard[1])
    del nib, sc
    return lin


def time_graph(torch, fn, steps, warmup, flush=None):
    """Captures fn() once into a CUDA graph and times `steps` replays with CUDA
    events on the launching stream (after `warmup` replays)."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(steps):
            graph.replay()
        stop.record(stream)
        stream.synchronize()
    return start.elapsed_time(stop) / steps   # ms per replay


def run_gpu(args):
    import torch
    import torch.distributed as dist

    import garnet_b200 as gb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = measured_peaks()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)

    # ---- the decode pass: 28 layers + lm_head (sharded along N when world > 1)
    m = 1
    layers = []
    for _ in range(LAYERS):
        layers.append([(make_linear(torch, gb, k, n, gen), k, n) for (_, k, n) in PROJ])
    _, hk, hn = LM_HEAD
    head = make_linear(torch, gb, hk, hn, gen, shard=(rank, world))
    hn_local = hn // world
    xs = {k: torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16) for k in (2048, 6144)}
    ys = {n: torch.empty(m, n, device="cuda", dtype=torch.bfloat16) for n in (1024, 2048, 6144)}
    y_head = torch.empty(m, hn_local, device="cuda", dtype=torch.bfloat16)
    logits = torch.empty(world, m, hn_local, device="cuda", dtype=torch.bfloat16) if world > 1 else None
    gather = None
    if world > 1:
        from garnet_b200.dist import Channel, Comm
        comm = Comm(4 * world * m * hn_local * 2 + (1 << 20))
        gather = Channel(comm, m * hn_local * 2)
    ws_bytes = max([lin.workspace_bytes(m) for layer in layers for (lin, _, _) in layer] + [head.workspace_bytes(m)])
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    # the whole pass is one prepared list: one persistent launch per step
    y_k = torch.empty(m, 1024, device="cuda", dtype=torch.bfloat16)
    y_v = torch.empty(m, 1024, device="cuda", dtype=torch.bfloat16)
    y_up = torch.empty(m, 6144, device="cuda", dtype=torch.bfloat16)
    y_o = torch.empty(m, 2048, device="cuda", dtype=torch.bfloat16)
    y_d = torch.empty(m, 2048, device="cuda", dtype=torch.bfloat16)
    calls = []
    for layer in layers:
        q, kk, v, o, gate, up, down = [lin for (lin, _, _) in layer]
        calls += [(q, xs[2048], ys[2048]), (kk, xs[2048], y_k), (v, xs[2048], y_v), (o, xs[2048], y_o),
                  (gate, xs[2048], ys[6144]), (up, xs[2048], y_up), (down, xs[6144], y_d)]
    calls.append((head, xs[hk], y_head))
    pass_list = gb.LinearList(calls, m=m)
    launches_per_step = 1 if world == 1 else 2

    def decode_pass():
        pass_list.run()
        if world > 1:
            gather.all_gather(y_head, logits)     # peer stores over NVLink: one kernel per rank, no library collective

    # The same 197 linears with the data dependencies their shapes allow, each consumer
    # waiting on the device for its producer (one launch as well).
    def chained_list():
        cc, prev_down = [], -1
        x_in = xs[2048]
        mk = lambda n: torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        for layer in layers:
            q, kk, v, o, gate, up, down = [lin for (lin, _, _) in layer]
            yq, yk2, yv2, yo, yg, yu, yd = mk(2048), mk(1024), mk(1024), mk(2048), mk(6144), mk(6144), mk(2048)
            iq = len(cc)
            cc += [(q, x_in, yq, prev_down), (kk, x_in, yk2, prev_down), (v, x_in, yv2, prev_down)]
            io = len(cc)
            cc.append((o, yq, yo, iq))
            ig = len(cc)
            cc += [(gate, yo, yg, io), (up, yo, yu, io)]
            prev_down = len(cc)
            cc.append((down, yg, yd, ig))
            x_in = yd
        cc.append((head, x_in, y_head, prev_down))
        return gb.LinearList(cc, m=m)

    step_bytes = LAYERS * sum(algo_bytes(k, n, m) for (_, k, n) in PROJ) + algo_bytes(hk, hn, m)

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = time_graph(torch, decode_pass, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    assert pass_list.fault() == 0, "a device-side wait gave up"
    chain = chained_list()
    chained_ms = time_graph(torch, chain.run, args.steps, args.warmup)
    assert chain.fault() == 0, "a device-side wait gave up"
    del chain
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = step_bytes / (ms * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point
    xh = {k: v.cpu().pin_memory() for k, v in xs.items()}
    yh = {n: torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for n in (1024, 2048, 6144)}
    yh_head = torch.empty(m, hn_local, dtype=torch.bfloat16).pin_memory()

    # Every linear is called with HOST buffers (pinned) through the prepared-batch C entry
    # points: each distinct input buffer is copied to the device once per pass, the 197
    # linears run as one launch, one kernel writes their 197 outputs to the host buffers, and
    # the pass synchronises once, when its results are read.  Two sets of seven output
    # buffers, alternating by layer.
    yh_all = [[torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for (_, _, n) in PROJ] for _ in range(2)]
    host_calls = []
    for li, layer in enumerate(layers):
        for j, (lin, k, n) in enumerate(layer):
            host_calls.append((lin, xh[k], yh_all[li & 1][j]))
    host_calls.append((head, xh[hk], yh_head))
    host_batch = gb.HostBatch(host_calls)

    def host_pass():
        host_batch.run()
        if world > 1:
            torch.cuda.current_stream().synchronize()
            y_head.copy_(yh_head, non_blocking=True)
            gather.all_gather(y_head, logits)
        torch.cuda.current_stream().synchronize()
        return float(yh_head[0, 0])   # the host reads the step's result

    for _ in range(max(3, args.warmup)):
        host_pass()
    e2e_steps = max(3, min(args.steps, 10))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_pass()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    # bytes actually copied in: the prepared batch copies every distinct host input once per pass
    h2d = sum(int(v.numel()) * 2 for v in xh.values())
    d2h = LAYERS * sum(m * n * 2 for (_, k, n) in PROJ) + m * hn_local * 2

    out = None
    if rank == 0:
        out = {
            "metric": "w4a16_weight_GBps", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int4 x bf16 (as 15-bit block fixed point) -> int32 per 128-group, fp32 across groups, bf16 out",
            "data": "synthetic",
            "config": {"workload": "qwen3_1p7b_w4a16_sweep: decode pass M=1 over 28x7 projections + lm_head (197 int4 group-128 linears)",
                       "bytes_per_step": step_bytes, "l2": "887 MB of weights per step > 126 MB L2; no flush needed",
                       "parallelism": f"lm_head N-sharded x{world} + all-gather by peer stores (garnet_b200_comm_all_gather)" if world > 1 else "single GPU",
                       "launch": "one persistent launch per pass (a prepared list of the 197 linears reading fixed activation buffers; no linear waits for another)"},
            "chained": {"ms_per_step": round(chained_ms, 5), "value": round(step_bytes / (chained_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                        "hbm_frac": round(step_bytes / (chained_ms * 1e-3) / 1e9 / peaks["hbm"], 4),
                        "what": "same pass, one launch, with the data dependencies the shapes allow (113 dependent stages: q/k/v <- previous down, o <- q, gate/up <- o, down <- gate, lm_head <- last down); a dependent linear polls its producer's output packets on the device"},
            "clocks": clocks,
            "e2e": {"value": round(step_bytes / (e2e_ms * 1e-3) / 1e9, 3), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": round(value, 2), "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": round(value / peaks["hbm"], 4), "peak_source": peaks["src"],
                         "traffic": round(step_bytes / launches_per_step * TRAFFIC_RATIO),
                         "traffic_source": TRAFFIC_SOURCE,
                         "kernel": "w4a16_list_kernel", "bytes_per_launch": round(step_bytes / launches_per_step),
                         "us_per_launch": round(ms * 1e3 / launches_per_step, 3)},
        }

    # ---- per-shape sweep on rotating copies (single GPU only)
    if world == 1 and not args.no_sweep:
        del layers, head
        torch.cuda.empty_cache()
        out["decode_step"] = bench_decode_step(torch, peaks, args)
        torch.cuda.empty_cache()
        sweep = []
        shapes = [("q_proj/o_proj", 2048, 2048), ("k_proj/v_proj", 2048, 1024), ("gate_proj/up_proj", 2048, 6144),
                  ("down_proj", 6144, 2048), ("lm_head", 2048, 151936)]
        for name, k, n in shapes:
            copies = max(2, int(np.ceil(2.2 * 126e6 / weight_bytes(k, n))))
            lins = [make_linear(torch, gb, k, n, gen) for _ in range(copies)]
            for mm in SWEEP_M:
                x = torch.randn(mm, k, device="cuda", generator=gen).to(torch.bfloat16)
                y = torch.empty(mm, n, device="cuda", dtype=torch.bfloat16)
                w = torch.empty(max(16, lins[0].workspace_bytes(mm)), dtype=torch.uint8, device="cuda")

                if mm <= 16 and mm <= (8 if k > 4096 else 16):
                    rot = gb.LinearList([(lin, x, y) for lin in lins], m=mm)   # one launch over the rotating copies
                    body = rot.run
                else:
                    def body():
                        for lin in lins:
                            lin.forward(x, out=y, workspace=w)

                t_ms = time_graph(torch, body, max(3, args.steps // 4), 3) / copies
                gbs = algo_bytes(k, n, mm) / (t_ms * 1e-3) / 1e9
                tfl = 2.0 * mm * n * k / (t_ms * 1e-3) / 1e12
                sweep.append({"shape": name, "K": k, "N": n, "M": mm, "us": round(t_ms * 1e3, 3), "GBps": round(gbs, 1),
                              "hbm_frac": round(gbs / peaks["hbm"], 4), "TFLOPs": round(tfl, 2),
                              "tensor_frac": round(tfl / peaks["tf"], 4), "copies": copies})
            del lins
            torch.cuda.empty_cache()
        out["sweep"] = sweep

    if world == 1 and not args.no_moe:
        torch.cuda.empty_cache()
        out["moe"] = bench_moe(torch, gb, peaks, args)
        out["gpt_oss_layer_ops"] = bench_gpt_oss_layer_ops(torch, args)
        out["moe_ep"] = bench_moe_ep(torch, dist, gb, args, 0, 1)
    if world > 1 and not args.no_moe:
        del layers, head
        torch.cuda.empty_cache()
        ep = bench_moe_ep(torch, dist, gb, args, rank, world)
        if rank == 0:
            out["moe_ep"] = ep

    if rank == 0:
        if world == 1:
            out["cpu_baseline"] = cpu_baseline(sample_seconds=10.0)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_decode_step(torch, peaks, args, context=2048):
    """BASELINE's config 3 as a real step: one token through the 28 Qwen3-1.7B layers at a context
    of 2048 positions (embedding, norms, packed q/k/v, head norms + RoPE, paged-KV attention,
    o_proj, packed gate/up with SiLU, down, residuals, final norm, lm_head, arg-max) as one CUDA
    graph of 2 launches per layer.  Synthetic weights and a random bf16 KV cache."""
    from garnet_b200 import decode as dec
    cfg = dec.DecoderConfig()
    w = dec.synthetic_decoder(cfg, seed=7)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    pages = context // cfg.page_size
    kps = [torch.randn(pages, cfg.page_size, cfg.kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(cfg.layers)]
    vps = [torch.randn(pages, cfg.page_size, cfg.kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(cfg.layers)]
    tables = torch.randperm(pages, generator=torch.Generator().manual_seed(2)).reshape(1, pages).to(torch.int32).cuda()
    step = dec.DecodeStep(cfg, w, 1, max_context=context, key_pages=kps, value_pages=vps, page_tables=tables)
    step.token_in.fill_(1234)
    step.positions.fill_(context - 1)            # the new token is the context's last position
    ms = time_graph(torch, step.enqueue, args.steps, args.warmup)
    assert step.fault() == 0, "a device-side wait gave up"
    H, I = cfg.hidden, cfg.intermediate
    weights = cfg.layers * sum(weight_bytes(k, n) for (k, n) in ((H, cfg.qkv_width), (cfg.q_heads * 128, H), (H, 2 * I), (I, H))) \
        + weight_bytes(H, cfg.vocab)
    kv = cfg.layers * context * cfg.kv_heads * 128 * 2 * 2
    nbytes = weights + kv
    return {"ms_per_step": round(ms, 5), "tok_per_s": round(1e3 / ms, 1), "context": context, "batch": 1,
            "bytes_per_step": nbytes, "weight_bytes": weights, "kv_bytes": kv,
            "GBps": round(nbytes / (ms * 1e-3) / 1e9, 1), "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm"], 4),
            "launches_per_step": step.launches,
            "what": "whole decode step in one CUDA graph: per layer one attention launch (head norms, RoPE, cache append, "
                    "split softmax and merge) and one list launch (o_proj + residual, norm + gate/up, SwiGLU + down + residual, "
                    "norm + next q/k/v); greedy token by arg-max"}


def gpt_oss_layer_case(torch, context=2048, layers=4):
    """Operands of the gpt-oss-120b attention block at decode (64 q heads, 8 kv heads of 64, pages of 16),
    one sequence with `context` positions, caches of `layers` layers filled with random bf16."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    logical = context // 16
    keys = torch.randn(layers, logical, 16, 8, 64, device="cuda", generator=gen).to(torch.bfloat16)
    values = torch.randn(layers, logical, 16, 8, 64, device="cuda", generator=gen).to(torch.bfloat16)
    table = torch.randperm(logical, generator=torch.Generator().manual_seed(1)).reshape(1, logical).to(torch.int32).cuda()
    qkv = torch.randn(1, 80 * 64, device="cuda", generator=gen).to(torch.bfloat16).float()
    lens = torch.tensor([context], dtype=torch.int32, device="cuda")
    starts = torch.tensor([context - 1], dtype=torch.int32, device="cuda")
    active = torch.ones(1, dtype=torch.int32, device="cuda")
    sinks = torch.randn(64, device="cuda", generator=gen)
    w_qkv = (torch.randn(80 * 64, 2880, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    w_o = (torch.randn(2880, 4096, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    x = torch.randn(2880, device="cuda", generator=gen).to(torch.bfloat16)
    a = torch.randn(4096, device="cuda", generator=gen).to(torch.bfloat16)
    return dict(keys=keys, values=values, table=table, qkv=qkv, lens=lens, starts=starts, active=active, sinks=sinks, w_qkv=w_qkv,
                w_o=w_o, x=x, a=a, logical=logical, layers=layers)


def bench_gpt_oss_layer_ops(torch, args):
    import garnet_b200 as gb
    """The gpt-oss attention block at decode, one launch sequence per layer over `layers` different cache slabs
    (so the KV rows come from HBM): attention with the cache append (full and with a 128-position window), and
    the q/k/v and output GEMVs."""
    from garnet_b200 import gpt_oss as go
    c = gpt_oss_layer_case(torch)
    out = {}
    for name, window in (("attention_full_2048", 0), ("attention_window_128", 128)):
        opts = [go.options(layer=l, window=window) for l in range(c["layers"])]
        import ctypes
        need = ctypes.c_size_t(0)
        gb._lib.check(gb.lib().garnet_b200_gpt_oss_attention_workspace(ctypes.byref(opts[0]), 1, c["logical"], ctypes.byref(need)))
        ws = torch.zeros(need.value, dtype=torch.uint8, device="cuda")

        def body():
            for o in opts:
                go.attention(o, c["qkv"], c["keys"], c["values"], c["table"], c["lens"], c["starts"], c["active"], c["sinks"], 1, 1,
                             c["logical"], workspace=ws)
        out[name + "_us"] = round(time_graph(torch, body, args.steps, 3) * 1e3 / c["layers"], 2)

    def gemvs():
        go.decode_gemv(c["x"], c["w_qkv"], 80 * 64, 2880)
        go.decode_gemv(c["a"], c["w_o"], 2880, 4096)
    out["qkv_and_o_gemv_us"] = round(time_graph(torch, gemvs, args.steps, 3) * 1e3, 2)
    return out


def reference_gpu_layer_ops():
    """The same operators through the reference's own kernels (RunGptOssAttention, RunGptOssDecodeGemv)."""
    try:
        import ctypes
        import torch
        from oracle import ref_gpu
    except Exception:
        return None
    if not ref_gpu.available() or not torch.cuda.is_available():
        return None
    R = ref_gpu.lib()
    c = gpt_oss_layer_case(torch)
    s = torch.cuda.current_stream().cuda_stream
    y = torch.empty(1, 4096, device="cuda")
    ws = torch.zeros(64 * 64 * 66 * 4, dtype=torch.uint8, device="cuda")
    ops = (ctypes.c_void_p * 8)(*[c[k].data_ptr() for k in ("qkv", "keys", "values", "table", "lens", "starts", "active", "sinks")])
    out = {}

    def timed(fn, per):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            fn()
        b.record()
        torch.cuda.synchronize()
        return round(a.elapsed_time(b) / 20 / per * 1e3, 2)

    for name, window in (("attention_full_2048", 0), ("attention_window_128", 128)):
        def body():
            for l in range(c["layers"]):
                R.ref_gpu_attention(ops, y.data_ptr(), ws.data_ptr(), 1, 1, c["logical"], c["logical"], 64, 8, 64, l, 16, window, 0, s)
        out[name + "_us"] = timed(body, c["layers"])
    yq = torch.empty(80 * 64, dtype=torch.bfloat16, device="cuda")
    yo = torch.empty(2880, dtype=torch.bfloat16, device="cuda")

    def gemvs():
        R.ref_gpu_decode_gemv(c["x"].data_ptr(), c["w_qkv"].data_ptr(), yq.data_ptr(), 80 * 64, 2880, 2880, 0, 0, 0, 0, 0, s)
        R.ref_gpu_decode_gemv(c["a"].data_ptr(), c["w_o"].data_ptr(), yo.data_ptr(), 2880, 4096, 4096, 0, 0, 0, 0, 0, s)
    out["qkv_and_o_gemv_us"] = timed(gemvs, 1)
    return out


def bench_moe(torch, gb, peaks, args, token_counts=(1, 8, 32, 512, 4096), cpu_rows=True):
    """gpt-oss-120b MoE layer (hidden = intermediate = 2880, 128 experts, top-4, MXFP4), one GPU.
    tok/s per token count; a step = one call of the operator.  To keep weight reads
    out of L2 at small T, a graph holds several calls on different token sets
    (different experts) and the time is divided by their number."""
    H = I = 2880
    E, K = 128, 4
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    u8 = lambda *shape, lo=0, hi=256: torch.randint(lo, hi, shape, dtype=torch.uint8, device="cuda", generator=gen)
    router_w = (torch.randn(E, H, device="cuda", generator=gen) / H ** 0.5).to(torch.bfloat16).float()
    router_b = torch.zeros(E, device="cuda")
    tensors = [router_w, router_b, u8(E, 2 * I, H // 32, 16), u8(E, 2 * I, H // 32, lo=117, hi=124),
               torch.zeros(E, 2 * I, device="cuda"), u8(E, H, I // 32, 16), u8(E, H, I // 32, lo=117, hi=124),
               torch.zeros(E, H, device="cuda")]
    moe = gb.GptOssMoe(H, I, E, K, io_dtype=torch.bfloat16).prepare(*tensors)
    host = [t.cpu().numpy() for t in tensors] if cpu_rows else None      # the same layer for the CPU restatement
    per_expert = 5760 * 2880 // 2 + 5760 * 90 + 2880 * 2880 // 2 + 2880 * 90
    rows = []
    for T in token_counts:
        rot = 16 if T == 1 else (4 if T <= 32 else 1)
        xs = [torch.randn(T, H, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(rot)]
        y = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
        ws = torch.empty(moe.workspace_bytes(T), dtype=torch.uint8, device="cuda")
        distinct = float(np.mean([len(torch.unique(moe.route(x)[1])) for x in xs]))

        def body():
            for x in xs:
                moe.run(x, out=y, workspace=ws)

        steps = max(3, min(args.steps, 20 if T <= 512 else 5))
        ms = time_graph(torch, body, steps, 3) / rot
        assert moe.fault() == 0, "a device-side wait gave up"
        # end to end: pinned host tokens in, the layer, pinned host result out, one synchronisation per call
        xh = [x.cpu().pin_memory() for x in xs]
        yh = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
        xd = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)

        def host_call(i):
            xd.copy_(xh[i % rot], non_blocking=True)
            moe.run(xd, out=y, workspace=ws)
            yh.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(yh[0, 0])

        for i in range(3):
            host_call(i)
        n_e2e = max(3, min(args.steps, 10))
        t0 = time.perf_counter()
        for i in range(n_e2e):
            host_call(i)
        e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
        bytes_ = distinct * per_expert + T * H * 2 * 2
        flops = 199065600.0 * T
        row = {"tokens": T, "ms": round(ms, 4), "tok_per_s": round(T / (ms * 1e-3), 1),
               "distinct_experts": round(distinct, 1), "GBps": round(bytes_ / (ms * 1e-3) / 1e9, 1),
               "hbm_frac": round(bytes_ / (ms * 1e-3) / 1e9 / peaks["hbm"], 4),
               "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 2),
               "tensor_frac_burst": round(flops / (ms * 1e-3) / 1e12 / peaks["tf"], 4),
               "tensor_frac_sustained": round(flops / (ms * 1e-3) / 1e12 / peaks["tf_sus"], 4), "calls_per_graph": rot,
               "e2e": {"ms": round(e2e_ms, 4), "tok_per_s": round(T / (e2e_ms * 1e-3), 1), "h2d_bytes_per_step": T * H * 2,
                       "d2h_bytes_per_step": T * H * 2}}
        if cpu_rows:
            row["cpu_baseline"] = moe_cpu_baseline(host, xs[0].float().cpu().numpy(), H, I, E, K)
        rows.append(row)
    del moe
    torch.cuda.empty_cache()
    return rows


def moe_cpu_baseline(host, x, H, I, E, K, budget_s=12.0):
    """The reference has no production CPU MoE; this times the C/OpenMP restatement of its
    arithmetic (oracle.moe_route + oracle.moe_experts) on the host cores, on all tokens
    when that fits the time budget, else on a leading subset (stated)."""
    import oracle
    T = x.shape[0]
    threads = os.cpu_count() or 1
    # a token costs 4 experts x 24.9 M multiply-adds with on-the-fly MXFP4 decode: ~0.15 s on one core
    est_per_token = 0.15 / max(1, min(threads, 16))
    sample = int(max(1, min(T, budget_s / est_per_token)))
    if sample < T:
        sample = max(threads, sample // threads * threads)
        sample = min(sample, T)
    xs = np.ascontiguousarray(x[:sample])
    t0 = time.perf_counter()
    _, sel, pr = oracle.moe_route(xs, host[0], host[1], E, K)
    oracle.moe_experts(xs, sel, pr, host[2], host[3], host[4].reshape(-1), host[5], host[6], host[7].reshape(-1), H, I, E, K)
    dt = time.perf_counter() - t0
    return {"value": round(sample / dt, 2), "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{sample} of {T} tokens (route + experts, C restatement with OpenMP over tokens), {dt:.1f} s"}


def bench_moe_ep(torch, dist, gb, args, rank, world, tokens_total=8192):
    """gpt-oss-120b MoE layer, expert parallel over `world` GPUs: 128/world experts per GPU,
    tokens_total tokens split evenly over the ranks, Zipf(1.1)-skewed expert popularity; rows
    and values travel by peer stores over NVLink (garnet_b200_moe_ep_run: no host
    synchronisation, no library collective).  Experts are placed by popularity (most popular
    first, dealt to the ranks in snake order) within the experts/world-per-GPU rule; the
    imbalance of plain contiguous blocks is reported beside it.  tok/s = tokens_total / time
    (device time, max over ranks).  With world = 1 the same call runs on one GPU (the anchor
    of the scaling curve).  Every rank also holds the whole layer once, to check its slice
    of the output against the single-GPU operator."""
    from garnet_b200.dist import Comm, ExpertParallel, ep_arena_bytes
    H = I = 2880
    E, K = 128, 4
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)                       # same weights on every rank; each keeps its block
    u8 = lambda *shape, lo=0, hi=256: torch.randint(lo, hi, shape, dtype=torch.uint8, device="cuda", generator=gen)
    router_w = (torch.randn(E, H, device="cuda", generator=gen) / H ** 0.5).to(torch.bfloat16).float()
    perm = torch.randperm(E, device="cuda", generator=gen).float() + 1.0
    pop = perm ** -1.1
    router_b = torch.log(pop / pop.sum() * E).to(torch.bfloat16).float()
    gu_b, gu_s = u8(E, 2 * I, H // 32, 16), u8(E, 2 * I, H // 32, lo=117, hi=124)
    dn_b, dn_s = u8(E, H, I // 32, 16), u8(E, H, I // 32, lo=117, hi=124)
    # placement: experts sorted by popularity, dealt to the ranks in snake order, then renumbered so
    # that rank r owns the contiguous block [r * per, (r + 1) * per) of the new numbering
    per = E // world
    by_pop = torch.argsort(pop, descending=True).tolist()
    owner_lists = [[] for _ in range(world)]
    for i, e in enumerate(by_pop):
        r = i % (2 * world)
        owner_lists[r if r < world else 2 * world - 1 - r].append(e)
    order = torch.tensor([e for lst in owner_lists for e in lst], device="cuda")
    router_w, router_b = router_w[order].contiguous(), router_b[order].contiguous()
    gu_b, gu_s, dn_b, dn_s = gu_b[order].contiguous(), gu_s[order].contiguous(), dn_b[order].contiguous(), dn_s[order].contiguous()
    zeros_up, zeros_dn = torch.zeros(E, 2 * I, device="cuda"), torch.zeros(E, H, device="cuda")
    full = gb.GptOssMoe(H, I, E, K, io_dtype=torch.bfloat16).prepare(router_w, router_b, gu_b, gu_s, zeros_up, dn_b, dn_s, zeros_dn)
    lo = rank * per
    if world > 1:
        moe = gb.GptOssMoe(H, I, E, K, io_dtype=torch.bfloat16, ep_rank=rank, ep_world=world,
                           expert_weights_sharded=True).prepare(
            router_w, router_b, gu_b[lo:lo + per].contiguous(), gu_s[lo:lo + per].contiguous(),
            zeros_up[:per].contiguous(), dn_b[lo:lo + per].contiguous(), dn_s[lo:lo + per].contiguous(), zeros_dn[:per].contiguous())
    else:
        moe = full
    t_local = tokens_total // world
    gx = torch.Generator(device="cuda")
    gx.manual_seed(1000 + rank)
    x = torch.randn(t_local, H, device="cuda", generator=gx).to(torch.bfloat16)
    comm = Comm(ep_arena_bytes(moe, world, t_local) + (1 << 20))
    ep = ExpertParallel(moe, comm, t_local)
    y = torch.empty_like(x)
    for _ in range(3):
        ep.run(x, out=y)
    torch.cuda.synchronize()
    expected = full.run(x)
    err = ((y.float() - expected.float()).abs() / (1 + expected.float().abs())).max()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    steps = max(3, min(args.steps, 10))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        ep.run(x, out=y)
    b.record()
    torch.cuda.synchronize()
    assert comm.fault() == 0 and moe.fault() == 0, "a device-side wait gave up"
    ms = a.elapsed_time(b) / steps
    # what contiguous blocks of the original numbering would have put on one GPU
    _, sel, _ = full.route(x)
    original = order[sel.reshape(-1).long()]
    contiguous_rows = torch.bincount(torch.div(original, per, rounding_mode="floor"), minlength=world).float()
    t = torch.tensor([ms, float(ep.rows_received()), float(err)], device="cuda")
    tmax, tsum = t.clone(), t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        dist.all_reduce(contiguous_rows, op=dist.ReduceOp.SUM)
    ms = float(tmax[0].item())
    return {"tokens": tokens_total, "ms": round(ms, 4), "tok_per_s": round(tokens_total / (ms * 1e-3), 1),
            "experts_per_gpu": per, "routing": "zipf(1.1) popularity over a seeded permutation",
            "placement": "experts dealt to the ranks by popularity (snake order)",
            "exchange": "peer stores over NVLink inside garnet_b200_moe_ep_run (no host synchronisation, no library collective)",
            "max_rows_on_one_gpu": int(tmax[1].item()), "mean_rows_per_gpu": round(float(tsum[1].item()) / world, 1),
            "max_rows_with_contiguous_blocks": int(contiguous_rows.max().item()),
            "TFLOPs": round(199065600.0 * tokens_total / (ms * 1e-3) / 1e12, 2),
            "parity_max_scaled_err_vs_single_gpu_operator": float(tmax[2].item())}


# ------------------------------------------------------------- CPU baseline

def cpu_linears():
    """The 197 linears of the decode pass as CPU operators, each with its own weights.
    Uses the reference's own compiled operator when oracle/_ref is present, else the
    restatement in oracle/oracle.c."""
    import oracle
    import oracle.ref as ref
    rng = np.random.default_rng(0)
    threads = min(16, os.cpu_count() or 1)      # the reference's pool is capped at 16 threads
    kind = "reference" if ref.available() else "port"
    ops = []
    xs = {k: rng.normal(0, 1, size=k).astype(np.float32) for k in (2048, 6144)}
    for name, k, n in PROJ * LAYERS + [LM_HEAD]:
        nib = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
        sc = (np.abs(rng.normal(0, 0.02, size=(n, k // GROUP))) / 7.0).astype(np.float32)
        x = xs[k]
        if kind == "reference":
            op = ref.Q4Q8Linear(nib, sc, n, k, GROUP)
            y = np.empty(n, np.float32)
            ops.append((name, k, n, (lambda op=op, x=x, y=y: op.forward(x, threads, out=y))))
        else:
            ops.append((name, k, n, (lambda nib=nib, sc=sc, n=n, k=k, x=x: oracle.q4q8_forward(nib, sc, n, k, GROUP, x, threads))))
    return ops, kind, threads


def cpu_baseline(sample_seconds=10.0):
    ops, kind, threads = cpu_linears()
    bytes_pass = sum(algo_bytes(k, n, 1) for (_, k, n, _) in ops)
    for (_, _, _, fn) in ops:
        fn()
    t0 = time.perf_counter()
    passes = 0
    while time.perf_counter() - t0 < sample_seconds or passes < 3:
        for (_, _, _, fn) in ops:
            fn()
        passes += 1
    dt = time.perf_counter() - t0
    return {"value": round(bytes_pass * passes / dt / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{passes} full decode passes (197 linears at M=1, {bytes_pass} B each), "
                      f"Q4Q8Linear::Forward (int8 activations), {dt:.1f} s"}


def reference_gpu_moe(token_counts=(1, 8, 32, 512, 4096)):
    """The reference's own GPU MoE on this box (oracle/_ref/libgarnet_ref_gpu.so, compiled unchanged from
    its sources): the gpt-oss-120b layer of bench_moe (same seed, same tensors), through RunGptOssMoe (the
    scalar path below 16 tokens, the grouped WMMA path from 16) and through GptOssMarlin::Run, the
    production GEMM.  Marlin takes 8 tokens at most in its default configuration; for the larger counts
    the reference's documented opt-in is set (GARNET_GPT_OSS_MARLIN_MAX_TOKENS=4096 with
    GARNET_GPT_OSS_MARLIN_PREFILL_BLOCK=32) and the rows say so.  CUDA events around repeated calls on
    rotating inputs; None when the library or a GPU is absent."""
    try:
        import torch
        from oracle import ref_gpu
    except Exception:
        return None
    if not ref_gpu.available() or not torch.cuda.is_available():
        return None
    os.environ.setdefault("GARNET_GPT_OSS_MARLIN_MAX_TOKENS", "4096")
    os.environ.setdefault("GARNET_GPT_OSS_MARLIN_PREFILL_BLOCK", "32")
    H = I = 2880
    E, K = 128, 4
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    u8 = lambda *shape, lo=0, hi=256: torch.randint(lo, hi, shape, dtype=torch.uint8, device="cuda", generator=gen)   # noqa: E731
    router_w = (torch.randn(E, H, device="cuda", generator=gen) / H ** 0.5).to(torch.bfloat16).float()
    tensors = [router_w, torch.zeros(E, device="cuda"), u8(E, 2 * I, H // 32, 16), u8(E, 2 * I, H // 32, lo=117, hi=124),
               torch.zeros(E, 2 * I, device="cuda"), u8(E, H, I // 32, 16), u8(E, H, I // 32, lo=117, hi=124),
               torch.zeros(E, H, device="cuda")]
    rows = []
    for T in token_counts:
        prefill = 1 if T > 8 else 0
        ref = ref_gpu.RefMoe(H, I, E, K, tensors, prefill=prefill)
        rot = 16 if T == 1 else (4 if T <= 32 else 1)
        xs = [torch.randn(T, H, device="cuda", generator=gen).to(torch.bfloat16).float() for _ in range(rot)]
        y = torch.empty(T, H, device="cuda")
        row = {"tokens": T}
        for name, fn in (("RunGptOssMoe", ref.run), ("GptOssMarlin", ref.run_marlin)):
            rc, _ = fn(xs[0], out=y)
            torch.cuda.synchronize()
            if rc != 0:
                row[name] = {"status": int(rc), "note": "cudaErrorNotSupported: the reference falls back" if rc == 801 else "error"}
                continue
            reps = 3 if T > 512 and name == "RunGptOssMoe" else 10
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for r in range(reps):
                for x in xs:
                    fn(x, out=y)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / (reps * rot)
            row[name] = {"ms": round(ms, 4), "tok_per_s": round(T / (ms * 1e-3), 1)}
            if name == "GptOssMarlin" and T > 8:
                row[name]["config"] = "GARNET_GPT_OSS_MARLIN_MAX_TOKENS=4096 GARNET_GPT_OSS_MARLIN_PREFILL_BLOCK=32, prefill=1"
        ref.close()
        rows.append(row)
    return rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ops, kind, threads = cpu_linears()
    bytes_pass = sum(algo_bytes(k, n, 1) for (_, k, n, _) in ops)
    for _ in range(max(1, args.warmup)):
        for (_, _, _, fn) in ops:
            fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for (_, _, _, fn) in ops:
            fn()
    dt = (time.perf_counter() - t0) / args.steps
    value = bytes_pass / dt / 1e9
    sample = (f"each step = the full decode pass, 197 linears at M=1 ({bytes_pass} B), Q4Q8Linear::Forward on host cores")
    moe_gpu = None if args.no_moe else reference_gpu_moe()
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_weight_GBps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int4 -> int32 (W4A8)",
        "data": "synthetic",
        "config": {"workload": "qwen3_1p7b_w4a16_sweep: decode pass M=1 over 28x7 projections + lm_head (197 int4 group-128 linears)",
                   "bytes_per_step": bytes_pass},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "moe_reference_gpu": moe_gpu,
        "gpt_oss_layer_ops_reference_gpu": None if args.no_moe else reference_gpu_layer_ops(),
    }), flush=True)


def run_profile_case(spec):
    """Small fixed case for profiler captures: `w4a16:K:N:M[:copies]` runs one linear
    a few times without a graph (one warm-up and one measured rotation over `copies`
    weight copies, at least 3 launches each) and prints the
    CUDA-event time per launch; `moe:T` runs the MoE layer on T tokens."""
    import torch

    import garnet_b200 as gb

    torch.cuda.set_device(0)
    if spec.startswith("moe:"):
        # `moe:T`: the gpt-oss-120b MoE layer on T tokens, 2 warm-up calls + 2 timed calls
        class A:
            steps = 2
        rows = bench_moe(torch, gb, measured_peaks(), A, token_counts=(int(spec.split(":")[1]),), cpu_rows=False)
        print(json.dumps({"case": spec, **rows[0]}))
        return
    if spec.startswith("list:"):
        # `list:L[:head]`: the headline's launch on L layers (7 projections each, M = 1), with
        # the lm_head when `head` is given; 3 warm-up launches + 3 timed ones, no graph.
        # `list:4` holds 0.2 GB of weights, more than the L2.
        f = spec.split(":")
        nl, with_head = int(f[1]), len(f) > 2 and f[2] == "head"
        gen = torch.Generator(device="cuda")
        gen.manual_seed(1234)
        xs = {k: torch.randn(1, k, device="cuda", generator=gen).to(torch.bfloat16) for k in (2048, 6144)}
        calls, nbytes = [], 0
        for _ in range(nl):
            for (_, k, n) in PROJ:
                calls.append((make_linear(torch, gb, k, n, gen), xs[k], torch.empty(1, n, device="cuda", dtype=torch.bfloat16)))
                nbytes += algo_bytes(k, n, 1)
        if with_head:
            _, k, n = LM_HEAD
            calls.append((make_linear(torch, gb, k, n, gen), xs[k], torch.empty(1, n, device="cuda", dtype=torch.bfloat16)))
            nbytes += algo_bytes(k, n, 1)
        lst = gb.LinearList(calls, m=1)
        for _ in range(3):
            lst.run()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            lst.run()
        b.record()
        torch.cuda.synchronize()
        assert lst.fault() == 0
        us = a.elapsed_time(b) / 3 * 1e3
        print(json.dumps({"case": spec, "linears": len(calls), "algorithmic_bytes": nbytes,
                          "us_per_launch_no_graph": round(us, 3), "GBps": round(nbytes / us / 1e3, 1)}))
        return
    parts = spec.split(":")
    kind, k, n, m = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    copies = int(parts[4]) if len(parts) > 4 else 2      # weight copies rotated through (to defeat L2)
    assert kind == "w4a16"
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    lins = [make_linear(torch, gb, k, n, gen) for _ in range(copies)]
    x = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
    y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    reps = max(3, copies)
    for i in range(reps):
        lins[i % copies].forward(x, out=y)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        lins[i % copies].forward(x, out=y)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) / reps * 1e3
    print(json.dumps({"case": spec, "us_per_launch": round(us, 3),
                      "GBps": round(algo_bytes(k, n, m) / us / 1e3, 1)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-moe", action="store_true")
    ap.add_argument("--profile", default=None,
                    help="w4a16:K:N:M[:copies] | moe:T | list:L[:head] - run one small case for a profiler capture")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args.profile)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
