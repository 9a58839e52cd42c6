#!/usr/bin/env python
"""Benchmark of the Kascade sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the Llama-3.1-8B-shaped prefill attention stack at 32 768 tokens —
32 layers, anchors {0,2,8,13,14}, batch 1, 32 query / 8 KV heads, head_dim 128, fp16, tile 32,
Top-k 10 %, rolling prefill, seeded synthetic Q/K/V with heavy-hitter keys.  One "step" is one
pass of all 32 attention layers through ``EfficientKascadeStrategy.attention_forward``.
The same JSON line also carries the paged sparse-decode configuration (batch 64, context 32 768,
16-token pages) under "decode", dense attention on the same GPU under "dense", the roofline of the
dominant kernel and the CPU baseline (the oracle port on the host cores).

With N > 1 (launched by torch.distributed.run) the KV heads of every layer are sharded over the
ranks (strong scaling); the anchors' index rows are all-gathered over NCCL because a reuse head may
map to an anchor head of another shard, per-head outputs are all-gathered at the end of each layer.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode attn µs/step & prefill attn ms @32k, 10% top-k, vs dense on B200"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "tflops_burst": p["bf16_tflops"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


class _Module:
    def __init__(self, layer_idx, groups=4):
        self.layer_idx = layer_idx
        self.num_key_value_groups = groups
        self.training = False


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (every 100 ms, each sample with nvidia-smi's own
    timestamp) and reports those that fall into a window of host time.  nvidia-smi takes a good part of a second to
    produce its first sample, so the sampler is started before the warm-up."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.thread = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t_begin=None, t_end=None):
        """t_begin / t_end: datetime.now() taken around the window; None = every sample."""
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in list(self.lines):
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                when = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                clock, top = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if (t_begin is not None and when < t_begin) or (t_end is not None and when > t_end):
                continue
            sm.append(clock)
            mx = top
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _time_cuda(fn, reps: int):
    """Mean milliseconds of fn() over reps back-to-back calls, CUDA events on the current stream."""
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for i in range(reps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's own PyTorch KascadeStrategy (staged by oracle/make_ref.py into the
# git-ignored oracle/_ref/) on the host cores; the oracle port only where those files are absent
# ------------------------------------------------------------------------------------------------
class _RefModule:
    training = False

    def __init__(self, layer_idx, groups):
        self.layer_idx = layer_idx
        self.num_key_value_groups = groups


def _reference_strategy(wl, block_size=512):
    """The reference's unmodified KascadeStrategy for workload `wl` (kind "reference"), or the oracle port
    (kind "port") when oracle/_ref is not staged.  Returns (kind, run) with run(layer, q, k, v, mask) -> out."""
    import tempfile
    import numpy as np
    from oracle import make_ref
    scaling = wl.D ** -0.5
    if make_ref.available():
        KS = make_ref.load_reference_strategy()
        with tempfile.TemporaryDirectory() as wd:           # the class reads ./results/head_mappings/<model>_layers_<..>.npy
            os.makedirs(os.path.join(wd, "results", "head_mappings"))
            np.save(os.path.join(wd, "results", "head_mappings",
                                 f"bench_layers_{'_'.join(map(str, wl.anchors))}.npy"),
                    np.asarray(wl.head_mapping(), dtype=np.int32))
            cwd = os.getcwd()
            os.chdir(wd)
            try:
                strat = KS(recompute_layers=list(wl.anchors), model_name="x/bench", k=wl.pct, tile_size=wl.tile,
                           rolling_prefill=wl.rolling, block_size=block_size)
            finally:
                os.chdir(cwd)
        groups = wl.H // wl.G
        return "reference", lambda layer, q, k, v, mask: strat.attention_forward(_RefModule(layer, groups), q, k, v,
                                                                                  mask, scaling)[0]
    from oracle.kascade_oracle import KascadeOracle
    orc = KascadeOracle(recompute_layers=wl.anchors, head_mapping=wl.head_mapping(), k=wl.pct, tile_size=wl.tile,
                        rolling_prefill=wl.rolling, row_block=block_size)
    return "port", lambda layer, q, k, v, mask: orc.attention_forward(layer, q, k, v, scaling)


def cpu_prefill_sample(seq_len: int, target_len: int = 32768, n_anchor: int = 4, n_reuse: int = 27):
    """Times one layer of each kind (layer 0, reuse, anchor > 0) of the reference's CPU strategy at `seq_len`
    tokens, fp32, and extrapolates the stack (1 + n_anchor + n_reuse layers) at `target_len` tokens by the L^2
    work ratio.  Returns (stack_ms, [t_layer0, t_reuse, t_anchor] in seconds, kind)."""
    from bench_workloads import PrefillWorkload
    wl = PrefillWorkload(seq_len=seq_len, layers=3, anchors=(0, 2))
    kind, run = _reference_strategy(wl)
    fmin = torch.finfo(torch.float32).min
    mask = torch.full((seq_len, seq_len), fmin).triu_(1)[None, None]
    times = []
    with torch.no_grad():
        for layer in range(3):
            q, k, v = wl.layer_inputs(layer, "cpu")
            q, k, v = (x.float().transpose(1, 2).contiguous() for x in (q, k, v))
            t0 = time.perf_counter()
            run(layer, q, k, v, mask)
            times.append(time.perf_counter() - t0)
    scale = (target_len / seq_len) ** 2
    stack_ms = (times[0] + n_anchor * times[2] + n_reuse * times[1]) * scale * 1e3
    return stack_ms, times, kind


def prefill_config(wl, world=1, parallelism=None):
    """The `config` object of the JSON line; the reference arm prints the same keys for the same workload."""
    name = ("llama31_8b_prefill_attention_stack_32k" if wl.seq_len == 32768 and not wl.qk_norm else
            f"qwen3_8b_prefill_attention_stack_{wl.seq_len}_qknorm" if wl.qk_norm else
            f"llama31_8b_prefill_attention_stack_{wl.seq_len}")
    return {"workload": name, "layers": wl.layers, "anchors": list(wl.anchors), "seq_len": wl.seq_len, "batch": wl.B,
            "q_heads": wl.H, "kv_heads": wl.G, "head_dim": wl.D, "topk_pct": wl.pct, "tile": wl.tile,
            "rolling": wl.rolling, "parallelism": parallelism or f"kv-head shard x{world}",
            "cache_policy": f"inputs larger than L2 ({wl.seq_len * (wl.H + 2 * wl.G) * wl.D * 2 / 1e6:.0f} MB "
                            f"per layer, {wl.layers} distinct layers)"}


def run_reference(args, rank):
    """--impl reference: the reference's CPU implementation of the path — its own PyTorch KascadeStrategy,
    unmodified, from oracle/_ref — on all host threads, same metric, unit and config as the GPU arm.  A step is
    a bounded sample: one layer of each kind at a sample length chosen so that the whole run stays within a few
    minutes; `value` is the 32-layer stack at 32 768 tokens extrapolated from it by the L^2 work ratio."""
    if rank != 0:
        return
    from bench_workloads import PrefillWorkload
    torch.set_num_threads(max(os.cpu_count() or 1, 1))     # a launcher may have pinned OMP_NUM_THREADS to 1
    cores = torch.get_num_threads()
    wl = PrefillWorkload()
    budget_s = 150.0
    n_runs = max(args.steps, 1) + max(args.warmup, 0)
    L = 1024
    _, probe_times, kind = cpu_prefill_sample(L)
    t_probe = sum(probe_times) * 1.25                       # + input generation and the mask
    while L < 8192 and t_probe * 4.4 * n_runs <= budget_s:  # the work grows ~4x per doubling of L
        L *= 2
        t_probe *= 4.4
    for _ in range(args.warmup):
        cpu_prefill_sample(L)
    t0 = time.perf_counter()
    samples = [cpu_prefill_sample(L) for _ in range(max(args.steps, 1))]
    wall = (time.perf_counter() - t0) / max(args.steps, 1)
    value = sum(s[0] for s in samples) / len(samples)
    tl = [sum(s[1][i] for s in samples) / len(samples) for i in range(3)]
    what = ("the reference's own KascadeStrategy (unmodified, oracle/_ref)" if kind == "reference"
            else "oracle port (oracle/_ref not staged)")
    sample = (f"{what}, fp32, {cores} threads, block_size 512: measured at L={L} layer 0 {tl[0]:.2f}s, reuse {tl[1]:.2f}s, "
              f"anchor>0 {tl[2]:.2f}s per layer; value = 32-layer stack at 32768 tokens extrapolated by (32768/{L})^2 "
              f"with 1/27/4 layer weights")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall * 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": prefill_config(wl, max(args.gpus, 1)),
            "measured": {"seq_len": L, "layer0_s": tl[0], "reuse_s": tl[1], "anchor_s": tl[2],
                         "extrapolation": f"(32768/{L})^2, 1 layer-0 + 27 reuse + 4 anchor layers"},
            "cpu_baseline": {"value": value, "unit": "ms", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def sharded_self_check(rank, world, dev, exchange, seq_len=2048):
    """N > 1: every rank runs three layers (layer 0, a reuse layer, an anchor > 0) of a short prompt both through
    the head-sharded strategy with the benchmark's exchange mode and through an unsharded strategy over all heads
    on its own GPU, and compares the gathered [B, L, H, D] outputs of every layer bit for bit.  Returns "ok" or a
    description of the first difference (the same string on all ranks)."""
    import torch.distributed as dist
    from bench_workloads import PrefillWorkload
    from kascade_b200 import EfficientKascadeStrategy
    wl = PrefillWorkload(seq_len=seq_len, layers=3, anchors=(0, 2))
    gpr = wl.G // world
    heads = list(range(rank * gpr, (rank + 1) * gpr))
    kw = dict(k=wl.pct, tile_size=wl.tile, rolling_prefill=wl.rolling, head_mapping=wl.head_mapping(), register=False)
    full = EfficientKascadeStrategy(list(wl.anchors), "x/check", **kw)
    part = EfficientKascadeStrategy(list(wl.anchors), "x/check", shard=(rank, world), exchange=exchange, **kw)
    worst, where = 0.0, None
    for layer in range(wl.layers):
        q, k, v = wl.layer_inputs(layer, dev)
        ref, _ = full.attention_forward(_Module(layer), q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None,
                                        wl.D ** -0.5)
        hg = wl.H // wl.G
        qh = [g * hg + i for g in heads for i in range(hg)]
        part.attention_forward(_Module(layer), q[:, :, qh].contiguous().transpose(1, 2),
                               k[:, :, heads].contiguous().transpose(1, 2), v[:, :, heads].contiguous().transpose(1, 2),
                               None, wl.D ** -0.5)
        part.wait_gathers()
        torch.cuda.synchronize()
        got = part.gathered_out
        if got.dim() == 5:                                            # NCCL layout [world, B, L, H/world, D]
            got = torch.cat([got[r] for r in range(world)], dim=2)
        diff = (got.float() - ref.float()).abs().max().item()
        if diff > worst:
            worst, where = diff, layer
        dist.barrier()                                                # nobody overwrites a buffer a peer still compares
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    del full, part
    torch.cuda.empty_cache()
    return "ok" if float(t.item()) == 0.0 else f"gathered outputs differ from the unsharded run by up to {float(t.item()):.3e}"


def bench_decode(args, dev, world, peaks, batch=None, ragged=False, rank=0):
    """Paged sparse decode, Llama-3.1-8B shape: batch 64 (split over the ranks), every sequence at context
    32 768, 16-token pages behind a seeded random block table, 32 layers with anchors {0,2,8,13,14}."""
    import torch.distributed as dist
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    from bench_workloads import DecodeWorkload
    scaling = 128 ** -0.5
    if ragged:                                                    # 256 sequences, contexts uniform in [4096, 65536]
        dw = DecodeWorkload.ragged(rank=rank, world=world, distinct_caches=2)
    else:
        dw = DecodeWorkload() if batch is None else DecodeWorkload(batch=batch)
        assert dw.batch % world == 0
        dw.batch //= world                                        # batch-sharded across ranks
    dstrat = EfficientKascadeStrategy(list(dw.anchors), "synthetic/llama31-8b-shape", k=dw.pct, tile_size=32,
                                      rolling_prefill=True, head_mapping=dw.head_mapping(), register=False)
    caches = [dw.make_cache(i, dev) for i in range(dw.distinct_caches)]
    qs = [dw.query(l, dev) for l in range(dw.layers)]
    seq_lens = torch.tensor(dw.seq_lens(), dtype=torch.int32, device=dev)
    mean_len = sum(dw.seq_lens()) / len(dw.seq_lens())            # the host knows its batch: a hint for the split count
    dout = {}

    def dstep(_i=0):
        for l in range(dw.layers):
            kc, vc, bt = caches[l % len(caches)]
            dout["o"] = dstrat.paged_decode_forward(l, qs[l], kc, vc, bt, seq_lens, scaling, dw.context, mean_seq_len=mean_len)

    for _ in range(args.warmup):
        dstep()
    if world > 1:
        dist.barrier()
    n0 = nat.launch_count
    t = torch.tensor([_time_cuda(dstep, args.steps)], device=dev)
    dl = (nat.launch_count - n0) // max(args.steps, 1)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us_eager = float(t.item()) * 1e3
    # the same step captured once into a CUDA graph and replayed (every buffer of the step exists after
    # the warm-up; the library allocates nothing and never synchronises)
    us_graph, graph_note = None, None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dstep()
        for _ in range(max(args.warmup, 1)):
            graph.replay()
        tg = torch.tensor([_time_cuda(lambda i: graph.replay(), args.steps)], device=dev)
        if world > 1:
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        us_graph = float(tg.item()) * 1e3
    except Exception as e:                                         # noqa: BLE001 - reported in the JSON line
        graph_note = f"{type(e).__name__}: {e}"[:200]
        torch.cuda.synchronize()
    us_step = min(us_graph, us_eager) if us_graph is not None else us_eager
    # reuse-layer kernel alone (the dominant decode kernel by launches: 27 of 32 layers)
    kc, vc, bt = caches[0]
    kv = nat.kv_layout_paged(kc, vc, bt)
    o = torch.empty(dw.batch, dw.H, dw.D, dtype=torch.float16, device=dev)
    kmax = dstrat._dec_kmax
    splits = nat.decode_default_splits(dw.batch, dw.G, kmax)
    ws = nat.decode_workspace(dw.batch, dw.H, splits, dev)

    def reuse(i):
        kc, vc, bt = caches[i % len(caches)]
        nat.decode_sparse_paged(qs[i % len(qs)], nat.kv_layout_paged(kc, vc, bt), dstrat._dec_idx, dstrat._dec_count,
                                kmax, None, scaling, o, None, ws, splits)
    reuse(0)
    t_reuse = _time_cuda(reuse, 20) * 1e3
    # dense decode of all layers with the library's own dense pass, for the "vs dense" figure
    stride = -(-dw.context // 4) * 4
    logits = torch.empty(dw.batch, dw.H, stride, dtype=torch.float32, device=dev)
    pooled = torch.empty(dw.batch, dw.G, stride, dtype=torch.float32, device=dev)
    lse2 = torch.empty(dw.batch, dw.H, dtype=torch.float32, device=dev)
    sa = nat.decode_default_splits(dw.batch, dw.G, dw.context)
    wsa = nat.decode_workspace(dw.batch, dw.H, sa, dev)

    # the same reuse layer over an FP8 (e4m3) copy of the cache, one scale per (page, KV head)
    fp8 = None
    try:
        kc, vc, bt = caches[0]
        k8, v8 = torch.empty_like(kc, dtype=torch.float8_e4m3fn), torch.empty_like(vc, dtype=torch.float8_e4m3fn)
        ks = torch.empty(kc.shape[0], kc.shape[2], dtype=torch.float32, device=dev)
        vs = torch.empty_like(ks)
        step_pages = max(1, kc.shape[0] // 32)
        for s0 in range(0, kc.shape[0], step_pages):               # bounded fp32 temporaries
            for src, dst8, sc in ((kc, k8, ks), (vc, v8, vs)):
                x = src[s0:s0 + step_pages].float()
                a = x.abs().amax(dim=(1, 3)).clamp(min=1e-6) / 448.0
                sc[s0:s0 + step_pages] = a
                dst8[s0:s0 + step_pages] = (x / a[:, None, :, None]).to(torch.float8_e4m3fn)
        kv8 = nat.kv_layout_paged(k8, v8, bt, ks, vs)
        o8 = torch.empty_like(o)
        f8 = lambda i: nat.decode_sparse_paged(qs[i % len(qs)], kv8, dstrat._dec_idx, dstrat._dec_count, kmax, None, scaling,
                                               o8, None, ws, splits)
        f8(0)
        t8 = _time_cuda(f8, 20) * 1e3
        d8 = lambda i: nat.decode_anchor_paged(qs[i % len(qs)], kv8, seq_lens, dw.context, scaling, logits, pooled, o8, lse2,
                                               wsa, sa)
        d8(0)
        t8_dense = _time_cuda(d8, 8) * 1e3
        keys = dw.G * sum(min(dstrat._dec_kmax, n) for n in dw.seq_lens())
        bytes8 = keys * (2 * dw.D + 4 + 8) + 2 * dw.batch * dw.H * dw.D * 2
        fp8 = {"reuse_layer_us": t8, "algorithmic_mb": bytes8 / 1e6, "achieved_gbs": bytes8 / (t8 * 1e-6) / 1e9,
               "frac": bytes8 / (t8 * 1e-6) / 1e9 / peaks["hbm_gbs"], "speedup_vs_fp16_cache": t_reuse / t8,
               "dense_layer_us": t8_dense, "dense_layer_gbs": dw.bytes_dense_k() / (t8_dense * 1e-6) / 1e9,
               "note": "e4m3 cache, one fp32 scale per (16-token page, KV head): half the cache bytes; the MMA operands are "
                       "made from the stored bytes in registers; this cache alone is the working set here (4.3 GB, "
                       "larger than L2)"}
        del k8, v8, ks, vs, kv8
    except Exception as ex:                                          # noqa: BLE001 - reported in the JSON line
        fp8 = {"error": f"{type(ex).__name__}: {ex}"[:200]}
    def dense_dec(i):
        kc, vc, bt = caches[i % len(caches)]
        nat.decode_anchor_paged(qs[i % len(qs)], nat.kv_layout_paged(kc, vc, bt), seq_lens, dw.context, scaling, logits,
                                pooled, o, lse2, wsa, sa)
    dense_dec(0)
    t_dense = _time_cuda(dense_dec, 8) * 1e3
    if fp8 and "dense_layer_us" in fp8:
        fp8["dense_speedup_vs_fp16_cache"] = t_dense / fp8["dense_layer_us"]
    gbs_reuse = dw.bytes_reuse() / (t_reuse * 1e-6) / 1e9
    decode = {"us_per_step": us_step, "us_per_step_eager": us_eager, "us_per_step_graph": us_graph,
              "cuda_graph": us_graph is not None,
              "cuda_graph_note": graph_note, "layers": dw.layers, "batch_per_gpu": dw.batch,
              "context": dw.context if dw.contexts is None else f"ragged, {min(dw.contexts)}..{max(dw.contexts)}",
              "page": dw.page, "topk": dw.budget(), "distinct_layer_caches": dw.distinct_caches,
              "gpu_launches": dl,
              "algorithmic_gb_per_step": dw.bytes_step() / 1e9,
              "achieved_gbs_step": dw.bytes_step() / (us_step * 1e-6) / 1e9,
              "frac_step": dw.bytes_step() / (us_step * 1e-6) / 1e9 / peaks["hbm_gbs"],
              "reuse_layer_us": t_reuse,
              "roofline": {"kernel": "decode_attn_kernel<sparse>", "bound": "hbm", "achieved": gbs_reuse,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs_reuse / peaks["hbm_gbs"],
                           # dram__bytes_read + write of the ncu capture at batch 8, context 32 768 (110.5 MB per launch,
                           # profiles/decode_sparse_paged_ncu.md), scaled by the gathered keys: every row is touched once
                           "traffic": (110.5e6 * dw.bytes_reuse() / DecodeWorkload(batch=8).bytes_reuse()),
                           "traffic_note": "bytes per launch, ncu capture at batch 8 scaled by the gathered keys",
                           "peak_source": peaks["source"]},
              "fp8_cache": fp8,
              "dense_layer_us": t_dense, "dense_us_per_step": t_dense * dw.layers,
              "dense_layer_gbs": 2 * dw.bytes_dense_k() / (t_dense * 1e-6) / 1e9,
              "speedup_vs_dense": t_dense * dw.layers / us_step}
    del caches, logits, pooled
    torch.cuda.empty_cache()
    return decode


def bench_decoder_generate(args, dev, world, rank):
    """The long-reasoning decode as a whole decoder: a random-init Llama-3.1-8B-architecture stack (32 layers, hidden
    4096, SwiGLU 14336, 32 / 8 heads, RoPE theta 500000, fp16, weights N(0, 0.02)) generates `--gen-tokens` tokens for
    256 sequences with contexts uniform in [4096, 65536] (batch-sharded over the ranks, weights replicated, no
    collective).  Per layer the step calls kb200_kv_write (RoPE + paged append) and the Kascade paged decode; the
    dense layers are torch GEMMs.  One step is captured into a CUDA graph and replayed.  The KV caches of 256 such
    sequences for 32 layers (1.2 TB) do not fit one GPU, so `distinct_layer_caches` caches are cycled over the
    layers (the bytes every layer reads are those of a real run; what it appends lands in a shared cache)."""
    import torch.distributed as dist
    from bench_decoder import DecoderConfig, KascadeLlamaDecoder
    from bench_workloads import DecodeWorkload
    gen = int(args.gen_tokens)
    cfg = DecoderConfig()
    dw = DecodeWorkload.ragged(rank=rank, world=world, distinct_caches=2, reserve=gen)
    model = KascadeLlamaDecoder(cfg, dev, dw.head_mapping())
    caches = [dw.make_cache(i, dev) for i in range(dw.distinct_caches)]
    block_table = caches[0][2]                                    # one page table: the caches share their page layout
    caches = [(kc, vc) for kc, vc, _ in caches]
    lens0 = torch.tensor(dw.seq_lens(), dtype=torch.int32, device=dev)
    seq_lens = lens0.clone()
    max_len = dw.context + gen
    tokens = torch.randint(0, cfg.vocab, (dw.batch,), device=dev, generator=torch.Generator(device=dev).manual_seed(11))
    model._qkv_cache = [None] * cfg.layers
    model.mean_len = sum(dw.seq_lens()) / len(dw.seq_lens())

    def step():
        nxt = model.step(tokens, lambda l: caches[l % len(caches)], block_table, seq_lens, max_len)
        tokens.copy_(nxt)
        seq_lens.add_(1)

    for _ in range(3):                                            # warm-up: every scratch buffer of a step exists afterwards
        step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    seq_lens.copy_(lens0)
    for _ in range(2):
        graph.replay()
    seq_lens.copy_(lens0)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_ms = torch.tensor([_time_cuda(lambda i: graph.replay(), gen) * gen], device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    total_ms = float(t_ms.item())
    # the library's part of a step alone: the same kernels on the q / k / v of the last step
    seq_lens.copy_(lens0)
    agraph = torch.cuda.CUDAGraph()
    model.step(tokens, lambda l: caches[l % len(caches)], block_table, seq_lens, max_len, attention_only=True)
    torch.cuda.synchronize()
    with torch.cuda.graph(agraph):
        model.step(tokens, lambda l: caches[l % len(caches)], block_table, seq_lens, max_len, attention_only=True)
    agraph.replay()
    t_att = torch.tensor([_time_cuda(lambda i: agraph.replay(), 16)], device=dev)
    if world > 1:
        dist.all_reduce(t_att, op=dist.ReduceOp.MAX)
    batch_total = 256
    res = {"tokens_per_s": batch_total * gen / (total_ms * 1e-3), "generated_tokens_per_sequence": gen,
           "ms_per_token_step": total_ms / gen, "attention_us_per_step": float(t_att.item()) * 1e3,
           "attention_share": float(t_att.item()) / (total_ms / gen), "batch_total": batch_total, "batch_per_gpu": dw.batch,
           "contexts": f"uniform {min(dw.contexts)}..{max(dw.contexts)} on this rank, seed 0", "cuda_graph": True,
           "model": "random-init Llama-3.1-8B architecture: 32 layers, hidden 4096, SwiGLU 14336, 32/8 heads, RoPE theta "
                    "500000, vocab 128256 (tied), fp16, weights N(0, 0.02)",
           "per_layer": "torch GEMMs (qkv, o, gate/up, down) + kb200_kv_write (RoPE, paged append) + Kascade paged decode",
           "distinct_layer_caches": dw.distinct_caches, "parallelism": f"batch shard x{world}, weights replicated, no collective"}
    del caches, model
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------------
def bench_kv_write(dev, peaks, seq_len=32768, H=32, G=8, D=128, page=16):
    """KV-cache write path (RoPE of Q and K, paged append of K and V) for one layer of a prefill at seq_len
    and for one decode append at batch 64; bytes = every operand read once and written once."""
    from kascade_b200 import _native as nat
    g = torch.Generator(device="cpu").manual_seed(7)
    q = torch.randn(1, seq_len, H, D, generator=g).half().to(dev)
    k = torch.randn(1, seq_len, G, D, generator=g).half().to(dev)
    v = torch.randn(1, seq_len, G, D, generator=g).half().to(dev)
    pps = seq_len // page
    kc = torch.empty(pps + 4, page, G, D, dtype=torch.float16, device=dev)
    vc = torch.empty_like(kc)
    bt = torch.randperm(pps + 4, generator=g)[:pps].view(1, pps).to(torch.int32).to(dev)
    qo = torch.empty_like(q)
    inv = (1.0 / (500000.0 ** (torch.arange(0, D, 2).float() / D))).to(dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    kv = nat.kv_layout_paged(kc, vc, bt)
    fn = lambda i: nat.kv_write(q, qo, k, v, zero, None, kv, inv_freq=inv)
    _time_cuda(fn, 3)
    ms = _time_cuda(fn, 20)
    byts = 2 * 2 * (q.numel() + k.numel() + v.numel())
    gbs = byts / (ms * 1e-3) / 1e9
    B2, ctx = 64, 32768
    q1 = torch.randn(B2, 1, H, D, generator=g).half().to(dev)
    k1 = torch.randn(B2, 1, G, D, generator=g).half().to(dev)
    v1 = torch.randn(B2, 1, G, D, generator=g).half().to(dev)
    q1o = torch.empty_like(q1)
    kc2 = torch.empty(B2 * 4, page, G, D, dtype=torch.float16, device=dev)     # only the page being appended to
    vc2 = torch.empty_like(kc2)
    bt2 = (torch.arange(B2, dtype=torch.int32) * 4).view(B2, 1).repeat(1, ctx // page + 1).to(dev)
    pos = torch.full((B2,), ctx, dtype=torch.int32, device=dev)
    kv2 = nat.kv_layout_paged(kc2, vc2, bt2)
    fn2 = lambda i: nat.kv_write(q1, q1o, k1, v1, pos, None, kv2, inv_freq=inv)
    _time_cuda(fn2, 3)
    us = _time_cuda(fn2, 50) * 1e3
    return {"kernel": "kv_write_kernel", "workload": f"one layer, {seq_len} tokens, RoPE + paged append ({page}-token pages)",
            "ms": ms, "bytes": byts, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": gbs / peaks["hbm_gbs"], "bound": "hbm", "peak_source": peaks["source"],
            "decode_append_us": us, "decode_append_workload": f"batch {B2}, one token each at context {ctx}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", type=int, default=32768, help="prefill length (default: the benchmark's 32768)")
    ap.add_argument("--config", type=int, default=2, choices=[2, 4, 5],
                    help="2 (default): the headline, prefill stack @32k + paged decode B=64; 4: the 131 072-token "
                         "prefill stack (36 layers, QK-norm, KV heads sharded over the GPUs); 5: attention of the "
                         "long-reasoning decode (256 sequences, contexts 4096..65536, batch-sharded)")
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-dense", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "push", "push_slices", "peer_store", "multicast", "nccl", "local"],
                    help="N > 1: how the per-head outputs reach the other GPUs: copy-engine pushes on side streams "
                         "(push), stores from the kernel epilogue to every peer (peer_store) or once to an NVLink multicast "
                         "address (multicast), NCCL all-gather (nccl); auto = peer_store on 2 GPUs, multicast from 4 on; local = measurement aid: like push with the copies left "
                         "out (every rank keeps only its own heads), which gives the step time without any output exchange")
    ap.add_argument("--no-peer-store", action="store_true", help="same as --exchange nccl")
    ap.add_argument("--wait-every-layer", action="store_true",
                    help="N > 1: synchronise the GPUs after every layer (what a consumer of each layer's gathered "
                         "outputs needs) instead of once per step")
    ap.add_argument("--skip-decoder", action="store_true", help="--config 5: attention only, without the decoder around it")
    ap.add_argument("--gen-tokens", type=int, default=128, help="--config 5: tokens generated per sequence")
    ap.add_argument("--decode-only", action="store_true", help="profiling aid: run only the decode configuration")
    ap.add_argument("--kv-write-only", action="store_true", help="profiling aid: run only the KV-cache write path")
    ap.add_argument("--decode-batch", type=int, default=None, help="profiling aid: decode batch (default 64)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist
    from kascade_b200 import EfficientKascadeStrategy, _native as nat
    from bench_workloads import DecodeWorkload, PrefillWorkload

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = _peaks()
    if args.kv_write_only:
        if rank == 0:
            print(json.dumps({"metric": "kv write only (profiling aid)", "kv_write": bench_kv_write(dev, peaks)}), flush=True)
        return
    if args.decode_only:
        decode = bench_decode(args, dev, world, peaks, args.decode_batch)
        if rank == 0:
            print(json.dumps({"metric": "decode only (profiling aid)", "decode": decode}), flush=True)
        return
    if args.config == 5:
        decode = bench_decode(args, dev, world, peaks, ragged=True, rank=rank)
        decoder = None if args.skip_decoder else bench_decoder_generate(args, dev, world, rank)
        if rank == 0:
            line = {"metric": "long-reasoning decode: tokens/s of a Llama-3.1-8B-architecture decoder and attention us/step, "
                              "256 sequences with contexts 4096..65536, 10% top-k",
                    "value": decode["us_per_step"], "unit": "us", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": decode["us_per_step"] / 1e3,
                    "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                    "data": "synthetic",
                    "config": {"workload": "llama31_8b_decode_attention_ragged_b256", "parallelism":
                               f"batch shard x{world}", "cache_policy": "caches larger than L2"},
                    "gpu_launches": decode["gpu_launches"], "device_status": nat.read_status(),
                    "decode": decode}
            if decoder:
                line["decoder"] = decoder
                line["tokens_per_s"] = decoder["tokens_per_s"]
                line["attention_us_per_step"] = decoder["attention_us_per_step"]
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- prefill stack (headline) -----------------------------------------------------
    if args.config == 4:
        from bench_workloads import QWEN3_ANCHORS
        wl = PrefillWorkload(seq_len=131072 if args.seq_len == 32768 else args.seq_len, layers=36,
                             anchors=QWEN3_ANCHORS, qk_norm=True)
        args.skip_decode = True
    else:
        wl = PrefillWorkload(seq_len=args.seq_len)
    assert wl.G % world == 0, "KV heads must divide over the ranks"
    gpr = wl.G // world
    my_heads = list(range(rank * gpr, (rank + 1) * gpr))
    exchange = "nccl" if args.no_peer_store else args.exchange
    if exchange == "auto":
        exchange = "peer_store" if world == 2 else "multicast"
    local_only = exchange == "local"
    if local_only:
        exchange = "push"
    sharded_check = sharded_self_check(rank, world, dev, exchange) if world > 1 else None
    if local_only:
        nat.peer_push = lambda *a, **k: None                       # the copies are left out on purpose (see --exchange)
    strat = EfficientKascadeStrategy(list(wl.anchors), "synthetic/llama31-8b-shape", k=wl.pct, tile_size=wl.tile,
                                     rolling_prefill=wl.rolling, head_mapping=wl.head_mapping(), register=False,
                                     shard=(rank, world) if world > 1 else None, exchange=exchange)
    inputs = [wl.layer_inputs(l, dev, my_heads if world > 1 else None) for l in range(wl.layers)]
    scaling = wl.D ** -0.5
    mods = [_Module(l) for l in range(wl.layers)]
    result = {}

    def step(_i=0):
        out = None
        for l in range(wl.layers):
            q, k, v = inputs[l]
            out, _ = strat.attention_forward(mods[l], q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, scaling)
            if world > 1 and args.wait_every_layer:
                strat.wait_gathers()
        if world > 1:
            strat.wait_gathers()
        result["out"] = out

    import datetime
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    n0 = nat.launch_count
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = datetime.datetime.now()
    s.record()
    for _ in range(args.steps):
        step()
    e.record()
    torch.cuda.synchronize()
    launches = (nat.launch_count - n0) // max(args.steps, 1)
    if world > 1:
        dist.barrier()
    ms = torch.tensor([s.elapsed_time(e) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item())
    # A timed region shorter than a few sampling periods holds no clock sample: the same steps go on, untimed,
    # until the load has lasted 0.6 s (every rank derives the same count from the all-reduced step time).
    repeat = 0
    if ms_step * args.steps < 600.0:
        repeat = min(500, int((600.0 - ms_step * args.steps) / max(ms_step, 1e-3)) + 1)
        for _ in range(repeat):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    clocks = sampler.stop(t_begin, datetime.datetime.now())
    clocks["window"] = "timed region" if repeat == 0 else f"timed region + {repeat} more of the same steps, untimed"
    status = nat.read_status()

    # ---------------- per-kernel timing and the roofline of the dominant kernel ------------------
    kernels = {}
    roof = None
    if world == 1:
        B, L, H, G, D = wl.B, wl.seq_len, wl.H, wl.G, wl.D
        T = -(-L // 32)
        out = torch.empty(B, L, H, D, dtype=torch.float16, device=dev)
        lse = torch.empty(B, L, H, dtype=torch.float32, device=dev)
        pooled = strat._buf["pooled"][: B * G * T * (-(-L // 128) * 128)].view(B, G, T, -1)
        nl = len(inputs)
        reps = 4
        kernels["prefill_dense_attn"] = (_time_cuda(lambda i: nat.prefill_dense(*inputs[i % nl], scaling, out, lse), reps),
                                         wl.flops_dense(), 1)
        kernels["prefill_dense_lse"] = (_time_cuda(lambda i: nat.prefill_dense(inputs[i % nl][0], inputs[i % nl][1], None,
                                                                               scaling, None, lse), reps),
                                        wl.flops_qk_causal(), 4)
        kernels["prefill_pool_scores"] = (_time_cuda(lambda i: nat.prefill_pool_scores(inputs[i % nl][0], inputs[i % nl][1],
                                                                                       lse, scaling, pooled), reps),
                                          wl.flops_qk_causal(), 5)
        nv, kr = strat._buf["n_valid"][: B * G * T].view(B, G, T), strat._buf["k_row"][: B * G * T].view(B, G, T)
        kk = strat._tile_idx.shape[-1]
        kernels["topk_select"] = (_time_cuda(lambda i: nat.topk_select(pooled, nv, kr, kk, strat._tile_idx,
                                                                       strat._tile_count, n_cols=L), reps), 0.0, 5)
        kernels["prefill_sparse"] = (_time_cuda(lambda i: nat.prefill_sparse(*inputs[i % nl], strat._tile_idx,
                                                                             strat._tile_count, None, scaling, out), reps),
                                     wl.flops_sparse(), 31)
        share = {k: v[0] * v[2] for k, v in kernels.items()}
        top = max(share, key=share.get)
        t_ms, flops, _n = kernels[top]
        achieved = flops / (t_ms * 1e-3) / 1e12
        # dram__bytes_read + dram__bytes_write per launch from the ncu capture at 16 384 tokens
        # (profiles/tile_prefill_kernels_16k_ncu.md), scaled linearly in L: every operand grows linearly
        ncu_mb_16k = {"prefill_dense_attn": 490.7, "prefill_dense_lse": 174.2, "prefill_pool_scores": 289.3,
                      "prefill_sparse": 315.8}
        traffic = ncu_mb_16k.get(top)
        traffic = None if traffic is None else traffic * 1e6 * (L / 16384)
        roof = {"kernel": "tile_prefill_kernel<%s>" % top, "bound": "tensor", "achieved": achieved,
                "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"], "traffic": traffic,
                "traffic_note": "bytes per launch, ncu capture at L=16384 scaled by L/16384",
                "peak_source": peaks["source"] + " (sustained bf16 GEMM)",
                "per_kernel_ms": {k: round(v[0], 4) for k, v in kernels.items()},
                "per_kernel_tflops": {k: round(v[1] / (v[0] * 1e-3) / 1e12, 1) for k, v in kernels.items() if v[1]},
                "launches_per_step": {k: v[2] for k, v in kernels.items()}}

    # ---------------- end to end through the plugin call with host buffers ------------------------
    e2e = None
    if not args.skip_e2e:
        n_host = min(4, wl.layers)
        host = [tuple(x.cpu().pin_memory() for x in inputs[l]) for l in range(n_host)]
        host_out = torch.empty(inputs[0][0].shape, dtype=torch.float16).pin_memory()
        dbuf = [tuple(torch.empty_like(x) for x in inputs[0]) for _ in range(2)]   # double-buffered device inputs
        h2d = sum(x.numel() * 2 for x in inputs[0]) * wl.layers
        d2h = host_out.numel() * 2 * wl.layers
        in_s, out_s = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(_i=0):
            # three streams: H2D of layer l+1 and D2H of layer l-1 overlap the kernels of layer l; every copy and
            # every kernel of the step lies between the two timing events on the current stream
            cur = torch.cuda.current_stream()
            in_s.wait_stream(cur)
            out_s.wait_stream(cur)
            for l in range(wl.layers):
                slot = l & 1
                dq, dk, dv = dbuf[slot]
                hq, hk, hv = host[l % n_host]
                with torch.cuda.stream(in_s):
                    if l >= 2:
                        in_s.wait_event(ev_free[slot])            # layer l-2 has finished reading this slot
                    dq.copy_(hq, non_blocking=True)
                    dk.copy_(hk, non_blocking=True)
                    dv.copy_(hv, non_blocking=True)
                    ev_in[slot].record(in_s)
                cur.wait_event(ev_in[slot])
                o, _ = strat.attention_forward(mods[l], dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2), None, scaling)
                ev_free[slot].record(cur)
                out_s.wait_event(ev_free[slot])
                with torch.cuda.stream(out_s):
                    host_out.copy_(o, non_blocking=True)
                o.record_stream(out_s)
            cur.wait_stream(in_s)
            cur.wait_stream(out_s)

        e2e_step()
        if world > 1:
            dist.barrier()
        t = torch.tensor([_time_cuda(e2e_step, max(1, min(args.steps, 2)))], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": float(t.item()), "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "note": f"{n_host} distinct pinned host layers cycled over {wl.layers} layers; H2D, kernels and D2H of "
                       "consecutive layers overlap on three streams (double-buffered device inputs)"}
        dq = dk = dv = None
        del host, host_out, dbuf, dq, dk, dv

    # ---------------- dense attention on the same GPU ----------------------------------------------
    dense = None
    if world == 1 and not args.skip_dense:
        out = torch.empty(wl.B, wl.seq_len, wl.H, wl.D, dtype=torch.float16, device=dev)
        t_own = _time_cuda(lambda i: nat.prefill_dense(*inputs[i % len(inputs)], scaling, out, None), 3)
        dense = {"own_kernel_ms_per_layer": t_own, "own_kernel_ms_stack": t_own * wl.layers,
                 "own_tflops": wl.flops_dense() / (t_own * 1e-3) / 1e12}
        try:
            import torch.nn.functional as F

            def sdpa(i):
                q, k, v = inputs[i % len(inputs)]
                F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=True)
            sdpa(0)
            t_lib = _time_cuda(sdpa, 3)
            dense.update({"torch_sdpa_ms_per_layer": t_lib, "torch_sdpa_ms_stack": t_lib * wl.layers})
        except Exception as ex:                                      # library comparator only
            dense["torch_sdpa_error"] = str(ex)[:120]
        dense["speedup_vs_own_dense"] = dense["own_kernel_ms_stack"] / ms_step
        # the headline "vs dense" figure is taken against the FASTER dense attention on this GPU
        fastest = min(dense["own_kernel_ms_stack"], dense.get("torch_sdpa_ms_stack", float("inf")))
        dense["speedup_vs_dense"] = fastest / ms_step
        dense["speedup_vs_dense_against"] = ("torch SDPA (library)" if fastest != dense["own_kernel_ms_stack"]
                                             else "this library's dense kernel")
    del inputs
    strat._buf.clear()
    torch.cuda.empty_cache()

    decode = None if args.skip_decode else bench_decode(args, dev, world, peaks)
    kvw = bench_kv_write(dev, peaks) if (world == 1 and rank == 0 and not args.skip_decode) else None
    status |= nat.read_status()

    # ---------------- CPU baseline (rank 0, N = 1) --------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        L = 4096
        n_anchor = len([a for a in wl.anchors if a != 0])
        n_reuse = wl.layers - n_anchor - 1
        stack_ms, times, kind = cpu_prefill_sample(L, wl.seq_len, n_anchor, n_reuse)
        what = ("the reference's own KascadeStrategy (unmodified, oracle/_ref)" if kind == "reference"
                else "oracle port (oracle/_ref not staged)")
        cpu = {"value": stack_ms, "unit": "ms", "cores": torch.get_num_threads(), "kind": kind,
               "sample": (f"{what}, fp32, block_size 512: layer 0 {times[0]:.1f}s, reuse {times[1]:.1f}s, anchor>0 "
                          f"{times[2]:.1f}s measured at L={L}; {wl.layers}-layer stack at {wl.seq_len} extrapolated by "
                          f"({wl.seq_len}/{L})^2 with 1/{n_reuse}/{n_anchor} layer weights")}

    if rank == 0:
        line = {"metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": prefill_config(wl, world),
                "exchange": (None if world == 1 else "NONE (measurement aid): outputs stay on their rank" if local_only
                             else strat.exchange_description()),
                "gpu_sync": (None if world == 1 else "after every layer" if args.wait_every_layer else
                             "once per step (the layers' outputs are not consumed in between)"),
                "sharded_check": sharded_check,
                "algorithmic_tflop_per_step": wl.flops_stack() / 1e12,
                "achieved_tflops": wl.flops_stack() / (ms_step * 1e-3) / 1e12,
                "gpu_launches": launches, "device_status": status, "clocks": clocks}
        if roof:
            line["roofline"] = roof
        if cpu:
            line["cpu_baseline"] = cpu
        if e2e:
            line["e2e"] = e2e
        if dense:
            line["dense"] = dense
        if decode:
            line["decode"] = decode
        if kvw:
            line["kv_write"] = kvw
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
