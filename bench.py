"""Benchmark of the LSA selection-plus-attention path: prefill tokens/s of one flat D-LSA layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload` = "C2"): one causal global-attention layer, B=1, 131,072 tokens, 40 query heads over
8 KV heads of 128 dims, bf16; linear key and query maps [1024, 64]; keys pooled by 16 and Ward-merged into 32
buckets per 1,024-key cluster block (4,096 buckets, cap 64); every query reads its top 64 buckets (at most 4,096
keys), 4 sinks and a 1,024-key window; queries are taken in chunks of 8,192 rows. Inputs are seeded synthetic
tensors with a 256-centre mixture structure. A step is one whole prefill: index map of keys and queries, pooling,
Ward, bucket table, and per chunk the bucket scan with its top-p, the expansion and the gather-sparse attention.

`value` times the step with q, k, v resident in HBM; `e2e` times the same call from pinned host buffers with the
host-to-device copies of q, k, v and the device-to-host copy of the output inside the timed region.
`--impl reference` times the CPU oracle (the port of the reference's PyTorch specification) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _path in (ROOT, os.path.join(ROOT, "latent-sparse-attention_b200")):
    if _path not in sys.path:
        sys.path.insert(0, _path)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "LSA layer prefill tokens/s (D-LSA flat, 128k ctx, one layer)"
UNIT = "tokens/s"

C2 = dict(workload="C2", tokens=131072, heads=40, kv_heads=8, head_dim=128, index_dim=64, pool_size=16,
          bucket_size=32, bucket_cap=64, cluster_block_size=1024, top_p=64, top_k=4096, sink_size=4,
          window_size=1024, chunk=8192, centres=256, seed=0)

# DRAM bytes per algorithmic byte of a sparse_attend launch, from a one-pass ncu capture of the 16 launches of a
# full-size step (dram__bytes_read.sum + dram__bytes_write.sum: 0.3 GB for the first chunk up to 55.9 GB for the
# last, 37.2 GB on average, against 66.4 GB of algorithmic bytes; summarised in profiles/). The traffic reported is
# this ratio times the launch's algorithmic bytes.
ATTEND_DRAM_BYTES_PER_ALGORITHMIC_BYTE = 0.561
# DRAM bytes of one bucket-major attend call (the six kernels of a chunk): dram__bytes_read.sum +
# dram__bytes_write.sum over the 96 launches of a full-size step in a one-pass ncu capture, 189.7 GB, a sixteenth of
# it a call (the attend pass writes 5.4 GB of partials, the merge reads them back; summarised in profiles/).
BUCKET_DRAM_TRAFFIC_PER_CALL = 11.85e9


def small(cfg: dict, tokens: int) -> dict:
    out = dict(cfg)
    out["tokens"] = tokens
    return out


def make_inputs(cfg: dict, pin: bool):
    """Seeded q [T,Hq,dh], k, v [T,Hkv,dh] bf16 on the host, and the two maps [Hkv*dh, index_dim] bf16."""
    gen = torch.Generator().manual_seed(cfg["seed"])
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    mu = torch.randn(cfg["centres"], Hkv, dh, generator=gen)
    label = torch.randint(0, cfg["centres"], (T,), generator=gen)
    half = 0.5 ** 0.5
    k = half * mu[label] + half * torch.randn(T, Hkv, dh, generator=gen)
    q = torch.empty(T, Hq, dh, dtype=torch.bfloat16)
    group = Hq // Hkv
    grouped = q.view(T, Hkv, group, dh)  # head h reads KV head h // group
    for g in range(group):  # one query head of every group at a time keeps the fp32 scratch small
        grouped[:, :, g] = (half * k + half * torch.randn(T, Hkv, dh, generator=gen)).bfloat16()
    v = torch.randn(T, Hkv, dh, generator=gen).bfloat16()
    k = k.bfloat16()
    d_in = Hkv * dh
    wq = (torch.randn(d_in, cfg["index_dim"], generator=gen) / d_in ** 0.5).bfloat16()
    wk = (torch.randn(d_in, cfg["index_dim"], generator=gen) / d_in ** 0.5).bfloat16()
    if pin:
        q, k, v = q.pin_memory(), k.pin_memory(), v.pin_memory()
    return q, k, v, wq, wk


def design_of(cfg: dict):
    from lsa_b200.layer import FlatDesign

    return FlatDesign(pool_size=cfg["pool_size"], bucket_size=cfg["bucket_size"], bucket_cap=cfg["bucket_cap"],
                      cluster_block_size=cfg["cluster_block_size"], top_p=cfg["top_p"], top_k=cfg["top_k"],
                      sink_size=cfg["sink_size"], window_size=cfg["window_size"])


# ------------------------------------------------------------------------------------------------ clocks


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs (read-only)."""

    def __init__(self, index: int, period: float = 0.2):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        n = self._nvml
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
                try:
                    bits = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for bit, name in names.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------ CPU baseline


def cpu_prefill_rate(cfg: dict, host, buckets_np, index_q_np, threads: int) -> dict:
    """Tokens/s of the CPU oracle on a bounded sample of the workload, stage by stage.

    Map: 8 cluster blocks of tokens of q and k. Pool + Ward + table: those 8 blocks. Search + expansion and attention: 128 rows
    spread evenly over the context, against the whole index and cache. Each stage's time per token is summed.
    """
    import oracle

    q, k, v, wq, wk = host
    os.environ["OMP_NUM_THREADS"] = str(threads)
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    n_map = min(T, 8 * cfg["cluster_block_size"])
    qs, ks = q[:n_map].float().numpy(), k[:n_map].float().numpy()
    t0 = time.perf_counter()
    oracle.project(oracle.regroup_queries(qs, Hkv), wq.float().numpy())
    index_k_sample = oracle.project(ks.reshape(n_map, -1), wk.float().numpy())
    t_map = (time.perf_counter() - t0) / n_map
    blocks = n_map // cfg["cluster_block_size"]
    n_build = blocks * cfg["cluster_block_size"]
    t0 = time.perf_counter()
    oracle.build_buckets(index_k_sample[:n_build], cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"],
                         cfg["cluster_block_size"])
    t_build = (time.perf_counter() - t0) / n_build
    rows = np.linspace(0, T - 1, 128).astype(np.int64)
    t0 = time.perf_counter()
    lists, lengths = oracle.read(index_q_np[rows], rows, buckets_np, cfg["top_p"], cfg["top_k"], cfg["sink_size"],
                                 cfg["window_size"])
    t_read = (time.perf_counter() - t0) / len(rows)
    kf, vf = k.float().numpy(), v.float().numpy()
    qrows = q[torch.from_numpy(rows)].float().numpy()
    t0 = time.perf_counter()
    oracle.sparse_attend(qrows, kf, vf, lists, rows, 0, 0, dh ** -0.5, lengths=lengths)
    t_attend = (time.perf_counter() - t0) / len(rows)
    per_token = t_map + t_build + t_read + t_attend
    return {"value": 1.0 / per_token, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"map {n_map} tokens, build {blocks} blocks, search+expand and attend 128 rows spread over "
                       f"{T} positions; per-token stage times summed "
                       f"(map {t_map * 1e6:.1f} build {t_build * 1e6:.1f} read {t_read * 1e6:.1f} "
                       f"attend {t_attend * 1e6:.1f} us)")}


def host_threads() -> int:
    return len(os.sched_getaffinity(0))


# ------------------------------------------------------------------------------------------------ runs


def attend_algorithmic_bytes(cfg: dict, gathered_total: int) -> float:
    """Algorithmic bytes of a step's gather attention: the K/V rows each query gathers (its selected keys; the
    window and the sinks are the band kernel's), Q in, the band's partial result in (fp32 output and log-sum-exp),
    and O out."""
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    row = Hkv * dh * 2 * 2
    return gathered_total * row + T * Hq * dh * (2 + 4 + 2) + T * Hq * 4


def bucket_attend_algorithmic_bytes(cfg: dict, pairs: int) -> float:
    """Algorithmic bytes of a step's bucket-major attention (starts, invert, attend, merge): per (row, pick) pair and
    query head one query vector in, one bf16 partial output and one log-sum-exp out of the attend pass and back
    into the merge; per row the band's fp32 partial in and the bf16 output out. A bucket's K/V rows are read once
    per 128 pairs and do not show at this scale."""
    T, Hq, dh = cfg["tokens"], cfg["heads"], cfg["head_dim"]
    return pairs * Hq * (3 * dh * 2 + 2 * 4) + T * Hq * ((dh + 1) * 4 + dh * 2)


def band_algorithmic_bytes(cfg: dict) -> float:
    """Algorithmic bytes of a step's band attention: the band's K/V once per 128-query tile, the sinks, Q in and
    the fp32 partial result out."""
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    row = Hkv * dh * 2 * 2
    tiles = (T + 127) // 128
    return tiles * (cfg["window_size"] + 128 + cfg["sink_size"]) * row + T * Hq * dh * (2 + 4) + T * Hq * 4


def run_ours(args, cfg: dict) -> dict:
    import torch.distributed as dist

    from lsa_b200 import _lib, probe
    from lsa_b200.layer import FlatLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun), found WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    host = make_inputs(cfg, pin=True)
    q_h, k_h, v_h, wq, wk = host
    base = FlatLayer(design_of(cfg), wq.cuda(), wk.cuda(), cfg["heads"], cfg["kv_heads"], cfg["head_dim"])
    base.bucket_tensor_memory = args.bucket_kernel == "tensor-memory"
    layer = base
    if world > 1:
        from lsa_b200.parallel import ShardedFlatLayer, deal

        # a rank holds only its own share of the KV rows, on the host and on the device; the queries are split by
        # rows (every rank reads the gathered cache for its own rows) or replicated (context parallel: every rank
        # reads the keys it stores for all rows and the partial outputs are merged)
        layer = ShardedFlatLayer(base, rank, world)
        k_h, v_h = deal(k_h, rank, world).clone().pin_memory(), deal(v_h, rank, world).clone().pin_memory()
        if args.parallel == "rows":
            q_h = layer.rows_of(q_h, cfg["chunk"] * world).clone().pin_memory()
    q, k, v = q_h.cuda(), k_h.cuda(), v_h.cuda()
    out_d = torch.empty(cfg["tokens"] // world, cfg["heads"], cfg["head_dim"], dtype=torch.bfloat16, device="cuda")
    out_h = torch.empty(out_d.shape, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    q_in, k_in, v_in = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    by_rows = world > 1 and args.parallel == "rows"

    def prefill(q_, k_, v_):
        if by_rows:
            # the ranks take a chunk of 8,192 rows each, side by side
            return layer.prefill_by_rows(q_, k_, v_, cfg["tokens"], chunk=cfg["chunk"] * world, out=out_d)
        return layer.prefill(q_, k_, v_, chunk=cfg["chunk"], out=out_d)

    def resident_step():
        prefill(q, k, v)

    def e2e_step():
        if world == 1:
            # the layer's own call for host-resident inputs: copies in and out overlapped with the chunks' work
            base.prefill_from_host(q_h, k_h, v_h, out_h, chunk=cfg["chunk"])
            return
        q_in.copy_(q_h, non_blocking=True)
        k_in.copy_(k_h, non_blocking=True)
        v_in.copy_(v_h, non_blocking=True)
        out_h.copy_(prefill(q_in, k_in, v_in), non_blocking=True)

    for _ in range(args.warmup):
        resident_step()
    gathered, index, index_q = None, None, None
    if world == 1:
        # One more untimed pass counts the gathered keys the roofline figure needs, and keeps what the CPU baseline
        # reads.
        _, index = base.prefill(q, k, v, chunk=cfg["chunk"], return_index=True)
        gathered = pairs = 0
        index_q = base.index_queries(q)
        for start in range(0, cfg["tokens"], cfg["chunk"]):
            pos = torch.arange(start, min(cfg["tokens"], start + cfg["chunk"]), device="cuda")
            pairs += int((base.pick(index_q[start:start + cfg["chunk"]], pos, index)[0] >= 0).sum())
            _, lengths = base.select(index_q[start:start + cfg["chunk"]], pos, index)
            window_start = (pos + 1 - cfg["window_size"]).clamp_min(0)
            fixed = (pos + 1 - window_start) + torch.minimum(window_start, torch.full_like(pos, cfg["sink_size"]))
            gathered += int((lengths.to(torch.int64) - fixed).sum())

    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    launches_before = _lib.LAUNCHES
    with ClockSampler(local) as clocks:
        ms = timed(resident_step, args.steps)
    launches = (_lib.LAUNCHES - launches_before) // args.steps
    stage_ms = recorder.totals_ms()
    probe.uninstall()
    for _ in range(min(args.warmup, 3)):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps)

    tokens = cfg["tokens"]
    attend_ms, attend_launches = stage_ms.get("attend", (0.0, 0))
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_kind = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_kind = 6650.0, "fallback"
    per_launch_bytes = achieved = useful_tflops = None
    bucket_major = world == 1 or by_rows  # these prefills read the selected keys bucket by bucket
    if gathered is not None and attend_launches:
        stage_bytes = bucket_attend_algorithmic_bytes(cfg, pairs) if bucket_major else \
            attend_algorithmic_bytes(cfg, gathered)
        per_launch_bytes = stage_bytes / max(1, attend_launches // args.steps)
        achieved = per_launch_bytes / (attend_ms / attend_launches * 1e-3) / 1e9
        useful_tflops = 4.0 * gathered * cfg["heads"] * cfg["head_dim"] / (attend_ms / args.steps * 1e-3) / 1e12
    result = {
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["workload"], "tokens": tokens, "heads": cfg["heads"], "kv_heads": cfg["kv_heads"],
                   "head_dim": cfg["head_dim"], "index_dim": cfg["index_dim"], "buckets": tokens // cfg["bucket_size"],
                   "top_p": cfg["top_p"], "top_k": cfg["top_k"], "window": cfg["window_size"],
                   "sink": cfg["sink_size"], "chunk": cfg["chunk"], "bucket_kernel": args.bucket_kernel,
                   "l2": "inputs (1.9 GB of q, k, v per step) exceed the 126 MB L2",
                   "parallelism": "1 GPU" if world == 1 else (
                       f"KV rows and cluster blocks dealt round-robin over {world} GPUs; " + (
                           "the cache all-gathered once a step, query rows split over the ranks" if by_rows else
                           "every rank reads the keys it stores, partial outputs merged (context parallel)"))},
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": (q_h.numel() * world + (k_h.numel() + v_h.numel()) * world) * 2,
                "d2h_bytes_per_step": out_h.numel() * world * 2, "ms_per_step": e2e_ms},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "roofline": {"kernel": "bucket-major attend (bucket_starts, scan, scatter, segments, bucket_attend, "
                               "bucket_merge: one call a chunk)" if bucket_major else "sparse_attend_kernel",
                     "bound": "hbm", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                     "traffic": (BUCKET_DRAM_TRAFFIC_PER_CALL if bucket_major else
                                 ATTEND_DRAM_BYTES_PER_ALGORITHMIC_BYTE * per_launch_bytes) if per_launch_bytes else None,
                     "algorithmic_bytes_per_launch": per_launch_bytes,
                     "useful_tflops": useful_tflops,
                     "launches_per_step": attend_launches // args.steps,
                     "ms_per_launch": attend_ms / max(1, attend_launches)},
        "stages_ms_per_step": {name: total / args.steps for name, (total, _) in sorted(stage_ms.items())},
    }
    if rank == 0 and world == 1:
        from lsa_b200.core import Buckets  # noqa: F401
        import oracle

        b = index.buckets
        buckets_np = oracle.Buckets(b.bucket_centroids.cpu().numpy(), b.bucket_members.cpu().numpy(),
                                    b.bucket_sizes.cpu().numpy(), b.block_bucket_count, b.cluster_block_size)
        result["cpu_baseline"] = cpu_prefill_rate(cfg, host, buckets_np, index_q.cpu().numpy(), host_threads())
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else None


def run_reference(args, cfg: dict) -> dict | None:
    """The CPU arm: the oracle port of the reference's PyTorch path, timed on the host cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return None
    import oracle

    oracle.build()
    threads = host_threads()
    host = make_inputs(small(cfg, cfg["tokens"]), pin=False)
    q, k, v, wq, wk = host
    # The sample's search and attention need the whole index: build it once, untimed, with the same oracle.
    index_k = oracle.project(k.float().numpy().reshape(cfg["tokens"], -1), wk.float().numpy())
    buckets = oracle.build_buckets(index_k, cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"],
                                   cfg["cluster_block_size"])
    rows = np.linspace(0, cfg["tokens"] - 1, 128).astype(np.int64)
    index_q = np.zeros((cfg["tokens"], cfg["index_dim"]), dtype=np.float32)
    index_q[rows] = oracle.project(oracle.regroup_queries(q[torch.from_numpy(rows)].float().numpy(), cfg["kv_heads"]),
                                   wq.float().numpy())
    rates = []
    for step in range(args.warmup + args.steps):
        rate = cpu_prefill_rate(cfg, host, buckets, index_q, threads)
        if step >= args.warmup:
            rates.append(rate)
    value = statistics.median(r["value"] for r in rates)
    base = dict(rates[-1], value=value)
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cfg["tokens"] / value * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg["workload"], "tokens": cfg["tokens"]},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--tokens", type=int, default=None, help="a smaller context of the same workload (profiling)")
    parser.add_argument("--bucket-kernel", default="tensor-memory", choices=["warp", "tensor-memory"],
                        help="the form of the bucket-major attend pass: warp-level MMA tiles or tcgen05 tiles in tensor memory")
    parser.add_argument("--parallel", default="rows", choices=["rows", "context"],
                        help="at N > 1: split the query rows over the ranks (the cache is all-gathered once a step), "
                             "or keep every rank on the keys it stores and merge partial outputs")
    args = parser.parse_args()
    cfg = dict(C2)
    if args.tokens:
        cfg = small(cfg, args.tokens)
        cfg["workload"] = f"C2 cut to {args.tokens} tokens"
    result = run_reference(args, cfg) if args.impl == "reference" else run_ours(args, cfg)
    if result is not None:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
