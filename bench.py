"""Benchmark of the LSA selection-plus-attention path: one global-attention layer at 1M-10M tokens of context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C4|C2|C3|C5]
                    [--also C2,C3,C5|none] [--tokens T]

The headline workload (`config.workload` = "C4") is the flat design over an MLA-style layer: 64 query heads over a
shared latent cache of 10,485,760 tokens (512 value dims + 64 rope dims a token, bf16), two-layer key and query maps
576 -> 2048 -> 64, keys pooled by 64 and Ward-merged into 8 buckets per 5,120-key cluster block (16,384 buckets, cap
1,280), every query reading its top 128 buckets, 4 sinks and a 5,120-key window. A STEP is one prefill chunk of 8,192
queries at the END of the context, as the reference times its layers (the last chunk before each context length,
src/lsa/evaluation/performance/kernels/measure/layer.py:393): the index keys of the chunk's own tokens, the pools,
Ward and bucket table of the cluster blocks they close, the query map, the bucket scan with its top-p, the expansion
and the gather attention of all 8,192 rows. `value` is chunk tokens / step time with the cache and the chunk resident
in HBM; `e2e` times the same step with the chunk's queries and latent rows copied from pinned host memory and the
output copied back inside the timed region. `decode` is one query row at the last position (CUDA-graph replay).

Before anything is timed, sample rows of the very path that is timed are compared with the CPU oracle (read lists
equal, attention within max-abs 2e-2 and mean-abs 2e-3); a miss ends the run with a non-zero exit code.

The other configurations ride along as `also`: C2 (flat prefill of 128k tokens, GQA), C3 (tree decode over 1M
tokens), C5 (batched paged decode of 64 requests). Inputs are seeded synthetic tensors (`lsa_b200.workloads`).
`--impl reference` times the CPU oracle - a C port of the reference's PyTorch specification - on the host cores.
"""

from __future__ import annotations

import argparse
import json
import math
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

METRIC = "LSA layer prefill tokens/s (one layer, last 8,192-query chunk of a 10M-token context) and decode us/step"
UNIT = "tokens/s"
TOLERANCE = {"attention_max_abs": 2e-2, "attention_mean_abs": 2e-3}

# DRAM bytes per algorithmic byte of the dominant kernel of a workload, from the ncu capture summarised in the named
# file under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum over the launch's algorithmic bytes, on a cut of
# the workload small enough to capture; traffic grows in proportion to the rows a launch reads).
TRAFFIC = {
    "C4": {"ratio": 0.718, "profile": "profiles/latent_attend_tc_kernel_c4_cut.md"},
    "C2": {"ratio": None, "profile": "profiles/bucket_attend_tc_kernel_c2_49152tok.md"},
}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        found = json.load(open(path))
        return {"hbm_gbs": found["hbm_gbs"], "tensor_tflops": found["bf16_tflops_sustained"],
                "tensor_tflops_burst": found["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "tensor_tflops_burst": 1590.0, "kind": "fallback"}


def roof_ms(nbytes: float, flops: float, pk: dict) -> tuple:
    """The roofline time of a stage and what bounds it: max(bytes / HBM, flops / sustained dense bf16)."""
    t_hbm = nbytes / (pk["hbm_gbs"] * 1e9) * 1e3
    t_tensor = flops / (pk["tensor_tflops"] * 1e12) * 1e3
    return (t_hbm, "hbm") if t_hbm >= t_tensor else (t_tensor, "tensor")


def stage_table(work: dict, measured: dict, pk: dict, ms_per_step: float, gpus: int = 1) -> dict:
    """Per stage: algorithmic bytes and flops of the whole job, the roofline time they imply on `gpus` GPUs that share
    them evenly, the measured time and their ratio; and the stage-wise fraction = sum of the roofline times / the step
    time."""
    stages, total = {}, 0.0
    for name, (nbytes, flops) in work.items():
        roof, bound = roof_ms(nbytes / gpus, flops / gpus, pk)
        total += roof
        got = measured.get(name)
        stages[name] = {"bytes": nbytes, "flops": flops, "roof_ms": roof, "bound": bound, "ms": got,
                        "frac": roof / got if got else None}
    return {"stages": stages, "gpus": gpus, "roof_ms": total, "frac": total / ms_per_step if ms_per_step else None}


def host_threads() -> int:
    return len(os.sched_getaffinity(0))


# ------------------------------------------------------------------------------------------------ clocks


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs (read-only)."""

    def __init__(self, index: int, period: float = 0.2):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

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


# ------------------------------------------------------------------------------------------------ timing


class Env:
    """The ranks of this launch: one process a GPU under torchrun, or a single process."""

    def __init__(self, gpus: int):
        import torch.distributed as dist

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != gpus:
            raise SystemExit(f"--gpus {gpus} needs {gpus} ranks (torchrun), found WORLD_SIZE={self.world}")
        torch.cuda.set_device(self.local)
        self.dist = dist
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps: int) -> float:
        """Milliseconds a call: `steps` calls between two barriers, CUDA events on the launching stream, the
        maximum over ranks."""
        self.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        self.barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device="cuda")
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms) / steps

    def total(self, value: float) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t)
        return float(t)

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_graph(env: Env, step, warmup: int, steps: int) -> tuple:
    """Microseconds a step, the step captured in a CUDA graph and replayed; eager launches if capture is refused, and
    on several GPUs (the step then holds collectives). Returns (us, "graph" or "eager")."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    run, how = step, "eager"
    if env.world > 1:
        return env.timed(run, steps) * 1e3, how
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run, how = graph.replay, "graph"
    except Exception as failure:  # capture is an optimisation of the measurement, not of the result
        print(f"graph capture refused ({type(failure).__name__}); timing eager launches", file=sys.stderr)
        torch.cuda.synchronize()
    for _ in range(warmup):
        run()
    return env.timed(run, steps) * 1e3, how


def buckets_to_host(buckets):
    import oracle

    return oracle.Buckets(buckets.bucket_centroids.cpu().numpy(), buckets.bucket_members.cpu().numpy(),
                          buckets.bucket_sizes.cpu().numpy(), buckets.block_bucket_count, buckets.cluster_block_size)


def fail(message: str) -> None:
    print(f"bench: PARITY FAILURE - {message}", file=sys.stderr)
    raise SystemExit(3)


# ------------------------------------------------------------------------------------------------ C4: MLA, flat, 10M


def c4_config(cfg: dict, world: int) -> dict:
    """What both arms of the benchmark print as `config`: the workload, not what a run found in it."""
    T = cfg["tokens"]
    blocks = T // cfg["cluster_block_size"]
    return {"workload": cfg["workload"] if T == 10485760 else f"C4 cut to {T} tokens", "tokens": T,
            "chunk": min(cfg["chunk"], T // 2), "heads": cfg["heads"], "latent_dim": cfg["latent_dim"],
            "value_dim": cfg["value_dim"], "index_dim": cfg["index_dim"],
            "maps": f"two-layer {cfg['latent_dim']} -> {cfg['hidden_dim']} -> {cfg['index_dim']}",
            "buckets": blocks * (cfg["cluster_block_size"] // cfg["bucket_size"]), "top_p": cfg["top_p"],
            "top_k": cfg["top_k"], "window": cfg["window_size"], "sink": cfg["sink_size"],
            "l2": "a step gathers hundreds of GB of latent rows out of a 12 GB cache: far beyond the 126 MB L2, no "
                  "flush between steps",
            "parallelism": "1 GPU" if world == 1 else (
                f"context parallel: latent rows dealt in granules of 64 and cluster blocks round-robin over {world} "
                f"GPUs; candidates all-gathered and cut, partial outputs exchanged by all-to-all and merged by "
                f"log-sum-exp")}


def c4_expected(cfg, rows, index_q_np, positions_np, buckets_np, latent_of, q, decode: bool = False):
    """The oracle's read of sample rows: lists, lengths, and for `attend_rows` of them the attention output."""
    import oracle

    t0 = time.perf_counter()
    lists, lens = oracle.read(index_q_np, positions_np, buckets_np, cfg["top_p"], cfg["top_k"], cfg["sink_size"],
                              cfg["window_size"])
    t_read = time.perf_counter() - t0
    outs, t_attend = {}, 0.0
    for i in rows:
        ids = np.sort(lists[i, : lens[i]])
        gathered = latent_of(ids)
        t0 = time.perf_counter()
        ref, _ = oracle.sparse_attend(q[i:i + 1].float().cpu().numpy(), gathered[:, None, :], gathered[:, None, :],
                                      np.arange(len(ids), dtype=np.int32)[None], np.array([len(ids)]), 0, 0,
                                      _latent_scale(cfg))
        t_attend += time.perf_counter() - t0
        outs[i] = ref[0, :, : cfg["value_dim"]]
    return lists, lens, outs, t_read, t_attend


def _latent_scale(cfg):
    from lsa_b200 import workloads as W

    return W.latent_scale(cfg)


def run_c4(args, env: Env, cfg: dict) -> dict:
    import oracle
    from lsa_b200 import _lib, ops, probe
    from lsa_b200 import workloads as W
    from lsa_b200.core import Buckets
    from lsa_b200.latent import LatentLayer
    from lsa_b200.parallel import ShardedLatentLayer, gather_pieces

    world, rank = env.world, env.rank
    pk = peaks()
    T, chunk, Hq, dk, dv, d_idx = (cfg[k] for k in ("tokens", "chunk", "heads", "latent_dim", "value_dim",
                                                     "index_dim"))
    chunk = min(chunk, T // 2)
    first = T - chunk
    gen = torch.Generator(device="cuda").manual_seed(cfg["seed"])
    share, tail = W.latent_cache(cfg, gen, world=world, rank=rank, keep_tail=chunk)
    qmap, kmap = W.latent_maps(cfg, gen)
    q = W.latent_queries(cfg, tail, gen)
    layer = LatentLayer(W.design_of(cfg), qmap, kmap, Hq, dk, dv, scale=W.latent_scale(cfg))
    q1, pos1 = q[-1:].contiguous(), torch.tensor([T - 1], device="cuda")
    own_rows = chunk // world
    out_d = torch.empty(own_rows, Hq, dv, dtype=torch.bfloat16, device="cuda")
    start_ev, stop_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start_ev.record()
    if world == 1:
        index = layer.build_index(share)
        sharded = None
    else:
        sharded = ShardedLatentLayer(layer, rank, world)
        sharded.build_index(share, T)
        index = None
    stop_ev.record()
    torch.cuda.synchronize()
    build_ms = start_ev.elapsed_time(stop_ev)

    def step():
        if world == 1:
            layer.extend_index(share, first, chunk)
            layer.prefill_rows(q, first, share, index, out_d)
        else:
            sharded.extend_index(share, first, chunk)
            sharded.prefill_rows(q, first, share, out_d)

    def decode():
        if world == 1:
            return layer.decode(q1, pos1, share, index, splits=args.decode_splits)
        return sharded.decode(q1, pos1, share, splits=max(16, args.decode_splits // world))

    # ---- parity of the timed path, before anything is timed
    step()
    out1 = decode()
    torch.cuda.synchronize()
    layer.check()
    positions = torch.arange(first, T, device="cuda")
    if world == 1:
        buckets = index.buckets
        full = share
        lists_d, lens_d = layer.select(layer.index_queries(q), positions, index)
        gathered_total = float(lens_d.sum())
    else:
        per_block, blocks = layer.design.block_bucket_count, T // layer.design.cluster_block_size
        centroids = gather_pieces(sharded.centroids).view(world, blocks // world, per_block, d_idx).transpose(
            0, 1).reshape(blocks * per_block, d_idx)
        members = sharded.members
        buckets = Buckets(centroids, members, (members >= 0).sum(1, dtype=torch.int32), per_block,
                          layer.design.cluster_block_size)
        lists_d, lens_d = sharded.select(q, positions)
        gathered_total = env.total(float(lens_d.sum()))
        full = None
        if rank == 0:  # the checker's copy of the whole cache: the same generator walked again
            full, _ = W.latent_cache(cfg, torch.Generator(device="cuda").manual_seed(cfg["seed"]))
    # rows of rank 0's share of the chunk (their outputs are checked), and the chunk's last row (the decode row)
    sample = sorted({0, own_rows - 1} | set(np.random.default_rng(0).choice(own_rows, 4, replace=False).tolist()))
    owned = list(range(len(sample)))
    if sample[-1] != chunk - 1:
        sample.append(chunk - 1)
    parity, cpu = None, None
    if world > 1:  # every rank's share of the sample rows' lists, as positions
        local = lists_d[sample].to(torch.int64)
        as_positions = torch.full((len(sample), layer.design.list_width), -1, dtype=torch.int32, device="cuda")
        as_positions[:, : local.shape[1]] = torch.where(local >= 0, (local // 64 * world + rank) * 64 + local % 64, local)
        every_lists = gather_pieces(as_positions).cpu().numpy()
    if rank == 0:
        oracle.set_threads(host_threads())
        b_np = buckets_to_host(buckets)
        index_q = layer.index_queries(q)
        iq_np, pos_np = index_q[sample].cpu().numpy(), positions[sample].cpu().numpy()
        # the decode row maps its query through the few-rows kernels: one more sample row, at the last position
        iq_np = np.concatenate([iq_np, layer.index_queries(q1).cpu().numpy()])
        pos_np = np.concatenate([pos_np, [T - 1]])
        q_sample = torch.cat([q[sample], q1])
        attend_at = [owned[-1], len(sample)]  # an owned row of the chunk and the decode row
        latent_of = lambda ids: full[torch.from_numpy(ids.astype(np.int64)).cuda()].float().cpu().numpy()
        want_lists, want_lens, want_out, t_read, t_attend = c4_expected(cfg, attend_at, iq_np, pos_np, b_np, latent_of,
                                                                       q_sample)
        if world == 1:
            same = all(int(lens_d[r]) == int(want_lens[i]) and np.array_equal(
                lists_d[r, : int(lens_d[r])].cpu().numpy(), want_lists[i, : want_lens[i]]) for i, r in enumerate(sample))
        else:
            same = True
            for i in range(len(sample)):
                union = every_lists[:, i].reshape(-1)
                union = np.sort(union[union >= 0])
                same = same and np.array_equal(union, np.sort(want_lists[i, : want_lens[i]]))
        worst, mean = 0.0, 0.0
        for i in (owned[-1],):
            gap = np.abs(out_d[sample[i]].float().cpu().numpy() - want_out[i])
            worst, mean = max(worst, float(gap.max())), max(mean, float(gap.mean()))
        decode_gap = float(np.abs(out1[0].float().cpu().numpy() - want_out[len(sample)]).max())
        worst = max(worst, decode_gap)
        parity = {"rows_checked": len(sample), "lists_equal": bool(same), "attention_max_abs": worst,
                  "attention_mean_abs": mean, "decode_max_abs": decode_gap, "tolerance": TOLERANCE,
                  "against": "CPU oracle on the device's own index vectors"
                             + ("; the ranks' lists are united before they are compared" if world > 1 else "")}
        if not same:
            detail = ""
            if world > 1:
                for i in range(len(sample)):
                    union = every_lists[:, i].reshape(-1)
                    got_set, want_set = set(union[union >= 0].tolist()), set(want_lists[i, : want_lens[i]].tolist())
                    if got_set != want_set or len(got_set) != int((union >= 0).sum()):
                        detail = (f" (row {sample[i]}: {int((union >= 0).sum())} listed, {len(got_set)} distinct, "
                                  f"{len(want_set)} wanted, {len(want_set - got_set)} missing, "
                                  f"{len(got_set - want_set)} extra)")
                        break
            fail("C4 read lists differ from the oracle's" + detail)
        if worst > TOLERANCE["attention_max_abs"] or mean > TOLERANCE["attention_mean_abs"]:
            fail(f"C4 attention differs from the oracle: max-abs {worst}, mean-abs {mean}")
        # the CPU baseline on the same sample: per-token stage times summed
        n_map = 512
        rows_host = tail[:n_map].float().cpu().numpy()
        t0 = time.perf_counter()
        oracle.project_mlp(rows_host, kmap[0].float().t().cpu().numpy(), kmap[1].float().t().cpu().numpy())
        oracle.project_mlp(rows_host, qmap[0].float().t().cpu().numpy(), qmap[1].float().t().cpu().numpy())
        t_map = (time.perf_counter() - t0) / n_map
        per_token = t_map + t_read / (len(sample) + 1) + t_attend / len(attend_at)
        cpu = {"value": 1.0 / per_token, "unit": UNIT, "cores": host_threads(), "kind": "port",
               "sample": (f"maps of {n_map} tokens, read of {len(sample)} rows, attention of {len(attend_at)} rows "
                          f"({int(want_lens[attend_at[0]])} keys a row); per-token stage times summed (map "
                          f"{t_map * 1e3:.2f} read {t_read / len(sample) * 1e3:.1f} attend "
                          f"{t_attend / len(attend_at) * 1e3:.0f} ms)")}
        del full
    env.barrier()

    # ---- the timed regions
    for _ in range(args.warmup):
        step()
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    launches_before = _lib.LAUNCHES
    with ClockSampler(env.local) as clocks:
        ms = env.timed(step, args.steps)
    launches = (_lib.LAUNCHES - launches_before) // args.steps
    stage_ms = {name: total / args.steps for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()
    (sharded or layer).check()

    # What a kernel that does nothing but read the same rows reaches: the lists of 148 neighbouring query rows (what
    # the attention launch has in flight at once, a row an SM), walked 64 ids at a time across the rows as the
    # launch walks them, through the page-fingerprint kernel (a warp a 1,152-byte row, a wrapping sum of its words).
    gather_probe = None
    if world == 1:
        tile, mid = 64, chunk // 2
        group = min(148, chunk - mid)
        walked = int(lens_d[mid:mid + group].min()) // tile * tile
        ids = lists_d[mid:mid + group, :walked].reshape(group, walked // tile, tile).permute(1, 0, 2).reshape(-1)
        ids = ids.to(torch.int64)
        probe_gen = torch.Generator(device="cuda").manual_seed(1)
        by_word = torch.randint(-(1 << 62), 1 << 62, (dk * 2 // 8,), generator=probe_gen, device="cuda") | 1
        by_row = torch.randint(-(1 << 62), 1 << 62, (tile,), generator=probe_gen, device="cuda") | 1
        rows_2d = share.view(share.shape[0], -1)

        def read_rows():
            ops.page_fingerprints(rows_2d, tile, by_word, by_row, slots=ids)

        read_rows()
        probe_ms = max(env.timed(read_rows, 3), 1e-6)
        gather_probe = {"GB/s": ids.numel() * dk * 2 / (probe_ms * 1e-3) / 1e9, "rows_read": int(ids.numel()),
                        "ms": probe_ms,
                        "note": "lsa_page_fingerprints over the listed rows of 148 neighbouring query rows in the "
                                "attention launch's own order: a read-only gather of the same 1,152-byte rows"}
        del ids

    # from pinned host memory: the chunk's queries and (this rank's share of) its latent rows in, the output back
    from lsa_b200.parallel import deal

    # (on several GPUs a rank copies its own rows of the chunk's queries and the ranks all-gather them over NVLink:
    # every rank needs every row, but the host link need carry each row only once)
    pieces = 4
    if world == 1:
        q_h = q.cpu().pin_memory()
    else:  # this rank's rows of each of the four pieces the chunk crosses the host link in
        q_h = q.view(pieces, world, chunk // pieces // world, Hq, dk)[:, rank].reshape(own_rows, Hq, dk).cpu().pin_memory()
    tail_h = (tail if world == 1 else deal(tail, rank, world)).cpu().pin_memory()
    out_h = torch.empty(out_d.shape, dtype=out_d.dtype).pin_memory()

    def e2e_step():
        if world == 1:  # (the copies ride beside the work, a quarter of the chunk at a time)
            layer.prefill_from_host(q_h, tail_h, first, share, index, out_h)
            return
        sharded.prefill_from_host(q_h, tail_h, first, chunk, share, out_h, pieces=pieces)

    for _ in range(min(args.warmup, 3)):
        e2e_step()
    e2e_ms = env.timed(e2e_step, args.steps)

    decode_us, how = timed_graph(env, decode, 5, args.decode_steps)
    q1_h, out1_h = q1.cpu().pin_memory(), torch.empty(1, Hq, dv, dtype=torch.bfloat16).pin_memory()

    def decode_e2e():
        q1.copy_(q1_h, non_blocking=True)
        out1_h.copy_(decode(), non_blocking=True)

    # (the copies are part of the captured step: the row comes in from pinned host memory and its output goes back
    # inside the same graph, as a serving loop would replay it)
    decode_e2e_us, e2e_how = timed_graph(env, decode_e2e, 5, min(args.decode_steps, 64))
    torch.cuda.synchronize()
    if not torch.equal(out1_h, decode().cpu()):
        fail("the decode step replayed with its host copies does not return the resident step's output")
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    for _ in range(20):
        decode()
    decode_stages = {name: total * 1e3 / 20 for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()
    layer.check()

    # ---- the algorithmic work of a step, stage by stage (whole job: all ranks together)
    d = layer.design
    hidden = cfg["hidden_dim"]
    blocks_closed = T // d.cluster_block_size - first // d.cluster_block_size
    visible_total = float((positions // d.cluster_block_size * d.block_bucket_count).sum())
    picked_keys = gathered_total - chunk * (d.window_size + d.sink_size)  # ids the expansion writes
    map_flops = 2.0 * chunk * (dk * hidden + hidden * d_idx)
    work = {
        "index map": (chunk * Hq * dk * 2 + chunk * dk * 2 * 2 + 2 * chunk * d_idx * 4, 2 * map_flops),
        "pool": (blocks_closed * d.cluster_block_size * d_idx * 4 * 1.0, 0.0),
        "ward": (blocks_closed * (d.cluster_block_size // d.pool_size) * (d_idx * 4 + 8) * 1.0, 0.0),
        "bucket table": (blocks_closed * (d.cluster_block_size * d_idx * 4 + d.block_bucket_count * d.bucket_cap * 4)
                         * 1.0, 0.0),
        "select": (buckets.bucket_centroids.shape[0] * d_idx * 4 + chunk * d_idx * 4 + chunk * d.top_p * 12.0,
                   2.0 * visible_total * d_idx),
        "expand": (picked_keys * 4 + chunk * d.top_p * 4 + gathered_total * 4.0, 0.0),
        "attend": (gathered_total * dk * 2 + chunk * Hq * (dk + dv) * 2 + chunk * Hq * 4.0,
                   2.0 * gathered_total * Hq * (dk + dv)),
    }
    table = stage_table(work, stage_ms, pk, ms, world)
    attend = table["stages"]["attend"]
    attend_ms = stage_ms.get("attend")
    achieved = attend["bytes"] / world / (attend_ms * 1e-3) / 1e9 if attend_ms else None
    ratio = TRAFFIC["C4"]["ratio"]
    decode_list = float(lens_d[-1]) if world == 1 else env.total(float(lens_d[-1]))
    decode_bytes = decode_list * dk * 2 + float(buckets.bucket_centroids.shape[0]) * d_idx * 4
    result = {
        "metric": METRIC, "value": chunk / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": c4_config(cfg, world),
        "workload_stats": {"keys_read_per_row": gathered_total / chunk, "gathered_GB_per_step": attend["bytes"] / 1e9},
        "decode": {"us_per_step": decode_us, "timed": how, "steps": args.decode_steps,
                   "e2e_us_per_step": decode_e2e_us, "e2e_timed": e2e_how, "stages_us_eager": decode_stages,
                   "keys_read": decode_list,
                   "hbm_floor_us": decode_bytes / (pk["hbm_gbs"] * 1e3) / world,
                   "note": "one query row at the last position; the floor is its bytes at the copy bandwidth, the "
                           "step itself is a chain of dependent launches"},
        "e2e": {"value": chunk / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": (q_h.numel() * world + tail_h.numel() * world) * 2,
                "d2h_bytes_per_step": out_h.numel() * world * 2},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "parity": parity,
        "roofline": {"kernel": "latent_attend_tc_kernel (gather attention of a chunk's 8,192 rows: 1 launch a step)",
                     "bound": attend["bound"], "achieved": achieved, "peak": pk["hbm_gbs"], "peak_kind": pk["kind"],
                     "unit": "GB/s", "frac": achieved / pk["hbm_gbs"] if achieved else None,
                     "traffic": ratio * attend["bytes"] / world if ratio else None,
                     "traffic_from": TRAFFIC["C4"]["profile"],
                     "algorithmic_bytes_per_launch": attend["bytes"] / world,
                     "useful_tflops": attend["flops"] / world / (attend_ms * 1e-3) / 1e12 if attend_ms else None,
                     "tensor_frac": attend["flops"] / world / (attend_ms * 1e-3) / 1e12 / pk["tensor_tflops"]
                     if attend_ms else None,
                     "ms_per_launch": attend_ms, "gather_probe": gather_probe,
                     "note": "algorithmic bytes = every listed latent row once per query row (1,152 bytes) + Q in + "
                             "O out, per GPU; achieved = those bytes over the launch's CUDA-event time"},
        "stagewise": table,
        "stages_ms_per_step": stage_ms,
        "build_ms": build_ms,
    }
    if cpu:
        result["cpu_baseline"] = cpu
    return result if rank == 0 else None


# ------------------------------------------------------------------------------------------------ C2: GQA flat 128k


def run_c2(args, env: Env, cfg: dict, steps: int, cpu_baseline: bool = True) -> dict:
    import oracle
    from lsa_b200 import _lib, probe
    from lsa_b200 import workloads as W
    from lsa_b200.layer import FlatLayer
    from lsa_b200.parallel import ShardedFlatLayer, deal

    world, rank = env.world, env.rank
    pk = peaks()
    host = W.gqa_inputs(cfg, pin=True)
    q_h, k_h, v_h, wq, wk = host
    T, Hq, Hkv, dh, chunk = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["chunk"]
    base = FlatLayer(W.design_of(cfg), wq.cuda(), wk.cuda(), Hq, Hkv, dh)
    layer = base
    by_rows = world > 1 and args.parallel == "rows"
    if world > 1:
        layer = ShardedFlatLayer(base, rank, world)
        k_h, v_h = deal(k_h, rank, world).clone().pin_memory(), deal(v_h, rank, world).clone().pin_memory()
        if by_rows:
            q_h = layer.rows_of(q_h, chunk * world).clone().pin_memory()
    q, k, v = q_h.cuda(), k_h.cuda(), v_h.cuda()
    out_d = torch.empty(T // world, Hq, dh, dtype=torch.bfloat16, device="cuda")
    out_h = torch.empty(out_d.shape, dtype=torch.bfloat16).pin_memory()
    q_in, k_in, v_in = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def prefill(q_, k_, v_):
        if by_rows:  # the ranks take a chunk of 8,192 rows each, side by side
            return layer.prefill_by_rows(q_, k_, v_, T, chunk=chunk * world, out=out_d)
        return layer.prefill(q_, k_, v_, chunk=chunk, out=out_d)

    def resident_step():
        prefill(q, k, v)

    def e2e_step():
        if world == 1:  # the layer's own call for host-resident inputs: copies overlapped with the chunks' work
            base.prefill_from_host(q_h, k_h, v_h, out_h, chunk=chunk)
            return
        q_in.copy_(q_h, non_blocking=True)
        k_in.copy_(k_h, non_blocking=True)
        v_in.copy_(v_h, non_blocking=True)
        out_h.copy_(prefill(q_in, k_in, v_in), non_blocking=True)

    for _ in range(max(1, args.warmup)):
        resident_step()
    torch.cuda.synchronize()
    base.check()
    parity = cpu = None
    pairs = gathered = None
    if world == 1:
        # parity of sample rows of the timed output, and the counts the roofline needs
        out, index = base.prefill(q, k, v, chunk=chunk, return_index=True)
        index_q = base.index_queries(q)
        pairs = gathered = 0
        for start in range(0, T, chunk):
            pos = torch.arange(start, min(T, start + chunk), device="cuda")
            picked = base.pick(index_q[start:start + chunk], pos, index)[0]
            pairs += int((picked >= 0).sum())
            _, lengths = base.select(index_q[start:start + chunk], pos, index)
            window_start = (pos + 1 - cfg["window_size"]).clamp_min(0)
            fixed = (pos + 1 - window_start) + torch.minimum(window_start, torch.full_like(pos, cfg["sink_size"]))
            gathered += int((lengths.to(torch.int64) - fixed).sum())
        oracle.set_threads(host_threads())
        b_np = buckets_to_host(index.buckets)
        rows = np.unique(np.concatenate([np.linspace(0, T - 1, 24).astype(np.int64), [T - 1, chunk, chunk - 1]]))
        rows_d = torch.from_numpy(rows).cuda()
        lists_d, lens_d = base.select(index_q[rows_d], rows_d, index)
        iq_np = index_q[rows_d].cpu().numpy()
        t0 = time.perf_counter()
        want_lists, want_lens = oracle.read(iq_np, rows, b_np, cfg["top_p"], cfg["top_k"], cfg["sink_size"],
                                            cfg["window_size"])
        t_read = (time.perf_counter() - t0) / len(rows)
        same = bool(np.array_equal(lists_d.cpu().numpy(), want_lists) and np.array_equal(lens_d.cpu().numpy(),
                                                                                         want_lens))
        kf, vf = k_h.float().numpy(), v_h.float().numpy()
        t0 = time.perf_counter()
        want, _ = oracle.sparse_attend(q_h[torch.from_numpy(rows)].float().numpy(), kf, vf, want_lists, rows, 0, 0,
                                       dh ** -0.5, lengths=want_lens)
        t_attend = (time.perf_counter() - t0) / len(rows)
        gap = np.abs(out_d[rows_d].float().cpu().numpy() - want)
        parity = {"rows_checked": int(len(rows)), "lists_equal": same, "attention_max_abs": float(gap.max()),
                  "attention_mean_abs": float(gap.mean()), "tolerance": TOLERANCE}
        if not same:
            fail("C2 read lists differ from the oracle's")
        if gap.max() > TOLERANCE["attention_max_abs"] or gap.mean() > TOLERANCE["attention_mean_abs"]:
            fail(f"C2 attention differs from the oracle: max-abs {gap.max()}, mean-abs {gap.mean()}")
        if cpu_baseline:
            n_map = 8 * cfg["cluster_block_size"]
            qs, ks = q_h[:n_map].float().numpy(), k_h[:n_map].float().numpy()
            t0 = time.perf_counter()
            oracle.project(oracle.regroup_queries(qs, Hkv), wq.float().numpy())
            sample_keys = oracle.project(ks.reshape(n_map, -1), wk.float().numpy())
            t_map = (time.perf_counter() - t0) / n_map
            t0 = time.perf_counter()
            oracle.build_buckets(sample_keys, cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"],
                                 cfg["cluster_block_size"])
            t_build = (time.perf_counter() - t0) / n_map
            cpu = {"value": 1.0 / (t_map + t_build + t_read + t_attend), "unit": UNIT, "cores": host_threads(),
                   "kind": "port", "sample": f"map and build of {n_map} tokens, read and attention of {len(rows)} rows "
                                             f"spread over the context; per-token stage times summed"}
        del kf, vf

    for _ in range(max(3, args.warmup)):  # (the checks above left the GPU idle: warm it again)
        resident_step()
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    launches_before = _lib.LAUNCHES
    with ClockSampler(env.local) as clocks:
        ms = env.timed(resident_step, steps)
    launches = (_lib.LAUNCHES - launches_before) // steps
    stage_ms = {name: total / steps for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()
    for _ in range(2):
        e2e_step()
    e2e_ms = env.timed(e2e_step, steps)
    base.check()
    arms = None
    if world > 1:
        # the other way to part the same prefill over the ranks, timed for the record beside the one the line reports
        other_rows = not by_rows
        q_other = (layer.rows_of(host[0], chunk * world) if other_rows else host[0]).cuda()

        def other_step():
            if other_rows:
                layer.prefill_by_rows(q_other, k, v, T, chunk=chunk * world, out=out_d)
            else:
                layer.prefill(q_other, k, v, chunk=chunk, out=out_d)

        other_step()
        other_ms = env.timed(other_step, max(1, min(steps, 2)))
        base.check()
        rows_ms, context_ms = (ms, other_ms) if by_rows else (other_ms, ms)
        arms = {"rows split, cache all-gathered": {"value": T / (rows_ms * 1e-3), "ms_per_step": rows_ms},
                "context parallel over the dealt cache": {"value": T / (context_ms * 1e-3), "ms_per_step": context_ms}}
        del q_other

    result = {"metric": "LSA layer prefill tokens/s (flat, GQA, 128k tokens from position 0)", "value": T / (ms * 1e-3),
              "unit": UNIT, "n_gpus": world, "steps": steps, "ms_per_step": ms,
              "config": {"workload": cfg["workload"] if T == 131072 else f"C2 cut to {T} tokens", "tokens": T,
                         "heads": Hq, "kv_heads": Hkv, "head_dim": dh, "buckets": T // cfg["bucket_size"],
                         "top_p": cfg["top_p"], "window": cfg["window_size"], "chunk": chunk,
                         "parallelism": "1 GPU" if world == 1 else (
                             "rows of every chunk split over the ranks, the dealt cache all-gathered once a step"
                             if by_rows else "context parallel over the dealt cache, partial outputs merged")},
              "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": (q_h.numel() + k_h.numel() + v_h.numel()) * world * 2,
                      "d2h_bytes_per_step": out_h.numel() * world * 2},
              "gpu_launches": launches, "clocks": clocks.summary(), "parity": parity,
              "stages_ms_per_step": stage_ms}
    if arms is not None:
        result["arms"] = arms
    if world == 1:
        d_idx, d_in = cfg["index_dim"], Hkv * dh
        row = Hkv * dh * 2 * 2
        tiles = (T + 127) // 128
        chunks = (T + chunk - 1) // chunk
        kv_once = sum(min(T, (c + 1) * chunk) * row for c in range(chunks))
        visible_total = sum((p // cfg["cluster_block_size"]) * (cfg["cluster_block_size"] // cfg["bucket_size"])
                            for p in range(0, T, cfg["cluster_block_size"])) * cfg["cluster_block_size"]
        work = {
            "index map": (T * (Hq + Hkv) * dh * 2 + 2 * T * d_idx * 4.0, 2.0 * T * 2 * d_in * d_idx),
            "pool": (T * d_idx * 4 * 1.0625, 0.0),
            "ward": (T / cfg["pool_size"] * (d_idx * 4 + 8), 0.0),
            "bucket table": (T * d_idx * 4 + T / cfg["bucket_size"] * cfg["bucket_cap"] * 4.0, 0.0),
            "select": (chunks * (T / cfg["bucket_size"]) * d_idx * 4 * 0.5 + T * d_idx * 4 + T * cfg["top_p"] * 12.0,
                       2.0 * visible_total * d_idx),
            "band": (tiles * (cfg["window_size"] + 128 + cfg["sink_size"]) * row + T * Hq * dh * (2 + 4) + T * Hq * 4.0,
                     4.0 * T * (cfg["window_size"] + cfg["sink_size"]) * Hq * dh),
            # the selected keys, read bucket by bucket: a chunk's rows share their keys on chip, so the bytes the stage
            # MUST move are Q in, the band's partial in, O out and the visible K/V once a chunk
            "attend": (T * Hq * dh * (2 + 2) + T * Hq * (dh + 1) * 4 + kv_once * 1.0, 4.0 * gathered * Hq * dh),
        }
        table = stage_table(work, stage_ms, pk, ms, world)
        attend = table["stages"]["attend"]
        calls = chunks
        result["stagewise"] = table
        result["roofline"] = {
            "kernel": "bucket-major attend (bucket_starts, scan, scatter, segments, bucket_attend_tc, bucket_merge: "
                      "one call a chunk)",
            "bound": attend["bound"], "achieved": attend["flops"] / (stage_ms["attend"] * 1e-3) / 1e12,
            "peak": pk["tensor_tflops"], "peak_kind": pk["kind"], "unit": "TFLOP/s",
            "frac": attend["frac"], "launches_per_step": calls, "ms_per_launch": stage_ms["attend"] / calls,
            "traffic": None, "traffic_from": TRAFFIC["C2"]["profile"],
            "note": "frac = roofline time / measured time of the stage; the stage's floor is its products "
                    "(4 x gathered keys x heads x head dim) on the tensor cores at the sustained bf16 rate, its minimum "
                    "bytes (Q, the band's partial, O, visible K/V once a chunk) are the smaller term"}
        if cpu:
            result["cpu_baseline"] = cpu
    return result if rank == 0 else None


# ------------------------------------------------------------------------------------------------ C3: tree decode, 1M


def run_c3(args, env: Env, cfg: dict) -> dict:
    """One query a step over a 1M-token cache, a two-level tree of 64-child node buckets (single GPU)."""
    import oracle
    from lsa_b200 import probe
    from lsa_b200 import workloads as W
    from lsa_b200.decode import TreeDecoder
    from lsa_b200.hierarchy import build_hierarchy
    from lsa_b200.layer import FlatLayer

    pk = peaks()
    gen = torch.Generator(device="cuda").manual_seed(cfg["seed"])
    T, Hq, Hkv, dh = cfg["tokens"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    k, v = W.clustered_cache(T, Hkv, dh, cfg["centres"], gen)
    w = (torch.randn(2, Hkv * dh, cfg["index_dim"], generator=gen, device="cuda") / (Hkv * dh) ** 0.5).bfloat16()
    layer = FlatLayer(W.design_of(cfg), w[0], w[1], Hq, Hkv, dh)
    index = layer.build_index(k)
    tree = build_hierarchy(index.index_keys, index.buckets, cfg["top_level"], cfg["node_bucket_size"],
                           cfg["node_cluster_block_size"])
    position = T - 1
    decoder = TreeDecoder(layer, index.buckets, tree, cfg["beam_width"], None, cfg["page_size"], cfg["growth_buckets"],
                          splits=args.tree_splits)
    decoder.prepare(position)
    q = (0.7071 * k[position].repeat_interleave(Hq // Hkv, dim=0) + 0.7071 * torch.randn(
        Hq, dh, generator=gen, device="cuda").bfloat16())[None].contiguous()
    out = decoder.step(q, k, v)
    lists, lengths = decoder.select(q)
    torch.cuda.synchronize()
    layer.check()
    # parity: the oracle reads the same step from the device's own index
    oracle.set_threads(host_threads())
    b_np = buckets_to_host(index.buckets)
    tree_np = oracle.Hierarchy([c.cpu().numpy() for c in tree.node_centroids], [c.cpu().numpy() for c in tree.children],
                               cfg["node_bucket_size"], (cfg["node_cluster_block_size"],))
    index_q = layer.index_queries_rows(q).cpu().numpy()
    t0 = time.perf_counter()
    want_lists, want_len = oracle.read_hierarchy(index_q, np.array([position]), b_np, tree_np, cfg["beam_width"], None,
                                                 cfg["top_p"], cfg["top_k"], cfg["sink_size"], cfg["window_size"],
                                                 cfg["page_size"], cfg["growth_buckets"])
    t_read = time.perf_counter() - t0
    same = bool(np.array_equal(lists.cpu().numpy(), want_lists) and int(lengths[0]) == int(want_len[0]))
    ids = np.sort(want_lists[0, : want_len[0]])
    rows = torch.from_numpy(ids).cuda().long()
    kf, vf = k[rows].float().cpu().numpy(), v[rows].float().cpu().numpy()
    t0 = time.perf_counter()
    want, _ = oracle.sparse_attend(q.float().cpu().numpy(), kf, vf, np.arange(len(ids), dtype=np.int32)[None],
                                   np.array([len(ids)]), 0, 0, dh ** -0.5)
    t_attend = time.perf_counter() - t0
    gap = np.abs(out.float().cpu().numpy() - want)
    if not same:
        fail("C3 tree read list differs from the oracle's")
    if gap.max() > TOLERANCE["attention_max_abs"] or gap.mean() > TOLERANCE["attention_mean_abs"]:
        fail(f"C3 attention differs from the oracle: max-abs {gap.max()}")
    us, how = timed_graph(env, lambda: decoder.step(q, k, v), 5, args.decode_steps)
    recorder = probe.CudaEventRecorder()
    probe.install(recorder)
    for _ in range(20):
        decoder.step(q, k, v)
    stages = {name: total * 1e3 / 20 for name, (total, _) in recorder.totals_ms().items()}
    probe.uninstall()
    nodes = int(tree.children[0].shape[0])
    node_bytes = (nodes + cfg["beam_width"] * cfg["node_bucket_size"] + cfg["growth_buckets"]) * cfg["index_dim"] * 4
    kv_bytes = int(want_len[0]) * Hkv * dh * 2 * 2
    return {"metric": "tree decode us/step (1M-token cache, one request)", "value": us, "unit": "us", "timed": how,
            "higher_is_better": False, "n_gpus": 1,
            "config": {"workload": "C3", "tokens": T, "buckets": int(index.buckets.bucket_sizes.shape[0]),
                       "nodes": nodes, "beam": cfg["beam_width"], "top_p": cfg["top_p"], "keys_read": int(want_len[0])},
            "stages_us_eager": stages,
            "parity": {"lists_equal": same, "attention_max_abs": float(gap.max()), "attention_mean_abs": float(gap.mean())},
            "hbm_floor_us": (node_bytes + kv_bytes) / (pk["hbm_gbs"] * 1e3),
            "cpu_baseline": {"value": (t_read + t_attend) * 1e6, "unit": "us", "kind": "port", "cores": host_threads(),
                             "sample": "one step: tree read + attention"}}


# ------------------------------------------------------------------------------------------------ C5: batched decode


def run_c5(args, env: Env, cfg: dict) -> dict:
    """One decode step of 64 requests of 32k-512k tokens over a paged bf16 KV pool (page 64) and a paged bucket
    cache, flat design (single GPU)."""
    import oracle
    from lsa_b200 import ops
    from lsa_b200 import workloads as W
    from lsa_b200.layer import FlatLayer
    from lsa_b200.serving import BucketCache, Selector

    pk = peaks()
    gen = torch.Generator(device="cuda").manual_seed(cfg["seed"])
    rng = np.random.default_rng(cfg["seed"])
    B, Hq, Hkv, dh, kv_page = cfg["requests"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["kv_page"]
    design = W.design_of(cfg)
    lengths = W.request_lengths(cfg)
    total = int(lengths.sum())
    pool_pages = total // kv_page + B
    k, v = W.clustered_cache(pool_pages * kv_page, Hkv, dh, cfg["centres"], gen)
    w = (torch.randn(2, Hkv * dh, cfg["index_dim"], generator=gen, device="cuda") / (Hkv * dh) ** 0.5).bfloat16()
    layer = FlatLayer(design, w[0], w[1], Hq, Hkv, dh)
    # KV pages dealt to the requests in a shuffled order; a request's position p is slot pages[p / 64] * 64 + p % 64
    order = torch.from_numpy(rng.permutation(pool_pages).astype(np.int32)).cuda()
    kv_pages = torch.full((B, int(lengths.max()) // kv_page), -1, dtype=torch.int32, device="cuda")
    cache = BucketCache(design, cfg["index_dim"], pages=total // 8192 + 2 * B, page_buckets=cfg["page_buckets"],
                        max_requests=B, max_request_pages=int(lengths.max()) // 8192 + 1)
    taken = 0
    for r, n in enumerate(lengths.tolist()):
        count = n // kv_page
        kv_pages[r, :count] = order[taken:taken + count]
        taken += count
        slots = (kv_pages[r, :count].long()[:, None] * kv_page + torch.arange(kv_page, device="cuda")[None]).reshape(-1)
        for start in range(0, n, 1 << 17):  # index keys of the request, in position order, a piece at a time
            cache.append(r, layer.index_keys(k[slots[start:start + (1 << 17)]]))
    selector = Selector(cache, kv_page)
    rows = torch.arange(B, device="cuda")
    positions = torch.from_numpy(lengths - 1).cuda()
    last_slot = kv_pages[rows, (positions // kv_page)].long() * kv_page + positions % kv_page
    q = (0.7071 * k[last_slot].repeat_interleave(Hq // Hkv, dim=1) + 0.7071 * torch.randn(
        B, Hq, dh, generator=gen, device="cuda")).bfloat16().contiguous()
    visible = selector.visible(rows, positions)

    def step():
        lists, lens = selector.decode_flat(layer.index_queries(q), rows, positions, kv_pages, visible=visible,
                                           splits=4)
        return ops.sparse_attend(q, k, v, lists, lens, layer.scale, splits=args.tree_splits)[0], lists, lens

    out, lists, lens = step()
    torch.cuda.synchronize()
    layer.check()
    # parity on a few requests, the oracle reading each from the device's own index vectors
    oracle.set_threads(host_threads())
    index_q = layer.index_queries(q).cpu().numpy()
    order_by_len = np.argsort(lengths)
    checked, worst, mean, t_cpu = 0, 0.0, 0.0, 0.0
    for r in [int(order_by_len[0]), int(order_by_len[B // 2])]:
        n = int(lengths[r])
        slots = (kv_pages[r, : n // kv_page].long()[:, None] * kv_page + torch.arange(kv_page, device="cuda")[None]
                 ).reshape(-1)
        index_k = torch.cat([layer.index_keys(k[slots[s:s + (1 << 17)]]) for s in range(0, n, 1 << 17)]).cpu().numpy()
        buckets = oracle.build_buckets(index_k, cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"],
                                       cfg["cluster_block_size"])
        t0 = time.perf_counter()
        want, want_len = oracle.read(index_q[r:r + 1], np.array([n - 1]), buckets, cfg["top_p"], cfg["top_k"],
                                     cfg["sink_size"], cfg["window_size"])
        ids = want[0, : want_len[0]]
        mine = lists[r, : int(lens[r])].cpu().numpy()
        want_slots = slots[torch.from_numpy(ids.astype(np.int64)).cuda()].cpu().numpy()
        if int(lens[r]) != int(want_len[0]) or not np.array_equal(mine, want_slots):
            fail(f"C5 request {r}: read list differs from the oracle's")
        gathered = torch.from_numpy(want_slots).cuda().long()
        ref, _ = oracle.sparse_attend(q[r:r + 1].float().cpu().numpy(), k[gathered].float().cpu().numpy(),
                                      v[gathered].float().cpu().numpy(), np.arange(len(ids), dtype=np.int32)[None],
                                      np.array([len(ids)]), 0, 0, dh ** -0.5)
        t_cpu += time.perf_counter() - t0
        gap = np.abs(out[r].float().cpu().numpy() - ref[0])
        worst, mean = max(worst, float(gap.max())), max(mean, float(gap.mean()))
        checked += 1
    if worst > TOLERANCE["attention_max_abs"] or mean > TOLERANCE["attention_mean_abs"]:
        fail(f"C5 attention differs from the oracle: max-abs {worst}")
    us, how = timed_graph(env, lambda: step(), 3, min(args.decode_steps, 64))
    listed = int(lens.sum())
    centroid_bytes = int(visible.sum()) * cfg["index_dim"] * 4
    kv_bytes = listed * Hkv * dh * 2 * 2
    return {"metric": "batched decode steps/s (64 requests, paged KV)", "value": 1e6 / us, "unit": "steps/s",
            "us_per_step": us, "timed": how, "higher_is_better": True, "n_gpus": 1,
            "config": {"workload": "C5", "requests": B, "tokens_total": total, "min_len": int(lengths.min()),
                       "max_len": int(lengths.max()), "kv_page": kv_page, "top_p": cfg["top_p"], "keys_read": listed},
            "parity": {"requests_checked": checked, "lists_equal": True, "attention_max_abs": worst,
                       "attention_mean_abs": mean},
            "hbm_floor_us": (centroid_bytes + kv_bytes) / (pk["hbm_gbs"] * 1e3),
            "roofline_frac": (centroid_bytes + kv_bytes) / (pk["hbm_gbs"] * 1e3) / us,
            "cpu_baseline": {"value": 1.0 / (t_cpu / max(checked, 1) * B), "unit": "steps/s", "kind": "port",
                             "cores": host_threads(), "sample": f"read + attention of {checked} requests, scaled to {B}"}}


# ------------------------------------------------------------------------------------------------ the CPU arm


def run_reference(args, cfg: dict) -> dict | None:
    """The CPU arm: the oracle - a C port of the reference's PyTorch specification of this path - timed on the host
    cores, on a bounded sample of the C4 step. The index the sample's rows search is built over a stand-in context of
    64 cluster blocks (327,680 tokens, 512 buckets) with linear stand-ins for the key vectors: a row still scores
    every visible bucket, picks 128 and reads their members plus its window and sinks, which is what its cost is."""
    if int(os.environ.get("RANK", "0")) != 0:
        return None
    import oracle
    from lsa_b200 import workloads as W

    oracle.build()
    threads = oracle.set_threads(host_threads())
    rng = np.random.default_rng(cfg["seed"])
    dk, dv, d_idx, hidden, Hq = cfg["latent_dim"], cfg["value_dim"], cfg["index_dim"], cfg["hidden_dim"], cfg["heads"]
    block = cfg["cluster_block_size"]
    tokens = 64 * block
    mu = rng.standard_normal((cfg["centres"], dv), dtype=np.float32)
    latent = np.empty((tokens, dk), dtype=np.float32)
    latent[:, :dv] = 0.7071 * mu[rng.integers(0, cfg["centres"], tokens)] + 0.7071 * rng.standard_normal(
        (tokens, dv), dtype=np.float32)
    latent[:, dv:] = rng.standard_normal((tokens, dk - dv), dtype=np.float32)
    w1 = (rng.standard_normal((dk, hidden), dtype=np.float32) / dk ** 0.5)
    w2 = (rng.standard_normal((hidden, d_idx), dtype=np.float32) / hidden ** 0.5)
    # untimed: index keys of the stand-in context through a random LINEAR map (the timed sample maps its own rows
    # through the two-layer map), and its buckets
    index_keys = oracle.project(latent, (w1[:, :d_idx] + w1[:, d_idx:2 * d_idx]).copy())
    buckets = oracle.build_buckets(index_keys, cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"], block)
    n_map, n_read, n_attend, attend_keys = 256, 4, 1, 16384
    positions = np.full(n_read, tokens - 1, dtype=np.int64) - np.arange(n_read)
    q = (0.7071 * latent[positions][:, None, :] + 0.7071 * rng.standard_normal((n_read, Hq, dk), dtype=np.float32))
    scale = W.latent_scale(cfg)
    rates, last = [], None
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        oracle.project_mlp(latent[:n_map], w1, w2)
        index_q = oracle.project_mlp(q[:, :, :].sum(1), w1, w2)
        t_map = (time.perf_counter() - t0) / (n_map + n_read) * 2  # a token maps its key row and its query row
        t0 = time.perf_counter()
        oracle.build_buckets(index_keys[:block], cfg["pool_size"], cfg["bucket_size"], cfg["bucket_cap"], block)
        t_build = (time.perf_counter() - t0) / block
        t0 = time.perf_counter()
        lists, lens = oracle.read(index_q, positions, buckets, cfg["top_p"], cfg["top_k"], cfg["sink_size"],
                                  cfg["window_size"])
        t_read = (time.perf_counter() - t0) / n_read
        # (attention is linear in the keys a row reads: the first `attend_keys` of the list are timed and the time is
        # scaled to the whole list, which keeps a step of this arm to a few seconds)
        t_attend = 0.0
        for i in range(n_attend):
            ids = lists[i, : min(int(lens[i]), attend_keys)]
            rows = latent[ids]
            t0 = time.perf_counter()
            oracle.sparse_attend(q[i:i + 1], rows[:, None, :], rows[:, None, :], np.arange(len(ids), dtype=np.int32)[None],
                                 np.array([len(ids)]), 0, 0, scale)
            t_attend += (time.perf_counter() - t0) * int(lens[i]) / len(ids) / n_attend
        last = (t_map, t_build, t_read, t_attend, int(lens[0]))
        if step >= args.warmup:
            rates.append(1.0 / (t_map + t_build + t_read + t_attend))
    value = statistics.median(rates)
    t_map, t_build, t_read, t_attend, keys = last
    sample = (f"maps of {n_map} tokens, clustering of one block, read of {n_read} rows and attention of {n_attend} row "
              f"(its first {attend_keys} of {keys} keys, scaled to all of them) at the end of a {tokens}-token stand-in "
              f"context; per-token stage times summed (map "
              f"{t_map * 1e3:.2f} build {t_build * 1e3:.3f} read {t_read * 1e3:.1f} attend {t_attend * 1e3:.0f} ms)")
    chunk = cfg["chunk"]
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": chunk / value * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": c4_config(cfg, args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ------------------------------------------------------------------------------------------------ main


def main() -> None:
    from lsa_b200 import workloads as W

    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="C4", choices=["C4", "C2", "C3", "C5"])
    parser.add_argument("--also", default=None, help="workloads that ride along as `also` (comma-separated, or "
                                                     "'none'); default: C2,C3,C5 on one GPU, C2 on several")
    parser.add_argument("--tokens", type=int, default=None, help="a shorter context of the same workload (profiling)")
    parser.add_argument("--decode-steps", type=int, default=256)
    parser.add_argument("--decode-splits", type=int, default=148, help="CTAs a decode row's list is divided over")
    parser.add_argument("--tree-splits", type=int, default=16)
    parser.add_argument("--parallel", default="rows", choices=["rows", "context"],
                        help="C2 at N > 1: split the query rows over the ranks (the cache is all-gathered once a "
                             "step), or keep every rank on the keys it stores and merge partial outputs")
    args = parser.parse_args()
    if args.impl == "reference":
        result = run_reference(args, dict(W.C4))
        if result is not None:
            print(json.dumps(result))
        return

    env = Env(args.gpus)
    cfgs = {name: dict(cfg) for name, cfg in W.CONFIGS.items()}
    if args.tokens:
        cfgs[args.workload] = W.cut(cfgs[args.workload], args.tokens)
    also = args.also if args.also is not None else ("C2,C3,C5" if env.world == 1 else "C2")
    also = [name for name in also.split(",") if name and name != "none" and name != args.workload]

    def run(name: str, headline: bool):
        steps = args.steps if headline else min(args.steps, 10)
        if name == "C4":
            return run_c4(args, env, cfgs["C4"])
        if name == "C2":
            return run_c2(args, env, cfgs["C2"], steps, cpu_baseline=headline)
        if env.world > 1:
            return None  # (single-GPU workloads)
        return run_c3(args, env, cfgs["C3"]) if name == "C3" else run_c5(args, env, cfgs["C5"])

    result = run(args.workload, True)
    torch.cuda.empty_cache()
    extras = {}
    for name in also:
        got = run(name, False)
        torch.cuda.empty_cache()
        if got is not None:
            extras[name] = got
    env.close()
    if env.rank == 0 and result is not None:
        result.setdefault("warmup", args.warmup)
        result.setdefault("higher_is_better", True)
        result.setdefault("scaling", "strong")
        result.setdefault("vs_baseline", None)
        result.setdefault("dtype", "bf16")
        result.setdefault("data", "synthetic")
        if extras:
            result["also"] = extras
        print(json.dumps(result))


if __name__ == "__main__":
    main()
