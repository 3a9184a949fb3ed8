"""Benchmark of the paged KV-cache hot path (append + gather) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl barqkv|reference]

Workload (the Llama-3-8B-shaped decode configuration): 32 layers, 8 KV heads
(sharded N ways by KV head), head_dim 128, bf16, page size 16; 64 sequences
with seeded prompt lengths uniform in [512, 4096] prefilled into a pool whose
free list is a seeded permutation; then decode steps.  One STEP is one pass of
the hot path over the batch: for every layer, append one new token per
sequence through the block table, then gather every sequence's pages into
contiguous ``[H, sum_len, D]`` K and V (the attention operand).

The printed JSON line follows the driver's contract; ``value`` is whole-job
GB/s of ALGORITHMIC bytes (append 4*N_tok*H*D*e + gather 4*sum_len*H*D*e per
layer, K and V, read + write; index traffic excluded) with inputs resident in
HBM; ``e2e`` is the same metric through the public Python API with the step's
new K/V rows coming from pinned host memory and the status word read back.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "paged KV append+gather HBM GB/s"
UNIT = "GB/s"
NOMINAL_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0

CFG = dict(name="llama3-8b-decode", layers=32, kv_heads=8, head_dim=128, dtype="bf16", page_size=16, batch=64,
           prompt_lo=512, prompt_hi=4096, seed=1236)


def init_nccl(dist, device) -> None:
    """Create the process group and its communicator with file descriptor 1 pointed at stderr: NCCL
    prints its version banner to stdout when the communicator comes up, and stdout carries the JSON line."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
        torch.cuda.synchronize(device)
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_PEAK_GBS, "fallback"


def seeded_lengths():
    g = torch.Generator().manual_seed(CFG["seed"])
    lens = torch.randint(CFG["prompt_lo"], CFG["prompt_hi"] + 1, (CFG["batch"],), generator=g).tolist()
    return g, lens


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[3:7]):
                if flag.lower() == "active":
                    reasons.add(name)
        if sm:
            self.summary = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                            "samples": len(sm)}


# ---------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------
class DecodeWorkload:
    def __init__(self, world: int, rank: int, device: torch.device, total_steps: int, fused: bool = True,
                 heads: int = 0):
        self.fused = fused          # one update() launch per layer instead of append() + gather()
        self.graph = None
        from barqtrain_b200 import BlockTableKVCache
        from barqtrain_b200.sharding import kv_head_shard

        self.L, self.D, self.ps, self.B = CFG["layers"], CFG["head_dim"], CFG["page_size"], CFG["batch"]
        if CFG["kv_heads"] % world:
            raise SystemExit(f"--gpus must divide the {CFG['kv_heads']} KV heads")
        self.first_head, self.H = kv_head_shard(CFG["kv_heads"], world, rank)   # this rank's KV heads
        if heads:                    # experiments: another shard size on this GPU (1 = an 8-GPU rank's work)
            self.H = heads
        self.dtype = torch.bfloat16
        self.device = device
        g, self.prompts = seeded_lengths()
        final = [n + total_steps for n in self.prompts]
        num_pages = sum(-(-n // self.ps) for n in final)
        order = torch.randperm(num_pages, generator=g).tolist()
        self.cache = BlockTableKVCache(self.L, self.H, self.D, page_size=self.ps, num_pages=num_pages,
                                       max_seqs=self.B, max_blocks_per_seq=-(-max(final) // self.ps),
                                       dtype=self.dtype, device=device, free_order=order, zero_pages=False)
        self.slots = [self.cache.open(i) for i in range(self.B)]
        self.row_bytes = self.D * 2

        # prefill (untimed set-up): the prompts' K/V through the same append kernel, 2048-token chunks
        gen = torch.Generator(device=device).manual_seed(CFG["seed"] + rank)
        chunk = 2048
        done = [0] * self.B
        while any(d < n for d, n in zip(done, self.prompts)):
            counts = [min(chunk, n - d) for d, n in zip(done, self.prompts)]
            total = sum(counts)
            k = torch.randn(total, self.H, self.D, generator=gen, device=device, dtype=torch.float32).to(self.dtype)
            v = torch.randn(total, self.H, self.D, generator=gen, device=device, dtype=torch.float32).to(self.dtype)
            batch = self.cache.begin_append(self.slots, counts)
            for layer in range(self.L):
                self.cache.append(layer, batch, k, v)
            self.cache.end_append(batch)
            done = [d + c for d, c in zip(done, counts)]
        # per-step new rows, [L, B, H, D]; a few distinct sets cycled
        self.new_k = [torch.randn(self.L, self.B, self.H, self.D, generator=gen, device=device,
                                  dtype=torch.float32).to(self.dtype) for _ in range(4)]
        self.new_v = [torch.randn(self.L, self.B, self.H, self.D, generator=gen, device=device,
                                  dtype=torch.float32).to(self.dtype) for _ in range(4)]
        max_total = sum(final)
        self.out = [(torch.empty(self.H, max_total, self.D, dtype=self.dtype, device=device),
                     torch.empty(self.H, max_total, self.D, dtype=self.dtype, device=device)) for _ in range(2)]
        self.host_k = torch.empty(self.L, self.B, self.H, self.D, dtype=self.dtype).pin_memory()
        self.host_v = torch.empty(self.L, self.B, self.H, self.D, dtype=self.dtype).pin_memory()
        self.host_k.copy_(self.new_k[0])
        self.host_v.copy_(self.new_v[0])
        self.stage_k = torch.empty_like(self.new_k[0])
        self.stage_v = torch.empty_like(self.new_v[0])
        self.host_status = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.step_no = 0
        torch.cuda.synchronize(device)

    def sum_len(self) -> int:
        return int(sum(self.cache.lengths[s] for s in self.slots))

    def step_bytes(self, sum_len_after: int):
        """Algorithmic bytes of one step on THIS rank: (append, gather)."""
        per_tok = 4 * self.H * self.row_bytes
        return self.B * per_tok * self.L, sum_len_after * per_tok * self.L

    def step(self, k_all: torch.Tensor, v_all: torch.Tensor, events=None):
        """One pass of the hot path: per layer, append B tokens then gather all sequences."""
        cache = self.cache
        ab = cache.begin_append(self.slots, [1] * self.B)
        cache.end_append(ab)                       # lengths now include this step's token
        gb = cache.begin_gather(self.slots)
        total = gb.total
        # [H, total, D] prefixes of the two reusable output buffers (layers alternate between them)
        n = self.H * total * self.D
        outs = [(ko.view(-1)[:n].view(self.H, total, self.D), vo.view(-1)[:n].view(self.H, total, self.D))
                for ko, vo in self.out]
        k_rows, v_rows = k_all.unbind(0), v_all.unbind(0)
        for layer in range(self.L):
            timed = events is not None and (layer & 7) == 0       # a sample of launches carries event pairs
            if timed:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            if self.fused:
                cache.update(layer, ab, gb, k_rows[layer], v_rows[layer], "HND", out=outs[layer & 1])
            else:
                cache.append(layer, ab, k_rows[layer], v_rows[layer])
                cache.gather(layer, gb, "HND", out=outs[layer & 1])
            if timed:
                e1.record()
                events.append((e0, e1, total))
        self.step_no += 1
        return total

    def enable_graph(self):
        """Replay the step's launches from a CUDA graph (``DecodeStepGraph``): eager step, record, replay."""
        from barqtrain_b200 import DecodeStepGraph

        self.graph = DecodeStepGraph(self.cache, self.slots, capacity_tokens=self.out[0][0].size(1))
        self.graph.k_in.copy_(self.new_k[0])
        self.graph.v_in.copy_(self.new_v[0])
        self.out = None                                    # the graph owns its output buffers
        self.graph.step()
        self.graph.record()
        self.graph.step()
        self.step_no += 2

    def append_only_leg(self, steps: int, barrier, max_over_ranks, backend):
        """Decode tokens appended per second with nothing but the append in the timed region: every step
        appends one token per sequence in every layer - one launch per layer (what a model's forward pass
        issues), and again with one launch for all layers - replayed from a CUDA graph."""
        from barqtrain_b200 import DecodeStepGraph

        out = {}
        for name, what in (("per_layer", "append"), ("all_layers_one_launch", "append_layers")):
            g = DecodeStepGraph(self.cache, self.slots, capacity_tokens=0, what=what)
            g.k_in.copy_(self.new_k[1])
            g.v_in.copy_(self.new_v[1])
            g.step()
            g.record()
            for _ in range(3):
                g.step()
            half = max(steps // 2, 1)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(half):
                g.step()
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1))
            out[name] = {"tokens_per_s": round(self.B * half / (ms * 1e-3), 1), "us_per_step": round(ms * 1e3 / half, 2),
                         "steps": half, "launches_per_step": g.launches_per_replay,
                         "gbs_per_gpu": round(self.step_bytes(0)[0] * half / (ms * 1e-3) / 1e9, 1)}
        out["note"] = ("a token = its K and V rows in all %d layers; the append moves %.1f MiB per step per GPU, so "
                       "these steps are bound by launches, not by bandwidth" % (self.L, self.step_bytes(0)[0] / 2 / 2**20))
        return out

    def resident_step(self, events=None):
        if self.graph is not None:                          # inputs stay in the graph's resident buffers
            self.step_no += 1
            return self.graph.step()
        i = self.step_no % 4
        return self.step(self.new_k[i], self.new_v[i], events)

    def e2e_step(self):
        """Public-API step with host inputs: H2D of the step's new K/V, the hot path, D2H of the status word."""
        if self.graph is not None:
            self.graph.k_in.copy_(self.host_k, non_blocking=True)
            self.graph.v_in.copy_(self.host_v, non_blocking=True)
            total = self.graph.step()
            self.step_no += 1
        else:
            self.stage_k.copy_(self.host_k, non_blocking=True)
            self.stage_v.copy_(self.host_v, non_blocking=True)
            total = self.step(self.stage_k, self.stage_v)
        self.host_status.copy_(self.cache._status, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        if int(self.host_status[0]) != 0:
            raise RuntimeError(f"device guard fired: status {int(self.host_status[0])}")
        return total


def _median(xs):
    return statistics.median(xs)


def run_barqkv(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N > 1")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        init_nccl(dist, device)

    from barqtrain_b200 import _ffi

    backend = _ffi.require_cuda_backend()
    K, W = args.steps, max(args.warmup, 3)
    e2e_steps = max(3, min(K, 10))
    # The K-step region is timed again and again until a second has gone by (at most 256 decode steps in
    # all, the configuration's length), so that clock samples exist; the line reports the median region.
    max_regions = max(1, min(12, 256 // max(K, 1)))
    append_steps = 64
    total_steps = W + K * max_regions + 3 + e2e_steps + 8 + append_steps + 8 + (K + 4)
    if args.tune:
        backend.set_tuning(**{k: int(v) for k, v in (kv.split("=") for kv in args.tune.split(","))})
    wl = DecodeWorkload(world, rank, device, total_steps, fused=not args.two_launches, heads=args.shard_heads)
    use_graph = not args.eager and not args.two_launches
    if use_graph:
        wl.enable_graph()

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- resident leg: `value` -------------------------------------------------
    for _ in range(W):
        wl.resident_step()
    barrier()
    events = []
    regions = []          # (ms, append bytes, gather bytes, launches) of every timed K-step region
    with ClockSampler(local) as clocks:
        spent = 0.0
        while True:
            launches0 = backend.launches
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            app_bytes = gat_bytes = 0
            barrier()
            start.record()
            for _ in range(K):
                total = wl.resident_step(events)
                a, g = wl.step_bytes(total)
                app_bytes += a
                gat_bytes += g
            stop.record()
            barrier()
            launches = backend.launches - launches0
            if use_graph:
                # kernel nodes replayed (a replay makes no library call) plus what the library launched itself in
                # the region: the small table-scatter kernel of the steps in which a sequence enters a new page
                launches += K * wl.graph.launches_per_replay
            ms = max_over_ranks(start.elapsed_time(stop))
            regions.append((ms, app_bytes, gat_bytes, launches))
            spent += ms
            if spent >= 1000.0 * args.min_seconds or len(regions) >= max_regions:
                break
    rates = [(a + g) * world / (ms * 1e-3) / 1e9 for ms, a, g, _ in regions]
    value = _median(rates)
    ms = _median([r[0] for r in regions])
    app_bytes = _median([r[1] for r in regions])
    gat_bytes = _median([r[2] for r in regions])
    launches = sum(r[3] for r in regions)
    status = backend.read_status(device)
    if status:
        raise SystemExit(f"device guard fired during the timed region: status {status}")

    # ---- roofline of the dominant kernel (gather), per launch ---------------------
    peak, peak_kind = measured_peak()
    per_tok = 4 * wl.H * wl.row_bytes
    if events:
        durs = [e0.elapsed_time(e1) * 1e-3 for e0, e1, _ in events]
        # a sampled launch moves the gather's bytes plus (fused) the appended rows' bytes
        gbytes = [(t + wl.B) * per_tok for _, _, t in events]
        avg_dur = sum(durs) / len(durs)
        avg_bytes = sum(gbytes) / len(gbytes)
        how = f"event pairs around {len(events)} sampled launches inside the timed regions"
    else:
        # graph replay: a timed region is nothing but these launches back to back, so its CUDA-event
        # time divided by the launch count is the launch duration (kernel plus the gap to the next one)
        n_launch = len(regions) * K * wl.L
        avg_dur = sum(r[0] for r in regions) * 1e-3 / n_launch
        avg_bytes = sum(r[1] + r[2] for r in regions) / n_launch
        how = (f"{len(regions)} timed regions / {n_launch} launches of the replayed graph; neighbouring layers' launches "
               "overlap at their ends, so this is the interval between launches, not a lone launch's duration")
    achieved = avg_bytes / avg_dur / 1e9
    roofline = {"bound": "hbm", "kernel": "gather_bulk_kernel" + (" (append fused)" if wl.fused else " + append_rows_kernel"),
                "how": how, "achieved": round(achieved, 1), "peak": peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "frac_of_nominal_8TBs": round(achieved / NOMINAL_PEAK_GBS, 4),
                "avg_launch_us": round(avg_dur * 1e6, 2), "bytes_per_launch": int(avg_bytes),
                "traffic": None}
    tpath = ROOT / "profiles" / "gather_bulk_traffic.json"
    if tpath.exists():
        try:
            t = json.loads(tpath.read_text())
            # DRAM bytes per algorithmic byte measured by ncu on a smaller case with the same number of KV
            # heads per GPU, scaled to this launch; null for a head count nobody captured
            ratio = t.get("by_heads", {}).get(str(wl.H))
            if ratio is not None:
                roofline["traffic"] = int(ratio * roofline["bytes_per_launch"])
                roofline["traffic_source"] = t.get("source")
        except Exception:  # noqa: BLE001
            pass

    # ---- end-to-end leg ---------------------------------------------------------
    for _ in range(3):
        wl.e2e_step()
    barrier()
    e2e_bytes = 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        total = wl.e2e_step()
        a, g = wl.step_bytes(total)
        e2e_bytes += a + g
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_value = e2e_bytes * world / e2e_s / 1e9
    h2d = 2 * wl.host_k.numel() * wl.host_k.element_size()

    # ---- the same step with every layer on one stream, each launch behind the one before ------
    one_stream = None
    if use_graph:
        wl.graph.one_stream = True
        wl.graph.record()
        for _ in range(3):
            wl.resident_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        chain_bytes = 0
        e0.record()
        for _ in range(K):
            total = wl.resident_step()
            a, g = wl.step_bytes(total)
            chain_bytes += a + g
        e1.record()
        barrier()
        chain_ms = max_over_ranks(e0.elapsed_time(e1))
        one_stream = {"value": round(chain_bytes * world / (chain_ms * 1e-3) / 1e9, 1), "unit": UNIT,
                      "ms_per_step": round(chain_ms / K, 4), "steps": K,
                      "note": "one region of the same step recorded with every layer's launch on one stream, each a "
                              "programmatic dependent of the one before (a layer waits for the layer before it, as in a "
                              "model's forward pass); `value` above lets neighbouring layers overlap at their ends"}
        wl.graph.one_stream = False
        wl.graph.record()

    # ---- the metric's second half: decode tokens appended per second, append only -------
    append_only = wl.append_only_leg(append_steps, barrier, max_over_ranks, backend) if use_graph else None

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": decode_config(world),
        "run": {"kv_heads_per_gpu": wl.H, "sum_len_tokens": wl.sum_len(),
                "pool_gb_read_per_step_per_gpu": round(gat_bytes / K / 2 / 1e9, 1),
                "launch": ("one update() kernel per layer" if wl.fused else "append() + gather() per layer")
                + (", odd layers on a second stream so that neighbouring layers overlap at their ends (a layer is "
                   "ordered behind the layer two before it, whose output buffer it reuses), replayed from a CUDA graph"
                   if use_graph else ", called from Python")},
        "timed_regions": {"count": len(regions), "steps_each": K, "ms_median": round(ms, 3),
                          "ms_min": round(min(r[0] for r in regions), 3), "ms_max": round(max(r[0] for r in regions), 3),
                          "value_min": round(min(rates), 1), "value_max": round(max(rates), 1),
                          "note": "value and ms_per_step are the median region's; every region is exactly `steps` steps "
                                  "between barriers, max over ranks"},
        "pct_of_nominal_8TBs": round(100 * value / world / NOMINAL_PEAK_GBS, 2),
        "pct_of_measured_copy": round(100 * value / world / peak, 2),
        "decode_tokens_per_s": round(wl.B * K / (ms * 1e-3), 1),
        "append_gb_per_step": round(app_bytes * world / K / 1e9, 4),
        "gather_gb_per_step": round(gat_bytes * world / K / 1e9, 3),
        "roofline": roofline,
        "one_stream": one_stream,
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": 4 * world, "steps": e2e_steps,
                "ms_per_step": round(e2e_s * 1e3 / e2e_steps, 4),
                "note": "per step: the new K/V rows of all layers come from pinned host memory, the step runs, and "
                        "the 4-byte device status word is read back and checked; the gathered K/V stay on the device "
                        "on purpose - they are the attention operand, not a result the host consumes"},
        "gpu_launches": launches,
        "clocks": clocks.summary,
    }
    if append_only is not None:
        line["decode_append_tokens_per_s"] = append_only["per_layer"]["tokens_per_s"]
        line["decode_append"] = append_only

    # ---- the other configurations, short legs -----------------------------------------
    if not args.no_legs and not args.shard_heads:
        del wl
        gc.collect()
        torch.cuda.empty_cache()
        line["configs"] = run_legs(world, rank, local, device, barrier, max_over_ranks, backend, peak, peak_kind,
                                   quick=args.quick_legs)

    # ---- CPU baseline beside it (rank 0, N = 1 only) ------------------------------
    if world == 1:
        line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_seconds)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_legs(world, rank, local, device, barrier, max_over_ranks, backend, peak, peak_kind, quick=False):
    """Short legs of the other configurations (chunked prefill at page 16 and 32, the 70B-shaped gather,
    continuous-batching churn, the decode configuration with attention from the pages), each through ``barqtrain_b200.benchmarks.workloads`` at the
    configuration's full shape for this rank's KV-head shard; one entry per leg."""
    from barqtrain_b200.benchmarks.workloads import WORKLOADS

    plan = [
        # (name, workload, arguments, timed steps, warm-up steps): step counts sized for about a second of device
        # time at one GPU; the churn configuration's 1000 steps are the configuration's own
        ("chunked-prefill-ps16", "prefill", dict(page_size=16), 640, 8),
        ("chunked-prefill-ps32", "prefill", dict(page_size=32), 640, 8),
        ("llama3-70b-gather", "gather70b", {}, 44, 3),
        ("continuous-batching-churn", "churn", {}, 1000, 20),
        # the decode configuration once more with attention reading the pages instead of the gather (K/V read once)
        ("decode-attention-from-pages", "decode-attn", {}, 200, 5),
    ]
    out = {}
    for name, key, kwargs, steps, warmup in plan:
        if quick:
            steps, warmup = max(4, steps // 8), 3
            if key not in ("churn", "decode-attn"):
                kwargs = dict(kwargs, layers=8)
        try:
            with ClockSampler(local) as clocks:
                res = WORKLOADS[key](world, rank, device, steps, warmup, sync=barrier, **kwargs)
            ms = max_over_ranks(res["ms"])
            value = res["bytes"] * world / (ms * 1e-3) / 1e9
            entry = {"workload": res["config"], "value": round(value, 1), "unit": UNIT, "steps": steps, "warmup": warmup,
                     "ms_per_step": round(ms / steps, 4), "seconds_timed": round(ms * 1e-3, 3),
                     "frac_of_%s_copy" % peak_kind: round(value / world / peak, 4),
                     "frac_of_nominal_8TBs": round(value / world / NOMINAL_PEAK_GBS, 4),
                     "tokens_per_s": round(res["tokens"] / (ms * 1e-3), 1), "gpu_launches": res["launches"],
                     "us_per_launch": round(ms * 1e3 / max(res["launches"], 1), 2), "clocks": clocks.summary}
            if "extra" in res:
                entry["extra"] = res["extra"]
            status = backend.read_status(device)
            if status:
                entry["device_status"] = status
        except Exception as exc:  # noqa: BLE001 - a leg that cannot run must not take the headline with it
            entry = {"error": f"{type(exc).__name__}: {str(exc)[:200]}"}
        out[name] = entry
        gc.collect()                       # the workload's cache sits in reference cycles of its closures
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------
# the CPU arm: the oracle's port of the reference's CPU path
# ---------------------------------------------------------------------------
def cpu_baseline(budget_s: float = 15.0, want_native: bool = True, steps_max: int = 2000, warmup: int = 1):
    """Time the reference's CPU algorithm (per-token strided assignment loop for append,
    flattened view + ``.contiguous()`` for gather) on ONE layer of the workload, all 64
    sequences at their prompt lengths, for whole decode steps until ``budget_s`` is used.

    The layer class is the reference's own ``BarqPagedKVCacheLayer`` when its byte-compiled CPU path is at
    hand (``oracle/ref_python.py`` -> ``oracle/_ref``; ``kind: "reference"``), else the oracle's restatement
    of it (``kind: "port"``).  Only the class's public methods are used, so both run the same script."""
    from oracle import ref_python

    kind, layer_cls = "port", None
    try:
        module = ref_python.load()
        if module is not None:
            kind, layer_cls = "reference", module.BarqPagedKVCacheLayer
    except Exception:  # noqa: BLE001 - e.g. bytecode of another Python version: the port runs instead
        layer_cls = None
    if layer_cls is None:
        from oracle.paged_kv_oracle import OracleLayer as layer_cls

    torch.set_num_threads(os.cpu_count() or 1)
    g, prompts = seeded_lengths()
    H, D, ps, B = CFG["kv_heads"], CFG["head_dim"], CFG["page_size"], CFG["batch"]
    dtype = torch.bfloat16
    layers = []
    for n in prompts:                                   # set-up (untimed): caches already holding the prompts
        lay = layer_cls(1, -(-(n + steps_max + warmup + 1) // ps) * ps, ps)
        prompt = torch.randn(1, H, n, D, generator=g).to(dtype)
        lay.append(prompt, prompt)
        layers.append(lay)
    k_new = torch.randn(B, 1, H, 1, D, generator=g).to(dtype)
    per_tok = 4 * H * D * 2

    def one_step():
        for b, lay in enumerate(layers):
            lay.append(k_new[b], k_new[b])
        for lay in layers:
            ks, vs = lay.current_tensors()
            ks.contiguous()
            vs.contiguous()

    for _ in range(warmup):
        one_step()
    steps, moved = 0, 0
    t0 = time.perf_counter()
    while True:
        one_step()
        steps += 1
        moved += (B + sum(lay.get_seq_length() for lay in layers)) * per_tok
        if time.perf_counter() - t0 > budget_s or steps >= steps_max:
            break
    dt = time.perf_counter() - t0
    out = {"value": round(moved / dt / 1e9, 3), "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
           "host_cpus": os.cpu_count(), "steps": steps, "ms_per_step": round(dt * 1e3 / steps, 3),
           "what": ("the reference's own BarqPagedKVCacheLayer (python/barqtrain/kv_cache.py), CPU path, byte-compiled "
                    "from its checkout" if kind == "reference" else "the oracle's restatement of the reference's CPU path"),
           "sample": f"1 of {CFG['layers']} layers, all {B} sequences, {steps} decode steps "
                     f"(append loop + view.contiguous() gather), {dt:.1f} s; GB/s is per-layer work / time, "
                     f"so it compares directly with the GPU figure",
           "decode_tokens_per_s": round(B * steps / dt / CFG["layers"], 2)}
    if want_native:
        try:
            out["native_c_openmp"] = cpu_baseline_native(prompts, budget_s=min(5.0, budget_s))
        except Exception as exc:  # noqa: BLE001
            out["native_c_openmp"] = {"unavailable": str(exc)[:120]}
    return out


def cpu_baseline_native(prompts, budget_s: float = 5.0):
    """The same layer-sample through the C/OpenMP restatement with a shuffled block table."""
    from oracle import c_oracle

    H, D, ps, B = CFG["kv_heads"], CFG["head_dim"], CFG["page_size"], CFG["batch"]
    g = torch.Generator().manual_seed(1)
    lens = list(prompts)
    blocks = [-(-(n + 64) // ps) for n in lens]
    P = sum(blocks)
    perm = torch.randperm(P, generator=g).to(torch.int32)
    table = torch.full((B, max(blocks)), -1, dtype=torch.int32)
    at = 0
    for b, nb in enumerate(blocks):
        table[b, :nb] = perm[at:at + nb]
        at += nb
    k_pool = torch.zeros(H, P, ps, D, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    k_new = torch.randn(B, H, D, generator=g).to(torch.bfloat16)
    cu_new = torch.arange(B + 1, dtype=torch.int32)
    total_cap = sum(lens) + 64 * B
    k_out = torch.empty(total_cap, H, D, dtype=torch.bfloat16)
    v_out = torch.empty_like(k_out)
    per_tok = 4 * H * D * 2
    steps, moved = 0, 0
    t0 = time.perf_counter()
    while steps < 60:
        start = torch.tensor(lens, dtype=torch.int32)
        c_oracle.append_paged(k_pool, v_pool, table, None, start, cu_new, k_new, k_new)
        lens = [n + 1 for n in lens]
        lt = torch.tensor(lens, dtype=torch.int32)
        cu = torch.zeros(B, dtype=torch.int32)
        cu[1:] = torch.cumsum(lt, 0)[:-1]
        total = sum(lens)
        # head-major output [H, total, D] addressed as [token, head, dim]
        ko = k_out.view(-1)[: H * total * D].view(H, total, D).transpose(0, 1)
        vo = v_out.view(-1)[: H * total * D].view(H, total, D).transpose(0, 1)
        c_oracle.gather_paged(k_pool, v_pool, table, None, lt, cu, ko, vo)
        steps += 1
        moved += (B + total) * per_tok
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return {"value": round(moved / dt / 1e9, 3), "unit": UNIT, "cores": c_oracle.threads(), "steps": steps}


# ---------------------------------------------------------------------------
# single-kernel cases (the commands the ncu summaries under profiles/ were made with)
# ---------------------------------------------------------------------------
def run_micro_legacy(args):
    """The reference's native entry point on the reference's own cache layout, one layer:
    ``paged_kv_append_(key_cache[B,H,blocks,ps,D], value_cache, seq_lens, key_states[B,H,T,D], value_states)``.
    ``--impl barqkv`` times libbarqkv's implementation of it, ``--impl reference`` the reference's own CUDA
    kernel (built from a reference checkout into ``oracle/_ref`` by ``oracle/ref_cuda.py``)."""
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if args.impl == "reference":
        from oracle import ref_cuda

        module = ref_cuda.load()
        if module is None:
            print(json.dumps({"micro": "append-legacy", "impl": "reference",
                              "unavailable": "oracle/_ref holds no build of the reference kernel"}))
            return
        call = module.paged_kv_append_
    else:
        from barqtrain_b200 import _ffi

        call = _ffi.require_cuda_backend().paged_kv_append_
    H, D, ps, dtype = args.heads, CFG["head_dim"], args.page_size, torch.float16
    gen = torch.Generator(device=device).manual_seed(7)
    cases = {"prefill": (16, args.chunk, 4 * args.chunk), "decode": (CFG["batch"], 1, 4096)}
    out = {"micro": "append-legacy", "impl": args.impl, "heads": H, "page_size": ps, "dtype": "fp16", "cases": {}}
    for name, (B, T, capacity) in cases.items():
        blocks = capacity // ps
        keys = torch.zeros(B, H, blocks, ps, D, dtype=dtype, device=device)
        values = torch.zeros_like(keys)
        seq_lens = torch.zeros(B, dtype=torch.int32, device=device)
        k = torch.randn(B, H, T, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
        v = torch.randn(B, H, T, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
        per_round = min(capacity // T, 64)            # calls before the lengths are reset
        samples = []
        for it in range(args.warmup + args.steps):
            seq_lens.zero_()
            torch.cuda.synchronize(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(per_round):
                call(keys, values, seq_lens, k, v)
            e1.record()
            torch.cuda.synchronize(device)
            if it >= args.warmup:
                samples.append(e0.elapsed_time(e1) * 1e3 / per_round)
        us = statistics.median(samples)
        nbytes = 4 * B * T * H * D * 2
        out["cases"][name] = {"batch": B, "tokens_per_sequence": T, "calls_per_sample": per_round,
                              "us_per_call": round(us, 2), "bytes_per_call": nbytes,
                              "gbs": round(nbytes / us / 1e3, 1)}
        if args.impl != "reference":
            # the drop-in cache layer mirrors the lengths on the host, so its calls carry the largest
            # length with them and never read the device
            samples = []
            for it in range(args.warmup + args.steps):
                seq_lens.zero_()
                torch.cuda.synchronize(device)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(per_round):
                    call(keys, values, seq_lens, k, v, max_start=i * T)
                e1.record()
                torch.cuda.synchronize(device)
                if it >= args.warmup:
                    samples.append(e0.elapsed_time(e1) * 1e3 / per_round)
            us = statistics.median(samples)
            out["cases"][name]["host_mirrored_lengths"] = {"us_per_call": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)}
    print(json.dumps(out))


def run_micro(args):
    """One kernel alone on a small case of the workload's shape: per-launch CUDA-event times."""
    from barqtrain_b200 import BlockTableKVCache, _ffi

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    backend = _ffi.require_cuda_backend()
    if args.tune:
        backend.set_tuning(**{k: int(v) for k, v in (kv.split("=") for kv in args.tune.split(","))})
    H, D, ps = args.heads, CFG["head_dim"], args.page_size
    dtype = torch.bfloat16
    gen = torch.Generator(device=device).manual_seed(7)
    g = torch.Generator().manual_seed(CFG["seed"])
    if args.micro in ("gather", "update", "update-layers", "attention", "decode-update"):
        if args.lengths == "loguniform":          # the 70B-shaped gather configuration: 32 sequences in [1k, 32k]
            import math
            u = torch.rand(32, generator=g, dtype=torch.float64)
            lens = [int(round(math.exp(math.log(1024) + float(x) * (math.log(32768) - math.log(1024))))) for x in u]
        else:
            lens = torch.randint(CFG["prompt_lo"], CFG["prompt_hi"] + 1, (CFG["batch"],), generator=g).tolist()
    elif args.micro == "append-prefill":
        lens = [args.chunk * 4] * 16
    else:
        lens = [1024] * CFG["batch"]
    B = len(lens)
    pages = sum(-(-(n + 64) // ps) for n in lens)
    cache = BlockTableKVCache(1, H, D, page_size=ps, num_pages=pages, max_seqs=B,
                              max_blocks_per_seq=-(-(max(lens) + 64) // ps), dtype=dtype, device=device,
                              free_order=torch.randperm(pages, generator=g).tolist(), zero_pages=False)
    slots = [cache.open(i) for i in range(B)]
    per_tok = 4 * H * D * 2
    times, nbytes = [], 0

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        return e0, e1

    # Each case prepares its batch description on the stream it will launch on and returns
    # (launch function, launches per call, algorithmic bytes per call).
    def prepare():
        if args.micro == "gather":
            total = sum(lens)
            if cache.lengths[slots[0]] == 0:
                k = torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
                cache.append_step(slots, lens, [k], [k])
            gb = cache.begin_gather(slots)
            shape = (H, total, D) if args.layout == "HND" else (total, H, D)
            out = (torch.empty(shape, dtype=dtype, device=device), torch.empty(shape, dtype=dtype, device=device))

            def launch():
                for _ in range(args.reps):
                    cache.gather(0, gb, args.layout, out=out, mode=args.mode)
            if args.impl == "torch":
                # Comparison point, not a product path: the same pages collected by torch's index_select
                # (whole pages, so the rows past a sequence's end in its last page travel too; the bytes
                # counted are those pages').
                ids = torch.tensor([p for s_ in slots for p in cache.pages_of[s_]], dtype=torch.int64, device=device)
                k_pool, v_pool = cache.pools[0, 0], cache.pools[0, 1]                  # [H, P, ps, D]
                outs = (torch.empty(H, ids.numel(), ps, D, dtype=dtype, device=device),
                        torch.empty(H, ids.numel(), ps, D, dtype=dtype, device=device))

                def launch_torch():
                    for _ in range(args.reps):
                        torch.index_select(k_pool, 1, ids, out=outs[0])
                        torch.index_select(v_pool, 1, ids, out=outs[1])
                return launch_torch, 2 * args.reps, ids.numel() * ps * per_tok * args.reps
            return launch, args.reps, total * per_tok * args.reps
        if args.micro == "update":
            total = sum(lens)
            k = torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            if cache.lengths[slots[0]] == 0:
                cache.append_step(slots, lens, [k], [k])
            new = cache.begin_append(slots, [1] * B)     # every launch re-appends the same token: same work each time
            cache.end_append(new)
            full = cache.begin_gather(slots)
            shape = (H, full.total, D) if args.layout == "HND" else (full.total, H, D)
            out = (torch.empty(shape, dtype=dtype, device=device), torch.empty(shape, dtype=dtype, device=device))
            k1 = k[:B].contiguous()

            def launch():
                for _ in range(args.reps):
                    cache.update(0, new, full, k1, k1, args.layout, out=out, mode=args.mode)
            return launch, args.reps, (full.total + B) * per_tok * args.reps
        if args.micro == "update-layers":
            # the decode step's launches: `layers` fused append + gather kernels issued by one native call
            many = BlockTableKVCache(args.layers, H, D, page_size=ps, num_pages=pages, max_seqs=B,
                                     max_blocks_per_seq=-(-(max(lens) + 64) // ps), dtype=dtype, device=device,
                                     free_order=torch.randperm(pages, generator=g).tolist(), zero_pages=False)
            mslots = [many.open(i) for i in range(B)]
            fill = many.begin_append(mslots, lens)          # lengths only: the pools' contents do not matter for timing
            many.end_append(fill)
            new = many.begin_append(mslots, [1] * B)
            many.end_append(new)
            full = many.begin_gather(mslots)
            outs = [(torch.empty(H, full.total, D, dtype=dtype, device=device),
                     torch.empty(H, full.total, D, dtype=dtype, device=device)) for _ in range(2)]
            k_all = torch.randn(args.layers, B, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)

            def launch():
                for _ in range(args.reps):
                    many.update_layers(new, full, k_all, k_all, outs, "HND", mode=args.mode)
            return launch, args.layers * args.reps, (full.total + B) * per_tok * args.layers * args.reps
        if args.micro == "decode-update":
            # a decode layer in one call: the step's rows stored and attended by the same kernel
            total = sum(lens)
            k = torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            if cache.lengths[slots[0]] == 0:
                cache.append_step(slots, lens, [k], [k])
            new = cache.begin_append(slots, [1] * B)     # every launch stores the same token again: same work each time
            cache.end_append(new)
            full = cache.begin_gather(slots)
            q = torch.randn(B, H * args.group, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            out = torch.empty_like(q)
            k1 = k[:B].contiguous()
            cache.decode_update(0, full, k1, k1, q, out=out)       # sizes the workspace outside any capture

            def launch():
                for _ in range(args.reps):
                    cache.decode_update(0, full, k1, k1, q, out=out)
            return launch, args.reps, (full.total * 2 + 4 * B) * H * D * 2 * args.reps
        if args.micro == "attention":
            total = sum(lens)
            k = torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            if cache.lengths[slots[0]] == 0:
                cache.append_step(slots, lens, [k], [k])
            full = cache.begin_gather(slots)
            q = torch.randn(B, H * args.group, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            out = torch.empty_like(q)
            cache.decode_attention(0, full, q, out=out)            # sizes the workspace outside any capture

            def launch():
                for _ in range(args.reps):
                    cache.decode_attention(0, full, q, out=out)
            # K and V are read once: 2 * tokens * H * D * e bytes (q and out are negligible)
            return launch, args.reps, total * 2 * H * D * 2 * args.reps
        if args.micro == "append-prefill":
            total = args.chunk * B
            # four source sets taken in turn, so that consecutive launches read different memory (1 GB at 8 heads)
            srcs = [(torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype),
                     torch.randn(total, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype))
                    for _ in range(4)]
            if args.src_head_major:           # head-major sources: rows of a head adjacent in memory
                srcs = [(k.transpose(0, 1).contiguous().transpose(0, 1), v.transpose(0, 1).contiguous().transpose(0, 1))
                        for k, v in srcs]
            batch = cache.begin_append(slots, [args.chunk] * B)   # the same chunk lands on the same pages every launch

            def launch():
                for i in range(args.reps):
                    cache.append(0, batch, *srcs[i & 3])
            return launch, args.reps, total * per_tok * args.reps
        if args.micro == "append-layers":
            # one decode token per sequence for `layers` layers in ONE launch (pools of all layers are one tensor)
            many = BlockTableKVCache(args.layers, H, D, page_size=ps, num_pages=sum(-(-(n + 64) // ps) for n in lens),
                                     max_seqs=B, max_blocks_per_seq=-(-(max(lens) + 64) // ps), dtype=dtype,
                                     device=device, seed=5, zero_pages=False)
            mslots = [many.open(i) for i in range(B)]
            fill = many.begin_append(mslots, lens)          # lengths only: the decode rows land after them
            many.end_append(fill)
            k_all = torch.randn(args.layers, B, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
            batch = many.begin_append(mslots, [1] * B)

            def launch():
                for _ in range(args.reps):
                    many.append_layers(batch, k_all, k_all)
            return launch, args.reps, B * per_tok * args.layers * args.reps
        # append-decode: `layers` back-to-back single-token appends form one timed group
        k = torch.randn(B, H, D, generator=gen, device=device, dtype=torch.float32).to(dtype)
        if cache.lengths[slots[0]] == 0:
            fill = k.repeat(1024, 1, 1)[: sum(lens)]
            cache.append_step(slots, lens, [fill], [fill])
        batch = cache.begin_append(slots, [1] * B)

        def launch():
            for _ in range(args.layers):
                cache.append(0, batch, k, k)
        return launch, args.layers, B * per_tok * args.layers

    if args.graph:
        # the launches recorded into a CUDA graph: what the kernels take back to back, without host call overhead
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            launch, reps, nbytes = prepare()
            for _ in range(max(args.warmup, 1)):
                launch()
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            counted = backend.launches
            with torch.cuda.graph(graph, stream=side):
                launch()
            kernels = backend.launches - counted
            graph.replay()
            torch.cuda.synchronize(device)
            evs = [timed(graph.replay) for _ in range(args.steps)]
    else:
        launch, reps, nbytes = prepare()
        for _ in range(args.warmup):
            launch()
        torch.cuda.synchronize(device)
        counted = backend.launches
        evs = [timed(launch) for _ in range(args.steps)]
        kernels = (backend.launches - counted) // max(args.steps, 1)
    args.warmup = 0
    torch.cuda.synchronize(device)
    times = sorted(e0.elapsed_time(e1) * 1e-3 for e0, e1 in evs[args.warmup:])
    med = times[len(times) // 2]
    peak, kind = measured_peak()
    status = backend.read_status(device)
    # `launches_per_sample` counts calls of the library; `kernels_per_sample` what they enqueued (a decode
    # attention call is two kernels when sequences are split; --impl torch / reference are not counted)
    print(json.dumps({"micro": args.micro, "impl": args.impl, "tune": args.tune, "graph": bool(args.graph), "launches_per_sample": reps,
                      "kernels_per_sample": kernels,
                      "us_per_launch": round(med * 1e6 / reps, 2), "mode": args.mode, "layout": args.layout, "heads": H, "page_size": ps,
                      "sequences": B, "tokens": sum(lens) if args.micro == "gather" else None,
                      "bytes_per_launch": nbytes, "us_median": round(med * 1e6, 2), "us_min": round(times[0] * 1e6, 2),
                      "gbs_median": round(nbytes / med / 1e9, 1), "gbs_best": round(nbytes / times[0] / 1e9, 1),
                      "frac_of_%s_peak" % kind: round(nbytes / med / 1e9 / peak, 4), "status": status}), flush=True)


# ---------------------------------------------------------------------------
# the other configurations (chunked prefill, 70B-shaped gather, continuous-batching churn)
# ---------------------------------------------------------------------------
def run_extra(args):
    import torch.distributed as dist

    from barqtrain_b200 import _ffi
    from barqtrain_b200.benchmarks.workloads import WORKLOADS

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        init_nccl(dist, device)
    backend = _ffi.require_cuda_backend()
    if args.tune:
        backend.set_tuning(**{k: int(v) for k, v in (kv.split("=") for kv in args.tune.split(","))})

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    kwargs = {"page_size": args.page_size, "all_layers": args.all_layers,
              "calls_per_layer": args.eager} if args.workload == "prefill" else {}
    if args.workload == "gather70b":
        kwargs["all_layers"] = args.all_layers
        kwargs["calls_per_layer"] = args.eager
    if args.workload == "decode-attn":
        kwargs["eager"] = args.eager
    if args.workload == "churn":
        kwargs["attend"] = args.attend
    if args.layers_override:
        kwargs["layers"] = args.layers_override
    if args.shard_heads:
        kwargs["heads"] = args.shard_heads
    with ClockSampler(local) as clocks:
        res = WORKLOADS[args.workload](world, rank, device, args.steps, max(args.warmup, 3), sync=barrier, **kwargs)
    ms = res["ms"]
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    peak, kind = measured_peak()
    value = res["bytes"] * world / (ms * 1e-3) / 1e9
    line = {"metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": res["config"]["dtype"], "data": "synthetic",
            "config": dict(res["config"], sharding=f"kv-head x{world}"),
            "pct_of_nominal_8TBs": round(100 * value / world / NOMINAL_PEAK_GBS, 2),
            "pct_of_%s_copy" % kind: round(100 * value / world / peak, 2),
            "tokens_per_s": round(res["tokens"] / (ms * 1e-3), 1),
            "us_per_launch": round(ms * 1e3 / max(res["launches"], 1), 2),
            "gpu_launches": res["launches"], "clocks": clocks.summary}
    if "extra" in res:
        line["extra"] = res["extra"]
    status = backend.read_status(device)
    if status:
        raise SystemExit(f"device guard fired: status {status}")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_generate(args):
    """The reference's generation benchmark method (notebook cell 3: warm-up, resident snapshot with the peak
    reset, measured runs, peak snapshot, overhead) on a seeded random-weight Llama, for the stock dynamic
    cache, the drop-in paged cache and the block-table cache gathered and from the pages."""
    from barqtrain_b200.benchmarks import inference

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    layers = args.layers_override or 16
    rows = inference.run_table(device=device, batch=args.gen_batch, layers=layers)
    print(json.dumps({"workload": "generate", "model": f"seeded random-weight Llama: {layers} layers, hidden 1024, 8 query / 2 KV "
                      "heads of 128, vocabulary 32000, bf16", "batch": args.gen_batch,
                      "method": "warm-up runs, cuda_memory_snapshot(reset_peak=True), measured runs, peak snapshot; "
                                "generation_overhead_mb = peak max_allocated - resident allocated",
                      "rows": rows}), flush=True)


def decode_config(world: int) -> dict:
    """The workload of the default run, in the same words on both arms' lines."""
    return {"workload": CFG["name"], "layers": CFG["layers"], "kv_heads": CFG["kv_heads"], "head_dim": CFG["head_dim"],
            "page_size": CFG["page_size"], "batch": CFG["batch"], "prompt_lengths": "uniform[512,4096] seeded",
            "sharding": f"kv-head x{world}",
            "step": "per layer: append 1 token/seq, gather all sequences to [H,sum_len,D]",
            "l2": "inputs larger than L2: a step reads every layer's pages of all sequences once (~21 GB over 32 layers "
                  "at 8 KV heads)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    K, W = args.steps, args.warmup
    base = cpu_baseline(budget_s=max(args.cpu_seconds, 30.0), steps_max=K, warmup=W)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": base["steps"], "warmup": W, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": decode_config(args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's CPU PyTorch path (_python_append + current_tensors().contiguous(); see cpu_baseline.kind "
                "and .what) on the host cores; each step is a bounded sample (one layer) of the workload",
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="barqkv", choices=["barqkv", "reference", "torch"],
                    help="reference: the reference's CPU path (default run) or CUDA kernel (--micro append-legacy); "
                         "torch: --micro gather with torch.index_select over the pages, for comparison")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="repeat the timed K-step region until this much device time has been measured")
    ap.add_argument("--gen-batch", type=int, default=1, help="--workload generate: sequences per generate() call")
    ap.add_argument("--attend", action="store_true",
                    help="--workload churn: every decode step also attends over the pages (graph of fused launches)")
    ap.add_argument("--no-legs", action="store_true", help="skip the short legs of the other configurations")
    ap.add_argument("--quick-legs", action="store_true", help="legs with fewer layers and steps (smoke runs)")
    ap.add_argument("--eager", action="store_true",
                    help="call update() per layer from Python every step instead of replaying a CUDA graph")
    ap.add_argument("--two-launches", action="store_true",
                    help="per layer call append() then gather() instead of the single update() launch")
    ap.add_argument("--micro", choices=["gather", "update", "update-layers", "attention", "decode-update", "append-prefill", "append-decode", "append-layers", "append-legacy"],
                    help="time one kernel alone on a one-layer case instead of the full step")
    ap.add_argument("--mode", default="auto", choices=["auto", "vector", "bulk"])
    ap.add_argument("--layout", default="HND", choices=["HND", "NHD"])
    ap.add_argument("--src-head-major", action="store_true",
                    help="micro append-prefill: new rows laid out [H, tokens, D] instead of [tokens, H, D]")
    ap.add_argument("--heads", type=int, default=8, help="KV heads on this GPU (micro cases)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--chunk", type=int, default=2048, help="tokens per sequence per append (append-prefill)")
    ap.add_argument("--layers", type=int, default=32, help="appends per timed group (append-decode)")
    ap.add_argument("--lengths", default="uniform", choices=["uniform", "loguniform"])
    ap.add_argument("--group", type=int, default=4, help="micro attention: query heads per KV head")
    ap.add_argument("--reps", type=int, default=1, help="micro gather/append-prefill: launches per timed sample")
    ap.add_argument("--graph", action="store_true", help="micro cases: time a CUDA-graph replay of the launches")
    ap.add_argument("--tune", default="", help="gather knobs, e.g. stages=8,ctas=3,interleave=1 (micro cases)")
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "prefill", "gather70b", "churn", "decode-attn", "generate"],
                    help="decode = the headline configuration; the others print the same line for their configuration")
    ap.add_argument("--all-layers", action="store_true",
                    help="--workload prefill / gather70b: all layers with one launch (all layers' rows / outputs at hand)")
    ap.add_argument("--shard-heads", type=int, default=0,
                    help="--workload: KV heads on this GPU instead of 8/N (1 = an 8-GPU shard's work on one GPU)")
    ap.add_argument("--layers-override", type=int, default=0, help="fewer layers for a quick run of --workload")
    args = ap.parse_args()
    if args.workload == "generate":
        run_generate(args)
    elif args.micro == "append-legacy":
        run_micro_legacy(args)
    elif args.micro:
        run_micro(args)
    elif args.workload != "decode" and args.impl != "reference":
        run_extra(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_barqkv(args)


if __name__ == "__main__":
    main()
