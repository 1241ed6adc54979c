"""Benchmark of the DSA sparse-attention forward (indexer + top-k + attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--tokens T]
    python bench.py --workload {dsa_variants,block_sparse,nsa,encoder,static,static2d}     # other configurations

Workload ("dsa_fwd_64k"): one DSA attention layer, 65536 tokens, 8 heads x 64,
4 x 64 indexer, top-2048, bf16, batch 1, non-causal; seeded synthetic inputs with
the shapes and distributions of the reference's Virchow2 feature bags (q, k, v ~
N(0,1), q scaled by 1/8; indexer q/k ~ N(0, 1/64); W ~ N(0,1)).  One step = one
forward over the whole slide.  With N > 1 (torchrun, one rank per GPU) the slide
is sequence-sharded: total work is fixed ("strong" scaling), every step
all-gathers the indexer keys, K and V over NCCL.

Prints ONE JSON line (rank 0).  `value` is whole-job tokens/s with inputs resident
in HBM; `e2e` is the same through the public API with inputs in pinned host
memory and the output read back, copies inside the timed region.
"""
import argparse
import datetime
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, D, IH, ID, TOP_K = 8, 64, 4, 64, 2048
METRIC = "dsa_sparse_attn_fwd_tokens_per_s"
# kernels of this library launched per forward on one GPU: 2 head collapses; the selection -- for a
# sparse top-k on a long key range estimate, collect, select and 5 launches of the exact passes that
# return at once unless a query tile was flagged (8), otherwise 6 radix-select tile passes (4 of them
# returning at once unless flagged) and emit (7); valid fill; key-norm maximum; attention.  When the
# selection is sparse enough for the list-driven attention kernel: + the tile-list build and the launch
# of the dense sweep for flagged tiles (returns at once unless a tile was flagged).  The sharded step
# launches the same on every rank.
def kernels_per_step(T):
    from sparse_wsi_vit_b200 import ops
    k_eff = min(TOP_K, T)
    # the library sizes a larger workspace exactly where it takes the two-sweep form of the selection
    two_sweep = ops.workspace_bytes(1, T, T, TOP_K) > ops.workspace_bytes(1, T, T)
    lists = TOP_K % 4 == 0 and k_eff <= ops.LISTS_MAX_DENSITY * T
    return 2 + (8 if two_sweep else 7) + 1 + (4 if lists else 2)


def uses_list_kernel(T):
    from sparse_wsi_vit_b200 import ops
    return TOP_K % 4 == 0 and min(TOP_K, T) <= ops.LISTS_MAX_DENSITY * T

# DRAM bytes (read + write) of one dsa_attn_masked_kernel launch, from one-pass ncu captures
# (dram__bytes_read.sum + dram__bytes_write.sum): 3.15 GB + 0.07 GB on the 65536-token workload -- K, V
# of all heads and the indexer keys, 144 MiB, do not fit the 126 MB L2, so key tiles are re-fetched;
# 62.7 MB + 64.8 MB at 16384 tokens, where they fit.  A profiler figure cannot be taken inside a timed
# run, so the JSON line carries it with `traffic_source` saying so.
ATTN_DRAM_BYTES_PER_LAUNCH = {65536: 3.225e9, 16384: 127.5e6}
# the same for dsa_attn_lists_kernel (65536 tokens; it also reads the 1.6 GB of tile lists once per head pair)
ATTN_LISTS_DRAM_BYTES_PER_LAUNCH = {65536: 4.12e9}


def workload_config(T, world):
    """The `config` object of the JSON line; both arms print exactly this."""
    return {"workload": f"dsa_fwd_{T // 1024}k", "tokens": T, "heads": H, "head_dim": D,
            "indexer": f"{IH}x{ID} tf32", "top_k": TOP_K, "batch": 1,
            "parallelism": f"sp{world}" if world > 1 else "single",
            "l2": "inputs+outputs per step (>1.9 GiB) exceed the 126 MB L2"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p.get("bf16_tflops_sustained", 1411.6), p.get("hbm_gbs", 6453.1), "measured"
    return 1400.0, 6650.0, "fallback"


def make_inputs(T, seed, device, pinned=False):
    """Token-major tensors (1, T, H, D) / (1, T, IH, ID), bf16, seeded on the CPU."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(1, T, H, D, generator=g) / D ** 0.5).to(torch.bfloat16)
    k = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16)
    qi = (torch.randn(1, T, IH, ID, generator=g) / ID ** 0.5).to(torch.bfloat16)
    ki = (torch.randn(1, T, IH, ID, generator=g) / ID ** 0.5).to(torch.bfloat16)
    w = torch.randn(IH, generator=g)
    ts = [q, k, v, qi, ki]
    if pinned:
        ts = [t.pin_memory() for t in ts]
    elif device is not None:
        ts = [t.to(device) for t in ts]
    return (*ts, w.to(device) if device is not None else w)


class ClockSampler:
    """nvidia-smi polling every 100 ms in a child process.  It is started before the warm-up steps
    (its start-up takes longer than a short timed region) and every sample carries its time stamp;
    `stop()` keeps the samples between `begin()` and `end()`."""
    QUERY = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    MIN_WINDOW_S = 1.0

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def begin(self):
        self.t_begin = datetime.datetime.now()

    def end(self):
        self.t_end = datetime.datetime.now()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []                                  # (inside the window?, sm, max sm, reasons)
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 10:
                        continue
                    try:
                        vals = (float(c[2]), float(c[3]))
                    except ValueError:
                        continue
                    try:
                        ts = datetime.datetime.strptime(c[0], "%Y/%m/%d %H:%M:%S.%f")
                        inside = self.t_begin is None or self.t_begin <= ts <= (self.t_end or ts)
                    except ValueError:
                        inside = False
                    rows.append((inside, *vals, [name for name, val in zip(
                        ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[6:10])
                        if val.lower().startswith("active")]))
            os.unlink(self.path)
        except Exception:
            pass
        kept = [r for r in rows if r[0]]
        if not kept and rows and self.t_begin is not None and self.t_end is not None:
            # time stamps unreadable or in another zone: the last samples cover the window, which
            # ended just before the sampler was stopped
            n = max(1, int((self.t_end - self.t_begin).total_seconds() / 0.1))
            kept = rows[-n:]
        sm = [r[1] for r in kept]
        mx = [r[2] for r in kept]
        reasons = {name for r in kept for name in r[3]}
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


# ----------------------------------------------------------------- CPU baseline
_CPU_INPUTS = {}


def cpu_baseline(T, budget_s=15.0, threads=None):
    """The CPU oracle (a port of the reference's arithmetic) on a bounded sample of the same
    workload: `rows` query rows against all T keys, all heads.  Returns tokens/s."""
    from oracle import dsa as O
    if threads:
        torch.set_num_threads(threads)
    if T not in _CPU_INPUTS:
        q, k, v, qi, ki, w = make_inputs(T, seed=0, device=None)
        q, k, v = (t[0].transpose(0, 1).float() for t in (q, k, v))        # (H, T, D)
        _CPU_INPUTS[T] = (q, k, v, qi[0].float(), ki[0].float(), w)
    q, k, v, qi, ki, w = _CPU_INPUTS[T]

    def run(rows):
        t0 = time.perf_counter()
        wq = O.collapse_heads(qi[:rows], w)
        wk = O.collapse_heads(ki, w)
        s = torch.relu(wq @ wk.T)
        idx, valid, sel = O.topk_lower_index(s, TOP_K)
        O.dsa_attention(q[:, :rows], k, v, idx, valid, sel * valid, chunk=64)
        return time.perf_counter() - t0

    rows = 32
    t = run(rows)
    target = max(rows, min(T, int(rows * budget_s / max(t, 1e-3))))
    target = max(32, min(target, 4096))
    if target > rows * 2:
        rows = target
        t = run(rows)
    return {"value": rows / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{rows} of {T} query rows against all {T} keys, {H} heads, fp32, {t:.1f} s"}


def triton_reference_baseline(src, T=1024, top_k=32):
    """The reference's OWN kernels (LightningIndexerFunction + DSAAttentionFunction of
    deepseek_sparse_attention_kernels/kernels.py) executed on CPU tensors by Triton's interpreter,
    from a checkout whose `src` directory is given.  The interpreter needs about a minute per
    forward at 1024 tokens and four times that per doubling, so this is a small-size figure beside
    the full-size port, at the same selection density (top_k / T = 1/32) and head shapes."""
    os.environ["TRITON_INTERPRET"] = "1"
    sys.path.insert(0, src)
    from sparse_wsi_vit.models.deepseek_sparse_attention_kernels import kernels as ref_kernels
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, H, T, D, generator=g) / D ** 0.5
    k = torch.randn(1, H, T, D, generator=g)
    v = torch.randn(1, H, T, D, generator=g)
    qi = torch.randn(1, T, IH, ID, generator=g) / ID ** 0.5
    ki = torch.randn(1, T, IH, ID, generator=g) / ID ** 0.5
    w = torch.randn(IH, generator=g)
    t0 = time.perf_counter()
    idx, valid, scores = ref_kernels.LightningIndexerFunction.apply(qi, ki, w, 1, T, IH, ID, top_k, 64, 64, 64, IH)
    o = torch.zeros(1, H, T, D)
    ref_kernels.DSAAttentionFunction.apply(q, k, v, idx, valid, scores * valid, o, 1, H, T, D, top_k, 64, 64, H, 64)
    dt = time.perf_counter() - t0
    return {"value": T / dt, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "reference",
            "sample": f"whole forward at {T} tokens, top-{top_k}, {H}x{D} heads, {IH}x{ID} indexer, fp32, Triton "
                      f"interpreter on CPU tensors, {dt:.1f} s"}


def run_reference(args):
    """`--impl reference`: the reference's forward arithmetic on the host cores.  The reference is
    Python + Triton (no compiled CPU library to build), and its kernels only run on a CPU under
    Triton's interpreter at toy sizes, so the full-size workload is timed with the CPU port in
    oracle/ (pinned to the reference by the golden fixtures).  One step = one bounded sample of the
    workload: `rows` query rows against all keys; `ms_per_step` is the time that sample took, the
    extrapolation to all rows is a separate field.  With --reference-src (or SWV_REFERENCE_SRC)
    pointing at the `src` directory of a checkout, the reference's own kernels are also timed, at
    1024 tokens, and reported in `triton_interpreter`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    T = args.tokens
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    per_step, per_step_s, base = [], [], None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        base = cpu_baseline(T, budget_s=4.0 if i >= args.warmup else 1.0, threads=threads)
        if i >= args.warmup:
            per_step.append(base["value"])
            per_step_s.append(time.perf_counter() - t0)
    value = statistics.mean(per_step)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(per_step_s),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(T, world),
        "step_is": "one bounded sample of the workload (see cpu_baseline.sample); value = sample rows / sample time",
        "extrapolated_ms_full_workload": 1e3 * T / value,
        "cpu_baseline": {**base, "value": value},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    src = args.reference_src or os.environ.get("SWV_REFERENCE_SRC")
    if src and os.path.isdir(src):
        try:
            line["triton_interpreter"] = triton_reference_baseline(src)
        except Exception as e:                                   # a checkout that does not import here
            line["triton_interpreter"] = {"skipped": f"{type(e).__name__}: {e}"[:200]}
    else:
        line["triton_interpreter"] = {"skipped": "no reference checkout given (--reference-src / SWV_REFERENCE_SRC)"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch.distributed as dist

    import sparse_wsi_vit_b200 as swv
    from sparse_wsi_vit_b200 import ops
    from sparse_wsi_vit_b200.dist import plan_shards, sharded_dsa_attention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T = args.tokens
    plan = plan_shards(T, world, rank, align=128)
    sl = slice(plan.start, plan.stop)

    host = make_inputs(T, seed=0, device=None)
    w = host[5].to(dev)
    pinned = [t[:, sl].contiguous().pin_memory() for t in host[:5]]
    q, k, v, qi, ki = (t.to(dev) for t in pinned)
    comm = torch.cuda.Stream(dev) if world > 1 else None
    cur = torch.cuda.current_stream(dev)

    ev_a = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ev_b = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    attn_events = []

    def step(qd, kd, vd, qid, kid, timed_idx=None, qkv_ready=None):
        if world == 1:
            B = 1
            qv, kv, vv = (t.transpose(1, 2) for t in (qd, kd, vd))
            idx, valid, scores, sel = ops.dsa_indexer_topk(qid, kid, w, TOP_K, want_mask=True)
            o = torch.empty((B, H, qd.shape[1], D), dtype=torch.bfloat16, device=dev)
            if qkv_ready is not None:
                cur.wait_event(qkv_ready)
            if timed_idx is not None:
                ev_a[timed_idx].record(cur)
            ops.dsa_attention_dense(qv, kv, vv, idx, scores, sel, o)
            if timed_idx is not None:
                ev_b[timed_idx].record(cur)
            return o, idx
        o, idx, valid, scores = sharded_dsa_attention(qd, kd, vd, qid, kid, w, TOP_K, plan, out_dtype=torch.bfloat16,
                                                      return_topk=True, comm_stream=comm)
        return o, idx

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step(q, k, v, qi, ki)
    ops.check_status(dev, "bench warm-up")

    # ---- device-resident timing
    barrier()
    sampler.begin()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record(cur)
    _h0 = time.perf_counter()
    for i in range(args.steps):
        step(q, k, v, qi, ki, timed_idx=i)
    _h1 = time.perf_counter()
    t1.record(cur)
    barrier()
    ms = t0.elapsed_time(t1) / args.steps
    # A timed region shorter than a few sampling periods gives the clock sampler nothing to read:
    # the same step keeps running, untimed, until the sampled window is MIN_WINDOW_S long (the
    # count comes from rank 0, so that every rank issues the same collectives).
    extra = torch.tensor([max(0, math.ceil((ClockSampler.MIN_WINDOW_S * 1e3 - ms * args.steps) / ms))], device=dev)
    if world > 1:
        dist.broadcast(extra, 0)
    for _ in range(int(extra.item())):
        step(q, k, v, qi, ki)
    barrier()
    sampler.end()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = (f"the {args.steps} timed steps" if int(extra.item()) == 0 else
                            f"the {args.steps} timed steps and {int(extra.item())} identical untimed steps after them")
    ops.check_status(dev, "bench timed region")

    # ---- end to end: pinned host inputs -> device, forward, output back to pinned host
    o_host = torch.empty((1, H, plan.local, D), dtype=torch.bfloat16).pin_memory()
    dbuf = [torch.empty_like(t, device=dev) for t in pinned]

    copy_stream = torch.cuda.Stream(dev)

    # A double-buffered pipeline, as a service that streams slides would run it.  The five input
    # tensors of step s + 1 are copied from pinned host memory (upload stream, second set of device
    # buffers) while step s computes; the output of step s goes back on the download stream while
    # step s + 1 computes.  Every step's uploads and download happen inside the timed region; the
    # first step's upload and the last step's download are not hidden.  On one GPU the step starts as
    # soon as the two indexer tensors are up (the attention waits for q, k, v); a sharded step
    # starts when all five are up, because its K/V all-gather is issued at once.
    up_stream = torch.cuda.Stream(dev)
    dbuf2 = [torch.empty_like(t) for t in dbuf]

    idx_host = torch.empty((1, plan.local, TOP_K), dtype=torch.int32).pin_memory()

    def e2e_pipeline(n, with_idx=False):
        sets = (dbuf, dbuf2)
        done = [None, None]                    # compute of the step that last read each buffer set
        outs = [None, None]                    # output of that step, kept until its download is ordered
        dl_done = [None, None]                 # ... and the download of it

        def upload(slot):
            with torch.cuda.stream(up_stream):
                if done[slot] is not None:
                    up_stream.wait_event(done[slot])
                sets[slot][3].copy_(pinned[3], non_blocking=True)
                sets[slot][4].copy_(pinned[4], non_blocking=True)
                ev_idx = up_stream.record_event()
                for i in range(3):
                    sets[slot][i].copy_(pinned[i], non_blocking=True)
                return ev_idx, up_stream.record_event()

        up_stream.wait_stream(cur)
        nxt = upload(0)
        for s_ in range(n):
            ev_idx, ev_qkv = nxt
            slot = s_ & 1
            if s_ + 1 < n:
                nxt = upload(slot ^ 1)
            # The output of two steps ago is released here, after this stream has been ordered behind
            # its download: the allocator hands the block to this step at once.  (Marking the output
            # as in use by the download stream instead would keep every block out of the pool until
            # the GPU catches up with the host, one device allocation per step.)
            if dl_done[slot] is not None:
                cur.wait_event(dl_done[slot])
                outs[slot] = None
            if world == 1:
                cur.wait_event(ev_idx)
                o, ix = step(*sets[slot], qkv_ready=ev_qkv)
            else:
                cur.wait_event(ev_qkv)
                o, ix = step(*sets[slot])
            done[slot] = cur.record_event()
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(done[slot])
                o_host.copy_(o, non_blocking=True)
                if with_idx:
                    idx_host.copy_(ix, non_blocking=True)
                dl_done[slot] = copy_stream.record_event()
            outs[slot] = (o, ix) if with_idx else o
            del o, ix
        cur.wait_stream(copy_stream)           # the last download belongs to the timed region
        cur.wait_stream(up_stream)

    e2e_pipeline(2)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(cur)
    _h2 = time.perf_counter()
    e2e_pipeline(args.steps)
    _h3 = time.perf_counter()
    e1.record(cur)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    # the same pipeline with the selected-key indices (the operator's second checked output) downloaded too
    barrier()
    e2 = torch.cuda.Event(enable_timing=True)
    e3 = torch.cuda.Event(enable_timing=True)
    e2.record(cur)
    e2e_pipeline(args.steps, with_idx=True)
    e3.record(cur)
    barrier()
    ms_e2e_idx = e2.elapsed_time(e3) / args.steps

    if world > 1:
        tt = torch.tensor([ms, ms_e2e, ms_e2e_idx], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e, ms_e2e_idx = float(tt[0]), float(tt[1]), float(tt[2])

    if rank == 0:
        tf_peak, hbm_peak, peak_src = measured_peaks()
        line = {
            "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(T, world),
            # host time rank 0 spends issuing one step (no waiting): far below ms_per_step = not launch-bound
            "host_issue_ms_per_step": (_h1 - _h0) * 1e3 / args.steps,
            "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "host_issue_ms_per_step": (_h3 - _h2) * 1e3 / args.steps,
                    "mode": "double-buffered uploads/downloads overlapped with the neighbouring steps",
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in pinned) * world,
                    "d2h_bytes_per_step": o_host.numel() * o_host.element_size() * world,
                    "outputs_downloaded": "the attention output o; idx / valid / scores stay on the device",
                    "with_idx": {"value": T / (ms_e2e_idx * 1e-3), "ms_per_step": ms_e2e_idx,
                                 "d2h_bytes_per_step": (o_host.numel() * o_host.element_size() +
                                                        idx_host.numel() * 4) * world,
                                 "outputs_downloaded": "o and the int32 index lists idx"}},
            "gpu_launches": args.steps * kernels_per_step(T) * world,
            "clocks": clocks,
        }
        if world == 1:
            attn_ms = statistics.mean(a.elapsed_time(b) for a, b in zip(ev_a, ev_b))
            lists = uses_list_kernel(T)
            kept = 4.0 * T * min(TOP_K, T) * H * D
            # dense tiles on the tensor cores: the sweep multiplies Q K^T and P V over all keys (+ the
            # routing-weight tiles); the list-driven kernel Q K^T and P [V | 1] with an 80-wide accumulator
            executed = (2.0 * D + 2.0 * 80) * T * T * H if lists else 4.0 * T * T * H * D
            ach = kept / (attn_ms * 1e-3) / 1e12
            line["roofline"] = {
                "kernel": ("dsa_attn_lists_kernel (timed with dsa_tile_lists_kernel and key_norm_max_kernel, which "
                           "it needs)" if lists else "dsa_attn_masked_kernel"),
                "bound": "tensor", "achieved": ach, "peak": tf_peak,
                "unit": "TFLOP/s", "frac": ach / tf_peak,
                "traffic": (ATTN_LISTS_DRAM_BYTES_PER_LAUNCH if lists else ATTN_DRAM_BYTES_PER_LAUNCH).get(T),
                "traffic_source": "one-pass ncu capture of this kernel on this workload, taken in a separate "
                                  "run (a constant of bench.py, not measured by this run)",
                "peak_source": f"bf16_tflops_sustained of {peak_src}",
                "kernel_ms": attn_ms, "algorithmic_flops": kept,
                "executed_flops": executed, "executed_tflops": executed / (attn_ms * 1e-3) / 1e12,
                "executed_frac": executed / (attn_ms * 1e-3) / 1e12 / tf_peak,
                "other_kernels_ms": ms - attn_ms,
            }
            if lists:
                # what bounds the list-driven kernel: the tensor pipe is occupied nearly all the time (24 MMA
                # instructions per (128 x 128 tile, head pair): 2 x 4 for Q K^T, 2 x 8 for P [V | 1]) although its
                # math units are active only ~40 % of it.  Those 24 instructions take 1634 cycles when nothing
                # else runs on the SM (micro-benchmark); the floor below is that figure over all tile pairs.
                tiles = (T / 128.0) ** 2 * (H / 2)
                line["roofline"]["mma_issue_floor_ms"] = tiles * 1634.0 / (148 * (clocks.get("sm_mhz") or 1965.0) * 1e6) * 1e3
                line["roofline"]["mma_issue_frac"] = line["roofline"]["mma_issue_floor_ms"] / attn_ms
            else:
                # what bounds the sweep: one exp per (query, key, head) on the 16 exp lanes per SM
                line["roofline"]["exp_unit_floor_ms"] = T * float(T) * H / (16.0 * 148 * (clocks.get("sm_mhz") or 1965.0) * 1e6) * 1e3
                line["roofline"]["exp_unit_frac"] = line["roofline"]["exp_unit_floor_ms"] / attn_ms
            line["cpu_baseline"] = cpu_baseline(T, budget_s=15.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="sequence length (default 65536; with --workload "
                    "block_sparse / nsa: run only this size)")
    ap.add_argument("--reference-src", default=None, help="with --impl reference: `src` directory of a "
                    "sparse-wsi-vit checkout; its own Triton kernels are then timed too (interpreter, 1024 tokens)")
    ap.add_argument("--top-k", type=int, default=None, help="keys per query of the dsa_fwd workload (default 2048; "
                    "e.g. --tokens 16384 --top-k 512 is a small case with the bench workload's one key in 32)")
    ap.add_argument("--workload", default="dsa_fwd", choices=["dsa_fwd", "dsa_variants", "dsa_backward", "block_sparse", "nsa", "encoder", "static", "static2d"])
    args = ap.parse_args()
    if args.top_k is not None:
        global TOP_K
        TOP_K = args.top_k
    if args.workload != "dsa_fwd":
        from sparse_wsi_vit_b200.benchmarks import WORKLOADS
        kw = {}
        if args.tokens is not None and args.workload in ("block_sparse", "dsa_variants", "dsa_backward"):
            kw["sizes"] = (args.tokens,)
        elif args.tokens is not None and args.workload in ("nsa", "static"):
            kw["tokens"] = args.tokens
        if args.workload == "static2d":
            # the CPU baseline of this workload: the oracle's fp32 restatement, timed on the host cores
            from oracle import encoder as E
            kw["cpu_forward"] = lambda sd, x, c, rp, ci: E.block2d_encoder_forward(sd, x, c, rp, ci, 64, 2, 6, 1, 64.0)
        WORKLOADS[args.workload](**kw)
        return
    if args.tokens is None:
        args.tokens = 65536
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
