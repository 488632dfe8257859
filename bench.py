"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg4|cfg5] [--impl ours|reference]

One step = one decoded token's worth of the path on one attention-layer pair:
a token-selection layer (full attention over the whole context + head-summed
fp32 logits + top-k) followed by a sparse layer over the selected positions.
Prints ONE JSON line (rank 0).  Under torchrun (N > 1) the KV cache is sharded by
sequence across the ranks and the step includes the two packed all-gathers.

Workloads (synthetic, seeded; shapes of the benchmark configurations):
    cfg2  B=1, 32 heads x 128 MHA fp16, context 32768, top_k 256, 64 planted keys   (default)
    cfg4  B=4, 32 q / 8 kv heads x 128 bf16, context 131072, top_k 128
    cfg5  B=8, 64 q / 8 kv heads x 128 bf16, context 1048576, top_k 1024 (needs >= 2 GPUs' memory at 1 layer pair: 64 GiB)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "cfg2": dict(B=1, Hq=32, Hkv=32, D=128, dtype="float16", N=32768, k=256, planted=64, layer_pairs=4),
    "cfg4": dict(B=4, Hq=32, Hkv=8, D=128, dtype="bfloat16", N=131072, k=128, planted=64, layer_pairs=2),
    "cfg5": dict(B=8, Hq=64, Hkv=8, D=128, dtype="bfloat16", N=1048576, k=1024, planted=10486, layer_pairs=1),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one selection-layer launch at one GPU, from the ncu captures
# summarised under profiles/ (cfg5 holds 64 GiB and is not captured; its traffic is left null)
NCU_TRAFFIC_BYTES = {"cfg2": 536.97e6 + 4.30e6, "cfg4": 2147.76e6 + 8.41e6}
METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown") else 0x8: "hw_slowdown",
            0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t is not None:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def synth_shard(w, lo, hi, seed, dtype, device):
    """K,V ~ N(0,1) for positions [lo,hi) of every sequence, written straight into a pool
    [B*(hi-lo), 2, 1, Hkv, D] on the device; planted keys are added by the caller."""
    B, Hkv, D = w["B"], w["Hkv"], w["D"]
    n = hi - lo
    g = torch.Generator(device=device).manual_seed(seed)
    pool = torch.empty(B * max(n, 1), 2, 1, Hkv, D, dtype=dtype, device=device)
    step = 1 << 16
    flat = pool.view(B * max(n, 1), -1)
    for s in range(0, flat.shape[0], step):
        e = min(flat.shape[0], s + step)
        flat[s:e] = torch.randn(e - s, flat.shape[1], generator=g, device=device, dtype=torch.float32).to(dtype)
    return pool


def plant(w, pool, q, lo, hi, seed):
    """Planted positions: K[p,h,:] = 3*q_h/|q_h| + N(0,0.1), positions from a seeded randperm."""
    B, Hq, Hkv, D, N = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"]
    G = Hq // Hkv
    g = torch.Generator().manual_seed(seed)
    for b in range(B):
        pos = torch.randperm(N, generator=g)[: w["planted"]]
        noise = 0.1 * torch.randn(w["planted"], Hkv, D, generator=g)
        mine = (pos >= lo) & (pos < hi)
        if not bool(mine.any()):
            continue
        qh = q[b, ::G].float().cpu()                                    # first q head of each KV head
        rows = 3.0 * qh / qh.norm(dim=-1, keepdim=True)                 # [Hkv, D]
        vals = (rows[None] + noise[mine]).to(pool.dtype).to(pool.device)
        idx = (b * (hi - lo) + (pos[mine] - lo)).to(pool.device)
        pool[idx, 0, 0] = vals


def run_ours(args, rank, world, device):
    import torch.distributed as dist

    import tidaldecode_b200.ops as T
    from tidaldecode_b200.sharded import ShardPlan, ShardedDecodeAttention

    w = WORKLOADS[args.workload]
    dtype = getattr(torch, w["dtype"])
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    es = 2
    plan = ShardPlan.contiguous(N, world)
    lo, hi = plan.range_of(rank)
    n_loc = hi - lo
    pairs = args.layer_pairs if args.layer_pairs > 0 else w["layer_pairs"]
    gq = torch.Generator().manual_seed(1)
    q_host = torch.randn(pairs * 2, B, Hq, D, generator=gq).to(dtype).pin_memory()
    q_dev = q_host.to(device)
    # distinct KV pools per layer so that consecutive steps never hit the same lines in L2
    pools = []
    for layer in range(pairs * 2):
        p = synth_shard(w, lo, hi, 1000 + layer * 64 + rank, dtype, device)
        plant(w, p, q_dev[layer], lo, hi, 7 + layer)
        pools.append(p)
    bytes_kv_layer = 2 * B * n_loc * Hkv * D * es
    l2_note = (f"{pairs * 2} distinct layer pools of {bytes_kv_layer / 2**20:.0f} MiB per GPU rotate; "
               f"every selection pass streams more than the 126 MB L2")

    sh = None
    if world > 1:
        sh = ShardedDecodeAttention(B, Hq, Hkv, D, dtype, plan, rank, k, "sum", device=device, exchange=args.exchange)
    ws = T.Workspace(B, Hq, D, B, max(n_loc, 1), device=device)
    scores = torch.empty(B, max(n_loc, 1), dtype=torch.float32, device=device)
    idx = torch.zeros(B, k, dtype=torch.int32, device=device)
    o_both = torch.empty(2, B, Hq, D, dtype=dtype, device=device)       # both layers' outputs: one device-to-host copy per step
    o_sel, o_sp = o_both[0], o_both[1]
    out_host = torch.empty(2, B, Hq, D, dtype=dtype).pin_memory()
    q_step = torch.empty(2, B, Hq, D, dtype=dtype, device=device)
    ev_sel = []

    def step(i, timed_kernel=False, e2e=False, sync=True):
        ls, lp = (2 * i) % (2 * pairs), (2 * i + 1) % (2 * pairs)
        if e2e:
            q_step.copy_(q_host[ls:ls + 2], non_blocking=True)    # ls is even and lp == ls + 1
            qs, qp = q_step[0], q_step[1]
        else:
            qs, qp = q_dev[ls], q_dev[lp]
        if sh is None:
            if timed_kernel:
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            T.decode_attention(qs, pools[ls], n_loc, ws, pages_per_seq=n_loc, scores=scores, hist=ws.hist, out=o_sel)
            if timed_kernel:
                b_.record()
                ev_sel.append((a, b_))
            T.topk(scores, k, ws, out_idx=idx, hist=ws.hist)
            T.decode_attention(qp, pools[lp], n_loc, ws, pages_per_seq=n_loc, sel_idx=idx, out=o_sp)
            outs = (o_sel, o_sp)
        else:
            a1 = sh.selection_layer(qs, pools[ls], pages_per_seq=max(n_loc, 1), timing=ev_sel if timed_kernel else None)
            if e2e:
                out_host[0].copy_(a1, non_blocking=True)
            a2 = sh.sparse_layer(qp, pools[lp], pages_per_seq=max(n_loc, 1))
            outs = (None, a2)
        if e2e:
            if sh is None:
                out_host.copy_(o_both, non_blocking=True)
            else:
                out_host[1].copy_(outs[1], non_blocking=True)
            if sync:
                torch.cuda.current_stream().synchronize()     # the caller reads the step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    use_graph = args.graph != 0
    graphs = {}

    def step_graph(i, e2e):
        """One CUDA graph per (layer pair, variant): the sharded step is a dozen small launches and two
        collectives, which the host cannot issue as fast as the GPUs retire them."""
        key = (i % pairs, e2e)
        g = graphs.get(key)
        if g is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step(i % pairs, e2e=e2e, sync=False)
            graphs[key] = g
        return g

    done_ev = torch.cuda.Event()

    def run_step(i, timed_kernel=False, e2e=False):
        if use_graph and not timed_kernel:
            step_graph(i, e2e).replay()
            if e2e:
                # the caller reads the step's result: poll the event instead of a blocking wait (a few us less)
                done_ev.record()
                while not done_ev.query():
                    pass
        else:
            step(i, timed_kernel=timed_kernel, e2e=e2e)

    def block_graph():
        """All `pairs` layer pairs back to back in one graph: the resident-input loop is launch-bound between graphs."""
        g = graphs.get("block")
        if g is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(pairs):
                    step(i, sync=False)
            graphs["block"] = g
        return g

    def timed(n_steps, **kw):
        barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if use_graph and not kw and n_steps % pairs == 0:
            g = block_graph()
            for _ in range(n_steps // pairs):
                g.replay()
        else:
            for i in range(n_steps):
                run_step(i, **kw)
        b_.record()
        barrier()
        ms = a.elapsed_time(b_)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    for i in range(args.warmup):
        step(i)
        step(i, e2e=True)
    torch.cuda.synchronize()
    if sh is not None and sh.peer is not None and args.exchange == "auto":
        # a peer exchange whose bounded waits ran out on any rank (a rank that cannot reach a peer's memory):
        # every rank falls back to the library all-gather together
        bad = torch.tensor([sh.exchange_status()], device=device)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad):
            if rank == 0:
                print("bench: peer exchange reported fault bits %d during warm-up, using NCCL" % int(bad), file=sys.stderr)
            sh = ShardedDecodeAttention(B, Hq, Hkv, D, dtype, plan, rank, k, "sum", device=device, exchange="nccl")
            for i in range(args.warmup):
                step(i)
                step(i, e2e=True)
            torch.cuda.synchronize()
    assert ws.status() == 0 and (sh is None or (sh.ws.status() | sh.exchange_status()) == 0), "device-side fault bits set during warm-up"
    if use_graph:
        block_graph().replay()
        for i in range(pairs):
            step_graph(i, False)
            step_graph(i, True)
        for i in range(args.warmup):
            run_step(i)
            run_step(i, e2e=True)
        torch.cuda.synchronize()

    launches0 = T.lib.tidal_launch_count()
    launches_eager = None
    with ClockSampler(torch.cuda.current_device()) as cs:
        if use_graph:
            # kernel-level events cannot be recorded inside a graph: time the dominant kernel in an eager pass
            # over the same steps first, then the graph-replayed region
            for i in range(min(args.steps, 4 * pairs)):
                step(i, timed_kernel=True)
            launches_eager = T.lib.tidal_launch_count() - launches0
            ms = timed(args.steps)
        else:
            ms = timed(args.steps, timed_kernel=True)
    launches = T.lib.tidal_launch_count() - launches0
    if use_graph:
        # graph replays do not pass through the library's host entry points: count what one captured step
        # launches (measured in the eager pass) times the steps
        launches = int(round(launches_eager / min(args.steps, 4 * pairs) * args.steps))
    ms_e2e = timed(args.steps, e2e=True)
    assert ws.status() == 0 and (sh is None or (sh.ws.status() | sh.exchange_status()) == 0), "device-side fault bits set"

    ms_step = ms / args.steps
    value = B / (ms_step * 1e-3)
    hbm, which = peaks()
    roof = None
    if ev_sel:
        sel_ms = sum(a.elapsed_time(b_) for a, b_ in ev_sel) / len(ev_sel)
        alg = bytes_kv_layer + 4 * B * n_loc
        ach = alg / (sel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "decode_attn_kernel (selection layer: K,V streamed once, fp32 logits written)",
                "achieved": round(ach, 1), "peak": hbm, "peak_source": which, "unit": "GB/s", "frac": round(ach / hbm, 4),
                "algorithmic_bytes": alg, "us_per_launch": round(sel_ms * 1e3, 2), "traffic": None}
        if args.workload in NCU_TRAFFIC_BYTES:
            # measured at one GPU; a shard's launch streams n_loc / N of the tokens and traffic follows the tokens
            roof["traffic"] = int(NCU_TRAFFIC_BYTES[args.workload] * n_loc / N)
            roof["traffic_source"] = "ncu capture of this launch at 1 GPU (profiles/), scaled by the tokens a shard holds"
    per_layer = None
    if sh is None:
        # steady-state device time of each layer type: 2*pairs back-to-back launches (distinct pools) replayed as a graph
        def op_us(fn, reps=2 * pairs, iters=10):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(reps):
                    fn(i % (2 * pairs))
            g.replay()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                g.replay()
            b_.record()
            torch.cuda.synchronize()
            return round(a.elapsed_time(b_) * 1e3 / (reps * iters), 2)

        kn = torch.randn(B, Hkv, D, device=device).to(dtype)
        vn = torch.randn(B, Hkv, D, device=device).to(dtype)
        qr = q_dev[0].clone()

        def sel_layer(i):
            T.decode_attention(q_dev[i], pools[i], n_loc, ws, pages_per_seq=n_loc, scores=scores, hist=ws.hist, out=o_sel)
            T.topk(scores, k, ws, out_idx=idx, hist=ws.hist)

        per_layer = {
            "full_attention": op_us(lambda i: T.decode_attention(q_dev[i], pools[i], n_loc, ws, pages_per_seq=n_loc, out=o_sel)),
            "selection_attention_plus_topk": op_us(sel_layer),
            "sparse_attention": op_us(lambda i: T.decode_attention(q_dev[i], pools[i], n_loc, ws, pages_per_seq=n_loc,
                                                                    sel_idx=idx, out=o_sp), reps=8 * pairs),
            "rope_append": op_us(lambda i: T.rope_append(qr, kn, vn, pools[i], batch=B, pos0=n_loc - 1, rope_mode=2,
                                                         rope_theta=1e4), reps=8 * pairs),
            "note": "steady-state device time per launch group, back-to-back launches on distinct layer pools replayed as a CUDA graph",
        }
        full_bytes = bytes_kv_layer
        per_layer["full_attention_frac_of_hbm_peak"] = round(full_bytes / (per_layer["full_attention"] * 1e-6) / 1e9 / peaks()[0], 4)
        per_layer["selection_frac_of_hbm_peak"] = round((bytes_kv_layer + 4 * B * n_loc) / (per_layer["selection_attention_plus_topk"] * 1e-6) / 1e9 / peaks()[0], 4)
        sparse_bytes = 2 * B * k * Hkv * D * es + 4 * B * k
        per_layer["sparse_frac_of_hbm_peak"] = round(sparse_bytes / (per_layer["sparse_attention"] * 1e-6) / 1e9 / peaks()[0], 4)
        assert ws.status() == 0
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": {"float16": "f16", "bfloat16": "bf16"}[w["dtype"]], "data": "synthetic",
        "config": {"workload": f"{args.workload}: selection layer + sparse layer, B={B}, {Hq}q/{Hkv}kv heads x {D}, "
                               f"context {N}, top_k {k}, head-summed scores",
                   "kv_sharding": f"sequence-sharded over {world} GPU(s)" + (("; per-layer exchange: " + ("peer stores (tidal_peer_all_gather)" if sh.peer is not None else "NCCL all-gather")) if sh is not None else ""), "l2": l2_note},
        "e2e": {"value": round(B / (ms_e2e / args.steps * 1e-3), 2), "unit": UNIT,
                "h2d_bytes_per_step": 2 * B * Hq * D * es, "d2h_bytes_per_step": 2 * B * Hq * D * es},
        "gpu_launches": int(launches),
        "clocks": cs.summary(),
    }
    if use_graph:
        line["config"]["launch"] = ("each step is the public operator calls captured once into a CUDA graph and replayed "
                                    "(kernels, copies, NCCL all-gathers): the resident-input loop replays graphs of "
                                    f"{pairs} consecutive steps when the step count divides, the end-to-end loop one step per graph, "
                                    "polling its completion; the roofline kernel is timed with CUDA events in an eager pass over the same steps")

    if roof:
        line["roofline"] = roof
    if per_layer:
        line["us_per_layer"] = per_layer
    return line


def cpu_reference_leg(workload, budget_s, steps=None, warmup=1):
    """The reference's CPU path (PyTorch, all host threads) restated in oracle/: dense
    logits + top-k + dense masked sparse layer, as src/tidal_build/modify_llama.py:105-133 does."""
    from oracle import tidal_oracle as O

    w = WORKLOADS[workload]
    dtype = getattr(torch, w["dtype"])
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    # bounded sample: one sequence of the batch, context capped so that a step stays near a second
    Bs = 1
    Ns = min(N, 131072)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(Bs, Hq, 1, D, generator=g).to(dtype)
    K = torch.randn(Bs, Hkv, Ns, D, generator=g).to(dtype)
    V = torch.randn(Bs, Hkv, Ns, D, generator=g).to(dtype)
    times = []
    t_end = time.time() + budget_s
    n = 0
    with torch.no_grad():
        while True:
            t0 = time.time()
            _, _, mask = O.selection_layer(q, K, V, k, "sum")
            O.sparse_layer(q, K, V, mask)
            dt = time.time() - t0
            n += 1
            if n > warmup:
                times.append(dt)
            if steps is not None and len(times) >= steps:
                break
            if steps is None and time.time() > t_end and len(times) >= 3:
                break
    per_step = statistics.mean(times)
    # a step of the full workload is B sequences of N tokens; the sample scales linearly in B and N
    scale = (B / Bs) * (N / Ns)
    tokens_per_s = B / (per_step * scale)
    sample = (f"{len(times)} steps of 1 sequence x {Ns} context ({w['dtype']}, {Hq}q/{Hkv}kv x {D}), "
              f"{per_step * 1e3:.1f} ms each; scaled x{scale:g} to B={B}, context {N}")
    return tokens_per_s, per_step * scale * 1e3, sample, len(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", choices=["auto", "nccl", "peer"], default="auto",
                    help="per-layer exchange of sharded KV: this library's peer-store all-gather, or NCCL")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", type=int, default=-1, help="replay each step as one CUDA graph (default); 0: issue every launch from the host")
    ap.add_argument("--layer-pairs", type=int, default=0, help="distinct (selection, sparse) KV pool pairs to rotate over")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    threads = torch.get_num_threads()

    if args.impl == "reference":
        if rank != 0:
            return
        steps = min(args.steps, 20)
        v, ms, sample, n = cpu_reference_leg(args.workload, 30.0, steps=steps, warmup=min(args.warmup, 3))
        w = WORKLOADS[args.workload]
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": round(v, 3), "unit": UNIT, "n_gpus": args.gpus, "steps": n,
            "warmup": min(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": {"float16": "f16", "bfloat16": "bf16"}[w["dtype"]], "data": "synthetic",
            "config": {"workload": f"{args.workload}: selection layer + sparse layer (dense masked, as the reference's "
                                   f"PyTorch path computes it) on the host CPU"},
            "cpu_baseline": {"value": round(v, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": round(v, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    line = run_ours(args, rank, world, device)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            v, ms, sample, _ = cpu_reference_leg(args.workload, 12.0)
            line["cpu_baseline"] = {"value": round(v, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
