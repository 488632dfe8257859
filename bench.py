"""Benchmark of the decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5|cfg4|cfg2] [--impl ours|reference]

One step = one decoded token's worth of the path on one attention-layer pair:
RoPE on the new token's q,k + append of its k,v to the paged pool, a token-selection
layer (full attention over the whole context + head-summed fp32 logits + top-k), then
RoPE + append and a sparse layer over the selected positions on the next layer's pool.
Prints ONE JSON line (rank 0).  Under torchrun (N > 1) the KV cache is sharded by
sequence across the ranks and the step includes the per-layer exchanges.

Workloads (synthetic, seeded; tidaldecode_b200/workloads.py):
    cfg5  B=8, 64 q / 8 kv heads x 128 bf16, context 1048576, top_k 1024   (default: the 1 M-context
          workload the 1 -> 8 GPU scaling target is stated on; one layer pair is 64 GiB and fits one GPU)
    cfg4  B=4, 32 q / 8 kv heads x 128 bf16, context 131072, top_k 128
    cfg2  B=1, 32 heads x 128 MHA fp16, context 32768, top_k 256, 64 planted keys
At one GPU the line also carries the per-layer figures of the workloads not chosen (`other_workloads`).

Before anything is timed, the first step's outputs (rotated queries, appended rows, selection-layer
output, selected set, sparse-layer output) are compared with the CPU oracle on the same bits
(`parity_checked`); a mismatch aborts the run.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tidaldecode_b200.workloads import WORKLOADS, describe  # noqa: E402  (host-side tables only; no CUDA needed)

METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"
DTYPE_TAG = {"float16": "f16", "bfloat16": "bf16"}
ROPE_THETA = {"cfg2": 1e4, "cfg4": 5e5, "cfg5": 1e4}
MIN_TIMED_S = 0.5          # the timed region is repeated until it is at least this long


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum per token streamed by one selection-layer launch,
    from the ncu captures summarised under profiles/ (profiles/ncu_traffic.json names the capture)."""
    p = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        t = json.load(f)
    return t.get(workload)


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
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
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
            self._stop.wait(0.01)

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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def workload_dict(name, args):
    """The workload's table entry; --context shortens the context (a small case of the same kernels for a
    profiler capture), the planted keys keep their share of it."""
    w = dict(WORKLOADS[name])
    ctx = getattr(args, "context", 0)
    if ctx and ctx != w["N"]:
        w["planted"] = max(1, w["planted"] * ctx // w["N"])
        w["N"] = ctx
        w["k"] = min(w["k"], ctx)
    return w


def describe_w(name, w):
    s = describe(name)
    return s if w["N"] == WORKLOADS[name]["N"] else s.replace(f"context {WORKLOADS[name]['N']}", f"context {w['N']} (shortened)")


def inv_freq(D, theta, device):
    """1 / theta^(2i/D) in fp32, computed on the host as model code does, so that the device and any checker
    form the same fp32 angle position * inv_freq (at a position of 10^6 one ulp of the frequency is 0.05 rad)."""
    return (1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.int64).float() / D))).to(device)


class Workload:
    """Buffers and the step function of one workload on one rank."""

    def __init__(self, name, args, rank, world, device):
        import tidaldecode_b200.ops as T
        from tidaldecode_b200 import workloads as WL
        from tidaldecode_b200.sharded import ShardPlan, ShardedDecodeAttention

        self.T, self.name, self.args, self.rank, self.world, self.device = T, name, args, rank, world, device
        w = self.w = workload_dict(name, args)
        self.dtype = dtype = getattr(torch, w["dtype"])
        B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
        self.plan = plan = ShardPlan.contiguous(N, world)
        self.lo, self.hi = plan.range_of(rank)
        self.n_loc = n_loc = self.hi - self.lo
        self.pairs = pairs = args.layer_pairs if args.layer_pairs > 0 else w["layer_pairs"]
        self.theta = ROPE_THETA[name]
        self.inv_freq = inv_freq(D, self.theta, device)
        # the new token sits at position N - 1: its k,v are appended by the rank that owns that position
        self.owner = plan.owner_of(N - 1) == rank
        # per layer: raw q, and the new token's k, v — one pinned block per layer so that a step's inputs are one copy
        g = torch.Generator().manual_seed(1)
        self.tok = Hq + 2 * Hkv                                   # head rows of one token: q heads, k heads, v heads
        # flat per layer: q [B,Hq,D], then k [B,Hkv,D], then v [B,Hkv,D]
        host = torch.randn(pairs * 2, B * self.tok * D, generator=g).to(dtype)
        self.in_host = host.pin_memory()
        self.in_dev = host.to(device)                              # resident inputs
        self.in_step = torch.empty(2, B * self.tok * D, dtype=dtype, device=device)   # landing buffer of the per-step copy
        self.q_rot = torch.empty(2, B, Hq, D, dtype=dtype, device=device)
        # distinct KV pools per layer so that consecutive steps never hit the same lines in L2
        self.pools = []
        for layer in range(pairs * 2):
            p = WL.synth_shard(w, self.lo, self.hi, 1000 + layer * 64 + rank, dtype, device)
            # planted keys follow the ROTATED query of the layer (what the attention sees)
            WL.plant(w, p, self._rotated_q_host(layer), self.lo, self.hi, 7 + layer)
            self.pools.append(p)
        self.bytes_kv_layer = 2 * B * n_loc * Hkv * D * 2
        l2_mb = 126
        if self.bytes_kv_layer > l2_mb * 1e6:
            self.l2_note = (f"{pairs * 2} distinct layer pools of {self.bytes_kv_layer / 2**20:.0f} MiB per GPU rotate; "
                            f"every selection pass streams more than the {l2_mb} MB L2")
        elif pairs * 2 * self.bytes_kv_layer > l2_mb * 1e6:
            self.l2_note = (f"{pairs * 2} distinct layer pools of {self.bytes_kv_layer / 2**20:.0f} MiB per GPU rotate "
                            f"({pairs * 2 * self.bytes_kv_layer / 2**20:.0f} MiB in all, more than the {l2_mb} MB L2): a pool's "
                            "lines are evicted before it is streamed again")
        else:
            self.l2_note = (f"WARNING: this rank's {pairs * 2} layer pools ({pairs * 2 * self.bytes_kv_layer / 2**20:.0f} MiB) "
                            f"fit the {l2_mb} MB L2; raise --layer-pairs for an L2-cold number")
        self.sh = None
        if world > 1:
            self.sh = ShardedDecodeAttention(B, Hq, Hkv, D, dtype, plan, rank, k, "sum", device=device, exchange=args.exchange)
        self.ws = T.Workspace(B, Hq, D, B, max(n_loc, 1), device=device)
        self.scores = torch.empty(B, max(n_loc, 1), dtype=torch.float32, device=device)
        self.idx = torch.zeros(B, k, dtype=torch.int32, device=device)
        self.o_both = torch.empty(2, B, Hq, D, dtype=dtype, device=device)    # both layers' outputs: one device-to-host copy per step
        self.out_host = torch.empty(2, B, Hq, D, dtype=dtype).pin_memory()
        self.rope_status = torch.zeros(1, dtype=torch.int32, device=device)
        self.ev_sel = []
        self.h2d = 2 * B * self.tok * D * 2
        self.d2h = 2 * B * Hq * D * 2

    def _rotated_q_host(self, layer):
        """RoPE (fp32, rounded once) of the layer's raw queries at position N - 1, on the host: only to place the
        planted keys; the timed path rotates on the device."""
        w = self.w
        q = self.split(self.in_host[layer])[0].float()             # [B, Hq, D]
        D = w["D"]
        ang = float(w["N"] - 1) * self.inv_freq.cpu().float()
        cos, sin = torch.cat((ang, ang)).cos(), torch.cat((ang, ang)).sin()
        rot = torch.cat((-q[..., D // 2:], q[..., : D // 2]), dim=-1)
        return (q * cos + rot * sin).to(self.dtype)

    def split(self, flat):
        """(q [B,Hq,D], k [B,Hkv,D], v [B,Hkv,D]) views of one layer's flat input block."""
        w = self.w
        B, Hq, Hkv, D = w["B"], w["Hq"], w["Hkv"], w["D"]
        a, b_ = B * Hq * D, B * (Hq + Hkv) * D
        return flat[:a].view(B, Hq, D), flat[a:b_].view(B, Hkv, D), flat[b_:].view(B, Hkv, D)

    # ------------------------------------------------------------------ one step
    def rope_append(self, src, layer, slot):
        """RoPE of the layer's q (out of place, into q_rot[slot]) and of the new k at position N - 1, and the
        append of k,v to that position's slot on the rank that owns it (the others only rotate)."""
        w, T = self.w, self.T
        q_src, k_new, v_new = self.split(src)
        T.rope_append(self.q_rot[slot], k_new, v_new if self.owner else None, self.pools[layer] if self.owner else None,
                      batch=w["B"], pos0=w["N"] - 1, kv_pos_base=self.lo, pages_per_seq=max(self.n_loc, 1),
                      rope_mode=2, inv_freq=self.inv_freq, rope_theta=self.theta, rotate_k_in_place=False,
                      status=self.rope_status, q_src=q_src)

    def step(self, i, timed_kernel=False, e2e=False, sync=True, keep=False):
        T, w, pairs = self.T, self.w, self.pairs
        ls, lp = (2 * i) % (2 * pairs), (2 * i + 1) % (2 * pairs)
        if e2e:
            self.in_step.copy_(self.in_host[ls:ls + 2], non_blocking=True)     # ls is even and lp == ls + 1
            src_s, src_p = self.in_step[0], self.in_step[1]
        else:
            src_s, src_p = self.in_dev[ls], self.in_dev[lp]
        n_loc, k = self.n_loc, w["k"]
        self.rope_append(src_s, ls, 0)
        if self.sh is None:
            if timed_kernel:
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
            T.decode_attention(self.q_rot[0], self.pools[ls], n_loc, self.ws, pages_per_seq=n_loc, scores=self.scores,
                               hist=self.ws.hist, out=self.o_both[0])
            if timed_kernel:
                b_.record()
                self.ev_sel.append((a, b_))
            T.topk(self.scores, k, self.ws, out_idx=self.idx, hist=self.ws.hist)
            self.rope_append(src_p, lp, 1)
            T.decode_attention(self.q_rot[1], self.pools[lp], n_loc, self.ws, pages_per_seq=n_loc, sel_idx=self.idx,
                               out=self.o_both[1])
            if e2e:
                self.out_host.copy_(self.o_both, non_blocking=True)
        else:
            a1 = self.sh.selection_layer(self.q_rot[0], self.pools[ls], pages_per_seq=max(n_loc, 1),
                                         timing=self.ev_sel if timed_kernel else None)
            if e2e:
                self.out_host[0].copy_(a1, non_blocking=True)
            elif keep:                                          # the checker wants both layers' outputs side by side
                self.o_both[0].copy_(a1)
            self.rope_append(src_p, lp, 1)
            a2 = self.sh.sparse_layer(self.q_rot[1], self.pools[lp], pages_per_seq=max(n_loc, 1))
            if e2e:
                self.out_host[1].copy_(a2, non_blocking=True)
            elif keep:
                self.o_both[1].copy_(a2)
        if e2e and sync:
            torch.cuda.current_stream().synchronize()          # the caller reads the step's result

    def status(self):
        s = self.ws.status() | int(self.rope_status.item())
        if self.sh is not None:
            s |= self.sh.ws.status() | self.sh.exchange_status()
        return s


# ---------------------------------------------------------------------- parity (outside every timed region)
def parity_check(wl: Workload, seqs):
    """The first step's results against the CPU oracle on the bits the kernels read and wrote.  Returns
    {"max_abs_err": ..., "sequences": ...}; raises on a mismatch.  Sharded: every rank evaluates the
    oracle on its own shard, rank 0 merges the partials exactly as the oracle's merge prescribes."""
    import torch.distributed as dist

    from oracle import tidal_oracle as O          # the checker; never on a timed or shipped path
    from tidaldecode_b200 import workloads as WL

    w, T = wl.w, wl.T
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    dtype, n_loc, world, rank = wl.dtype, wl.n_loc, wl.world, wl.rank
    tol = dict(rtol=2e-3, atol=1e-2)             # the tolerance stated for fp16/bf16 attention outputs
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    wl.step(0, keep=True)
    torch.cuda.synchronize()
    assert wl.status() == 0, "device-side fault bits set in the first step"
    worst = 0.0

    def close(got, want, what):
        nonlocal worst
        got, want = got.float().cpu(), want.float().cpu()
        err = (got - want).abs().max().item() if got.numel() else 0.0
        worst = max(worst, err)
        if not torch.allclose(got, want, **tol):
            raise SystemExit(f"bench: PARITY MISMATCH in {what}: max abs err {err:.3e} (rtol {tol['rtol']}, atol {tol['atol']})")

    # RoPE of q and the appended rows (fp32 rotation rounded once: within one unit of the storage type)
    pos = torch.full((B,), N - 1)
    ang_inv = wl.inv_freq.cpu()
    for slot, layer in ((0, 0), (1, 1)):
        xq, xk, xv = wl.split(wl.in_host[layer])

        def rope(x):
            ang = float(N - 1) * ang_inv
            cos, sin = torch.cat((ang, ang)).cos(), torch.cat((ang, ang)).sin()
            xf = x.float()
            return (xf * cos + O.rotate_half(xf) * sin).to(dtype)

        got_q = wl.q_rot[slot].cpu()
        if not torch.allclose(got_q.float(), rope(xq).float(), rtol=2 * ulp, atol=2 * ulp):
            raise SystemExit("bench: PARITY MISMATCH in RoPE of q")
        if wl.owner:
            rows = torch.stack([wl.pools[layer][b * n_loc + n_loc - 1, :, 0] for b in range(B)]).cpu()   # [B, 2, Hkv, D]
            if not torch.allclose(rows[:, 0].float(), rope(xk).float(), rtol=2 * ulp, atol=2 * ulp):
                raise SystemExit("bench: PARITY MISMATCH in the appended K row")
            if not torch.equal(rows[:, 1], xv):
                raise SystemExit("bench: PARITY MISMATCH in the appended V row")

    q_sel, q_sp = wl.q_rot[0].cpu(), wl.q_rot[1].cpu()
    o_sel, o_sp = wl.o_both[0].cpu(), wl.o_both[1].cpu()
    if wl.sh is None:
        idx = wl.idx.cpu()
        for b in seqs:
            K, V = WL.dense_of_sequence(w, wl.pools[0], b, n_loc)
            qb = q_sel[b:b + 1, :, None, :]
            want_o, want_s = O.attention_chunked(qb, K, V, "sum")
            close(o_sel[b:b + 1], want_o, f"selection-layer output, sequence {b}")
            ok, why = O.topk_sets_match(want_s, idx[b:b + 1], k, tie_band=1e-4)
            if not ok:
                raise SystemExit(f"bench: PARITY MISMATCH in the selected set, sequence {b}: {why}")
            K, V = WL.dense_of_sequence(w, wl.pools[1], b, n_loc)
            close(o_sp[b:b + 1], O.gathered_attention_gqa(q_sp[b:b + 1, :, None, :], K, V, idx[b:b + 1]),
                  f"sparse-layer output, sequence {b}")
        return {"max_abs_err": worst, "sequences": list(seqs)}
    # sharded
    sh = wl.sh
    cnt = sh.sel_count.cpu()
    nb = len(seqs)
    pack = torch.zeros(nb, 2, Hq, D + 2, dtype=torch.float32)      # [seq][layer kind][head][m, l, o...]
    sc = torch.full((nb, max(wl.plan.bounds[r + 1] - wl.plan.bounds[r] for r in range(world))), -float("inf"))
    chosen = torch.full((nb, k), -1, dtype=torch.int64)
    for j, b in enumerate(seqs):
        mine = sh.sel_local[b, : int(cnt[b])].cpu().long()
        chosen[j, : mine.numel()] = mine + wl.lo
        if n_loc > 0:
            K, V = WL.dense_of_sequence(w, wl.pools[0], b, n_loc)
            (m, l, o), s = O.attention_chunked(q_sel[b:b + 1, :, None, :], K, V, "sum", return_partials=True)
            sc[j, :n_loc] = s[0]
            pack[j, 0, :, 0], pack[j, 0, :, 1], pack[j, 0, :, 2:] = m[0], l[0], o[0]
            K, V = WL.dense_of_sequence(w, wl.pools[1], b, n_loc)
            m, l, o = O.partial_attention(q_sp[b:b + 1, :, None, :], K[:, :, mine], V[:, :, mine])
            pack[j, 1, :, 0], pack[j, 1, :, 1], pack[j, 1, :, 2:] = m[0], l[0], o[0]
        else:
            pack[j, :, :, 0] = -float("inf")
    dev = wl.device
    gp = [torch.empty_like(pack, device=dev) for _ in range(world)]
    gs = [torch.empty_like(sc, device=dev) for _ in range(world)]
    gc = [torch.empty_like(chosen, device=dev) for _ in range(world)]
    dist.all_gather(gp, pack.to(dev))
    dist.all_gather(gs, sc.to(dev))
    dist.all_gather(gc, chosen.to(dev))
    if rank == 0:
        gp, gs, gc = [t.cpu() for t in gp], [t.cpu() for t in gs], [t.cpu() for t in gc]
        for j, b in enumerate(seqs):
            for kind, got, what in ((0, o_sel, "merged selection-layer output"), (1, o_sp, "merged sparse-layer output")):
                parts = [(t[j, kind, :, 0][None], t[j, kind, :, 1][None], t[j, kind, :, 2:][None]) for t in gp]
                close(got[b:b + 1], O.merge_partials(parts), f"{what}, sequence {b}")
            full = torch.cat([gs[r][j, : wl.plan.bounds[r + 1] - wl.plan.bounds[r]] for r in range(world)])[None]
            union = torch.cat([t[j][t[j] >= 0] for t in gc])[None]
            ok, why = O.topk_sets_match(full, union, k, tie_band=1e-4)
            if not ok:
                raise SystemExit(f"bench: PARITY MISMATCH in the union of the ranks' selected positions, sequence {b}: {why}")
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"max_abs_err": float(t), "sequences": list(seqs)}


# ---------------------------------------------------------------------- timing
def run_workload(name, args, rank, world, device):
    import torch.distributed as dist

    wl = Workload(name, args, rank, world, device)
    T, w, pairs = wl.T, wl.w, wl.pairs
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    n_loc = wl.n_loc
    steps = args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    parity = None
    if not args.no_parity:
        # cfg2 and cfg4 in full; the 1 M workload on one sequence (4 GiB of K,V through the host per sequence)
        parity = parity_check(wl, range(B) if name != "cfg5" else [0])

    use_graph = args.graph != 0
    graphs = {}

    def step_graph(i, e2e):
        """One CUDA graph per (layer pair, variant): a step is a dozen small launches (and two exchanges when
        sharded), which the host cannot issue as fast as the GPUs retire them."""
        key = (i % pairs, e2e)
        g = graphs.get(key)
        if g is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                wl.step(i % pairs, e2e=e2e, sync=False)
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
            wl.step(i, timed_kernel=timed_kernel, e2e=e2e)

    def block_graph():
        """All `pairs` layer pairs back to back in one graph: the resident-input loop is launch-bound between graphs."""
        g = graphs.get("block")
        if g is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(pairs):
                    wl.step(i, sync=False)
            graphs["block"] = g
        return g

    def timed_block(**kw):
        """EXACTLY `steps` steps between a barrier + synchronize on both sides, CUDA events, max over ranks."""
        barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if use_graph and not kw and steps % pairs == 0:
            g = block_graph()
            for _ in range(steps // pairs):
                g.replay()
        else:
            for i in range(steps):
                run_step(i, **kw)
        b_.record()
        barrier()
        ms = a.elapsed_time(b_)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    def timed(**kw):
        """Blocks of `steps` steps until the timed region is at least MIN_TIMED_S long (at least 3 blocks);
        the median block is reported."""
        first = timed_block(**kw)
        reps = max(3, min(200, int(math.ceil(MIN_TIMED_S * 1e3 / max(first, 1e-3)))))
        if world > 1:                               # every rank runs the same number of blocks
            t = torch.tensor([reps], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            reps = int(t)
        blocks = [first] + [timed_block(**kw) for _ in range(reps - 1)]
        return statistics.median(blocks), blocks

    for i in range(args.warmup):
        wl.step(i)
        wl.step(i, e2e=True)
    torch.cuda.synchronize()
    if wl.sh is not None and wl.sh.peer is not None and args.exchange == "auto":
        # a peer exchange whose bounded waits ran out on any rank (a rank that cannot reach a peer's memory):
        # every rank falls back to the library all-gather together
        from tidaldecode_b200.sharded import ShardedDecodeAttention
        bad = torch.tensor([wl.sh.exchange_status()], device=device)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad):
            if rank == 0:
                print("bench: peer exchange reported fault bits %d during warm-up, using NCCL" % int(bad), file=sys.stderr)
            wl.sh = ShardedDecodeAttention(B, Hq, Hkv, D, wl.dtype, wl.plan, rank, k, "sum", device=device, exchange="nccl")
            for i in range(args.warmup):
                wl.step(i)
                wl.step(i, e2e=True)
            torch.cuda.synchronize()
    assert wl.status() == 0, "device-side fault bits set during warm-up"
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
    eager_steps = min(steps, 4 * pairs)
    with ClockSampler(torch.cuda.current_device()) as cs:
        # kernel-level events cannot be recorded inside a graph: the dominant kernel is timed in an eager pass
        # over the same steps, then the (graph-replayed) timed region
        for i in range(eager_steps):
            wl.step(i, timed_kernel=True)
        launches_eager = T.lib.tidal_launch_count() - launches0
        ms, blocks = timed() if use_graph else timed(timed_kernel=True)
        ms_e2e, blocks_e2e = timed(e2e=True)
    assert wl.status() == 0, "device-side fault bits set"
    # graph replays do not pass through the library's host entry points: what one step launches (counted in
    # the eager pass) times the steps of one timed block
    launches = int(round(launches_eager / eager_steps * steps))

    ms_step = ms / steps
    value = B / (ms_step * 1e-3)
    hbm, which = peaks()
    roof = None
    per_layer = per_layer_times(wl)
    if wl.ev_sel and per_layer["selection_attention"] > 0:
        # the dominant launch (selection-layer attention + its chunk merge): CUDA events around back-to-back launches
        # on distinct pools replayed as a graph (steady state); the eager pass's events bracket the same launch inside a
        # whole step but also count the host's launch gaps, and are kept beside it
        eager_ms = statistics.median(a.elapsed_time(b_) for a, b_ in wl.ev_sel)
        sel_ms = per_layer["selection_attention"] * 1e-3
        alg = wl.bytes_kv_layer + 4 * B * n_loc
        ach = alg / (sel_ms * 1e-3) / 1e9
        kern = "decode_attn_mma_kernel" if Hq != Hkv else "decode_attn_kernel"
        roof = {"bound": "hbm", "kernel": f"{kern} + merge_chunks_kernel (selection layer: K,V streamed once, fp32 logits written)",
                "achieved": round(ach, 1), "peak": hbm, "peak_source": which, "unit": "GB/s", "frac": round(ach / hbm, 4),
                "algorithmic_bytes": alg, "us_per_launch": round(sel_ms * 1e3, 2),
                "us_per_launch_inside_an_eager_step": round(eager_ms * 1e3, 2), "traffic": None}
        tr = ncu_traffic(name)
        if tr:
            # captured on a case of tr["tokens"] tokens (all sequences); traffic follows the tokens streamed
            roof["traffic"] = int(tr["dram_bytes"] * (B * n_loc) / tr["tokens"])
            roof["traffic_source"] = tr["source"]
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": DTYPE_TAG[w["dtype"]], "data": "synthetic",
        "config": {"workload": describe_w(name, w),
                   "step": "RoPE + KV append of the new token, selection layer (attention over the whole context, head-summed "
                           "logits, top-k), RoPE + append, sparse layer over the selected positions",
                   "kv_sharding": f"sequence-sharded over {world} GPU(s)" + (
                       ("; per-layer exchange: " + ("peer stores (tidal_peer_all_gather)" if wl.sh.peer is not None else "NCCL all-gather"))
                       if wl.sh is not None else ""),
                   "l2": wl.l2_note},
        "timing": {"blocks": len(blocks), "steps_per_block": steps, "block_ms_median": round(ms, 4),
                   "block_ms_min": round(min(blocks), 4), "block_ms_max": round(max(blocks), 4),
                   "timed_region_s": round(sum(blocks) * 1e-3, 3),
                   "note": "each block is exactly `steps` steps between barrier + synchronize, CUDA events, max over ranks; "
                           "blocks repeat until the timed region is at least 0.5 s; ms_per_step = median block / steps"},
        "e2e": {"value": round(B / (ms_e2e / steps * 1e-3), 2), "unit": UNIT, "h2d_bytes_per_step": wl.h2d,
                "d2h_bytes_per_step": wl.d2h, "blocks": len(blocks_e2e)},
        "gpu_launches": launches,
        "clocks": cs.summary(),
    }
    if parity is not None:
        line["parity_checked"] = True
        line["parity"] = {"max_abs_err": round(parity["max_abs_err"], 6), "sequences_checked": parity["sequences"],
                          "against": "CPU oracle on the bits the kernels read (first step, outside the timed region): rotated q, "
                                     "appended rows, selection output, selected set (tie band 1e-4), sparse output; "
                                     "tolerance 2e-3 rel / 1e-2 abs"}
    else:
        line["parity_checked"] = False
    if use_graph:
        line["config"]["launch"] = ("each step is the public operator calls captured once into a CUDA graph and replayed "
                                    "(kernels, copies, exchanges): the resident-input loop replays graphs of "
                                    f"{pairs} consecutive steps when the step count divides, the end-to-end loop one step per graph, "
                                    "polling its completion; the roofline kernel is timed with CUDA events in an eager pass over the same steps")
    if roof:
        line["roofline"] = roof
    if per_layer:
        line["us_per_layer"] = per_layer
    return line


def per_layer_times(wl: Workload):
    """Steady-state device time of each layer type: back-to-back launches on distinct pools replayed as a graph."""
    T, w, pairs = wl.T, wl.w, wl.pairs
    B, Hq, Hkv, D, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["k"]
    n_loc = wl.n_loc
    hbm = peaks()[0]

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

    q0, q1 = wl.q_rot[0], wl.q_rot[1]

    def sel_attention(i):
        if wl.sh is None:
            T.decode_attention(q0, wl.pools[i], n_loc, wl.ws, pages_per_seq=n_loc, scores=wl.scores, hist=wl.ws.hist, out=wl.o_both[0])
        else:       # a rank's local launch: partials out, no normalised output
            sh = wl.sh
            m, l, o, _, _ = sh._send_views()
            T.decode_attention(q0, wl.pools[i], n_loc, sh.ws, pages_per_seq=n_loc, scores=sh.scores, hist=sh.ws.hist[: sh.rows],
                               partials=(m, l, o), want_out=False)

    iters = 3 if wl.bytes_kv_layer > (1 << 30) else 10          # launches of several ms need fewer repeats
    if n_loc > 0:
        sel_us = op_us(sel_attention, iters=iters)
        (wl.ws if wl.sh is None else wl.sh.ws).hist.zero_()      # no top-k consumed the digit counts of these launches
    else:
        sel_us = 0.0
    if wl.sh is not None:
        return {"selection_attention": sel_us,
                "note": "this rank's selection-layer attention launch, back-to-back on distinct layer pools replayed as a CUDA graph"}

    def sel_layer(i):
        T.decode_attention(q0, wl.pools[i], n_loc, wl.ws, pages_per_seq=n_loc, scores=wl.scores, hist=wl.ws.hist, out=wl.o_both[0])
        T.topk(wl.scores, k, wl.ws, out_idx=wl.idx, hist=wl.ws.hist)

    per = {
        "selection_attention": sel_us,
        "full_attention": op_us(lambda i: T.decode_attention(q0, wl.pools[i], n_loc, wl.ws, pages_per_seq=n_loc, out=wl.o_both[0]),
                                iters=iters),
        "selection_attention_plus_topk": op_us(sel_layer, iters=iters),
        "sparse_attention": op_us(lambda i: T.decode_attention(q1, wl.pools[i], n_loc, wl.ws, pages_per_seq=n_loc, sel_idx=wl.idx,
                                                               out=wl.o_both[1]), reps=8 * pairs),
        "rope_append": op_us(lambda i: wl.rope_append(wl.in_dev[i], i, 0), reps=8 * pairs),
        "note": "steady-state device time per launch group, back-to-back launches on distinct layer pools replayed as a CUDA graph",
    }
    sel_bytes = wl.bytes_kv_layer + 4 * B * n_loc
    sparse_bytes = 2 * B * k * Hkv * D * 2 + 4 * B * k
    per["full_attention_frac_of_hbm_peak"] = round(wl.bytes_kv_layer / (per["full_attention"] * 1e-6) / 1e9 / hbm, 4)
    per["selection_frac_of_hbm_peak"] = round(sel_bytes / (per["selection_attention_plus_topk"] * 1e-6) / 1e9 / hbm, 4)
    per["sparse_frac_of_hbm_peak"] = round(sparse_bytes / (per["sparse_attention"] * 1e-6) / 1e9 / hbm, 4)
    per["sparse_bytes"] = sparse_bytes
    assert wl.status() == 0
    return per


# ---------------------------------------------------------------------- the reference's CPU path
def cpu_reference_leg(workload, w, steps, warmup, budget_s=150.0):
    """The reference's CPU path (PyTorch, all host threads) restated in oracle/: RoPE of the new token, dense
    logits + top-k + dense masked sparse layer, as src/tidal_build/modify_llama.py:105-133 does.  Each step is a
    bounded sample of the workload — one sequence, a context cut so that the whole run stays inside budget_s —
    scaled linearly in batch and context to the full workload."""
    from oracle import tidal_oracle as O

    dtype = getattr(torch, w["dtype"])
    B, Hq, Hkv, D, N, k = w["B"], w["Hq"], w["Hkv"], w["D"], w["N"], w["k"]
    g = torch.Generator().manual_seed(0)

    def make(ns):
        return (torch.randn(1, Hq, 1, D, generator=g).to(dtype), torch.randn(1, Hkv, ns, D, generator=g).to(dtype),
                torch.randn(1, Hkv, ns, D, generator=g).to(dtype))

    def one_step(q, K, V):
        cos, sin = O.rope_cos_sin(torch.tensor([[K.shape[2] - 1]]), D, ROPE_THETA[workload], dtype)
        qr = O.apply_rope_path_a(q, cos[:, None], sin[:, None])
        K[:, :, -1:] = O.apply_rope_path_a(K[:, :, -1:], cos[:, None], sin[:, None])      # the new token's key, rotated and "appended"
        _, _, mask = O.selection_layer(qr, K, V, k, "sum")
        O.sparse_layer(qr, K, V, mask)

    with torch.no_grad():
        # calibrate on a short context, then take the longest power-of-two context that keeps the run inside the budget
        ns = min(N, 8192)
        q, K, V = make(ns)
        one_step(q, K, V)
        t0 = time.time()
        one_step(q, K, V)
        per_tok = (time.time() - t0) / ns
        total = steps + warmup
        ns = min(N, 131072)
        while ns > 8192 and per_tok * ns * total > budget_s:
            ns //= 2
        q, K, V = make(ns)
        times = []
        for i in range(total):
            t0 = time.time()
            one_step(q, K, V)
            if i >= warmup:
                times.append(time.time() - t0)
    per_step = statistics.mean(times)
    scale = B * (N / ns)
    tokens_per_s = B / (per_step * scale)
    sample = (f"{len(times)} steps of 1 sequence x {ns} context ({w['dtype']}, {Hq}q/{Hkv}kv x {D}), "
              f"{per_step * 1e3:.1f} ms each; scaled x{scale:g} to B={B}, context {N}")
    return tokens_per_s, per_step * scale * 1e3, sample


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", choices=["auto", "nccl", "peer"], default="auto",
                    help="per-layer exchange of sharded KV: this library's peer-store all-gather, or NCCL")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison of the first step")
    ap.add_argument("--no-others", action="store_true", help="one GPU: do not add the per-layer figures of the other workloads")
    ap.add_argument("--graph", type=int, default=-1, help="replay each step as one CUDA graph (default); 0: issue every launch from the host")
    ap.add_argument("--layer-pairs", type=int, default=0, help="distinct (selection, sparse) KV pool pairs to rotate over")
    ap.add_argument("--context", type=int, default=0, help="shorten the workload's context (a small case for a profiler capture)")
    args = ap.parse_args()
    if args.warmup < 3:
        print("bench: --warmup raised to 3 (at least three untimed steps)", file=sys.stderr)
        args.warmup = 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    threads = torch.get_num_threads()
    w = workload_dict(args.workload, args)

    if args.impl == "reference":
        if rank != 0:
            return
        v, ms, sample = cpu_reference_leg(args.workload, w, args.steps, args.warmup)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": round(v, 4), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE_TAG[w["dtype"]], "data": "synthetic",
            "config": {"workload": describe_w(args.workload, w),
                       "how": "the reference's PyTorch path on the host CPU (dense logits, top-k, dense masked sparse layer), "
                              "each step a bounded sample scaled to the workload"},
            "cpu_baseline": {"value": round(v, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": round(v, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    line = run_workload(args.workload, args, rank, world, device)
    if world == 1 and not args.no_others:
        others = {}
        for name in sorted(WORKLOADS):
            if name == args.workload or args.context:
                continue
            torch.cuda.empty_cache()
            o = run_workload(name, args, rank, world, device)
            others[name] = {"workload": o["config"]["workload"], "tokens_per_s": o["value"], "ms_per_step": o["ms_per_step"],
                            "e2e_tokens_per_s": o["e2e"]["value"], "parity_checked": o["parity_checked"],
                            "roofline_frac": o.get("roofline", {}).get("frac"), "us_per_layer": o.get("us_per_layer")}
        line["other_workloads"] = others
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            v, ms, sample = cpu_reference_leg(args.workload, w, 5, 1, budget_s=20.0)
            line["cpu_baseline"] = {"value": round(v, 4), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
