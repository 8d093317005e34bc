#!/usr/bin/env python3
"""Benchmark of the fused MAC decode step (one JSON line on stdout).

Metric: microseconds per decode step under CUDA-graph replay, with the HBM GB/s
it corresponds to, on the reference's headline workload: GQA-4 (Hq 32 / Hkv 8 /
D 128), bf16 paged KV (page 16), batch 64, context 126976, ring capacity 2048,
semantic_pos_ahead 256, per-query-head hit fraction 0.9 chosen by the
reference's own synthetic decision hash (its published curves were measured the
same way), match lag 64.  Inputs are seeded synthetic tensors of those shapes
(``mac_attention_b200/synth.py``).

    python bench.py [--gpus N] [--steps K] [--warmup W]     this library
    python bench.py --impl reference ...                     the reference's own CUDA kernel
    python bench.py --sweep ...                              hit/batch/context table
    python bench.py --config4 ...                            mixed serving step + prefill rows

The line of this library also carries: ``parity`` (the timed tensors checked
against the CPU oracle on a sample of requests), ``gpu_baselines`` (FlashInfer
full decode with and without tensor cores and the reference kernel on the same
tensors), ``config3`` (the Llama-70B attention shape split by KV head over the
N ranks), ``cpu_baseline`` and ``real_scan``.

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank
owns its own requests, KV pool and ring (the path shards by request with no
collective inside attention); the step time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HQ, HKV, DIM = 32, 8, 128
CAPACITY, SEM, TILE, MTS, MAX_CONTEXT = 2048, 256, 32, 32, 131072
LAG = 64
# dram__bytes_read+write / bytes requested by the kernel, from the ncu captures
# summarised under profiles/ (small cases, scaled by the units processed)
NCU_TRAFFIC_RATIO = 1.02
METRIC = "us_per_decode_step_cuda_graph_replay"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=126976)
    ap.add_argument("--hit", type=float, default=0.9)
    ap.add_argument("--hq", type=int, default=HQ)
    ap.add_argument("--hkv", type=int, default=HKV)
    ap.add_argument("--front-sink", type=int, default=0)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--capacity", type=int, default=CAPACITY)
    ap.add_argument("--bench-mode", type=int, default=1)
    ap.add_argument("--sweep", action="store_true", help="print the hit/batch/context table")
    ap.add_argument("--sweep-out", default=None, help="also write the sweep rows to this file")
    ap.add_argument("--baselines", default="",
                    help="comma list for --sweep/--config4: flashinfer,flashinfer_tc,refkernel")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the oracle legs (parity sample and cpu_baseline)")
    ap.add_argument("--no-gpu-baselines", action="store_true")
    ap.add_argument("--no-config3", action="store_true")
    ap.add_argument("--parity-requests", type=int, default=6)
    ap.add_argument("--matched-prefix", default="",
                    help="with --sweep: 'mean,std' of the matched prefix length as a fraction of "
                         "the context (BASELINE config 1 draws it from [0.5, 0.95]: 0.725,0.13). "
                         "Labelled extension: lifts the reference's rule that a reused entry lies "
                         "within the last M positions, for synthetic decisions only")
    ap.add_argument("--shard", default="request", choices=["request", "kv_head"])
    ap.add_argument("--config4", action="store_true",
                    help="mixed serving step with readiness gating + prefill ring build timing")
    ap.add_argument("--config4-part", choices=["all", "prefill"], default="all",
                    help="with --config4: run every row, or only the prefill ring-build rows")
    ap.add_argument("--prompt-len", type=int, default=32768,
                    help="with --config4: prompt length of the prefill ring-build rows")
    ap.add_argument("--config4-out", default=None, help="also write the config-4 rows to this file")
    return ap.parse_args()


# --------------------------------------------------------------------------- workload
def workload_config(args, world, hq=None, hkv=None, shard=None):
    """What is measured, in the same words for every arm of the benchmark."""
    hq = args.hq if hq is None else hq
    hkv = args.hkv if hkv is None else hkv
    shard = args.shard if shard is None else shard
    return {
        "workload": f"GQA-{hq // hkv} MAC decode step, Hq{hq}/Hkv{hkv}/D128, "
                    f"batch {args.batch} per GPU, context {args.ctx}, per-head hit fraction {args.hit} "
                    f"(reference synthetic_head decisions, lag {LAG}), ring M={args.capacity}, "
                    f"S={SEM}, F={args.front_sink}, paged KV page {args.page_size}",
        "batch": args.batch, "context": args.ctx, "hit_fraction": args.hit,
        "hq": hq, "hkv": hkv, "ring_capacity": args.capacity, "front_sink": args.front_sink,
        "page_size": args.page_size,
        "sharding": f"{shard} x{world}, no collective in attention",
        "l2": "inputs larger than L2 (K/V + ring streamed per step >> 126 MB)",
    }


def alg_bytes(ws, batch, hq, hkv, F, capacity, past_lens, eligible=True):
    """Bytes of one step from the decision arrays the kernel reports: K/V rows
    actually needed (512 B per token and KV head), the ring scan, reused prefix
    states, ring write, output, queries and the page-table entries.

    ``total`` counts full 256 B ring rows for every scanned slot (the convention
    of the reference's own accounting); ``requested`` counts what this kernel
    asks the memory system for: the 128 B probe half of every row (the second
    half is fetched only for rows that survive the probe, a handful per step).
    ``per_row`` is ``requested`` split by batch row."""
    from mac_attention_b200 import workspace as W

    head_hit = ws[W.HEAD_HIT][:batch].cpu()
    head_rect = ws[W.HEAD_RECT_START][:batch].cpu()
    new_end = ws[W.HEAD_NEW_END][:batch].cpu()
    mode = ws[W.GROUP_MODE][:batch].cpu()
    G = hq // hkv
    kv = pt = scan = 0
    per_row = []
    for n in range(batch):
        P = int(past_lens[n])
        kv_len = P + 1
        ne = int(new_end[n, 0])
        distinct = row_kv = 0
        for g in range(hkv):
            if int(mode[n, g]) != 0:
                t = kv_len
            else:
                lo = int(head_rect[n, g * G:(g + 1) * G].min())
                t = min(F, lo) + (ne - lo) + (kv_len - ne)
            row_kv += t * 512
            distinct = max(distinct, t)
        row_scan = min(capacity, P) * hq * 256 if eligible else 0
        row_small = int(head_hit[n].sum()) * 260 + hq * (516 + 256 + 512) + 4 * distinct
        kv += row_kv
        pt += 4 * distinct
        scan += row_scan
        per_row.append(row_kv + row_scan // 2 + row_small)
    hits = int(head_hit.sum())
    heads = batch * hq
    total = kv + scan + hits * 260 + heads * 516 + heads * 256 + heads * 512 + pt
    return dict(total=total, requested=total - scan // 2, kv=kv, scan=scan, hit_heads=hits,
                per_row=per_row, non_hit_groups=int((mode != 0).sum()),
                full_groups=int((mode == 1).sum()))


class ClockSampler:
    """nvidia-smi clock/throttle samples of one GPU while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "100", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


def build_case(args, device, seed, batch, ctx, hq, hkv):
    from mac_attention_b200 import synth

    case = synth.make_decode_case(batch=batch, ctx=ctx, hq=hq, hkv=hkv, capacity=args.capacity,
                                  page_size=args.page_size, seed=seed, device=device,
                                  sink_boost=64 if args.front_sink > 0 else 0)
    return case


def make_launch(ext, case, ws, scal, out, lse):
    import torch

    e = torch.empty(0)

    def launch():
        ext.mac_persistent_decode_bf16(
            case.q_post, case.q_pre, case.k, case.v, case.req_to_token, case.req_ids,
            case.past_lens, case.out_cache_loc, case.query_cache, case.attn_cache, case.lse_cache,
            out, lse, *ws, *scal, case.query_cache, e, e, e)
    return launch


def scalars(args, hit, debug=0, front_sink=None):
    """The operator's 21 scalars in positional order (reference benchmark defaults)."""
    F = args.front_sink if front_sink is None else front_sink
    skip, skip_std = -1.0, 0.0
    if getattr(args, "matched_prefix", ""):
        skip, skip_std = (float(x) for x in args.matched_prefix.split(","))
    return (MAX_CONTEXT, TILE, MTS, SEM, F, 0, 0, 0, 0.45, 1.0 / math.sqrt(DIM),
            debug, args.bench_mode, hit, 0.0, skip, skip_std, float(LAG), 0.0, 1, -1, 0)


def time_graph(launch, steps, warmup, barrier=None):
    """Mean ms per replay of a CUDA graph holding one step, CUDA events on the
    stream the graph is replayed on."""
    import torch

    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()
    for _ in range(max(warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        graph.replay()
    t1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return t0.elapsed_time(t1) / steps, graph


def replay_blocks(graph, steps, blocks=5):
    """Further blocks of `steps` replays of an already-timed graph, each between
    its own CUDA events: the spread of the headline number inside one process."""
    import torch

    out = []
    for _ in range(blocks):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            graph.replay()
        t1.record()
        torch.cuda.synchronize()
        out.append(t0.elapsed_time(t1) * 1e3 / steps)
    out.sort()
    return {"blocks": blocks, "steps_per_block": steps, "us_min": out[0],
            "us_median": out[len(out) // 2], "us_max": out[-1]}


class HostStep:
    """One step's host-side inputs the way a serving engine would send them: the
    two query tensors and the three per-row integer vectors packed into ONE
    pinned buffer, uploaded with one copy into a device buffer whose typed
    views are what the operator is called with."""

    def __init__(self, case, device):
        import copy

        import torch

        n = case.q_post.shape[0]
        parts = [("q_post", case.q_post), ("q_pre", case.q_pre), ("req_ids", case.req_ids[:n]),
                 ("past_lens", case.past_lens[:n]), ("out_cache_loc", case.out_cache_loc[:n])]
        off, layout = 0, []
        for name, t in parts:
            nbytes = t.numel() * t.element_size()
            layout.append((name, t, off, nbytes))
            off = (off + nbytes + 255) // 256 * 256
        self.host = torch.empty(off, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(off, dtype=torch.uint8, device=device)
        self.case = copy.copy(case)
        self.h2d_bytes = off
        for name, t, o, nbytes in layout:
            self.host[o:o + nbytes].copy_(t.contiguous().view(torch.uint8).reshape(-1).cpu())
            setattr(self.case, name, self.dev[o:o + nbytes].view(t.dtype).view(t.shape))

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)


def time_e2e(ext, case, ws, scal, out, lse, dev, n_steps, barrier, count_launches=None,
             host_out=True):
    """The step through the operator with HOST buffers: one pinned H2D copy of
    the step's inputs, the eager operator call with ``out`` in pinned host
    memory (the kernel writes the output rows over the bus itself), a stream
    synchronise; host wall clock per step.  The variant with the output on the
    device and a D2H copy after the kernel is timed beside it; it is the only
    one with ``host_out=False`` (the reference's operator wants device tensors)."""
    import torch

    hs = HostStep(case, dev)
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    launch_direct = make_launch(ext, hs.case, ws, scal, out_host, lse)
    launch_staged = make_launch(ext, hs.case, ws, scal, out, lse)
    stream = torch.cuda.current_stream()

    def step():
        hs.upload()
        launch_direct()
        stream.synchronize()

    def step_staged():
        hs.upload()
        launch_staged()
        out_host.copy_(out, non_blocking=True)
        stream.synchronize()

    def wall(fn, n):
        for _ in range(3):
            fn()
        barrier()
        w0 = time.perf_counter()
        for _ in range(n):
            fn()
        return (time.perf_counter() - w0) * 1e3 / n

    staged_ms = wall(step_staged, n_steps)
    d2h_bytes = out_host.numel() * out_host.element_size()
    if not host_out:
        return staged_ms, hs.h2d_bytes, d2h_bytes, None, {}
    staged_out = out_host.clone()
    out_host.zero_()
    before = count_launches() if count_launches else 0
    ms = wall(step, n_steps)
    launches = (count_launches() - before - 3) if count_launches else None
    same = bool(torch.equal(out_host, staged_out))

    def copy_us(fn):   # one copy alone, CUDA events on the same stream
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        stream.synchronize()
        t0.record()
        for _ in range(10):
            fn()
        t1.record()
        stream.synchronize()
        return t0.elapsed_time(t1) * 100.0

    parts = {"h2d_copy_us": copy_us(hs.upload),
             "d2h": "the kernel writes out into pinned host memory",
             "with_out_on_device_and_d2h_copy_us": staged_ms * 1e3,
             "d2h_copy_us": copy_us(lambda: out_host.copy_(out, non_blocking=True)),
             "host_out_equals_device_out": same}
    return ms, hs.h2d_bytes, d2h_bytes, launches, parts


def time_real_scan(args, ext, case, ws, out, lse, dev):
    """Times the step with ``bench_mode = 0`` on planted ring rows; restores the
    planted rows and the overwritten slot afterwards so the caller's case is intact."""
    import torch

    from mac_attention_b200 import synth
    from mac_attention_b200.workspace import HEAD_HIT

    G = args.hq // args.hkv
    ring = (case.query_cache, case.attn_cache, case.lse_cache)
    P = case.past_lens.long()
    req = case.req_ids.long()
    M = args.capacity
    touched = torch.stack([(P % M), ((P - LAG) % M)], dim=1)            # [N,2] slots per request
    saved = [t[req[:, None], touched].clone() for t in ring]
    planted = synth.plant_matches(case, hit_fraction=args.hit, noise=0.05, lag_lo=LAG, lag_hi=LAG,
                                  seed=5, heads_per_draw=G)
    keep = [t[req, P % M].clone() for t in ring]                         # the slot a step overwrites
    # earlier replays left this step's own query there (a distance-0 candidate): make it a stranger
    keep[0] = torch.randn(keep[0].shape, device=dev).to(keep[0].dtype)
    scal = list(scalars(args, args.hit))
    scal[11] = 0                                                         # bench_mode off
    e = torch.empty(0)

    def launch():
        ext.mac_persistent_decode_bf16(
            case.q_post, case.q_pre, case.k, case.v, case.req_to_token, case.req_ids,
            case.past_lens, case.out_cache_loc, case.query_cache, case.attn_cache, case.lse_cache,
            out, lse, *ws, *scal, case.query_cache, e, e, e)
        for t, k in zip(ring, keep):
            t[req, P % M] = k

    for t, k in zip(ring, keep):
        t[req, P % M] = k
    ms, _ = time_graph(launch, max(10, min(args.steps, 50)), args.warmup)
    hits = ws[HEAD_HIT][:case.q_post.shape[0]].bool().cpu()
    ab = alg_bytes(ws, case.q_post.shape[0], args.hq, args.hkv, args.front_sink, args.capacity,
                   case.past_lens.cpu().tolist())
    for t, sv in zip(ring, saved):
        t[req[:, None], touched] = sv
    return {"us": ms * 1e3, "includes": "3 ring-slot restore copies per step",
            "planted_hit_heads": int(planted.sum()), "hit_heads": int(hits.sum()),
            "decisions_match_planted": bool(torch.equal(hits, planted)),
            "requested_gbs": ab["requested"] / (ms * 1e-3) / 1e9,
            "non_hit_groups": ab["non_hit_groups"]}


# --------------------------------------------------------------------------- parity on the timed tensors
def parity_sample(args, case, ws, out, lse, per_row_bytes, hq, hkv, front_sink, max_rows):
    """Checks the step that was just timed against the CPU oracle on a sample of
    its requests: the SAME tensors, copied to the host.  The sample holds rows of
    every kind the step has (a request with a full-attention group, one with a
    mixed group, all-hit requests); their K/V rows are gathered through the page
    table into a compact host pool, their ring rows are taken whole, and the
    oracle runs with the full batch's row indices (the synthetic decision hash
    depends on them) restricted to the sampled rows.  Returns the parity record
    and the oracle's wall time with the share of the step's bytes it covered."""
    import torch

    from mac_attention_b200 import workspace as W
    from oracle import mac_oracle as O

    N = case.q_post.shape[0]
    M = case.query_cache.shape[1]
    mode = ws[W.GROUP_MODE][:N].cpu()
    kinds = {"full": [], "mixed": [], "hit": []}
    for n in range(N):
        row = mode[n]
        kinds["mixed" if bool((row == 2).any()) else "full" if bool((row == 1).any()) else "hit"].append(n)
    rows = []
    quota = max(1, max_rows // 3)
    for k in ("full", "mixed", "hit"):
        rows += kinds[k][:quota]
    for k in ("hit", "full", "mixed"):           # fill up from whatever is left
        for n in kinds[k][quota:]:
            if len(rows) < max_rows:
                rows.append(n)
    rows = sorted(rows)[:max_rows]
    dev = case.q_post.device
    P = case.past_lens.cpu().tolist()
    req = case.req_ids.cpu().tolist()
    stride = max(P[n] + 1 for n in rows)
    r2t_sub = torch.zeros(len(rows), stride, dtype=torch.int32)
    req_sub = torch.zeros(N, dtype=torch.int32)
    ocl_sub = torch.zeros(N, dtype=case.out_cache_loc.dtype)
    k_parts, v_parts = [], []
    base = 0
    for i, n in enumerate(rows):
        toks = torch.cat([case.req_to_token[req[n], :P[n]].long(),
                          case.out_cache_loc[n:n + 1].long()])
        k_parts.append(case.k.index_select(0, toks).cpu())
        v_parts.append(case.v.index_select(0, toks).cpu())
        r2t_sub[i, :P[n]] = torch.arange(base, base + P[n], dtype=torch.int32)
        ocl_sub[n] = base + P[n]
        req_sub[n] = i
        base += P[n] + 1
    sel = torch.tensor([req[n] for n in rows], device=dev)
    gpu_ring = [t.index_select(0, sel).cpu() for t in (case.query_cache, case.attn_cache, case.lse_cache)]
    qc, ac, lc = (t.clone() for t in gpu_ring)
    mask = torch.zeros(N, dtype=torch.uint8)
    mask[rows] = 1
    cfg = O.DecodeConfig(max_context=MAX_CONTEXT, tile_tokens=TILE, match_tile_slots=MTS,
                         semantic_pos_ahead=SEM, front_sink_tokens=front_sink,
                         bench_mode=args.bench_mode, bench_hit_rate=args.hit,
                         bench_match_lag_mean=float(LAG), bench_seed=1)
    k_sub, v_sub = torch.cat(k_parts), torch.cat(v_parts)
    del k_parts, v_parts
    t0 = time.perf_counter()
    res = O.decode_step(case.q_post.cpu(), case.q_pre.cpu(), k_sub, v_sub, r2t_sub, req_sub,
                        case.past_lens.cpu()[:N].contiguous(), ocl_sub, qc, ac, lc, cfg,
                        row_mask=mask)
    oracle_s = time.perf_counter() - t0
    ridx = torch.tensor(rows)
    pairs = [(W.HEAD_HIT, res.head_hit), (W.HEAD_MATCH_SLOT, res.head_match_slot),
             (W.HEAD_MATCH_POS, res.head_match_pos), (W.HEAD_PREFIX_END, res.head_prefix_end),
             (W.HEAD_RECT_START, res.head_rect_start), (W.HEAD_NEW_END, res.head_new_end),
             (W.GROUP_RECT_BEGIN, res.group_rect_begin), (W.GROUP_MODE, res.group_mode)]
    decisions_equal = all(torch.equal(ws[i][:N].cpu()[ridx], ref[ridx]) for i, ref in pairs)
    got_out = out.float().cpu()[ridx]
    out_err = O.rel_l2(got_out, res.out_f32[ridx])
    slot = torch.tensor([P[n] % M for n in rows])
    ar = torch.arange(len(rows))
    ring_q_equal = bool(torch.equal(gpu_ring[0][ar, slot], qc[ar, slot]))
    ring_err = O.rel_l2(gpu_ring[1][ar, slot].float(), res.ring_o_f32[ridx])
    l_gpu, l_ref = lse.cpu()[ridx], res.lse[ridx]
    fin = torch.isfinite(l_ref)
    lse_err = float((l_gpu[fin] - l_ref[fin]).abs().max()) if bool(fin.any()) else 0.0
    rl_gpu, rl_ref = gpu_ring[2][ar, slot], lc[ar, slot]
    rfin = torch.isfinite(rl_ref)
    ring_lse_err = float((rl_gpu[rfin] - rl_ref[rfin]).abs().max()) if bool(rfin.any()) else 0.0
    parity = {
        "checked_against": "CPU oracle (oracle/mac_oracle.c) on the timed tensors copied to the host",
        "requests_checked": len(rows), "rows": rows,
        "rows_with_full_group": sum(n in kinds["full"] for n in rows),
        "rows_with_mixed_group": sum(n in kinds["mixed"] for n in rows),
        "all_hit_rows": sum(n in kinds["hit"] for n in rows),
        "decisions_equal": bool(decisions_equal), "out_rel_l2": out_err,
        "ring_query_rows_equal": ring_q_equal, "ring_rel_l2": ring_err,
        "lse_max_abs": lse_err, "ring_lse_max_abs": ring_lse_err,
        "finite_pattern_equal": bool(torch.equal(torch.isfinite(l_gpu), fin)
                                     and torch.equal(torch.isfinite(rl_gpu), rfin)),
        "tolerance": {"out_rel_l2": 1e-2, "ring_rel_l2": 1e-2, "lse_max_abs": 2e-2},
    }
    parity["ok"] = bool(decisions_equal and ring_q_equal and parity["finite_pattern_equal"]
                        and out_err <= 1e-2 and ring_err <= 1e-2 and lse_err <= 2e-2
                        and ring_lse_err <= 2e-2)
    share = sum(per_row_bytes[n] for n in rows) / max(1, sum(per_row_bytes))
    return parity, oracle_s, share


def cpu_baseline_from_sample(parity, oracle_s, share, args):
    """``cpu_baseline`` of the main line: the oracle's time on the parity sample,
    scaled to the whole step by the share of the step's bytes the sample holds."""
    from oracle import mac_oracle as O

    return {"value": oracle_s / max(share, 1e-9) * 1e6, "unit": "us",
            "cores": O.lib().mac_oracle_num_threads(), "kind": "port",
            "sample": f"{parity['requests_checked']} of {args.batch} requests of the timed step "
                      f"(rows {parity['rows']}: {parity['rows_with_full_group']} with a full-attention "
                      f"group, {parity['rows_with_mixed_group']} with a mixed group, "
                      f"{parity['all_hit_rows']} all-hit) = {share * 100:.1f} % of the step's bytes, "
                      f"{oracle_s:.3f} s on the host cores, scaled by bytes"}


def cpu_port_arm(args, steps, warmup):
    """The CPU restatement of the path (oracle port) timed on the host cores on
    the first requests of a step of the same shape; used only when the
    reference's CUDA kernel is not available to ``--impl reference``."""
    import torch  # noqa: F401

    from mac_attention_b200 import synth
    from oracle import mac_oracle as O

    ns = max(1, min(4, args.batch))
    case = synth.make_decode_case(batch=ns, ctx=args.ctx, hq=args.hq, hkv=args.hkv,
                                  capacity=args.capacity, page_size=args.page_size, seed=1000,
                                  device="cpu")
    cfg = O.DecodeConfig(max_context=MAX_CONTEXT, tile_tokens=TILE, match_tile_slots=MTS,
                         semantic_pos_ahead=SEM, front_sink_tokens=args.front_sink,
                         bench_mode=args.bench_mode, bench_hit_rate=args.hit,
                         bench_match_lag_mean=float(LAG), bench_seed=1)
    times = []
    for i in range(warmup + steps):
        c = case.clone() if i == 0 else case
        t0 = time.perf_counter()
        O.decode_step(c.q_post, c.q_pre, c.k, c.v, c.req_to_token, c.req_ids, c.past_lens,
                      c.out_cache_loc, c.query_cache, c.attn_cache, c.lse_cache, cfg)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    per_sample = sum(times) / len(times)
    scale = args.batch / ns
    return {"value": per_sample * scale * 1e6, "unit": "us", "cores": O.lib().mac_oracle_num_threads(),
            "kind": "port", "extrapolated": True, "factor": scale,
            "sample": f"{ns} of {args.batch} requests (all heads, full context {args.ctx}, hit "
                      f"{args.hit}), {per_sample:.3f} s per sample step, scaled x{scale:g}"}


# --------------------------------------------------------------------------- same-box GPU baselines
def gpu_baselines(args, case, ws, scal, out, lse, hq, hkv, budget_s=240.0):
    """FlashInfer full decode (CUDA-core and tensor-core decode paths) and the
    reference's own kernel (built for sm_100a from its source) on the tensors of
    the timed step.  An arm that cannot run reports why instead of a number."""
    import torch

    res = {}
    t_start = time.perf_counter()
    steps = max(5, min(args.steps, 20))
    for key, tc in (("flashinfer_us", False), ("flashinfer_tc_us", True)):
        if time.perf_counter() - t_start > budget_s:
            res[key] = "unavailable on this box: time budget of the baseline leg used up"
            continue
        try:
            ms, fi_out = bench_flashinfer(case, hq, hkv, args.page_size, steps, 3, use_tensor_cores=tc)
            res[key] = ms * 1e3
            del fi_out
        except Exception as exc:  # noqa: BLE001
            res[key] = f"unavailable on this box: {type(exc).__name__}: {str(exc)[:160]}"
        torch.cuda.empty_cache()
    nums = [v for v in (res.get("flashinfer_us"), res.get("flashinfer_tc_us")) if isinstance(v, float)]
    res["flashinfer_best_us"] = min(nums) if nums else None
    try:
        from oracle import build_ref

        ref_ext = build_ref.load_decode()
        if ref_ext is None:
            res["refkernel_us"] = "unavailable on this box: oracle/_ref holds no prebuilt reference kernel"
        else:
            keep = [t.clone() for t in (out, lse)]
            ms, _ = time_graph(make_launch(ref_ext, case, ws, scal, out, lse), steps, 3)
            res["refkernel_us"] = ms * 1e3
            out.copy_(keep[0]); lse.copy_(keep[1])
    except Exception as exc:  # noqa: BLE001
        res["refkernel_us"] = f"unavailable on this box: {type(exc).__name__}: {str(exc)[:160]}"
    res["what"] = ("same tensors as the timed step; FlashInfer BatchDecodeWithPagedKVCacheWrapper "
                   "(page 16, plan once, graph replay) with use_tensor_cores False / True; "
                   "refkernel = the reference's mac_persistent_decode_bf16 built for sm_100a")
    return res


# --------------------------------------------------------------------------- config 3
def config3_leg(args, dev, rank, world, dist, ext, peak_gbs):
    """BASELINE config 3: the Llama-3.1-70B attention shape (Hq 64 / Hkv 8, batch
    64, context 126976, hit 0.9) split by KV head over the ranks; every rank owns
    its KV-head slice of the pool and of the ring, no collective.  Strong
    scaling: the aggregate work is fixed."""
    import torch

    from mac_attention_b200 import make_decode_workspace, sharding

    hq_all, hkv_all, batch, ctx, hit = 64, 8, 64, 126976, 0.9
    if hkv_all % world != 0:
        return {"skipped": f"Hkv {hkv_all} does not split over {world} ranks"}
    q_sl, kv_sl = sharding.head_slices(hq_all, hkv_all, world, rank)
    hq, hkv = q_sl.stop - q_sl.start, kv_sl.stop - kv_sl.start
    case = build_case(args, dev, 3000 + rank, batch, ctx, hq, hkv)
    ws = make_decode_workspace(batch, hq, hkv, args.capacity, MAX_CONTEXT, TILE, MTS, SEM, 0,
                               device=dev, partial_dtype=torch.bfloat16)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(batch, hq, device=dev)
    scal = scalars(args, hit, front_sink=0)

    def barrier():
        if dist is not None:
            dist.barrier()

    ms, _ = time_graph(make_launch(ext, case, ws, scal, out, lse), args.steps, args.warmup, barrier)
    ab = alg_bytes(ws, batch, hq, hkv, 0, args.capacity, case.past_lens.cpu().tolist())
    t = torch.tensor([ms, float(ab["requested"]), float(ab["total"])], device=dev, dtype=torch.float64)
    tmax = t.clone()
    if dist is not None:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    ms_max = float(tmax[0])
    req_all, alg_all = float(t[1]), float(t[2])
    del case, ws, out, lse
    torch.cuda.empty_cache()
    return {"workload": f"Hq{hq_all}/Hkv{hkv_all}/D128 split by KV head over {world} GPU(s), batch "
                        f"{batch}, context {ctx}, hit {hit}, ring M={args.capacity}",
            "us": ms_max * 1e3, "scaling": "strong", "hq_per_rank": hq, "hkv_per_rank": hkv,
            "requested_gbs_aggregate": req_all / (ms_max * 1e-3) / 1e9,
            "alg_gbs_aggregate": alg_all / (ms_max * 1e-3) / 1e9,
            "frac": req_all / (ms_max * 1e-3) / 1e9 / (peak_gbs * world),
            "frac_of": "requested bytes / (measured copy bandwidth x ranks)",
            "non_hit_groups_rank0": ab["non_hit_groups"]}


# --------------------------------------------------------------------------- this library's arm
def dist_setup():
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    saved_stdout = None
    if world > 1:
        import torch.distributed as dist_mod

        # libraries print banners on fd 1 during set-up; keep stdout for the JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    return rank, local_rank, world, dev, dist, saved_stdout


def dist_finish(dist, saved_stdout):
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if saved_stdout is not None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)


def measured_peak():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        return float(json.loads(pk.read_text()).get("hbm_gbs", 6650.0)), \
            "MEASURED_PEAKS.json hbm_gbs (of measured)"
    return 6650.0, "6650 GB/s (of fallback)"


def run_ours(args):
    import torch

    rank, local_rank, world, dev, dist, saved_stdout = dist_setup()

    from mac_attention_b200 import load_mac_persistent_decode_extension, make_decode_workspace
    from mac_attention_b200 import ops, sharding

    ext = load_mac_persistent_decode_extension()
    hq, hkv, batch = args.hq, args.hkv, args.batch
    if args.shard == "kv_head" and world > 1:
        q_sl, kv_sl = sharding.head_slices(hq, hkv, world, rank)
        hq, hkv = q_sl.stop - q_sl.start, kv_sl.stop - kv_sl.start
        seed = 1000
    else:
        seed = 1000 + rank
    case = build_case(args, dev, seed, batch, args.ctx, hq, hkv)
    ws = make_decode_workspace(batch, hq, hkv, args.capacity, MAX_CONTEXT, TILE, MTS, SEM,
                               args.front_sink, device=dev, partial_dtype=torch.bfloat16)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(batch, hq, device=dev)
    scal = scalars(args, args.hit)
    launch = make_launch(ext, case, ws, scal, out, lse)

    def barrier():
        if dist is not None:
            dist.barrier()

    profiler_range = os.environ.get("MAC_BENCH_PROFILER_RANGE") == "1"
    if profiler_range:  # lets a profiler attach to the measured launches only
        torch.cuda.profiler.start()
    with ClockSampler(local_rank) as clk:
        ms, graph = time_graph(launch, args.steps, args.warmup, barrier)
    clocks = clk.summary()
    if profiler_range:   # the side legs below are not part of the launch list
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    stability = replay_blocks(graph, args.steps)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t)
    ab = alg_bytes(ws, batch, hq, hkv, args.front_sink, args.capacity,
                   case.past_lens.cpu().tolist())
    bytes_all = torch.tensor([float(ab["requested"]), float(ab["total"])], device=dev,
                             dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(bytes_all, op=dist.ReduceOp.SUM)
    status = ops.query_status(dev)

    # the timed tensors against the CPU oracle (rank 0), which also gives the CPU baseline
    parity = cpu_base = None
    if rank == 0 and not args.no_cpu_baseline:
        try:
            parity, oracle_s, share = parity_sample(args, case, ws, out, lse, ab["per_row"], hq, hkv,
                                                    args.front_sink, args.parity_requests)
            cpu_base = cpu_baseline_from_sample(parity, oracle_s, share, args)
        except Exception as exc:  # reported, never fatal for the main line
            parity = {"ok": False, "error": f"{type(exc).__name__}: {exc}"[:300]}
    barrier()

    # the same step with decisions from the REAL match scan (synthetic-decision mode
    # off): ring rows planted so that about the same fraction of KV groups hit at the
    # same lag; the ring slot the step overwrites is put back inside the graph, else
    # the row written by one replay is a distance-0 match for the next
    real_scan = None
    if world == 1 and args.bench_mode != 0:
        try:
            real_scan = time_real_scan(args, ext, case, ws, out, lse, dev)
        except Exception as exc:  # reported, never fatal for the main line
            real_scan = {"error": f"{type(exc).__name__}: {exc}"[:200]}

    n_e2e = max(5, min(args.steps, 50))
    e2e_ms, h2d, d2h, launches_e2e, e2e_parts = time_e2e(
        ext, case, ws, scal, out, lse, dev, n_e2e, barrier,
        count_launches=lambda: ops.launch_info(dev)["kernel_launches"])
    te = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te)

    baselines = None
    if world == 1 and not args.no_gpu_baselines:
        baselines = gpu_baselines(args, case, ws, scal, out, lse, hq, hkv)

    info = ops.launch_info(dev)
    peak_gbs, peak_source = measured_peak()
    del case, ws, graph, launch
    torch.cuda.empty_cache()
    config3 = None
    if not args.no_config3 and args.shard == "request":
        try:
            config3 = config3_leg(args, dev, rank, world, dist, ext, peak_gbs)
        except Exception as exc:  # reported, never fatal for the main line
            config3 = {"error": f"{type(exc).__name__}: {exc}"[:200]}

    requested = ab["requested"]
    achieved = requested / (ms * 1e-3) / 1e9
    line = {
        "metric": METRIC,
        "value": ms_max * 1e3,
        "unit": "us",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": ms_max,
        "higher_is_better": False,
        "scaling": "weak" if args.shard == "request" else "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args, world),
        "non_hit_groups": ab["non_hit_groups"], "full_attention_groups": ab["full_groups"],
        "grid": info["last_grid"], "regs": info["regs_per_thread"],
        "hbm_gbs": float(bytes_all[0]) / (ms_max * 1e-3) / 1e9,
        "hbm_gbs_full_row_convention": float(bytes_all[1]) / (ms_max * 1e-3) / 1e9,
        "request_steps_per_s": world * batch / (ms_max * 1e-3),
        # five more blocks of `steps` replays of the same graph on this rank, after the timed one
        "stability": stability,
        "e2e": {"value": e2e_ms * 1e3, "unit": "us", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "h2d_copies_per_step": 1, "d2h_copies_per_step": 0,
                # the output is written by the kernel into the caller's pinned host buffer;
                # beside it: the variant with a D2H copy after the kernel, and the two copies
                # timed alone (back to back, CUDA events)
                **e2e_parts},
        "gpu_launches": args.steps,
        "gpu_launches_e2e_region": int(launches_e2e),
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                   "reasons": clocks["reasons"]},
        # achieved = bytes this kernel asks the memory system for (K/V rows, the
        # 128-byte probe half of every scanned ring row, states, outputs) per
        # launch / CUDA-event time of one launch; DRAM traffic measured by ncu
        # on smaller captures is 1.02x that and grows in proportion (profiles/).
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                     "frac": achieved / peak_gbs, "traffic": int(requested * NCU_TRAFFIC_RATIO),
                     "traffic_gbs": requested * NCU_TRAFFIC_RATIO / (ms * 1e-3) / 1e9,
                     "requested_bytes_per_launch": requested,
                     "kernel": "mac_decode_persistent_kernel",
                     "alg_bytes_full_row_convention": ab["total"],
                     "alg_gbs_full_row_convention": ab["total"] / (ms * 1e-3) / 1e9,
                     "kv_bytes": ab["kv"], "scan_bytes_full_rows": ab["scan"],
                     "peak_source": peak_source},
        "parity": parity,
        "gpu_baselines": baselines,
        "config3": config3,
        "device_status": status, "real_scan": real_scan,
    }
    if cpu_base is not None:
        line["cpu_baseline"] = cpu_base
    dist_finish(dist, saved_stdout)
    if rank == 0:
        print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- reference arm
def run_reference_arm(args):
    """``--impl reference``: the reference's own decode kernel, compiled for
    sm_100a from its unmodified source by ``oracle/build_ref.py`` (prebuilt into
    ``oracle/_ref``), through its own operator on the same workload, timed the
    same way (graph replay, CUDA events, max over ranks; ``e2e`` with the same
    host copies).  The reference has no CPU implementation of the path; when
    its kernel cannot be loaded the CPU oracle port is timed instead and the
    line says so."""
    import torch

    from oracle import build_ref

    ref_ext = None
    why = ""
    try:
        ref_ext = build_ref.load_decode()
        if ref_ext is None:
            why = "oracle/_ref holds no prebuilt reference kernel"
    except Exception as exc:  # noqa: BLE001
        why = f"{type(exc).__name__}: {str(exc)[:160]}"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if ref_ext is None or not torch.cuda.is_available():
        if int(os.environ.get("RANK", "0")) != 0:
            return
        cb = cpu_port_arm(args, steps=max(1, min(args.steps, 5)), warmup=1)
        line = {
            "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "us",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": cb["value"] / 1e3, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": workload_config(args, world), "extrapolated": True,
            "reference_kind": f"CPU oracle port (reference kernel unavailable: {why})",
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "us", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return

    rank, local_rank, world, dev, dist, saved_stdout = dist_setup()
    from mac_attention_b200 import make_decode_workspace

    hq, hkv, batch = args.hq, args.hkv, args.batch
    case = build_case(args, dev, 1000 + rank, batch, args.ctx, hq, hkv)
    ws = make_decode_workspace(batch, hq, hkv, args.capacity, MAX_CONTEXT, TILE, MTS, SEM,
                               args.front_sink, device=dev, partial_dtype=torch.bfloat16)
    out = torch.empty_like(case.q_post)
    lse = torch.empty(batch, hq, device=dev)
    scal = scalars(args, args.hit)

    def barrier():
        if dist is not None:
            dist.barrier()

    with ClockSampler(local_rank) as clk:
        ms, graph = time_graph(make_launch(ref_ext, case, ws, scal, out, lse), args.steps,
                               args.warmup, barrier)
    clocks = clk.summary()
    ab = alg_bytes(ws, batch, hq, hkv, args.front_sink, args.capacity, case.past_lens.cpu().tolist())
    e2e_ms, h2d, d2h, _, _ = time_e2e(ref_ext, case, ws, scal, out, lse, dev,
                                      max(5, min(args.steps, 50)), barrier, host_out=False)
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_max = float(t[0]), float(t[1])
    peak_gbs, peak_source = measured_peak()
    line = {
        "impl": "reference", "metric": METRIC, "value": ms_max * 1e3, "unit": "us",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_max, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
        "reference_kind": "the reference's mac_persistent_decode_bf16 CUDA kernel, built for sm_100a "
                          "from its unmodified source (oracle/_ref), its own operator and workspace",
        "non_hit_groups": ab["non_hit_groups"], "full_attention_groups": ab["full_groups"],
        "hbm_gbs_full_row_convention": ab["total"] / (ms * 1e-3) / 1e9,
        "e2e": {"value": e2e_max * 1e3, "unit": "us", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "h2d_copies_per_step": 1},
        "gpu_launches": args.steps,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"],
                   "reasons": clocks["reasons"]},
        "peak": peak_gbs, "peak_source": peak_source,
    }
    dist_finish(dist, saved_stdout)
    if rank == 0:
        print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- sweep
def bench_flashinfer(case, hq, hkv, page_size, steps, warmup, use_tensor_cores=False):
    """FlashInfer full decode over the same paged KV (plan once, capture run, time replay).
    ``use_tensor_cores`` selects its tensor-core decode path (the prefill template run on
    decode queries) instead of the CUDA-core decode kernel the reference's harness uses."""
    import torch
    import flashinfer

    batch = case.q_post.shape[0]
    dev = case.q_post.device
    kv_lens = (case.past_lens + 1).cpu()
    pages = (kv_lens + page_size - 1) // page_size
    indptr = torch.zeros(batch + 1, dtype=torch.int32)
    indptr[1:] = torch.cumsum(pages, 0)
    idx = []
    r2t = case.req_to_token.cpu()
    ocl = case.out_cache_loc.cpu()
    for n in range(batch):
        toks = torch.cat([r2t[int(case.req_ids[n]), :int(kv_lens[n]) - 1].long(), ocl[n:n + 1].long()])
        idx.append((toks[::page_size] // page_size).to(torch.int32))
    indices = torch.cat(idx).to(dev)
    last = ((kv_lens - 1) % page_size + 1).to(torch.int32).to(dev)
    indptr = indptr.to(dev)
    kc = case.k.view(-1, page_size, hkv, DIM)
    vc = case.v.view(-1, page_size, hkv, DIM)
    wsb = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
    wrapper = flashinfer.decode.BatchDecodeWithPagedKVCacheWrapper(
        wsb, kv_layout="NHD", use_cuda_graph=True, use_tensor_cores=use_tensor_cores,
        paged_kv_indptr_buffer=indptr,
        paged_kv_indices_buffer=indices, paged_kv_last_page_len_buffer=last)
    wrapper.plan(indptr, indices, last, hq, hkv, DIM, page_size, q_data_type=torch.bfloat16,
                 kv_data_type=torch.bfloat16, sm_scale=1.0 / math.sqrt(DIM))
    out = torch.empty_like(case.q_post)
    lse = torch.empty(batch, hq, device=dev, dtype=torch.float32)

    def launch():
        wrapper.run(case.q_post, (kc, vc), out=out, lse=lse, return_lse=True)

    ms, _ = time_graph(launch, steps, warmup)
    return ms, out


def run_sweep(args):
    import torch

    from mac_attention_b200 import load_mac_persistent_decode_extension, make_decode_workspace
    from mac_attention_b200 import ops

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ext = load_mac_persistent_decode_extension()
    if args.matched_prefix:
        # the operator reads this switch from the environment at every call, like the
        # reference's own launcher knobs; the reference kernel ignores it and demotes
        os.environ["MAC_B200_BENCH_LONG_BAND"] = "1"
    baselines = [b for b in args.baselines.split(",") if b]
    ref_ext = None
    if "refkernel" in baselines:
        from oracle import build_ref

        ref_ext = build_ref.load_decode()
    rows = []
    hits = [0.0, 0.25, 0.5, 0.75, 0.9, 1.0]
    shapes = [(b, c) for b in (1, 16, 64) for c in (32768, 65536, 126976)]
    if os.environ.get("MAC_SWEEP_SHAPES"):
        shapes = [tuple(int(x) for x in s.split("x")) for s in os.environ["MAC_SWEEP_SHAPES"].split(",")]
    if os.environ.get("MAC_SWEEP_HITS"):
        hits = [float(x) for x in os.environ["MAC_SWEEP_HITS"].split(",")]
    for batch, ctx in shapes:
        case = build_case(args, dev, 1000, batch, ctx, args.hq, args.hkv)
        ws = make_decode_workspace(batch, args.hq, args.hkv, args.capacity, MAX_CONTEXT, TILE, MTS,
                                   SEM, args.front_sink, device=dev, partial_dtype=torch.bfloat16)
        out = torch.empty_like(case.q_post)
        lse = torch.empty(batch, args.hq, device=dev)
        fi_ms = fi_tc_ms = None
        for name, tc in (("flashinfer", False), ("flashinfer_tc", True)):
            if name not in baselines:
                continue
            try:
                v, _ = bench_flashinfer(case, args.hq, args.hkv, args.page_size, args.steps,
                                        args.warmup, use_tensor_cores=tc)
            except Exception as exc:  # noqa: BLE001
                v = f"unavailable on this box: {type(exc).__name__}: {str(exc)[:200]}"
            if tc:
                fi_tc_ms = v
            else:
                fi_ms = v
        for hit in hits:
            scal = scalars(args, hit)
            ms, _ = time_graph(make_launch(ext, case, ws, scal, out, lse), args.steps, args.warmup)
            ab = alg_bytes(ws, batch, args.hq, args.hkv, args.front_sink, args.capacity,
                           case.past_lens.cpu().tolist())
            # one eager launch with phase timestamps (ns) for the breakdown
            make_launch(ext, case, ws, scalars(args, hit, debug=2), out, lse)()
            torch.cuda.synchronize()
            ph = ws[29].cpu().tolist()
            row = dict(batch=batch, ctx=ctx, hit=hit, mac_us=ms * 1e3,
                       matched_prefix=args.matched_prefix or None,
                       requested_gbs=ab["requested"] / (ms * 1e-3) / 1e9,
                       phase_us=dict(scan=(ph[1] - ph[0]) / 1e3, classify=(ph[2] - ph[1]) / 1e3,
                                     attend_cta0=(ph[3] - ph[2]) / 1e3),
                       alg_gbs=ab["total"] / (ms * 1e-3) / 1e9, kv_gb=ab["kv"] / 1e9,
                       non_hit_groups=ab["non_hit_groups"], full_groups=ab["full_groups"],
                       flashinfer_us=(fi_ms * 1e3 if isinstance(fi_ms, float) else fi_ms),
                       flashinfer_tc_us=(fi_tc_ms * 1e3 if isinstance(fi_tc_ms, float) else fi_tc_ms))
            if ref_ext is not None:
                try:
                    rms, _ = time_graph(make_launch(ref_ext, case, ws, scal, out, lse), args.steps,
                                        args.warmup)
                    row["refkernel_us"] = rms * 1e3
                except Exception as exc:  # noqa: BLE001
                    row["refkernel_us"] = f"failed: {str(exc)[:120]}"
            rows.append(row)
            print(json.dumps(row), flush=True)
        del case, ws
        torch.cuda.empty_cache()
    if args.sweep_out:
        Path(args.sweep_out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.sweep_out).write_text(json.dumps(dict(rows=rows, status=ops.query_status(dev),
                                                        hq=args.hq, hkv=args.hkv,
                                                        front_sink=args.front_sink), indent=1))


def run_config4(args):
    """Mixed serving step (contexts uniform in [8K,127K], 20 % of the requests not
    ready, 10 % with a stale cache epoch, the rest hitting at 0.8) and the prefill
    ring build from 32K-token prompts with q_post_cache supplied."""
    import torch

    from mac_attention_b200 import (load_mac_persistent_decode_extension,
                                    load_mac_prefill_update_cache_extension, make_decode_workspace)
    from mac_attention_b200 import ops, synth

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ext = load_mac_persistent_decode_extension()
    pre = load_mac_prefill_update_cache_extension()
    batch = args.batch
    rows = []
    if args.config4_part == "all":
        g = torch.Generator().manual_seed(4)
        ctxs = torch.randint(8192, 126977, (batch,), generator=g).tolist()
        case = synth.make_decode_case(batch=batch, ctx=0, ctx_list=ctxs, hq=args.hq, hkv=args.hkv,
                                      capacity=args.capacity, page_size=args.page_size, seed=44,
                                      device=dev)
        synth.add_readiness_gate(case, not_ready_fraction=0.2, stale_fraction=0.1, seed=4)
        ws = make_decode_workspace(batch, args.hq, args.hkv, args.capacity, MAX_CONTEXT, TILE, MTS, SEM,
                                   0, device=dev, partial_dtype=torch.bfloat16)
        out = torch.empty_like(case.q_post)
        lse = torch.empty(batch, args.hq, device=dev)
        scal = scalars(args, 0.8)

        def launch():
            ext.mac_persistent_decode_bf16(
                case.q_post, case.q_pre, case.k, case.v, case.req_to_token, case.req_ids,
                case.past_lens, case.out_cache_loc, case.query_cache, case.attn_cache, case.lse_cache,
                out, lse, *ws, *scal, case.query_cache, case.cache_ready, case.cache_epoch,
                case.request_epoch)

        ms, _ = time_graph(launch, args.steps, args.warmup)
        ab = alg_bytes(ws, batch, args.hq, args.hkv, 0, args.capacity, case.past_lens.cpu().tolist())
        gated = int(case.meta["gated_off"].sum())
        # the scan only runs for requests that pass the gate
        scan = sum(min(args.capacity, c) for c, off in zip(ctxs, case.meta["gated_off"].tolist())
                   if not off) * args.hq * 256
        total = ab["total"] - ab["scan"] + scan
        rows = [dict(kind="mixed_decode_step", batch=batch, ctx_min=min(ctxs), ctx_max=max(ctxs),
                     gated_off_requests=gated, hit=0.8, us=ms * 1e3, alg_gbs=total / (ms * 1e-3) / 1e9,
                     kv_gb=ab["kv"] / 1e9, non_hit_groups=ab["non_hit_groups"],
                     full_groups=ab["full_groups"])]
        print(json.dumps(rows[-1]), flush=True)
        del case, ws
        torch.cuda.empty_cache()

    # prefill ring build: 32K-token prompts, last M rows kept, q_post_cache rows stamped
    H, D, M, plen = args.hq, DIM, args.capacity, args.prompt_len
    R = batch
    qc = torch.zeros(R, M, H, D, device=dev, dtype=torch.bfloat16)
    ac = torch.zeros_like(qc)
    lc = torch.zeros(R, M, H, device=dev)
    qpc = torch.zeros_like(qc)
    src_q = torch.empty(batch * plen, H, D, device=dev, dtype=torch.bfloat16)
    src_a = torch.empty_like(src_q)
    for t in (src_q, src_a):
        for r0 in range(0, t.shape[0], 1 << 16):
            t[r0:r0 + (1 << 16)].normal_()
    src_l = torch.randn(batch * plen, H, device=dev)
    req_ids = torch.arange(batch, device=dev, dtype=torch.int32)
    offsets = (torch.arange(batch + 1, device=dev, dtype=torch.int32) * plen).contiguous()
    lens = torch.full((batch,), plen, device=dev, dtype=torch.int32)
    rl = torch.zeros(batch, device=dev, dtype=torch.int32)   # by-batch: read-only lengths

    def prefill():
        pre.mac_prefill_update_cache(qc, ac, lc, rl, req_ids, src_q, src_a, src_l, offsets, lens,
                                     M, H, D, qpc)

    pms, _ = time_graph(prefill, args.steps, args.warmup)
    ref_us = {}
    want_ref = "refkernel" in args.baselines
    if want_ref:
        from oracle import build_ref

        rpre = build_ref.load_prefill()
        if rpre is not None:
            rms_, _ = time_graph(lambda: rpre.mac_prefill_update_cache(
                qc, ac, lc, rl, req_ids, src_q, src_a, src_l, offsets, lens, M, H, D, qpc),
                args.steps, args.warmup)
            ref_us["prefill"] = rms_ * 1e3
    keep = min(plen, M)
    pbytes = batch * keep * (2 * (2 * H * 256 + H * 4) + H * 256)
    rows.append(dict(kind="prefill_update_cache", batch=batch, prompt_len=plen, capacity=M,
                     us=pms * 1e3, alg_gbs=pbytes / (pms * 1e-3) / 1e9, alg_bytes=pbytes,
                     refkernel_us=ref_us.get("prefill")))
    print(json.dumps(rows[-1]), flush=True)

    # the same ring build from the un-downdated prefill outputs: one pass
    # (band-LSE scale + downdate + ring write + ready mark) against the hook's
    # sequence of operators, which downdates every prompt row
    band_a = torch.empty_like(src_q)
    for r0 in range(0, band_a.shape[0], 1 << 16):
        band_a[r0:r0 + (1 << 16)].normal_()
    full_l = src_l + 8
    band_l2 = (full_l - torch.rand_like(full_l) * 4 - 0.1) / math.log(2.0)   # log2-domain producer
    ready = torch.zeros(R, device=dev, dtype=torch.bool)
    cache_epoch = torch.full((R,), -1, device=dev, dtype=torch.int64)
    request_epoch = torch.zeros(R, device=dev, dtype=torch.int64)

    def build_one_pass():
        pre.mac_prefill_downdate_update_cache(
            qc, ac, lc, rl, req_ids, src_q, src_a, full_l, band_a, band_l2, offsets, lens, M, H, D,
            qpc, band_lse_scale=math.log(2.0), ready=ready, cache_epoch=cache_epoch,
            request_epoch=request_epoch)

    bms, _ = time_graph(build_one_pass, args.steps, args.warmup)
    from mac_attention_b200 import load_mac_merge_downdate_cache_extension as _load_dd

    def sequence(dd_mod, pre_mod):
        band_l = band_l2 * math.log(2.0)
        dd_mod.mac_update_then_downdate_bf16_inplace(src_a, full_l, band_a, band_l)
        pre_mod.mac_prefill_update_cache(qc, ac, lc, rl, req_ids, src_q, band_a, band_l, offsets,
                                         lens, M, H, D, qpc)
        pre_mod.mac_mark_persistent_ready(ready, cache_epoch, request_epoch, req_ids)

    few = max(3, min(args.steps, 10))
    sms, _ = time_graph(lambda: sequence(_load_dd(), pre), few, 3)
    if want_ref:
        rdd_, rpre_ = build_ref.load_downdate(), build_ref.load_prefill()
        if rdd_ is not None and rpre_ is not None:
            rms_, _ = time_graph(lambda: sequence(rdd_, rpre_), few, 3)
            ref_us["build_sequence"] = rms_ * 1e3
    bbytes = batch * keep * H * (3 * 256 + 8 + 3 * 256 + 4)
    rows.append(dict(kind="prefill_downdate_update_cache (one pass)", batch=batch, prompt_len=plen,
                     capacity=M, us=bms * 1e3, alg_gbs=bbytes / (bms * 1e-3) / 1e9,
                     alg_bytes=bbytes, operator_sequence_us=sms * 1e3,
                     refkernel_sequence_us=ref_us.get("build_sequence")))
    print(json.dumps(rows[-1]), flush=True)
    # sink-exclusive rows (F = 128): the same pass plus each row's attention over
    # the sink tokens, computed in the kernel from q_post and the paged K/V
    Fs = int(os.environ.get("MAC_BENCH_SINK_F", "128"))   # sink size of the sink-exclusive leg
    q_post_rows = torch.empty_like(src_q)
    for r0 in range(0, q_post_rows.shape[0], 1 << 16):
        q_post_rows[r0:r0 + (1 << 16)].normal_()
    pool_k = torch.randn(batch * Fs, args.hkv, D, device=dev).to(torch.bfloat16)
    pool_v = torch.randn(batch * Fs, args.hkv, D, device=dev).to(torch.bfloat16)
    r2t = torch.arange(batch * Fs, device=dev, dtype=torch.int32).view(batch, Fs).contiguous()

    def build_sink_exclusive():
        pre.mac_prefill_downdate_update_cache(
            qc, ac, lc, rl, req_ids, src_q, src_a, full_l, band_a, band_l2, offsets, lens, M, H, D,
            qpc, band_lse_scale=math.log(2.0), sink_mode=ops.SINK_EXCLUDE, ready=ready,
            cache_epoch=cache_epoch, request_epoch=request_epoch, q_post=q_post_rows,
            k_buffer=pool_k, v_buffer=pool_v, req_to_token=r2t, front_sink_tokens=Fs,
            semantic_pos_ahead=SEM)

    xms, _ = time_graph(build_sink_exclusive, args.steps, args.warmup)
    xbytes = bbytes + batch * keep * H * 256
    xflops = 4.0 * batch * keep * H * Fs * D
    rows.append(dict(kind=f"prefill_downdate_update_cache (sink-exclusive, F={Fs})", batch=batch,
                     prompt_len=plen, capacity=M, us=xms * 1e3,
                     alg_gbs=xbytes / (xms * 1e-3) / 1e9, alg_bytes=xbytes,
                     sink_attention_tflops=xflops / (xms * 1e-3) / 1e12))
    print(json.dumps(rows[-1]), flush=True)
    del src_q, src_a, src_l, qc, ac, lc, qpc, band_a, full_l, band_l2, q_post_rows, pool_k, pool_v
    torch.cuda.empty_cache()

    if args.config4_part == "prefill":
        write_config4(args, rows, ops.query_status(dev))
        return
    # the producer of the prefill rows: downdate of the last M rows of every prompt
    from mac_attention_b200 import (load_mac_decode_rope_preserve_extension,
                                    load_mac_merge_downdate_cache_extension)

    dd = load_mac_merge_downdate_cache_extension()
    rows_dd = batch * keep
    o_full = torch.randn(rows_dd, H, D, device=dev).to(torch.bfloat16)
    o_win = torch.randn(rows_dd, H, D, device=dev).to(torch.bfloat16)
    l_full = torch.randn(rows_dd, H, device=dev) + 8
    l_win0 = l_full - torch.rand(rows_dd, H, device=dev) * 4 - 0.1
    l_win = l_win0.clone()

    def downdate():
        dd.mac_update_then_downdate_bf16_inplace(o_full, l_full, o_win, l_win)

    dms, _ = time_graph(downdate, args.steps, args.warmup)
    if want_ref:
        rdd = build_ref.load_downdate()
        if rdd is not None:
            rms_, _ = time_graph(lambda: rdd.mac_update_then_downdate_bf16_inplace(
                o_full, l_full, o_win, l_win), args.steps, args.warmup)
            ref_us["downdate"] = rms_ * 1e3
    dbytes = rows_dd * H * (3 * D * 2 + 3 * 4)
    rows.append(dict(kind="update_then_downdate", rows=rows_dd * H, us=dms * 1e3,
                     alg_gbs=dbytes / (dms * 1e-3) / 1e9, alg_bytes=dbytes,
                     refkernel_us=ref_us.get("downdate")))
    print(json.dumps(rows[-1]), flush=True)
    del o_full, o_win, l_full, l_win, l_win0
    torch.cuda.empty_cache()

    # the step before the decode path: RoPE + q preserve + KV write for the batch
    rp = load_mac_decode_rope_preserve_extension()
    qkv = torch.randn(batch, (args.hq + 2 * args.hkv) * D, device=dev).to(torch.bfloat16)
    q, k, v = (qkv[:, :args.hq * D], qkv[:, args.hq * D:(args.hq + args.hkv) * D],
               qkv[:, (args.hq + args.hkv) * D:])
    q_pre = torch.empty(batch, args.hq, D, device=dev, dtype=torch.bfloat16)
    pool = torch.zeros(1 << 16, args.hkv, D, device=dev, dtype=torch.bfloat16)
    pool_v = torch.zeros_like(pool)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=dev).float() / D))
    ang = torch.arange(131072, device=dev).float()[:, None] * inv[None, :]
    cache = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous()
    positions = torch.randint(8192, 126977, (batch,), device=dev)
    locs = torch.randperm(1 << 16, device=dev)[:batch]

    def rope():
        rp.mac_decode_rope_preserve_q_bf16(q, k, v, q_pre, pool, pool_v, cache, positions, locs, D,
                                           True)

    rms, _ = time_graph(rope, args.steps, args.warmup)
    if want_ref:
        rrp = build_ref.load_rope()
        if rrp is not None:
            rms_, _ = time_graph(lambda: rrp.mac_decode_rope_preserve_q_bf16(
                q, k, v, q_pre, pool, pool_v, cache, positions, locs, D, True),
                args.steps, args.warmup)
            ref_us["rope"] = rms_ * 1e3
    rbytes = batch * ((args.hq * 3 + args.hkv * 5) * D * 2 + D * 4)
    rows.append(dict(kind="decode_rope_preserve", batch=batch, us=rms * 1e3,
                     alg_gbs=rbytes / (rms * 1e-3) / 1e9, alg_bytes=rbytes,
                     refkernel_us=ref_us.get("rope")))
    print(json.dumps(rows[-1]), flush=True)
    write_config4(args, rows, ops.query_status(dev))


def write_config4(args, rows, status):
    if args.config4_out:
        Path(args.config4_out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.config4_out).write_text(json.dumps(dict(rows=rows, status=status), indent=1))



def main():
    args = parse_args()
    if args.config4:
        run_config4(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.sweep:
        run_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
