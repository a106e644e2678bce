#!/usr/bin/env python
"""Paged-decode benchmark: tokens/s and KV-read HBM bandwidth at Llama-3-8B geometry.

One step = one decode step of the whole batch through all layers: per layer one head-major KV
store of the new token plus paged GQA attention over the whole context, each layer on its own
KV pool.  Default workload (N = 1): batch 256, every context 4096 tokens, 32 query / 8 KV heads,
head_dim 128, KV block 128 tokens, pool of batch*32 blocks + 10 % spare, shuffled block tables,
bf16, 32 layers.  With N > 1 the KV heads are sharded over the ranks (tensor parallel) and the
attention output is gathered along the last dimension (strong scaling: the batch is fixed).

Inputs are synthetic (seeded); pool contents are N(0,1) bf16.  The pools together are far
larger than L2 (4.7 GB per layer), so consecutive launches never hit in cache.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python bench.py --impl reference          # the CPU restatement of the reference on host cores
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "paged_decode_tokens_per_s"
# DRAM bytes moved per algorithmic KV byte by the attention kernel: (dram__bytes_read.sum +
# dram__bytes_write.sum) of one ncu capture on a batch-128 launch; traffic is one pass over the
# visible K/V rows, so it is scaled to the benchmark launch by its KV bytes.
TRAFFIC_PER_KV_BYTE = 1.0037
TRAFFIC_SOURCE = "profiles/paged_attn_kernel_decode_b128_ctx4096_ncu_full.md, scaled by KV bytes"
GEOM = dict(batch=256, ctx=4096, q_heads=32, kv_heads=8, head_dim=128, block=128, layers=32)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=GEOM["layers"], help="for experiments only; 32 is the workload")
    ap.add_argument("--batch", type=int, default=GEOM["batch"], help="for experiments only")
    ap.add_argument("--ctx", type=int, default=GEOM["ctx"], help="for experiments only")
    ap.add_argument("--cpu-seqs", type=int, default=64, help="sequences in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's CPU path on a bounded sample
# --------------------------------------------------------------------------------------------
def cpu_case(args, n_seqs):
    from tests import cases
    g = GEOM
    blocks = n_seqs * (args.ctx // g["block"]) + 4
    return cases.decode_case(n_seqs, g["q_heads"], g["kv_heads"], g["head_dim"], g["block"], blocks,
                             [args.ctx] * n_seqs, seed=20261102)


def cpu_pass(case):
    """Store + attend for the sample's sequences of ONE layer on the host cores (all threads):
    seconds per (sequence, layer)."""
    import oracle
    g = GEOM
    pool = case.pool.clone()
    t0 = time.perf_counter()
    oracle.kv_store_head_major(pool, case.k, case.v, case.locations)
    kp, vp = oracle.pool_views(pool)
    oracle.direct_bf16_pv(case.q, kp, vp, case.requests, case.positions, case.mapping, g["q_heads"],
                          g["kv_heads"], g["head_dim"], case.scale)
    return (time.perf_counter() - t0) / case.q.size(0)


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the path (its Python restatement
    in oracle/, all host threads), each step one bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = args.cpu_seqs
    case = cpu_case(args, n)
    for _ in range(min(args.warmup, 2)):
        cpu_pass(case)
    t0 = time.perf_counter()
    per = [cpu_pass(case) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    sec_per_seq_layer = statistics.mean(per)
    value = 1.0 / (sec_per_seq_layer * args.layers)          # tokens/s of the full workload
    sample = f"{n} of {args.batch} sequences x 1 of {args.layers} layers per step, scaled linearly"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_seq_layer * args.batch * args.layers * 1e3,
            "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(args, 1),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": wall}
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    g = GEOM
    return {"workload": f"Llama-3-8B-geometry paged decode: batch {args.batch}, ctx {args.ctx}, "
                        f"{g['q_heads']}q/{g['kv_heads']}kv heads, head_dim {g['head_dim']}, block {g['block']}, "
                        f"{args.layers} layers (independent pools), KV store + attention per layer",
            "parallelism": f"tp{world} (KV heads sharded, output gathered along the last dim)" if world > 1 else "single GPU",
            "cache": "inputs larger than L2: 4.7 GB of KV per layer, every layer its own pool"}


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_b200(args):
    import torch.distributed as dist
    import gaudirt_b200 as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    g = GEOM
    B, ctx, d, blk, L = args.batch, args.ctx, g["head_dim"], g["block"], args.layers
    assert g["kv_heads"] % world == 0, "KV heads must divide over the ranks"
    hq, hkv = g["q_heads"] // world, g["kv_heads"] // world
    blocks_per_seq = ctx // blk
    n_blocks = int(B * blocks_per_seq * 1.1)
    slots = n_blocks * blk

    # ---- metadata (replicated on every rank): shuffled block tables, new token at ctx-1 -------
    gen = torch.Generator().manual_seed(20261102)
    tables = torch.randperm(n_blocks, generator=gen)[: B * blocks_per_seq].reshape(B, blocks_per_seq).to(torch.int32)
    pos = torch.arange(ctx)
    mapping = (tables.long()[:, pos // blk] * blk + pos % blk).to(torch.int32).contiguous()
    requests = torch.arange(B, dtype=torch.int32)
    positions = torch.full((B,), ctx - 1, dtype=torch.int32)
    locations = mapping[:, ctx - 1].contiguous()
    scale = 1.0 / math.sqrt(d)

    # ---- pools: layer 0 is drawn N(0,1); the others are that data rotated by a layer-specific
    # offset (same distribution, distinct HBM, seconds instead of minutes to fill) ---------------
    pool = rt._C._allocate_paged_kv(L, slots, hkv, d)
    flat0 = pool[0].view(-1)
    step_elems = 1 << 28
    for off in range(0, flat0.numel(), step_elems):
        flat0[off:off + step_elems].normal_()
    for l in range(1, L):
        shift = (l * 7919 * d) % flat0.numel()
        dst = pool[l].view(-1)
        dst[: flat0.numel() - shift].copy_(flat0[shift:])
        dst[flat0.numel() - shift:].copy_(flat0[:shift])
    views = [(pool[l, 0].transpose(0, 1), pool[l, 1].transpose(0, 1)) for l in range(L)]

    hgen = torch.Generator().manual_seed(20261102 + rank)
    host_q = torch.randn(L, B, hq * d, generator=hgen).to(torch.bfloat16).pin_memory()
    host_k = torch.randn(L, B, hkv * d, generator=hgen).to(torch.bfloat16).pin_memory()
    host_v = torch.randn(L, B, hkv * d, generator=hgen).to(torch.bfloat16).pin_memory()
    host_out = torch.empty(L, B, hq * d * world, dtype=torch.bfloat16).pin_memory()
    dq, dk, dv = host_q.to(dev), host_k.to(dev), host_v.to(dev)
    gathered = torch.empty(world, B, hq * d, dtype=torch.bfloat16, device=dev) if world > 1 else None

    def gather_last(out):
        """AllGatherDimLast: [B, cols] per rank -> [B, world*cols], rank-major along the last dim."""
        if world == 1:
            return out
        dist.all_gather_into_tensor(gathered.view(world * B, -1), out)
        return gathered.permute(1, 0, 2).reshape(B, -1)

    md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
    md.attention_plan(hq, hkv, d)

    def resident_step():
        last = None
        for l in range(L):
            out = torch.ops.gaudirt.paged_attn(dq[l], dk[l], dv[l], views[l][0], views[l][1], md, d, scale)
            last = gather_last(out)
        return last

    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        """The same step from HOST buffers: metadata built from CPU tensors, per layer q/k/v copied
        in from pinned memory and the layer's result copied back, copies overlapped with compute."""
        main = torch.cuda.current_stream()
        step_md = rt.PagedMetadata(locations, requests, positions, mapping, slots)
        step_md.attention_plan(hq, hkv, d)
        staged = {}

        def stage(l):
            with torch.cuda.stream(copy_in):
                t = (host_q[l].to(dev, non_blocking=True), host_k[l].to(dev, non_blocking=True),
                     host_v[l].to(dev, non_blocking=True))
                ev = torch.cuda.Event()
                ev.record(copy_in)
            staged[l] = (t, ev)

        stage(0)
        for l in range(L):
            if l + 1 < L:
                stage(l + 1)
            (q, k, v), ev = staged.pop(l)
            main.wait_event(ev)
            for t in (q, k, v):
                t.record_stream(main)
            out = gather_last(torch.ops.gaudirt.paged_attn(q, k, v, views[l][0], views[l][1], step_md, d, scale))
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                out.record_stream(copy_out)
                host_out[l].copy_(out, non_blocking=True)
        main.wait_stream(copy_out)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.barrier()
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        resident_step()
    with ClockSampler(local) as clocks:
        total_ms = timed(resident_step, args.steps)
    for _ in range(2):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps)
    status = rt._C._take_device_status()
    assert status == 0, f"device status {status}"

    # ---- dominant kernel alone: CUDA events around every attention launch of one step ---------
    from gaudirt_b200 import raw as H
    from gaudirt_b200 import abi
    seq, page = H.validate(locations, requests, positions, mapping, slots)
    work, combine, entries = H.plan(seq, hq, hkv, d, sm_count=torch.cuda.get_device_properties(dev).multi_processor_count)
    work_d = torch.from_numpy(work).to(dev)
    table = md.request_mapping()
    out = torch.empty(B, hq * d, dtype=torch.bfloat16, device=dev)
    pml, po = torch.empty(max(entries, 1) * 2, device=dev), torch.empty(max(entries, 1) * d, device=dev)
    lib, s = abi.lib(), H.stream_ptr()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(L)]
    for rep in range(2):
        for l in range(L):
            events[l][0].record()
            abi.check(lib.gk_paged_attn_bf16(dq[l].data_ptr(), dq[l].stride(0), pool[l, 0].data_ptr(), pool[l, 1].data_ptr(),
                                             slots, table.data_ptr(), table.stride(0), page, page, None, work_d.data_ptr(),
                                             len(work), out.data_ptr(), out.stride(0), pml.data_ptr(), po.data_ptr(), scale,
                                             0.0, -1, hq, hkv, d, None, s), "gk_paged_attn_bf16")
            events[l][1].record()
        torch.cuda.synchronize()
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_per_step = total_ms / args.steps
    tokens_s = B / ms_per_step * 1e3
    e2e_tokens_s = B / (e2e_ms / args.steps) * 1e3
    kv_bytes = B * ctx * hkv * d * 2 * 2
    algo_bytes = kv_bytes + 2 * B * hq * d * 2 + B * (ctx // page) * 4 + len(work) * 32
    peak, which = peaks()
    achieved = algo_bytes / kernel_ms / 1e6
    line = {
        "metric": METRIC, "value": tokens_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, world),
        "kv_read_gbs_whole_step": kv_bytes * L * world / ms_per_step / 1e6,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": f"{which} copy bandwidth", "kernel": "paged_attn_kernel<128,4,3>",
                     "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": algo_bytes,
                     "frac_of_8TBs_nominal": achieved / 8000.0},
        "e2e": {"value": e2e_tokens_s, "unit": "tokens/s",
                "h2d_bytes_per_step": int(L * B * (hq + 2 * hkv) * d * 2 + (3 * B + mapping.numel() + 1) * 4 + work.nbytes),
                "d2h_bytes_per_step": int(L * B * hq * world * d * 2)},
        "gpu_launches": args.steps * L * (2 + (1 if len(combine) else 0)),
        "clocks": clocks.summary(),
    }
    line["roofline"]["traffic"] = TRAFFIC_PER_KV_BYTE * kv_bytes
    line["roofline"]["traffic_source"] = TRAFFIC_SOURCE
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        case = cpu_case(args, args.cpu_seqs)
        cpu_pass(case)
        sec = min(cpu_pass(case), cpu_pass(case))
        line["cpu_baseline"] = {"value": 1.0 / (sec * L), "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{args.cpu_seqs} of {B} sequences x 1 of {L} layers (store + direct_bf16_pv), "
                                          "best of 2 after a warm-up, scaled linearly"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
