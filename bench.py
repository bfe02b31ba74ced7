"""Benchmark of the sparse-decode hot path.

Workload (one "step"): a Qwen3-1.7B-shaped decode step — 28 attention layers, 16 query heads,
8 KV heads, head_dim 128, bf16 KV, batch 64, every request at 8192 tokens, page_size 16,
top-k 30 + 1 BOS + 1 EOS page, layer 0 dense and layers 1-27 sparse.  Per step: block-table
build, then per layer KV write, centroid maintenance (the new token closes a page), fused
indexer and paged decode attention.  Data are seeded synthetic N(0,1) values; each layer has its
own 2.1 GB K/V pool in seeded random physical page order, so a step touches far more than L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the same
workload on its own shard of requests (weak scaling, no hot-path communication); NCCL is used
for the barrier, the max-over-ranks time and to gather verification verdicts.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "vortex_torch-dev_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

METRIC = "sparse-decode steps/s (Qwen3-1.7B-shape, bs64 per GPU, 8k ctx)"
CFG = dict(layers=28, Hq=16, Hkv=8, D=128, bs=64, ctx=8192, P=16, K=30, bos=1, eos=1, skip=[0])


def algorithmic_bytes(cfg):
    """Centroid rows scanned + K/V bytes of the attended pages (q, outputs, index lists excluded)."""
    S = cfg["bs"] * cfg["Hkv"]
    pages = cfg["ctx"] // cfg["P"]
    row = cfg["D"] * 2
    page_kv = 2 * cfg["P"] * cfg["D"] * 2
    budget = cfg["K"] + cfg["bos"] + cfg["eos"]
    cent = S * (pages - cfg["bos"] - cfg["eos"]) * row
    sparse_kv = S * budget * page_kv
    dense_kv = S * pages * page_kv
    n_sparse = cfg["layers"] - len(cfg["skip"])
    return dict(centroids_per_layer=cent, sparse_kv_per_layer=sparse_kv, dense_kv_per_layer=dense_kv,
                step=n_sparse * (cent + sparse_kv) + len(cfg["skip"]) * dense_kv)


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return json.loads(f.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def ncu_traffic_bytes(name: str):
    """DRAM bytes (read + written) of one launch of a kernel, from the figures recorded beside its ncu summary
    (``profiles/<name>_ncu.json``); None when no capture has been recorded."""
    f = ROOT / "profiles" / f"{name}_ncu.json"
    if not f.exists():
        return None
    d = json.loads(f.read_text())
    return float(d["dram_bytes_read"]) + float(d["dram_bytes_write"])


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline (oracle port)
def cpu_baseline(cfg, sample_requests: int = 16, repeats: int = 3):
    """Time the CPU port of the path on a bounded sample and scale it to one full step.

    Sample: ``sample_requests`` requests of the workload (all 8 KV heads each); one dense layer and
    one sparse layer (plan + indexer + decode) are timed and scaled by batch and layer counts.
    """
    from oracle import vortex_oracle as vo

    torch.set_num_threads(os.cpu_count() or 1)
    P, H, G, D, K = cfg["P"], cfg["Hkv"], cfg["Hq"] // cfg["Hkv"], cfg["D"], cfg["K"]
    seq = [cfg["ctx"]] * sample_requests
    prob = vo.make_paged_problem(0, seq, H, G, D, P)
    best_sparse, best_dense = float("inf"), float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, cfg["bos"],
                              cfg["eos"], 64, 16)
        t_plan = time.perf_counter() - t0
        t0 = time.perf_counter()
        vo.forward_indexer(prob["q"], prob["centroids"], plan, K, cfg["bos"], cfg["eos"])
        vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                      plan["kv_last_page_len"])
        best_sparse = min(best_sparse, time.perf_counter() - t0)
        t0 = time.perf_counter()
        vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["dense_kv_indptr"], plan["dense_kv_indices"],
                      plan["kv_last_page_len"])
        best_dense = min(best_dense, time.perf_counter() - t0)
    scale = cfg["bs"] / sample_requests
    n_sparse = cfg["layers"] - len(cfg["skip"])
    step_s = scale * (t_plan + n_sparse * best_sparse + len(cfg["skip"]) * best_dense)
    return dict(value=1.0 / step_s, unit="steps/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{sample_requests} of {cfg['bs']} requests x (plan + 1 sparse layer + 1 dense layer), "
                       f"scaled by batch and by {n_sparse} sparse + {len(cfg['skip'])} dense layers",
                sparse_layer_s=best_sparse, dense_layer_s=best_dense)


def run_reference_arm(args, cfg):
    """The reference has no CPU (or Blackwell) implementation of this path; its arithmetic restated in
    PyTorch eager on the host cores is what gets timed here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup):
        cpu_baseline(cfg, sample_requests=4, repeats=1)
    cb = None
    for _ in range(max(1, min(args.steps, 5))):
        cb = cpu_baseline(cfg, sample_requests=8, repeats=1)
        vals.append(cb["value"])
    v = float(np.median(vals))
    cb["value"] = v
    line = dict(metric=METRIC, value=v, unit="steps/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1000.0 / v, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic", impl="reference", config=workload_config(cfg, args.gpus), cpu_baseline=cb,
                e2e=dict(value=v, unit="steps/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


def workload_config(cfg, n):
    return dict(workload="Qwen3-1.7B-shaped decode step: 28 layers (layer 0 dense, 1-27 sparse), 16 q heads, "
                         "8 KV heads, head_dim 128, bf16, batch 64 per GPU at 8192 tokens, page_size 16, "
                         "topk 30 + 1 BOS + 1 EOS",
                global_batch=cfg["bs"] * n, sharding=f"requests x{n}, no hot-path collective",
                l2="per-layer pools (2.1 GB K/V each, 60 GB per step working set) exceed L2; no flush needed",
                flow="block_sparse_attention")


# --------------------------------------------------------------------------- GPU arm
def build_runtime(cfg, device, seed, flow_name="block_sparse_attention"):
    from vortex_torch import _cabi
    from vortex_torch.runtime import GraphedDecodeStep, ServerArgs, VortexDecodeRuntime

    P, H, bs = cfg["P"], cfg["Hkv"], cfg["bs"]
    pages_per_req = cfg["ctx"] // P
    num_pages = bs * pages_per_req
    sa = ServerArgs(page_size=P, vortex_topk_val=cfg["K"], vortex_page_reserved_bos=cfg["bos"],
                    vortex_page_reserved_eos=cfg["eos"], vortex_layers_skip=list(cfg["skip"]),
                    vortex_max_seq_lens=cfg["ctx"], vortex_module_name=flow_name)
    rt = VortexDecodeRuntime(cfg["layers"], cfg["Hq"], H, cfg["D"], num_pages=num_pages, max_bs=bs,
                             context_len=cfg["ctx"], server_args=sa, dtype=torch.bfloat16, device=device)
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g)
    slots = (perm.view(bs, pages_per_req, 1) * P + torch.arange(P).view(1, 1, P)).view(bs, -1)
    rt.model_runner.req_to_token_pool.req_to_token.copy_(slots.to(torch.int32))
    torch.manual_seed(seed)
    closing = (torch.arange(num_pages, device=device, dtype=torch.int64) * P + (P - 1))
    for l in range(cfg["layers"]):
        buf = rt.pool.buffers[l]
        buf["k"].normal_()
        buf["v"].normal_()
        if "centroids" in buf:
            _cabi.cmean(buf["k"], buf["centroids"], closing, H, P)
        if "max" in buf:
            _cabi.creduce(buf["k"], buf["max"], closing, H, P, 1)
            _cabi.creduce(buf["k"], buf["min"], closing, H, P, 2)
    step = GraphedDecodeStep(rt, bs)
    step.seq_lens.fill_(cfg["ctx"])
    step.req_indices.copy_(torch.arange(bs))
    step.loc.copy_(slots[:, cfg["ctx"] - 1].to(torch.int64))
    step.q.normal_()
    step.new_k.normal_()
    step.new_v.normal_()
    torch.cuda.synchronize(device)
    return rt, step, slots


def verify_sample(rt, step, cfg, slots):
    """Check request 0 of the last sparse layer and of the dense layer against the CPU oracle."""
    from oracle import vortex_oracle as vo

    P, H, G, D, K = cfg["P"], cfg["Hkv"], cfg["Hq"] // cfg["Hkv"], cfg["D"], cfg["K"]
    pages = cfg["ctx"] // P
    seq = np.asarray([cfg["ctx"]], dtype=np.int32)
    r2t = slots[:1].numpy().astype(np.int32)
    plan = vo.plan_decode(seq, r2t, np.zeros(1, dtype=np.int64), P, H, K, cfg["bos"], cfg["eos"], 64, 16)
    rows = torch.as_tensor(plan["dense_kv_indices"], dtype=torch.long)
    ok = True
    for layer in (cfg["layers"] - 1, cfg["skip"][0] if cfg["skip"] else None):
        if layer is None:
            continue
        buf = rt.pool.buffers[layer]
        # compact copy of request 0's rows so the CPU side stays small
        remap = {int(r): i for i, r in enumerate(rows.tolist())}
        k = buf["k"][rows.to(rt.device)].cpu()
        v = buf["v"][rows.to(rt.device)].cpu()
        c = buf["centroids"][rows.to(rt.device)].cpu()
        p2 = {kk: vv.copy() for kk, vv in plan.items()}
        p2["dense_kv_indices"] = np.arange(len(rows), dtype=np.int32)
        for s in range(H):
            a, b = int(p2["sparse_kv_indptr"][s]), int(p2["sparse_kv_indptr"][s + 1])
            p2["sparse_kv_indices"][a:b] = [remap.get(int(x), -1) for x in plan["sparse_kv_indices"][a:b]]
        q = step.q[layer, 0].view(H, G, D).cpu()
        got = step.out[layer, 0].view(H, G, D).float().cpu()
        if layer in cfg["skip"]:
            want = vo.decode_gqa(q, k, v, p2["dense_kv_indptr"], p2["dense_kv_indices"], p2["kv_last_page_len"])
        else:
            vo.forward_indexer(q, c, p2, K, cfg["bos"], cfg["eos"])
            ns = int(p2["sparse_kv_indptr"][H])
            if layer == cfg["layers"] - 1:  # the index buffers hold the last layer's selection
                dev_sel = rt.backend.kv_indices_decode[1][:ns].cpu().numpy()
                want_sel = rows.numpy()[p2["sparse_kv_indices"][:ns]]
                ok = ok and bool(np.array_equal(dev_sel, want_sel))
            want = vo.decode_gqa(q, k, v, p2["sparse_kv_indptr"], p2["sparse_kv_indices"], p2["kv_last_page_len"])
        ok = ok and bool(((got - want.float()).abs() <= 2e-2 * want.float().abs().clamp(min=1)).all())
    return ok


def time_kernels(rt, step, cfg, reps, pdl):
    """Average device time per launch of each kernel kind, from CUDA events around graph replays.

    For each kind (fused sparse layer, fused indexer, sparse decode, dense decode, KV write + centroid
    update) one CUDA graph holds that kernel's launches of every layer of a step, back to back on each
    layer's own pool, launched the way the step launches them (``pdl``: programmatic dependent launch,
    with the early prologue of the fused layer kernel when 2); the graph is replayed ``reps`` times
    between two events on the launching stream.
    """
    from vortex_torch import _cabi
    from vortex_torch.cache import set_kv_buffer_launcher

    dev = rt.device
    b = rt.backend
    eff_bs = cfg["bs"] * cfg["Hkv"]
    sparse_layers = [l for l in range(cfg["layers"]) if l not in rt.skip]
    dense_layers = [l for l in range(cfg["layers"]) if l in rt.skip]

    def views(l):
        return step.q[l].view(-1, rt.G, rt.D), step.out[l].view(-1, rt.G, rt.D), rt.pool.buffers[l]

    def run_indexer():
        for l in sparse_layers:
            qv, _, cache = views(l)
            _cabi.indexer_fused(qv, cache["centroids"], b.kv_indptr_decode[0], b.kv_indptr_decode[1],
                                b.kv_indices_decode[0], b.kv_indices_decode[1], eff_bs, cfg["K"], cfg["bos"],
                                cfg["eos"], rt.ictx.max_num_pages_per_request)

    def run_decode(layers, sparse):
        for l in layers:
            qv, ov, _ = views(l)
            rt.attention(qv, l, ov, sparse=sparse)

    def run_cache():
        for l in range(cfg["layers"]):
            cache = rt.pool.buffers[l]
            _cabi.set_kv_cmean(cache["k"], cache["v"], step.new_k[l], step.new_v[l], cache["centroids"], step.loc,
                               rt.P)

    def run_fused():
        for l in sparse_layers:
            qv, ov, cache = views(l)
            # the page lists are static here (no planner launch in this graph), so the early prologue is safe
            _cabi.sparse_layer_fused(qv, cache["centroids"], cache["k"], cache["v"], ov, b.kv_indptr_decode[0],
                                     b.kv_indptr_decode[1], b.kv_indices_decode[0], b.kv_indices_decode[1],
                                     b.kv_last_page_len_decode, eff_bs, rt.P, cfg["K"], cfg["bos"], cfg["eos"],
                                     rt.ictx.max_num_pages_per_request, rt.sm_scale, step.new_k[l], step.new_v[l],
                                     step.loc, workspace=rt.layer_workspace, early_prologue=pdl == 2)

    kinds = dict(sparse_layer_fused=(run_fused, len(sparse_layers)),
                 indexer=(run_indexer, len(sparse_layers)),
                 decode_sparse=(lambda: run_decode(sparse_layers, True), len(sparse_layers)),
                 decode_dense=(lambda: run_decode(dense_layers, False), len(dense_layers)),
                 kv_write_cmean=(run_cache, cfg["layers"]))
    out = {}
    for name, (fn, n) in kinds.items():
        if n == 0:
            out[name] = None
            continue
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        _cabi.set_programmatic_launch(1 if pdl else 0)
        try:
            with torch.cuda.graph(g):
                fn()
        finally:
            _cabi.set_programmatic_launch(0)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        out[name] = e0.elapsed_time(e1) * 1e-3 / (reps * n)
    return out


def measure_mla(dev, steps, layers=4, mla_path=0, pdl=True):
    """The MLA block-table sparse decode configuration (config 5), one layer = page selection + decode in one
    launch (`vtx_mla_sparse_layer`); the two kernels are also timed on their own and as two launches.

    bs128, 16 heads, 576-dim latent (values = first 512), page 64, 16384 tokens, topk 32 + 1 + 1.
    ``layers`` distinct 2.4 GB latent pools are cycled so that consecutive launches never share L2 lines.
    Returns a dict with per-kernel and per-layer times, bytes and fractions of the measured HBM peak.
    """
    from oracle import vortex_oracle as vo
    from vortex_torch import _cabi

    _cabi.set_mla_path(mla_path)
    bs, Hq, Dl, Dv, P, ctx, K, bos, eos, L = 128, 16, 576, 512, 64, 16384, 32, 1, 1, layers
    pages_per_req = ctx // P
    num_pages = bs * pages_per_req
    g = torch.Generator().manual_seed(7)
    perm = torch.randperm(num_pages, generator=g)
    slots = (perm.view(bs, pages_per_req, 1) * P + torch.arange(P).view(1, 1, P)).view(bs, -1).to(torch.int32)
    i32 = dict(dtype=torch.int32, device=dev)
    r2t = slots.to(dev)
    seq = torch.full((bs,), ctx, **i32)
    ridx = torch.arange(bs, device=dev)
    budget = K + bos + eos
    dip, sip = torch.zeros(bs + 1, **i32), torch.zeros(bs + 1, **i32)
    din, sin_ = torch.zeros(num_pages, **i32), torch.zeros(bs * budget, **i32)
    last = torch.zeros(bs, **i32)
    w = [torch.zeros(num_pages // 16 + bs, **i32) for _ in range(3)] + [torch.zeros(1, **i32), torch.zeros(1, **i32)]
    dpt, spt = torch.zeros(bs, pages_per_req, **i32), torch.zeros(bs, pages_per_req, **i32)
    dsl, ssl = torch.zeros(bs, **i32), torch.zeros(bs, **i32)
    _cabi.plan_decode(seq, r2t, ridx, dip, din, sip, sin_, last, *w, P, 1, K, bos, eos, 64, 16, dpt, dsl, spt, ssl)
    torch.manual_seed(7)
    closing = torch.arange(num_pages, device=dev, dtype=torch.int64) * P + (P - 1)
    lat, cent, qs, outs = [], [], [], []
    for _ in range(L):
        x = torch.empty(num_pages, P, Dl, dtype=torch.bfloat16, device=dev).normal_()
        c = torch.zeros(num_pages, 1, Dl, dtype=torch.bfloat16, device=dev)
        _cabi.cmean(x, c, closing, 1, P)
        lat.append(x); cent.append(c)
        qs.append(torch.randn(bs, Hq, Dl, device=dev).bfloat16())
        outs.append(torch.empty(bs, Hq, Dv, dtype=torch.bfloat16, device=dev))
    scale = 1.0 / math.sqrt(192.0)

    def run_indexer():
        for l in range(L):
            _cabi.indexer_fused(qs[l], cent[l], dip, sip, din, sin_, bs, K, bos, eos, pages_per_req,
                                sparse_page_table=spt)

    def run_decode():
        for l in range(L):
            _cabi.decode_mla(qs[l], lat[l], outs[l], spt, ssl, P, scale)

    def run_layer():  # selection + decode as one launch (two in the mma.sync form)
        for l in range(L):
            _cabi.mla_sparse_layer(qs[l], cent[l], lat[l], outs[l], dip, sip, din, sin_, spt, ssl, P, K, bos, eos,
                                   pages_per_req, scale)

    def run_two_launches():
        for l in range(L):
            _cabi.indexer_fused(qs[l], cent[l], dip, sip, din, sin_, bs, K, bos, eos, pages_per_req,
                                sparse_page_table=spt)
            _cabi.decode_mla(qs[l], lat[l], outs[l], spt, ssl, P, scale)

    res = {}
    for name, fn in (("indexer", run_indexer), ("decode_mla", run_decode), ("layer_two_launches", run_two_launches),
                     ("layer", run_layer)):
        fn()
        torch.cuda.synchronize(dev)
        gr = torch.cuda.CUDAGraph()
        _cabi.set_programmatic_launch(1 if pdl else 0)  # launches of the graph chained as in the headline step
        try:
            with torch.cuda.graph(gr):
                fn()
        finally:
            _cabi.set_programmatic_launch(0)
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        res[name] = e0.elapsed_time(e1) * 1e-3 / (steps * L)
    # parity of request 0 of the last layer against the CPU oracle (selection bit-exact, output within 2e-2)
    rows = dpt[0].cpu().long()
    plan = vo.plan_decode([ctx], np.arange(ctx, dtype=np.int32).reshape(1, -1), [0], P, 1, K, bos, eos, 64, 16,
                          page_table_stride=pages_per_req)
    q0 = qs[-1][:1].cpu()
    vo.forward_indexer(q0, cent[-1][rows.to(dev)].cpu(), plan, K, bos, eos)
    want_sel = rows.numpy()[plan["sparse_kv_indices"]]
    ok = bool(np.array_equal(spt[0, :budget].cpu().numpy(), want_sel))
    want = vo.decode_mla(q0, lat[-1][rows.to(dev)].cpu(), plan["sparse_page_table"], plan["sparse_cache_seqlens"], Dv,
                         scale)
    got = outs[-1][:1].float().cpu()
    ok = ok and bool(((got - want.float()).abs() <= 2e-2 * want.float().abs().clamp(min=1)).all())
    peaks, kind = measured_peaks()
    cent_b = bs * (pages_per_req - bos - eos) * Dl * 2
    kv_b = bs * budget * P * Dl * 2
    flops = bs * budget * P * (2 * Hq * Dl + 2 * Hq * Dv)
    gb = lambda nbytes, secs: nbytes / secs / 1e9
    return dict(workload="config 5: MLA block-table sparse decode, bs128, 16 heads x 576 latent, page 64, 16k ctx, "
                         "topk 32+1+1",
                us=dict((k, v * 1e6) for k, v in res.items()),
                indexer=dict(bytes=cent_b, achieved_gbs=gb(cent_b, res["indexer"]),
                             frac=gb(cent_b, res["indexer"]) / peaks["hbm_gbs"]),
                decode_mla=dict(bytes=kv_b, achieved_gbs=gb(kv_b, res["decode_mla"]),
                                frac=gb(kv_b, res["decode_mla"]) / peaks["hbm_gbs"],
                                tflops=flops / res["decode_mla"] / 1e12),
                layer=dict(bytes=cent_b + kv_b, us=res["layer"] * 1e6,
                           achieved_gbs=gb(cent_b + kv_b, res["layer"]),
                           frac=gb(cent_b + kv_b, res["layer"]) / peaks["hbm_gbs"]),
                mla_form="mma.sync + cp.async" if mla_path else "tcgen05 + TMA",
                programmatic_launch=1 if pdl else 0, mla_fault_bits=_cabi.mla_fault_bits(),
                parity_sample_ok=ok, peak_kind=f"of {kind}")


def run_mla_workload(args):
    print(json.dumps(measure_mla(torch.device("cuda", 0), args.steps, layers=args.layers or 4,
                                 mla_path=args.mla_path, pdl=bool(args.pdl))))


def measure_ragged(dev, dist, rank, world, steps, warmup, head_shards=1):
    """The ragged-batch configuration (config 3), one sparse layer, sharded over the ranks (strong scaling).

    256 requests, context lengths uniform in [1024, 32768], 32 q heads / 8 KV heads / head_dim 128, bf16,
    page 16, topk 64 + 1 + 1.  The ranks form a grid of (world / head_shards) request shards x head_shards head
    shards: requests are dealt to the request shards by total page count, and a rank holds a pool with only its
    own requests' pages and its own KV heads.  No collective on the timed path; NCCL gathers the selections
    of sampled requests for verification afterwards.  Returns the result dict on every rank.
    """
    from oracle import vortex_oracle as vo
    from vortex_torch import _cabi
    from vortex_torch.runtime import gather_for_verification, shard_grid

    nreq, Hq, H_all, D, P, K, bos, eos = 256, 32, 8, 128, 16, 64, 1, 1
    G = Hq // H_all
    g = torch.Generator().manual_seed(33)
    seq_all = torch.randint(1024, 32769, (nreq,), generator=g).tolist()
    pages_all = [(x + P - 1) // P for x in seq_all]
    grid = shard_grid(pages_all, H_all, world, head_shards)
    mine, H = list(grid[rank].requests), grid[rank].num_heads   # from here on H is this rank's head count
    seq = [seq_all[r] for r in mine]
    n = [pages_all[r] for r in mine]
    bs, total, maxp = len(mine), sum(n), max(n)
    gl = torch.Generator().manual_seed(1000 + rank)
    perm = torch.randperm(total, generator=gl)
    r2t = torch.zeros(bs, maxp * P, dtype=torch.int32)
    off = 0
    for i in range(bs):
        pg = perm[off:off + n[i]]
        r2t[i, : n[i] * P] = (pg.view(-1, 1) * P + torch.arange(P).view(1, -1)).reshape(-1).to(torch.int32)
        off += n[i]
    i32 = dict(dtype=torch.int32, device=dev)
    budget = K + bos + eos
    S = bs * H
    seq_d, r2t_d, ridx = torch.tensor(seq, **i32), r2t.to(dev), torch.arange(bs, device=dev)
    dip, sip = torch.zeros(S + 1, **i32), torch.zeros(S + 1, **i32)
    din, sin_ = torch.zeros(total * H, **i32), torch.zeros(S * budget, **i32)
    last = torch.zeros(S, **i32)
    w = [torch.zeros(total * H // 16 + S, **i32) for _ in range(3)] + [torch.zeros(1, **i32), torch.zeros(1, **i32)]
    torch.manual_seed(1000 + rank)
    k = torch.empty(total * H, P, D, dtype=torch.bfloat16, device=dev).normal_()
    v = torch.empty(total * H, P, D, dtype=torch.bfloat16, device=dev).normal_()
    cent = torch.zeros(total * H, 1, D, dtype=torch.bfloat16, device=dev)
    _cabi.cmean(k, cent, torch.arange(total, device=dev, dtype=torch.int64) * P + (P - 1), H, P)
    q = torch.randn(S, G, D, device=dev).bfloat16()
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(D)
    # scratch that lets the long segments of this batch be scanned by several CTAs each
    ws = torch.zeros(max(1, _cabi.sparse_layer_workspace_bytes(S, maxp, K, bos, eos) // 4), **i32)

    def layer():
        _cabi.plan_decode(seq_d, r2t_d, ridx, dip, din, sip, sin_, last, *w, P, H, K, bos, eos, 64, 16)
        _cabi.sparse_layer_fused(q, cent, k, v, out, dip, sip, din, sin_, last, S, P, K, bos, eos, maxp, scale,
                                 workspace=ws)

    layer()
    torch.cuda.synchronize(dev)
    gr = torch.cuda.CUDAGraph()
    _cabi.set_programmatic_launch(1)
    try:
        with torch.cuda.graph(gr):
            layer()
    finally:
        _cabi.set_programmatic_launch(0)
    for _ in range(max(3, warmup)):
        gr.replay()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        gr.replay()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(dev)
    secs = e0.elapsed_time(e1) * 1e-3 / steps
    # the layer launch alone (a model step plans once for all its layers; the figure above plans per layer)
    gk = torch.cuda.CUDAGraph()
    _cabi.set_programmatic_launch(1)
    try:
        with torch.cuda.graph(gk):
            for _ in range(4):
                _cabi.sparse_layer_fused(q, cent, k, v, out, dip, sip, din, sin_, last, S, P, K, bos, eos, maxp, scale,
                                         workspace=ws)
    finally:
        _cabi.set_programmatic_launch(0)
    gk.replay()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(steps):
        gk.replay()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(dev)
    secs_kernel = e0.elapsed_time(e1) * 1e-3 / (steps * 4)
    if dist is not None:
        tt = torch.tensor([secs, secs_kernel], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        secs, secs_kernel = float(tt[0]), float(tt[1])
    # ---- verification of two sampled local requests (the longest one and request bs/2) against the CPU
    # oracle, then gathered over NCCL
    sel_local, ok = {}, _cabi.device_status() == 0
    sip_h = sip.cpu().numpy()
    for i in sorted({max(range(bs), key=lambda r: n[r]), bs // 2}):
        ni = n[i]
        plan = vo.plan_decode([seq[i]], (np.arange(ni * P, dtype=np.int32)).reshape(1, -1), [0], P, H, K, bos, eos, 64, 16)
        # oracle rows are page*H + h over a compact pool holding only this request, in logical order
        rows = ((r2t[i, : ni * P : P].long() // P).view(-1, 1) * H + torch.arange(H).view(1, -1)).reshape(-1).to(dev)
        kk, vv, cc = k[rows].cpu(), v[rows].cpu(), cent[rows].cpu()
        qi = q[i * H:(i + 1) * H].cpu()
        vo.forward_indexer(qi, cc, plan, K, bos, eos)
        a, b = sip_h[i * H], sip_h[(i + 1) * H]
        got_rows = sin_[a:b].cpu().numpy()
        # translate device rows (physical page * H + h) to the compact numbering (logical page * H + h)
        phys_to_log = {int(r2t[i, pg * P].item()) // P: pg for pg in range(ni)}
        got = np.asarray([phys_to_log[int(r) // H] * H + int(r) % H for r in got_rows], dtype=np.int32)
        ok = ok and bool(np.array_equal(got, plan["sparse_kv_indices"]))
        want = vo.decode_gqa(qi, kk, vv, plan["sparse_kv_indptr"], plan["sparse_kv_indices"], plan["kv_last_page_len"])
        gotv = out[i * H:(i + 1) * H].float().cpu()
        ok = ok and bool(((gotv - want.float()).abs() <= 2e-2 * want.float().abs().clamp(min=1)).all())
        sel_local[mine[i] * H_all + grid[rank].head_lo] = torch.as_tensor(got.astype(np.int64), device=dev)
    gathered = gather_for_verification(sel_local, dtype=torch.int64)
    flags = torch.tensor([int(ok)], device=dev, dtype=torch.int32)
    if dist is not None:
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    # ---- algorithmic bytes of the whole batch (all ranks)
    cent_b = sum(H_all * max(0, p - bos - eos) * D * 2 for p in pages_all if p - bos - eos > K)
    kv_b = 0
    for s_len, p in zip(seq_all, pages_all):
        toks = s_len if p <= budget else (budget - 1) * P + (s_len % P or P)
        kv_b += H_all * toks * D * 2 * 2
    peaks, kind = measured_peaks()
    return dict(workload="config 3: ragged batch, 256 requests ctx U[1024,32768], 32q/8kv heads, D128, page 16, "
                         "topk 64+1+1, one sparse layer (plan + selection and attention in one launch, long "
                         "segments split over CTAs)",
                n_gpus=world, scaling="strong", sharding=f"{world // head_shards} request shards x {head_shards} head shards",
                requests_per_rank=[len(x.requests) for x in grid], kv_heads_per_rank=H,
                us_per_layer=secs * 1e6, layers_per_s=1.0 / secs, algorithmic_bytes=cent_b + kv_b,
                achieved_gbs=(cent_b + kv_b) / secs / 1e9,
                frac_of_n_x_peak=(cent_b + kv_b) / secs / 1e9 / (world * peaks["hbm_gbs"]),
                layer_launch_only=dict(us=secs_kernel * 1e6,
                                       frac_of_n_x_peak=(cent_b + kv_b) / secs_kernel / 1e9 / (world * peaks["hbm_gbs"])),
                peak_kind=f"of {kind}", parity_sample_ok=bool(int(flags.item())), verified_requests=sorted({int(x) // H_all for x in gathered}))


def run_ragged_workload(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    line = measure_ragged(dev, dist, rank, world, args.steps, args.warmup, head_shards=args.head_shards)
    if rank == 0:
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def side_flow_measurement(args, cfg, rt, step, json_fd):
    """Side measurement (not the headline line): the same decode step with another shipped flow choosing
    the pages.  Prints steps/s of the graphed step; parity of these flows is covered by the tests."""
    dev = rt.device
    step.capture(programmatic_launch=args.pdl)
    for _ in range(max(3, args.warmup)):
        step.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    secs = e0.elapsed_time(e1) * 1e-3 / args.steps
    peaks, kind = measured_peaks()
    ab = algorithmic_bytes(cfg)
    n_sparse = cfg["layers"] - len(cfg["skip"])
    extra = ab["centroids_per_layer"] * n_sparse if args.flow == "gqa_quest_sparse_attention" else 0  # two summary rows
    total = ab["step"] + extra
    line = dict(flow=args.flow, workload=workload_config(cfg, 1)["workload"], steps_per_s=1.0 / secs,
                ms_per_step=secs * 1e3, algorithmic_bytes=total, achieved_gbs=total / secs / 1e9,
                frac=total / secs / 1e9 / peaks["hbm_gbs"], peak_kind=f"of {kind}", programmatic_launch=int(args.pdl))
    sys.stdout.flush()
    os.write(json_fd, (json.dumps(line) + "\n").encode())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="debug: fewer layers (number is invalid as a bench)")
    ap.add_argument("--batch", type=int, default=None, help="debug: smaller batch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--head-shards", type=int, default=1,
                    help="--workload c3: ranks per request shard that split its KV heads (divides --gpus and 8)")
    ap.add_argument("--no-side", action="store_true", help="skip the side measurements (configs 3 and 5)")
    ap.add_argument("--pdl", type=int, default=2, choices=[0, 1, 2],
                    help="programmatic dependent launch inside the step graph: 0 off, 1 on, 2 on + early prologue")
    ap.add_argument("--flow", default="block_sparse_attention",
                    choices=["block_sparse_attention", "gqa_block_sparse_attention", "gqa_quest_sparse_attention"],
                    help="which shipped flow selects the pages (the headline line uses the default)")
    ap.add_argument("--mla-path", type=int, default=0, choices=[0, 1],
                    help="c5 workload: 0 = tcgen05 + TMA form of the MLA decode (default), 1 = mma.sync + cp.async form")
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c5"],
                    help="c2 = the headline decode step; c5 = side measurement of the MLA block-table decode")
    args = ap.parse_args()
    if args.workload == "c5":
        run_mla_workload(args)
        return
    if args.workload == "c3":
        run_ragged_workload(args)
        return
    cfg = dict(CFG)
    if args.layers:
        cfg["layers"] = args.layers
    if args.batch:
        cfg["bs"] = args.batch
    if args.impl == "reference":
        run_reference_arm(args, cfg)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    # Libraries (NCCL's version banner, for one) write to stdout; the JSON line must be the only thing
    # there, so everything else goes to stderr until the line is printed.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    rt, step, slots = build_runtime(cfg, device, seed=1234 + rank, flow_name=args.flow)
    if args.flow != "block_sparse_attention":
        side_flow_measurement(args, cfg, rt, step, json_fd)
        return
    if not args.no_graph:
        step.capture(programmatic_launch=args.pdl)
    W = max(3, args.warmup)
    for _ in range(W):
        step.replay()
    torch.cuda.synchronize(device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    # ---- device-resident timing
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step.replay()
    e1.record()
    barrier()
    dev_s = e0.elapsed_time(e1) * 1e-3
    # ---- end to end from pinned host buffers
    h = step.host_buffers()
    for n in ("seq_lens", "req_indices", "loc", "q", "new_k", "new_v"):
        h[n].copy_(getattr(step, n).cpu())
    if not args.no_graph:
        step.capture_host_pipeline(programmatic_launch=args.pdl)
    for _ in range(3):
        step.run_from_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step.run_from_host()
    torch.cuda.synchronize(device)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    if dist is not None:
        tt = torch.tensor([dev_s, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_s, e2e_s = float(tt[0]), float(tt[1])

    ok = verify_sample(rt, step, cfg, slots)
    if dist is not None:
        flags = [torch.zeros(1, device=device, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(flags, torch.tensor([int(ok)], device=device, dtype=torch.int32))
        ok = all(int(f.item()) == 1 for f in flags)

    kt = time_kernels(rt, step, cfg, reps=10, pdl=0 if args.no_graph else args.pdl)
    # ---- side measurements, outside the timed region of the headline workload: the ragged batch sharded by
    # request over the same ranks (its strong-scaling point at this N) and, on rank 0, the MLA configuration
    side = None
    if not args.no_side:
        side = dict(c3=measure_ragged(device, dist, rank, world, steps=20, warmup=3))
        if world > 1:  # the same batch with every request's KV heads spread over the ranks as well
            t = max(d for d in (1, 2, 4, 8) if world % d == 0)
            side["c3_head_split"] = measure_ragged(device, dist, rank, world, steps=20, warmup=3, head_shards=t)
        if rank == 0:
            side["c5"] = measure_mla(device, steps=20)
    peaks, peak_kind = measured_peaks()
    ab = algorithmic_bytes(cfg)
    peak = float(peaks["hbm_gbs"])

    def roof(bytes_, secs):
        if not secs:
            return None
        a = bytes_ / secs / 1e9
        return dict(bound="hbm", achieved=a, peak=peak, unit="GB/s", frac=a / peak, peak_kind=f"of {peak_kind}")

    if rank == 0:
        n_sparse = cfg["layers"] - len(cfg["skip"])
        launches_per_step = 1 + n_sparse + 2 * len(cfg["skip"])
        value = world * args.steps / dev_s
        line = dict(
            metric=METRIC, value=value, unit="steps/s", n_gpus=world, steps=args.steps, warmup=W,
            ms_per_step=1000.0 * dev_s / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
            dtype="bf16", data="synthetic", config=workload_config(cfg, world),
            e2e=dict(value=world * args.steps / e2e_s, unit="steps/s", h2d_bytes_per_step=step.h2d_bytes,
                     d2h_bytes_per_step=step.d2h_bytes),
            gpu_launches=launches_per_step * args.steps, clocks=clocks, parity_sample_ok=ok,
            cuda_graph=not args.no_graph, programmatic_launch=int(args.pdl if not args.no_graph else 0),
            roofline=dict(kernel="sparse_layer_kernel (token write + indexer + decode, 27 launches per step)",
                          traffic=ncu_traffic_bytes("sparse_layer_kernel_c2"),
                          algorithmic_bytes_per_launch=ab["centroids_per_layer"] + ab["sparse_kv_per_layer"],
                          **roof(ab["centroids_per_layer"] + ab["sparse_kv_per_layer"], kt["sparse_layer_fused"])),
            kernels=dict(sparse_layer_fused=roof(ab["centroids_per_layer"] + ab["sparse_kv_per_layer"],
                                                 kt["sparse_layer_fused"]),
                         indexer_fused=roof(ab["centroids_per_layer"], kt["indexer"]),
                         decode_sparse=roof(ab["sparse_kv_per_layer"], kt["decode_sparse"]),
                         decode_dense=roof(ab["dense_kv_per_layer"], kt["decode_dense"]),
                         us=dict((k, v * 1e6 if v else None) for k, v in kt.items())),
            step_hbm=dict(algorithmic_bytes=ab["step"], achieved_gbs=ab["step"] * args.steps / dev_s / 1e9,
                          frac_of_measured_peak=ab["step"] * args.steps / dev_s / 1e9 / peak,
                          frac_of_nominal_8000=ab["step"] * args.steps / dev_s / 1e9 / 8000.0),
        )
        if side is not None:
            line["side"] = side
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(cfg)
        elif not args.no_cpu_baseline:
            line["cpu_baseline"] = None
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
