#!/usr/bin/env python
"""bench.py -- decode tokens/s of the crabml CUDA backend on synthetic Llama-2-7B shapes (BASELINE.json metric).

One "step" = one decoded token = one pass of the hot path (225 quantized matvecs + the small ops around them).
  value : device-resident throughput (weights + KV in HBM, no host<->device traffic inside the timed region)
  e2e   : the same loop through the reference-facing runner API with HOST buffers: per step the token id goes
          host->device and the 128 KB logits come device->host (Llama2Runner::forward -> export, llama2.rs:209),
          then the host samples (argmax) and feeds the next token.
  roofline : the dominant kernel (the ffn_gate/ffn_up-shaped matvec, 11008x4096) timed with CUDA events
  cpu_baseline : the CPU restatement of the reference's AVX2 path (oracle/, all host threads) on a bounded sample
`--impl reference` runs ONLY that CPU path and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SEED = 0x5EED
WORKLOADS = {
    # name: (config name, body weight type, classifier weight type)
    "llama2-7b-q8_0": ("LLAMA2_7B", "Q8_0", "Q8_0"),
    "llama2-7b-q4_0": ("LLAMA2_7B", "Q4_0", "Q4_0"),
    "llama2-7b-q4_0-q6k": ("LLAMA2_7B", "Q4_0", "Q6_K"),
    "llama2-7b-q4_k": ("LLAMA2_7B", "Q4_K", "Q6_K"),
    "tinyllamas-15m-q8_0": ("TINYLLAMAS_15M", "Q8_0", "Q8_0"),
    # BASELINE.json config 5: the dense matmuls of a 4096-token prefill (TMA + tcgen05 path, csrc/prefill_gemm.cu); see run_prefill
    "mistral-7b-q8_0-prefill": ("MISTRAL_7B", "Q8_0", "Q8_0"),
    "llama2-7b-q8_0-prefill": ("LLAMA2_7B", "Q8_0", "Q8_0"),
    # the Zatorax family at layer sizes of a real model (random weights), beside a llama stack of equal size; see run_zatorax
    "zatorax-w1024": ("ZATORAX", "BF16", "BF16"),
    "zatorax-w2048": ("ZATORAX", "BF16", "BF16"),
    # the Meresun family at the same layer sizes, beside the Zatorax stack of equal width and depth; see run_meresun
    "meresun-w1024": ("MERESUN", "BF16", "BF16"),
    "meresun-w2048": ("MERESUN", "BF16", "BF16"),
    # the Vuzinex family at the same layer sizes, beside the Zatorax stack of equal width and depth; see run_vuzinex
    "vuzinex-w1024": ("VUZINEX", "BF16", "BF16"),
    "vuzinex-w2048": ("VUZINEX", "BF16", "BF16"),
    # the Lifesun family at the same layer sizes, beside the Vuzinex stack of equal width and depth; see run_lifesun
    "lifesun-w1024": ("LIFESUN", "BF16", "BF16"),
    "lifesun-w2048": ("LIFESUN", "BF16", "BF16"),
    "lifesun-w4096": ("LIFESUN", "BF16", "BF16"),
}
# dram bytes per megakernel launch from the committed ncu --set full capture (profiles/); None until captured
TRAFFIC = {("llama2-7b-q8_0", 1): 7040893000 + 49879296}     # profiles/r02p_mega_ring_q8_0_ncu_raw.csv (mega_ring_kernel: dram__bytes_read.sum + dram__bytes_write.sum)
MEGA_NAMES = {1: ("mega_kernel", "mega.cu, weights through registers"), 2: ("mega_ring_kernel", "mega_ring.cu, weights through a TMA-fed shared-memory ring")}
TYPE_ID = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def usable_cpus():
    """CPUs this process may actually use: affinity mask capped by the cgroup CPU quota (spin-waiting workers beyond the
    quota get throttled by CFS and make the CPU arm erratic)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        with open("/sys/fs/cgroup/cpu.max") as f:
            quota, period = f.read().split()
        if quota != "max":
            n = min(n, max(1, int(int(quota) / int(period))))
    except (OSError, ValueError):
        pass
    return n


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured (MEASURED_PEAKS.json)"
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0}, "fallback (B200_PROFILING.md)"


class ClockSampler:
    """nvidia-smi clocks/throttle reasons DURING the timed region (B200_PROFILING.md recipe)."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's CPU path restated (oracle/), AVX2 order, all host threads, bounded sample
# --------------------------------------------------------------------------------------------------------------
def cpu_reference_tokens_per_s(workload: str, steps: int = 8, warmup: int = 2, sample_layers: int = 8):
    from crabml_b200 import runner as R          # config table + byte accounting only (no GPU use)
    from oracle import oracle as oc
    from oracle.llama_replay import Llama2Runner, LlamaConfig, LlamaWeights
    from oracle.synth import synth_weight
    from oracle.tensor_ref import OracleDevice, OracleTensor

    cname, wt_name, ct_name = WORKLOADS[workload]
    conf = getattr(R, cname)
    wt, ct = TYPE_ID[wt_name], TYPE_ID[ct_name]
    dim, hid, kv = conf.embedding_dim, conf.hidden_dim, conf.head_size() * conf.n_kv_heads
    # thread count: the reference takes it from the command line; use the count that is fastest for the dominant matvec on
    # this host (ascending, stop when it gets slower -- oversubscribed spin-waiting workers are pathological on big hosts)
    probe_w = synth_weight(wt, 2048, dim, SEED, 99, R.synth_scale(wt, dim))
    probe_x = np.random.default_rng(0).standard_normal(dim).astype(np.float32)
    threads, best = 1, float("inf")
    cpus = min(usable_cpus(), oc.hw_threads())
    for cand in sorted({c for c in (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, cpus) if c <= cpus}):
        oc.gemv(wt, probe_w, 2048, dim, probe_x, threads=cand, flags=oc.ORDER_AVX2)
        dt = float("inf")
        for _ in range(3):                       # best of 3 batches of 5
            t0 = time.perf_counter()
            for _ in range(5):
                oc.gemv(wt, probe_w, 2048, dim, probe_x, threads=cand, flags=oc.ORDER_AVX2)
            dt = min(dt, time.perf_counter() - t0)
        if dt < best * 0.97:
            threads, best = cand, dt
        elif dt > best * 1.3:
            break
    dev = OracleDevice(thread_num=threads, flags=oc.ORDER_AVX2)
    n_sample_layers = min(sample_layers, conf.n_layers)

    def syn(rows, cols, t, tid):
        return OracleTensor.from_cpu(synth_weight(t, rows, cols, SEED, tid, R.synth_scale(t, cols)), [rows, cols], t, dev)
    rng = np.random.default_rng(SEED)

    def norm():
        return OracleTensor.from_cpu((1.0 + 0.05 * rng.standard_normal(dim)).astype(np.float32), [dim], oc.F32, dev)
    L = conf.n_layers
    w = dict(wq=[], wk=[], wv=[], wo=[], gate=[], up=[], down=[], ra=[], rf=[])
    for l in range(n_sample_layers):            # same tensor ids as crabml_b200.runner.synthetic_weights
        b = 7 * l
        w["wq"].append(syn(dim, dim, wt, b + 1)); w["wk"].append(syn(kv, dim, wt, b + 2)); w["wv"].append(syn(kv, dim, wt, b + 3))
        w["wo"].append(syn(dim, dim, wt, b + 4)); w["gate"].append(syn(hid, dim, wt, b + 5)); w["up"].append(syn(hid, dim, wt, b + 6))
        w["down"].append(syn(dim, hid, wt, b + 7)); w["ra"].append(norm()); w["rf"].append(norm())
    tok_embed = syn(conf.vocab_size, dim, wt, 7 * L + 1)
    out_w = syn(conf.vocab_size, dim, ct, 7 * L + 2)
    # REAL decode steps (warm-up, then `steps` timed tokens, mean) on two models cut from the same weights: 1 layer and
    # n_sample_layers layers (+ embedding, final norm, classifier).  A full token = the 1-layer token + (L - 1) x the per-layer
    # difference -- every layer of these shapes costs the same on the CPU (weights stream from DRAM once per token).
    times = {}
    for nl in sorted({1, n_sample_layers}):
        c = LlamaConfig(conf.n_heads, conf.n_kv_heads, nl, dim, hid, conf.seq_len, conf.vocab_size, conf.rms_norm_eps, conf.rope_dim or None)
        lw = LlamaWeights(tok_embed, w["wq"][:nl], w["wk"][:nl], w["wv"][:nl], w["wo"][:nl], w["gate"][:nl], w["down"][:nl], w["up"][:nl],
                          w["ra"][:nl], w["rf"][:nl], norm(), out_w)
        r = Llama2Runner(OracleTensor, c, lw, dev, warmup + steps + 8)
        pos = 0
        for i in range(warmup):
            r.forward([1 + i], pos); pos += 1
        t0 = time.perf_counter()
        for i in range(steps):
            r.forward([100 + i], pos); pos += 1
        times[nl] = (time.perf_counter() - t0) / max(1, steps)
    if n_sample_layers > 1:
        per_layer = (times[n_sample_layers] - times[1]) / (n_sample_layers - 1)
        if per_layer <= 0:                       # timer noise: split the sampled time by streamed bytes instead
            lb = 4 * R.weight_bytes(wt, dim, dim) + 3 * R.weight_bytes(wt, hid, dim)
            per_layer = times[n_sample_layers] * lb / (n_sample_layers * lb + R.weight_bytes(ct, conf.vocab_size, dim))
        rest = times[1] - per_layer
    else:
        per_layer, rest = times[1], 0.0
    per_token = per_layer * conf.n_layers + max(rest, 0.0)
    detail = {"layers_timed": n_sample_layers, "layers_model": conf.n_layers, "steps_timed": steps, "warmup_run": warmup,
              "ms_per_token_1_layer_model": times[1] * 1e3, f"ms_per_token_{n_sample_layers}_layer_model": times[n_sample_layers] * 1e3,
              "ms_per_layer": per_layer * 1e3, "extrapolated": n_sample_layers < conf.n_layers, "threads": threads, "usable_cpus": cpus,
              "hw_threads": oc.hw_threads(), "thread_probe": "ascending counts on a 2048-row matvec of the body type, fastest kept"}
    sample = (f"{steps} timed decode steps (after {warmup} warm-up) of a 1-layer and a {n_sample_layers}-layer cut of {workload} (same synthetic weights, seed "
              f"{SEED:#x}, embedding + final norm + classifier included); token time = 1-layer token + {conf.n_layers - 1} x per-layer difference; "
              f"AVX2-order C restatement of the reference, {threads} threads ({cpus} usable CPUs, {oc.hw_threads()} hardware threads)")
    return 1.0 / per_token, threads, sample, per_token, detail


def run_reference(args, rank, world):
    if rank != 0:
        return
    tps, threads, sample, per_token, detail = cpu_reference_tokens_per_s(args.workload, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_token * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"{args.workload}-decode-synthetic", "note": "reference CPU path restated in C (oracle/): the Rust reference cannot be built here"},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample, **detail},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def quick_decode(workload: str, local_rank: int, K: int, W: int, start_pos: int):
    """Second measurement of the default run: the same decode loop (device-resident and e2e) for another weight type, so that one
    bench line covers the whole metric (Q8_0 AND Q4_0).  Returns a dict that is embedded in the main JSON line."""
    from crabml_b200 import CudaTensorDevice
    from crabml_b200 import runner as R
    cname, wt_name, ct_name = WORKLOADS[workload]
    conf = getattr(R, cname)
    wt, ct = TYPE_ID[wt_name], TYPE_ID[ct_name]
    dev = CudaTensorDevice(local_rank, lazy=2)
    try:
        weights = R.synthetic_weights(dev, conf, wt, ct, seed=SEED)
        runner = R.LlamaRunner(dev, conf, weights, min(conf.seq_len, start_pos + 2 * (W + K) + 8))
        bytes_per_token = runner.weight_bytes_per_token()
        pos, tok = 0, 1
        for _ in range(start_pos):
            runner.forward([tok], pos, export=False); pos += 1; tok = (tok * 7 + 3) % conf.vocab_size

        def step_e2e(t, p):
            lg = runner.forward([t], p, export=True)
            return int(np.flatnonzero(lg == lg.max())[-1])
        for _ in range(W):
            tok = step_e2e(tok, pos); pos += 1
        dev.synchronize()
        p0 = pos                                           # both timed regions decode at the same KV positions [p0, p0 + K)
        dev.timer_begin(); t0 = time.perf_counter()
        for _ in range(K):
            tok = step_e2e(tok, pos); pos += 1
        e2e_ms = max(dev.timer_end(), (time.perf_counter() - t0) * 1e3)
        pos = p0
        l0 = dev.launch_count()
        dev.timer_begin()
        for i in range(K):
            runner.forward([(tok * 31 + 7 * i) % conf.vocab_size], pos, export=False); pos += 1
        val_ms = dev.timer_end()
        launches = dev.launch_count() - l0
        peaks, _ = measured_peaks()
        gbs = bytes_per_token / (val_ms / K * 1e-3) / 1e9
        out = {"workload": f"{workload}-decode-synthetic", "weights": wt_name, "classifier": ct_name, "value": K / (val_ms * 1e-3), "unit": "tok/s",
               "ms_per_step": val_ms / K, "e2e": {"value": K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": conf.vocab_size * 4},
               "gpu_launches_device_resident": int(launches), "steps": K, "warmup": W,
               "roofline": {"bound": "hbm", "kernel": MEGA_NAMES.get(dev.mega_variant(), MEGA_NAMES[1])[0] if launches == K else "fused kernels (CUDA graph)", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes_per_launch": bytes_per_token, "frac_of_8TBs_nominal": gbs / 8000.0}}
        runner.close()
        return out
    finally:
        dev.close()


# --------------------------------------------------------------------------------------------------------------
def run_b200(args, rank, world, local_rank):
    from crabml_b200 import CudaTensor, CudaTensorDevice
    from crabml_b200 import runner as R

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("cpu:gloo,cuda:nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    sharded = world > 1 and args.multi == "sharded"

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cname, wt_name, ct_name = WORKLOADS[args.workload]
    conf = getattr(R, cname)
    wt, ct = TYPE_ID[wt_name], TYPE_ID[ct_name]
    transport = args.comm
    lazy = args.lazy if not (sharded and transport == "nccl" and args.lazy == 2) else 1     # NCCL cannot run inside the megakernel
    dev = CudaTensorDevice(local_rank, lazy=lazy)
    plan = None
    if sharded:
        from crabml_b200 import sharding

        def exchange(blob):
            out = [None] * world
            dist.all_gather_object(out, blob)
            return out
        plan = sharding.make_plan(conf.n_heads, conf.n_kv_heads, conf.embedding_dim, conf.hidden_dim, conf.vocab_size, wt, rank, world)
        dev.init_comm(rank, world, exchange, transport)
    args.lazy = lazy
    weights = R.synthetic_weights(dev, conf, wt, ct, seed=SEED, plan=plan)
    K, W = args.steps, args.warmup
    kv_len = min(conf.seq_len, args.start_pos + 3 * (W + K) + 8)
    runner = R.LlamaRunner(dev, conf, weights, kv_len, plan=plan)
    bytes_per_token = runner.weight_bytes_per_token()

    # context: fill the KV cache up to start_pos with untimed steps so that decode runs at a realistic position
    pos, tok = 0, 1
    for _ in range(args.start_pos):
        runner.forward([tok], pos, export=False); pos += 1; tok = (tok * 7 + 3) % conf.vocab_size

    def step_e2e(t, p):
        lg = runner.forward([t], p, export=True)      # token id H2D (8 B) + logits D2H (vocab*4 B)
        return int(np.flatnonzero(lg == lg.max())[-1])   # sampler.rs:109-116 argmax (last max)

    for _ in range(W):
        tok = step_e2e(tok, pos); pos += 1
    # ---- timed region 1: e2e through the runner's public decode call with HOST buffers ---------------------------------------
    # ccr_runner_generate_greedy_ex: the prompt id goes host->device, the logits of EVERY step come device->host (pinned staging, async)
    # and the ids too; the host samples (argmax, sampler.rs:109-116) from those logits inside the timed region and must agree with the
    # device-side sampler that fed the next step.  No step waits for the host, so the GPU never idles between tokens.
    sampler = ClockSampler(local_rank); sampler.start()
    dev.synchronize(); barrier()
    p0 = pos              # every timed region decodes K tokens at the SAME KV positions [p0, p0 + K): the regions differ in how the host is involved, not in context length
    launches0 = dev.launch_count()
    dev.timer_begin(); t0 = time.perf_counter()
    tok_first = tok
    ids, lgs = runner.generate_greedy_logits([tok], K)
    host_ids = [int(np.flatnonzero(lg == lg.max())[-1]) for lg in lgs]
    e2e_ms_dev = dev.timer_end(); e2e_wall = time.perf_counter() - t0
    assert host_ids == ids and len(ids) == K, "host sampler and device sampler disagree"
    pos = p0; tok = tok_first                     # the synchronous variant reproduces the same greedy sequence
    launches_e2e = dev.launch_count() - launches0
    barrier()
    e2e_ms = max_over_ranks(max(e2e_ms_dev, e2e_wall * 1e3))      # host work (sampling) is part of e2e
    # the synchronous variant (one forward + blocking export + host argmax per token), for comparison
    dev.synchronize(); barrier()
    dev.timer_begin(); t0 = time.perf_counter()
    for _ in range(K):
        tok = step_e2e(tok, pos); pos += 1
    e2e_sync_ms = max_over_ranks(max(dev.timer_end(), (time.perf_counter() - t0) * 1e3))
    pos = p0
    barrier()
    # ---- timed region 2: device-resident (no per-step host<->device traffic) -----------------------------------
    toks = [tok_first] + ids[:-1]          # the same K input tokens at the same positions as the e2e region: identical device work, no host round trips
    dev.synchronize(); barrier()
    launches1 = dev.launch_count()
    st0 = dev.lazy_stats() if args.lazy else None
    dev.timer_begin(); th0 = time.perf_counter()
    for i in range(K):
        runner.forward([toks[i]], pos, export=False); pos += 1
    host_issue_ms = (time.perf_counter() - th0) * 1e3          # host time to record+submit K tokens (GPU runs behind)
    val_ms = max_over_ranks(dev.timer_end())
    st1 = dev.lazy_stats() if args.lazy else None
    launches_val = dev.launch_count() - launches1
    clocks = sampler.stop()
    barrier()

    # ---- roofline of the dominant kernel: ffn_gate/ffn_up-shaped matvec over all layers' weights (>> L2) ----------
    # (timed through an eager-mode device handle on the same GPU so that each matmul_vec is its own launch pair)
    m, k = weights["ffn_gate"][0].shape()
    dev.synchronize()
    edev = CudaTensorDevice(local_rank, lazy=False) if args.lazy else dev
    x = CudaTensor.new(np.random.default_rng(1).standard_normal(k).astype(np.float32), [k], edev)
    mats = [CudaTensor(wm.buf, wm.strider(), edev) for wm in weights["ffn_gate"] + weights["ffn_up"]]
    for wmat in mats[:4]:
        wmat.matmul_vec(x)
    reps = 3
    edev.synchronize()
    l0 = edev.launch_count()
    edev.timer_begin()
    for _ in range(reps):
        for wmat in mats:
            wmat.matmul_vec(x)
    mv_ms = edev.timer_end()
    n_mv = reps * len(mats)
    launches_per_mv = (edev.launch_count() - l0) / n_mv
    mv_bytes = R.weight_bytes(wt, m, k)
    mv_gbs = mv_bytes / (mv_ms / n_mv * 1e-3) / 1e9
    peaks, peak_src = measured_peaks()

    if rank == 0:
        streams = 1 if sharded or world == 1 else world       # sharded: ONE token stream over N GPUs; replicas: N streams
        value = streams * K / (val_ms * 1e-3)
        e2e = streams * K / (e2e_ms * 1e-3)
        if lazy == 2 and launches_val == K:
            # the dominant kernel IS the step: one mega_kernel launch per token streams every weight byte of this rank once
            mega_gbs = bytes_per_token / (val_ms / K * 1e-3) / 1e9
            mk_name, mk_file = MEGA_NAMES.get(dev.mega_variant(), MEGA_NAMES[1])
            roofline = {"bound": "hbm", "kernel": f"{mk_name} ({mk_file}): one persistent launch per decoded token, all matvec/attention/norm phases",
                        "achieved": mega_gbs, "peak": peaks["hbm_gbs"], "peak_source": peak_src, "unit": "GB/s", "frac": mega_gbs / peaks["hbm_gbs"],
                        "traffic": TRAFFIC.get((args.workload, world)), "traffic_source": "profiles/ (ncu --set full, dram__bytes_read.sum + dram__bytes_write.sum per launch)" if TRAFFIC.get((args.workload, world)) else None,
                        "algorithmic_bytes_per_launch": bytes_per_token, "us_per_launch": val_ms / K * 1e3, "frac_of_8TBs_nominal": mega_gbs / 8000.0}
        else:
            roofline = {"bound": "hbm", "kernel": f"matvec_stream_kernel<{wt_name}> {m}x{k} (+ activation quantize: {launches_per_mv:.0f} launches per matmul_vec)",
                        "achieved": mv_gbs, "peak": peaks["hbm_gbs"], "peak_source": peak_src, "unit": "GB/s",
                        "frac": mv_gbs / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": mv_bytes,
                        "us_per_launch": mv_ms / n_mv * 1e3, "frac_of_8TBs_nominal": mv_gbs / 8000.0}
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": val_ms / K, "higher_is_better": True, "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}-decode-synthetic", "weights": wt_name, "classifier": ct_name, "kv_cache": "f32",
                       "start_pos": args.start_pos, "kv_positions": [int(p0), int(p0 + K)], "mode": "lazy: plan not megakernel-eligible (matvec types outside Q8_0/Q4_0 use the warp-per-row kernels): fused kernels, CUDA-graph replay" if (lazy == 2 and launches_val != K) else {0: "eager (one launch per trait call)", 1: "lazy: fused kernels, CUDA-graph replay", 2: "lazy: one persistent megakernel per token, CUDA-graph replay"}[args.lazy],
                       "multi_gpu": ("single GPU" if world == 1 else
                                     f"one token stream sharded over {world} GPUs: rows of wq/wk/wv/gate/up/classifier, block columns of wo/down; "
                                     f"exchange = {'one-shot NVLink peer stores fused into the megakernel' if transport == 'p2p' and lazy == 2 else 'one-shot NVLink peer-store kernel' if transport == 'p2p' else 'ncclAllReduce/ncclAllGather'} "
                                     f"(2 allreduce of [dim] f32 per layer + 1 allgather of logits)" if sharded else f"{world} independent replicas"),
                       "weight_bytes_per_token_per_gpu": bytes_per_token,
                       "l2_policy": f"weights streamed once per token ({bytes_per_token / 1e9:.2f} GB >> 126 MB L2): inputs larger than L2",
                       "weight_bytes_per_token": bytes_per_token,
                       "hbm_frac_whole_step": bytes_per_token / (val_ms / K * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": conf.vocab_size * 4 + 8,
                    "ms_per_step": e2e_ms / K,
                    "api": "ccr_runner_generate_greedy_ex: sampling on the device feeds the next step, logits + ids exported asynchronously every step, host argmax checked in the timed region",
                    "synchronous_variant": {"value": streams * K / (e2e_sync_ms * 1e-3), "unit": "tok/s", "api": "ccr_runner_forward + blocking export + host argmax per token"}},
            "gpu_launches": int(launches_e2e),
            "gpu_launches_device_resident": int(launches_val),
            "roofline": roofline,
            "roofline_matvec_eager": {"kernel": f"matvec_stream_kernel<{wt_name}> {m}x{k} + activation quantize ({launches_per_mv:.0f} launches per matmul_vec, eager handle, not in the timed region)",
                                      "achieved": mv_gbs, "unit": "GB/s", "frac": mv_gbs / peaks["hbm_gbs"], "algorithmic_bytes_per_launch": mv_bytes,
                                      "us_per_launch": mv_ms / n_mv * 1e3},
            "clocks": clocks,
            "lazy_stats": dev.lazy_stats() if args.lazy else None,
            "host_ms_per_step": {"issue_total": host_issue_ms / K,
                                 **({k: (st1[k] - st0[k]) / 1e3 / K for k in ("host_us_record", "host_us_fuse", "host_us_submit")} if args.lazy else {})},
        }
        if world == 1 and not args.no_cpu_baseline:
            tps, threads, sample, _, detail = cpu_reference_tokens_per_s(args.workload, steps=min(K, 8), warmup=2)
            line["cpu_baseline"] = {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample, **detail}
    runner.close()
    dev.close()
    if rank == 0:
        if world == 1 and args.workload == "llama2-7b-q8_0" and not args.no_also:
            # the metric names Q8_0 AND Q4_0: same loop, same shapes, Q4_0 blocks (llama.cpp-style Q4_0 files keep a Q6_K classifier:
            # run `--workload llama2-7b-q4_0-q6k` for that variant)
            weights = None
            try:
                line["also"] = {"llama2-7b-q4_0": quick_decode("llama2-7b-q4_0", local_rank, K, W, args.start_pos)}
            except Exception as e:      # the second block must never cost the main line
                line["also"] = {"llama2-7b-q4_0": {"error": repr(e)}}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()



def run_prefill(args, rank, world, local_rank):
    """BASELINE.json config 5: every matmul_vec of a `--prefill-tokens`-token prompt pass (Tensor::matmul_vec with a (b, k) rhs) on the
    tensor-core path: per layer wq, wk, wv, wo, ffn_gate, ffn_up, ffn_down on (b, k) activations, then the classifier on the last row.
    A step = all 225 matmuls once.  This is the DENSE part of a prefill (58 of ~63 TFLOP for Mistral-7B at 4096 tokens); attention,
    norms and RoPE of a batched forward are not part of this workload (the reference has no batched forward: llama2.rs:111-139 walks
    the prompt token by token)."""
    from crabml_b200 import CudaTensor, CudaTensorDevice
    from crabml_b200 import runner as R
    if rank != 0:
        return
    cname, wt_name, ct_name = WORKLOADS[args.workload]
    conf = getattr(R, cname)
    wt, ct = TYPE_ID[wt_name], TYPE_ID[ct_name]
    b = args.prefill_tokens
    dev = CudaTensorDevice(local_rank, lazy=0)
    weights = R.synthetic_weights(dev, conf, wt, ct, seed=SEED)
    dim, hid = conf.embedding_dim, conf.hidden_dim
    rng = np.random.default_rng(SEED)
    x_dim = CudaTensor.new(rng.standard_normal(b * dim).astype(np.float32), [b, dim], dev)
    x_hid = CudaTensor.new(rng.standard_normal(b * hid).astype(np.float32), [b, hid], dev)
    x_last = CudaTensor.new(rng.standard_normal(dim).astype(np.float32), [dim], dev)
    flops = 0
    for key, kk in (("wq", dim), ("wk", dim), ("wv", dim), ("wo", dim), ("ffn_gate", dim), ("ffn_up", dim), ("ffn_down", hid)):
        for t in weights[key]:
            flops += 2 * b * t.shape()[0] * kk
    wbytes = sum(R.weight_bytes(t.dtype(), *t.shape()) for key in ("wq", "wk", "wv", "wo", "ffn_gate", "ffn_up", "ffn_down") for t in weights[key])

    def step():
        for l in range(conf.n_layers):
            for key in ("wq", "wk", "wv", "wo", "ffn_gate", "ffn_up"):
                weights[key][l].matmul_vec(x_dim)
            weights["ffn_down"][l].matmul_vec(x_hid)
        return weights["output_weight"].matmul_vec(x_last)
    K, W = args.steps, args.warmup
    for _ in range(W):
        step()
    sampler = ClockSampler(local_rank); sampler.start()
    dev.synchronize()
    l0 = dev.launch_count()
    dev.timer_begin()
    for _ in range(K):
        step()
    ms = dev.timer_end()
    launches = dev.launch_count() - l0
    # e2e: what crosses the host boundary in a prompt pass -- the token ids go host->device (the embedding rows are gathered on the
    # device, llama2.rs:223-224), the logits of the last position come back
    ids = [int(v) for v in rng.integers(0, conf.vocab_size, b)]
    from crabml_b200 import capi as _capi
    dev.synchronize()
    dev.timer_begin(); t0 = time.perf_counter()
    for _ in range(K):
        xd = CudaTensor.alloc([b, dim], _capi.F32, dev)
        xd.copy_rows_from(weights["token_embed"], ids)
        for l in range(conf.n_layers):
            for key in ("wq", "wk", "wv", "wo", "ffn_gate", "ffn_up"):
                weights[key][l].matmul_vec(xd)
            weights["ffn_down"][l].matmul_vec(x_hid)
        weights["output_weight"].matmul_vec(x_last).export()
    e2e_ms = max(dev.timer_end(), (time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop()
    peaks, peak_src = measured_peaks()
    tf = flops / (ms / K * 1e-3) / 1e12
    peak_tf = peaks.get("bf16_tflops_sustained", 1431.9)
    line = {"metric": "prefill_tokens_per_s", "value": b * K / (ms * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operand tiles (dequantised Q8_0 weights, quantised activations), f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}-dense-matmuls-synthetic", "prompt_tokens": b, "weights": wt_name,
                       "scope": "the 225 matmul_vec calls of a prompt pass (per-call activation quantisation and weight dequantisation included); attention / norms / RoPE of a "
                                "batched forward are not part of this workload",
                       "l2_policy": f"{wbytes / 1e9:.2f} GB of weights and {b * hid * 4 / 1e6:.0f} MB activations per step: inputs larger than L2",
                       "flop_per_step": flops},
            "e2e": {"value": b * K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": b * 8, "d2h_bytes_per_step": conf.vocab_size * 4, "ms_per_step": e2e_ms / K},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "umma_gemm_kernel (prefill_gemm.cu): TMA -> smem ring -> tcgen05.mma kind::f16 -> TMEM -> tcgen05.ld epilogue",
                         "achieved": tf, "peak": peak_tf, "peak_source": peak_src + " bf16_tflops_sustained", "unit": "TFLOP/s", "frac": tf / peak_tf, "traffic": None,
                         "note": "whole step (dequantise + quantise + GEMM launches) over the dense FLOPs; the GEMM kernel alone is profiled in profiles/"},
            "clocks": clocks}
    print(json.dumps(line))
    dev.close()


def zatorax_bench_config(width: int, n_layers: int = 4, vocab: int = 32000):
    """delta, attention, attention reading the previous layer's keys / values, delta; 128-wide heads, 4 query heads per key head,
    16 experts of width/2 (top 4) plus a shared expert of the model's width: 3 x width of active feed-forward per token"""
    H = width // 128
    G = max(1, H // 4)
    mlp = {"kind": "moe", "expert": {"ff": width // 2}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}}, "shared": {"ff": width}}
    delta = {"type": "delta", "mixer": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "conv": 4}, "mlp": mlp}
    layers = []
    for i in range(n_layers):
        if i % 4 in (0, 3):
            layers.append(delta)
        else:
            m = {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 128 ** -0.5}
            if i % 4 == 2:
                m["kv_from"] = i - 1
            layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Zatorax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers}


def measure_seq_model(dev, model, prompt, K, W, params):
    """prefill and decode of one slot-based model (seqmodel.SeqModel) through its step function; device time and wall time"""
    Tp = len(prompt)
    l0 = dev.launch_count()
    for rep in range(2):                                             # first pass warms up (tensor maps, pool, function attributes)
        slot = model.open()
        dev.synchronize(); dev.timer_begin(); t0 = time.perf_counter()
        model.step(slot, prompt, [Tp - 1])
        pre_ms = dev.timer_end(); pre_wall = (time.perf_counter() - t0) * 1e3
        if rep == 0:
            model.close_seq(slot)
    pre_launches = (dev.launch_count() - l0) // 2
    tok = prompt[-1]
    for _ in range(W):
        model.step(slot, [tok], [0])
    l0 = dev.launch_count()
    dev.synchronize(); dev.timer_begin(); t0 = time.perf_counter()
    for _ in range(K):
        lg = model.step(slot, [tok], [0])                            # token id host -> device, logits device -> host, every step
        tok = int(np.argmax(lg[0]))
    dec_ms = dev.timer_end(); dec_wall = (time.perf_counter() - t0) * 1e3
    dec_launches = dev.launch_count() - l0
    return {"params": params, "prefill_tok_s": Tp / (pre_ms * 1e-3), "prefill_ms": pre_ms, "prefill_wall_ms": pre_wall, "prefill_launches": int(pre_launches),
            "decode_tok_s": K / (dec_ms * 1e-3), "decode_ms_per_token": dec_ms / K, "decode_wall_ms_per_token": dec_wall / K,
            "decode_launches_per_token": dec_launches / K, "state": model.stats()}


def meresun_bench_config(width: int, vocab: int = 32000):
    """four layers (dense, routed, dense, routed), each run once, so that depth and active feed-forward width (3 x width per token) equal
    the Zatorax stack's; 128 + 64 wide query heads over a latent of 512, window 1024, 16 experts of 3/4 width (top 4 of the best 2 of 4 groups)"""
    H = width // 128
    mixer = {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * width // 4, "kv_rank": 512, "mask": {"size": 1024}, "scale": 192 ** -0.5,
             "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "expert": {"ff": 3 * width // 4, "limit": 7.0}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "latent_attention", "mixer": mixer, "mlp": m} for m in (dense, moe, dense, moe)]
    return {"architecture": "Meresun", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6, "groups": 4}, "token_side": {"dim": 64},
            "loop": {"start": 0, "stop": 0, "times": 1}, "layers": layers}


def run_meresun(args, rank, world, local_rank):
    """Prefill and decode throughput of the Meresun family at real layer sizes, beside the closest existing model -- the Zatorax stack of
    the same width, depth and active feed-forward width (run_zatorax's configuration) -- through the same step function and slots."""
    from crabml_b200 import CudaTensorDevice, meresun, zatorax
    if rank != 0:
        return
    width = int(args.workload.split("-w")[1])
    Tp, K, W = args.prefill_tokens, args.steps, args.warmup
    rng = np.random.default_rng(SEED)
    prompt = [int(v) for v in rng.integers(0, 32000, Tp)]
    sampler = ClockSampler(local_rank); sampler.start()
    out = {}
    for name, mod, cls, raw in (("meresun", meresun, "MeresunModel", meresun_bench_config(width)), ("zatorax", zatorax, "ZatoraxModel", zatorax_bench_config(width))):
        conf = mod.parse_config(raw)
        dev = CudaTensorDevice(local_rank, lazy=0)
        model = getattr(mod, cls)(dev, conf, mod.random_weights(conf, SEED), "bfloat16", chunk=args.zatorax_chunk)
        params = sum(int(np.prod(sh)) if sh else 1 for sh in mod.expected_tensors(conf).values())
        out[name] = measure_seq_model(dev, model, prompt, K, W, params)
        model.close(); dev.close()
    clocks = sampler.stop()
    z = out["meresun"]
    line = {"metric": "decode_tokens_per_s", "value": z["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": z["decode_ms_per_token"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 matrices and product inputs, f32 everything else", "data": "synthetic",
            "config": {"workload": args.workload, "model": meresun_bench_config(width), "prefill_tokens": Tp, "chunk": args.zatorax_chunk,
                       "closest_model": {"family": "zatorax", "model": zatorax_bench_config(width)}},
            "e2e": {"value": 1e3 / z["decode_wall_ms_per_token"], "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 32000 * 4},
            "gpu_launches": int(z["decode_launches_per_token"] * K), "detail": out, "clocks": clocks}
    print(json.dumps(line))


def vuzinex_bench_config(width: int, vocab: int = 32000):
    """four layers, each run once, each with a dense feed-forward of 3 x width, so that depth and active feed-forward width equal the
    Zatorax stack's: attention in blocks of 1024 positions with a sink beside the matrix memory; causal attention with biases, norms and a
    gate beside the decayed linear attention; two state-space layers.  128-wide attention heads, 4 query heads per key head."""
    H = width // 128
    G = max(1, H // 4)
    rot = {"dims": 128, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    rot2 = {"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    mlp = {"kind": "dense", "ff": 3 * width}
    a = {"type": "parallel", "mlp": mlp, "mixer": {"left": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": rot, "mask": {"size": 1024}},
                                                   "right": {"heads": max(1, H // 2), "dim": 128, "vdim": 128, "gate_cap": 20.0}, "left_scale": 1.0, "right_scale": 1.0}}
    b = {"type": "parallel_2", "mlp": mlp, "mixer": {"left": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": rot2},
                                                     "right": {"heads": max(1, H // 2), "dim": 64, "vdim": 128, "tau": 8.0}, "left_scale": 1.0, "right_scale": 1.0}}
    c = {"type": "mamba2", "mlp": mlp, "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}}
    return {"architecture": "Vuzinex", "vocab": vocab, "width": width, "embedding": {"scale": 1.0, "bigram": {"buckets": 65536, "mul_prev": 1000003, "mul_cur": 31}},
            "norm": {"eps": 1e-6}, "residual_mult": 1.0, "logit_scale": 1.0, "layers": [a, b, c, c]}


def time_recurrences(dev, width, T):
    """The recurrence kernels alone at the bench's sizes, beside the closest model's (the gated delta rule): device time of one call over T
    tokens, and the rate at which state elements are updated (token x head x dk x dv per second)."""
    from crabml_b200 import CudaTensor, capi, seqops
    rng = np.random.default_rng(SEED)

    def rand(*shape, scale=1.0):
        return CudaTensor.new((rng.standard_normal(shape) * scale).astype(np.float32), list(shape), dev)

    def zeros(*shape):
        return CudaTensor.alloc(list(shape), capi.F32, dev)
    H = max(1, width // 256)
    out = {}

    def timed(name, heads, dk, dv, f):
        f()
        dev.synchronize(); dev.timer_begin()
        for _ in range(3):
            f()
        ms = dev.timer_end() / 3
        out[name] = {"heads": heads, "dk": dk, "dv": dv, "tokens": T, "ms": ms, "state_updates_per_s": T * heads * dk * dv / (ms * 1e-3)}
    q, k, v = rand(T, H * 128, scale=0.1), rand(T, H * 128, scale=0.1), rand(T, H * 128)
    gi, gf, bz = rand(T, H), rand(T, H), zeros(H)
    S, ms_ = zeros(H, 128, 129), zeros(H)
    timed("matrix_memory", H, 128, 128, lambda: seqops.matrix_memory(q, k, v, gi, gf, bz, bz, 20.0, 128 ** -0.5, S, ms_, H, 128, 128))
    q2, k2, z2, zb = rand(T, H * 64, scale=0.1), rand(T, H * 64, scale=0.1), rand(T, H * 64), zeros(H * 64)
    S2 = zeros(H, 64, 128)
    timed("decayed_linear_attention", H, 64, 128, lambda: seqops.decayed_linear_attention(q2, k2, v, z2, zb, 8.0, 0.125, S2, H, 64, 128))
    Hs = 2 * width // 64
    xbc, dt, hb = rand(T, Hs * 64 + 256, scale=0.3), rand(T, Hs), zeros(Hs)
    S3 = zeros(Hs, 128, 64)
    timed("state_space_scan", Hs, 128, 64, lambda: seqops.state_space_scan(xbc, dt, hb, hb, hb, S3, Hs, 1, 128, 64))
    a, b, S4 = rand(T, H), rand(T, H), zeros(H, 128, 128)
    timed("gated_delta_rule (closest model)", H, 128, 128, lambda: seqops.gated_delta_rule(q, k, v, a, b, bz, bz, S4, H, H, 128, 128))
    return out


def run_vuzinex(args, rank, world, local_rank):
    """Prefill and decode throughput of the Vuzinex family at real layer sizes, beside the closest existing model -- the Zatorax stack of
    the same width, depth and active feed-forward width (run_zatorax's configuration) -- through the same step function and slots; then
    the recurrence kernels alone beside the closest model's."""
    from crabml_b200 import CudaTensorDevice, vuzinex, zatorax
    if rank != 0:
        return
    width = int(args.workload.split("-w")[1])
    Tp, K, W = args.prefill_tokens, args.steps, args.warmup
    rng = np.random.default_rng(SEED)
    prompt = [int(v) for v in rng.integers(0, 32000, Tp)]
    sampler = ClockSampler(local_rank); sampler.start()
    out = {}
    for name, mod, cls, raw in (("vuzinex", vuzinex, "VuzinexModel", vuzinex_bench_config(width)), ("zatorax", zatorax, "ZatoraxModel", zatorax_bench_config(width))):
        conf = mod.parse_config(raw)
        dev = CudaTensorDevice(local_rank, lazy=0)
        kw = {"max_seq": Tp + K + W + 8} if name == "vuzinex" else {}
        weights = mod.random_weights(conf, SEED)
        model = getattr(mod, cls)(dev, conf, weights, "bfloat16", chunk=args.zatorax_chunk, **kw)
        params = sum(int(np.prod(np.shape(a))) for a in weights.values())
        del weights
        out[name] = measure_seq_model(dev, model, prompt, K, W, params)
        model.close()
        if name == "vuzinex":
            out["recurrence_kernels"] = time_recurrences(dev, width, min(Tp, 2048))
        dev.close()
    clocks = sampler.stop()
    z = out["vuzinex"]
    line = {"metric": "decode_tokens_per_s", "value": z["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": z["decode_ms_per_token"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 matrices and product inputs, f32 everything else", "data": "synthetic",
            "config": {"workload": args.workload, "model": vuzinex_bench_config(width), "prefill_tokens": Tp, "chunk": args.zatorax_chunk,
                       "closest_model": {"family": "zatorax", "model": zatorax_bench_config(width)}},
            "e2e": {"value": 1e3 / z["decode_wall_ms_per_token"], "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 32000 * 4},
            "gpu_launches": int(z["decode_launches_per_token"] * K), "detail": out, "clocks": clocks}
    print(json.dumps(line))


def lifesun_bench_config(width: int, vocab: int = 32000):
    """four layers, each run once, each with a dense feed-forward of 3 x width, so that depth and active feed-forward width equal the
    Vuzinex stack's: windowed attention (1024 positions, half of every head rotated, capped scores) beside retention, and attention in blocks
    of 1024 positions beside the gated diagonal recurrence (as wide as the model, gate blocks of 128 channels, 4 taps), alternating; the two
    middle layers form a loop that runs once.  128-wide attention heads, 4 query heads per key head."""
    H = width // 128
    G = max(1, H // 4)
    R = max(1, H // 2)
    mlp = {"kind": "dense", "ff": 3 * width}
    a = {"type": "parallel_2", "mlp": mlp,
         "mixer": {"left": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0, "rot": {"dims": 64, "base": 200000.0}, "mask": {"size": 1024}},
                   "right": {"heads": R, "dim": 64, "vdim": 128, "decay": [1.0 - 0.5 ** (4.5 + h) for h in range(R)], "rot": {"dims": 64, "base": 10000.0}},
                   "left_scale": 1.0, "right_scale": 1.0}}
    b = {"type": "parallel", "mlp": mlp, "mixer": {"left": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024}},
                                                   "right": {"width": width, "blocks": width // 128, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}}
    return {"architecture": "Lifesun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "loop": {"start": 1, "stop": 3, "times": 1}, "layers": [a, b, a, b]}


def time_lifesun_recurrences(dev, width, T):
    """The recurrence kernels of the Lifesun family alone at the bench's sizes, beside the like kernel of the closest model (linear attention
    with a decay per key channel): device time of one call over T tokens, the rate at which state elements are updated, and for the diagonal
    recurrence (one state number per channel: its bound is the traffic of its operands) the bytes it moves per second."""
    from crabml_b200 import CudaTensor, capi, seqops
    rng = np.random.default_rng(SEED)

    def rand(*shape, scale=1.0):
        return CudaTensor.new((rng.standard_normal(shape) * scale).astype(np.float32), list(shape), dev)

    def zeros(*shape):
        t = CudaTensor.alloc(list(shape), capi.F32, dev)
        seqops.tensor_zero(t)
        return t
    H = max(1, width // 256)
    out = {}

    def timed(name, f, **what):
        f()
        dev.synchronize(); dev.timer_begin()
        for _ in range(3):
            f()
        ms = dev.timer_end() / 3
        out[name] = dict(what, tokens=T, ms=ms)
        return ms
    q, k, v = rand(T, H * 64, scale=0.1), rand(T, H * 64, scale=0.1), rand(T, H * 128)
    decay, S = CudaTensor.new(np.asarray([1.0 - 0.5 ** (4.5 + h) for h in range(H)], np.float32), [H], dev), zeros(H, 64, 128)
    ms = timed("retention", lambda: seqops.retention(q, k, v, decay, 0.125, S, H, 64, 128), heads=H, dk=64, dv=128)
    out["retention"]["state_updates_per_s"] = T * H * 64 * 128 / (ms * 1e-3)
    z2, zb, S2 = rand(T, H * 64), zeros(H * 64), zeros(H, 64, 128)
    ms = timed("decayed_linear_attention (closest model)", lambda: seqops.decayed_linear_attention(q, k, v, z2, zb, 8.0, 0.125, S2, H, 64, 128), heads=H, dk=64, dv=128)
    out["decayed_linear_attention (closest model)"]["state_updates_per_s"] = T * H * 64 * 128 / (ms * 1e-3)
    C, B = width, width // 128
    u, y, yb, lam, st = rand(T, C), rand(T, C), zeros(C), CudaTensor.new(rng.uniform(-5, -1, C).astype(np.float32), [C], dev), zeros(C)
    gw, gb = rand(2 * C, C // B, scale=(C // B) ** -0.5), zeros(2 * C)
    gates = seqops.head_project(u, gw, B)
    ms = timed("gated_diagonal_recurrence", lambda: seqops.gated_diagonal_recurrence(u, gates, gb, lam, 8.0, B, st, y=y, y_bias=yb, y_act=capi.ACT_GELU_TANH), channels=C, blocks=B)
    out["gated_diagonal_recurrence"].update(bytes=5 * T * C * 4, bytes_per_s=5 * T * C * 4 / (ms * 1e-3))
    ms = timed("gate products of the diagonal recurrence (one per block, 32-bit)", lambda: seqops.head_project(u, gw, B), channels=C, blocks=B)
    out["gate products of the diagonal recurrence (one per block, 32-bit)"]["flop_per_s"] = 2 * T * 2 * C * (C // B) / (ms * 1e-3)
    xw, xb, tail = rand(C, 4), zeros(C), zeros(3, C)
    timed("short_conv_bias (4 taps, no activation)", lambda: seqops.short_conv_bias(u, xw, xb, tail, act=capi.ACT_NONE), channels=C)
    Hs = 2 * width // 64
    xbc, dt, hb, S3 = rand(T, Hs * 64 + 256, scale=0.3), rand(T, Hs), zeros(Hs), zeros(Hs, 128, 64)
    ms = timed("state_space_scan (closest model)", lambda: seqops.state_space_scan(xbc, dt, hb, hb, hb, S3, Hs, 1, 128, 64), heads=Hs, dk=128, dv=64)
    out["state_space_scan (closest model)"]["state_updates_per_s"] = T * Hs * 128 * 64 / (ms * 1e-3)
    return out


def run_lifesun(args, rank, world, local_rank):
    """Prefill and decode throughput of the Lifesun family at real layer sizes, beside the closest existing model -- the Vuzinex stack of
    the same width, depth and feed-forward width (run_vuzinex's configuration) -- through the same step function and slots; then the
    recurrence kernels alone beside the closest model's."""
    from crabml_b200 import CudaTensorDevice, lifesun, vuzinex
    if rank != 0:
        return
    width = int(args.workload.split("-w")[1])
    Tp, K, W = args.prefill_tokens, args.steps, args.warmup
    rng = np.random.default_rng(SEED)
    prompt = [int(v) for v in rng.integers(0, 32000, Tp)]
    sampler = ClockSampler(local_rank); sampler.start()
    out = {}
    for name, mod, cls, raw in (("lifesun", lifesun, "LifesunModel", lifesun_bench_config(width)), ("vuzinex", vuzinex, "VuzinexModel", vuzinex_bench_config(width))):
        conf = mod.parse_config(raw)
        dev = CudaTensorDevice(local_rank, lazy=0)
        weights = mod.random_weights(conf, SEED)
        model = getattr(mod, cls)(dev, conf, weights, "bfloat16", chunk=args.zatorax_chunk, max_seq=Tp + K + W + 8)
        params = sum(int(np.prod(np.shape(a))) for a in weights.values())
        del weights
        out[name] = measure_seq_model(dev, model, prompt, K, W, params)
        model.close()
        if name == "lifesun":
            out["recurrence_kernels"] = time_lifesun_recurrences(dev, width, min(Tp, 2048))
        dev.close()
    clocks = sampler.stop()
    z = out["lifesun"]
    line = {"metric": "decode_tokens_per_s", "value": z["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": z["decode_ms_per_token"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 matrices and product inputs, f32 everything else", "data": "synthetic",
            "config": {"workload": args.workload, "model": lifesun_bench_config(width), "prefill_tokens": Tp, "chunk": args.zatorax_chunk,
                       "closest_model": {"family": "vuzinex", "model": vuzinex_bench_config(width)}},
            "e2e": {"value": 1e3 / z["decode_wall_ms_per_token"], "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 32000 * 4},
            "gpu_launches": int(z["decode_launches_per_token"] * K), "detail": out, "clocks": clocks}
    print(json.dumps(line))


def run_zatorax(args, rank, world, local_rank):
    """Prefill and decode throughput of the Zatorax family at real layer sizes, beside the closest existing model -- a llama stack of the
    same width, depth, head layout and ACTIVE feed-forward width (Q8_0 weights, its serving format) -- through each family's runner.
    A prefill step = one `--prefill-tokens` prompt through model.step (logits of the last position read back); a decode step = one token."""
    from crabml_b200 import CudaTensorDevice, zatorax
    from crabml_b200 import runner as R
    if rank != 0:
        return
    width = int(args.workload.split("-w")[1])
    conf = zatorax.parse_config(zatorax_bench_config(width))
    Tp, K, W = args.prefill_tokens, args.steps, args.warmup
    rng = np.random.default_rng(SEED)
    prompt = [int(v) for v in rng.integers(0, conf["vocab"], Tp)]
    sampler = ClockSampler(local_rank); sampler.start()
    out = {}
    dev = CudaTensorDevice(local_rank, lazy=0)
    model = zatorax.ZatoraxModel(dev, conf, zatorax.random_weights(conf, SEED), "bfloat16", chunk=args.zatorax_chunk)
    params = sum(int(np.prod(sh)) if sh else 1 for sh in zatorax.expected_tensors(conf).values())
    out["zatorax"] = measure_seq_model(dev, model, prompt, K, W, params)
    dec_launches = out["zatorax"]["decode_launches_per_token"] * K
    model.close(); dev.close()
    # the closest existing model at equal size
    H = width // 128
    lconf = R.LlamaConfig(H, max(1, H // 4), len(conf["layers"]), width, 3 * width, Tp + K + W + 8, conf["vocab"], 1e-5, 128)
    for lazy in (0, 2):
        dev = CudaTensorDevice(local_rank, lazy=lazy)
        weights = R.synthetic_weights(dev, lconf, TYPE_ID["Q8_0"], TYPE_ID["Q8_0"], seed=SEED)
        r = R.LlamaRunner(dev, lconf, weights, Tp + K + W + 8)
        rec = {}
        if lazy == 0:
            r.forward(prompt[:64], 0)                                   # warm-up of the batched path, then a fresh runner for the timed prompt
            r.close()
            r = R.LlamaRunner(dev, lconf, weights, Tp + K + W + 8)
            dev.synchronize(); dev.timer_begin()
            r.forward(prompt, 0)
            rec["prefill_ms"] = dev.timer_end()
            rec["prefill_tok_s"] = Tp / (rec["prefill_ms"] * 1e-3)
            pos = Tp
        else:
            for i, t in enumerate(prompt[:32]):
                r.forward([t], i, export=False)
            pos = 32
        for _ in range(W):
            r.forward([prompt[0]], pos); pos += 1
        l0 = dev.launch_count()
        dev.synchronize(); dev.timer_begin()
        for _ in range(K):
            r.forward([prompt[0]], pos); pos += 1
        ms = dev.timer_end()
        rec.update({"decode_tok_s": K / (ms * 1e-3), "decode_ms_per_token": ms / K, "decode_launches_per_token": (dev.launch_count() - l0) / K, "kv_len_at_decode": pos})
        out["llama_q8_0_lazy%d" % lazy] = rec
        r.close(); dev.close()
    clocks = sampler.stop()
    z = out["zatorax"]
    line = {"metric": "decode_tokens_per_s", "value": z["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": z["decode_ms_per_token"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 matrices and product inputs, f32 everything else", "data": "synthetic",
            "config": {"workload": args.workload, "model": zatorax_bench_config(width), "prefill_tokens": Tp, "chunk": args.zatorax_chunk,
                       "closest_model": {"family": "llama", "weights": "Q8_0", "n_layers": lconf.n_layers, "dim": width, "hidden_dim": 3 * width, "heads": H, "kv_heads": lconf.n_kv_heads}},
            "e2e": {"value": K / (z["decode_wall_ms_per_token"] * K * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": conf["vocab"] * 4},
            "gpu_launches": int(dec_launches), "detail": out, "clocks": clocks}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="llama2-7b-q8_0", choices=sorted(WORKLOADS))
    ap.add_argument("--start-pos", type=int, default=32, help="KV-cache length before the timed decode steps")
    ap.add_argument("--lazy", type=int, default=2, help="2 = record+fuse, one persistent megakernel per token (default); 1 = fused kernels in a CUDA graph; 0 = one launch per trait call")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=4096)
    ap.add_argument("--no-also", action="store_true", help="skip the second (Q4_0) measurement of the default run")
    ap.add_argument("--multi", default="sharded", choices=["sharded", "replicas"], help="N > 1: shard one token stream (strong scaling, default) or run N independent replicas")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"], help="exchange transport of the sharded path: one-shot NVLink peer stores (default) or the NCCL baseline")
    ap.add_argument("--zatorax-chunk", type=int, default=512, help="zatorax / meresun / vuzinex / lifesun workloads: longest run of prompt tokens one pass takes")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload.startswith("zatorax-"):
        run_zatorax(args, rank, world, local_rank)
    elif args.workload.startswith("meresun-"):
        run_meresun(args, rank, world, local_rank)
    elif args.workload.startswith("vuzinex-"):
        run_vuzinex(args, rank, world, local_rank)
    elif args.workload.startswith("lifesun-"):
        run_lifesun(args, rank, world, local_rank)
    elif args.workload.endswith("-prefill"):
        run_prefill(args, rank, world, local_rank)
    else:
        run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
