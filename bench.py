#!/usr/bin/env python
"""Benchmark of the per-step decode sampling path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: configuration 3 of the baseline - batch 1024, vocab 128256, bf16 logits ~ N(0, 2.5^2), mixed
per-row top-k in {0,1,40,1024} / top-p in {0,0.5,0.95}, repetition penalty 1.1 over a 512-token prompt
plus everything generated so far, 8 bad words per row, end id 128001, length criterion.  Seeded synthetic
logits stand in for a model (no dataset is involved).  A step is one pass of the path over the batch:
the fused sampling step (the single-pass kernels of the top-p and of the top-k rows side by side, then the
general kernel on the rows they leave), the stop-criteria kernel and the host read of should_stop.

One JSON line on stdout (rank 0):
  value      sampled tokens/s with the logits resident in HBM (4 distinct 263 MB buffers rotate, so no
             step finds its logits in the 126 MB L2), CUDA events around exactly K steps, max over ranks
  e2e        same metric with the step's logits starting in pinned HOST memory and the sampled ids read
             back to the host, copies inside the timed region
  roofline   algorithmic bytes of one step / the mean CUDA-event duration of its sampling launches,
             against the measured HBM copy bandwidth (MEASURED_PEAKS.json)
  e2e_cpp_classes  (N = 1) the end-to-end leg once more with the host side in C++ (the driver of the C++
             decode layers, fastertransformer_b200/lib/shim_driver)
  other_configs    (N > 1) config 5 (vocabulary in N shards, one all-gather per step) and config 4 (beam
             search, batch-sharded) measured in the same process group
  cpu_baseline  the CPU oracle (oracle/ft_oracle.cpp) on a bounded sample, all host cores
--impl reference times the unmodified FasterTransformer kernels (oracle/_ref, built for sm_100a from the
reference sources) on the same workload, seeds and rank layout through the reference's own
DynamicDecodeLayer<float> (on every rank at N > 1); the reference has no bf16 path, so it is fed the lossless
fp32 up-cast, as its own models do.
"""
import argparse
import copy
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))  # ft_oracle / ft_reference drivers (checkers, not product)

import numpy as np  # noqa: E402
import torch  # noqa: E402

N_BUFFERS = 4
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index, period=0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=1.0)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        # NCCL prints its version banner on stdout when the communicator is created; stdout carries the JSON line
        # only, so file descriptor 1 points at stderr until the first collective has run
        torch.cuda.set_device(local)
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def cpu_baseline(w, rows=64):
    """The CPU oracle on the first `rows` rows of step 0 of the workload, all host cores."""
    from ft_oracle import OracleDynamicDecodeLayer, bf16_bits
    rows = min(rows, w.batch)
    args = {}
    for k, v in w.runtime_args.items():
        v = np.atleast_1d(np.asarray(v))
        args[k] = v[:rows] if v.size == w.batch else v
    orc = OracleDynamicDecodeLayer(w.vocab, w.vocab_padded, "bfloat16")
    orc.setup(rows, 1, args)
    g = np.random.default_rng(w.seed)
    logits = (g.standard_normal((rows, w.vocab_padded), dtype=np.float32) * w.sigma)
    out = {"output_ids": np.zeros((w.max_input_length + 2, rows), np.int32),
           "finished": np.zeros(rows, np.bool_),
           "sequence_length": np.full(rows, w.max_input_length, np.int32)}
    out["output_ids"][: w.max_input_length] = w.prompt[:, :rows]
    inp = {"logits": bf16_bits(logits), "step": w.max_input_length, "max_input_length": w.max_input_length,
           "end_id": np.full(rows, w.end_id, np.int32),
           "input_lengths": np.full(rows, w.max_input_length, np.int32),
           "bad_words_list": None if w.bad_words is None else w.bad_words[:rows]}
    u = 1.0 - g.random(rows, dtype=np.float32)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0 or reps < 2:
        orc.forward(out, inp, u, u)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": rows / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": "%d rows x 1 step of the same workload, %d repetitions, OpenMP over rows" % (rows, reps)}


def workload_seed(wname, rank):
    """Seed of the synthetic logits: the same for both arms, one stream per rank."""
    return (1237 if wname == "c3" else 1234 + int(wname[1])) + rank


def metric_name(wname, B, vocab):
    if wname == "c3":
        return "sampled tokens/sec and achieved HBM GB/s (% of roofline) at batch 1024, vocab 128256"
    return "sampled tokens/sec and achieved HBM GB/s (config %s: batch %d, vocab %d)" % (wname[1], B, vocab)


def workload_config(wname, B, vocab, first_step, K, n_buffers, world):
    """The `config` object of the JSON line: identical for both arms on the same workload."""
    label = {"c1": "c1: top-k 50, T 1.0, repetition 1.2, batch %d x vocab %d fp32",
             "c2": "c2: top-p 0.9, T 0.8, presence 0.5, min_length 16, batch %d x vocab %d fp16",
             "c3": "c3: mixed per-row top-k/top-p, batch %d x vocab %d bf16, repetition 1.1, "
                   "8 bad words/row, length criterion"}[wname] % (B, vocab)
    return {"workload": label, "rows_per_gpu": B, "history_tokens": "%d..%d" % (first_step, first_step + K),
            "l2": "%d logits buffers rotate, every one larger than the 126 MB L2 or all of them together "
                  "more than twice its size; each time round the batch starts one row further down its buffer" % n_buffers,
            "parallelism": "batch-sharded, no collective" if world > 1 else "single GPU"}


def n_buffers_for(B, vocab_padded, element_size):
    # enough rotating buffers that a step never finds its logits in the 126 MB L2
    return max(4, min(200, -(-300_000_000 // (B * vocab_padded * element_size))))


POOL_EXTRA_ROWS = 61  # a buffer holds this many rows more than the batch (see step_logits)


def make_pool(w, device, dtype, n):
    """`n` logits buffers of batch + POOL_EXTRA_ROWS rows each."""
    wide = copy.copy(w)
    wide.batch = w.batch + POOL_EXTRA_ROWS
    pool = []
    for i in range(n):
        x = wide.logits(10_000 + i, device)
        pool.append(x if dtype == w.dtype else x.to(dtype))
    return pool


def step_logits(pool, it, batch):
    """Logits of the `it`-th step of a run: the buffers rotate (so that no step finds its logits in L2), and each
    time round the batch starts one row further down its buffer, so that a row does not meet the same logits
    again every len(pool) steps - a model never repeats them, and a row that decodes greedily would otherwise put
    the largest columns of those few vectors into its own history one by one.  A contiguous view; the row pitch
    is a multiple of 16 bytes for every configuration."""
    buf = pool[it % len(pool)]
    off = (it // len(pool)) % (POOL_EXTRA_ROWS + 1)
    return buf[off:off + batch]


def run_ours(a, rank, world, local):
    from fastertransformer_b200 import DynamicDecodeLayer
    from fastertransformer_b200.workloads import algorithmic_bytes_per_step, make_workload
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    K, W = a.steps, a.warmup
    e2e_steps = min(K, 16)
    wname = a.workload if a.workload in ("c1", "c2") else "c3"
    w = make_workload(wname, batch=a.batch, steps=W + K + e2e_steps + 40, seed=workload_seed(wname, rank))
    B = w.batch
    layer = DynamicDecodeLayer(w.vocab, w.vocab_padded, w.dtype, device)
    layer.setup(B, 1, w.runtime_args)
    st = w.initial_state(device)
    inputs = w.static_inputs(device)
    N_BUFFERS = n_buffers_for(B, w.vocab_padded, torch.empty(0, dtype=w.dtype).element_size())
    pool = make_pool(w, device, w.dtype, N_BUFFERS)
    torch.cuda.synchronize()

    step_no = [w.max_input_length]

    def one_step(logits=None):
        it = step_no[0] - w.max_input_length
        layer.forward(st, dict(inputs, logits=step_logits(pool, it, B) if logits is None else logits, step=step_no[0]))
        step_no[0] += 1

    for i in range(W):
        one_step()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    launches0 = layer.launches
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    first_step = step_no[0]
    ev0.record()
    for i in range(K):
        # the event pair brackets the fused sampling launch; the criteria kernel follows it
        kev[i][0].record()
        one_step()
        kev[i][1].record()
    ev1.record()
    torch.cuda.synchronize()
    barrier(world)
    clocks = sampler.stop()
    launches = layer.launches - launches0
    ms_total = ev0.elapsed_time(ev1)
    ms_total = max_over_ranks(ms_total, world, device)
    step_ms = [p[0].elapsed_time(p[1]) for p in kev]

    # kernel-only duration of the fused launch: events directly around the C-ABI call
    layer.time_kernels = True
    for i in range(min(K, 32)):
        one_step()
    torch.cuda.synchronize()
    layer.time_kernels = False
    kern_ms = [e0.elapsed_time(e1) for e0, e1 in layer.kernel_events]
    kern_ms_mean = float(np.mean(kern_ms))

    # end to end: logits start in pinned host memory, ids come back to the host, every step
    host_pool = [torch.empty(B, w.vocab_padded, dtype=w.dtype).pin_memory() for _ in range(2)]
    for h, d in zip(host_pool, pool):
        h.copy_(d[:B])
    # two device buffers: the copy of the next step's logits (copy stream) runs under this step's kernel; every
    # copy, every kernel and every read-back of the ids lies inside the timed region
    dev_logits = [torch.empty_like(pool[0][:B]) for _ in range(2)]
    ids_host = torch.empty(B, dtype=torch.int32).pin_memory()
    copy_stream = torch.cuda.Stream(device=device)
    main = torch.cuda.current_stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def start_copy(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])      # the kernel that read this buffer last has finished
            dev_logits[b].copy_(host_pool[b], non_blocking=True)
            copied[b].record(copy_stream)

    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for b in range(2):
        consumed[b].record(main)
    start_copy(0)
    for i in range(e2e_steps):
        if i + 1 < e2e_steps:
            start_copy(i + 1)
        main.wait_event(copied[i % 2])
        s = step_no[0]
        one_step(dev_logits[i % 2])
        consumed[i % 2].record(main)
        ids_host.copy_(st["output_ids"][s], non_blocking=True)
        main.synchronize()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, device)

    peak, peak_kind = measured_peak()
    alg_bytes = float(np.mean([algorithmic_bytes_per_step(w, first_step + i) for i in range(K)]))
    achieved = alg_bytes / (kern_ms_mean * 1e-3) / 1e9
    es = pool[0].element_size()
    line = {
        "metric": metric_name(wname, B, w.vocab),
        "value": world * B * K / (ms_total * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_total / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"c1": "fp32", "c2": "fp16 logits and probabilities", "c3": "bf16 logits, fp32 arithmetic"}[wname],
        "data": "synthetic",
        "config": workload_config(wname, B, w.vocab, first_step, K, N_BUFFERS, world),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": a.traffic if wname == "c3" and B == 1024 else None, "peak_kind": peak_kind,
                     "kernel": ("decode_sampling_kernel<f32>" if wname == "c1" else
                                "fused sampling step: fast_sampling_kernel<%s> (top-k rows) and (top-p rows) side by side, "
                                "then decode_sampling_kernel on the rows they leave" % {"c2": "f16", "c3": "bf16"}[wname]),
                     "kernel_ms": kern_ms_mean,
                     "algorithmic_bytes_per_launch": alg_bytes},
        "e2e": {"value": world * B * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": B * w.vocab_padded * es, "d2h_bytes_per_step": B * 4 + 4,
                "steps": e2e_steps},
        "gpu_launches": launches,
        "clocks": clocks,
        "step_ms_median": float(np.median(step_ms)),
    }
    if rank == 0 and world == 1 and not a.no_cpu:
        line["cpu_baseline"] = cpu_baseline(w)
    return line


def e2e_through_cpp_classes(rows=1024, vocab=128256, steps=12):
    """The end-to-end leg once more with the host side in C++: the driver of the C++ decode layers
    (tests/cpp/shim_driver.cc, built to fastertransformer_b200/lib/shim_driver) copies bf16 logits from pinned host
    memory, calls fastertransformer::DynamicDecodeLayer<__nv_bfloat16>::forward and reads the ids back, every step,
    and prints the rate itself.  Rows mix k in {0, 1, 8, 64} with p in {0, 0.5, 0.9}, repetition penalty 1.2."""
    exe = os.path.join(ROOT, "fastertransformer_b200", "lib", "shim_driver")
    if not os.path.exists(exe):
        return {"unavailable": "fastertransformer_b200/lib/shim_driver is not built"}
    try:
        r = subprocess.run([exe, "bf16", str(rows), str(vocab), str(steps), "e2e"], capture_output=True, text=True,
                           timeout=600)
    except subprocess.TimeoutExpired:
        return {"unavailable": "shim_driver did not finish in 600 s"}
    for ln in r.stdout.split("\n"):
        if ln.startswith("e2e "):
            f = dict(kv.split("=") for kv in ln.split()[1:])
            return {"value": float(f["tokens_per_s"]), "unit": "tokens/s", "ms_per_step": float(f["ms_per_step"]),
                    "steps": int(f["steps"]), "h2d_bytes_per_step": int(f["h2d_bytes"]),
                    "d2h_bytes_per_step": int(f["d2h_bytes"]),
                    "workload": "batch %d x vocab %d bf16 through DynamicDecodeLayer<__nv_bfloat16> (C++)" % (rows, vocab)}
    return {"unavailable": "shim_driver exit %d: %s" % (r.returncode, r.stderr[-200:])}


def run_beam(a, rank, world, local, reference=False):
    """Config 4: beam search via online-softmax top-k. Batch 64 x beam 4 x vocab 32000 fp16, length penalty 1.0,
    cum_log_probs ~ N(-5, 1), end id 2; the batch is the unit that shards over GPUs (weak scaling here)."""
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    B, K, V, mil = 64, 4, 32000, 4
    steps, W = a.steps, a.warmup
    L = mil + steps + W + 2
    if reference:
        import ft_reference
        if rank != 0:
            return None
        if not ft_reference.available():
            return {"impl": "reference", "unavailable": "oracle/_ref/libft_decode_ref.so is not built on this box"}
        layer = ft_reference.RefDynamicDecodeLayer(V, V, torch.float16, device)
    else:
        from fastertransformer_b200 import DynamicDecodeLayer
        layer = DynamicDecodeLayer(V, V, torch.float16, device)
    g = torch.Generator(device=device)
    g.manual_seed(4 + rank)
    st = {"output_ids": torch.zeros(L, B, K, dtype=torch.int32, device=device),
          "parent_ids": torch.zeros(L, B, K, dtype=torch.int32, device=device),
          "finished": torch.zeros(B * K, dtype=torch.bool, device=device),
          "sequence_length": torch.full((B * K,), mil, dtype=torch.int32, device=device),
          "cum_log_probs": torch.randn(B * K, generator=g, device=device) - 5.0,
          "tgt_cache_indirection": torch.zeros(B, K, L, dtype=torch.int32, device=device)}
    src = torch.zeros(B, K, L, dtype=torch.int32, device=device)
    args = {"len_penalty": np.asarray([1.0], np.float32)}
    layer.setup(B, K, args)
    pool = [(torch.randn(B, K, V, generator=g, device=device) * 2.0).half() for _ in range(4)]
    work = torch.empty_like(pool[0])
    end = torch.full((B,), 2, dtype=torch.int32, device=device)
    il = torch.full((B, K), mil, dtype=torch.int32, device=device)
    total_ms, n = 0.0, 0
    for i in range(W + steps):
        work.copy_(pool[i % 4])
        inp = dict(args, logits=work, step=mil + i, max_input_length=mil, ite=0, local_batch_size=B, end_id=end,
                   input_lengths=il, src_cache_indirection=src)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        layer.forward(st, inp)
        e1.record()
        torch.cuda.synchronize()
        src, st["tgt_cache_indirection"] = st["tgt_cache_indirection"], src
        if i >= W:
            total_ms += e0.elapsed_time(e1)
            n += 1
    total_ms = max_over_ranks(total_ms, world, device)
    peak, peak_kind = measured_peak()
    alg = B * K * V * 2.0
    line = {"metric": "beam-search tokens/sec (config 4: batch 64 x beam 4 x vocab 32000 fp16)",
            "value": world * B * K * n / (total_ms * 1e-3), "unit": "beam-tokens/s", "n_gpus": world, "steps": steps,
            "warmup": W, "ms_per_step": total_ms / n, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 logits, fp32 soft-max statistics", "data": "synthetic",
            "config": {"workload": "c4: online-softmax beam top-k, batch 64 x beam 4 x vocab 32000, len_penalty 1.0"},
            "roofline": {"bound": "hbm", "achieved": alg / (total_ms / n * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (total_ms / n * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                         "note": "16 MB per step: launch- and latency-bound, reported for completeness"}}
    if reference:
        line["impl"] = "reference"
    return line


def run_vocab_parallel(a, rank, world, local):
    """Config 5: batch 2048, vocab 256000 as `world` column shards, bf16 N(0, 3^2), k=64, p=0.92, T=0.7.
    Each rank reads its shard once, one NCCL all-gather moves (64+64+1)*8 bytes per row per rank, every rank
    merges and draws.  With one GPU all shards run on it (no communication) so that the arithmetic can be timed."""
    from fastertransformer_b200.vocab_parallel import VocabParallelSampler
    import torch.distributed as dist
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    B, V, k, mil = 2048, 256000, 64, 4
    n_shards = world if world > 1 else 8
    shard = V // n_shards
    steps, W = a.steps, a.warmup
    args = {"runtime_top_k": np.asarray([k], np.uint32), "runtime_top_p": np.asarray([0.92], np.float32),
            "temperature": np.asarray([0.7], np.float32), "random_seed": np.asarray([3], np.uint64)}
    vp = VocabParallelSampler(V, shard, n_shards, torch.bfloat16, device)
    vp.setup(B, 1, args)
    g = torch.Generator(device=device)
    g.manual_seed(500 + rank)
    my_shards = [rank] if world > 1 else list(range(n_shards))
    pool = [[(torch.randn(B, shard, generator=g, device=device) * 3.0).bfloat16() for _ in my_shards] for _ in range(2)]
    st = {"output_ids": torch.zeros(mil + steps + W + 1, B, dtype=torch.int32, device=device),
          "finished": torch.zeros(B, dtype=torch.bool, device=device),
          "sequence_length": torch.full((B,), mil, dtype=torch.int32, device=device)}
    end = torch.full((B,), V - 1, dtype=torch.int32, device=device)
    for i in range(W):
        inp = {"step": mil + i, "max_input_length": mil, "end_id": end}
        vp.forward_rank(st, inp, pool[i % 2][0], rank) if world > 1 else vp.forward_shards(st, inp, pool[i % 2])
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(W, W + steps):
        inp = {"step": mil + i, "max_input_length": mil, "end_id": end}
        vp.forward_rank(st, inp, pool[i % 2][0], rank) if world > 1 else vp.forward_shards(st, inp, pool[i % 2])
    e1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1), world, device)
    if world > 1:
        ids = st["output_ids"][mil + W].clone()
        ref = ids.clone()
        dist.broadcast(ref, 0)
        same = int(torch.equal(ids, ref))
        t = torch.tensor([same], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        same = int(t.item())
    else:
        same = 1
    peak, peak_kind = measured_peak()
    alg = B * shard * 2.0 * (1 if world > 1 else n_shards)
    return {"metric": "vocabulary-parallel sampled tokens/sec (config 5: batch 2048, vocab 256000)",
            "value": B * steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": W,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 logits", "data": "synthetic",
            "config": {"workload": "c5: vocab 256000 in %d shards of %d, batch 2048, k=64, p=0.92, T=0.7" % (n_shards, shard),
                       "allgather_bytes_per_rank": B * (2 + vp.cap) * 8, "ids_identical_on_all_ranks": bool(same),
                       "overflow_rows": vp.overflow_count()},
            "roofline": {"bound": "hbm", "achieved": alg / (ms / steps * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms / steps * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind},
            "gpu_launches": vp.launches}


def run_reference(a, rank, world, local):
    """The unmodified reference on the same workload: every rank runs its own batch (the rank's seed, as in the
    other arm), value = all rows of all ranks / the slowest rank's time."""
    import ft_reference
    from fastertransformer_b200.workloads import make_workload
    if not ft_reference.available():
        return {"impl": "reference", "unavailable": "oracle/_ref/libft_decode_ref.so is not built on this box"}
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    K, W = a.steps, a.warmup
    wname = a.workload if a.workload in ("c1", "c2") else "c3"
    w = make_workload(wname, batch=a.batch, steps=W + K + 4, seed=workload_seed(wname, rank))
    B = w.batch
    ref_dt = torch.float32 if w.dtype == torch.bfloat16 else w.dtype  # the reference has float and half only
    layer = ft_reference.RefDynamicDecodeLayer(w.vocab, w.vocab_padded, ref_dt, device)
    layer.setup(B, 1, w.runtime_args)
    st = w.initial_state(device)
    inputs = w.static_inputs(device)
    n_buffers = n_buffers_for(B, w.vocab_padded, torch.empty(0, dtype=w.dtype).element_size())
    pool = make_pool(w, device, ref_dt, min(n_buffers, 4))
    work = torch.empty_like(pool[0][:B])
    sampler = ClockSampler(local, period=0.02)
    total_ms, n = 0.0, 0
    barrier(world)
    for i in range(W + K):
        if i == W:
            sampler.start()
        step = w.max_input_length + i
        work.copy_(step_logits(pool, i, B))  # the reference overwrites its logits; a model would produce fresh ones
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        layer.forward(st, dict(inputs, logits=work.view(B, 1, w.vocab_padded), step=step))
        e1.record()
        torch.cuda.synchronize()
        if i >= W:
            total_ms += e0.elapsed_time(e1)
            n += 1
    clocks = sampler.stop()
    total_ms = max_over_ranks(total_ms, world, device)
    val = world * B * n / (total_ms * 1e-3)
    return {
        "impl": "reference",
        "metric": metric_name(wname, B, w.vocab),
        "value": val, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": total_ms / n,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (up-cast of the bf16 logits; the reference has no bf16 path)" if wname == "c3"
        else str(ref_dt).replace("torch.", ""), "data": "synthetic",
        "config": workload_config(wname, B, w.vocab, w.max_input_length + W, K, n_buffers, world),
        "reference": "unmodified FasterTransformer DynamicDecodeLayer compiled for sm_100a (oracle/_ref), logits "
                     "resident in HBM, CUDA events around each forward(), every rank its own batch",
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": 0, "kind": "reference",
                         "sample": "the reference's own CUDA kernels on the GPU, full batch, %d steps" % n},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "clocks": clocks,
    }


def run_log_probs(a, rank, world, local, reference=False):
    """Context log-probs (invokeLogProbFromLogits): 512 positions x 32 sequences x vocab 50257 fp16, 1.65 GB of
    logits per step per GPU (larger than L2, so no flush is needed); sequences shard over GPUs, no collective."""
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    L, B, V = 512, 32, 50257
    steps, W = a.steps, a.warmup
    if reference:
        import ft_reference
        if rank != 0:
            return None
        if not ft_reference.available():
            return {"impl": "reference", "unavailable": "oracle/_ref/libft_decode_ref.so is not built on this box"}
        fn = ft_reference.ref_lib().ftref_log_prob_from_logits
    else:
        from fastertransformer_b200 import lib
        fn = lib.ftb200_log_prob_from_logits
    g = torch.Generator(device=device)
    g.manual_seed(40 + rank)
    logits = torch.empty(L, B, V, dtype=torch.float16, device=device)
    for t in range(0, L, 64):   # filled in slices: no fp32 copy of the whole tensor
        logits[t:t + 64] = (torch.rand(64, B, V, generator=g, device=device) * 6 - 3).half()
    ids = torch.randint(0, V, (L, B), generator=g, device=device, dtype=torch.int32)
    lens = torch.full((B,), L, dtype=torch.int32, device=device)
    ws = torch.zeros(L * B, dtype=torch.float32, device=device)
    cum = torch.zeros(B, dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        rc = fn(cum.data_ptr(), logits.data_ptr(), 1, ids.data_ptr(), lens.data_ptr(), L, B, V, V, ws.data_ptr(),
                ws.numel() * 4, stream, 0)
        assert rc == 0, rc

    sampler = ClockSampler(local)
    for _ in range(W):
        step()
    barrier(world)
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    barrier(world)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world, device) / steps
    peak, peak_kind = measured_peak()
    alg = float(L - 1) * B * V * 2.0
    tokens = float(L - 1) * B
    line = {"metric": "context log-prob positions/sec (512 x 32 x vocab 50257 fp16)",
            "value": world * tokens / (ms * 1e-3), "unit": "positions/s", "n_gpus": world, "steps": steps, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16 logits, fp32 soft-max statistics", "data": "synthetic",
            "config": {"workload": "lp: log softmax(logits)[ids] summed per sequence, 512 positions x 32 sequences x "
                                   "vocab 50257 fp16 per GPU", "l2": "1.65 GB of logits per step, larger than L2"},
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                         "note": "algorithmic bytes = scored positions x vocab x 2 B; both kernels of the entry timed"},
            "gpu_launches": 2 * steps, "clocks": clocks}
    if reference:
        line["impl"] = "reference"
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="rows per GPU (default: the configuration's own)")
    ap.add_argument("--workload", default="c3", choices=["c1", "c2", "c3", "c4", "c5", "lp"],
                    help="c3 (default, the headline) | c1 / c2 the small sampling configurations | c4 beam search | "
                         "c5 vocabulary-parallel | lp context log-probs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg and the C++-classes leg")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="at N > 1: skip the config 5 / config 4 measurements added to the line")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the fused kernel from an ncu capture (profiles/)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if a.traffic is None:
        p = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(p):
            try:
                a.traffic = float(json.load(open(p))["dram_bytes_per_launch_c3"])
            except Exception:
                a.traffic = None
    rank, world, local = dist_setup(a.gpus)
    if a.workload == "c4":
        line = run_beam(a, rank, world, local, reference=a.impl == "reference")
    elif a.workload == "c5":
        line = run_vocab_parallel(a, rank, world, local)
    elif a.workload == "lp":
        line = run_log_probs(a, rank, world, local, reference=a.impl == "reference")
    elif a.impl == "reference":
        line = run_reference(a, rank, world, local)
    else:
        line = run_ours(a, rank, world, local)
        if world > 1 and a.workload == "c3" and not a.no_other_configs:
            # the configurations that exist only on several GPUs, measured in the same process group: config 5
            # (vocabulary in `world` shards, one all-gather per step) and config 4 (beam search, batch sharded)
            b = copy.copy(a)
            b.steps, b.warmup, b.batch = min(a.steps, 32), 3, None
            other = {}
            for name, leg in (("c5", run_vocab_parallel), ("c4", run_beam)):
                got = leg(b, rank, world, local)
                other[name] = {"ms_per_step": got["ms_per_step"], "value": got["value"], "unit": got["unit"],
                               "scaling": got["scaling"], "steps": got["steps"], "config": got["config"],
                               "roofline_frac": got["roofline"]["frac"]}
            line["other_configs"] = other
        if world == 1 and rank == 0 and a.workload == "c3" and not a.no_cpu:
            line["e2e_cpp_classes"] = e2e_through_cpp_classes()
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
