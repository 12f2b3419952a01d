#!/usr/bin/env python
"""Benchmark of the dense-matmul / policy-MLP hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `holdem_train`: one SGD training step (forward, cross-entropy
backward with dgrad + wgrad GEMMs, gradient all-reduce when N > 1, SGD) of the
NL-Hold'em-sized policy MLP 512-1024x4-10, bf16 inputs / fp32 accumulate, global
batch 262144 sharded over the N GPUs (strong scaling), synthetic seeded inputs
resident in HBM.  One JSON line is printed by rank 0:

  value      samples/s of the whole job, device-timed (CUDA events, max over ranks)
  e2e        the same step through the public Python API with host buffers: every step
             copies its inputs from pinned host memory and reads the loss back
  roofline   the dominant kernel (tcgen05 GEMM): algorithmic flops / CUDA-event time of
             the GEMM launches, against the measured cuBLAS bf16 peak of this pool
  cpu_baseline  the NumPy oracle's training step on the host cores (bounded sample)
  extra      GEMM TFLOP/s of the 4096^3 layout sweep and the other policy workloads

`--impl reference` times the CPU implementation (NumPy, all host threads) of the
same step on a bounded sample; under torchrun only rank 0 runs it.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "spiral-s-ml-library_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

HOLDEM_SIZES = [512, 1024, 1024, 1024, 1024, 10]
LEDUC_SIZES = [32, 256, 256, 256, 3]
WORKLOADS = {
    # name: (sizes, global batch, in_dtype, training)
    "holdem_train": (HOLDEM_SIZES, 262144, "bf16", True),
    "holdem_infer": (HOLDEM_SIZES, 262144, "bf16", False),
    "leduc_train": (LEDUC_SIZES, 65536, "bf16", True),
    "leduc_infer": (LEDUC_SIZES, 16384, "f16", False),
}
LR = 1e-3
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["source"] = "fallback"
    return d


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            if t0 is not None and not (t0 <= ts <= t1 + 0.2):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class PinnedBuffer:
    """Page-locked host memory viewed as a NumPy array (source of the end-to-end copies)."""

    def __init__(self, array):
        import ctypes
        from spiral_b200 import _lib
        array = np.ascontiguousarray(array)
        p = ctypes.c_void_p()
        _lib.call("sb_malloc_host", ctypes.byref(p), array.nbytes)
        self.ptr, self.nbytes = p.value, array.nbytes
        buf = (ctypes.c_char * array.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=array.dtype).reshape(array.shape)
        self.array[...] = array

    def copy_to(self, dev, stream=None):
        from spiral_b200 import _lib
        _lib.call("sb_memcpy_h2d", dev.ptr, self.ptr, self.nbytes, stream)


def numpy_step(x, ws, bs, mask, target, training):
    from oracle import spiral_oracle as so
    if training:
        so.mlp_train_step(x, ws, bs, mask, target, LR, exact=False)
    else:
        so.mlp_forward(x, ws, bs, mask, exact=False)


def cpu_reference(workload, steps, warmup, sample_rows):
    """Times the NumPy restatement (float32 BLAS, all host threads) on `sample_rows` rows per step."""
    from oracle import spiral_oracle as so
    sizes, _, _, training = WORKLOADS[workload]
    ws, bs = so.mlp_weights(5, sizes)
    if sizes[0] == 32:
        x, mask = so.leduc_inputs(5, sample_rows)
    else:
        x, mask = so.holdem_inputs(5, sample_rows, features=sizes[0], actions=sizes[-1])
    target = so.random_target(55, mask)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host thread it may.
    try:
        from threadpoolctl import threadpool_limits, threadpool_info
        limiter = threadpool_limits(limits=cores)
    except Exception:
        limiter, threadpool_info = None, None
    try:
        for _ in range(warmup):
            numpy_step(x, ws, bs, mask, target, training)
        t0 = time.perf_counter()
        for _ in range(steps):
            numpy_step(x, ws, bs, mask, target, training)
        dt = (time.perf_counter() - t0) / max(1, steps)
        if threadpool_info is not None:
            used = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
            cores = max(used) if used else 1
    finally:
        if limiter is not None:
            limiter.restore_original_limits()
    return sample_rows / dt, dt * 1e3, cores


def run_reference(args, rank):
    if rank != 0:
        return
    workload = args.workload
    sizes, gbatch, in_dtype, training = WORKLOADS[workload]
    rows = 8192 if sizes[0] == 512 else 65536
    value, ms, cores = cpu_reference(workload, args.steps, args.warmup, rows)
    sample = "NumPy float32 %s step on %d rows of the workload per step" % ("training" if training else "forward", rows)
    line = {
        "impl": "reference", "metric": "policy_mlp_%s_samples_per_sec" % ("train" if training else "infer"),
        "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "layers": sizes, "global_batch": gbatch, "sample_rows_per_step": rows},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample,
                         "sample_rows_per_step": rows},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def gemm_sweep(sb, iters=10):
    """GEMM TFLOP/s at 4096^3 (benchmark configuration 2): layouts NN/NT/TN, bf16 / f16 / tf32 inputs."""
    out = {}
    m = n = k = 4096
    rng = np.random.Generator(np.random.Philox(2))
    host = rng.standard_normal((4096, 4096), dtype=np.float32)
    flush = sb.DeviceArray((192 * 1024 * 1024,), "u8")
    for dt in ("bf16", "f16", "tf32"):
        a = sb.DeviceArray.from_numpy(host, dt)
        b = sb.DeviceArray.from_numpy(host.T.copy(), dt)
        c = sb.DeviceArray((m, n), "f32")
        for name, (at, bt) in (("NT", (False, True)), ("NN", (False, False)), ("TN", (True, False))):
            for _ in range(3):
                sb.matmul(at, bt, 1.0, a, b, 0.0, c, in_dtype=dt)
            total = 0.0
            for _ in range(iters):
                flush.fill_zero()                      # 192 MiB write: evicts the 126 MB L2
                e0, e1 = sb.Event().record(), None
                sb.matmul(at, bt, 1.0, a, b, 0.0, c, in_dtype=dt)
                e1 = sb.Event().record()
                total += e0.elapsed_ms(e1)
            out["%s_%s" % (dt, name)] = round(2.0 * m * n * k / (total / iters) / 1e9, 1)
    return out


def gemm_small_cases(sb, iters=20):
    """Benchmark configuration 1 (512^3 NT fp32, uniform[-1,1), in the fp32-exact and TF32 classes)
    and configuration 2's ragged case (4000 x 3000 x 1000), as microseconds and TFLOP/s."""
    out = {}
    rng = np.random.Generator(np.random.Philox(1))
    cases = [("cfg1_512_fp32_NT", 512, 512, 512, "f32", False, True), ("cfg1_512_tf32_NT", 512, 512, 512, "tf32", False, True),
             ("ragged_bf16_NT", 4000, 3000, 1000, "bf16", False, True), ("ragged_bf16_NN", 4000, 3000, 1000, "bf16", False, False),
             ("ragged_bf16_TN", 4000, 3000, 1000, "bf16", True, False), ("ragged_tf32_NT", 4000, 3000, 1000, "tf32", False, True)]
    for name, m, n, k, dt, at, bt in cases:
        a = sb.DeviceArray.from_numpy(rng.uniform(-1, 1, size=(k, m) if at else (m, k)).astype(np.float32), "f32" if dt == "f32" else dt)
        b = sb.DeviceArray.from_numpy(rng.uniform(-1, 1, size=(n, k) if bt else (k, n)).astype(np.float32), "f32" if dt == "f32" else dt)
        c = sb.DeviceArray((m, n), "f32")
        for _ in range(3):
            sb.matmul(at, bt, 1.0, a, b, 0.0, c, in_dtype=dt)
        e0 = sb.Event().record()
        for _ in range(iters):
            sb.matmul(at, bt, 1.0, a, b, 0.0, c, in_dtype=dt)
        e1 = sb.Event().record()
        ms = e0.elapsed_ms(e1) / iters
        out[name] = {"us": round(ms * 1e3, 2), "tflops": round(2.0 * m * n * k / ms / 1e9, 1)}
    return out


def reference_kernel_row(sb):
    """The reference's own TF32 WMMA GEMM (recompiled for sm_100a by oracle/build_ref.py) and this
    library's TF32 GEMM on the reference's baked shape, 8192 x 8192 x 4096 NT, alpha = beta = 1."""
    try:
        from oracle import ref_kernel
        if not ref_kernel.available():
            return None
        m, n, k = 8192, 8192, 4096
        a = sb.DeviceArray.zeros((m, k), "f32")
        b = sb.DeviceArray.zeros((n, k), "f32")
        c = sb.DeviceArray.zeros((m, n), "f32")
        rng = np.random.Generator(np.random.Philox(11))
        a.upload(rng.standard_normal((m, k), dtype=np.float32))
        b.upload(rng.standard_normal((n, k), dtype=np.float32))
        ref = ref_kernel.ReferenceMatmul()
        out = {}
        for name, fn in (("reference", lambda: ref.launch(a.ptr, b.ptr, c.ptr)),
                         ("ours", lambda: sb.matmul_tf32(False, True, 1.0, a, b, 1.0, c))):
            c.fill_zero()
            fn()
            sb.synchronize()
            e0 = sb.Event().record()
            fn()
            fn()
            e1 = sb.Event().record()
            out[name + "_tflops"] = round(2.0 * m * n * k / (e0.elapsed_ms(e1) / 2) / 1e9, 1)
        return out
    except Exception as exc:          # the row is context, never a reason to lose the bench line
        return {"error": str(exc)[:200]}


def run_ours(args, rank, world, local_rank):
    import spiral_b200 as sb
    from oracle import spiral_oracle as so   # only for the synthetic input generators and the CPU baseline leg

    workload = args.workload
    sizes, gbatch, in_dtype, training = WORKLOADS[workload]
    if args.batch:
        gbatch = args.batch
    if gbatch % world:
        raise SystemExit("global batch %d is not divisible by %d GPUs" % (gbatch, world))
    batch = gbatch // world
    sb.set_device(local_rank)

    dist = None
    torch = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier_sync():
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        sb.synchronize()

    # ---- synthetic inputs of this rank's shard (seeded; stand in for game states) ----------
    # Compact game states (one byte per one-hot field + the continuous values) are what the host
    # holds; the dense input is their encoding (on the device in the end-to-end path).
    gen_rows = min(batch, 32768)            # generate a block once and tile it: values/shape are what matter
    if sizes[0] == 32:
        fieldsh, maskh = so.leduc_states(100 + rank, gen_rows)
        denseh, widths = None, so.LEDUC_WIDTHS
    else:
        fieldsh, denseh, maskh = so.holdem_states(100 + rank, gen_rows, features=sizes[0], actions=sizes[-1])
        widths = so.HOLDEM_WIDTHS
    reps = (batch + gen_rows - 1) // gen_rows
    fieldsh = np.tile(fieldsh, (reps, 1))[:batch]
    maskh = np.tile(maskh, (reps, 1))[:batch]
    if denseh is not None:
        denseh = np.tile(denseh, (reps, 1))[:batch]
    xh = so.encode_states(fieldsh, widths, denseh)
    targeth = so.random_target(200 + rank, maskh)
    from spiral_b200 import dtypes

    def to_store(a):
        if in_dtype == "bf16":
            return dtypes.f32_to_bf16_bits(a).reshape(a.shape)
        if in_dtype == "f16":
            return a.astype(np.float16)
        return dtypes.round_tf32(a)

    x_store = to_store(xh)
    dense_store = to_store(denseh) if denseh is not None else None

    grads = None
    peer_mode = training and world > 1 and args.update in ("peer", "peer-overlap")
    if training and world > 1 and not peer_mode:
        n_params = sb.param_offsets(sizes)[-1]
        grads = torch.zeros(n_params, dtype=torch.float32, device="cuda")
    head = ("masked_softmax",) if training else ("masked_softmax", "regret_matching", "argmax")
    net = sb.PolicyMLP(sizes, batch, in_dtype=in_dtype, head=head, training=training, grads=grads)
    ws, bs = so.mlp_weights(5, sizes)        # same seed on every rank: replicated weights
    net.load_weights(ws, bs)

    x_dev = sb.DeviceArray(xh.shape, in_dtype)
    mask_dev = sb.DeviceArray(maskh.shape, "u8")
    target_dev = sb.DeviceArray(targeth.shape, "f32")
    x_pin, mask_pin, target_pin = PinnedBuffer(x_store), PinnedBuffer(maskh), PinnedBuffer(targeth)
    fields_pin = PinnedBuffer(fieldsh)
    dense_pin = PinnedBuffer(dense_store) if dense_store is not None else None
    x_pin.copy_to(x_dev)
    mask_pin.copy_to(mask_dev)
    target_pin.copy_to(target_dev)
    loss_pin = PinnedBuffer(np.zeros(1, np.float32))
    sb.synchronize()

    # narrow nets run inference as one persistent fused kernel
    fused = (not training) and max(sizes[1:-1]) <= 256 and in_dtype in ("f16", "bf16") and not args.layerwise
    seg = None
    if dist is not None and args.overlap:
        # per-layer asynchronous all-reduce: NCCL's stream picks each segment up as soon as that layer's
        # gradients are enqueued and runs beside the backward of the layers below.  Measured slower than
        # one all-reduce at the end on 2 and 8 B200s (the persistent GEMMs leave NCCL no free SM, and
        # five small messages cost more than one of 14.7 MB), so it is off by default.
        seg = lambda g, b, e: dist.all_reduce(g[b:e], async_op=True)
    peer = None
    if peer_mode:
        # The library's own reduce + update + redistribute kernel over peer memory; torch.distributed
        # only carries the 64-byte memory handles at set-up.
        def exchange(payload):
            out = [None] * world
            dist.all_gather_object(out, payload)
            return out
        peer = sb.PeerUpdate(net, world, rank, exchange, fused_reduce=args.fused_reduce)
    dp = sb.DataParallel(net, gbatch, all_reduce=(lambda g: dist.all_reduce(g)) if dist is not None else None,
                         world_size=world, rank=rank, all_reduce_segment=seg, peer_update=peer,
                         overlap_update=args.update == "peer-overlap", reserve_smem=args.reserve_smem)

    def step():
        if training:
            dp.train_step(x_dev, mask_dev, target_dev, LR)
        elif fused:
            net.forward_fused(x_dev, mask_dev)
        else:
            dp.infer(x_dev, mask_dev)

    # End-to-end step: the compact states of step i+1 (field bytes, continuous values, mask, target)
    # are copied from pinned host memory on a second stream into the other of two device buffer sets
    # while step i computes; every step still pays one full copy of its inputs, their encoding into
    # the dense input on the device and one read-back of its result.
    copy_stream = sb.Stream()

    def compact_set():
        return (sb.DeviceArray(fieldsh.shape, "u8"),
                sb.DeviceArray(dense_store.shape, in_dtype) if dense_store is not None else None,
                sb.DeviceArray(maskh.shape, "u8"), sb.DeviceArray(targeth.shape, "f32"))

    sets = [compact_set(), compact_set()]
    x_enc = sb.DeviceArray(xh.shape, in_dtype)     # the encoder's output, consumed by the same step
    ready = [sb.Event(), sb.Event()]     # inputs of a set have landed
    free = [sb.Event(), sb.Event()]      # the compute that read a set has finished
    e2e_state = {"i": 0, "primed": False}

    def enqueue_copy(k):
        copy_stream.wait_event(free[k])
        fields_pin.copy_to(sets[k][0], copy_stream.ptr)
        if dense_pin is not None:
            dense_pin.copy_to(sets[k][1], copy_stream.ptr)
        mask_pin.copy_to(sets[k][2], copy_stream.ptr)
        if training:
            target_pin.copy_to(sets[k][3], copy_stream.ptr)
        ready[k].record(copy_stream.ptr)

    def step_e2e():
        from spiral_b200 import _lib
        if not e2e_state["primed"]:
            free[0].record()
            free[1].record()
            enqueue_copy(0)
            e2e_state["primed"] = True
        cur = e2e_state["i"] & 1
        e2e_state["i"] += 1
        enqueue_copy(cur ^ 1)                      # next step's inputs, overlapping this step's compute
        sb.wait_event(None, ready[cur])
        fs, ds, ms, ts = sets[cur]
        xs = sb.primitives.encode_states(fs, widths, ds, x_enc)
        if training:
            dp.train_step(xs, ms, ts, LR)
        elif fused:
            net.forward_fused(xs, ms)
        else:
            dp.infer(xs, ms)
        free[cur].record()
        if training:
            _lib.call("sb_memcpy_d2h", loss_pin.ptr, net.loss.ptr, 4, None)
        else:
            _lib.call("sb_memcpy_d2h", act_pin.ptr, net.actions.ptr, act_pin.nbytes, None)
        _lib.call("sb_stream_sync", None)

    act_pin = None if training else PinnedBuffer(np.zeros(batch, np.int32))

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier_sync()
        l0 = sb.launch_count()
        t_wall0 = time.time()
        e0 = sb.Event().record()
        for _ in range(steps):
            fn()
        e1 = sb.Event().record()
        ms = e0.elapsed_ms(e1)
        barrier_sync()
        t_wall1 = time.time()
        launches = sb.launch_count() - l0
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches, (t_wall0, t_wall1)

    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    ms_total, launches, window = timed(step, args.steps, max(3, args.warmup))
    clocks = sampler.stop(*window) if sampler else None
    ms_step = ms_total / args.steps
    value = gbatch / (ms_step * 1e-3)

    # ---- dominant kernel: event-timed GEMM launches of two more steps --------------------
    with sb.GemmProfile() as prof:
        step()
        step()
    sb.synchronize()

    e2e_steps = max(2, min(args.steps, 10))
    ms_e2e, _, _ = timed(step_e2e, e2e_steps, 3)
    copy_stream.synchronize()
    e2e_value = gbatch / (ms_e2e / e2e_steps * 1e-3)
    h2d = (fields_pin.nbytes + (dense_pin.nbytes if dense_pin is not None else 0) + mask_pin.nbytes +
           (target_pin.nbytes if training else 0))
    d2h = 4 if training else act_pin.nbytes
    achieved = prof.flops / (prof.ms * 1e-3) / 1e12 if prof.ms > 0 else 0.0
    peaks = measured_peaks()
    # Denominator by the length of the timed window: the burst cuBLAS figure for a region shorter than
    # a second (the GPU has not settled under its power cap yet), the sustained one for longer runs.
    window_s = ms_total * 1e-3
    peak_key = "bf16_tflops" if window_s < 1.0 else "bf16_tflops_sustained"
    peak = float(peaks.get(peak_key, FALLBACK_PEAKS[peak_key]))
    status = sb.device_status()
    if status != (0, 0):
        raise SystemExit("device-side wait expired during the benchmark: %s" % (status,))
    dp_check = None
    leduc_dp = None
    if peer is not None:
        peer.check()
        # Outside every timed region: are the replicas the peer-memory kernel left behind identical,
        # and does it compute what all-reduce + SGD computes?  A failed check fails the run.
        dp_check = data_parallel_check(sb, dist, torch, net, peer, dp, ws, bs, x_dev, mask_dev, target_dev,
                                       gbatch, world, rank, barrier_sync)
        barrier_sync()
        peer.close()
        barrier_sync()                       # every rank has unmapped its peers' buffers
        if workload == "holdem_train" and not args.no_sweep:
            leduc_dp = leduc_train_data_parallel(sb, so, dist, torch, world, rank, barrier_sync)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    extra = {"dp_check": dp_check, "leduc_train_data_parallel": leduc_dp,
             "gemm_kernel_share_of_step": round(prof.ms / 2 / ms_step, 3),
             "gemm_launches_per_step": prof.launches // 2,
             # [microseconds, TFLOP/s] of every tensor-core GEMM launch of one step, in launch order
             "gemm_launch_us_tflops": [[round(ms * 1e3, 1), round(fl / ms / 1e9) if ms > 0 else 0]
                                       for ms, fl in prof.entries[prof.launches // 2:]],
             "peak_burst_tflops": peaks.get("bf16_tflops"), "peaks_source": peaks["source"],
             "model_tflops": round(net.flops_per_sample(training) * value / 1e12, 1)}
    if not training:
        # North-star view of the small-MLP case: algorithmic bytes of one forward pass (inputs, mask,
        # probabilities, actions, weights once) over the step time, against the measured HBM copy rate.
        n_params = sb.param_offsets(sizes)[-1]
        alg_bytes = (x_pin.nbytes + mask_pin.nbytes + batch * sizes[-1] * 4 + batch * 4) * world + n_params * 2
        hbm_peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        gbs = alg_bytes / (ms_step * 1e-3) / 1e9
        extra["hbm_view"] = {"algorithmic_bytes": int(alg_bytes), "achieved_gbs": round(gbs, 1), "peak_gbs": hbm_peak,
                             "frac": round(gbs / hbm_peak / world, 4)}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rows = 8192 if sizes[0] == 512 else 65536
        v, ms_cpu, cores = cpu_reference(workload, 3, 1, rows)
        cpu = {"value": v, "unit": "samples/s", "cores": cores, "kind": "port", "sample_rows_per_step": rows,
               "sample": "NumPy float32 %s step on %d rows, mean of 3" % ("training" if training else "forward", rows)}
        if not args.no_sweep:
            extra["gemm_4096_tflops"] = gemm_sweep(sb)
            extra["gemm_small_cases"] = gemm_small_cases(sb)
            extra["leduc_infer_batch_asymptote"] = leduc_infer_asymptote(sb, so, peaks)
            ref = reference_kernel_row(sb)
            if ref is not None:
                extra["reference_wmma_kernel_8192x8192x4096_tf32"] = ref
    # Bytes one step streams through HBM at least once: inputs, kept activations and (training) dY.
    touched = x_pin.nbytes + sum(batch * w for w in sizes[1:-1]) * x_store.itemsize * (2 if training else 1)
    if touched > 126e6:
        l2_note = "working set (%.0f MB of inputs and activations per step) larger than the 126 MB L2; no flush" % (touched / 1e6)
    else:
        l2_note = "working set (%.1f MB per step) fits in the 126 MB L2 and is left there: the steady state of this workload" % (touched / 1e6)
    traffic = NCU_TRAFFIC.get((workload, batch))
    line = {
        "metric": "policy_mlp_%s_samples_per_sec" % ("train" if training else "infer"),
        "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": in_dtype, "data": "synthetic",
        "config": {"workload": workload, "layers": sizes, "global_batch": gbatch, "batch_per_gpu": batch,
                   "parallelism": "dp%d" % world, "lr": LR,
                   "gradient_exchange": (("peer-memory reduce+update kernel" + (", per layer beside the backward pass" if args.update == "peer-overlap" else ""))
                                         if peer_mode else "nccl all-reduce") if (training and world > 1) else "none",
                   "l2": l2_note},
        "roofline": {"bound": "tensor", "kernel": "mlp_fused_kernel" if fused else "umma_gemm_kernel",
                     "achieved": round(achieved, 1), "peak": peak,
                     "unit": "TFLOP/s", "frac": round(achieved / peak, 4) if peak else None,
                     "traffic": traffic["bytes"] if traffic else None,
                     "traffic_source": traffic["source"] if traffic else
                     "no ncu capture backs this (workload, rows per GPU); see algorithmic_bytes",
                     "algorithmic_bytes": dominant_launch_bytes(sizes, batch, x_store.itemsize, training),
                     "peak_kind": "%s cuBLAS bf16, %s (timed window %.2f s)"
                                  % (peaks["source"], "burst" if peak_key == "bf16_tflops" else "sustained", window_s),
                     "frac_of_datasheet": round(achieved / DATASHEET_DENSE_TFLOPS[in_dtype], 4),
                     "datasheet_peak": DATASHEET_DENSE_TFLOPS[in_dtype],
                     "clock_normalised": clock_normalised(achieved, clocks)},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": int(h2d) * world,
                "d2h_bytes_per_step": int(d2h) * world, "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "extra": extra,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def replica_digest(net):
    """SHA-256 over this rank's fp32 master parameters and its compute copy (bit patterns)."""
    import hashlib
    h = hashlib.sha256()
    h.update(net.params.numpy().tobytes())
    raw = np.empty(net.w_compute.nbytes, np.uint8)
    from spiral_b200 import _lib
    _lib.call("sb_memcpy_d2h", raw.ctypes.data, net.w_compute.ptr, raw.nbytes, None)
    _lib.call("sb_stream_sync", None)
    h.update(raw.tobytes())
    return h.hexdigest()


def data_parallel_check(sb, dist, torch, net, peer, dp, ws, bs, x_dev, mask_dev, target_dev, gbatch, world, rank,
                        barrier_sync, steps=3):
    """Correctness of the peer-memory update on the hardware it runs on (all ranks call this).

    1. After the steps the benchmark has just run: every owner's master slice is gathered, then each
       rank hashes its master parameters and compute copy; the digests of all ranks must be equal
       (replicas bit-identical) and the loss finite.
    2. From the same seeded weights, `steps` training steps through the peer-memory kernel and `steps`
       through NCCL all-reduce + the SGD kernel: the two weight vectors may differ only by the order
       of the fp32 sums.  Reported relative to the size of the update itself; above 1e-3 the run fails.
    """
    from spiral_b200 import _lib
    peer.gather_master()
    barrier_sync()
    loss = float(net.loss.numpy()[0])
    digests = [None] * world
    dist.all_gather_object(digests, replica_digest(net))
    identical = len(set(digests)) == 1
    if not identical or not np.isfinite(loss):
        raise SystemExit("data-parallel check failed: replicas identical = %s, loss = %r" % (identical, loss))

    def reload():
        barrier_sync()                       # nobody still reads or writes a peer's buffers
        net.load_weights(ws, bs)
        peer.zero_gradients()                # the ranges peers add their weight-gradient tiles into start at zero
        barrier_sync()

    w0 = None
    reload()
    w0 = net.params.numpy().copy()
    for _ in range(steps):
        dp.train_step(x_dev, mask_dev, target_dev, LR)
    peer.gather_master()
    barrier_sync()
    peer.check()
    by_peer = net.params.numpy().copy()
    digests = [None] * world
    dist.all_gather_object(digests, replica_digest(net))
    identical = identical and len(set(digests)) == 1

    reload()
    tg = torch.zeros(net.n_params, dtype=torch.float32, device="cuda")
    for _ in range(steps):
        net.loss.fill_zero()
        net.forward(x_dev, mask_dev)
        net.backward(x_dev, mask_dev, target_dev, global_batch=gbatch)
        _lib.call("sb_memcpy_d2d", tg.data_ptr(), net.grads.ptr, net.grads.nbytes, None)
        dist.all_reduce(tg)
        _lib.call("sb_memcpy_d2d", net.grads.ptr, tg.data_ptr(), net.grads.nbytes, None)
        net.sgd(LR)
    barrier_sync()
    by_nccl = net.params.numpy().copy()
    update = np.linalg.norm((by_nccl - w0).astype(np.float64))
    diff = np.linalg.norm((by_peer - by_nccl).astype(np.float64))
    rel = float(diff / update) if update > 0 else float(diff)
    worst = torch.tensor([rel], dtype=torch.float64, device="cuda")
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    rel = float(worst.item())
    if not identical or not rel <= 1e-3:
        raise SystemExit("data-parallel check failed: replicas identical = %s, peer vs NCCL update differs by %g "
                         "of the update" % (identical, rel))
    return {"replicas_identical": bool(identical), "digest": digests[0][:16], "steps": steps,
            "peer_vs_nccl_rel_diff_of_update": rel, "loss": loss}


def leduc_train_data_parallel(sb, so, dist, torch, world, rank, barrier_sync, steps=50):
    """Benchmark configuration 4 as it is stated: the Leduc training step at a global batch of 65536,
    data-parallel over the ranks of this launch with the peer-memory update (all ranks call this)."""
    sizes, gbatch, in_dtype, _ = WORKLOADS["leduc_train"]
    batch = gbatch // world
    net = sb.PolicyMLP(sizes, batch, in_dtype=in_dtype, head=("masked_softmax",), training=True)
    ws, bs = so.mlp_weights(5, sizes)
    net.load_weights(ws, bs)
    x, mask = so.leduc_inputs(300 + rank, batch)
    target = so.random_target(400 + rank, mask)
    xd, md, td = sb.to_storage(x, in_dtype), sb.DeviceArray.from_numpy(mask), sb.DeviceArray.from_numpy(target)

    def exchange(payload):
        out = [None] * world
        dist.all_gather_object(out, payload)
        return out

    peer = sb.PeerUpdate(net, world, rank, exchange)
    dp = sb.DataParallel(net, gbatch, world_size=world, rank=rank, peer_update=peer)
    for _ in range(5):
        dp.train_step(xd, md, td, LR)
    barrier_sync()
    e0 = sb.Event().record()
    for _ in range(steps):
        dp.train_step(xd, md, td, LR)
    e1 = sb.Event().record()
    t = torch.tensor([e0.elapsed_ms(e1) / steps], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    barrier_sync()
    peer.check()
    peer.close()
    barrier_sync()                           # every rank has unmapped its peers' buffers before they are freed
    ms = float(t.item())
    return {"global_batch": gbatch, "n_gpus": world, "ms_per_step": round(ms, 4),
            "samples_per_s": round(gbatch / (ms * 1e-3), 1), "steps": steps}


def leduc_infer_asymptote(sb, so, peaks):
    """The narrow-net forward (fused persistent kernel) at the benchmark batch and at 16x and 64x of
    it: microseconds per forward, states per second, and the algorithmic bytes (input, mask,
    probabilities, actions, weights once) over that time against the measured HBM copy rate.  At 16384
    states one launch is latency-bound; the larger batches show what the kernel sustains."""
    sizes, base, in_dtype, _ = WORKLOADS["leduc_infer"]
    ws, bs = so.mlp_weights(5, sizes)
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    out = {}
    for mult in (1, 16, 64):
        batch = base * mult
        net = sb.PolicyMLP(sizes, batch, in_dtype=in_dtype, head=("masked_softmax", "regret_matching", "argmax"))
        net.load_weights(ws, bs)
        x, mask = so.leduc_inputs(7, min(batch, 65536))
        reps = batch // x.shape[0]
        xd = sb.to_storage(np.tile(x, (reps, 1)), in_dtype)
        md = sb.DeviceArray.from_numpy(np.tile(mask, (reps, 1)))
        for _ in range(3):
            net.forward_fused(xd, md)
        iters = 20
        e0 = sb.Event().record()
        for _ in range(iters):
            net.forward_fused(xd, md)
        e1 = sb.Event().record()
        ms = e0.elapsed_ms(e1) / iters
        alg = xd.nbytes + md.nbytes + batch * sizes[-1] * 4 + batch * 4 + net.n_params * 2
        gbs = alg / (ms * 1e-3) / 1e9
        out["batch_%d" % batch] = {"us": round(ms * 1e3, 2), "states_per_s": round(batch / (ms * 1e-3), 0),
                                   "algorithmic_gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm, 4),
                                   "tflops": round(net.flops_per_sample(False) * batch / ms / 1e9, 1)}
    return out


# DRAM bytes (read + write) of one launch of the dominant GEMM shape of a workload, from an ncu capture
# of a quarter of the batch rows scaled by the rows; keyed by (workload, rows per GPU).  The bound of
# that kernel is the tensor pipe; the figure shows that its operands are read from DRAM once.  The
# algorithmic bytes of the same launch are computed for every batch (dominant_launch_bytes).
NCU_TRAFFIC = {("holdem_train", 262144): {
    "bytes": 4 * (136450560 + 100710656),
    "source": "ncu capture of the hidden-layer training forward at 65536 rows (dram__bytes_read.sum + "
              "dram__bytes_write.sum), scaled x4 by the rows: profiles/umma_gemm_kernel_holdem_layer_fwd_bits.md"}}
# NVIDIA's dense (no 2:4 sparsity) tensor peaks of one B200, TFLOP/s.
DATASHEET_DENSE_TFLOPS = {"bf16": 2250.0, "f16": 2250.0, "tf32": 1125.0}


def dominant_launch_bytes(sizes, rows, es, training):
    """Algorithmic bytes of one launch of the dominant GEMM of a step, the widest hidden layer's forward:
    input and output activations once, the weights once, the bias, and (training) the ReLU sign words."""
    i = max(range(len(sizes) - 2), key=lambda j: sizes[j] * sizes[j + 1]) if len(sizes) > 2 else 0
    k, n = sizes[i], sizes[i + 1]
    total = rows * k * es + n * k * es + rows * n * es + n * 4
    if training:
        total += rows * (n // 32) * 4
    return int(total)


def clock_normalised(achieved, clocks):
    """The achieved figure scaled to the maximum SM clock from the median clock SAMPLED during the timed
    region (nothing is locked or set): what the same launches would give if the part held its top
    clock.  None when no clock sample exists."""
    if not clocks or not clocks.get("sm_mhz") or not clocks.get("sm_max_mhz"):
        return None
    return {"tflops_at_max_clock": round(achieved * clocks["sm_max_mhz"] / clocks["sm_mhz"], 1),
            "sm_mhz_median": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"]}

PROFILE_CASES = {
    # name: (a_trans, b_trans, M, N, K, in_dtype, out_dtype, epilogue)
    "gemm4096_bf16_nt": (False, True, 4096, 4096, 4096, "bf16", "f32", ()),
    "gemm4096_bf16_nn": (False, False, 4096, 4096, 4096, "bf16", "f32", ()),
    "gemm4096_bf16_tn": (True, False, 4096, 4096, 4096, "bf16", "f32", ()),
    "gemm4096_tf32_nt": (False, True, 4096, 4096, 4096, "tf32", "f32", ()),
    "holdem_layer_fwd": (False, True, 65536, 1024, 1024, "bf16", "bf16", ("bias", "relu")),
    "holdem_layer_plain": (False, True, 65536, 1024, 1024, "bf16", "bf16", ()),
    "holdem_layer_plain_f32": (False, True, 65536, 1024, 1024, "bf16", "f32", ()),
    "holdem_layer_dgrad": (False, False, 65536, 1024, 1024, "bf16", "bf16", ("relu_grad",)),
    "holdem_layer_wgrad": (True, False, 1024, 1024, 65536, "bf16", "f32", ()),
    "holdem_layer_dgrad_bits": (False, False, 65536, 1024, 1024, "bf16", "bf16", ("relu_grad_mask",)),
    "holdem_head_dgrad_bits": (False, False, 65536, 1024, 16, "bf16", "bf16", ("relu_grad_mask",)),
    "holdem_layer_fwd_bits": (False, True, 65536, 1024, 1024, "bf16", "bf16", ("bias", "relu", "relu_mask_out")),
    "holdem_layer0_fwd_bits": (False, True, 65536, 1024, 512, "bf16", "bf16", ("bias", "relu", "relu_mask_out")),
    "holdem_layer_dgrad_colsum": (False, False, 65536, 1024, 1024, "bf16", "bf16", ("relu_grad_mask", "colsum_out")),
    "holdem_head_dgrad_colsum": (False, False, 65536, 1024, 16, "bf16", "bf16", ("relu_grad_mask", "colsum_out")),
}


def run_profile_case(name, iters):
    """A few launches of one GEMM shape with seeded random operands, for ncu captures (no JSON line)."""
    import spiral_b200 as sb
    at, bt, m, n, k, dt, odt, epi = PROFILE_CASES[name]
    sb.set_device(0)
    rng = np.random.Generator(np.random.Philox(7))
    a = sb.DeviceArray.from_numpy(rng.standard_normal((k, m) if at else (m, k), dtype=np.float32), dt)
    b = sb.DeviceArray.from_numpy(rng.standard_normal((n, k) if bt else (k, n), dtype=np.float32), dt)
    c = sb.DeviceArray((m, n), odt)
    bias = sb.DeviceArray.from_numpy(rng.standard_normal(n, dtype=np.float32)) if "bias" in epi else None
    aux = sb.DeviceArray.from_numpy(rng.standard_normal((m, n), dtype=np.float32), odt) if "relu_grad" in epi else None
    if "relu_grad_mask" in epi:
        aux = sb.DeviceArray.from_numpy(rng.integers(-2**31, 2**31 - 1, size=(n // 32, m), dtype=np.int32))
    aux_out = None
    if "relu_mask_out" in epi:
        aux_out = sb.DeviceArray.zeros((n // 32, m), "i32")
    elif "colsum_out" in epi:
        aux_out = sb.DeviceArray.zeros((n,), "f32")
    kw = dict(in_dtype=dt, epilogue=epi, bias=bias, aux_in=aux, aux_out=aux_out)
    sb.matmul(at, bt, 1.0, a, b, 0.0, c, **kw)   # first-launch set-up
    sb.synchronize()
    e0 = sb.Event().record()
    for _ in range(iters):
        sb.matmul(at, bt, 1.0, a, b, 0.0, c, **kw)
    e1 = sb.Event().record()
    ms = e0.elapsed_ms(e1) / iters
    print("profile case %s: %.4f ms per launch, %.1f TFLOP/s, status %s"
          % (name, ms, 2.0 * m * n * k / ms / 1e9, sb.device_status()), flush=True)


def run_exchange_profile(args, rank, world, local_rank):
    """Times the data-parallel exchange of the Hold'em net by itself (under torchrun, N >= 2): the
    library's peer-memory update and its parts (remote reads only, remote stores only, local memory
    with and without the flag barriers) beside NCCL all-reduce + SGD.  One table on rank 0."""
    import ctypes
    import torch
    import torch.distributed as dist
    import spiral_b200 as sb
    from spiral_b200 import _lib
    torch.cuda.set_device(local_rank)
    sb.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    sizes = WORKLOADS["holdem_train"][0]
    net = sb.PolicyMLP(sizes, 1024, in_dtype="bf16", training=True)

    def exchange(payload):
        out = [None] * world
        dist.all_gather_object(out, payload)
        return out

    peer = sb.PeerUpdate(net, world, rank, exchange)
    tg = torch.zeros(net.n_params, dtype=torch.float32, device="cuda")

    def timed(fn):
        for _ in range(5):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        sb.synchronize()
        e0 = sb.Event().record()
        for _ in range(args.iters):
            fn()
        e1 = sb.Event().record()
        ms = e0.elapsed_ms(e1) / args.iters
        torch.cuda.synchronize()
        return ms * 1e3

    g, p, w, f = peer._tables

    def own(table):
        return (ctypes.c_void_p * world)(*[table[rank]] * world)

    def call(gt, pt, wt, mode, barriers=1):
        _lib.call("sb_dp_sgd_update", world, rank, gt, pt, wt, f, ctypes.c_uint(peer.epoch), ctypes.c_longlong(0),
                  ctypes.c_longlong(net.n_params), ctypes.c_float(1e-3), _lib.DTYPE_CODES["bf16"], mode,
                  peer._ranges, peer._n_ranges, 0, 2000, barriers, None)
        peer.epoch += 2

    rows = [
        ("peer update, sharded master (the default)", lambda: call(g, p, w, 1)),
        ("peer update, replicated master", lambda: call(g, p, w, 0)),
        ("  remote reads only (stores to own memory)", lambda: call(g, own(p), own(w), 0)),
        ("  remote stores only (reads from own memory)", lambda: call(own(g), p, w, 0)),
        ("  own memory only, both barriers", lambda: call(own(g), own(p), own(w), 0)),
        ("  own memory only, no barrier", lambda: call(own(g), own(p), own(w), 0, 0)),
        ("nccl all-reduce + sgd kernel", lambda: (dist.all_reduce(tg), net.sgd(1e-3))),
        ("nccl all-reduce", lambda: dist.all_reduce(tg)),
    ]
    results = [(name, timed(fn)) for name, fn in rows]
    status = peer.status()
    if rank == 0:
        print("exchange of %d parameters (%.1f MB of fp32 gradients) on %d GPUs, microseconds per step:"
              % (net.n_params, net.n_params * 4 / 1e6, world))
        for name, us in results:
            print("  %-48s %7.1f" % (name, us))
        print("status 0x%x" % status, flush=True)
    dist.barrier()
    peer.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="holdem_train")
    ap.add_argument("--batch", type=int, default=0, help="override the global batch (tests only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--overlap", action="store_true", help="per-layer asynchronous all-reduce instead of one at the end")
    ap.add_argument("--update", choices=("peer", "peer-overlap", "nccl"), default="peer",
                    help="N > 1 training: the library's reduce+update kernel over peer memory (one launch after the "
                         "backward pass, or per layer beside it), or NCCL all-reduce + SGD")
    ap.add_argument("--fused-reduce", action="store_true",
                    help="peer update: the weight-gradient GEMMs add their tiles straight into the owning rank's "
                         "buffer over peer memory (measured slower than letting the update kernel read the peers)")
    ap.add_argument("--reserve-smem", type=int, default=4096,
                    help="peer-overlap: shared memory per SM the backward GEMMs leave free for the update CTAs")
    ap.add_argument("--layerwise", action="store_true", help="narrow-net inference through one GEMM per layer")
    ap.add_argument("--profile-case", choices=sorted(PROFILE_CASES), default=None,
                    help="run a few launches of one GEMM shape (for ncu) and exit")
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--profile-exchange", action="store_true",
                    help="under torchrun: time the data-parallel exchange and its parts (no JSON line)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case, args.iters)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.profile_exchange:
        if world < 2:
            raise SystemExit("--profile-exchange needs a torchrun launch with at least 2 ranks")
        run_exchange_profile(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus %d needs a torchrun launch with %d ranks" % (args.gpus, args.gpus))
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
