#!/usr/bin/env python3
"""Benchmark of the BERT forward pass through the cuBERT C API on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: BERT-base, binary16 weight/activation storage with float32
arithmetic, seq_length 128, batch 256 per GPU, per-sequence valid length uniform in [8, 128]
(prefix mask), seeded random-init weights N(0, 0.02) and uniform token ids; outputs
cuBERT_SEQUENCE_OUTPUT and cuBERT_POOLED_OUTPUT. One step = one forward pass over one batch.
One process per GPU, each with its own model replica; the batch dimension is the only parallel
axis, so there is no collective on the data path ("weak" scaling: per-GPU work is fixed).

Printed by rank 0 as ONE JSON line:
  value      sequences/s, whole job, inputs already resident in device memory, timed with CUDA
             events on the replica's stream (max over ranks)
  e2e        the same through cuBERT_compute_m with pinned HOST buffers: host-to-device copy of
             ids/mask/segments and device-to-host copy of both outputs inside the timed region
  roofline   the fused kernel with the largest share of the step: algorithmic bytes / its mean
             launch duration, from CUDA events around every launch in a second timed region of the
             same K steps (the first region replays the step as one CUDA graph, which events
             cannot subdivide)
  kernels    the same figures for every kernel family
  cpu_baseline  the reference's own CPU code (oracle/_ref) or, failing that, its C restatement,
             timed on this machine's host cores on a bounded sample (N = 1 only)

--impl reference times only that CPU implementation, on the same workload definition.

--workload large_seq512 runs the second full-model case instead: BERT-large,
binary16 storage, seq_length 512, ONE batch of 512 sequences split evenly over the GPUs ("strong"
scaling), full masks, mean pooler, output cuBERT_POOLED_OUTPUT, seed 3.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

RANK = int(os.environ.get("RANK", "0"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))

# base_seq128 is the workload the headline metric is quoted on (per-GPU batch fixed: weak scaling);
# large_seq512 is the second full-model case: one 512-sequence batch split evenly over the GPUs
# (strong scaling), mean pooler, pooled_output only.
WORKLOADS = {
    # the reference's own published case (its README: batch 128, seq 32, float32)
    "base_seq32_f32": dict(model="base", seq=32, batch=128, lengths=None, seed=0, scaling="weak", dtype="f32",
                           segments="half", outputs=("logits", "probs"), cpu_sample=128,
                           metric="BERT-base seq32 float32 seqs/s",
                           text="BERT-base (12 layers, hidden 768, 12 heads, intermediate 3072, vocab 21128, 2 labels) "
                                "forward, float32, seq_length 32, batch 128 per GPU, full masks, segment 0 for the "
                                "first 16 positions and 1 after, outputs logits + probs"),
    "base_seq128": dict(model="base", seq=128, batch=256, lengths=(8, 128), seed=2, scaling="weak",
                        outputs=("sequence_output", "pooled_output"), metric="BERT-base seq128 seqs/s",
                        text="BERT-base (12 layers, hidden 768, 12 heads, intermediate 3072, vocab 21128) forward, "
                             "seq_length 128, batch 256 per GPU, valid length U[8,128], outputs sequence_output + "
                             "pooled_output"),
    "large_seq512": dict(model="large", seq=512, batch=512, lengths=None, seed=3, scaling="strong", cpu_sample=4,
                         outputs=("pooled_output",), metric="BERT-large seq512 seqs/s",
                         text="BERT-large (24 layers, hidden 1024, 16 heads, intermediate 4096, vocab 30522) forward, "
                              "seq_length 512, one batch of 512 split evenly over the GPUs, full masks, mean pooler, "
                              "output pooled_output"),
}
WORKLOAD = WORKLOADS["base_seq128"]
WORKLOAD_NAME = "base_seq128"
UNIT = "sequences/s"
L2_NOTE = ("no explicit L2 flush: one step streams the model's weights (218 MB or more) and >1 GB of activations, "
           "far more than the 126 MB L2")


def device_for_rank(visible, local_rank):
    """The entry of a CUDA_VISIBLE_DEVICES list (None or "" = every GPU of the machine, in order) that a
    rank works on: its own entry, or its own number when the list is absent or too short. Entries may be
    indices or GPU UUIDs; the entry is returned as the string to put into CUDA_VISIBLE_DEVICES."""
    ids = [v.strip() for v in (visible or "").split(",") if v.strip() != ""]
    if ids and local_rank < len(ids):
        return ids[local_rank]
    return str(local_rank)


def narrow_to_one_gpu(env, local_rank):
    """Restrict the process to one GPU, whatever the launcher left visible: the library builds a replica
    on every GPU it can see (as the reference does), and a bench process times exactly one. This holds
    for a single process on a multi-GPU machine just as for one rank of many. The list the process
    inherited is kept in CUBERT_BENCH_PARENT_VISIBLE. Returns the chosen entry."""
    if "CUBERT_BENCH_PARENT_VISIBLE" not in env:
        env["CUBERT_BENCH_PARENT_VISIBLE"] = env.get("CUDA_VISIBLE_DEVICES", "")
    chosen = device_for_rank(env["CUBERT_BENCH_PARENT_VISIBLE"], local_rank)
    env["CUDA_VISIBLE_DEVICES"] = chosen
    return chosen


def physical_gpu_index():
    """nvidia-smi index of this rank's GPU (for the clock samples)."""
    vis = os.environ.get("CUBERT_BENCH_PARENT_VISIBLE", os.environ.get("CUDA_VISIBLE_DEVICES", ""))
    d = device_for_rank(vis, LOCAL_RANK)
    return int(d) if d.isdigit() else LOCAL_RANK


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed regions run."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(prefix="cubert_clocks_", suffix=".csv")
        self.proc = None
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    smax.append(float(p[2]))
                    power.append(float(p[3]))
                except ValueError:
                    continue
                for name, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        # "under load": samples in the upper half of the power range seen
        lo, hi = min(power), max(power)
        loaded = [c for c, w in zip(sm, power) if w >= lo + 0.5 * (hi - lo)] or sm
        return dict(sm_mhz=statistics.median(loaded), sm_max_mhz=max(smax), reasons=sorted(reasons),
                    samples=len(sm), power_w_max=hi)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s sustained inside a long step (the driver-written measurement), or None."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f).get("bf16_tflops_sustained")
    return None


# Per-launch DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the fused kernels on the headline
# workload's shapes, from the ncu captures summarised under profiles/. Each figure belongs to ONE kernel of ONE
# library version on ONE workload; ncu_traffic() hands it out only when all three still hold, else None.
NCU_TRAFFIC = {
    "bias_gelu": dict(bytes=346974336, kernel="bias_act_kernel<__half, 128, 2, 4, GeluTailFit<6>>",
                      note="201.3 MB read + 145.6 MB written (rest of the output still in L2)"),
    "bias_residual_ln": dict(bytes=108217344, kernel="bias_residual_ln_rows_kernel<__half, 3>",
                             note="100.7 MB read + 7.5 MB written"),
    "masked_softmax": dict(bytes=123932032, kernel="masked_softmax_kernel<__half, 4, 4, 1, 256, true, true>",
                           note="77.1 MB read (scores past each sequence's last kept key are not read) + 46.8 MB written"),
    "embed_ln": dict(bytes=29022592, kernel="embed_ln_rows_kernel<__half, 3, 3>",
                     note="26.0 MB read + 3.0 MB written: word rows are served by L2"),
}
NCU_TRAFFIC_SOURCE = dict(workload="base_seq128", cubk_version=110,
                          profile="profiles/fused_kernels_in_bench_f16_ncu_full.md")
NCU_TRAFFIC_BYTES = {k: v["bytes"] for k, v in NCU_TRAFFIC.items()}


def ncu_traffic(family, workload_name, cubk_version, default_switches):
    """DRAM bytes per launch that ncu measured for `family`, or None when the capture does not describe what
    runs now: another workload, another build of the kernel library, or kernel-selection switches
    (cubk_set_option / their environment variables, the CUBERT_* toggles that change what K4 reads) off their
    defaults."""
    entry = NCU_TRAFFIC.get(family)
    if (entry is None or workload_name != NCU_TRAFFIC_SOURCE["workload"] or
            cubk_version != NCU_TRAFFIC_SOURCE["cubk_version"] or not default_switches):
        return None
    return dict(bytes=entry["bytes"], kernel=entry["kernel"], profile=NCU_TRAFFIC_SOURCE["profile"], note=entry["note"])


def switches_at_defaults(env):
    """True when no variable that changes which kernel variant runs, or what it reads, is set."""
    names = ("CUBK_BULK_COPY", "CUBK_SOFTMAX_MASK_SMEM", "CUBK_EXACT_WIDTH_ROWS", "CUBK_EXACT_WIDTH_EMBED",
             "CUBERT_SKIP_MASKED_KEYS", "CUBERT_KEY_GEMM", "CUBERT_KEY_GRANULE")
    return not any(n in env for n in names)


def make_model_file(cfg, seed, half):
    import numpy as np
    from cubert_b200 import frozen_graph, synthetic
    var = synthetic.random_weights(cfg, seed)
    if half:
        var = {k: v.astype(np.float16) for k, v in var.items()}
    d = tempfile.mkdtemp(prefix="cubert_b200_bench_")
    path = os.path.join(d, "model.pb")
    frozen_graph.write_frozen_graph(path, var)
    return path, var


def cpu_reference_rate(cfg, var32, seq, sample_batch, lengths, seed, steps, warmup):
    """sequences/s of the reference's CPU implementation (float32; it has no binary16 path) on
    `sample_batch` sequences of the workload per step. Returns (rate, kind, cores, seconds/step)."""
    import numpy as np
    from cubert_b200 import synthetic
    from oracle import bindings
    geo = synthetic.model_geometry(cfg, seq)
    ids, mask, seg, _ = synthetic.random_inputs(cfg, sample_batch, seq, seed, lengths=lengths)
    # All the host threads there are: launchers such as torchrun pin OMP_NUM_THREADS to 1 for their
    # children, which would time a single-threaded reference. CUBERT_BENCH_CPU_THREADS overrides.
    cores = int(os.environ.get("CUBERT_BENCH_CPU_THREADS", "0")) or len(os.sched_getaffinity(0)) or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    os.environ.setdefault("KMP_BLOCKTIME", "0")  # as the reference's README recommends
    try:  # an OpenMP runtime that is already loaded has read the variable; tell it directly as well
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    times = []
    if os.path.exists(bindings.REF_CPU_SO):
        kind = "reference"
        ref = bindings.Reference()
        h = ref.bert_open(var32, geo, sample_batch)
        try:
            for i in range(warmup + steps):
                t0 = time.perf_counter()
                ref.bert_compute(h, ids, mask, seg)
                ref.bert_output(h, sample_batch, geo, "output_weights" in var32)
                if i >= warmup:
                    times.append(time.perf_counter() - t0)
        finally:
            ref.bert_close(h)
    else:
        kind = "port"
        bindings.build()
        orc = bindings.Oracle()
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            orc.bert_forward(var32, geo, ids, mask, seg)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return sample_batch / sec, kind, int(os.environ["OMP_NUM_THREADS"]), sec


def run_reference_arm(args):
    """--impl reference: the reference's own CPU implementation of the path, rank 0 only."""
    if RANK != 0:
        return
    import numpy as np  # noqa: F401
    from cubert_b200 import synthetic
    cfg = synthetic.config(WORKLOAD["model"])
    var32 = synthetic.random_weights(cfg, WORKLOAD["seed"])
    sample = WORKLOAD.get("cpu_sample", 32)
    rate, kind, cores, sec = cpu_reference_rate(cfg, var32, WORKLOAD["seq"], sample, WORKLOAD["lengths"] or "full",
                                                WORKLOAD["seed"], args.steps, max(1, min(args.warmup, 3)))
    line = {
        "impl": "reference", "metric": WORKLOAD["metric"], "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": WORKLOAD["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["text"] + "; float32 on host cores (the reference's CPU build has no "
                               "binary16)",
                   "sample_batch": sample, "full_batch": WORKLOAD["batch"], "seed": WORKLOAD["seed"]},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": "%d sequences per step (of the %d-sequence batch), %d timed steps" %
                                   (sample, WORKLOAD["batch"], args.steps)},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    # one replica per process: restrict the library to this rank's GPU before CUDA starts
    # (also when this is the only process: on a machine with several GPUs the library would otherwise
    # build a replica on each of them)
    narrow_to_one_gpu(os.environ, LOCAL_RANK)
    import numpy as np
    from cubert_b200 import model, synthetic
    model.load()  # before torch: the process then binds the toolkit's cuBLAS, not the older one torch bundles
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(0)
    if WORLD > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", 0))

    from cubert_b200 import replicas

    def barrier():
        if WORLD > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        return replicas.max_over_ranks(x, "cuda")

    def sum_over_ranks(x):
        return replicas.sum_over_ranks(x, "cuda")

    cfg = synthetic.config(WORKLOAD["model"])
    weak = WORKLOAD["scaling"] == "weak"
    if not weak and WORKLOAD["batch"] % WORLD != 0:
        sys.exit("the %d-sequence batch does not split evenly over %d GPUs" % (WORKLOAD["batch"], WORLD))
    B = WORKLOAD["batch"] if weak else WORKLOAD["batch"] // WORLD   # sequences per GPU and step
    S, H = WORKLOAD["seq"], cfg["hidden"]
    half = WORKLOAD.get("dtype", "f16") == "f16"
    elem = 2 if half else 4
    path, var16 = make_model_file(cfg, WORKLOAD["seed"], half=half)
    m = model.Model(path, B, S, cfg["layers"], cfg["heads"],
                    model.ComputeType.HALF if half else model.ComputeType.FLOAT)
    os.unlink(path)
    if m.info["replicas"] != 1:
        sys.exit("bench.py times one replica per process; the library built %d (CUDA_VISIBLE_DEVICES=%r, "
                 "CUBERT_NUM_MODELS_PER_GPU=%r)" % (m.info["replicas"], os.environ.get("CUDA_VISIBLE_DEVICES"),
                                                    os.environ.get("CUBERT_NUM_MODELS_PER_GPU")))

    # every rank works on its own batch of the seeded stream
    ids, mask, seg, lens = synthetic.random_inputs(cfg, B, S, replicas.stream_seed(WORKLOAD["seed"], RANK),
                                                   lengths=WORKLOAD["lengths"] or "full")
    pin = lambda a: torch.from_numpy(a).pin_memory()  # noqa: E731
    h_ids, h_mask, h_seg = pin(ids), pin(mask), pin(seg)
    d_ids, d_mask, d_seg = h_ids.cuda(), h_mask.cuda(), h_seg.cuda()
    out = model.Output()
    d2h_bytes = 0
    h_out = {}
    for name in WORKLOAD["outputs"]:
        shape = {"sequence_output": (B, S, H), "pooled_output": (B, H)}.get(name, (B, cfg["num_labels"]))
        h_out[name] = torch.empty(shape, dtype=torch.float16 if half else torch.float32).pin_memory()
        setattr(out, name, h_out[name].numpy())
        d2h_bytes += h_out[name].numel() * elem
    np_ids, np_mask, np_seg = h_ids.numpy(), h_mask.numpy(), h_seg.numpy()
    stream = torch.cuda.ExternalStream(m.replica_stream(0))

    sampler = ClockSampler(physical_gpu_index()) if RANK == 0 else None

    # ---- device-resident: `value` (the forward pass replayed as one CUDA graph, the library's default)
    for _ in range(args.warmup):
        m.forward_device(0, B, d_ids.data_ptr(), d_mask.data_ptr(), d_seg.data_ptr(), host_mask=np_mask)
    m.synchronize(0)
    m.profile_read(0)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        m.forward_device(0, B, d_ids.data_ptr(), d_mask.data_ptr(), d_seg.data_ptr(), host_mask=np_mask)
    stop.record(stream)
    m.synchronize(0)
    barrier()
    local_dev_ms = start.elapsed_time(stop)
    dev_ms = max_over_ranks(local_dev_ms)
    counted = m.profile_read(0)

    # ---- the same K steps again with CUDA events around every launch (plain stream launches, since
    #      events cannot bracket the nodes of a replayed graph): per-kernel durations for the roofline
    m.profile_enable(True, 0)
    p_start, p_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    p_start.record(stream)
    for _ in range(args.steps):
        m.forward_device(0, B, d_ids.data_ptr(), d_mask.data_ptr(), d_seg.data_ptr(), host_mask=np_mask)
    p_stop.record(stream)
    m.synchronize(0)
    barrier()
    prof_ms = p_start.elapsed_time(p_stop)
    prof = m.profile_read(0)
    m.profile_enable(False, 0)

    # ---- end to end through the C API with pinned host buffers
    for _ in range(args.warmup):
        m.compute_m(np_ids, np_mask, np_seg, out)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        m.compute_m(np_ids, np_mask, np_seg, out)
    e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = max_over_ranks(e2e_s)
    ok = all(bool(np.all(np.isfinite(h.numpy().astype(np.float32)))) for h in h_out.values())
    clocks = sampler.stop() if sampler else None

    launches = sum_over_ranks(sum(v["launches"] for k, v in counted.items() if k not in ("gemm", "event_overhead")))
    if RANK != 0:
        m.close()
        if WORLD > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    kernels = {}
    for k, v in prof.items():
        if v["launches"] == 0:
            continue
        entry = dict(launches=int(v["launches"]), ms_total=v["ms"], us_per_launch=1e3 * v["ms"] / v["launches"],
                     share_of_step=v["ms"] / prof_ms)
        if k != "gemm" and v["bytes"] > 0 and v["ms"] > 0:
            entry["bytes_per_launch"] = int(v["bytes"] / v["launches"])
            entry["gbs"] = v["bytes"] / (v["ms"] * 1e-3) / 1e9
            entry["frac_of_%s_peak" % peak_kind] = entry["gbs"] / peak
        kernels[k] = entry
    # With heads of 64 a binary16 model of up to 128 positions runs each layer's Q.K^T, masked softmax and P.V as
    # ONE launch in the masked-softmax slot (four library products per layer instead of six). That launch is a
    # pair of tensor-core products around a softmax, not an HBM-bound row kernel: it is listed under its own name
    # with both rulers, and the roofline object stays with the largest HBM-bound family.
    L = cfg["layers"]
    one_launch = ("masked_softmax" in kernels and "gemm" in kernels and
                  kernels["gemm"]["launches"] == kernels["masked_softmax"]["launches"] // L * (4 * L + 1))
    if one_launch:
        att = kernels.pop("masked_softmax")
        heads, d = cfg["heads"], cfg["hidden"] // cfg["heads"]
        att["flops_per_launch"] = 4 * B * heads * S * S * d
        att["tflops"] = att["flops_per_launch"] / (att["us_per_launch"] * 1e-6) / 1e12
        tensor_peak = measured_tensor_peak()
        if tensor_peak:
            att["frac_of_measured_bf16_sustained_peak"] = att["tflops"] / tensor_peak
        att["what"] = ("Q.K^T + masked softmax + P.V of a layer in one launch (mma.sync or tcgen05); bytes = Q | K | V read "
                       "+ context written; flops = both products over every key, as the reference computes them; "
                       "latency-bound, neither ruler applies well")
        kernels["attention_one_launch"] = att
    ours = {k: v for k, v in kernels.items() if k not in ("gemm", "attention_one_launch") and "gbs" in v}
    top = max(ours, key=lambda k: ours[k]["ms_total"])
    # What the event pair itself costs at least: the same bracket around nothing, once per pass. Fractions are
    # reported raw (event time as measured) first; `frac_net_of_event_overhead` takes only this floor off.
    overhead_us = kernels.get("event_overhead", {}).get("us_per_launch")
    from cubert_b200 import kernels as kernel_lib
    workload_name = WORKLOAD_NAME
    traffic = ncu_traffic(top, workload_name, kernel_lib.load().cubk_version(), switches_at_defaults(os.environ))
    roofline = {"bound": "hbm", "kernel": top, "achieved": ours[top]["gbs"], "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": ours[top]["gbs"] / peak,
                "bytes_per_launch": ours[top]["bytes_per_launch"], "us_per_launch": ours[top]["us_per_launch"],
                "traffic": traffic["bytes"] if traffic else None, "traffic_source": traffic,
                "event_bracket_overhead_us": overhead_us,
                "scope": "largest HBM-bound family of the step" +
                         ("; kernels.attention_one_launch (%.1f us per launch) is a contraction + softmax launch with "
                          "its own entry" % kernels["attention_one_launch"]["us_per_launch"] if one_launch else "")}
    if overhead_us:
        for k, v in list(ours.items()) + ([("attention_one_launch", kernels["attention_one_launch"])] if one_launch else []):
            net = v["us_per_launch"] - overhead_us
            if net > 0:
                v["frac_net_of_event_overhead"] = v["bytes_per_launch"] / (net * 1e-6) / 1e9 / peak
        roofline["frac_net_of_event_overhead"] = ours[top].get("frac_net_of_event_overhead")

    total_seqs = B * args.steps * WORLD
    line = {
        "metric": WORKLOAD["metric"], "value": total_seqs / (dev_ms * 1e-3), "unit": UNIT, "n_gpus": WORLD,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
        "higher_is_better": True, "scaling": WORKLOAD["scaling"], "vs_baseline": None,
        "dtype": "f16" if half else "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["text"],
                   "storage": ("binary16" if half else "float32") + " weights and activations",
                   "arithmetic": "float32 accumulate",
                   "global_batch": B * WORLD, "batch_per_gpu": B, "seq_len": S,
                   "parallelism": "replica per GPU, no collective",
                   "seed": WORKLOAD["seed"], "l2": L2_NOTE, "per_kernel_events": "second timed region of the same K steps, CUDA events around every "
                                        "launch, graph replay off; ms_per_step there = %.3f" % (prof_ms / args.steps)},
        "e2e": {"value": total_seqs / e2e_s, "unit": UNIT, "ms_per_step": 1e3 * e2e_s / args.steps,
                "h2d_bytes_per_step": int(B * S * 6), "d2h_bytes_per_step": int(d2h_bytes),
                "outputs_finite": ok},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "kernels": kernels,
        "clocks": clocks,
    }

    # ---- CPU baseline beside it (N = 1 only): bounded sample on this machine's host cores
    if WORLD == 1 and not args.no_cpu_baseline:
        try:
            var32 = {k: v.astype(np.float32) for k, v in var16.items()}
            sample = WORKLOAD.get("cpu_sample", 32)
            rate, kind, cores, sec = cpu_reference_rate(cfg, var32, S, sample, WORKLOAD["lengths"] or "full",
                                                        WORKLOAD["seed"], 3, 1)
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": kind,
                                    "sample": "%d sequences of the batch per step, float32 (the reference's CPU "
                                              "build has no binary16), 1 warm-up + 3 timed steps, %.2f s/step"
                                              % (sample, sec)}
        except Exception as e:  # the baseline must not take the benchmark down
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "unavailable",
                                    "sample": repr(e)}
    print(json.dumps(line), flush=True)
    m.close()
    if WORLD > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="base_seq128", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="sequences per step of the CPU reference (default: the workload's bounded sample)")
    args = ap.parse_args()
    global WORKLOAD, WORKLOAD_NAME
    WORKLOAD = WORKLOADS[args.workload]
    WORKLOAD_NAME = args.workload
    if args.cpu_sample > 0:
        WORKLOAD = dict(WORKLOAD, cpu_sample=min(args.cpu_sample, WORKLOAD["batch"]))
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
