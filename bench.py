#!/usr/bin/env python
"""Benchmark of the encoder-stack hot path on B200.

Workload (the configuration the headline metric is quoted on): a 12-layer post-LN encoder
stack, hidden 768, 12 heads x 64, FFN 3072, exact GELU, fp16 storage with fp32 accumulation,
sequence length 128, all-valid mask, a global batch of 256 sequences per step; weights i.i.d.
N(0, 0.02), biases 0, input N(0, 1), all seeded synthetic data.  A step is one pass of the
stack over one batch through the library's C ABI (mgpuEncoderStackRun).  With N GPUs the
batch is sharded: rank r runs sequences [r*256/N, (r+1)*256/N) on its own GPU, no collective
in the data path (strong scaling, the default), and `value` is the 256 sequences divided by
the slowest rank's time per step.  The line also carries, as `weak`, the same measurement
with 256 sequences on every rank (--scaling weak makes that the headline instead).

  python bench.py --gpus N --steps K --warmup W            one JSON line (rank 0)
  python bench.py --impl reference ...                     the CPU restatement of the
                                                           reference's path on the host cores

The timed region holds only library calls on device-resident buffers and is bracketed by
a barrier and a device synchronisation; time is taken with CUDA events on the launching
stream and the maximum over ranks is reported.  `e2e` repeats the measurement with pinned
HOST buffers (upload, compute and download of every step inside the timed region, host
wall clock): batches streamed through mgpuEncoderStackSubmitHost / WaitHost, and, as
`e2e.synchronous`, one blocking mgpuEncoderStackRunHost call per step.  `roofline` describes the dominant kernel (the tcgen05 Gemm, 48 launches
per step): its launches are bracketed by CUDA events in a second pass over the same K
steps (mgpuOpsProfileBegin/End), so the headline time is not perturbed by the extra events.
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
sys.path.insert(0, ROOT)

L, GLOBAL_BATCH, S, D, F, H = 12, 256, 128, 768, 3072, 12
B_PER_GPU = GLOBAL_BATCH  # weak scaling: sequences on every rank
WORKLOAD = "encoder-stack-12L-h768-ffn3072-12heads-seq128-batch256"
METRIC, UNIT = "encoder_stack_seqs_per_sec", "seq/s"

GEMM_LAUNCHES_PER_STEP = 4 * L


def gemm_flops_per_step(batch):
    """Algorithmic FLOPs of the 4 Gemms per layer over batch * S tokens."""
    return L * 2 * batch * S * (D * 3 * D + D * D + 2 * D * F)


def bytes_touched_per_step(batch):
    """Distinct device bytes one step reads or writes: packed weights + 16-bit activations +
    the fp32 boundary tensors.  Compared with the L2 size to say whether steps re-use L2."""
    t = batch * S
    return L * 2 * (D * 3 * D + D * D + 2 * D * F) + t * 2 * (4 * D + 3 * D + F) + 2 * t * D * 4
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each of the four
# Gemm shapes of a layer, from one-launch ncu captures of `bench.py --micro gemm_* --tokens T`;
# keyed by T.  The roofline's `traffic` is their mean at the step's token count, or, for a
# token count without a capture, the nearest capture with the token-proportional part (A,
# residual, output) scaled and the weights kept.
GEMM_DRAM_TRAFFIC = {
    # tokens: {shape: bytes}
    32768: {"gemm_qkv": 53925888 + 96961536, "gemm_proj": 51560192 + 10394880,
            "gemm_ffn1": 55139072 + 143000064, "gemm_ffn2": 206767872 + 37095936},
    4096: {"gemm_qkv": 9883904, "gemm_proj": 7518208, "gemm_ffn1": 11096832, "gemm_ffn2": 29931520 + 1280},
}


def gemm_operand_bytes(tokens):
    """Algorithmic bytes per launch of the four Gemms (A + W + residual + out, 16-bit)."""
    t = tokens
    return {"gemm_qkv": 2 * (t * D + 3 * D * D + t * 3 * D), "gemm_proj": 2 * (t * D + D * D + 2 * t * D),
            "gemm_ffn1": 2 * (t * D + D * F + t * F), "gemm_ffn2": 2 * (t * F + D * F + 2 * t * D)}


def gemm_traffic_per_launch(tokens):
    """Mean DRAM traffic of a Gemm launch of the step (bytes), or None without a capture."""
    if not GEMM_DRAM_TRAFFIC:
        return None
    near = min(GEMM_DRAM_TRAFFIC, key=lambda k: abs(np.log(k / max(tokens, 1))))
    table = GEMM_DRAM_TRAFFIC[near]
    if near == tokens:
        return sum(table.values()) / len(table)
    alg_near, alg = gemm_operand_bytes(near), gemm_operand_bytes(tokens)
    return sum(table[k] * alg[k] / alg_near[k] for k in table) / len(table)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "tflops_burst": p["bf16_tflops"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


def make_weights(seed=0):
    rng = np.random.default_rng(seed)
    layers = []
    for _ in range(L):
        layers.append({
            "wqkv": (0.02 * rng.standard_normal((D, 3 * D))).astype(np.float32), "bqkv": np.zeros(3 * D, np.float32),
            "wo": (0.02 * rng.standard_normal((D, D))).astype(np.float32), "bo": np.zeros(D, np.float32),
            "w1": (0.02 * rng.standard_normal((D, F))).astype(np.float32), "b1": np.zeros(F, np.float32),
            "w2": (0.02 * rng.standard_normal((F, D))).astype(np.float32), "b2": np.zeros(D, np.float32),
            "ln1_g": None, "ln1_b": None, "ln2_g": None, "ln2_b": None})
    return layers


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], None, [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # keep the samples taken under load (upper half of the power readings)
        if power:
            thr = 0.5 * max(power)
            loaded = [c for c, p in zip(sm, power) if p >= thr] or sm
        else:
            loaded = sm
        return {"sm_mhz": float(np.median(loaded)) if loaded else None, "sm_max_mhz": smax,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def max_over_ranks(value, dist, device):
    """The slowest rank's time: an all-reduce(MAX) over the process group (NCCL on GPUs;
    the CPU tests run the same code over gloo)."""
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def shard_of(rank, world, batch, scaling="strong"):
    """(first, count) of the sequences rank `rank` of `world` owns.
    strong: `batch` is the global batch; rank r takes [r*batch/world, (r+1)*batch/world).
    weak:   `batch` is what every rank runs; the global batch is world * batch."""
    if scaling == "weak":
        return rank * batch, batch
    first = rank * batch // world
    return first, (rank + 1) * batch // world - first


def pick_cpu_gemm(oracle, x, layers):
    """The CPU arm should be the fastest this port can be: times one layer over a few sequences
    with the oracle's own AVX2 loop and with cblas_sgemm of the OpenBLAS bundled with numpy
    (when the wheel carries one) and keeps the faster (the name goes into `gemm_kernel`)."""
    def once():
        t0 = time.perf_counter()
        oracle.encoder_stack(x, layers[:1], None, H, round_mode=oracle.ROUND_F16)
        return time.perf_counter() - t0
    oracle.use_blas(False)
    once()
    own = min(once(), once())
    if oracle.use_blas(True):
        once()
        blas = min(once(), once())
        if blas > own:
            oracle.use_blas(False)


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement of the reference's path (oracle/), all host
    threads, on a bounded sample of the same workload per step."""
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1; the CPU arm is meant to use every host thread
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    sample = 16  # sequences per step (the full step is 256)
    layers = make_weights()
    x = np.random.default_rng(1).standard_normal((sample, S, D)).astype(np.float32)
    pick_cpu_gemm(oracle, x[:8], layers)
    for _ in range(max(args.warmup, 0)):
        oracle.encoder_stack(x[:1], layers, None, H, round_mode=oracle.ROUND_F16)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.encoder_stack(x, layers, None, H, round_mode=oracle.ROUND_F16)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    cores = oracle.num_threads()
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": f"{sample} sequences per step"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "gemm_kernel": oracle.gemm_kernel_name(),
                             "gflops": value * (gemm_flops_per_step(1) + L * 4.0 * H * S * S * 64) / 1e9,
                             "sample": f"{sample} of 256 sequences x 12 layers per step, {args.steps} steps"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


MICRO = {
    # name: (kind, M-per-token-or-rows, N, K)   Gemm shapes of one layer + the standalone configs
    "gemm_qkv": ("gemm", None, 3 * D, D), "gemm_proj": ("gemm", None, D, D),
    "gemm_ffn1": ("gemm_gelu", None, F, D), "gemm_ffn2": ("gemm", None, D, F),
    "gemm_c1": ("gemm", 2048, 4096, 4096),
}


# Convolution layers for --micro: the reference's test layer and three ResNet-18 layers at
# batch 32.  N, IC, H, W, OC, KH, KW, stride, padding
CONV_MICRO = {
    "conv_ref": (16, 3, 256, 256, 64, 3, 3, 1, 1),       # test/End2End/GPU/conv.mlir
    "conv_stem": (32, 3, 224, 224, 64, 7, 7, 2, 3),
    "conv_56": (32, 64, 56, 56, 64, 3, 3, 1, 1),
    "conv_14": (32, 256, 14, 14, 256, 3, 3, 1, 1),
}


def run_micro(args):
    """One kernel, a few launches, on random data: the small case the ncu captures are taken
    on.  Prints one JSON line with the CUDA-event time per launch."""
    import __graft_entry__ as entry
    mdc = entry.load_package()
    mdc.init(0)
    rt, ops = mdc.runtime(), mdc.ops()
    rng = np.random.default_rng(0)
    tokens = args.tokens
    stream = rt.mgpuStreamCreate()
    ev0, ev1 = rt.mgpuEventEnableTimeCreate(), rt.mgpuEventEnableTimeCreate()
    name = args.micro
    if name in MICRO:
        kind, M, N, K = MICRO[name]
        M = M or tokens
        a = mdc.to_device(rng.standard_normal((M, K)).astype(np.float16), stream)
        w = mdc.to_device((0.02 * rng.standard_normal((N, K))).astype(np.float16), stream)
        bias = mdc.to_device(np.zeros(N, np.float32), stream)
        out = mdc.DeviceBuffer(M * N * 2, stream)
        act = mdc.ACT_GELU_ERF if kind == "gemm_gelu" else mdc.ACT_NONE
        fn = lambda: ops.mgpuMatmulEx16(a.ptr, w.ptr, bias.ptr, None, out.ptr, M, N, K, mdc.F16, mdc.F16, act, stream)
        work, unit = 2.0 * M * N * K, "TFLOP/s"
    elif name == "matmul_c1_abi":
        # the reference entry point with fp32 operands: cast + weight pack + Gemm per call
        M, N, K = 2048, 4096, 4096
        a = mdc.to_device(rng.standard_normal((M, K)).astype(np.float32), stream)
        w = mdc.to_device((0.02 * rng.standard_normal((K, N))).astype(np.float32), stream)
        bias = mdc.to_device((0.02 * rng.standard_normal(N)).astype(np.float32), stream)
        out = mdc.DeviceBuffer(M * N * 4, stream)
        fn = lambda: ops.mgpuMatmul(a.ptr, w.ptr, bias.ptr, out.ptr, M, N, K, stream)
        work, unit = 2.0 * M * N * K, "TFLOP/s"
    elif name == "layer_c3":
        # one post-LN layer, batch 32, seq 384, valid lengths uniform in [192, 384]
        Bc, Sc = 32, 384
        lw = make_weights()[:1]
        stack = mdc.EncoderStack(lw, H)
        x = mdc.to_device(rng.standard_normal((Bc, Sc, D)).astype(np.float32), stream)
        lens = mdc.to_device(rng.integers(192, 385, Bc).astype(np.int32), stream)
        y = mdc.DeviceBuffer(Bc * Sc * D * 4, stream)
        fn = lambda: ops.mgpuEncoderStackRun(stack.h, x.ptr, lens.ptr, y.ptr, Bc, Sc, stream)
        T3 = Bc * Sc
        work = 2.0 * T3 * (D * 3 * D + D * D + 2 * D * F) + 4.0 * Bc * H * Sc * Sc * 64  # dense count
        unit = "TFLOP/s"
    elif name == "attention_c3":
        Bc, Sc = 32, 384
        q = mdc.to_device(rng.standard_normal((Bc * Sc, 3 * H * 64)).astype(np.float16), stream)
        lens = mdc.to_device(rng.integers(192, 385, Bc).astype(np.int32), stream)
        out = mdc.DeviceBuffer(Bc * Sc * H * 64 * 2, stream)
        fn = lambda: ops.mgpuAttention(q.ptr, lens.ptr if args.hidden != 1 else None, out.ptr, Bc, Sc, H, 64, False, mdc.F16, stream)
        work, unit = 4.0 * Bc * H * Sc * Sc * 64, "TFLOP/s"
    elif name == "attention":
        Bq = max(tokens // S, 1)
        q = mdc.to_device(rng.standard_normal((Bq * S, 3 * H * 64)).astype(np.float16), stream)
        out = mdc.DeviceBuffer(Bq * S * H * 64 * 2, stream)
        fn = lambda: ops.mgpuAttention(q.ptr, None, out.ptr, Bq, S, H, 64, False, mdc.F16, stream)
        work, unit = 4.0 * Bq * H * S * S * 64, "TFLOP/s"
    elif name == "attention_d128":
        # the head geometry of the reference layer (8 heads x 128, causal), sequences of 256
        Sd, Hd, Dd = 256, 8, 128
        Bq = max(tokens // Sd, 1)
        q = mdc.to_device(rng.standard_normal((Bq * Sd, 3 * Hd * Dd)).astype(np.float16), stream)
        out = mdc.DeviceBuffer(Bq * Sd * Hd * Dd * 2, stream)
        fn = lambda: ops.mgpuAttention(q.ptr, None, out.ptr, Bq, Sd, Hd, Dd, True, mdc.F16, stream)
        work, unit = 4.0 * Bq * Hd * Sd * Sd * Dd, "TFLOP/s"  # dense count (the causal half is skipped)
    elif name == "layernorm_f16":
        rows, n = tokens, args.hidden
        a = mdc.to_device(rng.standard_normal((rows, n)).astype(np.float16), stream)
        c = mdc.DeviceBuffer(rows * n * 2, stream)
        fn = lambda: ops.mgpuLayerNormEx(a.ptr, None, None, None, None, c.ptr, 1e-5, rows, n, mdc.F16, mdc.F16, stream)
        work, unit = 2.0 * rows * n * 2, "GB/s"
    elif name in ("layernorm_f32", "add_f32"):
        rows, n = tokens, args.hidden
        a = mdc.to_device(rng.standard_normal((rows, n)).astype(np.float32), stream)
        b = mdc.to_device(rng.standard_normal((rows, n)).astype(np.float32), stream)
        c = mdc.DeviceBuffer(rows * n * 4, stream)
        if name == "layernorm_f32":
            fn = lambda: ops.mgpuLayerNormF32(a.ptr, None, None, c.ptr, 1e-5, rows, n, stream)
            work, unit = 2.0 * rows * n * 4, "GB/s"
        else:
            fn = lambda: ops.mgpuAdd(a.ptr, b.ptr, c.ptr, rows * n, stream)
            work, unit = 3.0 * rows * n * 4, "GB/s"
    elif name in CONV_MICRO:
        # N, IC, H, W, OC, KH, KW, stride, padding (symmetric), relu
        Nn, IC, Hh, Ww, OC, KH, KW, st, pd = CONV_MICRO[name]
        OH, OW = (Hh + 2 * pd - KH) // st + 1, (Ww + 2 * pd - KW) // st + 1
        x = mdc.to_device(rng.standard_normal((Nn, IC, Hh, Ww)).astype(np.float32), stream)
        w = mdc.to_device((rng.standard_normal((OC, IC, KH, KW)) / np.sqrt(IC * KH * KW)).astype(np.float32), stream)
        bias = mdc.to_device(np.zeros(OC, np.float32), stream)
        out = mdc.DeviceBuffer(Nn * OC * OH * OW * 4, stream)
        fn = lambda: ops.mgpuConv2d(x.ptr, w.ptr, bias.ptr, out.ptr, None, Nn, IC, Hh, Ww, OC, KH, KW, OH, OW,
                                    pd, pd, pd, pd, st, st, 1, 1, False, True, stream)
        work, unit = 2.0 * Nn * OH * OW * OC * IC * KH * KW, "TFLOP/s"
    elif name == "maxpool_ref":
        # test/End2End/GPU/pool.mlir scaled x8 in batch so the tensors exceed L2: 4x4 / stride 4
        Nn, Cc, Hh, Ww = 128, 3, 256, 256
        x = mdc.to_device(rng.standard_normal((Nn, Cc, Hh, Ww)).astype(np.float32), stream)
        out = mdc.DeviceBuffer(Nn * Cc * 64 * 64 * 4, stream)
        fn = lambda: ops.mgpuPool2d(x.ptr, out.ptr, Nn, Cc, Hh, Ww, 64, 64, 4, 4, 0, 0, 0, 0, 4, 4, 0, stream)
        work, unit = Nn * Cc * (Hh * Ww + 64 * 64) * 4.0, "GB/s"
    else:
        raise SystemExit(f"unknown --micro {name}")
    for _ in range(args.warmup):
        fn()
    rt.mgpuEventRecord(ev0, stream)
    for _ in range(args.steps):
        fn()
    rt.mgpuEventRecord(ev1, stream)
    rt.mgpuEventSynchronize(ev1)
    ms = rt.mgpuEventElapsedTime(ev0, ev1) / args.steps
    status = ops.mgpuOpsCheckDeviceStatus(stream)
    mdc.check("micro")
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"micro": name, "tokens": tokens, "ms_per_launch": ms, "rate": rate, "unit": unit,
                      "device_status": status}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, help="run one kernel only (for profiling): " + ", ".join(
        list(MICRO) + ["matmul_c1_abi", "layer_c3", "attention", "attention_c3", "attention_d128", "layernorm_f32", "layernorm_f16", "add_f32",
                     "maxpool_ref"] + list(CONV_MICRO)))
    ap.add_argument("--tokens", type=int, default=8192, help="--micro: rows / tokens of the small case")
    ap.add_argument("--hidden", type=int, default=768, help="--micro layernorm_f32 / add_f32: row length")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--chunks", type=int, default=3, help="pipeline depth of the host-buffer (e2e) path")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="progress messages on stderr")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: --batch is the global batch, sharded over the ranks; weak: every rank runs --batch")
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="sequences per step (see --scaling)")
    ap.add_argument("--no-weak", action="store_true", help="skip the secondary weak-scaling measurement at N > 1")
    ap.add_argument("--only-timed", action="store_true",
                    help="stop after the device-resident timed region (used for the ncu launch list)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.micro:
        run_micro(args)
        return

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    import __graft_entry__ as entry
    mdc = entry.load_package()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        # NCCL prints its version banner on stdout when the communicator is created; stdout
        # must carry the one JSON line only, so it points at stderr until NCCL is up
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier(device_ids=[local_rank])
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    note("process group up")
    mdc.init(local_rank)  # fails loudly without the CUDA libraries or a GPU
    rt, ops = mdc.runtime(), mdc.ops()

    def barrier():
        rt.mgpuStreamSynchronize(None)
        if dist is not None:
            dist.barrier(device_ids=[local_rank])
            import torch
            torch.cuda.synchronize()

    def _max(v):
        return max_over_ranks(v, dist, f"cuda:{local_rank}")

    def gather(values):
        """Every rank's list of floats, as a list of lists indexed by rank."""
        if dist is None:
            return [list(values)]
        import torch
        t = torch.tensor(list(values), dtype=torch.float64, device=f"cuda:{local_rank}")
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return [[float(v) for v in o.tolist()] for o in out]

    sampler = ClockSampler(local_rank)
    sampler.start()  # nvidia-smi needs a moment before its first sample; runs until the timed region ends
    layers = make_weights()
    stack = mdc.EncoderStack(layers, H, norm_first=False, causal=False, act=mdc.ACT_GELU_ERF, dtype=mdc.F16)
    first, batch = shard_of(rank, world, args.batch, args.scaling)
    global_batch = args.batch if args.scaling == "strong" else args.batch * world
    max_batch = max(batch, B_PER_GPU if (world > 1 and args.scaling == "strong" and not args.no_weak) else batch)
    # every rank draws the global input from one seed and keeps its own slice of it
    x_all = np.random.default_rng(1).standard_normal((max(global_batch, max_batch), S, D)).astype(np.float32)
    x = np.ascontiguousarray(x_all[first:first + batch])
    x_weak = x_all[:max_batch]
    # rank 0 re-computes the last rank's shard after the gather to check it bit for bit
    lf, lc = shard_of(world - 1, world, args.batch, args.scaling)
    x_last = np.ascontiguousarray(x_all[lf:lf + lc]) if (rank == 0 and world > 1 and args.scaling == "strong") else None
    del x_all
    stream = rt.mgpuStreamCreate()
    dx = mdc.to_device(x_weak, stream)
    dy = mdc.DeviceBuffer(x_weak.nbytes, stream)
    if max_batch > batch:
        rt.mgpuMemcpy(dx.ptr, x.ctypes.data, x.nbytes, stream)  # the rank's own shard in front
        rt.mgpuStreamSynchronize(stream)
    ev0, ev1 = rt.mgpuEventEnableTimeCreate(), rt.mgpuEventEnableTimeCreate()

    def timed_device(nb, steps, warmup):
        """warmup + steps passes over nb device-resident sequences; (max-over-ranks ms, launches)."""
        def step():
            ops.mgpuEncoderStackRun(stack.h, dx.ptr, None, dy.ptr, nb, S, stream)
        for _ in range(warmup):
            step()
        rt.mgpuStreamSynchronize(stream)
        barrier()
        launches0 = ops.mgpuOpsLaunchCount()
        t_host0 = time.perf_counter()
        rt.mgpuEventRecord(ev0, stream)
        for _ in range(steps):
            step()
        rt.mgpuEventRecord(ev1, stream)
        host_issue_ms = 1e3 * (time.perf_counter() - t_host0)
        rt.mgpuEventSynchronize(ev1)
        barrier()
        own = rt.mgpuEventElapsedTime(ev0, ev1)
        return _max(own), own, ops.mgpuOpsLaunchCount() - launches0, host_issue_ms

    note("weights packed")
    # ---------------- device-resident timed region ----------------
    ms_total, ms_own, launches, host_issue_ms = timed_device(batch, args.steps, args.warmup)
    clocks = sampler.stop()
    status = ops.mgpuOpsCheckDeviceStatus(stream)
    mdc.check("timed region")
    if status:
        raise mdc.MdcError(f"device status 0x{status:08x}")
    ms_per_step = ms_total / args.steps
    value = global_batch * args.steps / (ms_total / 1e3)
    if args.only_timed:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": ms_per_step, "gpu_launches": int(launches),
                              "batch_per_gpu": batch, "host_issue_ms_per_step": host_issue_ms / args.steps,
                              "note": "timed region only"}), flush=True)
        stack.close()
        return

    note(f"timed region done: {ms_per_step:.3f} ms/step")
    # ---------------- per-kernel pass: Gemm launch durations ----------------
    ms_cat = (mdc.C.c_double * 4)()
    n_cat = (mdc.C.c_uint64 * 4)()
    ops.mgpuOpsProfileBegin()
    for _ in range(args.steps):
        ops.mgpuEncoderStackRun(stack.h, dx.ptr, None, dy.ptr, batch, S, stream)
    ops.mgpuOpsProfileEnd(ms_cat, n_cat)
    pk = peaks()
    gemm_ms_per_launch = ms_cat[0] / max(n_cat[0], 1)
    flops_per_launch = gemm_flops_per_step(batch) / GEMM_LAUNCHES_PER_STEP
    achieved_tflops = flops_per_launch / (gemm_ms_per_launch * 1e-3) / 1e12
    roofline = {"kernel": "gemm_tcgen05_kernel", "bound": "tensor", "achieved": achieved_tflops, "peak": pk["tflops"],
                "unit": "TFLOP/s", "frac": achieved_tflops / pk["tflops"], "traffic": gemm_traffic_per_launch(batch * S),
                "peak_source": f"{pk['source']} (sustained bf16; burst {pk['tflops_burst']})",
                "frac_of_burst": achieved_tflops / pk["tflops_burst"],
                "algorithmic_flop_per_launch": flops_per_launch,
                "launches_per_step": int(n_cat[0] // args.steps), "ms_per_launch": gemm_ms_per_launch,
                "time_share_per_step": {"gemm_ms": ms_cat[0] / args.steps, "attention_ms": ms_cat[1] / args.steps,
                                        "layernorm_ms": ms_cat[2] / args.steps, "cast_ms": ms_cat[3] / args.steps}}

    # The instrumented pass runs eagerly with an event before and after every launch, so each
    # kernel's share includes the launch gap that programmatic dependent launch and graph replay
    # hide in the timed region; the same shares scaled to the timed step give the in-step rate.
    cat_sum = sum(ms_cat[i] for i in range(4)) / args.steps
    if cat_sum > 0:
        scale = min(1.0, ms_per_step / cat_sum)
        roofline["achieved_scaled_to_timed_step"] = achieved_tflops / scale
        roofline["frac_of_burst_scaled_to_timed_step"] = achieved_tflops / scale / pk["tflops_burst"]
        roofline["note"] = ("achieved = FLOP / event-bracketed launch time of the instrumented (eager) pass; "
                            "the timed step itself is %.3f of the sum of those times" % scale)
    note("per-kernel pass done")
    # ---------------- the other scaling mode, device-resident only ----------------
    weak = None
    if world > 1 and args.scaling == "strong" and not args.no_weak:
        w_ms, _, _, _ = timed_device(B_PER_GPU, args.steps, args.warmup)
        weak = {"value": world * B_PER_GPU * args.steps / (w_ms / 1e3), "unit": UNIT, "ms_per_step": w_ms / args.steps,
                "batch_per_gpu": B_PER_GPU, "global_batch": world * B_PER_GPU,
                "note": "every rank runs 256 sequences (replicas); device-resident inputs"}
        rt.mgpuMemcpy(dx.ptr, x.ctypes.data, x.nbytes, stream)
        rt.mgpuStreamSynchronize(stream)

    # ---------------- the one exchange of the path: the final gather of the output shards ----------------
    gather_info = None
    if world > 1 and args.scaling == "strong":
        import torch
        ops.mgpuEncoderStackRun(stack.h, dx.ptr, None, dy.ptr, batch, S, stream)
        rt.mgpuStreamSynchronize(stream)
        per = (global_batch + world - 1) // world  # equal-sized slots (the last shards may be shorter)
        mine = torch.zeros((per, S, D), dtype=torch.float32, device=f"cuda:{local_rank}")
        rt.mgpuMemcpy(mine.data_ptr(), dy.ptr, x.nbytes, stream)  # device to device
        rt.mgpuStreamSynchronize(stream)
        everyone = torch.empty((world * per, S, D), dtype=torch.float32, device=f"cuda:{local_rank}")
        for _ in range(2):
            dist.all_gather_into_tensor(everyone, mine)
        torch.cuda.synchronize()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            dist.all_gather_into_tensor(everyone, mine)
        g1.record()
        torch.cuda.synchronize()
        gather_ms = _max(g0.elapsed_time(g1)) / args.steps
        gather_info = {"ms_per_step": gather_ms, "bytes_per_rank": int(mine.numel() * 4),
                       "api": "torch.distributed.all_gather_into_tensor over NCCL",
                       "note": "not part of `value`: the stack has no collective; this is the final output gather"}
        if rank == 0:
            # the last rank's shard, recomputed here: sharding must not change a single bit
            dxl = mdc.to_device(x_last, stream)
            dyl = mdc.DeviceBuffer(x_last.nbytes, stream)
            ops.mgpuEncoderStackRun(stack.h, dxl.ptr, None, dyl.ptr, x_last.shape[0], S, stream)
            mine_again = mdc.to_host(dyl, x_last.shape, np.float32, stream)
            theirs = everyone[(world - 1) * per:(world - 1) * per + x_last.shape[0]].cpu().numpy()
            gather_info["last_shard_bit_identical_to_rank0_recompute"] = bool(np.array_equal(mine_again, theirs))
            dxl.release(stream)
            dyl.release(stream)
        del everyone, mine

    # ---------------- end to end through host buffers ----------------
    # (1) a stream of batches through SubmitHost / WaitHost: batch i+1 uploads while batch i
    #     computes and batch i-1 downloads; two pinned input and two pinned output buffers
    #     alternate, every step's upload and download lie inside the timed region;
    # (2) the synchronous RunHost call (returns when the result is in host memory), whose
    #     first upload and last download are exposed in every step.
    xs, ys = [x, x.copy()], [np.empty_like(x), np.empty_like(x)]
    for a in xs + ys:
        rt.mgpuMemHostRegister(a.ctypes.data, a.nbytes)

    def pipelined(steps):
        tickets = []
        for i in range(steps):
            tickets.append(stack.submit_host(xs[i & 1], ys[i & 1], None))
            if i >= 1:
                stack.wait_host(tickets[i - 1])  # the result of step i-1 is in ys[(i-1) & 1] here
        stack.wait_host(tickets[-1])

    pipelined(3)
    barrier()
    t0 = time.perf_counter()
    pipelined(args.steps)
    e2e_own = 1e3 * (time.perf_counter() - t0)
    e2e_ms = _max(e2e_own)
    barrier()
    for _ in range(2):
        stack.run_host(xs[0], ys[0], None, chunks=args.chunks)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        stack.run_host(xs[0], ys[0], None, chunks=args.chunks)  # returns when the result is complete
    sync_ms = _max(1e3 * (time.perf_counter() - t0))
    barrier()

    # where the end-to-end time goes, per rank: the upload alone, the download alone (all ranks
    # copying at the same time, as in the pipelined run) beside the device-resident step
    def copy_ms(dst, src, nbytes):
        for _ in range(2):
            rt.mgpuMemcpy(dst, src, nbytes, stream)
        rt.mgpuStreamSynchronize(stream)
        barrier()
        rt.mgpuEventRecord(ev0, stream)
        for _ in range(args.steps):
            rt.mgpuMemcpy(dst, src, nbytes, stream)
        rt.mgpuEventRecord(ev1, stream)
        rt.mgpuEventSynchronize(ev1)
        return rt.mgpuEventElapsedTime(ev0, ev1) / args.steps
    h2d_ms = copy_ms(dx.ptr, xs[0].ctypes.data, x.nbytes)
    d2h_ms = copy_ms(ys[0].ctypes.data, dy.ptr, x.nbytes)
    barrier()
    per_rank = gather([ms_own / args.steps, h2d_ms, d2h_ms, e2e_own / args.steps, host_issue_ms / args.steps])
    for a in xs + ys:
        rt.mgpuMemHostUnregister(a.ctypes.data)
    mdc.check("e2e region")
    split = {"per_rank": [{"rank": r, "compute_ms": v[0], "h2d_ms": v[1], "d2h_ms": v[2],
                           "h2d_gbs": x.nbytes / v[1] / 1e6, "d2h_gbs": x.nbytes / v[2] / 1e6,
                           "e2e_ms": v[3], "host_issue_ms": v[4]} for r, v in enumerate(per_rank)],
             "note": "per step; copies timed alone on every rank at the same time (pinned host memory); "
                     "the pipelined e2e step overlaps the three, so its floor is the largest of them"}
    e2e = {"value": global_batch * args.steps / (e2e_ms / 1e3), "unit": UNIT,
           "h2d_bytes_per_step": int(x.nbytes), "d2h_bytes_per_step": int(x.nbytes),
           "ms_per_step": e2e_ms / args.steps, "api": "mgpuEncoderStackSubmitHost / WaitHost, one batch in flight behind",
           "bytes_note": "per rank; the whole job moves n_gpus times as much",
           "synchronous": {"value": global_batch * args.steps / (sync_ms / 1e3), "ms_per_step": sync_ms / args.steps,
                           "api": "mgpuEncoderStackRunHost", "chunks": args.chunks},
           "split": split}

    note("e2e done")
    # ---------------- HBM-bound kernels of the metric: LayerNorm and Add ----------------
    hbm = {}
    if rank == 0:
        def time_ms(fn, iters=20):
            for _ in range(3):
                fn()
            rt.mgpuEventRecord(ev0, stream)
            for _ in range(iters):
                fn()
            rt.mgpuEventRecord(ev1, stream)
            rt.mgpuEventSynchronize(ev1)
            return rt.mgpuEventElapsedTime(ev0, ev1) / iters
        rows, n = 16384 * 8, 768  # 8 x the [32,512,768] config so the tensors exceed L2
        a = mdc.DeviceBuffer(rows * n * 4, stream)
        b = mdc.DeviceBuffer(rows * n * 4, stream)
        c = mdc.DeviceBuffer(rows * n * 4, stream)
        ms = time_ms(lambda: ops.mgpuLayerNormF32(a.ptr, None, None, b.ptr, 1e-5, rows, n, stream))
        hbm["layernorm_f32_gbs"] = 2 * rows * n * 4 / ms / 1e6
        ms = time_ms(lambda: ops.mgpuAdd(a.ptr, b.ptr, c.ptr, rows * n, stream))
        hbm["add_f32_gbs"] = 3 * rows * n * 4 / ms / 1e6
        hbm["peak_gbs"] = pk["hbm_gbs"]
        hbm["layernorm_frac"] = hbm["layernorm_f32_gbs"] / pk["hbm_gbs"]
        hbm["add_frac"] = hbm["add_f32_gbs"] / pk["hbm_gbs"]
        hbm["note"] = f"{rows}x{n} fp32 (805 MB per tensor, larger than L2); {pk['source']} peak"
        for buf in (a, b, c):
            buf.release(stream)

    # ---------------- CPU baseline (rank 0, N = 1 only) ----------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))
        oracle = entry.load_oracle()
        sample = min(64, batch)
        pick_cpu_gemm(oracle, x[:8], layers)
        oracle.encoder_stack(x[:1], layers[:1], None, H, round_mode=oracle.ROUND_F16)  # warm the threads
        t0 = time.perf_counter()
        ref = oracle.encoder_stack(x[:sample], layers, None, H, round_mode=oracle.ROUND_F16)
        dt = time.perf_counter() - t0
        ops.mgpuEncoderStackRun(stack.h, dx.ptr, None, dy.ptr, batch, S, stream)
        got = mdc.to_host(dy, x.shape, np.float32, stream)[:sample]
        cpu = {"value": sample / dt, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
               "gemm_kernel": oracle.gemm_kernel_name(),
               "gflops": sample * (gemm_flops_per_step(1) + L * 4.0 * H * S * S * 64) / dt / 1e9,
               "sample": f"{sample} of {batch} sequences x 12 layers, once ({dt:.1f} s)",
               "parity_max_rel_vs_gpu": oracle.max_rel_err(ref, got, floor_frac=1.0),
               "parity_max_rel_vs_gpu_floor_1e-2rms": oracle.max_rel_err(ref, got, floor_frac=1e-2)}

    note("printing")
    if rank == 0:
        touched = bytes_touched_per_step(batch)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD, "layers": L, "hidden": D, "ffn": F, "heads": H, "seq_len": S,
                           "batch_per_gpu": batch, "global_batch": global_batch,
                           "parallelism": f"batch sharded over {world} GPU(s), weights replicated, no collective",
                           "l2": f"a step touches {touched / 1e6:.0f} MB of distinct device memory per GPU "
                                 f"(weights + activations), {'more' if touched > 126e6 else 'LESS'} than the 126 MB L2; "
                                 "no explicit flush"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "hbm_kernels": hbm, "cpu_baseline": cpu}
        if weak is not None:
            line["weak"] = weak
        if gather_info is not None:
            line["gather"] = gather_info
        print(json.dumps(line), flush=True)
    stack.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
