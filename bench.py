"""Benchmark of the quantized matrix-product hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded
synthetic input; `value` is whole-job throughput with inputs resident in HBM, `e2e` the same metric
through the public ComputeContext API with host buffers (uploads and the result download inside the
timed region; the encoder workload feeds its batches through two recorded forwards on two streams, so one
batch's copies run under the other's compute - every step still uploads its inputs and reads its result).  `roofline` describes the dominant kernel, timed per launch with CUDA events on the
context's own stream; `cpu_baseline` is the CPU port of the reference's wasm kernels on a bounded
sample.  `--impl reference` times that CPU port alone with every host thread (rank 0 only).

Multi-GPU (torchrun, one process per GPU): the units of work (decode products / encoder windows)
are independent, so each rank runs its own share with no data-path collective ("weak" scaling);
the barrier and the max-over-ranks time are the only cross-rank steps.
"""
from __future__ import annotations

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

L2_BYTES = 126 * 1024 * 1024


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------

def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# --------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------

class Int4Decode:
    """Benchmark configuration 2 (int4 decode): int4 group-quantised decode products (Nemotron-style projection).
    K=2048, N=8192, M in {1,4,16}; a rotating set of distinct weight matrices larger than L2
    so every product streams its weights from HBM.  Seed 1."""

    name = "int4_decode_k2048_n8192_m1-4-16"
    metric = "int4_decode_weight_stream"
    unit = "GB/s"
    dtype = "u4 weights x f16 activations, f32 accumulate"
    dominant = "nbits"

    def __init__(self, quick=False):
        self.K, self.N, self.Ms = 2048, 8192, (1, 4, 16)
        self.nblk = self.K // 32
        self.nsets = 8 if quick else 32  # 32 x 10.3 MB = 330 MB > 2 x L2

    def weight_bytes(self):  # reference format: int4 + f32 scale per block + packed zero-points
        return self.N * self.K // 2 + self.N * self.nblk * 4 + self.N * (self.nblk // 2)

    def algorithmic_bytes(self, M):  # bytes of the reference's own storage format
        return self.weight_bytes() + 4 * M * self.K + 4 * M * self.N

    def host_data(self):
        rng = np.random.default_rng(1)
        sets = []
        for _ in range(self.nsets):
            s = rng.integers(-8, 8, (self.N, self.K), dtype=np.int8) + 8
            bq = (s[:, 0::2] | (s[:, 1::2] << 4)).astype(np.uint8).reshape(-1)
            scales = rng.uniform(5e-3, 2e-2, self.N * self.nblk).astype(np.float16).astype(np.float32)
            zp = np.full(self.N * (self.nblk // 2), 0x88, np.uint8)
            sets.append((bq, scales, zp))
        acts = {M: rng.standard_normal((M, self.K)).astype(np.float16).astype(np.float32) for M in self.Ms}
        return sets, acts

    def setup(self, ctx):
        sets, acts = self.host_data()
        self.host_acts = {}
        for M, a in acts.items():  # e2e uploads come from page-locked memory
            buf = ctx.pinnedArray(a.size)
            buf[:] = a.reshape(-1)
            self.host_acts[M] = buf
        self.dev_sets = [(ctx.uploadBytes(bq), ctx.upload(sc, 1, sc.size), ctx.uploadBytes(zp)) for bq, sc, zp in sets]
        self.dev_acts = {M: ctx.upload(a, M, self.K) for M, a in acts.items()}
        self.units_per_step = self.nsets * len(self.Ms)  # products
        self.bytes_per_step = sum(self.algorithmic_bytes(M) for M in self.Ms) * self.nsets

    def step_device(self, ctx):
        h = ctx.pushArena()
        for M in self.Ms:
            a = self.dev_acts[M]
            for bq, sc, zp in self.dev_sets:
                ctx.matmulNBits(a, bq, sc, zp, self.N)
        ctx.popArena(h)

    def step_e2e(self, ctx):
        h = ctx.pushArena()
        last = None
        for M in self.Ms:
            a = ctx.upload(self.host_acts[M], M, self.K)
            for bq, sc, zp in self.dev_sets:
                last = ctx.matmulNBits(a, bq, sc, zp, self.N)
            out = ctx.download(last)
            ctx.freeTensor(a)
        ctx.popArena(h)
        return out

    def e2e_bytes(self):
        return sum(4 * M * self.K for M in self.Ms), sum(4 * M * self.N for M in self.Ms)

    def value_from(self, steps, seconds):
        return self.bytes_per_step * steps / seconds / 1e9

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"].startswith(("gemv_nbits", "nbits", "tc_gemm"))]
        if not ent:
            return None
        e = max(ent, key=lambda x: x["ms"])
        per_launch_ms = e["ms"] / e["count"]
        alg = sum(self.algorithmic_bytes(M) for M in self.Ms) / len(self.Ms)
        ach = alg / (per_launch_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(ach / peaks["hbm_gbs"], 4), "traffic": None, "kernel": e["label"],
                "avg_launch_us": round(per_launch_ms * 1e3, 2), "peak_source": peaks["source"]}

    def roofline_live(self, ctx, peaks, timer):
        """The dominant kernel on its own: the M = 1 and M = 4 products (k_gemv_nbits) over the rotating weight
        sets, recorded back to back and replayed; achieved = their algorithmic bytes / CUDA-event time."""
        Ms = [M for M in self.Ms if M <= 4]

        def body():
            h = ctx.pushArena()
            for M in Ms:
                for bq, sc, zp in self.dev_sets:
                    ctx.matmulNBits(self.dev_acts[M], bq, sc, zp, self.N)
            ctx.popArena(h)

        body()
        batch, _ = ctx.recordBatch(body)
        reps = 20
        ms = timer(lambda _c: batch.launch(), reps)
        batch.free()
        n = len(Ms) * self.nsets * reps
        ach = sum(self.algorithmic_bytes(M) for M in Ms) * self.nsets * reps / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(ach / peaks["hbm_gbs"], 4),
                "traffic": 10.8e6, "traffic_note": "per launch, from an ncu capture of the M=4, K=2048, N=8192 launches "
                "(memory throughput x duration); algorithmic bytes per launch 10.6e6",
                "kernel": "k_gemv_nbits (label gemv_nbits), the M = 1 and M = 4 products", "launches_timed": n,
                "avg_launch_us": round(ms * 1e3 / n, 2), "peak_source": peaks["source"]}

    def cpu_sample(self, threads=True):
        """One M=4 product at full N,K on the CPU port; returns (value in GB/s, description)."""
        from oracle.wasm_oracle import T, WasmOracle

        ora = WasmOracle(threads=threads)
        sets, acts = self.host_data() if not hasattr(self, "_hd") else self._hd
        self._hd = (sets, acts)
        bq, sc, zp = sets[0]
        M = 4
        a = T(acts[M], M, self.K)
        bqh, zph, sch = ora.uploadBytes(bq), ora.uploadBytes(zp), T(sc, 1, sc.size)
        reps, t0 = 0, time.perf_counter()
        while True:
            ora.matmulNBits(a, bqh, sch, zph, self.N)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > 8 or reps >= 200:
                break
        return self.algorithmic_bytes(M) * reps / dt / 1e9, f"{reps} x (M=4, N={self.N}, K={self.K}) products, {dt:.1f} s"


class Int8Gemm:
    """Benchmark configuration 1: int8 GEMM in the reference's layout ([K][N] bytes, per-column f32 scales).
    A f32 [512,1024] ~ N(0,1), W int8 [1024][4096] uniform in [-127,127], scales U(1e-3,1e-2).  Seed 0.
    A rotating set of 48 weight matrices (> L2) keeps the weight reads on HBM."""

    name = "int8_gemm_512x1024x4096"
    metric = "int8_gemm_throughput"
    unit = "TOP/s"
    dtype = "s8 x s8 digits -> s32 (f32 activations split in int8 digits), f32 out"

    def __init__(self, quick=False):
        self.M, self.K, self.N = 512, 1024, 4096
        self.nsets = 8 if quick else 48

    def ops(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        return self.M * self.K * 4 + self.K * self.N + self.N * 4 + self.M * self.N * 4

    def host_data(self):
        rng = np.random.default_rng(0)
        a = rng.standard_normal((self.M, self.K)).astype(np.float32)
        ws = [rng.integers(-127, 128, (self.K, self.N), dtype=np.int8) for _ in range(self.nsets)]
        sc = rng.uniform(1e-3, 1e-2, self.N).astype(np.float32)
        return a, ws, sc

    def setup(self, ctx):
        a, ws, sc = self.host_data()
        self.host_a = ctx.pinnedArray(a.size)
        self.host_a[:] = a.reshape(-1)
        self.dev_a = ctx.upload(a, self.M, self.K)
        self.dev_w = [ctx.uploadBytes(w) for w in ws]
        self.dev_sc = ctx.upload(sc, 1, self.N)
        self.units_per_step = self.nsets
        # first use repacks each weight handle once; keep that out of the timed region
        h = ctx.pushArena()
        for w in self.dev_w:
            ctx.matmulInt8(self.dev_a, w, self.dev_sc, self.N, self.K)
        ctx.popArena(h)
        ctx.sync()

    def step_device(self, ctx):
        h = ctx.pushArena()
        for w in self.dev_w:
            ctx.matmulInt8(self.dev_a, w, self.dev_sc, self.N, self.K)
        ctx.popArena(h)

    def step_e2e(self, ctx):
        h = ctx.pushArena()
        out = None
        for w in self.dev_w:
            a = ctx.upload(self.host_a, self.M, self.K)
            out = ctx.download(ctx.matmulInt8(a, w, self.dev_sc, self.N, self.K))
            ctx.freeTensor(a)
        ctx.popArena(h)
        return out

    def e2e_bytes(self):
        return self.nsets * self.M * self.K * 4, self.nsets * self.M * self.N * 4

    def value_from(self, steps, seconds):
        return self.ops() * self.nsets * steps / seconds / 1e12

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"] == "tc_gemm_i8"]
        if not ent:
            return None
        e = ent[0]
        per_launch_ms = e["ms"] / e["count"]
        ach = self.algorithmic_bytes() / (per_launch_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(ach / peaks["hbm_gbs"], 4), "traffic": None, "kernel": e["label"],
                "avg_launch_us": round(per_launch_ms * 1e3, 2), "peak_source": peaks["source"],
                "tensor_tops": round(self.ops() / (per_launch_ms * 1e-3) / 1e12, 1)}

    def cpu_sample(self, threads=True):
        from oracle.wasm_oracle import T, WasmOracle

        ora = WasmOracle(threads=threads)
        a, ws, sc = self.host_data() if not hasattr(self, "_hd") else self._hd
        self._hd = (a, ws, sc)
        Ms = 64  # a 64-row slice of the 512 activation rows
        at, wh, st = T(a[:Ms], Ms, self.K), ora.uploadBytes(ws[0]), T(sc, 1, self.N)
        reps, t0 = 0, time.perf_counter()
        while True:
            ora.matmulInt8(at, wh, st, self.N, self.K)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > 8 or reps >= 100:
                break
        return 2.0 * Ms * self.N * self.K * reps / dt / 1e12, f"{reps} x ({Ms} of 512 rows, N={self.N}, K={self.K}), reference loop order, {dt:.1f} s"


class F16Gemm:
    """Benchmark configuration 3: f16-weight GEMM sweep over FastConformer encoder shapes.
    M in {256, 1024, 4096, 16384} x (K,N) in {(1024,3072), (1024,1024), (1024,4096), (4096,1024)};
    activations ~N(0,1) f32, weights ~N(0,1/K) rounded to f16, f32 accumulate.  Seed 2.
    One step = the 16 products once.  The M >= 4096 products move more than the 126 MB L2 per launch;
    the small ones are L2-resident by nature (8 MB of weights) and are reported as such."""

    name = "f16_gemm_sweep_fastconformer_shapes"
    metric = "f16_gemm_throughput"
    unit = "TFLOP/s"
    dtype = "f16 x f16 -> f32 accumulate, f32 out"
    nsets = 1

    def __init__(self, quick=False):
        self.Ms = (4096,) if quick else (256, 1024, 4096, 16384)
        self.KNs = ((1024, 4096),) if quick else ((1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024))

    def setup(self, ctx):
        rng = np.random.default_rng(2)
        self.W = {kn: ctx.uploadF16((rng.standard_normal(kn) / np.sqrt(kn[0])).astype(np.float32), kn[0], kn[1]) for kn in self.KNs}
        self.host_A, self.A = {}, {}
        for M in self.Ms:
            for K in sorted({k for k, _ in self.KNs}):
                buf = ctx.pinnedArray(M * K)
                buf[:] = rng.standard_normal(M * K).astype(np.float32)
                self.host_A[(M, K)] = buf
                self.A[(M, K)] = ctx.upload(buf, M, K)
        self.units_per_step = len(self.Ms) * len(self.KNs)
        self.flops_per_step = sum(2.0 * M * K * N for M in self.Ms for K, N in self.KNs)

    def step_device(self, ctx):
        h = ctx.pushArena()
        for M in self.Ms:
            for K, N in self.KNs:
                ctx.matmul(self.A[(M, K)], self.W[(K, N)])
        ctx.popArena(h)

    def step_e2e(self, ctx):
        h = ctx.pushArena()
        out = None
        for M in self.Ms:
            for K, N in self.KNs:
                a = ctx.upload(self.host_A[(M, K)], M, K)
                out = ctx.download(ctx.matmul(a, self.W[(K, N)]))
                ctx.freeTensor(a)
        ctx.popArena(h)
        return out

    def e2e_bytes(self):
        return (sum(4 * M * K for M in self.Ms for K, _ in self.KNs), sum(4 * M * N for M in self.Ms for _, N in self.KNs))

    def value_from(self, steps, seconds):
        return self.flops_per_step * steps / seconds / 1e12

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"].startswith("tc_gemm_f16")]
        if not ent:
            return None
        ms = sum(e["ms"] for e in ent)
        n = sum(e["count"] for e in ent)
        return {"bound": "tensor", "achieved": self.flops_per_step / (ms * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": None, "traffic": None, "kernel": "k_tc_gemm<f16>", "launches": n,
                "avg_launch_us": round(ms / n * 1e3, 2), "peak_source": peaks["source"] + " (burst bf16)"}

    def cpu_sample(self, threads=True):
        from oracle.wasm_oracle import T, WasmOracle

        ora = WasmOracle(threads=threads)
        rng = np.random.default_rng(2)
        M, K, N = 64, 1024, 1024
        a, b = T(rng.standard_normal((M, K)).astype(np.float32), M, K), T(rng.standard_normal((K, N)).astype(np.float32), K, N)
        reps, t0 = 0, time.perf_counter()
        while True:
            ora.matmul(a, b)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > 8 or reps >= 400:
                break
        return 2.0 * M * K * N * reps / dt / 1e12, f"{reps} x (64 rows of the 1024x1024 product), {dt:.1f} s"


class Encoder:
    """Benchmark configuration 4: Parakeet-TDT-0.6B-shaped FastConformer encoder (24 blocks, d_model 1024, 8 heads,
    FFN 4096, dw-conv 9, 8x conv subsampling, 128 mel bins), random-init weights stored int8 per output
    channel and dequantised at load as the reference loader does, 15 s windows of synthetic audio
    (pink noise + tones), batch of 32 windows per step per GPU.  Seed 3."""

    name = "fastconformer_0.6b_encoder_15s_windows_batch32"
    metric = "encoder_audio_seconds_per_second"
    unit = "audio-s/s"
    dtype = "f16 weights x f16 activations, f32 accumulate"
    nsets = 1

    weights_mode = "f16"  # "f16": the int8 artifact is dequantised at load to f16 storage, as the reference's loader does
                          # (the faster of the two today); "int8": its matrices stay int8 in HBM (matmulInt8Operand)

    def __init__(self, quick=False):
        self.W = 4 if quick else 32
        self.layers = 4 if quick else 24
        self.window_s = 15.0

    def _load(self, ctx):
        """The encoder from the int8 artifact (blob + manifest, the reference's shipping format)."""
        from fluidaudio_web_b200.engines import blob

        if not hasattr(self, "_artifact"):
            self._artifact = blob.write_int8_blob(self._weights)
        data, man = self._artifact
        return self.fc.load_encoder_blob(ctx, data, man, int8_resident=self.weights_mode == "int8")

    def setup(self, ctx):
        import __graft_entry__ as ge

        ge.load_package()
        from fluidaudio_web_b200.engines import fastconformer, synth

        self.fc = fastconformer
        cfg = dict(synth.PARAKEET_06B, layers=self.layers)
        self._weights = synth.encoder_weights(cfg, seed=3)
        self.enc = self._load(ctx)
        self.dtype = ("int8 weights (resident, widened to f16 in shared memory) x f16 activations, f32 accumulate"
                      if self.weights_mode == "int8" else "f16 weights x f16 activations, f32 accumulate")
        audio = synth.synth_audio(self.W, seed=3)  # one distinct 15 s window per batch slot
        self.n_samples = audio.shape[1]
        # device-resident leg: the windows' log-mel features, computed once by the device front end
        # (time-major, floor(N/160) = 1500 frames per window as the reference's ParakeetMel returns)
        pcm = ctx.upload(audio, self.W, self.n_samples)
        self.dev_mels = ctx.logMelWindows(pcm, 128)
        ctx.freeTensor(pcm)
        self.mel_len = self.dev_mels.cols
        # end-to-end leg: page-locked PCM, one array per pipeline slot (filled by _pcm_slot)
        self._audio = audio
        self.units_per_step = self.W
        self.e2e_batch = None

    def _pcm_slot(self, ctx):
        buf = ctx.pinnedArray(self.W * self.n_samples)
        buf[:] = self._audio.reshape(-1)
        return buf

    def step_device(self, ctx):
        h = ctx.pushArena()
        self.fc.encode_batch(ctx, self.enc, self.dev_mels)  # windows resident in HBM
        ctx.popArena(h)

    def step_e2e(self, ctx):
        # public API, host PCM in, host frames out: PipelinedEncoder keeps two recorded forwards (upload of the windows'
        # 16 kHz samples from page-locked memory, log-mel front end on the device, encoder, read-back of the frames) on
        # two streams of this GPU and alternates, so one batch's copies run under the other's compute; every step
        # uploads its windows and reads its frames back
        if self.e2e_batch is None:
            import __graft_entry__ as ge
            from fluidaudio_web_b200.engines import synth

            ctx2 = ge.load_package().CudaContext(ctx.device)
            enc2 = self._load(ctx2)
            slots = [self._pcm_slot(ctx), self._pcm_slot(ctx2)]
            self.e2e_batch = self.fc.PipelinedEncoder([ctx, ctx2], [self.enc, enc2], lambda s: slots[s], self.n_samples, from_pcm=True)
        return self.e2e_batch.submit()

    def e2e_drain(self):
        return self.e2e_batch.flush() if self.e2e_batch is not None else []

    def e2e_bytes(self):
        return self.W * self.n_samples * 4, self.W * 188 * 1024 * 4

    def value_from(self, steps, seconds):
        return self.W * self.window_s * steps / seconds

    def gemm_flops_per_step(self):
        D, DFF, T = 1024, 4096, 188
        per_frame_layer = 2 * (2 * D * DFF * 2 + 4 * D * D + D * 2 * D + D * D)
        return per_frame_layer * self.layers * T * self.W + 2 * 4096 * D * T * self.W

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"] in ("tc_gemm_f16", "tc_gemm_i8w_f16a")]
        if not ent:
            return None
        e = max(ent, key=lambda x: x["ms"])
        ach = self.gemm_flops_per_step() / (e["ms"] * 1e-3) / 1e12  # prof covers `steps` steps; caller scales
        return {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": None, "traffic": None, "kernel": "tc_gemm_f16", "launches": e["count"],
                "avg_launch_us": round(e["ms"] / e["count"] * 1e3, 2), "peak_source": peaks["source"] + " (sustained bf16)"}

    def roofline_live(self, ctx, peaks, timer):
        """The dominant kernel on its own: the weight products of one conformer block at this batch's
        M (2x FF up, 2x FF down, the fused q|k|v projection at D x 3D, out/pw2 at D x D, pw1 at D x 2D), recorded
        back to back and replayed;
        achieved = their algorithmic FLOPs / CUDA-event time.  The row operands are already packed, as they
        are inside the forward (producers hand them over as f16)."""
        D, DFF, M = 1024, 4096, self.W * 188
        rng = np.random.default_rng(5)
        x1 = ctx.upload(rng.standard_normal((M, D)).astype(np.float32), M, D)
        x4 = ctx.upload(rng.standard_normal((M, DFF)).astype(np.float32), M, DFF)
        L0 = self.enc["layers"][0]
        qkv = [(x1, L0["qkv"])] if "qkv" in L0 else [(x1, L0["q"]), (x1, L0["k"]), (x1, L0["v"])]
        seq = [(x1, L0["ff1w1"]), (x4, L0["ff1w2"])] + qkv + [(x1, L0["out"]), (x1, L0["pw1T"]), (x1, L0["pw2T"]),
                                                             (x1, L0["ff2w1"]), (x4, L0["ff2w2"])]
        flops = sum(2.0 * a.rows * a.cols * b.cols for a, b in seq)

        def body():
            h = ctx.pushArena()
            for a, b in seq:
                self.fc.mm(ctx, a, b)
            ctx.popArena(h)

        body()
        batch, _ = ctx.recordBatch(body)
        reps = 5
        ms = timer(lambda _c: batch.launch(), reps)
        batch.free()
        ctx.freeTensor(x1)
        ctx.freeTensor(x4)
        ach = flops * reps / (ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        return {"bound": "tensor", "achieved": round(ach, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(ach / peak, 4),
                "traffic": 26.3e6, "traffic_note": "ncu dram read+write of ONE launch of this kernel at M=4096, K=1024, N=4096 "
                "(a smaller case than the M=%d products timed here): 16.9 MB read = the two f16 operands once, 9.4 MB "
                "written (the rest of the 67 MB f32 result was still in the 126 MB L2 at kernel end); algorithmic bytes "
                "of that launch 84 MB" % M,
                "kernel": ("k_tc_gemm<int8 weights, f16 activations> (label tc_gemm_i8w_f16a)" if self.weights_mode == "int8"
                           else "k_tc_gemm<f16> (label tc_gemm_f16)"), "launches_timed": len(seq) * reps,
                "avg_launch_us": round(ms * 1e3 / (len(seq) * reps), 2),
                "what": "the %d weight products of one conformer block at M=%d, back to back (recorded batch)" % (len(seq), M),
                "peak_source": peaks["source"] + " (burst bf16: kernel timed alone)"}

    def cpu_sample(self, threads=True):
        """Twelve conformer blocks on one 15 s window on the CPU port, scaled to the full stack."""
        from oracle.wasm_oracle import WasmOracle
        from fluidaudio_web_b200.engines import fastconformer, synth

        nl = 12 if not threads else 4
        key = (threads,)
        if getattr(Encoder, "_cpu_enc", (None,))[0] != key:
            ora = WasmOracle(threads=threads)
            cfg = dict(synth.PARAKEET_06B, layers=nl)
            Encoder._cpu_enc = (key, ora, fastconformer.load_encoder(ora, synth.encoder_weights(cfg, seed=3)))
        _, ora, enc = Encoder._cpu_enc
        x0 = np.random.default_rng(3).standard_normal((188, 1024)).astype(np.float32)
        orig = fastconformer.pre_encode
        fastconformer.pre_encode = lambda c_, e_, m_: (c_.upload(m_, 188, 1024), 188)
        try:
            t0 = time.perf_counter()
            fastconformer.encode_batch(ora, enc, [x0])
            dt = time.perf_counter() - t0
        finally:
            fastconformer.pre_encode = orig
        # 24 blocks per window (the subsampling front end is <2% of the work and is left out of the sample)
        return self.window_s / (dt * 24 / nl), f"{nl} conformer blocks on one 15 s window ({dt:.2f} s), x{24 // nl} for the stack"


class Decoder:
    """Benchmark configuration 5: Whisper-large-v3-turbo-shaped decoder (4 layers, d_model 1280, 20 heads, FFN 5120,
    vocab 51866 padded to 51868), random-init weights, KV-cached greedy decoding of 64 concurrent streams of
    224 tokens after a 4-token forced prefix, cross-attention over 1500 x 1280 encoder states per stream.
    One step = the whole decode of the 64 streams (cross K/V products included).  Seed 5."""

    metric = "decode_tokens_per_second"
    unit = "tokens/s"
    nsets = 1
    quant = None
    profile_steps = 2  # a decode is ~30k launches: two of them are enough for per-launch statistics

    def __init__(self, quick=False):
        self.S = 8 if quick else 64
        self.n_tok = 16 if quick else 224
        self.Tenc = 1500
        self.prefix = [1, 2, 3, 4]
        v = "int8" if self.quant else "f16"
        self.name = f"whisper_large_v3_turbo_decoder_{v}_{self.S}streams_{self.n_tok}tok_greedy"
        self.dtype = ("int8 weights x 3 int8 activation digits, int32 accumulate" if self.quant else
                      "f16 weights x f16 value+residue activations, f32 accumulate")

    def setup(self, ctx):
        import __graft_entry__ as ge

        ge.load_package()
        from fluidaudio_web_b200.engines import synth, whisper_decoder

        self.dm = whisper_decoder
        self.cfg = dict(synth.WHISPER_TURBO_DEC, Tenc=self.Tenc)
        ctx.setOption("int8_limbs", 3)  # f32-grade activations on both weight variants, so that
        ctx.setOption("f16_hilo_rows", 1 << 30)  # greedy token picks follow the f32 reference arithmetic
        self.dec = whisper_decoder.load_decoder(ctx, synth.decoder_weights(self.cfg, seed=5), self.cfg["NH"], quant=self.quant)
        whisper_decoder.resident_tables(ctx, self.dec)
        D = self.cfg["D"]
        base = synth.encoder_states(self.cfg, 4, seed=7)  # 4 distinct clips, cycled over the streams
        self.host_enc = ctx.pinnedArray(self.S * self.Tenc * D)
        self.host_enc.reshape(self.S, self.Tenc, D)[:] = base[np.arange(self.S) % 4]
        self.enc_all = ctx.upload(self.host_enc, self.S * self.Tenc, D)
        self.prefix_idx = [ctx.upload(np.full(self.S, t, np.float32), self.S, 1) for t in self.prefix]
        self.st = whisper_decoder.decode_init_streams(ctx, self.dec, self.S, len(self.prefix) + self.n_tok)
        self.units_per_step = self.S * self.n_tok
        self.e2e_batch = None

    def _decode(self, ctx, enc_all):
        return self.dm.greedy_decode_streams_resident(ctx, self.dec, enc_all, self.S, self.prefix_idx, self.n_tok, st=self.st)

    def step_device(self, ctx):
        ctx.freeTensor(self._decode(ctx, self.enc_all))  # encoder states resident in HBM

    def _e2e_body(self, ctx):
        h = ctx.pushArena()
        enc = ctx.upload(self.host_enc, self.S * self.Tenc, self.cfg["D"])  # H2D from page-locked memory
        hist = ctx.pin(self._decode(ctx, enc), True)
        ctx.popArena(h)
        return hist

    def step_e2e(self, ctx):
        if self.e2e_batch is None:
            ctx.freeTensor(self._e2e_body(ctx))
            self.e2e_batch, self.e2e_out = ctx.recordBatch(lambda: self._e2e_body(ctx))
        self.e2e_batch.launch()
        return ctx.download(self.e2e_out)  # token ids [n_tok, S]

    def e2e_bytes(self):
        return self.S * self.Tenc * self.cfg["D"] * 4, self.n_tok * self.S * 4

    def value_from(self, steps, seconds):
        return self.S * self.n_tok * steps / seconds

    def attn_bytes_per_step(self):
        """Algorithmic bytes of the single-query attention kernels over one whole decode: each launch
        streams its key (or value) cache once, f32, plus the query/probability and result rows."""
        D, L, S = self.cfg["D"], self.cfg["layers"], self.S
        steps = len(self.prefix) + self.n_tok - 1
        cross = steps * L * S * self.Tenc * D * 4
        selfb = sum(L * S * (n + 1) * D * 4 for n in range(steps))
        return cross + selfb  # per kernel (qk reads K, pv reads V)

    def roofline(self, prof, peaks):
        ent = {e["label"]: e for e in prof}
        if "bmm_qk_t1" not in ent or "bmm_pv_t1" not in ent:
            return None
        ms = ent["bmm_qk_t1"]["ms"] + ent["bmm_pv_t1"]["ms"]
        launches = ent["bmm_qk_t1"]["count"] + ent["bmm_pv_t1"]["count"]
        ach = 2 * self.attn_bytes_per_step() / (ms * 1e-3) / 1e9  # per step; the caller scales by `steps`
        return {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None,
                "traffic": float(self.S * self.Tenc * self.cfg["D"] * 4),
                "traffic_note": "per cross-attention launch = its algorithmic bytes: an ncu capture of these launches shows "
                "1-2 % L2 hits, i.e. the cache is streamed from DRAM once",
                "kernel": "k_bmm_qk_t1 + k_bmm_pv_t1 (single-query attention over the f32 K/V caches)",
                "launches": launches, "avg_launch_us": round(ms / launches * 1e3, 2),
                "share_of_step": None, "peak_source": peaks["source"]}

    def cpu_sample(self, threads=True):
        """One stream, 128 tokens through the reference-form one-token step on the CPU port, full widths;
        the cross K/V of the clip are random stand-ins (their one-off products are left out of the sample)."""
        from oracle.wasm_oracle import WasmOracle
        from fluidaudio_web_b200.engines import synth, whisper_decoder

        if not hasattr(Decoder, "_cpu_dec") or Decoder._cpu_dec[0] != (self.quant, threads):
            ora = WasmOracle(threads=threads)
            cfg = dict(synth.WHISPER_TURBO_DEC)
            dec = whisper_decoder.load_decoder(ora, synth.decoder_weights(cfg, seed=5), cfg["NH"], quant=self.quant)
            rng = np.random.default_rng(9)
            kv = [dict(k=ora.upload(rng.standard_normal((1500, 1280), dtype=np.float32), 1500, 1280),
                       v=ora.upload(rng.standard_normal((1500, 1280), dtype=np.float32), 1500, 1280)) for _ in range(cfg["layers"])]
            Decoder._cpu_dec = ((self.quant, threads), ora, dec, kv)
        _, ora, dec, kv = Decoder._cpu_dec
        n = 128
        st = whisper_decoder.decode_init(ora, dec, n)
        tok = 1
        t0 = time.perf_counter()
        for _ in range(n):
            tok = int(np.argmax(whisper_decoder.decode_next(ora, dec, kv, st, tok)))
        dt = time.perf_counter() - t0
        return n / dt, f"1 stream x {n} tokens, one-token reference-form step, Tenc 1500 ({dt:.2f} s)"


class DecoderInt8(Decoder):
    quant = "int8"


class TdtDecode:
    """The stage after the encoder: greedy TDT decoding (prediction network + joint, int8 out-matrix) of the 32
    windows of one encoder batch, 188 pre-projected frames each, random-init weights with a bias on the blank logit so
    that most frames emit nothing (as with a trained model), frames ~ N(0,1).  One step = the whole decode of the
    batch, token ids and emission frames landed on the host.  Seed 5."""

    name = "parakeet_tdt_decode_32_windows_188_frames"
    metric = "tdt_decode_audio_seconds_per_second"
    unit = "audio-s/s"
    dtype = "int8 out-matrix x 3 int8 activation digits (joint), f32 multiply-adds (LSTM layers, projection)"
    nsets = 1
    graph = False  # the decode reads a device counter back every few rounds: eager steps

    def __init__(self, quick=False):
        self.W = 8 if quick else 32
        self.T = 188

    def setup(self, ctx):
        import __graft_entry__ as ge

        ge.load_package()
        from fluidaudio_web_b200.engines import tdt_decoder

        self.td = tdt_decoder
        self.weights = tdt_decoder.synth_tdt_weights(5)
        self.dec = tdt_decoder.TdtDecoder(ctx, self.weights, int8=True)
        self.host_proj = ctx.pinnedArray(self.W * self.T * 640)
        self.host_proj[:] = np.random.default_rng(6).standard_normal(self.W * self.T * 640).astype(np.float32)
        self.proj = ctx.upload(self.host_proj, self.W * self.T, 640)
        self.units_per_step = self.W
        self.tokens = 0

    def step_device(self, ctx):
        out = self.dec.decode_proj(self.proj, self.W, self.T)
        self.tokens = sum(len(i) for i, _ in out)

    def step_e2e(self, ctx):
        p = ctx.upload(self.host_proj, self.W * self.T, 640)
        out = self.dec.decode_proj(p, self.W, self.T)
        ctx.freeTensor(p)
        return out

    def e2e_bytes(self):
        return self.W * self.T * 640 * 4, 2 * 4 * max(1, self.tokens) + 4 * self.W

    def value_from(self, steps, seconds):
        return self.W * 15.0 * steps / seconds

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"] == "tc_gemm_i8"]
        if not ent:
            return None
        e = ent[0]
        per_launch = e["ms"] / e["count"]
        alg = 640 * 8198 + self.W * 640 * 4 + self.W * 8198 * 4 + 8198 * 4  # int8 out-matrix + J + logits + bias
        ach = alg / (per_launch * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4),
                "traffic": None, "kernel": "k_tc_gemm<i8> (the joint's 640 -> 8198 product, one per lock-step round)",
                "launches": e["count"], "avg_launch_us": round(per_launch * 1e3, 2), "rounds": self.dec.rounds,
                "note": "per-launch event pairs in an eager decode; the 5.2 MB out-matrix stays in L2 between rounds, so the "
                        "HBM figure says how far a round is from streaming its operands once; rounds are bound by launch and ramp",
                "peak_source": peaks["source"]}

    def cpu_sample(self, threads=True):
        from oracle.tdt_oracle import TdtOracle, synth_tdt_weights

        n = 8 if threads else 2
        ora = TdtOracle(getattr(self, "weights", None) or synth_tdt_weights(5), int8=True, threads=(os.cpu_count() or 1) if threads else 1)
        proj = np.random.default_rng(6).standard_normal((n, self.T, 640)).astype(np.float32)
        t0 = time.perf_counter()
        ora.decode_proj_batch(proj, n, self.T)
        dt = time.perf_counter() - t0
        return n * 15.0 / dt, f"{n} windows x {self.T} frames on the C restatement of rust/parakeet-decoder ({dt:.2f} s)"


class AsrPipeline(Encoder):
    """The reference's transcription pipeline for one batch of windows (src/engines/asr-parakeet/pipeline.js:32-61):
    16 kHz samples -> log-mel front end -> FastConformer encoder -> the joint's encoder projection riding the same
    submission (1024 -> 640) -> greedy TDT decoding of the 32 windows in lock step -> token ids and emission frames on
    the host.  Everything between the upload of the samples and the read-back of the ids stays on the device.  Batches
    alternate between two slots (contexts) of the GPU, the decode of one batch running under the encoder forward of the
    next, as the reference overlaps its decode workers with the next group's encode (pipeline.js `pipelined`); a step
    enqueues one batch and lands the token ids of the batch before it.  Weights
    random-init (encoder seed 3, decoder seed 5 with a bias on the blank logit so that most frames emit nothing)."""

    name = "parakeet_asr_pipeline_pcm_to_token_ids_batch32"
    metric = "asr_pipeline_audio_seconds_per_second"
    graph = False  # the decode reads a device counter back every few rounds: eager steps

    def setup(self, ctx):
        super().setup(ctx)
        from fluidaudio_web_b200.engines import tdt_decoder

        import __graft_entry__ as ge
        from fluidaudio_web_b200.engines import asr_pipeline

        self.tdt_weights = tdt_decoder.synth_tdt_weights(5)
        self.dec = tdt_decoder.TdtDecoder(ctx, self.tdt_weights, int8=True)
        self.dtype = "encoder: f16 x f16 -> f32; joint: int8 out-matrix x 3 int8 activation digits; prediction network f32"
        self.tokens = 0
        # one batch, stage after stage on one stream: the kernels a step launches
        l0 = ctx.launchCount()
        h = ctx.pushArena()
        x, tsub = self.fc.encode_batch(ctx, self.enc, self.dev_mels)
        self._count(self.dec.decode_proj(self.dec.project(x), self.W, tsub))
        ctx.popArena(h)
        self.launches_per_step = ctx.launchCount() - l0
        # the pipelined form the steps run: two slots (contexts), the decode of one batch under the forward of the next
        ctx2 = ge.load_package().CudaContext(ctx.device)
        enc2 = self._load(ctx2)
        dec2 = tdt_decoder.TdtDecoder(ctx2, self.tdt_weights, int8=True)
        pcm2 = ctx2.upload(self._audio, self.W, self.n_samples)
        mels2 = ctx2.logMelWindows(pcm2, 128)
        ctx2.freeTensor(pcm2)
        slots = [self._pcm_slot(ctx), self._pcm_slot(ctx2)]
        args = ([ctx, ctx2], [self.enc, enc2], [self.dec, dec2])
        self.pipe_dev = asr_pipeline.PipelinedAsr(*args, None, self.mel_len, self.W, from_pcm=False, resident=[self.dev_mels, mels2])
        self.pipe_e2e = asr_pipeline.PipelinedAsr(*args, lambda s: slots[s], self.n_samples, self.W, from_pcm=True)

    def _count(self, out):
        if out is not None:
            self.tokens = sum(len(i) for i, _ in out)

    def step_device(self, ctx):
        self._count(self.pipe_dev.submit())  # windows' features resident in HBM; token ids of the batch before land on the host

    def device_drain(self):
        for out in self.pipe_dev.flush():
            self._count(out)

    def step_e2e(self, ctx):
        out = self.pipe_e2e.submit()
        self._count(out)
        return out

    def e2e_drain(self):
        return self.pipe_e2e.flush()

    def e2e_bytes(self):
        return self.W * self.n_samples * 4, 2 * 4 * max(1, self.tokens) + 4 * self.W

    def cpu_sample(self, threads=True):
        from oracle.tdt_oracle import TdtOracle, synth_tdt_weights

        v_enc, d_enc = super().cpu_sample(threads=threads)
        n = 8 if threads else 2
        ora = TdtOracle(getattr(self, "tdt_weights", None) or synth_tdt_weights(5), int8=True,
                        threads=(os.cpu_count() or 1) if threads else 1)
        proj = np.random.default_rng(6).standard_normal((n, 188, 640)).astype(np.float32)
        t0 = time.perf_counter()
        ora.decode_proj_batch(proj, n, 188)
        v_dec = n * 15.0 / (time.perf_counter() - t0)
        return 1.0 / (1.0 / v_enc + 1.0 / v_dec), f"encoder: {d_enc}; decoder: {n} windows x 188 frames on the C restatement of rust/parakeet-decoder"


class F16GemmNSharded:
    """Benchmark configuration 3, its multi-GPU leg: the M = 16384 row of the f16 GEMM sweep with the output columns
    sharded over the ranks (each GPU holds N/world columns of every weight matrix) and an NCCL all-gather of
    the column blocks, so every rank ends with the whole row-major [M, N] product.  Total work is fixed as
    the number of GPUs grows ("strong" scaling); value = whole-product FLOPs / max-over-ranks time.  Seed 2."""

    name = "f16_gemm_m16384_n_sharded_allgather"
    metric = "f16_gemm_throughput"
    unit = "TFLOP/s"
    dtype = "f16 x f16 -> f32 accumulate, f32 out"
    nsets = 1
    scaling = "strong"
    graph = False  # the collective is enqueued by torch.distributed between the products: eager steps

    def __init__(self, quick=False):
        self.M = 4096 if quick else 16384
        self.KNs = ((1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024))

    def setup(self, ctx):
        import __graft_entry__ as ge

        ge.load_package()
        from fluidaudio_web_b200 import sharding

        self.sh = sharding
        rank, _lr, world = dist_env()
        self.world = world
        rng = np.random.default_rng(2)
        self.W = {}
        for kn in self.KNs:
            w = (rng.standard_normal(kn) / np.sqrt(kn[0])).astype(np.float32)
            ws = sharding.column_shard(w, world, rank)
            self.W[kn] = ctx.uploadF16(ws, ws.shape[0], ws.shape[1])
        self.host_A, self.A = {}, {}
        for K in sorted({k for k, _ in self.KNs}):
            buf = ctx.pinnedArray(self.M * K)
            buf[:] = rng.standard_normal(self.M * K).astype(np.float32)
            self.host_A[K] = buf
            self.A[K] = ctx.upload(buf, self.M, K)
        self.units_per_step = len(self.KNs)
        self.flops_per_step = sum(2.0 * self.M * K * N for K, N in self.KNs)
        # FA_NSHARD_FUSED=0 selects the NCCL all-gather + unshard form instead of the fused peer-store epilogue
        self.fused = os.environ.get("FA_NSHARD_FUSED", "1") != "0"
        self.res = {}
        if world > 1 and self.fused:
            self.res = {kn: sharding.ScatterResult(ctx, self.M, kn[1]) for kn in self.KNs}
            self.name = "f16_gemm_m16384_n_sharded_fused_peer_store_allgather"

    def step_device(self, ctx):
        if self.world > 1 and self.fused:
            # the all-gather rides the epilogue: peer stores into every rank's result, then one barrier
            for kn in self.KNs:
                self.sh.matmul_n_sharded_scatter(ctx, self.A[kn[0]], self.W[kn], self.res[kn])
            self.sh.stream_barrier(ctx)
            return
        h = ctx.pushArena()
        self.sh.matmul_n_sharded_many(ctx, [(self.A[kn[0]], self.W[kn]) for kn in self.KNs])
        ctx.popArena(h)

    def step_e2e(self, ctx):
        h = ctx.pushArena()
        outs = self.sh.matmul_n_sharded_many(ctx, [(ctx.upload(self.host_A[kn[0]], self.M, kn[0]), self.W[kn]) for kn in self.KNs])
        out = [ctx.download(o) for o in outs][-1]
        ctx.popArena(h)
        return out

    def nvlink_bytes_per_step(self):
        """Bytes every rank must receive over NVLink per step: (world-1)/world of each f32 product."""
        return sum(4 * self.M * N for _, N in self.KNs) * (self.world - 1) // self.world

    def e2e_bytes(self):
        return sum(4 * self.M * K for K, _ in self.KNs), sum(4 * self.M * N for _, N in self.KNs)

    def value_from(self, steps, seconds):
        return self.flops_per_step * steps / seconds / 1e12

    def roofline(self, prof, peaks):
        ent = [e for e in prof if e["label"].startswith("tc_gemm_f16")]
        if not ent:
            return None
        ms = sum(e["ms"] for e in ent)
        n = sum(e["count"] for e in ent)
        return {"bound": "tensor", "achieved": self.flops_per_step / self.world / (ms * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": None, "traffic": None, "kernel": "k_tc_gemm<f16> (this rank's column block)",
                "launches": n, "avg_launch_us": round(ms / n * 1e3, 2), "peak_source": peaks["source"] + " (burst bf16)",
                "nvlink_bytes_per_step_per_rank": self.nvlink_bytes_per_step(),
                "note": "with world > 1 the step is bound by the all-gather: f32 outputs leave a GPU faster than NVLink takes them "
                        "(K=1024 products make 1 output byte per 512 FLOP); step floor = nvlink bytes / 770 GB/s measured peer copy"}

    cpu_sample = F16Gemm.cpu_sample


def config4_sharded(ctx, wl, world, rank, local_rank):
    """The encoder configuration as BASELINE states it: 256 independent 15 s windows, batches of 32, sharded over the
    ranks in contiguous blocks (sharding.shard_range), frames gathered to rank 0 in window order and landed on the
    host.  The clock (wall, max over ranks) covers upload of this rank's PCM, log-mel, the encoder batches, the
    gather (NCCL, device to device) and rank 0's copy to host memory.  Rank 0 then re-encodes the last batch of the
    last rank's shard itself and requires the gathered frames to be identical."""
    import torch
    from fluidaudio_web_b200 import sharding
    from fluidaudio_web_b200.engines import synth

    n_win, B, D, T = 256, wl.W, 1024, 188
    lo, hi = sharding.shard_range(n_win, world, rank)
    base = wl._audio  # the batch's 32 distinct windows; window i of the job = base[i % 32] scaled by a per-window gain
    gain = (0.5 + 0.5 * np.random.default_rng(11).random(n_win)).astype(np.float32)
    mine = np.stack([base[i % B] * gain[i] for i in range(lo, hi)]) if hi > lo else np.zeros((0, wl.n_samples), np.float32)
    host = ctx.pinnedArray(max(1, mine.size))
    host[:mine.size] = mine.reshape(-1)
    out_host = ctx.pinnedArray(n_win * T * D) if rank == 0 else None
    stream = torch.cuda.ExternalStream(ctx.stream(), device=local_rank)

    def run():
        frames = []
        for i in range(0, hi - lo, B):
            nb = min(B, hi - lo - i)
            pcm = ctx.upload(host[i * wl.n_samples:(i + nb) * wl.n_samples], nb, wl.n_samples)
            x, _ = wl.fc.encode_batch(ctx, wl.enc, ctx.logMelWindows(pcm, 128))
            frames.append(x)
        local = ctx.concatRows(frames) if len(frames) > 1 else frames[0]
        if world == 1:
            ctx.downloadAsync(local, out_host)
            ctx.sync()
            return
        lt = sharding.as_torch(ctx, local)
        with torch.cuda.stream(stream):
            if rank == 0:
                parts = [torch.empty_like(lt) for _ in range(world)]
                torch.distributed.gather(lt, parts, dst=0)
                full = torch.cat(parts, 0)
                torch.from_numpy(out_host).view(n_win * T, D).copy_(full, non_blocking=True)
            else:
                torch.distributed.gather(lt, None, dst=0)
        ctx.sync()
        torch.cuda.synchronize()

    if n_win % (world * B):
        return {"skipped": f"256 windows do not split into batches of {B} over {world} ranks"}
    h = ctx.pushArena()
    run()  # warm-up (pool growth, NCCL set-up)
    ctx.popArena(h)
    if world > 1:
        torch.distributed.barrier()
    h = ctx.pushArena()
    t0 = time.perf_counter()
    run()
    dt = time.perf_counter() - t0
    ctx.popArena(h)
    if world > 1:
        t = torch.tensor([dt], device=f"cuda:{local_rank}")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dt = float(t.item())
    checked = None
    if rank == 0:
        h = ctx.pushArena()
        last = np.stack([base[i % B] * gain[i] for i in range(n_win - B, n_win)])
        x, _ = wl.fc.encode_batch(ctx, wl.enc, ctx.logMelWindows(ctx.upload(last, B, wl.n_samples), 128))
        want = ctx.download(x)
        ctx.popArena(h)
        checked = bool(np.array_equal(want.reshape(-1), out_host[(n_win - B) * T * D:]))
    return {"windows": n_win, "batch": B, "ms": round(dt * 1e3, 2), "audio_s_per_s": round(n_win * wl.window_s / dt, 1),
            "timing": "wall clock around upload of PCM, log-mel, encoder batches, gather to rank 0 and copy to host; max over ranks",
            "gathered_frames_identical_to_rank0_recompute": checked}


WORKLOADS = {"int4_decode": Int4Decode, "int8_gemm": Int8Gemm, "f16_gemm": F16Gemm, "encoder": Encoder,
             "decoder": Decoder, "decoder_int8": DecoderInt8, "f16_gemm_nsharded": F16GemmNSharded, "tdt_decode": TdtDecode, "asr_pipeline": AsrPipeline}
DEFAULT_WORKLOAD = "encoder"


# --------------------------------------------------------------------------------------------
# per-shape roofline records of the named GEMM / GEMV shapes
# --------------------------------------------------------------------------------------------

def shapes_report(ctx, peaks, timer, quick=False):
    """Every named product shape of the int8, int4 and f16 benchmark configurations, timed on its own:
    the product over a rotating set of weight matrices larger than L2 is recorded once (one CUDA graph) and
    replayed between CUDA events on the context's stream; `us` is the time per product.  `frac` = time floor
    / measured time, the floor being the larger of (algorithmic bytes / measured HBM copy bandwidth) and
    (operations / tensor peak), `bound` names which of the two it is.  Algorithmic bytes are those of the
    reference's own storage formats (f32 activations and results, int8 / int4+f32 scales / f16 weights).
    The int8 tensor peak is taken as 2x the measured bf16 figure (not measured on its own)."""
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = []
    l2x2 = 2 * L2_BYTES

    def time_products(make_body, n_products, reps):
        body = make_body
        body()
        ctx.sync()
        batch, _ = ctx.recordBatch(body)
        for _ in range(2):
            batch.launch()
        ms = timer(lambda _c: batch.launch(), reps)
        batch.free()
        return ms * 1e3 / (n_products * reps)

    def record(cfg, shape, kernel, us, bytes_, ops, ops_peak, extra=None):
        t_mem, t_ops = bytes_ / hbm, ops / ops_peak
        floor = max(t_mem, t_ops)
        r = {"config": cfg, "shape": shape, "kernel": kernel, "us": round(us, 2),
             "bound": "hbm" if t_mem >= t_ops else "tensor",
             "achieved": round((bytes_ / (us * 1e-6) / 1e9) if t_mem >= t_ops else (ops / (us * 1e-6) / 1e12), 1),
             "peak": round(peaks["hbm_gbs"] if t_mem >= t_ops else ops_peak / 1e12, 1),
             "unit": "GB/s" if t_mem >= t_ops else "TFLOP/s", "frac": round(floor / (us * 1e-6), 4),
             "algorithmic_bytes": int(bytes_), "ops": int(ops)}
        if extra:
            r.update(extra)
        out.append(r)

    # ---- int8 GEMM 512 x 1024 x 4096 (seed 0) -------------------------------------------------------
    rng = np.random.default_rng(0)
    M, K, N = 512, 1024, 4096
    nsets = 8 if quick else max(2, -(-l2x2 // (K * N)))
    a = ctx.upload(rng.standard_normal((M, K)).astype(np.float32), M, K)
    sc = ctx.upload(rng.uniform(1e-3, 1e-2, N).astype(np.float32), 1, N)
    ws = [ctx.uploadBytes(rng.integers(-127, 128, (K, N), dtype=np.int8)) for _ in range(nsets)]

    def body_i8():
        h = ctx.pushArena()
        for w in ws:
            ctx.matmulInt8(a, w, sc, N, K)
        ctx.popArena(h)

    us = time_products(body_i8, nsets, 10)
    ops = 2.0 * M * N * K
    record("int8_gemm", f"M={M} K={K} N={N}", "k_tc_gemm<i8> (+ activation digit prepass)", us,
           M * K * 4 + K * N + N * 4 + M * N * 4, ops, 2 * tf,
           {"tensor_tops": round(ops / (us * 1e-6) / 1e12, 1), "frac_of_int8_tensor_peak_2x_bf16": round(ops / (us * 1e-6) / (2 * tf), 4),
            "weight_sets": nsets})
    for w in ws:
        ctx.freeBytes(w)
    ctx.freeTensor(a)
    ctx.freeTensor(sc)

    # ---- int4 decode products K = 2048, N in {2048, 8192}, M in {1, 4, 16} (seed 1) -----------------------
    rng = np.random.default_rng(1)
    K = 2048
    nblk = K // 32
    for N in (2048, 8192):
        wbytes = N * K // 2 + N * nblk * 4 + N * (nblk // 2)
        nsets = 8 if quick else max(2, -(-l2x2 // wbytes))
        sets = []
        for _ in range(nsets):
            bq = rng.integers(0, 256, N * nblk * 16, dtype=np.uint8)
            scl = rng.uniform(5e-3, 2e-2, N * nblk).astype(np.float16).astype(np.float32)
            zp = np.full(N * (nblk // 2), 0x88, np.uint8)
            sets.append((ctx.uploadBytes(bq), ctx.upload(scl, 1, scl.size), ctx.uploadBytes(zp)))
        for M in (1, 4, 16):
            act = ctx.upload(rng.standard_normal((M, K)).astype(np.float16).astype(np.float32), M, K)

            def body_i4(act=act):
                h = ctx.pushArena()
                for bq, scl, zp in sets:
                    ctx.matmulNBits(act, bq, scl, zp, N)
                ctx.popArena(h)

            us = time_products(body_i4, nsets, 10)
            kern = ("k_gemv_nbits (dp4a on the raw nibbles)" if M <= 4 else
                    "k_nbits_mma (4-bit weights streamed once, mma.sync)" if N // 8 <= 5 * 148 else
                    "k_tc_gemm<f16> on the dequantised copy of the weights")
            record("int4_decode", f"M={M} K={K} N={N}", kern, us,
                   wbytes + 4 * M * K + 4 * M * N, 2.0 * M * N * K, tf, {"weight_sets": nsets})
            ctx.freeTensor(act)
        for bq, scl, zp in sets:
            ctx.freeBytes(bq)
            ctx.freeTensor(scl)
            ctx.freeBytes(zp)

    # ---- f16-weight GEMM sweep over the encoder's shapes (seed 2) ------------------------------------
    rng = np.random.default_rng(2)
    KNs = ((1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024))
    Ms = (4096,) if quick else (256, 1024, 4096, 16384)
    for K, N in KNs:
        w_host = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
        for M in Ms:
            abytes, cbytes = M * K * 4, M * N * 4
            # small products live in L2 unless the weights rotate; large ones stream activations and results anyway
            nsets = 1 if (abytes + cbytes > l2x2 or quick) else max(2, min(64, -(-l2x2 // (K * N * 2))))
            ws = [ctx.uploadF16(w_host, K, N) for _ in range(nsets)]
            act = ctx.upload(rng.standard_normal((M, K)).astype(np.float32), M, K)

            def body_f16(act=act, ws=ws):
                h = ctx.pushArena()
                for w in ws:
                    ctx.matmul(act, w)
                ctx.popArena(h)

            us = time_products(body_f16, nsets, 10 if M <= 4096 else 4)
            record("f16_gemm", f"M={M} K={K} N={N}", "k_tc_gemm<f16>", us, abytes + K * N * 2 + cbytes, 2.0 * M * N * K, tf,
                   {"weight_sets": nsets})
            ctx.freeTensor(act)
            for w in ws:
                ctx.freeTensor(w)

    # ---- layernorm on the encoder's residual stream (32 windows x 188 frames x 1024, seed 3) ------------------------
    # HBM-bound glue between the products: f32 rows in, the packed f16 operand of the next product out (and the f32
    # rows as well for the block-final form).  Inputs rotate through more than L2, which is the harsher case: inside
    # the encoder step the input was written by the kernel before and is still in L2.
    if not quick:
        rng = np.random.default_rng(3)
        M, D = 32 * 188, 1024
        nx = max(2, -(-l2x2 // (M * D * 4)))
        xs = [ctx.upload(rng.standard_normal((M, D)).astype(np.float32), M, D) for _ in range(nx)]
        g = ctx.upload(rng.standard_normal(D).astype(np.float32), 1, D)
        b = ctx.upload(rng.standard_normal(D).astype(np.float32), 1, D)
        for label, fn, nbytes in (("layernorm (f32 rows + packed f16 operand out)", ctx.layernorm, M * D * (4 + 4 + 2)),
                                  ("layernormOperand (packed f16 operand out only)", ctx.layernormOperand, M * D * (4 + 2))):
            def body_ln(fn=fn):
                h = ctx.pushArena()
                for x in xs:
                    fn(x, g, b, 1e-5)
                ctx.popArena(h)

            us = time_products(body_ln, nx, 10)
            record("encoder_glue", f"rows={M} cols={D}", "k_layernorm_warp: " + label, us, nbytes, 8.0 * M * D, tf, {"input_sets": nx})
        for x in xs:
            ctx.freeTensor(x)
        ctx.freeTensor(g)
        ctx.freeTensor(b)
    return out


# --------------------------------------------------------------------------------------------
# arms
# --------------------------------------------------------------------------------------------

def run_reference(args):
    rank, _lr, world = dist_env()
    if rank != 0:
        return
    from oracle.wasm_oracle import LIB
    import __graft_entry__ as ge

    ge.load_package()  # the engines' host logic (backend-agnostic) drives the CPU port for the model workloads
    wl = WORKLOADS[args.workload](quick=True)
    # all host threads, also under torchrun (which exports OMP_NUM_THREADS=1 to its workers)
    LIB.oracle_set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = LIB.oracle_num_threads()
    vals, desc = [], ""
    for _ in range(args.warmup):
        wl.cpu_sample(threads=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, desc = wl.cpu_sample(threads=True)
        vals.append(v)
    dt = time.perf_counter() - t0
    value = float(np.mean(vals))
    line = {"impl": "reference", "metric": wl.metric, "value": round(value, 6), "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
            "ms_per_step_is": "wall time of one bounded CPU sample (see cpu_baseline.sample), not of a full step of the workload",
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (CPU port of the wasm kernels)",
            "data": "synthetic", "config": {"workload": wl.name, "note": "Node/wasm runtime absent on the box: C port of rust/wasm-kernels timed instead"},
            "cpu_baseline": {"value": round(value, 6), "unit": wl.unit, "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": round(value, 6), "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_cuda(args):
    import torch
    import __graft_entry__ as ge

    rank, local_rank, world = dist_env()
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = ge.load_package()
    ctx = pkg.CudaContext(local_rank)
    torch.cuda.set_device(local_rank)
    stream = torch.cuda.ExternalStream(ctx.stream(), device=local_rank)
    wl = WORKLOADS[args.workload](quick=args.quick)
    if isinstance(wl, Encoder):
        wl.weights_mode = args.encoder_weights
    wl.setup(ctx)
    ctx.sync()

    def barrier():
        ctx.sync()
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()

    def timed(step_fn, steps, drain=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(steps):
                step_fn(ctx)
            if drain is not None:
                drain()  # a pipelined workload still owes its last batch (a host call that returns when it is done)
            e1.record(stream)
        ctx.sync()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=f"cuda:{local_rank}")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        return ms

    for _ in range(max(args.warmup, 3)):
        wl.step_device(ctx)
    ctx.sync()
    # the step is recorded once (one CUDA graph = the reference's one-submit batch) and replayed
    l0 = ctx.launchCount()
    use_graph = getattr(wl, "graph", True)
    if use_graph:
        batch, _ = ctx.recordBatch(lambda: wl.step_device(ctx))
    else:
        wl.step_device(ctx)
        batch = None
    launches_per_step = getattr(wl, "launches_per_step", ctx.launchCount() - l0)
    for _ in range(3):
        batch.launch() if use_graph else wl.step_device(ctx)
    drain = getattr(wl, "device_drain", None)
    if drain is not None:
        drain()
    ctx.sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed((lambda _ctx: batch.launch()) if use_graph else wl.step_device, args.steps, drain)
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    if use_graph:
        batch.free()
    scaling = getattr(wl, "scaling", "weak")
    units = world if scaling == "weak" else 1  # weak: every rank ran a whole step; strong: the ranks shared one
    value = wl.value_from(args.steps, ms * 1e-3) * units

    # per-launch durations of the dominant kernel: same steps again with an event pair around each launch
    psteps = min(args.steps, getattr(wl, "profile_steps", args.steps))
    ctx.startProfile(200000)
    for _ in range(psteps):
        wl.step_device(ctx)
    if drain is not None:
        drain()
    prof = ctx.endProfile()
    peaks = measured_peaks()
    roof = wl.roofline(prof, peaks)
    if hasattr(wl, "roofline_live"):
        in_step = roof
        roof = wl.roofline_live(ctx, peaks, timed)
        if in_step is not None:
            roof["in_step_profile"] = {"launches": in_step.get("launches"), "avg_launch_us": in_step.get("avg_launch_us"),
                                       "note": "per-launch event pairs inside the eager forward; includes launch gaps"}
    elif roof is not None and roof.get("frac") is None:  # per-step figure over a profile of `steps` steps
        roof["achieved"] = round(roof["achieved"] * psteps, 1)
        roof["frac"] = round(roof["achieved"] / roof["peak"], 4)

    # end to end through the public API with host buffers
    for _ in range(2):
        wl.step_e2e(ctx)
    if hasattr(wl, "e2e_drain"):
        wl.e2e_drain()  # nothing of the warm-up steps is still in flight when the clock starts
    ctx.sync()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.step_e2e(ctx)
    if hasattr(wl, "e2e_drain"):
        wl.e2e_drain()  # a pipelined workload still owes the read-back of its last batches
    ctx.sync()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=f"cuda:{local_rank}")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = wl.value_from(args.steps, e2e_s) * units
    h2d, d2h = wl.e2e_bytes()

    cfg4 = None
    if type(wl) is Encoder and not args.quick:
        cfg4 = config4_sharded(ctx, wl, world, rank, local_rank)

    shapes = None
    if world == 1 and not args.no_shapes:
        shapes = shapes_report(ctx, peaks, timed, quick=args.quick)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle.wasm_oracle import LIB

        v, desc = wl.cpu_sample(threads=False)
        cpu = {"value": round(v, 6), "unit": wl.unit, "cores": 1, "kind": "port", "sample": desc,
               "host_threads_available": LIB.oracle_num_threads()}

    if rank == 0:
        line = {"metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
                "scaling": scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
                "config": {"workload": wl.name, "l2": f"rotating weight set of {wl.nsets} matrices (> 126 MB L2)",
                           "timing": ("CUDA events on the context stream around K replays of the recorded step (CUDA graph), max over ranks"
                                      if use_graph else "CUDA events on the context stream around K eager steps, max over ranks"),
                           "roofline_timing": "per-launch CUDA event pairs, repeat pass of the same steps"},
                "roofline": roof, "cpu_baseline": cpu,
                "e2e": {"value": round(e2e_val, 3), "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": int(launches), "clocks": clocks, "config4_256_windows_sharded": cfg4, "shapes": shapes,
                "kernels": [{"label": e["label"], "launches": e["count"], "ms": round(e["ms"], 3)} for e in prof]}
        print(json.dumps(line), flush=True)
    ctx.destroy()
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--quick", action="store_true", help="smaller rotating set (for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-shapes", action="store_true", help="skip the per-shape roofline records of the GEMM / GEMV shapes")
    ap.add_argument("--encoder-weights", default="f16", choices=["int8", "f16"],
                    help="encoder workload: dequantise the int8 artifact to f16 storage at load (default) or keep its matrices int8 in HBM")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
