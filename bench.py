"""Benchmark driver: python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the hot path over one
batch of seeded synthetic input.  `value` is device-timed with inputs resident
in HBM; `e2e` is the same metric through the C ABI with HOST buffers (pinned
host memory, host->device and device->host copies inside the timed region).
`roofline` describes the dominant kernel against the measured HBM peak;
`cpu_baseline` is the CPU oracle timed on a bounded sample on this box's cores.
`--impl reference` times the reference's CPU path (restated in oracle/: the
reference is Rust + Metal and cannot be built here) on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.proc, self.device = None, device

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.device), "-lms", "100"], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
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


# --------------------------------------------------------------------------- workloads
class QuantMatvec:
    """Configs 1 and 2 at batch 1: a fused-dequant matvec over `copies` distinct weight
    matrices whose total size exceeds L2 twice over, launched back to back from one CUDA graph
    (the reference's own microbenchmark cycles 35 distinct weight sets so each read is cold,
    local-metal/src/kernels.rs:8898-8902).  One step = one pass over all copies."""

    def __init__(self, la, ctx, kernels, fmt: str, rows: int, cols: int, m: int = 1, min_copies: int = 8,
                 grouped: bool = False, f32out: bool = False):
        """grouped: the copies go through lc_matvec_*_group_into, up to 96 matrices per launch (the decode-time
        access pattern: many same-shape matrices against one vector), instead of one launch per matrix.
        f32out (Q4_0 matmul only): the f32-output entry point, as the vocabulary projection of a decode step uses."""
        self.la, self.ctx, self.k, self.fmt, self.rows, self.cols, self.m = la, ctx, kernels, fmt, rows, cols, m
        self.grouped = grouped and m == 1
        self.f32out = f32out and fmt == "q4_0" and m > 1
        self.obytes = 4 if self.f32out else 2
        l2 = ctx.caps()["l2_bytes"]
        gen = la.synth.q4_0_weights if fmt == "q4_0" else la.synth.tq2_0_weights
        w0 = gen(rows, cols, seed=1)
        self.wbytes = w0.size
        self.copies = max(min_copies, int(np.ceil(2.2 * l2 / self.wbytes)))
        self.weights = []
        for c in range(self.copies):
            w = w0 if c == 0 else np.roll(w0, c * 4099 * (18 if fmt == "q4_0" else 66))  # distinct rows order, same blocks
            self.weights.append(la.CudaBuffer.from_slice(ctx, w))
        self.w0 = w0
        self.x_host = la.synth.normal_f16((m, cols), seed=2)
        self.x = la.CudaBuffer.from_slice(ctx, self.x_host)
        self.out = [la.CudaBuffer.empty(ctx, m * rows * self.obytes) for _ in range(self.copies)]
        self.alg_bytes_per_launch = self.wbytes + m * cols * 2 + m * rows * self.obytes
        self.units_per_step = self.copies
        self.name = f"{fmt} fused dequant mat{'vec' if m == 1 else 'mul'} {rows}x{cols} batch {m}"
        if self.grouped:
            self.name += f", {min(96, self.copies)} matrices per launch"
        self.graph = None
        self.launches_per_step = self.copies if not self.grouped else -(-self.copies // 96)

    def _enqueue(self, b, c):
        if self.m == 1:
            fn = self.k.matvec_q4_0_into if self.fmt == "q4_0" else self.k.matvec_tq2_0_into
            fn(b, self.weights[c], self.x, self.out[c], self.rows, self.cols)
        else:
            if self.f32out:
                fn = self.k.matmul_nt_q4_0_f32out_into
            else:
                fn = self.k.matmul_nt_q4_0_into if self.fmt == "q4_0" else self.k.matmul_nt_tq2_0_into
            fn(b, self.x, self.weights[c], self.out[c], self.m, self.cols, self.rows)

    def _enqueue_all(self, b):
        if not self.grouped:
            for c in range(self.copies):
                self._enqueue(b, c)
            return
        fn = self.k.matvec_q4_0_group_into if self.fmt == "q4_0" else self.k.matvec_tq2_0_group_into
        for c0 in range(0, self.copies, 96):
            c1 = min(self.copies, c0 + 96)
            fn(b, self.weights[c0:c1], c1 - c0, self.x, self.out[c0:c1], self.rows, self.cols)

    def prepare(self):
        b = self.la.CommandBatch.new(self.ctx)
        self._enqueue_all(b)
        b.commit_and_wait()
        b = self.la.CommandBatch.capture(self.ctx)
        self._enqueue_all(b)
        self.graph = b.end_capture()

    def step(self):
        self.graph.launch()

    def check(self, orc):
        got = self.out[0].as_slice(np.float32 if self.f32out else np.float16).astype(np.float32).reshape(self.m, self.rows)
        f = orc.Q4_0 if self.fmt == "q4_0" else orc.TQ2_0
        mc = self.m if self.m * self.rows * self.cols <= 4e9 else 4    # bound the CPU time: the first batch rows only
        want = orc.matmul_nt(f, self.x_host[:mc], self.w0, mc, self.cols, self.rows)
        got = got[:mc]
        assert np.all(np.abs(got - want) <= 1e-3 * np.maximum(np.abs(want), 1.0)), "bench output differs from the oracle"

    # end to end through the C ABI with host buffers: upload x, run, download y, per copy
    def prepare_e2e(self):
        self.hx = self.la.PinnedHost(self.m * self.cols * 2)
        self.hy = self.la.PinnedHost(self.m * self.rows * self.obytes)
        self.hx.array[:] = self.x_host.view(np.uint8).reshape(-1)
        self.h2d, self.d2h = self.m * self.cols * 2 * self.copies, self.m * self.rows * self.obytes * self.copies

    def step_e2e(self):
        b = self.la.CommandBatch.new(self.ctx)
        for c in range(self.copies):
            b.upload(self.x, 0, self.hx.ptr, self.hx.nbytes)
            self._enqueue(b, c)
            b.download(self.out[c], 0, self.hy.ptr, self.hy.nbytes)
        b.commit_and_wait()

    def metric(self):
        return "fused_quant_matvec_hbm_gbs", "GB/s"

    def l2_note(self):
        return f"inputs larger than L2 ({self.copies} distinct weight copies, {self.copies * self.wbytes / 1e6:.0f} MB per pass)"

    def roofline(self, ms_per_step: float, peak: float, peak_kind: str, timed):
        launch_ms = ms_per_step / self.copies    # per matrix (a grouped launch covers several)
        achieved = self.alg_bytes_per_launch / (launch_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": peak_kind, "kernel": self.kernel_name(),
                "us_per_launch": launch_ms * 1e3, "algorithmic_bytes_per_launch": self.alg_bytes_per_launch,
                "frac_of_nominal_8tbs": achieved / 8000.0}

    def kernel_name(self) -> str:
        if self.grouped:
            return "qgemv_mma_stream_kernel (grouped)"
        if self.m == 1:
            return "qgemv_mma_stream_kernel" if self.rows >= 18944 else "qgemv_kernel"
        if self.f32out and 8 < self.m <= 64 and self.cols % 256 == 0 and self.rows >= 128 * 148:
            return "qgemm_tcv_kernel (tcgen05)"
        if self.fmt == "tq2_0" and 8 < self.m <= 64:
            return "qgemm_tcd_kernel (tcgen05)"
        return "qgemm_mma_kernel" if self.m <= 64 else "qgemm_tc_kernel (tcgen05)"

    def value(self, ms_per_step: float) -> float:
        return self.alg_bytes_per_launch * self.units_per_step / (ms_per_step * 1e-3) / 1e9

    def cpu_sample(self, orc, threads: int):
        """One matrix (all rows) on the CPU: returns (seconds, GB/s-equivalent, description)."""
        f = orc.Q4_0 if self.fmt == "q4_0" else orc.TQ2_0
        reps, t0 = 0, time.perf_counter()
        while True:
            orc.baseline_matmul_nt(f, self.x_host, self.w0, self.m, self.cols, self.rows, threads)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > 3.0 or reps >= 200:
                break
        return dt / reps, self.alg_bytes_per_launch / (dt / reps) / 1e9, f"{reps} passes over one {self.rows}x{self.cols} matrix"


class TqAttention:
    """Config 3: fused decode attention over tq2 codes (8 q heads, 1 kv head, head_dim 256, softmax scale 1/16) for
    `lanes` sequences at `context` cached positions each, every lane attending context + 1 keys.  A step is one
    pass over `pools` distinct KV pools (together larger than L2 twice over), one fused call each (query rotation,
    split-K attention over codes, merge, inverse rotation; f16 query in, f16 out), launched from one CUDA graph.
    Pools hold seeded random codes and norms ~ |N(0, I_256)|; the cost does not depend on the values."""

    def __init__(self, la, ctx, kernels, lanes: int, context: int):
        self.la, self.ctx, self.k, self.lanes, self.context = la, ctx, kernels, lanes, context
        self.hd, self.n_q, self.n_kv, self.bits = 256, 8, 1, 2
        cb = la.tq_code_bytes(self.hd, self.bits)
        self.cap = context + 1
        rows = lanes * self.cap
        self.alg_bytes_per_launch = rows * self.n_kv * (2 * cb + 4) + 2 * lanes * self.n_q * self.hd * 2
        l2 = ctx.caps()["l2_bytes"]
        self.pools_n = max(3, int(np.ceil(2.2 * l2 / self.alg_bytes_per_launch)))
        self.levels = la.CudaBuffer.from_slice(ctx, la.tq_levels(self.hd, self.bits))
        self.signs = la.CudaBuffer.from_slice(ctx, la.tq_signs(self.hd, la.TQ_SEED))
        self.q_host = la.synth.normal_f16((lanes, self.n_q, self.hd), 3)
        self.q = la.CudaBuffer.from_slice(ctx, self.q_host)
        self.out = la.CudaBuffer.empty(ctx, lanes * self.n_q * self.hd * 2)
        self.positions = la.CudaBuffer.from_slice(ctx, np.full(lanes, context, np.uint32))
        self.pools = []
        codes = la.synth.splitmix64(4242, rows * cb // 8).view(np.uint8)
        norms = (16.0 * la.synth.uniform(4243, rows, 0.9, 1.1)).astype(np.float16)
        for i in range(self.pools_n):
            # the same bytes at a different rotation per pool: distinct addresses, any code values
            kc = la.CudaBuffer.from_slice(ctx, np.roll(codes, 64 * (i + 1)))
            vc = la.CudaBuffer.from_slice(ctx, np.roll(codes, 64 * (i + 7)))
            kn = la.CudaBuffer.from_slice(ctx, np.roll(norms, i))
            vn = la.CudaBuffer.from_slice(ctx, np.roll(norms, i + 3))
            self.pools.append((kc, kn, vc, vn))
        self.name = f"fused tq2 decode attention, {lanes} lane(s) x {context + 1} keys, 8 q heads / 1 kv head of 256"
        self.units_per_step = self.pools_n
        self.graph, self.launches_per_step = None, None

    def _enqueue(self, b, i):
        kc, kn, vc, vn = self.pools[i]
        self.k.tq_attention_batched_into(b, self.q, kc, kn, vc, vn, self.levels, self.signs, self.out, self.positions,
                                         self.hd, self.cap, self.n_q, self.n_kv, 0, self.bits, self.lanes, 0, 1.0 / 16.0)

    def prepare(self):
        b = self.la.CommandBatch.new(self.ctx)
        for i in range(self.pools_n):
            self._enqueue(b, i)
        self.launches_per_step = b.dispatch_count()
        b.commit_and_wait()
        b = self.la.CommandBatch.capture(self.ctx)
        for i in range(self.pools_n):
            self._enqueue(b, i)
        self.graph = b.end_capture()

    def step(self):
        self.graph.launch()

    def check(self, orc):
        """Lane 0 of the last pool against the oracle's fused attention (2e-3 of max(|want|, 1): f16 output)."""
        kc, kn, vc, vn = self.pools[-1]
        cb = self.la.tq_code_bytes(self.hd, self.bits)
        n = self.cap
        want = orc.tq_attention_fused(self.q_host[:1], kc.as_slice(np.uint8, n * cb), kn.as_slice(np.float16, n),
                                      vc.as_slice(np.uint8, n * cb), vn.as_slice(np.float16, n),
                                      self.la.tq_levels(self.hd, self.bits), self.la.tq_signs(self.hd, self.la.TQ_SEED),
                                      np.array([self.context], np.uint32), self.hd, self.cap, self.n_q, self.n_kv, 0,
                                      self.bits, 1, 0, 1.0 / 16.0).astype(np.float32).reshape(-1)
        got = self.out.as_slice(np.float16, self.n_q * self.hd).astype(np.float32)
        assert np.all(np.abs(got - want) <= 2e-3 * np.maximum(np.abs(want), 1.0)), "attention differs from the oracle"

    def prepare_e2e(self):
        nb = self.lanes * self.n_q * self.hd * 2
        self.hq, self.ho = self.la.PinnedHost(nb), self.la.PinnedHost(nb)
        self.hq.array[:] = self.q_host.view(np.uint8).reshape(-1)
        self.h2d, self.d2h = nb * self.pools_n, nb * self.pools_n

    def step_e2e(self):
        b = self.la.CommandBatch.new(self.ctx)
        for i in range(self.pools_n):
            b.upload(self.q, 0, self.hq.ptr, self.hq.nbytes)
            self._enqueue(b, i)
            b.download(self.out, 0, self.ho.ptr, self.ho.nbytes)
        b.commit_and_wait()

    def metric(self):
        return "tq_decode_attention_hbm_gbs", "GB/s"

    def l2_note(self):
        return (f"inputs larger than L2 ({self.pools_n} distinct KV pools, "
                f"{self.pools_n * self.alg_bytes_per_launch / 1e6:.0f} MB per pass)")

    def value(self, ms_per_step: float) -> float:
        return self.alg_bytes_per_launch * self.units_per_step / (ms_per_step * 1e-3) / 1e9

    def roofline(self, ms_per_step: float, peak: float, peak_kind: str, timed):
        us = ms_per_step * 1e3 / self.pools_n
        achieved = self.alg_bytes_per_launch / (us * 1e-6) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": peak_kind,
                "kernel": "tq2_attn_mma_kernel (splits merged in the kernel through a thread-block cluster)", "us_per_launch": us,
                "algorithmic_bytes_per_launch": self.alg_bytes_per_launch, "frac_of_nominal_8tbs": achieved / 8000.0}

    def cpu_sample(self, orc, threads: int):
        kc, kn, vc, vn = self.pools[0]
        cb = self.la.tq_code_bytes(self.hd, self.bits)
        n = self.cap
        args = (self.q_host[:1], kc.as_slice(np.uint8, n * cb), kn.as_slice(np.float16, n), vc.as_slice(np.uint8, n * cb),
                vn.as_slice(np.float16, n), self.la.tq_levels(self.hd, self.bits),
                self.la.tq_signs(self.hd, self.la.TQ_SEED), np.array([self.context], np.uint32), self.hd, self.cap,
                self.n_q, self.n_kv, 0, self.bits, 1, 0, 1.0 / 16.0)
        reps, t0 = 0, time.perf_counter()
        while True:
            orc.tq_attention_fused(*args)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > 3.0 or reps >= 50:
                break
        per = dt / reps
        return per, n * (2 * cb + 4) / per / 1e9, f"{reps} passes over one lane of {n} keys (oracle, all host threads)"


class DecodeStep:
    """Config 4: one decode step of the synthetic Gemma-4-E2B-like dense decoder (35 layers, hidden 1536,
    8 q heads / 1 kv head of 256, GeGLU 6144, 4:1 SWA(512):full, TQ2_0 projections, Q4_0 tied 262144-row
    embedding / vocabulary projection, tq2 KV) at batch `lanes`, every sequence at context `context`.
    Random-init seeded weights; the KV pools are pre-filled with seeded random codes and norms ~ |N(0,I_256)|
    (attention cost does not depend on the values).  One step = one token for every lane, greedy argmax
    on the device, the whole step in one CUDA graph."""

    def __init__(self, la, ctx, kernels, lanes: int = 64, context: int = 8192, n_layers: int = 35,
                 vocab: int = 262144, share: "DecodeStep | None" = None):
        """`share`: another DecodeStep of the same architecture whose host-side weights are reused (the synthetic
        tensors depend on the layer shapes and the seed only)."""
        self.la, self.ctx, self.k, self.lanes, self.context = la, ctx, kernels, lanes, context
        self.cfg = la.e2b_like_config(max_lanes=lanes, max_context=context + 512, n_layers=n_layers, vocab=vocab)
        cfg = self.cfg
        self.model = la.DecodeModel(ctx, kernels, cfg)
        if share is not None:
            assert (share.cfg.n_layers, share.cfg.vocab) == (n_layers, vocab)
        self.host_layers = []
        for i in range(n_layers):
            t = share.host_layers[i] if share is not None else la.model.synth_layer(cfg, i, seed=4)
            self.model.set_layer(i, t)
            self.host_layers.append(t)
        self.emb, self.fnorm = (share.emb, share.fnorm) if share is not None else la.model.synth_embedding(cfg, seed=4)
        self.model.set_embedding(self.emb, self.fnorm)
        self.geo = []
        self.kv_bytes = 0
        cb = la.tq_code_bytes(cfg.head_dim, cfg.kv_bits)
        for i in range(n_layers):
            kv = self.model.kv_buffers(i)
            self.geo.append((kv["lane_rows"], kv["ring"], kv["window"]))
            rows = lanes * kv["lane_rows"] * cfg.n_kv_heads
            for j, name in enumerate(("k_codes", "v_codes")):
                kv[name].copy_from_bytes(la.synth.splitmix64(1000 + 2 * i + j, rows * cb // 8).view(np.uint8))
            for j, name in enumerate(("k_norms", "v_norms")):
                kv[name].copy_from_bytes((16.0 * la.synth.uniform(2000 + 2 * i + j, rows, 0.9, 1.1)).astype(np.float16))
            eff = min(context + 1, kv["window"]) if kv["window"] else context + 1
            self.kv_bytes += lanes * eff * cfg.n_kv_heads * (2 * cb + 4)
        tq = lambda r, c: r * (c // 256) * 66
        qd, kd = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        per_layer = (tq(qd, cfg.hidden) + 2 * tq(kd, cfg.hidden) + tq(cfg.hidden, qd) + 2 * tq(cfg.inter, cfg.hidden) +
                     tq(cfg.hidden, cfg.inter))
        self.weight_bytes = n_layers * per_layer + vocab * (cfg.hidden // 32) * 18
        self.alg_bytes_per_step = self.weight_bytes + self.kv_bytes
        self.tokens_host = (la.synth.splitmix64(7, lanes) % np.uint64(vocab)).astype(np.uint32)
        self.positions_host = np.full(lanes, context, np.uint32)
        self.tokens = la.CudaBuffer.from_slice(ctx, self.tokens_host)
        self.positions = la.CudaBuffer.from_slice(ctx, self.positions_host)
        self.next_tokens = la.CudaBuffer.empty(ctx, lanes * 4)
        self.name = (f"decode step, E2B-like dense decoder {n_layers} layers, batch {lanes}, context {context}, "
                     f"TQ2_0 weights + Q4_0 vocab {vocab}, tq{cfg.kv_bits} KV")
        self.copies, self.wbytes = 1, self.weight_bytes
        self.graph = None
        self.launches_per_step = None

    def prepare(self):
        b = self.la.CommandBatch.new(self.ctx)
        self.model.decode_batch_step_into(b, self.tokens, self.positions, self.lanes, False, self.next_tokens)
        self.launches_per_step = b.dispatch_count()
        b.commit_and_wait()
        b = self.la.CommandBatch.capture(self.ctx)
        self.model.decode_batch_step_into(b, self.tokens, self.positions, self.lanes, False, self.next_tokens)
        self.graph = b.end_capture()

    def step(self):
        self.graph.launch()

    def l2_note(self):
        return (f"inputs larger than L2: {self.weight_bytes / 1e6:.0f} MB of weights + {self.kv_bytes / 1e6:.0f} MB of KV "
                "read per step")

    def check(self, orc):
        """At full size: the first lanes' logits against the oracle's step on the same weights, tokens, positions
        and KV pools (the rule of the decode-step tests: 2e-3 of the logit scale when the rows written by the step
        come out byte-identical, the reference's 0.15 envelope otherwise, pipeline/batched.rs:471-477); tokens in
        range; the device argmax against its own logits."""
        la, cfg = self.la, self.cfg
        nl = min(2, self.lanes)
        self.tokens.copy_from_bytes(self.tokens_host.view(np.uint8))          # the end-to-end loop fed tokens back
        self.positions.copy_from_bytes(self.positions_host.view(np.uint8))
        om_cfg = la.e2b_like_config(max_lanes=nl, max_context=cfg.max_context, n_layers=cfg.n_layers, vocab=cfg.vocab)
        om = orc.OracleModel(om_cfg, self.host_layers, self.emb, self.fnorm, self.geo)
        cb = la.tq_code_bytes(cfg.head_dim, cfg.kv_bits)

        def lanes_of(i):   # the first nl lanes of layer i's device pools: (name, bytes)
            kv = self.model.kv_buffers(i)
            rows = nl * kv["lane_rows"] * cfg.n_kv_heads
            return [(n, kv[n].as_slice(np.uint8, rows * (cb if n.endswith("codes") else 2))) for n in
                    ("k_codes", "v_codes", "k_norms", "v_norms")]
        for i, pool in enumerate(om.pools):
            for name, dev in lanes_of(i):
                pool[name].view(np.uint8)[:] = dev
        want, _ = om.decode_batch_step(self.tokens_host[:nl], self.positions_host[:nl])
        b = la.CommandBatch.new(self.ctx)
        self.model.decode_batch_step_into(b, self.tokens, self.positions, self.lanes, True, self.next_tokens)
        b.commit_and_wait()
        nt = self.next_tokens.as_slice(np.uint32, self.lanes)
        assert np.all(nt < cfg.vocab), "argmax out of range"
        got = self.model.logits_buffer().as_slice(np.float32, nl * cfg.vocab).reshape(nl, -1)
        assert np.all(np.isfinite(got)), "non-finite logits"
        assert all(nt[i] == int(np.argmax(got[i])) for i in range(nl)), "argmax kernel disagrees with its logits"
        mism = sum(int(np.sum(dev != pool[name].view(np.uint8))) for i, pool in enumerate(om.pools)
                   for name, dev in lanes_of(i))
        scale = max(1.0, float(np.abs(want).max()))
        err = float(np.abs(got - want).max()) / scale
        tol = 2e-3 if mism == 0 else 0.15
        assert err <= tol, f"logits differ from the oracle by {err:.3e} of scale ({mism} differing KV bytes)"
        self.parity = {"lanes_checked": nl, "max_err_of_logit_scale": err, "kv_bytes_differing": mism, "tolerance": tol}

    def prepare_e2e(self):
        self.h_in = self.la.PinnedHost(2 * self.lanes * 4, dtype=np.uint32)
        self.h_out = self.la.PinnedHost(self.lanes * 4, dtype=np.uint32)
        self.h_in.array[: self.lanes] = self.tokens_host
        self.h_in.array[self.lanes:] = self.positions_host
        self.e2e_pos0 = self.positions_host.copy()
        self.e2e_steps = 0
        self.h2d, self.d2h = 2 * self.lanes * 4, self.lanes * 4

    def step_e2e(self):
        # host tokens + positions in, greedy tokens out, fed back as the next step's input.  The copies and the step's
        # graph go to the context's stream in order; the host waits once, for the tokens.
        b = self.la.CommandBatch.new(self.ctx)
        b.upload(self.tokens, 0, self.h_in.ptr, self.lanes * 4)
        b.upload(self.positions, 0, self.h_in.ptr + self.lanes * 4, self.lanes * 4)
        self.graph.launch()
        b.download(self.next_tokens, 0, self.h_out.ptr, self.lanes * 4)
        b.commit_and_wait()
        self.e2e_steps += 1
        self.h_in.array[: self.lanes] = self.h_out.array
        self.h_in.array[self.lanes:] = self.e2e_pos0 + (self.e2e_steps % 256)

    def metric(self):
        return f"decode_tok_s_batch{self.lanes}", "tok/s"

    def value(self, ms_per_step: float) -> float:
        return self.lanes / (ms_per_step * 1e-3)

    # dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel: mean over one GeGLU and one down
    # launch of an ncu capture (cold cache) of the 5-layer workload, whose launches have the full model's shapes.
    FFN_TRAFFIC = {"bytes": 4205056, "profile": "profiles/qgemm_tcd_tq2_0_m64.md",
                   "captured_on": "bench.py --workload decode_b64_small (same launch shapes as decode_b64)"}

    def roofline(self, ms_per_step: float, peak: float, peak_kind: str, timed):
        """The dominant kernel by time is the decode matmul (qgemm_tcd_kernel, TQ2_0, m = lanes): its two largest
        launch shapes, the fused GeGLU projection and the down projection of every layer, are run alone here (one
        graph, every layer's own weights, 2 x n_layers launches) and timed with CUDA events.  Algorithmic bytes per
        launch = rows * row_bytes + m * cols * 2 + m * rows * 2.  The whole-step figures are reported beside it."""
        la, ctx, cfg, m = self.la, self.ctx, self.cfg, self.lanes
        names = la.model.LAYER_TENSORS
        gi, ui, di = names.index("wgate"), names.index("wup"), names.index("wdown")
        x = la.CudaBuffer.from_slice(ctx, la.synth.normal_f16((m, cfg.hidden), 91))
        gate, up = la.CudaBuffer.empty(ctx, m * cfg.inter * 2), la.CudaBuffer.empty(ctx, m * cfg.inter * 2)
        ffn = la.CudaBuffer.empty(ctx, m * cfg.hidden * 2)

        def enqueue(b):
            for li in range(cfg.n_layers):
                bufs = self.model._keep[li]
                self.k.matmul_nt_tq2_0_geglu_into(b, x, bufs[gi], bufs[ui], gate, up, gate, m, cfg.hidden, cfg.inter)
                self.k.matmul_nt_tq2_0_into(b, gate, bufs[di], ffn, m, cfg.inter, cfg.hidden)
        b = la.CommandBatch.new(ctx)
        enqueue(b)
        n_launch = b.dispatch_count()
        b.commit_and_wait()
        b = la.CommandBatch.capture(ctx)
        enqueue(b)
        graph = b.end_capture()
        ms = timed(graph.launch, 10, 3)
        graph.destroy()
        tq = lambda r, c: r * (c // 256) * 66
        bytes_geglu = 2 * tq(cfg.inter, cfg.hidden) + m * cfg.hidden * 2 + m * cfg.inter * 2
        bytes_down = tq(cfg.hidden, cfg.inter) + m * cfg.inter * 2 + m * cfg.hidden * 2
        per_launch = (bytes_geglu + bytes_down) / 2
        us = ms * 1e3 / n_launch
        achieved = per_launch / (us * 1e-6) / 1e9
        whole = self.alg_bytes_per_step / (ms_per_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": self.FFN_TRAFFIC["bytes"] if m == 64 else None,
                "traffic_source": self.FFN_TRAFFIC if m == 64 else None, "peak_kind": peak_kind,
                "kernel": (f"{'qgemv_kernel' if m <= 8 else 'qgemm_tcd_kernel (tcgen05)' if m <= 64 else 'qgemm_tc_kernel (tcgen05) + gelu_mul'}"
                           f"<TQ2_0, m={m}>: GeGLU + down projections of {cfg.n_layers} layers, {n_launch} launches"),
                "us_per_launch": us, "algorithmic_bytes_per_launch": per_launch,
                "launches_timed_alone_share_of_step": ms / ms_per_step,
                "whole_step": {"achieved": whole, "frac": whole / peak, "algorithmic_bytes_per_step": self.alg_bytes_per_step,
                               "bound_tok_s": self.lanes / (self.alg_bytes_per_step / (peak * 1e9))}}

    def cpu_sample(self, orc, threads: int):
        lanes = min(2, self.lanes)
        cfg = self.la.e2b_like_config(max_lanes=lanes, max_context=self.cfg.max_context, n_layers=self.cfg.n_layers,
                                      vocab=self.cfg.vocab)
        om = orc.OracleModel(cfg, self.host_layers, self.emb, self.fnorm, self.geo)
        # the oracle's pools start empty (zero rows); the attention's cost does not depend on the values
        tok = self.tokens_host[:lanes].copy()
        pos = self.positions_host[:lanes].copy()
        orc.set_step_baseline_matmul(True)      # projections as the CPU baseline computes them: f16 weights, f32 dot
        try:
            t0 = time.perf_counter()
            om.decode_batch_step(tok, pos)
            dt = time.perf_counter() - t0
        finally:
            orc.set_step_baseline_matmul(False)
        return dt, lanes / dt, (f"1 step of {lanes} lane(s) at context {self.context}, all {self.cfg.n_layers} layers + "
                                "vocabulary projection (dequant to f16 + f32 dot, all host threads)")


class RaggedDecode(DecodeStep):
    """Config 5: 512 concurrent sequences of the config-4 model with lognormal context lengths (median 2048,
    sigma 1.0, clipped to [16, 131072]; seed fixed), sharded by request across the ranks (balanced by context
    sum), weights replicated, each lane's KV on its owner GPU.  Vocabulary projection:
      replicated  every rank projects its own lanes against the whole table; no collective (default);
      allgather   the table is row-split; hidden rows are all-gathered (1.5 MB), every rank projects its rows for
                  all 512 lanes and the f32 logit slices are all-gathered over NCCL (537 MB per step), as the
                  configuration states; greedy tokens are then taken on every rank (per-shard records + merge);
      pairs       as allgather up to the projection; then every rank reduces its slice to (max, first index) per
                  lane on the device and only those 8 bytes per lane are all-gathered and merged with the
                  first-maximum rule (local-engine/src/sampler.rs:148-158).
    The collectives go through the C ABI (lc_comm_*), enqueued on the step's stream.
    One step = one token for every one of the 512 sequences; value = 512 / step time (strong scaling)."""

    def __init__(self, la, ctx, kernels, rank: int, world: int, vocab_mode: str = "replicated", total: int = 512,
                 n_layers: int = 35, vocab: int = 262144, max_ctx: int = 131072, share: "DecodeStep | None" = None,
                 comm=None):
        self.la, self.ctx, self.k, self.comm = la, ctx, kernels, comm
        self.rank, self.world, self.vocab_mode, self.total = rank, world, vocab_mode, total
        ctxs = la.synth.lognormal_contexts(total, seed=55, hi=max_ctx)
        self.shards = la.sharding.shard_lanes(ctxs, world)
        self.my = self.shards[rank]
        self.lanes = len(self.my)
        self.context = int(ctxs[self.my].max())
        cfg = la.e2b_like_config(max_lanes=self.lanes, max_context=self.context + 260, n_layers=n_layers, vocab=vocab)
        self.cfg = cfg
        self.model = la.DecodeModel(ctx, kernels, cfg)
        self.host_layers = []
        for i in range(n_layers):
            t = share.host_layers[i] if share is not None else la.model.synth_layer(cfg, i, seed=4)
            self.model.set_layer(i, t)
        self.emb, self.fnorm = (share.emb, share.fnorm) if share is not None else la.model.synth_embedding(cfg, seed=4)
        self.emb_buf = la.CudaBuffer.from_slice(ctx, self.emb)
        self.model.set_embedding(self.emb_buf, self.fnorm)
        self.emb = None
        cb = la.tq_code_bytes(cfg.head_dim, cfg.kv_bits)
        self.kv_bytes = 0
        my_ctx = ctxs[self.my].astype(np.int64)
        for i in range(n_layers):
            kv = self.model.kv_buffers(i)
            for name in ("k_codes", "v_codes"):
                kv[name].fill(0x9C)          # codes 0,3,1,2 repeating: every level occurs
            for name in ("k_norms", "v_norms"):
                kv[name].fill(0x4C)          # f16 0x4C4C = 17.2, about |N(0, I_256)|
            eff = np.minimum(my_ctx + 1, kv["window"]) if kv["window"] else my_ctx + 1
            self.kv_bytes += int(eff.sum()) * cfg.n_kv_heads * (2 * cb + 4)
        tq = lambda r, c: r * (c // 256) * 66
        qd, kd = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        per_layer = (tq(qd, cfg.hidden) + 2 * tq(kd, cfg.hidden) + tq(cfg.hidden, qd) + 2 * tq(cfg.inter, cfg.hidden) +
                     tq(cfg.hidden, cfg.inter))
        vocab_rows = vocab if vocab_mode == "replicated" else (la.sharding.vocab_rows(vocab, world, rank)[1] -
                                                                la.sharding.vocab_rows(vocab, world, rank)[0])
        self.weight_bytes = n_layers * per_layer + vocab_rows * (cfg.hidden // 32) * 18
        self.alg_bytes_per_step = self.weight_bytes + self.kv_bytes
        self.tokens_host = (la.synth.splitmix64(7, total) % np.uint64(vocab)).astype(np.uint32)[self.my]
        self.positions_host = ctxs[self.my].astype(np.uint32)
        self.tokens = la.CudaBuffer.from_slice(ctx, self.tokens_host)
        self.positions = la.CudaBuffer.from_slice(ctx, self.positions_host)
        self.next_tokens = la.CudaBuffer.empty(ctx, max(self.lanes, total) * 4)
        self.name = (f"ragged decode, {total} sequences (lognormal contexts, median 2048) of the E2B-like decoder sharded by "
                     f"request over {world} GPU(s), vocabulary {vocab_mode}")
        self.copies, self.wbytes, self.graph, self.launches_per_step = 1, self.weight_bytes, None, None
        self.geo, self.n_layers_, self.vocab_ = [], n_layers, vocab

    def prepare(self):
        import torch
        import torch.distributed as dist
        la, ctx, cfg = self.la, self.ctx, self.cfg
        local_vocab = self.vocab_mode == "replicated"
        b = la.CommandBatch.new(ctx)
        self.model.decode_batch_step_into(b, self.tokens, self.positions, self.lanes, False,
                                          self.next_tokens if local_vocab else None)
        self.launches_per_step = b.dispatch_count()
        b.commit_and_wait()
        b = la.CommandBatch.capture(ctx)
        self.model.decode_batch_step_into(b, self.tokens, self.positions, self.lanes, False,
                                          self.next_tokens if local_vocab else None)
        self.graph = b.end_capture()
        if not local_vocab:
            assert self.total % self.world == 0, "the row-split variants need equal shards"
            assert self.world == 1 or self.comm is not None, "the row-split variants need a communicator"
            lo, hi = la.sharding.vocab_rows(self.vocab_, self.world, self.rank)
            self.rows, self.lo = hi - lo, lo
            rb = cfg.hidden // 32 * 18
            self.table_slice = la.CudaBuffer.wrap(ctx, self.emb_buf.device_ptr + lo * rb, self.rows * rb)
            if not hasattr(self, "hidden_all"):
                self.hidden_all = la.CudaBuffer.empty(ctx, self.total * cfg.hidden * 2)
                self.logits_slice = la.CudaBuffer.empty(ctx, self.total * self.rows * 4)
                self.pairs_all = la.CudaBuffer.empty(ctx, self.world * self.total * 8)
                self.next_all = la.CudaBuffer.empty(ctx, self.total * 4)
            if self.vocab_mode == "allgather" and not hasattr(self, "logits_all"):
                self.logits_all = la.CudaBuffer.empty(ctx, self.world * self.total * self.rows * 4)
            self.hidden_local = self.model.hidden_buffer()
            b = la.CommandBatch.new(ctx)
            self._enqueue_vocab(b)
            self.launches_per_step += b.dispatch_count()
            b.commit_and_wait()

    def _gather(self, b, buf, bytes_per_rank, send=None):
        """All-gather into `buf` ([world] x bytes_per_rank); `send` = None means in place (this rank's slot of buf)."""
        if self.world > 1:
            self.comm.all_gather_into(b, send if send is not None else buf, 0 if send is not None else self.rank * bytes_per_rank,
                                      buf, bytes_per_rank)
        elif send is not None:
            b.blit_buffer_copy(send, 0, buf, 0, bytes_per_rank)

    def _enqueue_vocab(self, b):
        la, ctx, cfg, n, total = self.la, self.ctx, self.cfg, self.lanes, self.total
        b.blit_buffer_copy(self.hidden_local, 0, self.hidden_all, self.rank * n * cfg.hidden * 2, n * cfg.hidden * 2)
        self._gather(b, self.hidden_all, n * cfg.hidden * 2)
        self.k.matmul_nt_q4_0_f32out_into(b, self.hidden_all, self.table_slice, self.logits_slice, total, cfg.hidden, self.rows)
        pair_slot = lambda r: la.CudaBuffer.wrap(ctx, self.pairs_all.device_ptr + r * total * 8, total * 8)
        if self.vocab_mode == "allgather":
            self._gather(b, self.logits_all, total * self.rows * 4, send=self.logits_slice)
            for r in range(self.world):
                sl = la.CudaBuffer.wrap(ctx, self.logits_all.device_ptr + r * total * self.rows * 4, total * self.rows * 4)
                self.k.argmax_pairs_f32_into(b, sl, pair_slot(r), total, self.rows, r * self.rows)
        else:
            self.k.argmax_pairs_f32_into(b, self.logits_slice, pair_slot(self.rank), total, self.rows, self.lo)
            self._gather(b, self.pairs_all, total * 8)
        self.k.merge_argmax_pairs_into(b, self.pairs_all, self.next_all, total, self.world)

    def gathers_alone(self):
        """The variant's collectives without the compute between them (timed alone by the bench)."""
        b = self.la.CommandBatch.new(self.ctx)
        self._gather(b, self.hidden_all, self.lanes * self.cfg.hidden * 2)
        if self.vocab_mode == "allgather":
            self._gather(b, self.logits_all, self.total * self.rows * 4, send=self.logits_slice)
        else:
            self._gather(b, self.pairs_all, self.total * 8)
        for p in getattr(self, "_pend2", []):
            p.wait()
        self._pend2 = [b.commit_async()]

    def step(self):
        self.graph.launch()
        if self.vocab_mode == "replicated":
            return
        for p in getattr(self, "_pend", []):   # the previous step's batch (long finished): release its event
            p.wait()
        b = self.la.CommandBatch.new(self.ctx)
        self._enqueue_vocab(b)
        self._pend = [b.commit_async()]

    def l2_note(self):
        return (f"inputs larger than L2: {self.weight_bytes / 1e6:.0f} MB of weights + {self.kv_bytes / 1e6:.0f} MB of KV "
                "read per step on this rank")

    def check(self, orc):
        if self.vocab_mode == "replicated":
            nt = self.next_tokens.as_slice(np.uint32, self.lanes)
            assert np.all(nt < self.cfg.vocab), "argmax out of range"
        else:
            self.ctx.synchronize()
            assert int(self.next_all.as_slice(np.uint32, self.total).max()) < self.cfg.vocab

    def prepare_e2e(self):
        self.h_in = self.la.PinnedHost(2 * self.lanes * 4, dtype=np.uint32)
        self.h_out = self.la.PinnedHost(self.lanes * 4, dtype=np.uint32)
        self.h_in.array[: self.lanes] = self.tokens_host
        self.h_in.array[self.lanes:] = self.positions_host
        self.e2e_pos0 = self.positions_host.copy()
        self.e2e_steps = 0
        self.h2d, self.d2h = 2 * self.lanes * 4, self.lanes * 4

    def step_e2e(self):
        b = self.la.CommandBatch.new(self.ctx)
        b.upload(self.tokens, 0, self.h_in.ptr, self.lanes * 4)
        b.upload(self.positions, 0, self.h_in.ptr + self.lanes * 4, self.lanes * 4)
        b.commit_and_wait()
        self.step()
        if self.vocab_mode == "replicated":
            b = self.la.CommandBatch.new(self.ctx)
            b.download(self.next_tokens, 0, self.h_out.ptr, self.lanes * 4)
            b.commit_and_wait()
            self.h_in.array[: self.lanes] = self.h_out.array
        else:
            b = self.la.CommandBatch.new(self.ctx)
            b.download(self.next_all, self.rank * self.lanes * 4, self.h_out.ptr, self.lanes * 4)
            b.commit_and_wait()
            self.h_in.array[: self.lanes] = self.h_out.array
        self.e2e_steps += 1
        self.h_in.array[self.lanes:] = self.e2e_pos0 + (self.e2e_steps % 200)

    def metric(self):
        return f"decode_tok_s_ragged{self.total}", "tok/s"

    def value(self, ms_per_step: float) -> float:
        return self.total / self.world / (ms_per_step * 1e-3)   # main() multiplies by world

    def cpu_sample(self, orc, threads: int):
        return 0.0, 0.0, "not timed for the ragged workload (see the batch-64 workload)"


WORKLOADS = {
    "matvec_tq2_0": lambda la, ctx, k: QuantMatvec(la, ctx, k, "tq2_0", 8192, 1536, 1),
    "matvec_tq2_0_grouped": lambda la, ctx, k: QuantMatvec(la, ctx, k, "tq2_0", 8192, 1536, 1, grouped=True),
    "matvec_q4_0_grouped": lambda la, ctx, k: QuantMatvec(la, ctx, k, "q4_0", 6144, 1536, 1, grouped=True),
    "matvec_q4_0": lambda la, ctx, k: QuantMatvec(la, ctx, k, "q4_0", 6144, 1536, 1),
    "matmul_tq2_0_m16": lambda la, ctx, k: QuantMatvec(la, ctx, k, "tq2_0", 8192, 1536, 16),
    "matmul_tq2_0_m64": lambda la, ctx, k: QuantMatvec(la, ctx, k, "tq2_0", 8192, 1536, 64),
    "matmul_tq2_0_m256": lambda la, ctx, k: QuantMatvec(la, ctx, k, "tq2_0", 8192, 1536, 256),
    "matvec_vocab_q4_0": lambda la, ctx, k: QuantMatvec(la, ctx, k, "q4_0", 262144, 1536, 1, min_copies=3),
    "matmul_vocab_q4_0_m64": lambda la, ctx, k: QuantMatvec(la, ctx, k, "q4_0", 262144, 1536, 64, min_copies=2, f32out=True),
    "decode_b64": lambda la, ctx, k: DecodeStep(la, ctx, k, 64, 8192),
    "decode_b1": lambda la, ctx, k: DecodeStep(la, ctx, k, 1, 8192),
    "decode_b64_small": lambda la, ctx, k: DecodeStep(la, ctx, k, 64, 2048, n_layers=5, vocab=32768),
    "attention_32768x1": lambda la, ctx, k: TqAttention(la, ctx, k, 1, 32767),
    "attention_131072x1": lambda la, ctx, k: TqAttention(la, ctx, k, 1, 131071),
    "attention_8193x64": lambda la, ctx, k: TqAttention(la, ctx, k, 64, 8192),
    "attention_2049x64": lambda la, ctx, k: TqAttention(la, ctx, k, 64, 2048),
    "ragged512": None, "ragged512_allgather": None, "ragged512_pairs": None,
    "ragged64_small": None, "ragged64_small_allgather": None, "ragged64_small_pairs": None,
}
DEFAULT_WORKLOAD = "decode_b64"


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def _load_module(name: str, path: Path):
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_extras(la, ctx, kernels, headline, timed_local, orc, peak: float, peak_kind: str, device: int) -> dict:
    """The other halves of the metric, measured in the same process after the headline (rank 0 only, no
    collective): batch-1 decode, the fused-dequant matvec / matmul configurations and decode attention at the
    configured contexts.  Each entry has its own CUDA-event time over about half a second of back-to-back steps,
    its own clock sample, its algorithmic bytes and its check against the oracle."""
    import gc
    out = {}

    def measure(key, make):
        try:
            wl = make()
            wl.prepare()
            ms1 = timed_local(wl.step, 3, 3)
            steps = int(min(2000, max(5, 0.5e3 / max(ms1, 1e-3))))
            sampler = ClockSampler(device)
            sampler.start()
            time.sleep(0.3)
            ms = timed_local(wl.step, steps, 3)
            clocks = sampler.stop()
            wl.check(orc)
            metric, unit = wl.metric()
            r = wl.roofline(ms, peak, peak_kind, timed_local)
            rec = {"metric": metric, "value": wl.value(ms), "unit": unit, "ms_per_step": ms, "steps": steps,
                   "workload": wl.name, "l2_policy": wl.l2_note(), "kernel": r["kernel"], "clocks": clocks}
            if isinstance(wl, DecodeStep):
                w = r["whole_step"]
                rec.update({"hbm_gbs": w["achieved"], "frac": w["frac"], "algorithmic_bytes_per_step": w["algorithmic_bytes_per_step"],
                            "gpu_launches_per_step": wl.launches_per_step, "parity": getattr(wl, "parity", None)})
            else:
                rec.update({"hbm_gbs": r["achieved"], "frac": r["frac"], "us_per_launch": r["us_per_launch"],
                            "algorithmic_bytes_per_launch": r["algorithmic_bytes_per_launch"]})
            rec["peak_kind"] = peak_kind
            out[key] = rec
            del wl
        except Exception as e:   # an extra must not take the headline down with it
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
        gc.collect()

    measure("decode_b1", lambda: DecodeStep(la, ctx, kernels, 1, 8192, share=headline))
    measure("matvec_q4_0", lambda: QuantMatvec(la, ctx, kernels, "q4_0", 6144, 1536, 1))
    measure("matvec_q4_0_grouped", lambda: QuantMatvec(la, ctx, kernels, "q4_0", 6144, 1536, 1, grouped=True))
    measure("matvec_tq2_0_m1_grouped", lambda: QuantMatvec(la, ctx, kernels, "tq2_0", 8192, 1536, 1, grouped=True))
    for m in (1, 16, 64):
        measure(f"matvec_tq2_0_m{m}", lambda m=m: QuantMatvec(la, ctx, kernels, "tq2_0", 8192, 1536, m))
    measure("matvec_vocab_q4_0", lambda: QuantMatvec(la, ctx, kernels, "q4_0", 262144, 1536, 1, min_copies=3))
    measure("matmul_vocab_q4_0_m64", lambda: QuantMatvec(la, ctx, kernels, "q4_0", 262144, 1536, 64, min_copies=2, f32out=True))
    measure("attention_32768x1", lambda: TqAttention(la, ctx, kernels, 1, 32767))
    measure("attention_131072x1", lambda: TqAttention(la, ctx, kernels, 1, 131071))
    measure("attention_8193x64", lambda: TqAttention(la, ctx, kernels, 64, 8192))
    return out


def run_ragged_extras(la, ctx, kernels, headline, timed, rank: int, world: int, comm, small: bool) -> dict:
    """Config 5 on `world` GPUs (every rank calls this): 512 ragged sequences sharded by request with the vocabulary
    projection (A) replicated, no collective; (B) row-split with the NCCL all-gather of the f32 logit slices; (C)
    row-split with per-shard (max, first index) records, 8 bytes per lane gathered and merged on the device.  For B and
    C the collectives are also timed alone, so that their share of the step is a measurement."""
    kw = dict(total=64, n_layers=5, vocab=32768, max_ctx=8192) if small else {}
    out, tag = {}, "ragged64_small" if small else "ragged512"
    wl = RaggedDecode(la, ctx, kernels, rank, world, "replicated", share=headline, comm=comm, **kw)
    for mode, label in (("replicated", "vocabulary replicated (no collective)"),
                        ("allgather", "vocabulary row-split + NCCL all-gather of f32 logits"),
                        ("pairs", "vocabulary row-split + all-gather of (max, index) records, 8 B per lane")):
        if mode != "replicated" and wl.total % world != 0:
            continue
        wl.vocab_mode = mode
        wl.prepare()
        ms = timed(wl.step, 5, 3)
        wl.check(None)
        rec = {"metric": wl.metric()[0], "value": wl.total / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms, "n_gpus": world,
               "workload": wl.name.replace("vocabulary replicated", label), "lanes_on_rank0": wl.lanes,
               "gpu_launches_per_step": wl.launches_per_step}
        if mode != "replicated":
            rec["collectives_ms_alone"] = timed(wl.gathers_alone, 5, 3)
            rec["collective_bytes_per_rank_per_step"] = wl.total // world * wl.cfg.hidden * 2 + (
                wl.total * wl.rows * 4 if mode == "allgather" else wl.total * 8)
        out[f"{tag}_{mode}"] = rec
    return out


def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU path for this workload on the host cores (rank 0 only): the reference is Rust +
    Metal and cannot be built or run here, so this arm times the oracle's restatement of what the reference
    computes on a CPU, with all host threads, on a bounded sample of the same workload."""
    if rank != 0:
        return
    orc = entry.load_oracle()
    synth = _load_module("la_synth", ROOT / "local-ai_b200" / "synth.py")
    name = args.workload
    orc.set_num_threads(orc.host_threads())   # torch.distributed.run exports OMP_NUM_THREADS=1 to every rank
    threads = orc.num_threads()
    note = ("CPU restatement of the reference's arithmetic (oracle/); the reference's Metal path is unavailable on "
            "this box and its Rust toolchain is absent")
    if name.startswith("decode") or name.startswith("ragged"):
        import ctypes as C

        class Cfg:  # the lc_model_config field names the oracle model reads
            pass

        ragged = name.startswith("ragged")
        lanes_full, context, n_layers, vocab = {"decode_b64": (64, 8192, 35, 262144), "decode_b1": (1, 8192, 35, 262144),
                                                "decode_b64_small": (64, 2048, 5, 32768),
                                                "ragged512": (512, 2048, 35, 262144), "ragged512_allgather": (512, 2048, 35, 262144),
                                                "ragged512_pairs": (512, 2048, 35, 262144),
                                                "ragged64_small": (64, 2048, 5, 32768), "ragged64_small_pairs": (64, 2048, 5, 32768),
                                                "ragged64_small_allgather": (64, 2048, 5, 32768)}[name]
        cfg = Cfg()
        cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.inter = 1536, 8, 1, 256, 6144
        cfg.vocab, cfg.n_layers, cfg.kv_bits = vocab, n_layers, 2
        sample_lanes = min(lanes_full, 2)
        cfg.max_lanes, cfg.max_context = sample_lanes, context + 512
        cfg.rms_eps, cfg.rope_theta, cfg.softmax_scale = 1e-6, 1e6, 1.0 / 16.0
        cfg.embed_scale = float(np.sqrt(np.float32(1536)))
        model = _load_module("la_model_shapes", ROOT / "oracle" / "synth_model.py")
        layers, emb, fnorm, geo = model.build(synth, cfg, context)
        om = orc.OracleModel(cfg, layers, emb, fnorm, geo)
        tok = (synth.splitmix64(7, sample_lanes) % np.uint64(vocab)).astype(np.uint32)
        pos = np.full(sample_lanes, context, np.uint32)
        orc.set_step_baseline_matmul(True)   # projections as a CPU would run them: weights to f16, naive f32 dot
        for _ in range(min(args.warmup, 1)):
            om.decode_batch_step(tok, pos)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            om.decode_batch_step(tok, pos)
        dt = (time.perf_counter() - t0) / args.steps
        val = sample_lanes / dt
        metric, unit = (f"decode_tok_s_ragged{lanes_full}" if ragged else f"decode_tok_s_batch{lanes_full}"), "tok/s"
        sample = (f"each step = {sample_lanes} of the {lanes_full} lanes, one token each at context {context}"
                  f"{' (the median of the lognormal contexts)' if ragged else ''}, all {n_layers} "
                  f"layers + vocabulary projection (dequant to f16 + f32 dot), {threads} OpenMP threads")
        wl_name = (f"ragged decode, {lanes_full} sequences (lognormal contexts, median 2048) of the E2B-like decoder" if ragged else
                   f"decode step, E2B-like dense decoder {n_layers} layers, batch {lanes_full}, context {context}, "
                   f"TQ2_0 weights + Q4_0 vocab {vocab}, tq2 KV")
    elif name.startswith("attention"):
        keys, lanes_full = {"attention_32768x1": (32768, 1), "attention_131072x1": (131072, 1),
                            "attention_8193x64": (8193, 64), "attention_2049x64": (2049, 64)}[name]
        hd, n_q, n_kv, bits, cb = 256, 8, 1, 2, 64
        codes = synth.splitmix64(4242, keys * cb // 8).view(np.uint8)
        norms = (16.0 * synth.uniform(4243, keys, 0.9, 1.1)).astype(np.float16)
        q = synth.normal_f16((1, n_q, hd), 3)
        a = (q, codes, norms, np.roll(codes, 64 * 7), np.roll(norms, 3), orc.tq_levels(hd, bits), orc.tq_signs(hd, 0x7459C0DE),
             np.array([keys - 1], np.uint32), hd, keys, n_q, n_kv, 0, bits, 1, 0, 1.0 / 16.0)
        for _ in range(min(args.warmup, 2)):
            orc.tq_attention_fused(*a)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            orc.tq_attention_fused(*a)
        dt = (time.perf_counter() - t0) / args.steps
        val = keys * (2 * cb + 4) / dt / 1e9
        metric, unit = "tq_decode_attention_hbm_gbs", "GB/s"
        sample = f"each step = one of the {lanes_full} lane(s), {keys} keys (fused code-space attention), {threads} OpenMP threads"
        wl_name = f"fused tq2 decode attention, {lanes_full} lane(s) x {keys} keys, 8 q heads / 1 kv head of 256"
    else:
        shapes = {"matvec_tq2_0": ("tq2_0", 8192, 1536, 1), "matvec_q4_0": ("q4_0", 6144, 1536, 1),
                  "matvec_tq2_0_grouped": ("tq2_0", 8192, 1536, 1), "matvec_q4_0_grouped": ("q4_0", 6144, 1536, 1),
                  "matmul_tq2_0_m16": ("tq2_0", 8192, 1536, 16), "matmul_tq2_0_m64": ("tq2_0", 8192, 1536, 64),
                  "matmul_tq2_0_m256": ("tq2_0", 8192, 1536, 256), "matvec_vocab_q4_0": ("q4_0", 262144, 1536, 1),
                  "matmul_vocab_q4_0_m64": ("q4_0", 262144, 1536, 64)}
        fmt, rows, cols, m = shapes[name]
        w = (synth.q4_0_weights if fmt == "q4_0" else synth.tq2_0_weights)(rows, cols, seed=1)
        x = synth.normal_f16((m, cols), seed=2)
        f = orc.Q4_0 if fmt == "q4_0" else orc.TQ2_0
        alg = w.size + m * cols * 2 + m * rows * (4 if name == "matmul_vocab_q4_0_m64" else 2)
        for _ in range(args.warmup):
            orc.baseline_matmul_nt(f, x, w, m, cols, rows, 0)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            orc.baseline_matmul_nt(f, x, w, m, cols, rows, 0)
        dt = (time.perf_counter() - t0) / args.steps
        val = alg / dt / 1e9
        metric, unit = "fused_quant_matvec_hbm_gbs", "GB/s"
        sample = f"each step = one {rows}x{cols} {fmt} matrix (dequant to f16 + naive f32 dot), {threads} OpenMP threads"
        wl_name = f"{fmt} fused dequant mat{'vec' if m == 1 else 'mul'} {rows}x{cols} batch {m}"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "l2_policy": "host memory: no device cache involved", "launch": "host threads (OpenMP)",
                   "replicas": 1, "note": note},
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra record (the metric's other halves)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    la = entry.load_package()
    ctx = la.CudaContext.new(local_rank)
    kernels = la.Kernels.new(ctx)
    comm = None

    def communicator():
        """NCCL through the C ABI; the unique id made on rank 0 travels over the process group."""
        nonlocal comm
        if comm is None and world > 1:
            uid = torch.zeros(la.Communicator.ID_BYTES, dtype=torch.uint8, device="cuda")
            if rank == 0:
                uid.copy_(torch.frombuffer(bytearray(la.Communicator.unique_id()), dtype=torch.uint8))
            dist.broadcast(uid, src=0)
            comm = la.Communicator(ctx, bytes(uid.cpu().numpy().tobytes()), rank, world)
        return comm

    if args.workload.startswith("ragged"):
        mode = "allgather" if args.workload.endswith("allgather") else "pairs" if args.workload.endswith("pairs") else "replicated"
        c = communicator() if mode != "replicated" else None
        if "small" in args.workload:
            wl = RaggedDecode(la, ctx, kernels, rank, world, mode, total=64, n_layers=5, vocab=32768, max_ctx=8192, comm=c)
        else:
            wl = RaggedDecode(la, ctx, kernels, rank, world, mode, comm=c)
    else:
        wl = WORKLOADS[args.workload](la, ctx, kernels)
    wl.prepare()
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))

    def barrier(collective: bool = True):
        ctx.synchronize()
        torch.cuda.synchronize()
        if world > 1 and collective:
            dist.barrier()

    def timed(step_fn, steps: int, warmup: int, collective: bool = True) -> float:
        """CUDA-event time per step; with `collective` every rank must call it (barrier on both sides, max over
        ranks), without it the measurement is local to the calling rank."""
        for _ in range(warmup):
            step_fn()
        barrier(collective)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            step_fn()
        e1.record(stream)
        barrier(collective)
        ms = e0.elapsed_time(e1) / steps
        if world > 1 and collective:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed_local(step_fn, steps: int, warmup: int) -> float:   # rank 0 alone (roofline of the dominant kernel)
        return timed(step_fn, steps, warmup, collective=False)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)  # let nvidia-smi come up so the timed region is covered
    ms = timed(wl.step, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    wl.prepare_e2e()
    ms_e2e = timed(wl.step_e2e, max(3, args.steps // 4), 3)
    extra = {}
    with_extra = not args.no_extra and args.workload in ("decode_b64", "decode_b64_small")
    if with_extra and world > 1:
        try:
            extra.update(run_ragged_extras(la, ctx, kernels, wl, timed, rank, world, communicator(),
                                           small=args.workload.endswith("small")))
        except Exception as e:
            extra["ragged"] = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    orc = entry.load_oracle()
    orc.set_num_threads(orc.host_threads())   # a launcher may have exported OMP_NUM_THREADS=1 to every rank
    wl.check(orc)
    peak, peak_kind = measured_peaks()
    metric, unit = wl.metric()
    value = wl.value(ms) * world
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if args.workload.startswith("ragged") else "weak",
        "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": wl.name, "l2_policy": wl.l2_note(), "launch": "one CUDA graph per step",
                   "replicas": world},
        "roofline": wl.roofline(ms, peak, peak_kind, timed_local),
        "e2e": {"value": wl.value(ms_e2e) * world, "unit": unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h},
        "gpu_launches": wl.launches_per_step * args.steps,
        "clocks": clocks,
    }
    if getattr(wl, "parity", None):
        line["parity"] = wl.parity
    if not args.no_cpu_baseline:
        threads = orc.num_threads()
        sec, gbs, desc = wl.cpu_sample(orc, 0)
        line["cpu_baseline"] = {"value": gbs, "unit": unit, "cores": threads, "kind": "port",
                                "sample": desc + f"; {sec * 1e3:.2f} ms"}
    if with_extra and args.workload == "decode_b64":
        extra.update(run_extras(la, ctx, kernels, wl, timed_local, orc, peak, peak_kind, local_rank))
    if extra:
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
