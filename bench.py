#!/usr/bin/env python
"""MoE-layer throughput benchmark (the reference's headline path, measured on B200).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A *step* is one pass of the MoE block over one batch of synthetic tokens (for
``decode20b``: over all 24 layers).  Workloads (shapes and value distributions
of the benchmark configurations; real checkpoints are not available offline, so
all tensors are seeded synthetic data):

  prefill120b (default)  gpt-oss-120b-shaped layer, E=128, 16384 tokens, uniform
                         routing; with N GPUs the tokens are split N ways and the
                         experts sharded 128/N per GPU (dispatch and return over
                         NVLink): strong scaling
  prefill20b_zipf        gpt-oss-20b-shaped layer, E=32, 8192 tokens, Zipf(1.1) router
                         bias scaled to a 4x busiest expert; N GPUs as above
  decode20b              24 gpt-oss-20b-shaped layers, 256 tokens per step (HBM-bound);
                         N GPUs = N independent replicas
  layer20b               one gpt-oss-20b-shaped layer, 64 tokens

Rank 0 prints ONE JSON line.  ``value`` is tokens/s with inputs resident in HBM;
``e2e`` is the same metric through ``moe_b200_forward_host`` (pinned host buffers,
host<->device copies inside the timed region); ``roofline`` describes the dominant
kernel (the gate/up expert GEMM) from CUDA-event timings taken on the launching
stream; ``parity`` compares output rows of this very run with the CPU oracle (the
run fails when they differ); ``cpu_baseline`` is the reference's CPU implementation
timed on this machine's host cores on a bounded token sample; ``sustained`` repeats
the timed region for at least two seconds (power-capped clocks); ``more`` holds the
same figures for the other workloads, measured after the headline.

``--impl reference`` times only that CPU implementation (rank 0; other ranks exit).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    "prefill120b": dict(E=128, T=16384, L=1, zipf=None, mode="ep", bound="tensor"),
    "prefill20b_zipf": dict(E=32, T=8192, L=1, zipf=1.1, mode="ep", bound="tensor"),
    "decode20b": dict(E=32, T=256, L=24, zipf=None, mode="replica", bound="hbm"),
    "layer20b": dict(E=32, T=64, L=1, zipf=None, mode="replica", bound="hbm"),
}
METRIC = "moe_layer_tokens_per_s"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum, bytes) of ONE launch of the
# dominant kernel on one GPU, from the ncu captures summarised under profiles/; reported
# only for the single-GPU shape the capture covers (a rank of an N-GPU run does 1/N of the
# work: no capture, no figure).
NCU_TRAFFIC = {
    "decode20b": dict(bytes=296.0e6, source="ncu capture of this launch: one layer, 256 tokens "
                                            "(profiles/expert_gemm_ts_layer20b_256tok_ncu_full.md)"),
    "layer20b": dict(bytes=None, source="not captured at 64 tokens"),
    "prefill120b": dict(bytes=1.80e9, source="ncu capture of the 20b-shaped layer at 2048 tokens, scaled to this "
                                             "launch by the units processed: weight bytes x4 (128 experts), row "
                                             "bytes x8 (profiles/expert_gemm_pair_prefill20b_zipf_2048tok_ncu_full.md)"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed regions run."""
    Q = ("uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, uuid):
        self.uuid, self.rows, self.proc = uuid, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) >= 8 and (self.uuid is None or self.uuid in f[0]):
                self.rows.append((time.monotonic(), f))

    def summary(self, t0=None, t1=None):
        """Median SM clock and the reasons seen between two time.monotonic() stamps
        (default: everything sampled so far)."""
        rows = [f for (t, f) in self.rows if (t0 is None or t >= t0) and (t1 is None or t <= t1)]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[4 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][2]) if rows[0][2].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}

    def stop(self):
        if self.proc:
            self.proc.terminate()


def cpu_reference_run(wl, shape, steps, warmup, sample_tokens, seed=0):
    """Times the reference's CPU MoE block (oracle/_ref when built, else the C
    restatement) on `sample_tokens` tokens of the workload with every host core
    this process may use; returns (tokens/s, seconds per step, descriptor dict)."""
    from gpt_oss_amd_b200 import synth
    from oracle import oracle

    impl = "reference" if oracle.have_reference() else "port"
    # explicit: torch.distributed.run exports OMP_NUM_THREADS=1 to its children
    oracle.use_all_cores()
    w_router, b_router = synth.make_router(shape, seed, wl["zipf"], synth.ZIPF_GAIN_4X)
    x = synth.bf16_bits_to_f32(synth.make_tokens(sample_tokens, shape.hidden, seed))
    cache = oracle.ExpertCache(None, None, None, None, None, None,
                               loader=lambda e: synth.make_experts(shape, seed, e, 1))
    wr = synth.bf16_bits_to_f32(w_router)
    # the CPU engine's own numerics (fp32 activations): round_mode 0
    run = lambda: oracle.moe_forward(x, wr, b_router, cache, top_k=shape.top_k, round_mode=0, impl=impl)
    run()  # decodes the experts the sample touches (not timed) and warms the caches
    for _ in range(max(0, warmup - 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    tps = sample_tokens / dt
    desc = {"value": tps, "unit": "tokens/s", "cores": oracle.num_threads(impl),
            "host_cores": oracle.host_cores(), "kind": impl,
            "sample": f"{sample_tokens} tokens of the workload's seeded input through one layer "
                      f"(src/run.cpp:628-707 token at a time, fp32 weights), {steps} timed passes"}
    return tps, dt, desc


class Bench:
    """One engine and the measurements taken on it."""

    def __init__(self, args, dist, rank, world, local_rank):
        self.args, self.dist, self.rank, self.world, self.local_rank = args, dist, rank, world, local_rank
        self.peaks = load_peaks()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *vals):
        if self.dist is None:
            return [float(v) for v in vals]
        t = torch.tensor(list(vals), dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    # ------------------------------------------------------------------ set-up
    def make_engine(self, E, n_layers, max_tokens, ep):
        import gpt_oss_amd_b200 as pkg
        shape = pkg.MoEShape(n_experts=E)
        eng = pkg.MoEEngine(shape, n_layers=n_layers, max_tokens=max_tokens,
                            ep_rank=self.rank if ep > 1 else 0, ep_size=ep, device=self.local_rank)
        if ep > 1:
            eng.ep_connect(self.dist, self.args.ep_exchange)
        return shape, eng

    # ------------------------------------------------------------------ one workload
    def measure(self, name, wl, eng, shape, layers, seeds, ep, steps, warmup, headline):
        """Times `steps` steps of workload `name` on `eng` (its layers `layers`, generated
        from `seeds`), then profiles the stages, checks a token sample against the oracle
        and, for the headline, measures the sustained and end-to-end figures."""
        from gpt_oss_amd_b200 import synth
        args, dist, rank, world = self.args, self.dist, self.rank, self.world
        H, I, K = shape.hidden, shape.intermediate, shape.top_k
        T_total = wl["T"]
        if wl["mode"] == "ep":
            T_local = T_total // world
            tokens_job = T_local * world
            x_bits = synth.make_tokens(T_total, H, seed=0)[rank * T_local:(rank + 1) * T_local]
        else:
            T_local = T_total
            tokens_job = T_total * world
            x_bits = synth.make_tokens(T_local, H, seed=0)
        x_host = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).view(torch.bfloat16).pin_memory()
        x_dev = x_host.cuda()
        out_dev = torch.empty(T_local, H, dtype=torch.float32, device="cuda")
        stream = torch.cuda.current_stream()
        L = len(layers)

        def step():
            for layer in layers:
                eng.forward(layer, x_dev, out=out_dev)

        def timed(n):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            t0 = time.monotonic()
            ev0.record(stream)
            for _ in range(n):
                step()
            ev1.record(stream)
            self.barrier()
            return ev0.elapsed_time(ev1), t0, time.monotonic()

        for _ in range(warmup):
            step()
        self.barrier()
        launches_per_step = eng.last_launch_count() * L

        # timed region: exactly `steps` steps, nothing else on the stream
        ms_total, t_begin, t_end = timed(steps)
        (ms_step,) = self.max_over_ranks(ms_total / steps)
        res = {"ms_per_step": ms_step, "value": tokens_job / (ms_step * 1e-3), "steps": steps,
               "tokens_per_step": tokens_job, "gpu_launches": launches_per_step * steps,
               "timed_window": (t_begin, t_end)}

        # the same steps once more with CUDA-event pairs around every stage (on the
        # launching stream) for the per-kernel durations behind `roofline`
        n_prof = min(steps * L, 2048)
        eng.profile(n_prof)
        for _ in range((n_prof + L - 1) // L):
            step()
        self.barrier()
        stage_ms = {}
        for c in range(n_prof):
            for k, v in eng.profile_read(c).items():
                stage_ms.setdefault(k, []).append(v)
        eng.profile(0)
        res["stage_ms"] = {k: statistics.mean(v) for k, v in stage_ms.items() if any(v)}
        counts = eng.last_expert_counts()

        # sustained: the same timed region again, at least two seconds long
        if headline:
            n_long = int(min(20000, max(steps, 2000.0 / max(ms_step, 1e-3))))
            if dist is not None:
                (n_long,) = self.max_over_ranks(n_long)
                n_long = int(n_long)
            ms_long, t0, t1 = timed(n_long)
            (ms_long_step,) = self.max_over_ranks(ms_long / n_long)
            res["sustained"] = {"steps": n_long, "ms_per_step": ms_long_step,
                                "value": tokens_job / (ms_long_step * 1e-3), "window": (t0, t1)}
        status = eng.device_status()
        if status != 0:
            raise SystemExit(f"{name}: device status word 0x{status:x}: a kernel wait ran out")

        # ---- parity record: rows of this run against the CPU oracle (outside any timed region)
        res["parity"] = self.parity(name, wl, eng, shape, layers[0], seeds[0], x_bits, x_dev, ep)

        # ---- roofline of the dominant kernel (gate/up GEMM + SwiGLU), per GPU
        rows_local = sum(counts)  # rows this rank's gate/up GEMM processed in the last call
        g1_ms = res["stage_ms"].get("gemm1", 0.0)
        peaks = self.peaks
        if wl["bound"] == "tensor":
            alg = 2.0 * rows_local * (2 * I) * H
            achieved = alg / (g1_ms * 1e-3) / 1e12 if g1_ms > 0 else None
            peak, unit = peaks["bf16_tflops"], "TFLOP/s"
        else:
            active = sum(1 for c in counts if c > 0)
            alg = active * ((2 * I * H) // 2 + (2 * I * H) // 32 + 2 * I * 4) + rows_local * H * 2 \
                + rows_local * I * 2  # packed W1 + scales + bias, rows in, h out
            achieved = alg / (g1_ms * 1e-3) / 1e9 if g1_ms > 0 else None
            peak, unit = peaks["hbm_gbs"], "GB/s"
        # the library picks the kernel from the rows per local expert (pick_bn in csrc/moe_b200.cu)
        small = (T_local * K) // max(eng.n_local, 1) <= 64
        kernel = "tc5::ts::expert_gemm_ts_kernel<0>" if small else "tc5::pair::expert_gemm_pair_kernel<0>"
        cap = NCU_TRAFFIC.get(name) if (world == 1 and T_total == WORKLOADS[name]["T"]) else None
        res["roofline"] = {"kernel": kernel + " (gate/up GEMM + SwiGLU)", "bound": wl["bound"],
                           "achieved": achieved, "peak": peak, "unit": unit,
                           "frac": (achieved / peak) if achieved else None, "peak_source": peaks["source"],
                           "traffic": cap["bytes"] if cap else None,
                           "traffic_source": cap["source"] if cap else "no ncu capture at this shape",
                           "launch_ms": g1_ms, "algorithmic_per_launch": alg, "per": "GPU (rank 0)"}
        # whole step, per GPU
        flops_gpu = synth.moe_flops(tokens_job, shape) * L / world
        whole = {"tflops_per_gpu": flops_gpu / (ms_step * 1e-3) / 1e12,
                 "frac_of_bf16_peak": flops_gpu / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        if wl["bound"] == "hbm":
            b = synth.moe_decode_bytes(T_local, shape, sum(1 for c in counts if c > 0)) * L
            whole.update({"gbs_per_gpu": b / (ms_step * 1e-3) / 1e9,
                          "frac_of_hbm_peak": b / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]})
        if "sustained" in res:
            s = res["sustained"]
            s["tflops_per_gpu"] = flops_gpu / (s["ms_per_step"] * 1e-3) / 1e12
            if peaks["bf16_tflops_sustained"]:
                s["frac_of_bf16_sustained_peak"] = s["tflops_per_gpu"] / peaks["bf16_tflops_sustained"]
        res["whole_step"] = whole

        # load balance over ALL ranks: rows per expert (global) and rows per rank
        all_counts = [counts]
        if dist is not None and ep > 1:
            all_counts = [None] * world
            dist.all_gather_object(all_counts, counts)
        flat = [c for cs in all_counts for c in cs]
        per_rank = [sum(cs) for cs in all_counts]
        res["load"] = {"expert_rows_max_over_mean": (max(flat) / (sum(flat) / len(flat))) if sum(flat) else None,
                       "rank_rows_max_over_mean": (max(per_rank) / (sum(per_rank) / len(per_rank))) if sum(per_rank) else None,
                       "expert_rows_min": min(flat), "expert_rows_max": max(flat)}

        # ---- end to end through the host-buffer entry point
        if headline or wl["bound"] == "hbm":
            out_host = torch.empty(T_local, H, dtype=torch.float32).pin_memory()
            e2e_steps = max(3, min(steps, 10))
            for _ in range(2):
                for layer in layers:
                    eng.forward_host(layer, x_host, out_host)
            eng.profile(e2e_steps * L)
            self.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                for layer in layers:
                    eng.forward_host(layer, x_host, out_host)
            self.barrier()
            (e2e_s,) = self.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
            e2e_stage = {}
            for c in range(e2e_steps * L):
                try:
                    for k, v in eng.profile_read(c).items():
                        e2e_stage.setdefault(k, []).append(v)
                except Exception:
                    break  # a chunked call records no per-stage events
            eng.profile(0)
            res["e2e"] = {"value": tokens_job / e2e_s, "unit": "tokens/s",
                          "h2d_bytes_per_step": T_local * H * 2 * L * world,
                          "d2h_bytes_per_step": T_local * H * 4 * L * world,
                          "ms_per_step": e2e_s * 1e3,
                          "stage_ms": {k: statistics.mean(v) for k, v in e2e_stage.items() if any(v)}}
        res["tokens_per_rank"] = T_local
        res["experts_per_rank"] = eng.n_local
        res["device_bytes_per_gpu"] = eng.device_bytes()
        return res

    def parity(self, name, wl, eng, shape, layer, seed, x_bits, x_dev, ep):
        """Rows of this run's output against the CPU oracle (bf16-weight / fp32-accumulate
        numerics): every rank checks a few of its own tokens -- the experts they touch are
        regenerated from the seed, whichever rank holds them -- and rank 0 gets the worst
        figures over the ranks."""
        from gpt_oss_amd_b200 import synth
        from oracle import oracle, parity
        oracle.use_all_cores()
        T_local = x_bits.shape[0]
        n = self.args.parity_tokens if self.world == 1 else max(2, self.args.parity_tokens // self.world)
        n = min(n, T_local)
        part = None
        if n > 0:
            out, _, ti, tw = eng.forward(layer, x_dev, side=True)
            h_bits = eng.last_intermediate(T_local) if ep == 1 else None
            torch.cuda.synchronize()
            rows = np.unique(np.linspace(0, T_local - 1, n).astype(np.int64))
            r_t = torch.from_numpy(rows).cuda()
            sub = {"out": out[r_t].cpu().numpy(), "topk_i": ti[r_t].cpu().numpy(), "topk_w": tw[r_t].cpu().numpy()}
            if h_bits is not None:
                sub["h_bits"] = h_bits[r_t].cpu().numpy().view(np.uint16)
            w_router, b_router = synth.make_router(shape, seed, wl["zipf"], synth.ZIPF_GAIN_4X)
            part = parity.compare_sampled(sub, x_bits[rows], w_router, b_router,
                                          lambda e: synth.make_experts(shape, seed, e, 1), shape.top_k,
                                          group=4, finished=False)
        elif ep > 1:
            eng.forward(layer, x_dev)  # the call is collective
            torch.cuda.synchronize()
        parts = [part]
        if self.dist is not None:
            parts = [None] * self.world
            self.dist.all_gather_object(parts, part)
        m = parity.finish(parity.merge([p for p in parts if p]))
        m["ranks_checked"] = sum(1 for p in parts if p)
        m["layer"], m["against"] = layer, "CPU oracle (oracle/moe_oracle.c), round_mode 1"
        return m


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="prefill120b", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-sample", type=int, default=16, help="tokens in the CPU baseline sample")
    ap.add_argument("--parity-tokens", type=int, default=16, help="tokens checked against the oracle (whole job)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-more", action="store_true", help="skip the other workloads after the headline")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: inside the kernels over NVLink peer memory, or NCCL")
    ap.add_argument("--tokens", type=int, default=0,
                    help="override the workload's tokens per step (for small profiling captures)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    warmup = max(args.warmup, 3)
    wl = dict(WORKLOADS[args.workload])
    if args.tokens > 0:
        wl["T"] = args.tokens

    import gpt_oss_amd_b200 as pkg
    from gpt_oss_amd_b200 import synth

    shape = pkg.MoEShape(n_experts=wl["E"])
    config = {"workload": args.workload, "n_experts": wl["E"], "hidden": shape.hidden,
              "intermediate": shape.intermediate, "top_k": shape.top_k, "layers": wl["L"],
              "tokens_per_step": wl["T"], "weights": "MXFP4 packed (e2m1 + e8m0/32)",
              "l2": "weights streamed per step exceed L2 (no flush needed)"}

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, min(args.steps, 5))
        tps, dt, desc = cpu_reference_run(wl, shape, steps, min(warmup, 2), args.cpu_sample)
        tps_step = tps / wl["L"] if wl["L"] > 1 else tps
        desc["value"] = tps_step
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": tps_step, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": min(warmup, 2),
            "ms_per_step": dt * 1e3 * wl["L"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": desc,
            "e2e": {"value": tps_step, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
        }))
        return

    # ------------------------------------------------------------------ B200 arm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    b = Bench(args, dist, rank, world, local_rank)
    ep = world if (wl["mode"] == "ep") else 1
    T_local = wl["T"] // world if wl["mode"] == "ep" else wl["T"]

    # clocks are sampled from here to the end of the measurements
    sampler = None
    if rank == 0:
        uuid = None
        try:
            uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        except Exception:
            pass
        sampler = ClockSampler(uuid)
        sampler.start()

    _, eng = b.make_engine(wl["E"], wl["L"], T_local, ep)
    for layer in range(wl["L"]):
        lw = synth.make_layer(shape, seed=layer, zipf_s=wl["zipf"], zipf_gain=synth.ZIPF_GAIN_4X,
                              first=eng.first_expert, n=eng.n_local)
        eng.load_layer(layer, lw)
        del lw
    res = b.measure(args.workload, wl, eng, shape, list(range(wl["L"])), list(range(wl["L"])), ep,
                    args.steps, warmup, headline=True)
    # every rank releases its handle at the same point (the NCCL variant's communicator
    # is destroyed collectively)
    b.barrier()
    eng.close()
    b.barrier()

    # ------------------------------------------------------------------ the other workloads
    more = {}
    want_more = (not args.no_more) and args.workload == "prefill120b" and args.tokens == 0
    if want_more and world == 1:
        # one engine holds the 24 decode layers (seeds 0..23) and, as layer 24, the experts
        # of seed 0 under the Zipf router: decode20b, layer20b and prefill20b_zipf
        shape32 = pkg.MoEShape(n_experts=32)
        _, eng2 = b.make_engine(32, 25, 8192, 1)
        for layer in range(24):
            lw = synth.make_layer(shape32, seed=layer)
            eng2.load_layer(layer, lw)
            if layer == 0:
                wz, bz = synth.make_router(shape32, 0, 1.1, synth.ZIPF_GAIN_4X)
                lw.w_router, lw.b_router = wz, bz
                eng2.load_layer(24, lw)
            del lw
        k = max(5, min(args.steps, 30))
        more["decode20b"] = b.measure("decode20b", WORKLOADS["decode20b"], eng2, shape32, list(range(24)),
                                      list(range(24)), 1, k, 3, headline=False)
        more["layer20b"] = b.measure("layer20b", WORKLOADS["layer20b"], eng2, shape32, [0], [0], 1,
                                     max(k, 20), 3, headline=False)
        more["prefill20b_zipf"] = b.measure("prefill20b_zipf", WORKLOADS["prefill20b_zipf"], eng2, shape32,
                                            [24], [0], 1, k, 3, headline=False)
        eng2.close()
    elif want_more and world == 2:
        wz = WORKLOADS["prefill20b_zipf"]
        shape32 = pkg.MoEShape(n_experts=32)
        _, eng2 = b.make_engine(32, 1, wz["T"] // world, world)
        lw = synth.make_layer(shape32, seed=0, zipf_s=1.1, zipf_gain=synth.ZIPF_GAIN_4X,
                              first=eng2.first_expert, n=eng2.n_local)
        eng2.load_layer(0, lw)
        del lw
        more["prefill20b_zipf"] = b.measure("prefill20b_zipf", wz, eng2, shape32, [0], [0], world,
                                            max(5, min(args.steps, 30)), 3, headline=False)
        b.barrier()
        eng2.close()
        b.barrier()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    clocks = sampler.summary(*res.pop("timed_window"))
    if "sustained" in res:
        res["sustained"]["clocks"] = sampler.summary(*res["sustained"].pop("window"))
    for m in more.values():
        m["clocks"] = sampler.summary(*m.pop("timed_window"))
    sampler.stop()
    if clocks["samples"] == 0:
        # a short timed region can fall between two 200 ms samples: report the run's samples
        clocks = sampler.summary()
        clocks["note"] = "no sample fell inside the timed region; figures are over the whole run"

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        tps, dt, cpu = cpu_reference_run(wl, shape, steps=2, warmup=1, sample_tokens=args.cpu_sample)
        if wl["L"] > 1:
            cpu["value"] = tps / wl["L"]
            cpu["sample"] += f"; reported per {wl['L']}-layer step"

    if ep > 1:
        config["ep_exchange"] = args.ep_exchange
    config.update({"parallelism": (f"ep{ep}" if ep > 1 else ("single" if world == 1 else f"replicas{world}")),
                   "tokens_per_rank": res.pop("tokens_per_rank"), "experts_per_rank": res.pop("experts_per_rank"),
                   "gemm_impl": "tcgen05"})
    scaling = "strong" if wl["mode"] == "ep" else "weak"
    line = {
        "metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "roofline": res["roofline"], "whole_step": res["whole_step"], "parity": res["parity"],
        "cpu_baseline": cpu, "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"],
        "stage_ms": res["stage_ms"], "sustained": res.get("sustained"), "load": res["load"],
        "clocks": clocks, "device_bytes_per_gpu": res["device_bytes_per_gpu"],
    }
    if more:
        for m in more.values():
            m.pop("tokens_per_rank", None)
            m.pop("experts_per_rank", None)
        line["more"] = more
    print(json.dumps(line))
    bad = [n for n, m in [("headline", res)] + list(more.items()) if not m["parity"]["ok"]]
    if bad:
        raise SystemExit("parity against the oracle failed for: " + ", ".join(
            f"{n} ({(res if n == 'headline' else more[n])['parity']['why']})" for n in bad))


if __name__ == "__main__":
    main()
