#!/usr/bin/env python
"""MoE-layer throughput benchmark (the reference's headline path, measured on B200).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A *step* is one pass of the MoE block over one batch of synthetic tokens (for
``decode20b``: over all 24 layers).  Workloads (shapes and value distributions
of the benchmark configurations; real checkpoints are not available offline, so
all tensors are seeded synthetic data):

  prefill120b (default)  gpt-oss-120b-shaped layer, E=128, 16384 tokens, uniform
                         routing; with N GPUs the tokens are split N ways and the
                         experts sharded 128/N per GPU (NCCL all-to-all dispatch and
                         return): strong scaling
  prefill20b_zipf        gpt-oss-20b-shaped layer, E=32, 8192 tokens, Zipf(1.1) router
                         bias; N GPUs as above
  decode20b              24 gpt-oss-20b-shaped layers, 256 tokens per step (HBM-bound);
                         N GPUs = N independent replicas
  layer20b               one gpt-oss-20b-shaped layer, 64 tokens

Rank 0 prints ONE JSON line.  ``value`` is tokens/s with inputs resident in HBM;
``e2e`` is the same metric through ``moe_b200_forward_host`` (pinned host buffers,
host<->device copies inside the timed region); ``roofline`` describes the dominant
kernel (the gate/up expert GEMM) from CUDA-event timings taken on the launching
stream during the timed steps; ``cpu_baseline`` is the reference's CPU
implementation timed on this machine's host cores on a bounded token sample.

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
    #                 E    tokens layers zipf   mode
    "prefill120b": dict(E=128, T=16384, L=1, zipf=None, mode="ep", bound="tensor"),
    "prefill20b_zipf": dict(E=32, T=8192, L=1, zipf=1.1, mode="ep", bound="tensor"),
    "decode20b": dict(E=32, T=256, L=24, zipf=None, mode="replica", bound="hbm"),
    "layer20b": dict(E=32, T=64, L=1, zipf=None, mode="replica", bound="hbm"),
}
ZIPF_GAIN = 1.0
METRIC = "moe_layer_tokens_per_s"

# DRAM traffic of one launch of the dominant kernel from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum), bytes; None until captured.
NCU_TRAFFIC = {"prefill120b": 1.80e9,   # 2048-token capture scaled by components (see profiles/)
               "prefill20b_zipf": None,
               "decode20b": 296.3e6,    # captured directly: one layer, 256 tokens
               "layer20b": None}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

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
                self.rows.append(f)

    def stop(self):
        if self.proc:
            self.proc.terminate()
        rows = self.rows
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[4 + i] == "Active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": float(rows[0][2]) if rows[0][2].replace(".", "").isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def cpu_reference_run(wl, shape, steps, warmup, sample_tokens, seed=0):
    """Times the reference's CPU MoE block (oracle/_ref when built, else the C
    restatement) on `sample_tokens` tokens of the workload; returns (tokens/s,
    seconds per step, descriptor dict)."""
    from gpt_oss_amd_b200 import synth
    from oracle import oracle

    impl = "reference" if oracle.have_reference() else "port"
    w_router, b_router = synth.make_router(shape, seed, wl["zipf"], ZIPF_GAIN)
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
    desc = {"value": tps, "unit": "tokens/s", "cores": oracle.num_threads(impl), "kind": impl,
            "sample": f"{sample_tokens} tokens of the workload's seeded input through one layer "
                      f"(src/run.cpp:628-707 token at a time, fp32 weights), {steps} timed passes"}
    return tps, dt, desc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="prefill120b", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "mma_sync", "tcgen05_1cta"])
    ap.add_argument("--cpu-sample", type=int, default=16, help="tokens in the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    from gpt_oss_amd_b200 import capi, synth

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
    ep = world if (wl["mode"] == "ep") else 1
    ep_rank = rank if ep > 1 else 0
    T_total = wl["T"]
    if wl["mode"] == "ep":
        T_local = T_total // world
        scaling = "strong"
        tokens_per_step_job = T_local * world
    else:
        T_local = T_total
        scaling = "weak"
        tokens_per_step_job = T_total * world
    gemm_impl = {"mma_sync": capi.GEMM_MMA_SYNC, "tcgen05_1cta": capi.GEMM_TCGEN05_1CTA}.get(
        args.impl, capi.GEMM_TCGEN05)
    eng = pkg.MoEEngine(shape, n_layers=wl["L"], max_tokens=T_local, ep_rank=ep_rank, ep_size=ep,
                        device=local_rank, gemm_impl=gemm_impl)
    if ep > 1:
        eng.ep_connect(dist, args.ep_exchange)
    for layer in range(wl["L"]):
        lw = synth.make_layer(shape, seed=layer, zipf_s=wl["zipf"], zipf_gain=ZIPF_GAIN,
                              first=eng.first_expert, n=eng.n_local)
        eng.load_layer(layer, lw)
        del lw
    # tokens: the workload's seeded batch; rank r owns rows [r*T_local, (r+1)*T_local)
    x_bits = synth.make_tokens(T_total if wl["mode"] == "ep" else T_local, shape.hidden, seed=0)
    if wl["mode"] == "ep":
        x_bits = x_bits[rank * T_local:(rank + 1) * T_local]
    x_host = torch.from_numpy(np.ascontiguousarray(x_bits).view(np.int16)).view(torch.bfloat16).pin_memory()
    x_dev = x_host.cuda()
    out_dev = torch.empty(T_local, shape.hidden, dtype=torch.float32, device="cuda")
    out_host = torch.empty(T_local, shape.hidden, dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()

    def step():
        for layer in range(wl["L"]):
            eng.forward(layer, x_dev, out=out_dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from the first warm-up step to the end of the timed steps
    sampler = None
    if rank == 0:
        uuid = None
        try:
            uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        except Exception:
            pass
        sampler = ClockSampler(uuid)
        sampler.start()

    for _ in range(warmup):
        step()
    barrier()
    launches_per_step = eng.last_launch_count() * wl["L"]

    # timed region: exactly args.steps steps, nothing else on the stream
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    ms_total = ev0.elapsed_time(ev1)

    # the same steps once more with CUDA-event pairs around every stage (on the
    # launching stream) for the per-kernel durations behind `roofline`
    n_prof = min(args.steps * wl["L"], 4096)
    eng.profile(n_prof)
    for _ in range((n_prof + wl["L"] - 1) // wl["L"]):
        step()
    barrier()
    # a short run can end before nvidia-smi has printed its first line: keep the same
    # load on the GPU (untimed steps, the same number on every rank) until the whole
    # sampled region is about a second long
    done_ms = (warmup + 2 * args.steps) * (ms_total / args.steps)
    extra = int(min(5000, max(0.0, 1000.0 - done_ms) / max(ms_total / args.steps, 1e-3)))
    if dist is not None:
        te = torch.tensor([extra], dtype=torch.int64, device="cuda")
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        extra = int(te[0])
    for _ in range(extra):
        step()
    barrier()
    clocks = sampler.stop() if sampler else None
    stage_ms = {}
    for c in range(n_prof):
        for k, v in eng.profile_read(c).items():
            stage_ms.setdefault(k, []).append(v)
    eng.profile(0)
    status = eng.device_status()
    if status != 0:
        raise SystemExit(f"device status word 0x{status:x}: a kernel wait ran out")
    counts = eng.last_expert_counts()

    # end to end through the host-buffer entry point
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        for layer in range(wl["L"]):
            eng.forward_host(layer, x_host, out_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for layer in range(wl["L"]):
            eng.forward_host(layer, x_host, out_host)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps

    ms_step = ms_total / args.steps
    if dist is not None:
        tt = torch.tensor([ms_step, e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_step, e2e_s = float(tt[0]), float(tt[1])
    # every rank releases its handle at the same point: destroying the library's
    # NCCL communicator is collective
    counts_dev_bytes = eng.device_bytes()
    if dist is not None:
        dist.barrier()
    eng.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    value = tokens_per_step_job / (ms_step * 1e-3)
    peaks = load_peaks()
    H, I, K = shape.hidden, shape.intermediate, shape.top_k
    rows_local = sum(counts)  # rows this rank's gate/up GEMM processed in the last call
    g1_ms = statistics.mean(stage_ms.get("gemm1", [0.0])) if stage_ms else 0.0
    if wl["bound"] == "tensor":
        alg = 2.0 * rows_local * (2 * I) * H  # flops of one gate/up launch on this rank
        achieved = alg / (g1_ms * 1e-3) / 1e12 if g1_ms > 0 else None
        peak, unit = peaks["bf16_tflops"], "TFLOP/s"
    else:
        active = sum(1 for c in counts if c > 0)
        alg = active * ((2 * I * H) // 2 + (2 * I * H) // 32 + 2 * I * 4) + rows_local * H * 2 \
            + rows_local * I * 2  # packed W1 + scales + bias, rows in, h out
        achieved = alg / (g1_ms * 1e-3) / 1e9 if g1_ms > 0 else None
        peak, unit = peaks["hbm_gbs"], "GB/s"
    # the library picks the kernel from the rows per local expert (pick_bn in csrc/moe_b200.cu)
    small = (T_local * K) // max(eng.n_local, 1) <= 96
    kernel = {capi.GEMM_MMA_SYNC: "expert_gemm_mma_kernel<0>",
              capi.GEMM_TCGEN05_1CTA: "tc5::swp::expert_gemm_swap_kernel<0>" if small
              else "tc5::expert_gemm_tc5_kernel<0,256>",
              capi.GEMM_TCGEN05: "tc5::swp::expert_gemm_swap_kernel<0>" if small
              else "tc5::pair::expert_gemm_pair_kernel<0>"}[gemm_impl]
    roofline = {"kernel": kernel + " (gate/up GEMM + SwiGLU)",
                "bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": unit,
                "frac": (achieved / peak) if achieved else None, "peak_source": peaks["source"],
                "traffic": NCU_TRAFFIC.get(args.workload), "launch_ms": g1_ms,
                "algorithmic_per_launch": alg}
    flops_step = synth.moe_flops(tokens_per_step_job, shape) * wl["L"]
    whole = {"tflops": flops_step / (ms_step * 1e-3) / 1e12,
             "frac_of_bf16_peak": flops_step / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    if wl["bound"] == "hbm":
        b = synth.moe_decode_bytes(T_local, shape, sum(1 for c in counts if c > 0)) * wl["L"] * world
        whole.update({"gbs": b / (ms_step * 1e-3) / 1e9,
                      "frac_of_hbm_peak": b / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]})

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        tps, dt, cpu = cpu_reference_run(wl, shape, steps=2, warmup=1, sample_tokens=args.cpu_sample)
        if wl["L"] > 1:
            cpu["value"] = tps / wl["L"]
            cpu["sample"] += f"; reported per {wl['L']}-layer step"

    if ep > 1:
        config["ep_exchange"] = args.ep_exchange
    config.update({"parallelism": (f"ep{ep}" if ep > 1 else ("single" if world == 1 else f"replicas{world}")),
                   "tokens_per_rank": T_local, "experts_per_rank": eng.n_local,
                   "gemm_impl": {capi.GEMM_TCGEN05: "tcgen05", capi.GEMM_MMA_SYNC: "mma_sync",
                                 capi.GEMM_TCGEN05_1CTA: "tcgen05_1cta"}[gemm_impl],
                   "expert_rows_max_over_mean": (max(counts) / (sum(counts) / len(counts))) if sum(counts) else None})
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "roofline": roofline, "whole_step": whole, "cpu_baseline": cpu,
        "e2e": {"value": tokens_per_step_job / e2e_s, "unit": "tokens/s",
                "h2d_bytes_per_step": T_local * H * 2 * wl["L"] * world,
                "d2h_bytes_per_step": T_local * H * 4 * wl["L"] * world},
        "gpu_launches": launches_per_step * args.steps,
        "stage_ms": {k: statistics.mean(v) for k, v in stage_ms.items()},
        "clocks": clocks,
    }
    line["device_bytes_per_gpu"] = counts_dev_bytes
    print(json.dumps(line))


if __name__ == "__main__":
    main()
