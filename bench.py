"""Benchmark of the SageAttention3 hot path (pre-pass + FP4 attention) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the hot path (smoothing, NVFP4 quantization, attention) over one batch of seeded
synthetic input.  Default workload: B=4, H=32, Nq=Nk=32768, D=128, bf16, non-causal -- the configuration the
reference's headline "attention TOPS at hd128, N=32k" is quoted on.  TOPS = 4*B*H*Nq*Nk*D / time
(halved for causal), the reference's formula (bench/bench_baseline.py:31 in the reference project).

With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the whole workload on its
own (batch, head) shard with no data-path collective (weak scaling); the reported value is the units all
ranks processed divided by the slowest rank's device time.

`--impl reference` times the reference's math on the host cores instead: the torch-fp32 CPU restatement of
the reference pipeline (the reference's own kernels only execute on sm_120 hardware), on a bounded sample
of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: B, Hq, Hkv, Nq, Nk, D, causal, layout, input kwargs
    "c2_hd128_32k": dict(B=4, Hq=32, Hkv=32, Nq=32768, Nk=32768, D=128, causal=False, layout="HND",
                         inp=dict(k_offset_std=3.0)),
    "c2_hd64_32k": dict(B=4, Hq=64, Hkv=64, Nq=32768, Nk=32768, D=64, causal=False, layout="HND",
                        inp=dict(k_offset_std=3.0)),
    "c3_cogvideox": dict(B=2, Hq=48, Hkv=48, Nq=17776, Nk=17776, D=64, causal=False, layout="HND",
                         inp=dict(k_outlier_channels=4)),
    "c4_hunyuan": dict(B=1, Hq=24, Hkv=24, Nq=119056, Nk=119056, D=128, causal=False, layout="HND",
                       inp=dict(k_offset_std=2.0)),
    "c5_llama_gqa": dict(B=8, Hq=32, Hkv=8, Nq=8192, Nk=8192, D=128, causal=True, layout="NHD",
                         inp=dict(rope_base=500000.0)),
    "ncu_small": dict(B=1, Hq=16, Hkv=16, Nq=16384, Nk=16384, D=128, causal=False, layout="HND",
                      inp=dict(k_offset_std=3.0)),
    "c1_small": dict(B=1, Hq=2, Hkv=2, Nq=1024, Nk=1024, D=128, causal=False, layout="HND",
                     inp=dict(k_offset_std=3.0)),
}
NOMINAL_FP4_TFLOPS = 9000.0     # dense NVFP4, B200 datasheet
FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS = 6650.0, 1590.0


def flops_of(w) -> float:
    f = 4.0 * w["B"] * w["Hq"] * w["Nq"] * w["Nk"] * w["D"]
    return f / 2 if w["causal"] else f


def prepass_bytes_of(w) -> float:
    """Algorithmic bytes of the pre-pass: every input element read once (2 B), its code (1/2 B) and scale
    (1/16 B) written once, plus delta_s and the means in 16 bit."""
    nqp, nkp = -(-w["Nq"] // 128) * 128, -(-w["Nk"] // 128) * 128
    nq_el = w["B"] * w["Hq"] * w["Nq"] * w["D"]
    nk_el = w["B"] * w["Hkv"] * w["Nk"] * w["D"]
    b = (nq_el + 2 * nk_el) * (2 + 0.5 + 1 / 16)
    b += 2.0 * w["B"] * w["Hq"] * (nqp // 128) * nkp
    b += 2.0 * (w["B"] * w["Hkv"] * w["D"] + w["B"] * w["Hq"] * (nqp // 128) * w["D"])
    return b


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        self.t.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [x for x in sm if x > 0]
        return dict(sm_mhz=statistics.median(busy) if busy else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------------------------------
def cpu_reference_sample(w, seconds_target: float = 2.0):
    """One bounded sample of the workload on the host cores with the CPU oracle: one (batch, head) at a
    reduced sequence length.  Returns (flops, seconds, description)."""
    import torch
    from oracle import sage3_oracle as O
    n = min(w["Nq"], 4096)
    group = w["Hq"] // w["Hkv"]
    q, k, v = O.make_inputs(1, group, 1, n, n, w["D"], seed=4242, **w["inp"])
    t0 = time.perf_counter()
    O.sageattn3_oracle(q, k, v, is_causal=w["causal"])
    dt = time.perf_counter() - t0
    f = 4.0 * group * n * n * w["D"] / (2 if w["causal"] else 1)
    return f, dt, f"{group} query head(s) of one (batch, kv-head) at Nq=Nk={n}, D={w['D']}, same distributions"


def run_reference(args, w):
    """`--impl reference`: the reference's math on the host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for _ in range(max(args.warmup, 0)):
        cpu_reference_sample(w)
    tot_f, tot_t, desc = 0.0, 0.0, ""
    for _ in range(args.steps):
        f, dt, desc = cpu_reference_sample(w)
        tot_f += f
        tot_t += dt
    tops = tot_f / tot_t / 1e12
    line = dict(impl="reference", metric="attention TOPS (4*B*H*Nq*Nk*D/t) of the smooth+NVFP4-quantize+attend path", value=tops,
                unit="TOPS", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=1e3 * tot_t / args.steps,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="fp4 (e2m1 x ue4m3), fp32 accumulate", data="synthetic",
                config=dict(workload=args.workload, **{k_: w[k_] for k_ in ("B", "Hq", "Hkv", "Nq", "Nk", "D", "causal", "layout")}),
                cpu_baseline=dict(value=tops, unit="TOPS", cores=cores, kind="port", sample=desc + " per step"),
                e2e=dict(value=tops, unit="TOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


def run_ulysses(args, w, q, k, v, flops, rank, world, local, dev):
    """Strong-scaling arm: one step = all-to-all, pre-pass, attention, all-to-all on every rank."""
    import torch
    import torch.distributed as dist
    from sageattention_b200.ulysses import ring_attention, ulysses_attention
    if args.ring:        # same token shards, K / V shards travel around the ring instead of the two all-to-alls
        ulysses_attention = lambda q_, k_, v_, tensor_layout, overlap_groups: ring_attention(q_, k_, v_, tensor_layout=tensor_layout)
    stream = torch.cuda.current_stream()
    hkv_l = w["Hkv"] // world
    groups = max(1, min(args.overlap_groups if args.overlap_groups else 1, hkv_l))      # ulysses_attention's own rule
    for _ in range(max(args.warmup, 3)):
        ulysses_attention(q, k, v, tensor_layout=w["layout"], overlap_groups=groups)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dist.barrier()
    torch.cuda.synchronize()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        ulysses_attention(q, k, v, tensor_layout=w["layout"], overlap_groups=groups)
    b_.record(stream)
    torch.cuda.synchronize()
    dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([a.elapsed_time(b_) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    if rank == 0:
        per_rank_bytes = 4 * (world - 1) / world * q.numel() * 2      # q, k, v out and o back, 16-bit
        print(json.dumps(dict(
            metric="attention TOPS (4*B*H*Nq*Nk*D/t) of the smooth+NVFP4-quantize+attend path", value=flops / (ms * 1e-3) / 1e12, unit="TOPS",
            n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="strong",
            vs_baseline=None, dtype="fp4 (e2m1 x ue4m3), fp32 accumulate", data="synthetic",
            config=dict(workload=args.workload, sharding=("ring attention: K/V shards sent around the ring (NCCL send/recv), partial results merged by LSE"
                                                          if args.ring else "ulysses sequence parallel: NCCL all-to-all before and after attention"),
                        tokens_per_rank=q.shape[2] if w["layout"] == "HND" else q.shape[1], heads_per_rank=w["Hq"] // world,
                        all_to_all_bytes_per_rank_per_step=per_rank_bytes, head_slices_in_flight=groups,
                        l2="inputs larger than L2"),
            clocks=clocks, gpu_launches=((6 + 1) * world if args.ring else 6 * groups + 4) * args.steps)))
    dist.destroy_process_group()


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2_hd128_32k", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="sage3_b200", choices=["sage3_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ulysses", action="store_true",
                    help="strong scaling: the workload's tokens are sharded over the ranks (all-to-all before and after attention)")
    ap.add_argument("--ring", action="store_true", help="with --ulysses: ring attention instead of the all-to-all exchange")
    ap.add_argument("--overlap-groups", type=int, default=0,
                    help="with --ulysses: head slices whose all-to-all overlaps the kernels of the others (0 = one slice, no overlap)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
        return

    import torch
    import torch.distributed as dist
    from sageattention_b200 import Sage3Problem, sageattn3_offload

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL prints its version banner to stdout while the communicator is created; stdout is for the one
        # JSON line, so file descriptor 1 points at stderr until the first collective has completed
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    # seeded synthetic input, generated on the device in chunks (the full tensors are several GB)
    g = torch.Generator(device=dev).manual_seed(2000 + rank)
    B, Hq, Hkv, Nq, Nk, D = (w[k_] for k_ in ("B", "Hq", "Hkv", "Nq", "Nk", "D"))
    if args.ulysses:
        if Nq % world or Nk % world or Hq % world or Hkv % world or w["causal"]:
            raise SystemExit("--ulysses needs token and head counts divisible by the number of GPUs and a non-causal workload")
        Nq, Nk = Nq // world, Nk // world       # this rank's token shard
    shp_q = (B, Hq, Nq, D) if w["layout"] == "HND" else (B, Nq, Hq, D)
    shp_k = (B, Hkv, Nk, D) if w["layout"] == "HND" else (B, Nk, Hkv, D)
    q = torch.empty(shp_q, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    k = torch.empty(shp_k, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    v = torch.empty(shp_k, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    off_std = w["inp"].get("k_offset_std", 0.0)
    if off_std:
        off_shape = (B, Hkv, 1, D) if w["layout"] == "HND" else (B, 1, Hkv, D)
        k += (off_std * torch.randn(off_shape, device=dev, generator=g)).to(torch.bfloat16)
    if w["inp"].get("k_outlier_channels"):
        idx = torch.randperm(D, device=dev, generator=g)[: w["inp"]["k_outlier_channels"]]
        k[..., idx] *= 2
    # (RoPE of the Llama-shaped workload changes values, not shapes or timing; the parity tests cover it.)

    flops = flops_of(w)
    stream = torch.cuda.current_stream()
    if args.ulysses and world > 1:
        run_ulysses(args, w, q, k, v, flops, rank, world, local, dev)
        return
    prob = Sage3Problem(q, k, v, tensor_layout=w["layout"], is_causal=w["causal"])

    def step(ev=None):
        if ev is not None:
            ev[0].record(stream)
        prob.prepass()
        if ev is not None:
            ev[1].record(stream)
        prob.attention()
        if ev is not None:
            ev[2].record(stream)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    prob.check_status()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for i in range(args.steps):
        step(evs[i])
    t_end.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_begin.elapsed_time(t_end)
    pre_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    att_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    prob.check_status()
    if world > 1:
        t = torch.tensor([total_ms, pre_ms, att_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, pre_ms, att_ms = t.tolist()

    # end to end through the public call: pinned host tensors in, host tensor out, copies inside the timed region
    e2e = None
    if args.e2e_steps > 0:
        qh, kh, vh = (t_.cpu().pin_memory() for t_ in (q, k, v))
        oh = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        del prob
        torch.cuda.synchronize()

        def e2e_step():
            # the public call for host-resident operands: copies in, pre-pass, attention and copy out, pipelined
            # over (batch, kv-head) chunks
            sageattn3_offload(qh, kh, vh, out=oh, tensor_layout=w["layout"], is_causal=w["causal"], device=dev)

        for _ in range(3):          # warm-up: allocator, pinned pages, clocks
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(args.e2e_steps):
            e2e_step()
        b_.record(stream)
        torch.cuda.synchronize()
        e2e_ms = a.elapsed_time(b_) / args.e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = t.item()
        nbytes = lambda t_: t_.numel() * t_.element_size()
        e2e = dict(value=world * flops / (e2e_ms * 1e-3) / 1e12, unit="TOPS", ms_per_step=e2e_ms,
                   h2d_bytes_per_step=world * (nbytes(qh) + nbytes(kh) + nbytes(vh)), d2h_bytes_per_step=world * nbytes(oh))     # whole job

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    ms_per_step = total_ms / args.steps
    att_tops = flops / (att_ms * 1e-3) / 1e12
    fp4_peak = 4.0 * peaks["bf16_sustained"]          # dense FP4 is 4x dense bf16 on this part
    # DRAM traffic of one attention launch: ncu measured 159.6 MB (dram__bytes_read.sum + dram__bytes_write.sum) on
    # the ncu_small case (16 heads x 16384 tokens, D=128; profiles/attn_fwd_kernel__ncu_small.md); the kernel reads
    # each head's operands once from DRAM and writes its output once, so traffic scales with B*H*N*D.
    traffic, traffic_src = None, None
    if D == 128 and not w["causal"]:
        traffic = 159.6e6 * (B * Hq * Nq) / (16 * 16384.0)
        traffic_src = "scaled from one ncu capture of the ncu_small case in proportion to B*H*N"
    line = dict(
        metric="attention TOPS (4*B*H*Nq*Nk*D/t) of the smooth+NVFP4-quantize+attend path", value=world * flops / (ms_per_step * 1e-3) / 1e12,
        unit="TOPS", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms_per_step, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="fp4 (e2m1 x ue4m3), fp32 accumulate", data="synthetic",
        config=dict(workload=args.workload, B=B, Hq=Hq, Hkv=Hkv, Nq=Nq, Nk=Nk, D=D, causal=w["causal"], layout=w["layout"],
                    in_dtype="bf16", l2="inputs larger than L2 (3.2 GB of q/k/v per step)" if flops > 1e12 else "small case, L2 resident",
                    sharding="independent (batch, head) shards per rank, no collective"),
        attn_kernel=dict(ms=att_ms, tops=att_tops), prepass=dict(ms=pre_ms, gbs=prepass_bytes_of(w) / (pre_ms * 1e-3) / 1e9,
                                                                 frac_of_hbm_peak=prepass_bytes_of(w) / (pre_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                                                 algorithmic_bytes=prepass_bytes_of(w)),
        roofline=dict(bound="tensor", kernel="attn_fwd_kernel", achieved=att_tops, peak=fp4_peak, unit="TFLOP/s", frac=att_tops / fp4_peak,
                      traffic=traffic, traffic_source=traffic_src, peak_source=f"4 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']})",
                      frac_of_nominal_fp4=att_tops / NOMINAL_FP4_TFLOPS),
        clocks=clocks, e2e=e2e, gpu_launches=6 * args.steps,
    )
    if not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        tot_f = tot_t = 0.0
        desc = ""
        t_start = time.perf_counter()
        while time.perf_counter() - t_start < 12.0:
            f, dt, desc = cpu_reference_sample(w)
            tot_f += f
            tot_t += dt
        line["cpu_baseline"] = dict(value=tot_f / tot_t / 1e12, unit="TOPS", cores=cores, kind="port",
                                    sample=f"{desc}; repeated for {tot_t:.1f} s")
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
