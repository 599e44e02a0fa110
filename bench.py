#!/usr/bin/env python
"""Throughput of the LoRA training step on the frozen quantised linears (trained tokens/s).

    python bench.py --gpus N --steps K --warmup W            # the CUDA path (this repository)
    python bench.py --impl reference --steps K --warmup W    # the CPU algorithm of the reference

One step = zero_grad + forward + backward over the local batch (+ one all-reduce of the flat
LoRA-gradient buffer when N > 1) + gradient clipping + AdamW, i.e. one iteration of the
reference's Trainer::run loop (src/train.rs:316-381).  Prints ONE JSON line on rank 0.
Model.checkpointing (src/model.rs:299) is on for the headline number, as the workload states and
as the CPU arm runs it: each block's forward runs again before its backward.  The library's own
default keeps every block's caches when they fit in device memory (here 12.6 GB); that variant
of the same step is timed in the same run and reported as `keep_caches`.

The headline workload: a synthetic Qwen3-0.6B-shaped GGUF model (28 layers, hidden 1024, 16 Q /
8 KV heads of 128, SwiGLU 3072, vocabulary 151 936, tied) with Q8_0 weights, 16 sequences x 512
uniform-random ids per GPU, loss on the last 30 % of each sequence, LoRA r=16 alpha=32 on the
seven projections, warm-up 2 + cosine LR.  For N > 1 every rank holds a replica; the global batch
is N x 16 sequences dealt round-robin (weak scaling), every target weighted with the GLOBAL
1/batch_tokens, and the ranks' gradient buffers are summed by the library's own NCCL all-reduce
(rt_model_allreduce_grads).  Before the timed region a fixed global batch is run both sharded
over the N ranks and whole on every rank, and the two gradients are compared (`dp_check`); after
it, the fixed-global-batch workload (Qwen2.5-0.5B shape, 32 x 1024, every position a target) is
timed at this N (`strong`).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the headline: Qwen3-0.6B shape, Q8_0, 16 x 512 per GPU, recomputation on
    "qwen3-0.6b-q8_0-16x512": dict(preset="qwen3-0.6b", quant="Q8_0", n_seq=16, seq_len=512, answer_frac=0.30, rank=16,
                                   alpha=32.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=2, lr_total=20, min_ratio=0.1),
    # the reference's own CPU-runnable case: the same shape in Q4_0, 4 x 256, one AdamW step
    "qwen3-0.6b-q4_0-4x256": dict(preset="qwen3-0.6b", quant="Q4_0", n_seq=4, seq_len=256, answer_frac=0.50, rank=16,
                                  alpha=32.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=0, lr_total=1, min_ratio=0.1),
    # Qwen2.5-0.5B shape (24 layers, hidden 896, 14 Q / 2 KV heads of 64, q/k/v bias), Q4_K where the row length allows it (ffn_down), Q4_0 elsewhere,
    # every position a target
    "qwen2.5-0.5b-q4_k-32x1024": dict(preset="qwen2.5-0.5b", quant="Q4_K", n_seq=32, seq_len=1024, answer_frac=1.0, rank=8,
                                      alpha=16.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=2, lr_total=20, min_ratio=0.1),
    # Llama-3.2-3B shape, Q6_K, every position a target (per GPU: 16 x 2048)
    "llama-3.2-3b-q6_k-16x2048": dict(preset="llama-3.2-3b", quant="Q6_K", n_seq=16, seq_len=2048, answer_frac=1.0, rank=16,
                                      alpha=32.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=2, lr_total=20, min_ratio=0.1),
    # Qwen3-4B shape, Q4_0, r = 32, last 25 % targets: the 64 x 2048 batch at its 8-GPU share
    "qwen3-4b-q4_0-8x2048": dict(preset="qwen3-4b", quant="Q4_0", n_seq=8, seq_len=2048, answer_frac=0.25, rank=32,
                                 alpha=64.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=2, lr_total=50, min_ratio=0.1),
    # two layers of the headline model (the same per-layer shapes and token count, about 1 GB on the device):
    # the case the per-kernel profiler captures run on
    "qwen3-0.6b-q8_0-16x512-2layers": dict(preset="qwen3-0.6b", quant="Q8_0", n_seq=16, seq_len=512, answer_frac=0.30, rank=16,
                                           alpha=32.0, lr=1e-4, wd=0.01, clip=1.0, lr_warmup=2, lr_total=20, min_ratio=0.1,
                                           n_layers=2),
    # small shape for quick checks of this script
    "tiny": dict(preset="tiny-qwen3", quant="Q8_0", n_seq=4, seq_len=64, answer_frac=0.5, rank=8, alpha=16.0, lr=1e-4,
                 wd=0.01, clip=1.0, lr_warmup=2, lr_total=20, min_ratio=0.1),
}
DEFAULT_WORKLOAD = "qwen3-0.6b-q8_0-16x512"
STRONG_WORKLOAD = "qwen2.5-0.5b-q4_k-32x1024"  # fixed GLOBAL batch, split over the ranks


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops=float(p["bf16_tflops_sustained"]), hbm=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1400.0, hbm=6650.0, source="fallback")


def make_batch(spec, wl, seed):
    from rust_trainer_b200 import synth

    toks = synth.token_batch(spec, wl["n_seq"], wl["seq_len"], seed)
    answer_start = int(np.ceil(wl["seq_len"] * (1.0 - wl["answer_frac"])))
    tps, tts = [], []
    for s in range(wl["n_seq"]):
        tp, tt = synth.answer_targets(toks[s], answer_start)
        tps.append(tp + s * wl["seq_len"])
        tts.append(tt)
    return toks, np.concatenate(tps), np.concatenate(tts), answer_start


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(smax) if smax else None,
                    reasons=sorted(reasons), samples=len(sm))


# ----------------------------------------------------------------------------- reference arm (CPU)
CPU_SAMPLE_TOKENS = 128  # the same bounded sample whatever --steps says


def cpu_reference_run(wl_name: str, steps: int, warmup: int):
    """Times the CPU restatement of the reference's algorithm (oracle/) on a bounded sample of
    the workload: ONE sequence of 128 ids of the same model, same LoRA shape, loss on the same
    trailing fraction, forward + recompute + backward + clip + AdamW per step, on every host core
    (a launcher's OMP_NUM_THREADS=1 is overridden)."""
    from oracle import oracle as O
    from rust_trainer_b200 import synth

    wl = WORKLOADS[wl_name]
    cores = O.set_num_threads(os.cpu_count() or 1)
    spec = synth.preset(wl["preset"], quant=wl["quant"], seed=0)
    tensors = synth.build_tensors(spec)
    om = O.OracleModel(spec.config(), tensors)
    om.attach_lora(synth.lora_adapters(spec, wl["rank"], wl["alpha"], seed=1234))
    sample_tokens = min(CPU_SAMPLE_TOKENS, wl["seq_len"])
    toks = synth.token_batch(spec, 1, sample_tokens, 99)[0]
    a0 = int(np.ceil(sample_tokens * (1.0 - wl["answer_frac"])))
    tp, tt = synth.answer_targets(toks, a0)
    w = np.full(tp.size, 1.0 / tp.size, np.float32)
    state = {}
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        om.zero_grad()
        om.forward_backward(toks, tp, tt, w)
        om.clip_grad_norm(wl["clip"])
        om.adamw_step(state, wl["lr"], wd=wl["wd"])
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    ms = 1e3 * float(np.mean(times))
    return dict(value=sample_tokens / (ms / 1e3), ms_per_step=ms, cores=cores,
                sample=f"1 sequence x {sample_tokens} tokens of the same model per step (loss on the last "
                       f"{int(wl['answer_frac'] * 100)} %), forward + recompute + backward + clip + AdamW"), spec


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return 0  # under a multi-rank launcher rank 0 alone runs the CPU arm
    wl = WORKLOADS[args.workload]
    # a few steps are enough for a CPU loop without caches to warm; bounded so the arm ends in about a minute
    steps, warmup = min(args.steps, 5), min(args.warmup, 1)
    r, spec = cpu_reference_run(args.workload, steps, warmup)
    line = {
        "impl": "reference", "metric": "trained_tokens_per_s", "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "model": wl["preset"], "quant": wl["quant"], "lora_rank": wl["rank"],
                   "note": "CPU restatement of the reference algorithm (oracle/), not the reference binary: no Rust "
                           "toolchain and rie-core is not vendored"},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------- CUDA arm
class StepRunner:
    """One replica of one workload on this rank's GPU: the local share of a global batch staged in
    HBM (or passed from pinned host buffers for the end-to-end arm), and the step around it."""

    def __init__(self, rt, ctx, wl, world, rank, checkpointing):
        from rust_trainer_b200 import dp, synth

        self.rt, self.ctx, self.wl, self.world, self.rank = rt, ctx, wl, world, rank
        over = {"n_layers": wl["n_layers"]} if "n_layers" in wl else {}
        self.spec = synth.preset(wl["preset"], quant=wl["quant"], seed=0, **over)
        tensors = synth.build_tensors(self.spec)
        self.model = rt.Model(ctx, self.spec.config(), tensors)
        self.n_params = self.model.attach_lora(wl["rank"], wl["alpha"], None, 1234)
        self.model.load_adapters(synth.lora_adapters(self.spec, wl["rank"], wl["alpha"], seed=1234))
        del tensors
        self.model.set_checkpointing({"on": 1, "off": 0, "auto": -1}[checkpointing])
        self.step_no = 0
        self.dp = dp

    def global_examples(self, n_seq_global, seed):
        from rust_trainer_b200 import synth

        wl = self.wl
        toks = synth.token_batch(self.spec, n_seq_global, wl["seq_len"], seed)
        self.answer_start = int(np.ceil(wl["seq_len"] * (1.0 - wl["answer_frac"])))
        return [(toks[i], self.answer_start) for i in range(n_seq_global)]

    def set_batch(self, examples, rank, world):
        """This rank's round-robin share of `examples` with the global 1/batch_tokens weights, in
        pinned host buffers."""
        import torch

        b = self.dp.local_batch(examples, rank, world)
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a).copy()).pin_memory().numpy()
        self.batch = b
        self.h_toks = pin(np.concatenate(b.seqs))
        offs = np.zeros(len(b.seqs) + 1, np.int32)
        offs[1:] = np.cumsum([s.size for s in b.seqs])
        self.h_offs, self.h_tpos, self.h_ttok, self.h_w = pin(offs), pin(b.target_pos), pin(b.target_tok), pin(b.weights)
        self.h_logp = torch.empty(b.target_pos.size, dtype=torch.float32).pin_memory().numpy()
        self.local_tokens = int(self.h_toks.size)

    def stage(self):
        L, m = self.L, self.model
        self.ctx.check(L.rt_model_stage_batch(m._h, _ip(self.h_toks), _ip(self.h_offs), len(self.batch.seqs), _ip(self.h_tpos),
                                              _ip(self.h_ttok), _fp(self.h_w), self.h_tpos.size))

    @property
    def L(self):
        from rust_trainer_b200._lib import lib

        return lib()

    def lr_now(self):
        wl = self.wl
        return self.rt.schedule_lr(wl["lr"], wl["lr_warmup"], wl["lr_total"], wl["min_ratio"], self.step_no % wl["lr_total"])

    def finish_step(self):
        self.model.allreduce_grads()  # sum over ranks on the ctx stream (nothing to do in a world of one)
        self.model.optim_step(self.lr_now(), self.wl["clip"], weight_decay=self.wl["wd"])
        self.step_no += 1

    def step_resident(self):
        self.model.zero_grad()
        self.ctx.check(self.L.rt_model_run_staged(self.model._h, 1))
        self.finish_step()

    def step_e2e(self):
        """The call a host makes: tokens, targets and weights from (pinned) host memory in, per-target
        log-probabilities back out, every step."""
        self.model.zero_grad()
        hits = C.c_int32()
        self.ctx.check(self.L.rt_model_forward_backward(self.model._h, _ip(self.h_toks), _ip(self.h_offs), len(self.batch.seqs),
                                                        _ip(self.h_tpos), _ip(self.h_ttok), _fp(self.h_w), self.h_tpos.size,
                                                        _fp(self.h_logp), C.byref(hits)))
        loss = self.dp.step_loss(self.h_logp, self.batch)
        self.finish_step()
        return loss

    def grads(self):
        return np.concatenate([np.concatenate([lo["ga"].ravel(), lo["gb"].ravel()])
                               for lo in (l.lora() for l in self.model.lora_linears())])

    def close(self):
        self.model.close()


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def dram_bytes_per_flop():
    """DRAM traffic of the frozen-matmul kernel per algorithmic flop, from the committed summary of
    its ncu capture (dram__bytes_read.sum + dram__bytes_write.sum of one launch over that launch's
    2*tokens*out*in); None when no summary of the current kernel is there."""
    path = os.path.join(ROOT, "profiles", "qgemm_kernel_dram_traffic.txt")
    try:
        for line in open(path):
            if line.startswith("dram_bytes_per_flop:"):
                return float(line.split(":", 1)[1].split()[0]), os.path.relpath(path, ROOT)
    except (OSError, ValueError):
        pass
    return None, None


def run_ours(args):
    import torch
    import rust_trainer_b200 as rt
    from rust_trainer_b200._lib import lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the CUDA path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod  # plumbing only: barriers, the max over ranks of the timings, handing out the communicator id
        dist.init_process_group("nccl", device_id=dev)
    wl = WORKLOADS[args.workload]
    L = lib()
    ctx = rt.Context(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    L.rt_ctx_set_stream(ctx._h, C.c_void_p(stream.cuda_stream))
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(rt.Context.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        ctx.comm_init_rank(world, rank, bytes(uid.cpu().numpy().tobytes()))

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        ms = max(e0.elapsed_time(e1), 0.0)
        t = torch.tensor([ms, wall], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
        return float(t[0]), float(t[1])

    run = StepRunner(rt, ctx, wl, world, rank, args.checkpointing)
    model = run.model

    # ---- N ranks on ONE global batch against one rank on the whole of it (before anything is timed)
    dp_check = None
    if world > 1:
        fixed = run.global_examples(wl["n_seq"], seed=7)
        run.set_batch(fixed, rank, world)
        model.zero_grad()
        hits = C.c_int32()
        ctx.check(L.rt_model_forward_backward(model._h, _ip(run.h_toks), _ip(run.h_offs), len(run.batch.seqs), _ip(run.h_tpos),
                                              _ip(run.h_ttok), _fp(run.h_w), run.h_tpos.size, _fp(run.h_logp), C.byref(hits)))
        loss_dp = torch.tensor([run.dp.step_loss(run.h_logp, run.batch)], dtype=torch.float64, device=dev)
        dist.all_reduce(loss_dp)
        model.allreduce_grads()
        ctx.synchronize()
        g_dp = run.grads()
        run.set_batch(fixed, 0, 1)  # the whole batch on this rank alone
        model.zero_grad()
        ctx.check(L.rt_model_forward_backward(model._h, _ip(run.h_toks), _ip(run.h_offs), len(run.batch.seqs), _ip(run.h_tpos),
                                              _ip(run.h_ttok), _fp(run.h_w), run.h_tpos.size, _fp(run.h_logp), C.byref(hits)))
        loss_one = run.dp.step_loss(run.h_logp, run.batch)
        g_one = run.grads()
        rel = float(np.linalg.norm(g_dp.astype(np.float64) - g_one) / np.linalg.norm(g_one.astype(np.float64)))
        t = torch.tensor([rel, abs(float(loss_dp[0]) - loss_one) / abs(loss_one)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dp_check = {"grad_rel_l2": float(t[0]), "loss_rel": float(t[1]), "bound": 1e-5, "ok": bool(float(t[0]) <= 1e-5),
                    "global_batch": f"{wl['n_seq']} x {wl['seq_len']}",
                    "what": "gradient buffer after the NCCL sum of N shards vs the whole batch on one rank, max over ranks"}
        model.zero_grad()

    # ---- the timed job: N x n_seq sequences dealt round-robin, inputs resident in HBM
    examples = run.global_examples(wl["n_seq"] * world, seed=100)
    run.set_batch(examples, rank, world)
    n_targets = run.h_tpos.size
    tokens_per_step = sum(int(t.size) for t, _ in examples)
    run.stage()
    for _ in range(args.warmup):
        run.step_resident()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = L.rt_ctx_launch_count(ctx._h)
    ms_total, _ = timed(run.step_resident, args.steps)
    launches = (L.rt_ctx_launch_count(ctx._h) - launches0) // max(args.steps, 1)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps

    if args.launch_list:
        if rank == 0:
            print(json.dumps({"launch_list_run": True, "ms_per_step": ms_step, "gpu_launches_per_step": int(launches),
                              "gpu_launches_before_timed": int(launches0)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end through the host-buffer call
    for _ in range(min(args.warmup, 2)):
        run.step_e2e()
    ms_e2e_total, wall_e2e = timed(run.step_e2e, args.steps)
    ms_e2e = max(ms_e2e_total, wall_e2e) / args.steps  # host copies are not all on the stream: take the slower clock

    # ---- roofline of the dominant kernel (the frozen matmul): per-launch CUDA events over profiled steps
    run.stage()
    L.rt_ctx_set_profiling(ctx._h, 1)
    prof_steps = min(args.steps, 2)
    for _ in range(prof_steps):
        run.step_resident()
    n_l, ms_l, fl, by = C.c_uint64(), C.c_double(), C.c_double(), C.c_double()
    ctx.check(L.rt_ctx_profile_read(ctx._h, C.byref(n_l), C.byref(ms_l), C.byref(fl), C.byref(by)))
    L.rt_ctx_set_profiling(ctx._h, 0)
    peaks = measured_peaks()
    achieved_tf = fl.value / (ms_l.value * 1e-3) / 1e12 if ms_l.value > 0 else 0.0
    bpf, bpf_src = dram_bytes_per_flop()
    avg_launch_flops = fl.value / max(n_l.value, 1)
    roofline = {"bound": "tensor", "achieved": achieved_tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": achieved_tf / peaks["tflops"], "traffic": None if bpf is None else bpf * avg_launch_flops,
                "traffic_source": None if bpf is None else f"{bpf_src}: ncu DRAM bytes per flop of one captured launch x flops of this run's average launch",
                "peak_source": peaks["source"] + " (sustained bf16 cuBLAS)",
                "kernel": "qgemm_kernel", "launches_per_step": int(n_l.value // prof_steps),
                "avg_launch_us": 1e3 * ms_l.value / max(n_l.value, 1), "share_of_step": (ms_l.value / prof_steps) / ms_step,
                "flops_per_step": fl.value / prof_steps}

    recompute_ran = bool(model.checkpointing)
    keep = None
    if args.checkpointing == "on":
        model.set_checkpointing(0)
        run.stage()
        for _ in range(args.warmup):
            run.step_resident()
        ms_keep, _ = timed(run.step_resident, args.steps)
        if not model.checkpointing:
            keep = {"value": tokens_per_step / (ms_keep / args.steps * 1e-3), "unit": "tokens/s", "ms_per_step": ms_keep / args.steps,
                    "what": "same step with Model.checkpointing off: every block's caches stay in HBM, no second forward"}
    n_params, lora_init = run.n_params, run.spec.describe()["lora_init"]
    h2d = run.h_toks.nbytes + run.h_offs.nbytes + run.h_tpos.nbytes + run.h_ttok.nbytes + run.h_w.nbytes + 2 * run.h_toks.size * 4
    d2h = run.h_logp.nbytes + 4 + 4
    answer_start = run.answer_start
    run.close()

    # ---- strong scaling: ONE fixed global batch split over the ranks
    strong = None
    if args.strong and args.workload == DEFAULT_WORKLOAD:
        swl = WORKLOADS[STRONG_WORKLOAD]
        if swl["n_seq"] % world == 0:
            srun = StepRunner(rt, ctx, swl, world, rank, args.checkpointing)
            sex = srun.global_examples(swl["n_seq"], seed=100)
            srun.set_batch(sex, rank, world)
            srun.stage()
            for _ in range(3):
                srun.step_resident()
            s_steps = min(args.steps, 5)
            ms_s, _ = timed(srun.step_resident, s_steps)
            stoks = swl["n_seq"] * swl["seq_len"]
            strong = {"workload": STRONG_WORKLOAD, "global_batch": f"{swl['n_seq']} x {swl['seq_len']}", "tokens_per_gpu": stoks // world,
                      "value": stoks / (ms_s / s_steps * 1e-3), "unit": "tokens/s", "ms_per_step": ms_s / s_steps, "steps": s_steps,
                      "recompute": bool(srun.model.checkpointing), "scaling": "strong"}
            srun.close()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    shapes = None
    if world == 1 and args.shape_table:
        shapes = qgemm_shape_table(rt, ctx, stream, peaks)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        r, _ = cpu_reference_run(args.workload, 1, 0)
        cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}

    line = {
        "metric": "trained_tokens_per_s", "value": tokens_per_step / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "model": wl["preset"], "quant": wl["quant"], "global_batch": wl["n_seq"] * world,
                   "seq_len": wl["seq_len"], "answer_targets_per_seq": wl["seq_len"] - answer_start, "lora_rank": wl["rank"],
                   "lora_params": n_params, "parallelism": f"dp{world}", "recompute": recompute_ran,
                   "l2": "activations and logits per step (>1 GB) exceed the 126 MB L2; no explicit flush",
                   "lora_init": lora_init, "seeds": {"weights": 0, "lora": 1234, "tokens": 100}},
        "roofline": roofline, "cpu_baseline": cpu, "keep_caches": keep,
        "e2e": {"value": tokens_per_step / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": ms_e2e},
        "gpu_launches": int(launches) * args.steps, "gpu_launches_per_step": int(launches), "clocks": clocks,
        "dp_check": dp_check, "strong": strong, "qgemm_shapes": shapes,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def qgemm_shape_table(rt, ctx, stream, peaks, token_counts=(4096, 8192), iters=10):
    """The frozen-matmul kernel alone on every projection shape of the five model configurations in
    its weight format, forward (f16 out) and backward (f32 out), CUDA events on the launching
    stream: [model, quant, dir, out, in, tokens, us, TFLOP/s, fraction of the measured peak]."""
    import torch
    from rust_trainer_b200 import quants as Q, synth
    from rust_trainer_b200._lib import lib

    L = lib()
    rng = np.random.default_rng(0)
    cases = [("qwen3-0.6b", "Q4_0"), ("qwen3-0.6b", "Q8_0"), ("qwen2.5-0.5b", "Q4_K"), ("llama-3.2-3b", "Q6_K"), ("qwen3-4b", "Q4_0")]
    rows = []
    seen = {}
    for preset, quant in cases:
        spec = synth.preset(preset, quant=quant)
        for (n, k) in sorted(set(spec.linear_shapes().values())):
            t = spec.quant_for(k)
            key = (n, k, t)
            if key not in seen:
                f = rt.Frozen(ctx, t, n, k, Q.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), t))
                res = []
                for M in token_counts:
                    x = torch.randn(M, k, device="cuda", dtype=torch.float16)
                    dy = torch.randn(M, n, device="cuda", dtype=torch.float16)
                    y = torch.empty(M, n, device="cuda", dtype=torch.float16)
                    dx = torch.empty(M, k, device="cuda", dtype=torch.float32)
                    for name, fn in (("fwd", lambda: L.rt_frozen_forward_dev(f._h, x.data_ptr(), 2, M, y.data_ptr(), 2, 0)),
                                     ("bwd", lambda: L.rt_frozen_backward_input_dev(f._h, dy.data_ptr(), 2, M, dx.data_ptr(), 0, 0))):
                        for _ in range(3):
                            ctx.check(fn())
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        for _ in range(iters):
                            ctx.check(fn())
                        e1.record(stream)
                        torch.cuda.synchronize()
                        us = 1e3 * e0.elapsed_time(e1) / iters
                        res.append((name, M, us))
                f.close()
                seen[key] = res
            for name, M, us in seen[key]:
                tf = 2.0 * M * n * k / us / 1e6
                rows.append([preset, Q.NAMES[t], name, n, k, M, round(us, 1), round(tf, 1), round(tf / peaks["tflops"], 3)])
    return {"columns": ["model", "quant", "dir", "out", "in", "tokens", "us", "tflops", "frac_of_peak"],
            "peak_tflops": peaks["tflops"], "peak_source": peaks["source"] + " (sustained bf16 cuBLAS)", "rows": rows}


def run_microbench(args):
    """Frozen-matmul kernel alone on the workload's projection shapes: forward (f16 out) and
    backward (f32 out) at `--tokens` tokens, CUDA events on the launching stream."""
    import torch
    import rust_trainer_b200 as rt
    from rust_trainer_b200 import quants as Q, synth
    from rust_trainer_b200._lib import lib

    wl = WORKLOADS[args.workload]
    spec = synth.preset(wl["preset"], quant=wl["quant"])
    L = lib()
    ctx = rt.Context(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    L.rt_ctx_set_stream(ctx._h, C.c_void_p(stream.cuda_stream))
    M = args.tokens
    rng = np.random.default_rng(0)
    peaks = measured_peaks()
    rows = []
    shapes = sorted(set(spec.linear_shapes().values()))
    if args.shape:
        n, k = (int(v) for v in args.shape.split("x"))
        shapes = [(n, k)]
    for (n, k) in shapes:
        t = spec.quant_for(k) if not args.quant else Q.BY_NAME[args.quant]
        f = rt.Frozen(ctx, t, n, k, Q.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), t))
        x = torch.randn(M, k, device="cuda", dtype=torch.float16)
        dy = torch.randn(M, n, device="cuda", dtype=torch.float16)
        y = torch.empty(M, n, device="cuda", dtype=torch.float16)
        dx = torch.empty(M, k, device="cuda", dtype=torch.float32)
        for name, fn in (("fwd", lambda: L.rt_frozen_forward_dev(f._h, x.data_ptr(), 2, M, y.data_ptr(), 2, 0)),
                         ("bwd", lambda: L.rt_frozen_backward_input_dev(f._h, dy.data_ptr(), 2, M, dx.data_ptr(), 0, 0))):
            for _ in range(3):
                ctx.check(fn())
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                ctx.check(fn())
            e1.record(stream)
            torch.cuda.synchronize()
            ctx.synchronize()
            us = 1e3 * e0.elapsed_time(e1) / args.steps
            tf = 2.0 * M * n * k / us / 1e6
            rows.append(dict(dir=name, out=n, inp=k, tokens=M, quant=Q.NAMES[t], us=us, tflops=tf, frac=tf / peaks["tflops"]))
        f.close()
    print(json.dumps({"microbench": "qgemm_kernel", "peak_tflops": peaks["tflops"], "peak_source": peaks["source"], "rows": rows}), flush=True)
    return 0


def run_attention_case(args):
    """The attention kernels alone on NSEQ sequences of T tokens (the workload's head geometry),
    through the one-op host entry points: forward, then backward.  For a profiler (the host calls
    copy their operands, so the wall time printed here is not a kernel time)."""
    import rust_trainer_b200 as rt
    from rust_trainer_b200 import ops, synth

    wl = WORKLOADS[args.workload]
    cfg = synth.preset(wl["preset"], quant=wl["quant"]).config()
    nseq, T = (int(v) for v in args.attention_case.split("x"))
    nh, nkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    M = nseq * T
    rng = np.random.default_rng(0)
    q = rng.standard_normal((M, nh, hd), dtype=np.float32)
    k = rng.standard_normal((M, nkv, hd), dtype=np.float32)
    v = rng.standard_normal((M, nkv, hd), dtype=np.float32)
    d_o = rng.standard_normal((M, nh, hd), dtype=np.float32)
    ss = np.repeat(np.arange(nseq, dtype=np.int32) * T, T)
    ctx = rt.Context(0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ops.attention(ctx, q, k, v, ss)
        ops.attention_backward(ctx, q, k, v, d_o, ss)
    ctx.synchronize()
    print(json.dumps({"attention_case": args.attention_case, "heads": nh, "kv_heads": nkv, "head_dim": hd, "steps": args.steps,
                      "host_ms_per_step_with_copies": 1e3 * (time.perf_counter() - t0) / args.steps}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--launch-list", action="store_true",
                    help="for a profiler's launch list: only the resident steps (no end-to-end, per-kernel or keep-caches "
                         "phases, fewer warm-up steps allowed); the printed number is not a bench value")
    ap.add_argument("--checkpointing", default="on", choices=["on", "off", "auto"],
                    help="Model.checkpointing for the headline number (the workload says on)")
    ap.add_argument("--no-strong", dest="strong", action="store_false",
                    help="skip the fixed-global-batch (strong scaling) workload after the headline")
    ap.add_argument("--no-shape-table", dest="shape_table", action="store_false",
                    help="skip the per-shape table of the frozen-matmul kernel (N = 1 only)")
    ap.add_argument("--microbench", action="store_true", help="time the frozen-matmul kernel alone")
    ap.add_argument("--attention-case", default="", help="NSEQxT: run the attention kernels alone (for a profiler)")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--quant", default="", help="microbench: weight format instead of the workload's")
    ap.add_argument("--shape", default="", help="microbench: one OUTxIN shape instead of the workload's")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours" and not args.launch_list:
        args.warmup = 3
    if args.attention_case:
        return run_attention_case(args)
    if args.microbench:
        return run_microbench(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
