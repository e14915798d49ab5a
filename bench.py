"""Benchmark of the hot path: GPT-2-small-shape greedy static decode on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json config 3): 12 layers, d_model 768, 12 heads, d_ff 3072, vocab 50257, fp32,
batch 32, static length 256 = 128 prompt tokens + 128 generated; weights ~N(0, 0.02) and prompt ids
uniform in [1, vocab) from a fixed seed (synthetic stand-ins: no dataset is involved).  Decode is the
reference's full-recompute loop (no KV cache): one STEP = rebuild the [B,1,T,T] mask, run the whole
graph on the [B,256] token buffer, argmax of one logits row, write the next token — 32 tokens per
step and per GPU.  K defaults to 128 steps (one complete decode), W to 3.

`value`   tokens/s with everything resident in HBM: mask kernel + captured CUDA Graph + argmax kernel
          per step, no host synchronisation inside the timed region (CUDA events, max over ranks).
`e2e`     the reference-shaped call with HOST buffers: every step builds the mask on the host, copies
          tokens + mask host->device from pinned memory through fxf_engine_run_host, runs the
          forward and the argmax, and reads the token buffer back device->host.
Inputs exceed L2 (weights 0.65 GB + 1.65 GB of logits written per step), so no explicit L2 flush.
N > 1: every rank runs an independent batch-32 replica (sequences are independent; no collective).
`--impl reference` times the reference's CPU backend arithmetic (its own compiled CPU kernels when
`oracle/_ref` is built, else the restated oracle) on the host cores, on a reduced batch per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

B, T, PROMPT = 32, 256, 128
METRIC = "gpt2_small_greedy_decode_tokens_per_s"
# DRAM bytes (read + written) of the dominant kernel's launches in ONE forward, from an ncu capture of
# this workload (profiles/decode_step_gpt2_small_b32_launch_list.md); bench.py cannot run ncu itself.
NCU_DRAM_BYTES_PER_FORWARD = {"gemm_tf32x3_tcgen05": (6591865088, 49)}
CPU_BUDGET_S = 150.0  # wall-clock budget of a CPU arm; the per-step batch is sized to fit it


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def build_graph_file(batch: int, tmpdir: str) -> str:
    from fxfusion_b200 import lowering, wire
    cfg = lowering.GPT2_SMALL
    g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=batch, seq=T, name=f"gpt2_small_b{batch}")
    path = os.path.join(tmpdir, f"{g.name}.bin")
    wire.dump(g, path)
    return path


def pick_cpu_batch(steps: int, warmup: int) -> int:
    """Largest power-of-two batch <= 32 whose (steps + warmup) decode steps fit CPU_BUDGET_S, from a
    one-step calibration at batch 2 (bigger batches cost ~2.2x more per sequence: the 1.65 GB logits
    tensor falls out of cache)."""
    _, s_per_step, _, _ = cpu_decode_steps(2, 1, 1)
    per_seq = s_per_step / 2 * 2.2
    b = 32
    while b > 1 and (steps + warmup) * per_seq * b > CPU_BUDGET_S:
        b //= 2
    return b


def cpu_decode_steps(batch: int, steps: int, warmup: int):
    """Reference CPU backend: graph walked node by node through the reference's CPU kernels."""
    import torch
    from fxfusion_b200 import lowering, wire
    from oracle.graph_oracle import KERNELS, GraphOracle, make_static_buffer, static_decoder_mask
    from oracle.ref_cpu.build import load as load_ref
    cfg = lowering.GPT2_SMALL
    graph = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=batch, seq=T, name="cpu")
    ref = load_ref()
    kernels, kind = None, "port"
    if ref is not None:
        def bind(op):
            def fn(reg, i, o, ints, floats):
                ref.call(op, [t if t is not None else torch.empty(0) for t in reg], list(i), list(o), list(ints), list(floats))
            return fn
        kernels, kind = {op: bind(op) for op in KERNELS}, "reference"
    orc = GraphOracle(graph, kernels=kernels)
    tokens = torch.from_numpy(lowering.decode_prompt(batch, PROMPT, cfg.vocab))
    buf = make_static_buffer(tokens, T)
    cur = PROMPT

    def step():
        nonlocal cur
        logits = orc.run([buf, static_decoder_mask(buf, cur)])[0]
        buf[:, cur] = logits[:, cur - 1, :].argmax(-1)
        cur = cur + 1 if cur + 1 < T else PROMPT

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return batch * steps / dt, dt / steps, kind, torch.get_num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = pick_cpu_batch(args.steps, args.warmup)
    tps, s_per_step, kind, cores = cpu_decode_steps(batch, args.steps, args.warmup)
    sample = f"{args.steps} full-recompute decode steps of the same model at batch {batch} (of {B}), seq {T}"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": s_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "GPT-2-small-shape greedy static decode, batch 32, 128 prompt + 128 generated, fp32, full recompute",
                   "cpu_step_batch": batch},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    from fxfusion_b200 import _lib, lowering, wire
    from fxfusion_b200.engine import ExecutionEngine
    import ctypes as C

    K, W = args.steps, max(args.warmup, 3)
    cfg = lowering.GPT2_SMALL
    tmp = tempfile.TemporaryDirectory()
    # layout: independent replicas (default), or tensor-parallel groups of 2 / 4 GPUs (12 heads do not divide by 8)
    tp_size, comm = 1, None
    if args.parallel == "tp" and world > 1:
        from fxfusion_b200.tp import Communicator
        tp_size = 4 if world % 4 == 0 else 2 if world % 2 == 0 else 1
        groups = [list(range(g * tp_size, (g + 1) * tp_size)) for g in range(world // tp_size)]
        handles = [dist.new_group(ranks=r) for r in groups]
        mine = rank // tp_size
        comm = Communicator.from_process_group(local, ranks=groups[mine], group=handles[mine]) if tp_size > 1 else None
    dp_size = world // tp_size
    dp_rank = rank // tp_size
    graph_path = build_graph_file(B, tmp.name)
    eng = ExecutionEngine(graph_path, f"cuda:{local}", precision=args.precision, comm=comm, shard_output=comm is not None)
    lib = _lib.lib()
    prompt = torch.from_numpy(lowering.decode_prompt(B, PROMPT, cfg.vocab, seed=dp_rank))
    start_buf = torch.zeros((B, T), dtype=torch.int64)
    start_buf[:, :PROMPT] = prompt
    tok_slot, mask_slot = eng.input_slots()
    logits = eng.outputs()[0]
    V = logits.shape[-1]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    h = eng.handle

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: device-resident loop ----------------------------------------------------------
    state = {"cur": PROMPT}

    def device_step():
        cur = state["cur"]
        _lib.check(lib.fxf_decode_build_mask(C.c_void_p(tok_slot.data_ptr()), C.c_void_p(mask_slot.data_ptr()), B, T, cur, 0, stream))
        _lib.check(lib.fxf_engine_run(h, (C.c_void_p * 2)(tok_slot.data_ptr(), mask_slot.data_ptr()), 2, stream))
        _lib.check(lib.fxf_engine_argmax_scatter(h, C.c_void_p(tok_slot.data_ptr()), cur, stream))
        state["cur"] = cur + 1 if cur + 1 < T else PROMPT

    tok_slot.copy_(start_buf)
    for _ in range(W):
        device_step()
    tok_slot.copy_(start_buf)
    state["cur"] = PROMPT
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K):
        device_step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    status = eng.device_status()
    generated = tok_slot.cpu()

    # ---- e2e: host buffers every step -------------------------------------------------------
    Ke = min(K, 32)
    host_tok = torch.zeros((B, T), dtype=torch.int64).pin_memory()
    host_mask = torch.zeros((B, 1, T, T), dtype=torch.bool).pin_memory()
    causal = torch.tril(torch.ones((T, T), dtype=torch.bool))
    ar = torch.arange(T)

    def host_step(cur):
        # the reference's mask rule, on the host (layers/masks.py:141-154)
        torch.logical_and(((ar < cur).view(1, 1, 1, T) & (host_tok != 0).view(B, 1, 1, T)), causal, out=host_mask)
        eng.run_host([host_tok.numpy(), host_mask.numpy().view(np.uint8)])
        _lib.check(lib.fxf_engine_argmax_scatter(h, C.c_void_p(tok_slot.data_ptr()), cur, stream))
        host_tok.copy_(tok_slot, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    host_tok.copy_(start_buf)
    for i in range(3):
        host_step(PROMPT + i)
    host_tok.copy_(start_buf)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(Ke):
        host_step(PROMPT + i)
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3 if world == 1 else 0.0)
    e2e_match = bool(torch.equal(host_tok[:, :PROMPT + Ke], generated[:, :PROMPT + Ke])) if K >= Ke else None

    # ---- opt-in loop: vocabulary projection only on the row the loop reads (whole 128-step decode) -----
    lr_ms, lr_match = None, None
    if eng.supports_last_row and not args.no_extras:
        lr_buf = start_buf.cuda()
        warm = start_buf.cuda()
        eng.decode_static(warm, T - 3, last_row_only=True)
        barrier()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        eng.decode_static(lr_buf, PROMPT, last_row_only=True)
        l1.record()
        barrier()
        lr_ms = l0.elapsed_time(l1)
        n_cmp = PROMPT + min(K, T - PROMPT)
        lr_match = bool(torch.equal(lr_buf.cpu()[:, :n_cmp], generated[:, :n_cmp]))

    # ---- optional bf16 mode (one GPU only): the same 128-step decode with bf16 tensor-core products --------------
    bf16 = None
    if world == 1 and not args.no_extras and args.precision != "bf16":
        try:   # an extra must never cost the headline line
            eng16 = ExecutionEngine(graph_path, f"cuda:{local}", precision="bf16")
            b16 = start_buf.cuda()
            eng16.decode_static(start_buf.cuda(), T - 3)
            torch.cuda.synchronize()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            eng16.decode_static(b16, PROMPT)
            b1.record()
            torch.cuda.synchronize()
            bms = b0.elapsed_time(b1)
            n_cmp = min(K, T - PROMPT)
            same = (b16.cpu()[:, PROMPT:PROMPT + n_cmp] == generated[:, PROMPT:PROMPT + n_cmp]).float().mean().item() if n_cmp else None
            bf16 = {"value": B * (T - PROMPT) / (bms * 1e-3), "unit": "tokens/s", "ms_per_step": bms / (T - PROMPT), "steps": T - PROMPT,
                    "tokens_equal_fp32_loop_fraction": same, "device_status": eng16.device_status(),
                    "note": "optional FXF_GEMM_BF16 mode, full-contract loop; greedy tokens diverge from the fp32 path after the first near-tie, by design not the headline"}
            eng16.close()
        except Exception as exc:  # noqa: BLE001
            bf16 = {"error": str(exc)[:300]}

    # ---- opt-in incremental decode (one GPU only): single-position step graph with cached keys / values -----------
    kv = None
    if world == 1 and not args.no_extras:
        try:
            cfg3 = lowering.GPT2_SMALL
            step_graph = lowering.gpt_step_graph(cfg3, lowering.gpt_params(cfg3, 0), batch=B, max_len=T, name="c3_step")
            step_path = os.path.join(tmp.name, "c3_step.bin")
            wire.dump(step_graph, step_path)
            del step_graph
            engs = ExecutionEngine(step_path, f"cuda:{local}", precision=args.precision)
            engs.decode_cached(start_buf.cuda(), PROMPT)          # warm-up: one whole decode
            kbuf = start_buf.cuda()
            torch.cuda.synchronize()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            engs.decode_cached(kbuf, PROMPT)
            k1.record()
            torch.cuda.synchronize()
            kms = k0.elapsed_time(k1)
            n_cmp = min(K, T - PROMPT)
            same = (kbuf.cpu()[:, PROMPT:PROMPT + n_cmp] == generated[:, PROMPT:PROMPT + n_cmp]).float().mean().item() if n_cmp else None
            kv = {"value": B * (T - PROMPT) / (kms * 1e-3), "unit": "tokens/s", "ms_total": kms, "positions_fed": T - 1, "ms_per_position": kms / (T - 1),
                  "tokens_equal_full_loop_fraction": same, "device_status": engs.device_status(), "launches_per_position": engs.launches_per_run + 2,
                  "note": "opt-in fxf_decode_cached (the reference's stated future work): 255 single-position forwards, prompt positions included in the time; "
                          "not the headline, whose contract is full recompute"}
            engs.close()
        except Exception as exc:  # noqa: BLE001
            kv = {"error": str(exc)[:300]}

    # ---- max over ranks ----------------------------------------------------------------------
    if world > 1:
        t = torch.tensor([ms, e2e_ms, lr_ms or 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t[0].item(), t[1].item()
        lr_ms = t[2].item() if lr_ms is not None else None

    # one traced forward (an event after every launch).  With tensor parallelism a forward contains
    # collectives, so every rank of the group has to run it, not only the rank that reports.
    trace = None
    if rank == 0 or comm is not None:
        tok_slot.copy_(start_buf)
        eng.profile_launches()
        trace = eng.profile_launches()
    if rank == 0:
        # ---- roofline of the dominant kernel -----
        by = {}
        for r in trace:
            a = by.setdefault(r["kernel"], {"ms": 0.0, "flops": 0.0, "bytes": 0.0, "n": 0})
            a["ms"] += r["ms"]; a["flops"] += r["flops"]; a["bytes"] += r["bytes"]; a["n"] += 1
        total_ms = sum(a["ms"] for a in by.values())
        top_name, top = max(by.items(), key=lambda kv: kv[1]["ms"])
        peaks = measured_peaks()
        achieved = top["flops"] / (top["ms"] * 1e-3) / 1e12
        traffic = NCU_DRAM_BYTES_PER_FORWARD.get(top_name)
        roofline = {"bound": "tensor", "kernel": top_name, "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": (traffic[0] / traffic[1]) if traffic and traffic[1] == top["n"] else None,
                    "algorithmic_bytes": top["bytes"] / top["n"], "peak_source": peaks["source"] + " cuBLAS bf16, sustained",
                    "launches_per_step": top["n"], "share_of_step": top["ms"] / total_ms,
                    # fp32 results from three TF32 products: TF32 runs at half the bf16 rate, so the ceiling of this arithmetic
                    # on the measured scale is peak / 6 (bf16 mode: the peak itself)
                    "fp32_emulation_ceiling": None if args.precision == "bf16" else peaks["bf16_tflops_sustained"] / 6.0,
                    "frac_of_fp32_emulation_ceiling": None if args.precision == "bf16" else achieved / (peaks["bf16_tflops_sustained"] / 6.0),
                    "note": "achieved = logical fp32 flops (2MNK, counted once) of all launches of this kernel in one forward / their summed device time"}
        kernels = {k: {"launches": v["n"], "ms": round(v["ms"], 4), "share": round(v["ms"] / total_ms, 4),
                       "tflops": round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 3) if v["ms"] > 0 else None,
                       "gbs": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1) if v["ms"] > 0 else None} for k, v in sorted(by.items(), key=lambda kv: -kv[1]["ms"])}
        # per-kernel fraction of its own roofline: tensor-core kernels against the ceiling of their arithmetic on the measured
        # scale (three TF32 products per fp32 product = sustained bf16 peak / 6; the bf16 peak itself in bf16 mode), every
        # other kernel against the measured copy bandwidth with its algorithmic bytes
        tensor_ceiling = peaks["bf16_tflops_sustained"] / (1.0 if args.precision == "bf16" else 6.0)
        for k, v in kernels.items():
            if "tcgen05" in k and v["tflops"] is not None:
                v["bound"], v["frac"] = "tensor", round(v["tflops"] / tensor_ceiling, 4)
            elif v["gbs"] is not None:
                v["bound"], v["frac"] = "hbm", round(v["gbs"] / peaks["hbm_gbs"], 4)
        # ---- CPU baseline on a bounded sample -------------------------------------------------------
        cpu = None
        if not args.no_cpu_baseline:
            cb = pick_cpu_batch(2, 1)
            tps, s_per_step, kind, cores = cpu_decode_steps(cb, 2, 1)
            cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind,
                   "sample": f"2 full-recompute decode steps of the same model at batch {cb} (of {B}), seq {T}; {s_per_step:.2f} s/step"}
        tokens_per_step = B * dp_size
        line = {
            "metric": METRIC, "value": tokens_per_step * K / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak" if tp_size == 1 else "strong", "vs_baseline": None, "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": "GPT-2-small-shape greedy static decode, batch 32 per replica, 128 prompt + 128 generated, fp32, full recompute",
                       "layers": 12, "d_model": 768, "heads": 12, "d_ff": 3072, "vocab": 50257, "batch_per_gpu": B, "seq": T,
                       "parallelism": (f"{world} independent replica(s), no collective" if tp_size == 1 else
                                       f"tp{tp_size} x dp{dp_size}: heads, FeedForward hidden units and vocabulary sharded over {tp_size} GPUs, "
                                       f"2 all-reduces per layer (own peer-memory kernel over NVLink, NCCL as fallback), {dp_size} replica group(s) of batch {B}"), "gemm": args.precision,
                       "l2": "inputs larger than L2 (0.65 GB weights read, 1.65 GB logits written per step)"},
            "e2e": {"value": tokens_per_step * Ke / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * T * 8 + B * T * T,
                    "d2h_bytes_per_step": B * T * 8, "steps": Ke, "tokens_equal_device_loop": e2e_match},
            "last_row_projection": None if lr_ms is None else {
                "value": tokens_per_step * (T - PROMPT) / (lr_ms * 1e-3), "unit": "tokens/s", "ms_per_step": lr_ms / (T - PROMPT), "steps": T - PROMPT,
                "tokens_equal_full_loop": lr_match,
                "note": "opt-in fxf_decode_static_last_row: same tokens, the final Linear evaluated on 1 of 256 positions; not the headline (the graph contract's output is full logits)"},
            "bf16_mode": bf16,
            "kv_cache_decode": kv,
            "gpu_launches": K * (eng.launches_per_run + 2),
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels,
            "device_status": status, "device_bytes": eng.device_bytes,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if comm is not None:
        comm.close()
    tmp.cleanup()
    if world > 1:
        dist.destroy_process_group()


def run_micro(args):
    """One op, outside any engine, through fxf_kernel_invoke — used to profile a single kernel on a
    small case (inputs larger than L2, a few hundred MB on the device)."""
    import math
    import torch
    from fxfusion_b200.kernels import invoke
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    M, N, K = args.m, args.n, args.k
    if args.micro == "linear":
        reg = [torch.randn(M, K, generator=g).cuda(), (torch.randn(N, K, generator=g) / math.sqrt(K)).cuda(), torch.randn(N, generator=g).cuda(),
               torch.empty(M, N, device="cuda")]
        call = lambda: invoke("Linear", reg, [0, 1, 2], [3], precision=args.precision)
        flops, nbytes = 2.0 * M * N * K, 4.0 * (M * K + N * K + N + M * N)
    elif args.micro == "layernorm":
        reg = [torch.randn(M, N, generator=g).cuda(), torch.ones(N).cuda(), torch.zeros(N).cuda(), torch.empty(M, N, device="cuda")]
        call = lambda: invoke("LayerNorm", reg, [0, 1, 2], [3], ints=[1, N], floats=[1e-5])
        flops, nbytes = 8.0 * M * N, 4.0 * (2 * M * N + 2 * N)
    elif args.micro == "add":
        reg = [torch.randn(M, N, generator=g).cuda(), torch.randn(M, N, generator=g).cuda(), torch.empty(M, N, device="cuda")]
        call = lambda: invoke("Add", reg, [0, 1], [2])
        flops, nbytes = 1.0 * M * N, 12.0 * M * N
    elif args.micro == "conv":  # 3x3, stride 1, pad 1, channels-last: batch = m, channels in = out = n, height = width = k
        cl = lambda t: t.contiguous(memory_format=torch.channels_last)
        reg = [cl(torch.randn(M, N, K, K, generator=g).cuda()), (torch.randn(N, N, 3, 3, generator=g) * 0.05).cuda(), torch.zeros(N).cuda(),
               cl(torch.empty(M, N, K, K, device="cuda"))]
        call = lambda: invoke("Conv2dRelu", reg, [0, 1, 2], [3], ints=[1, 1, 1, 1, 1, 1, 1], precision=args.precision)
        flops = 2.0 * M * K * K * N * N * 9
        nbytes = 4.0 * (2 * M * N * K * K + 9 * N * N + N)
    else:  # mha: B = m, T = n, D = k, 64-wide heads
        Bm, Tm, D = M, N, K
        H = D // 64
        mask = torch.tril(torch.ones(Tm, Tm, dtype=torch.bool)).view(1, 1, Tm, Tm).expand(Bm, 1, Tm, Tm).contiguous().cuda()
        reg = [torch.randn(Bm, Tm, D, generator=g).cuda(), mask, (torch.randn(3 * D, D, generator=g) * 0.02).cuda(), torch.zeros(3 * D).cuda(),
               (torch.randn(D, D, generator=g) * 0.02).cuda(), torch.zeros(D).cuda(), torch.empty(Bm, Tm, D, device="cuda")]
        call = lambda: invoke("MHA", reg, [0, 1, 2, 3, 4, 5], [6], ints=[H, 64, D, 3 * D], floats=[8.0], precision=args.precision)
        flops = 2.0 * Bm * Tm * 3 * D * D + 4.0 * Bm * H * Tm * Tm * 64 + 2.0 * Bm * Tm * D * D
        nbytes = 4.0 * (2 * Bm * Tm * D + 4 * D * D) + Bm * Tm * Tm
    for _ in range(max(args.warmup, 1)):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"micro": args.micro, "m": M, "n": N, "k": K, "precision": args.precision, "ms_per_call": ms,
                      "tflops": flops / ms / 1e9, "gbs": nbytes / ms / 1e6, "note": "includes the per-call weight split of the tensor-core path"}), flush=True)


def run_latency(args):
    """Forward latency of the two small configurations (secondary metrics): c1 = MLP, 16 layers of width 512,
    batch 32; c2 = GPT 4 layers d_model 256, batch 8 x seq 64.  CUDA-Graph replay, device-resident inputs."""
    import torch
    from fxfusion_b200 import lowering, wire
    from fxfusion_b200.engine import ExecutionEngine
    torch.cuda.set_device(0)
    tmp = tempfile.TemporaryDirectory()
    if args.workload == "c5":
        nb = args.m if args.m != 8192 else 256
        g = lowering.resnet50_graph(lowering.resnet50_params(0), batch=nb, name="c5_resnet50")
        inputs = [torch.randn(nb, 3, 224, 224, generator=torch.Generator().manual_seed(0)).cuda()]
        flops = sum(2.0 * float(np_.size) for np_ in ()) or 8.2e9 * nb
        weight_bytes = 4.0 * sum(int(v.size) for v in lowering.resnet50_params(0).values())
    elif args.workload == "c4":
        cfg = lowering.TRANSFORMER_C4
        nb = args.m if args.m != 8192 else 64
        L = 256
        g = lowering.transformer_graph(cfg, lowering.transformer_params(cfg, 0), batch=nb, src_len=L, tgt_len=L, name="c4_encdec")
        gen = torch.Generator().manual_seed(0)
        inputs = [torch.randint(1, cfg.vocab, (nb, L), generator=gen).cuda(), torch.randint(1, cfg.vocab, (nb, L), generator=gen).cuda(),
                  torch.ones(nb, 1, 1, L, dtype=torch.bool).cuda(),
                  torch.tril(torch.ones(L, L, dtype=torch.bool)).view(1, 1, L, L).expand(nb, 1, L, L).contiguous().cuda()]
        M, D, F, V, H = nb * L, cfg.d_model, cfg.d_ff, cfg.vocab, cfg.heads
        attn = 4.0 * nb * H * L * L * (D // H)
        enc = cfg.enc_layers * (2.0 * M * 3 * D * D + attn + 2.0 * M * D * D + 4.0 * M * D * F)
        dec = cfg.dec_layers * (2.0 * M * 3 * D * D + attn + 2.0 * M * D * D + (2.0 * M * D * D + 2.0 * M * 2 * D * D + attn + 2.0 * M * D * D) + 4.0 * M * D * F)
        flops = enc + dec + 2.0 * M * D * V
        weight_bytes = 4.0 * sum(int(v.size) for k, v in lowering.transformer_params(cfg, 0).items() if not k.endswith(".pe"))
    elif args.workload == "c1":
        g = lowering.mlp_graph(lowering.mlp_params(16, 512, 10, seed=0), batch=32, name="c1_mlp")
        inputs = [torch.randn(32, 512, generator=torch.Generator().manual_seed(0)).cuda()]
        flops, weight_bytes = 2.0 * 32 * 512 * (512 * 15 + 10), 4.0 * (512 * 512 * 15 + 512 * 10)
    else:
        cfg = lowering.GPT_C2
        g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=8, seq=64, name="c2_gpt")
        ids = torch.from_numpy(lowering.decode_prompt(8, 64, cfg.vocab))
        inputs = [ids.cuda(), torch.tril(torch.ones(64, 64, dtype=torch.bool)).view(1, 1, 64, 64).expand(8, 1, 64, 64).contiguous().cuda()]
        flops, weight_bytes = 3.62e9, 4.0 * sum(int(np_.size) for np_ in lowering.gpt_params(cfg, 0).values())
    path = os.path.join(tmp.name, g.name + ".bin")
    wire.dump(g, path)
    eng = ExecutionEngine(path, "cuda:0", precision=args.precision)
    for _ in range(max(args.warmup, 3)):
        eng.run(inputs)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = max(args.steps, 1)
    e0.record()
    for _ in range(n):
        eng.run(inputs)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / n
    trace = eng.profile_launches()
    print(json.dumps({"workload": args.workload, "forward_us": us, "items_per_s": (inputs[0].shape[0] / us * 1e6), "nodes": eng.num_nodes, "launches": eng.launches_per_run,
                      "gflops_per_forward": flops / 1e9, "tflops": flops / us / 1e6, "weight_mb": weight_bytes / 1e6,
                      "kernels_us": {r["kernel"]: round(sum(x["ms"] for x in trace if x["kernel"] == r["kernel"]) * 1e3, 2) for r in trace}}), flush=True)
    eng.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c3", choices=["c3", "c1", "c2", "c4", "c5"],
                    help="c3 = the decode benchmark (default); c1 / c2 = forward latency of the small configs; c4 = encoder-decoder forward "
                         "(batch --m, default 64; 256 source + 256 target positions); c5 = ResNet-50 forward (batch --m, default 256)")
    ap.add_argument("--micro", default=None, choices=["linear", "layernorm", "add", "mha", "conv"], help="profile one op instead of the decode workload")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="auto", choices=["auto", "fp32_simt", "fp32_3xtf32", "bf16"],
                    help="bf16 = optional reduced-precision mode (bf16 tensor-core products, fp32 accumulation); not the headline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the opt-in last-row-projection decode measurement (keeps profiler captures short)")
    ap.add_argument("--parallel", default="replicas", choices=["replicas", "tp"],
                    help="N > 1: independent batch replicas (default) or tensor-parallel groups (head-sharded MHA, split FeedForward, NCCL all-reduce)")
    args = ap.parse_args()
    if args.micro:
        return run_micro(args)
    if args.workload != "c3":
        return run_latency(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
