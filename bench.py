"""Benchmark of the hot path: GPT-2-small-shape greedy static decode on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3|c1|c2|c4|c5]

Workload (BASELINE.json config 3): 12 layers, d_model 768, 12 heads, d_ff 3072, vocab 50257, fp32,
batch 32, static length 256 = 128 prompt tokens + 128 generated; weights ~N(0, 0.02) and prompt ids
uniform in [1, vocab) from a fixed seed (synthetic stand-ins: no dataset is involved).  Decode is the
reference's full-recompute loop (no KV cache): one STEP = rebuild the [B,1,T,T] mask, run the whole
graph on the [B,256] token buffer, argmax of one logits row, write the next token — 32 tokens per
step and per batch.  K defaults to 128 steps (one complete decode), W to 3.

`value`   tokens/s with everything resident in HBM: mask kernel + captured CUDA Graph + argmax kernel
          per step, no host synchronisation inside the timed region (CUDA events, max over ranks).
`e2e`     the reference-shaped call with HOST buffers: every step builds the mask on the host, copies
          tokens + mask host->device from pinned memory through fxf_engine_run_host, runs the
          forward and the argmax, and reads the token buffer back device->host.
Inputs exceed L2 (weights 0.65 GB + 1.65 GB of logits written per step), so no explicit L2 flush.
N > 1 (default `--parallel tp`): the batch-32 decode is tensor-parallel — heads, FeedForward hidden units and the
vocabulary sharded over 2 or 4 GPUs, one fused exchange kernel (sum over the ranks + residual Add + LayerNorm) after
the attention output projection and one after the second FeedForward product; 12 heads do not divide by 8, so 8 GPUs
run two tensor-parallel groups of 4, each decoding its own batch of 32.  `--parallel replicas` runs N independent
batch-32 decodes instead (no collective).
`--impl reference` times the reference's CPU backend arithmetic (its own compiled CPU kernels when
`oracle/_ref` is built, else the restated oracle) on all host cores, on a reduced batch per step.
`--workload c1|c2|c4|c5` measures the other configurations (forward only) with the same kinds of evidence; the default
run folds their one-line results into `secondary`.
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
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel's launches in ONE forward of this
# workload on one GPU, summed over an ncu capture of a forward; bench.py cannot run ncu itself.
NCU_DRAM_BYTES_PER_FORWARD = {"gemm_tf32_bf16x2_tcgen05": (7092533248, 49),   # default arithmetic
                              "gemm_tf32x3_tcgen05": (7035996416, 49)}        # --precision fp32_3xtf32
CPU_BUDGET_S = 150.0  # wall-clock budget of a CPU arm; the per-step batch is sized to fit it
NVLINK_GBS_PER_DIRECTION = 770.0  # measured peer copy on this pool's B200s (nominal 900)


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
        return self

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


def layout(world: int, parallel: str):
    """(tp_size, dp_size) of an N-GPU run: tensor-parallel groups of 4 or 2 GPUs (12 heads divide by 2 and 4, not by 8)."""
    if parallel == "replicas" or world <= 1:
        return 1, max(world, 1)
    tp = 4 if world % 4 == 0 else 2 if world % 2 == 0 else 1
    return tp, world // tp


def workload_config(world: int, parallel: str, precision: str):
    """The `config` object of the c3 line; both arms (ours and --impl reference) print the same one."""
    tp, dp = layout(world, parallel)
    if tp == 1:
        par = f"{dp} independent batch-{B} replica(s), no collective"
    else:
        par = (f"tp{tp} x dp{dp}: heads, FeedForward hidden units and vocabulary sharded over {tp} GPUs, one fused exchange kernel "
               f"(sum over ranks + residual Add + LayerNorm, peer memory over NVLink) after each of the two row-parallel products of a layer, "
               f"{dp} group(s) of batch {B}")
    return {"workload": "GPT-2-small-shape greedy static decode, batch 32, 128 prompt + 128 generated, fp32, full recompute",
            "layers": 12, "d_model": 768, "heads": 12, "d_ff": 3072, "vocab": 50257, "batch": B, "global_batch": B * dp, "seq": T,
            "parallelism": par, "gemm": precision, "l2": "inputs larger than L2 (0.65 GB weights read, 1.65 GB logits written per step)"}


def use_all_host_cores() -> int:
    """A launcher may export OMP_NUM_THREADS=1 (torch.distributed.run does); the CPU arms use every core."""
    import torch
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0)) or n
    except AttributeError:
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def build_graph_file(batch: int, tmpdir: str) -> str:
    from fxfusion_b200 import lowering, wire
    cfg = lowering.GPT2_SMALL
    g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=batch, seq=T, name=f"gpt2_small_b{batch}")
    path = os.path.join(tmpdir, f"{g.name}.bin")
    wire.dump(g, path)
    return path


def reference_kernels():
    """Kernel table for the CPU arms: the reference's own compiled CPU kernels where `oracle/_ref` is built (this library's
    extension opcodes, for which the reference has no kernel, stay with the restated oracle), else the restated oracle
    alone.  Returns (table or None, kind)."""
    import torch
    from oracle.graph_oracle import KERNELS
    from oracle.ref_cpu.build import load as load_ref
    ref = load_ref()
    if ref is None:
        return None, "port"

    def bind(op):
        def fn(reg, i, o, ints, floats):
            ref.call(op, [t if t is not None else torch.empty(0) for t in reg], list(i), list(o), list(ints), list(floats))
        return fn
    table = dict(KERNELS)
    for op in KERNELS:
        if op <= 19:   # opcodes of the reference schema
            table[op] = bind(op)
    return table, "reference"


def cpu_decode_steps(batch: int, steps: int, warmup: int):
    """Reference CPU backend: the c3 graph walked node by node through the reference's CPU kernels, on the first `batch`
    sequences of the benchmark's prompts.  Returns (tokens/s, s/step, kind, threads, token buffer after all steps)."""
    import torch
    from fxfusion_b200 import lowering
    from oracle.graph_oracle import GraphOracle, make_static_buffer, static_decoder_mask
    cores = use_all_host_cores()
    cfg = lowering.GPT2_SMALL
    graph = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=batch, seq=T, name="cpu")
    kernels, kind = reference_kernels()
    orc = GraphOracle(graph, kernels=kernels)
    tokens = torch.from_numpy(lowering.decode_prompt(B, PROMPT, cfg.vocab))[:batch]
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
    return batch * steps / dt, dt / steps, kind, cores, buf.clone()


def pick_cpu_batch(steps: int, warmup: int) -> int:
    """Largest power-of-two batch <= 32 whose (steps + warmup) decode steps fit CPU_BUDGET_S, from a
    one-step calibration at batch 2 (bigger batches cost ~2.2x more per sequence: the 1.65 GB logits
    tensor falls out of cache)."""
    s_per_step = cpu_decode_steps(2, 1, 1)[1]
    per_seq = s_per_step / 2 * 2.2
    b = 32
    while b > 1 and (steps + warmup) * per_seq * b > CPU_BUDGET_S:
        b //= 2
    return b


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload != "c3":
        print(json.dumps(secondary_reference(args.workload, args)), flush=True)
        return
    batch = pick_cpu_batch(args.steps, args.warmup)
    tps, s_per_step, kind, cores, _ = cpu_decode_steps(batch, args.steps, args.warmup)
    tp, _ = layout(args.gpus, args.parallel)
    sample = f"{args.steps} full-recompute decode steps of the same model on the first {batch} of the {B} sequences, seq {T}, {cores} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": s_per_step * 1e3, "higher_is_better": True, "scaling": "weak" if tp == 1 else "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus, args.parallel, args.precision),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def measure_tf32_peak(device_index: int):
    """Dense TF32 rate of the library GEMM (torch.matmul with TF32 allowed, 8192^3), measured like the bf16 peak of
    MEASURED_PEAKS.json: best of 10 (burst) and back to back for about 2 s (sustained), SM clock sampled beside each.
    Three TF32 products make one fp32-grade product, so the ceiling of the 3xTF32 arithmetic is a third of these."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        sampler = ClockSampler(device_index).start()
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            a @ b
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        burst_clock = sampler.stop()
        sampler = ClockSampler(device_index).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = max(10, int(2000.0 / best))
        e0.record()
        for _ in range(iters):
            a @ b
        e1.record()
        torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / iters
        sus_clock = sampler.stop()
        return {"tf32_tflops_burst": flops / best / 1e9, "tf32_tflops_sustained": flops / sustained_ms / 1e9,
                "burst_sm_mhz": burst_clock.get("sm_mhz"), "sustained_sm_mhz": sus_clock.get("sm_mhz"), "sustained_reasons": sus_clock.get("reasons"),
                "how": "torch.matmul fp32 with allow_tf32 (library GEMM) 8192^3: best of 10, and back to back for ~2 s"}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def tf32_slots(kernel_name: str) -> float:
    """TF32-instruction-equivalents of tensor-core time per fp32 product of a kernel's arithmetic."""
    return 2.0 if "tf32_bf16x2" in kernel_name else 3.0


def kernel_table(trace, precision: str, peaks, tf32_peak):
    by = {}
    for r in trace:
        a = by.setdefault(r["kernel"], {"ms": 0.0, "flops": 0.0, "bytes": 0.0, "n": 0})
        a["ms"] += r["ms"]; a["flops"] += r["flops"]; a["bytes"] += r["bytes"]; a["n"] += 1
    total_ms = sum(a["ms"] for a in by.values()) or 1e-9
    kernels = {k: {"launches": v["n"], "ms": round(v["ms"], 4), "share": round(v["ms"] / total_ms, 4),
                   "tflops": round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 3) if v["ms"] > 0 else None,
                   "gbs": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1) if v["ms"] > 0 else None} for k, v in sorted(by.items(), key=lambda kv: -kv[1]["ms"])}
    # per-kernel fraction of its own roofline: tensor-core kernels against the ceiling of their arithmetic (the measured TF32
    # rate / the TF32-instruction-equivalents one fp32 product costs: 3 for three TF32 products, 2 for one TF32 product + two
    # bf16 corrections, a bf16 instruction covering twice the K of a TF32 one in the same time; the measured bf16 peak in
    # bf16 mode), exchange kernels against
    # the NVLink rate per direction (the kernel reports the bytes that ARRIVE at a rank during the exchange: the peers' partial
    # rows it fetches plus the normalised rows the peers store into it, 2 * (n-1)/n of the activation; as many leave it),
    # every other kernel against the measured copy bandwidth
    def tensor_ceiling(name):
        if "_bf16_tcgen05" in name:
            return peaks["bf16_tflops_sustained"]
        slots = tf32_slots(name)
        return tf32_peak["tf32_tflops_sustained"] / slots if tf32_peak else peaks["bf16_tflops_sustained"] / (2.0 * slots)
    for k, v in kernels.items():
        if "tcgen05" in k and v["tflops"] is not None:
            v["bound"], v["frac"] = "tensor", round(v["tflops"] / tensor_ceiling(k), 4)
        elif k in ("tp_exchange_add_layernorm", "p2p_all_reduce") and v["gbs"] is not None:
            v["bound"], v["frac"] = "nvlink", round(v["gbs"] / NVLINK_GBS_PER_DIRECTION, 4)
        elif v["gbs"] is not None:
            v["bound"], v["frac"] = "hbm", round(v["gbs"] / peaks["hbm_gbs"], 4)
    return by, kernels, total_ms, tensor_ceiling


def engine_options(args):
    """`--engine-option name=value` pairs (integer fields of FxfEngineOptions, e.g. tc_pair=1) for experiments."""
    out = {}
    for item in args.engine_option or []:
        k, _, v = item.partition("=")
        out[k] = int(v)
    return out


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
    tp_size, dp_size = layout(world, args.parallel)
    comm = None
    if tp_size > 1:
        from fxfusion_b200.tp import Communicator
        groups = [list(range(g * tp_size, (g + 1) * tp_size)) for g in range(world // tp_size)]
        handles = [dist.new_group(ranks=r) for r in groups]
        mine = rank // tp_size
        comm = Communicator.from_process_group(local, ranks=groups[mine], group=handles[mine])
    dp_rank = rank // tp_size
    graph_path = build_graph_file(B, tmp.name)
    eng = ExecutionEngine(graph_path, f"cuda:{local}", precision=args.precision, comm=comm, shard_output=comm is not None, **engine_options(args))
    lib = _lib.lib()
    prompt = torch.from_numpy(lowering.decode_prompt(B, PROMPT, cfg.vocab, seed=dp_rank))
    start_buf = torch.zeros((B, T), dtype=torch.int64)
    start_buf[:, :PROMPT] = prompt
    tok_slot, mask_slot = eng.input_slots()
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
            step_graph = lowering.gpt_step_graph(cfg, lowering.gpt_params(cfg, 0), batch=B, max_len=T, name="c3_step")
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
    # exchanges, so every rank of the group has to run it, not only the rank that reports.
    trace = None
    if rank == 0 or comm is not None:
        tok_slot.copy_(start_buf)
        eng.profile_launches()
        trace = eng.profile_launches()
    launches_per_run, device_bytes = eng.launches_per_run, eng.device_bytes
    describe_head = eng.describe().splitlines()[:3]
    eng.close()
    if comm is not None:
        comm.close()
    if rank == 0:
        report_c3(args, world, local, tp_size, dp_size, K, W, Ke, ms, e2e_ms, e2e_match, lr_ms, lr_match, bf16, kv, trace, clocks, status,
                  generated, launches_per_run, device_bytes, describe_head)
    tmp.cleanup()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def report_c3(args, world, local, tp_size, dp_size, K, W, Ke, ms, e2e_ms, e2e_match, lr_ms, lr_match, bf16, kv, trace, clocks, status,
              generated, launches_per_run, device_bytes, describe_head):
    """Rank 0, after the timed regions: roofline of the dominant kernel, TF32 peak, CPU baseline, secondary workloads, the line."""
    import torch
    peaks = measured_peaks()
    tf32_peak = None
    try:
        tf32_peak = measure_tf32_peak(local)
    except Exception as exc:  # noqa: BLE001
        sys.stderr.write(f"TF32 peak measurement failed: {exc}\n")
    by, kernels, total_ms, ceiling_of = kernel_table(trace, args.precision, peaks, tf32_peak)
    top_name, top = max(by.items(), key=lambda kv_: kv_[1]["ms"])
    tensor_ceiling = ceiling_of(top_name)
    achieved = top["flops"] / (top["ms"] * 1e-3) / 1e12
    traffic = NCU_DRAM_BYTES_PER_FORWARD.get(top_name) if tp_size == 1 else None
    step_mhz = clocks.get("sm_mhz") if clocks else None
    emulated = args.precision != "bf16"
    per_clock = None
    if emulated and tf32_peak and step_mhz:
        # flops per clock of the library GEMM: from its ~2 s loop (clock always sampled); the 15 ms burst only when a clock
        # sample fell inside it
        if tf32_peak.get("sustained_sm_mhz"):
            lib_per_mhz = tf32_peak["tf32_tflops_sustained"] / tf32_peak["sustained_sm_mhz"]
        elif tf32_peak.get("burst_sm_mhz"):
            lib_per_mhz = tf32_peak["tf32_tflops_burst"] / tf32_peak["burst_sm_mhz"]
        else:
            lib_per_mhz = None
        if lib_per_mhz:
            per_clock = (achieved / step_mhz) / (lib_per_mhz / tf32_slots(top_name))
    roofline = {"bound": "tensor", "kernel": top_name, "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": (traffic[0] / traffic[1]) if traffic and traffic[1] == top["n"] else None,
                "algorithmic_bytes": top["bytes"] / top["n"], "peak_source": peaks["source"] + " cuBLAS bf16, sustained",
                "launches_per_step": top["n"], "share_of_step": top["ms"] / total_ms,
                # fp32 results from one TF32 product + two bf16 corrections (or three TF32 products): the ceiling of this arithmetic
                # is the TF32 dense rate / 2 (/ 3), with the TF32 rate measured in this run the way the bf16 peak was (library
                # GEMM, burst and sustained, clocks beside them)
                "tf32_peak": tf32_peak,
                "tf32_instruction_equivalents_per_fp32_product": tf32_slots(top_name) if emulated else None,
                "fp32_emulation_ceiling": tensor_ceiling if emulated else None,
                "frac_of_fp32_emulation_ceiling": achieved / tensor_ceiling if emulated else None,
                # the same fraction with both sides divided by the SM clock they ran at (the library GEMM runs power-capped at a
                # lower clock than this kernel inside the step): flops per clock against flops per clock
                "frac_of_fp32_emulation_ceiling_per_clock": per_clock,
                "note": "achieved = logical fp32 flops (2MNK, counted once) of all launches of this kernel in one forward / their summed device time"}
    # ---- CPU baseline on a bounded sample; its tokens are compared with the device loop's -----------------
    cpu = None
    if not args.no_cpu_baseline and world == 1:   # the CPU baseline is a single-GPU figure (rank 0, N = 1)
        cb = pick_cpu_batch(2, 1)
        tps, s_per_step, kind, cores, cpu_buf = cpu_decode_steps(cb, 2, 1)
        n_steps = 3 if K >= 3 else 0   # one warm-up step + two timed steps, all starting at the prompt like the device loop
        eq = bool(torch.equal(cpu_buf[:, PROMPT:PROMPT + n_steps], generated[:cb, PROMPT:PROMPT + n_steps])) if n_steps else None
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": kind,
               "sample": f"2 full-recompute decode steps of the same model on the first {cb} of the {B} sequences, seq {T}; {s_per_step:.2f} s/step",
               "tokens_equal_reference_steps": (n_steps if eq else 0) if eq is not None else None,
               "tokens_compared": f"{cb} sequences x {n_steps} steps of the reference CPU path against the device loop" if n_steps else None}
    secondary = None
    if world == 1 and not args.no_extras:
        secondary = {}
        for w in ("c1", "c2", "c4", "c5"):
            try:
                secondary[w] = run_secondary(w, args, local, brief=True)
            except Exception as exc:  # noqa: BLE001
                secondary[w] = {"error": str(exc)[:300]}
    tokens_per_step = B * dp_size
    line = {
        "metric": METRIC, "value": tokens_per_step * K / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak" if tp_size == 1 else "strong", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
        "config": workload_config(world, args.parallel, args.precision),
        "e2e": {"value": tokens_per_step * Ke / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * T * 8 + B * T * T,
                "d2h_bytes_per_step": B * T * 8, "steps": Ke, "tokens_equal_device_loop": e2e_match},
        "last_row_projection": None if lr_ms is None else {
            "value": tokens_per_step * (T - PROMPT) / (lr_ms * 1e-3), "unit": "tokens/s", "ms_per_step": lr_ms / (T - PROMPT), "steps": T - PROMPT,
            "tokens_equal_full_loop": lr_match,
            "note": "opt-in fxf_decode_static_last_row: same tokens, the final Linear evaluated on 1 of 256 positions; not the headline (the graph contract's output is full logits)"},
        "bf16_mode": bf16,
        "kv_cache_decode": kv,
        "gpu_launches": K * (launches_per_run + 2),
        "launches_per_forward": launches_per_run,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels, "secondary": secondary,
        "device_status": status, "device_bytes": device_bytes, "engine": describe_head,
    }
    print(json.dumps(line), flush=True)


# ---- secondary workloads (forward only) ---------------------------------------------------------------------------------
def secondary_case(workload: str, batch=None):
    """Graph, inputs, logical flops, item count, metric name and description of a secondary configuration."""
    import torch
    from fxfusion_b200 import lowering
    gen = torch.Generator().manual_seed(0)
    if workload == "c1":
        nb = batch or 32
        g = lowering.mlp_graph(lowering.mlp_params(16, 512, 10, seed=0), batch=nb, name="c1_mlp")
        inputs = [torch.randn(nb, 512, generator=gen)]
        return (g, inputs, 2.0 * nb * 512 * (512 * 15 + 10), nb, "mlp16x512_forward_samples_per_s",
                "MLP, 16 layers of width 512 (14 LinearRelu + 1 FeedForward), batch 32, fp32")
    if workload == "c2":
        cfg = lowering.GPT_C2
        nb = batch or 8
        g = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=nb, seq=64, name="c2_gpt")
        ids = torch.from_numpy(lowering.decode_prompt(nb, 64, cfg.vocab))
        inputs = [ids, torch.tril(torch.ones(64, 64, dtype=torch.bool)).view(1, 1, 64, 64).expand(nb, 1, 64, 64).contiguous()]
        return (g, inputs, 3.62e9 * nb / 8, nb, "gpt4l_d256_forward_sequences_per_s",
                "GPT 4 layers d_model 256, 4 heads, vocab 1000, batch 8 x seq 64, fp32, single forward")
    if workload == "c4":
        cfg = lowering.TRANSFORMER_C4
        nb = batch or 64
        L = 256
        g = lowering.transformer_graph(cfg, lowering.transformer_params(cfg, 0), batch=nb, src_len=L, tgt_len=L, name="c4_encdec")
        inputs = [torch.randint(1, cfg.vocab, (nb, L), generator=gen), torch.randint(1, cfg.vocab, (nb, L), generator=gen),
                  torch.ones(nb, 1, 1, L, dtype=torch.bool),
                  torch.tril(torch.ones(L, L, dtype=torch.bool)).view(1, 1, L, L).expand(nb, 1, L, L).contiguous()]
        M, D, F, V, H = nb * L, cfg.d_model, cfg.d_ff, cfg.vocab, cfg.heads
        attn = 4.0 * nb * H * L * L * (D // H)
        enc = cfg.enc_layers * (2.0 * M * 3 * D * D + attn + 2.0 * M * D * D + 4.0 * M * D * F)
        dec = cfg.dec_layers * (2.0 * M * 3 * D * D + attn + 2.0 * M * D * D + (2.0 * M * D * D + 2.0 * M * 2 * D * D + attn + 2.0 * M * D * D) + 4.0 * M * D * F)
        return (g, inputs, enc + dec + 2.0 * M * D * V, nb, "encdec6x6_d512_forward_pairs_per_s",
                "encoder-decoder Transformer 6+6 layers d_model 512, 8 heads, vocab 32000, batch 64, 256 + 256 positions, fp32, single forward")
    nb = batch or 256
    g = lowering.resnet50_graph(lowering.resnet50_params(0), batch=nb, name="c5_resnet50")
    inputs = [torch.randn(nb, 3, 224, 224, generator=gen)]
    return (g, inputs, 8.2e9 * nb, nb, "resnet50_inference_images_per_s",
            "ResNet-50 inference, batch 256 x 3 x 224 x 224, fp32, BatchNorm folded, NCHW in / out")


def secondary_cpu(workload: str, budget_s: float = 12.0):
    """The reference CPU path on a bounded sample of a secondary workload: a reduced batch where the full one would not
    fit the budget; warm-up + timed iterations with perf_counter (the reference's methodology, benchmarks/utils.py:52-88)."""
    from oracle.graph_oracle import GraphOracle
    cores = use_all_host_cores()
    small = {"c1": 32, "c2": 8, "c4": 1, "c5": 4}[workload]
    g, inputs, _, items, _, _ = secondary_case(workload, small)
    kernels, kind = reference_kernels()
    orc = GraphOracle(g, kernels=kernels)
    orc.run(inputs)
    t0 = time.perf_counter()
    n = 0
    while True:
        orc.run(inputs)
        n += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or n >= 50:
            break
    return {"value": items * n / dt, "unit": "items/s", "cores": cores, "kind": kind,
            "sample": f"{n} forward(s) of the same graph at batch {small}, {dt / n * 1e3:.2f} ms each"}


def secondary_reference(workload: str, args):
    _, _, _, _, metric, desc = secondary_case(workload, {"c1": 32, "c2": 8, "c4": 1, "c5": 1}[workload])
    cpu = secondary_cpu(workload, budget_s=min(CPU_BUDGET_S, 30.0))
    return {"impl": "reference", "metric": metric, "value": cpu["value"], "unit": "items/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc}, "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": "items/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_secondary(workload: str, args, device_index: int = 0, brief: bool = False):
    """Forward throughput of c1 / c2 / c4 / c5 on one GPU: device-resident value (CUDA-Graph replay), e2e through
    fxf_engine_run_host with host buffers, roofline of the dominant kernel, CPU baseline on a bounded sample."""
    import numpy as np
    import torch
    from fxfusion_b200 import wire
    from fxfusion_b200.engine import ExecutionEngine
    g, inputs, flops, items, metric, desc = secondary_case(workload)
    tmp = tempfile.TemporaryDirectory()
    path = os.path.join(tmp.name, g.name + ".bin")
    wire.dump(g, path)
    del g
    eng = ExecutionEngine(path, f"cuda:{device_index}", precision=args.precision)
    dev_inputs = [t.cuda() for t in inputs]
    K = (200 if workload in ("c1", "c2") else 10) if brief else max(args.steps, 1)
    W = max(args.warmup, 3)
    for _ in range(W):
        eng.run(dev_inputs)
    torch.cuda.synchronize()
    sampler = ClockSampler(device_index).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        eng.run(dev_inputs)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K
    clocks = sampler.stop()
    # e2e: pinned host inputs in, every output back to the host, each call
    host_in = [t.contiguous().pin_memory() for t in inputs]
    host_out = [torch.empty(tuple(d.shape[i] for i in range(d.rank)), dtype=torch.float32).pin_memory() for d in eng.output_descs]
    as_np = lambda t: t.numpy().view(np.uint8) if t.dtype == torch.bool else t.numpy()
    Ke = max(2, min(K, 20))
    for _ in range(2):
        eng.run_host([as_np(t) for t in host_in], [as_np(t) for t in host_out])
    t0 = time.perf_counter()
    for _ in range(Ke):
        eng.run_host([as_np(t) for t in host_in], [as_np(t) for t in host_out])
    e2e_ms = (time.perf_counter() - t0) * 1e3 / Ke
    eng.profile_launches()
    trace = eng.profile_launches()
    peaks = measured_peaks()
    by, kernels, total_ms, ceiling_of = kernel_table(trace, args.precision, peaks, None)
    top_name, top = max(by.items(), key=lambda kv_: kv_[1]["ms"])
    tensor = "tcgen05" in top_name
    tensor_ceiling = ceiling_of(top_name) if tensor else None
    achieved = (top["flops"] / (top["ms"] * 1e-3) / 1e12) if tensor else (top["bytes"] / (top["ms"] * 1e-3) / 1e9)
    peak = peaks["bf16_tflops_sustained"] if tensor else peaks["hbm_gbs"]
    roofline = {"bound": "tensor" if tensor else "hbm", "kernel": top_name, "achieved": achieved, "peak": peak, "unit": "TFLOP/s" if tensor else "GB/s",
                "frac": achieved / peak, "traffic": None, "launches_per_step": top["n"], "share_of_step": top["ms"] / total_ms,
                "fp32_emulation_ceiling": tensor_ceiling if tensor else None,
                "frac_of_fp32_emulation_ceiling": achieved / tensor_ceiling if tensor else None,
                "peak_source": peaks["source"] + (" cuBLAS bf16, sustained (fp32 emulation ceiling = that / 6 for three TF32 products, / 4 for TF32 + two bf16 corrections)" if tensor else " copy bandwidth")}
    cpu = None if args.no_cpu_baseline else secondary_cpu(workload, budget_s=8.0 if brief else 20.0)
    status = eng.device_status()
    launches = eng.launches_per_run
    eng.close()
    tmp.cleanup()
    line = {"metric": metric, "value": items / (ms * 1e-3), "unit": "items/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": desc},
            "tflops_logical": flops / (ms * 1e-3) / 1e12,
            "e2e": {"value": items / (e2e_ms * 1e-3), "unit": "items/s", "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in inputs)),
                    "d2h_bytes_per_step": int(sum(t.numel() * 4 for t in host_out)), "steps": Ke},
            "gpu_launches": K * launches, "launches_per_forward": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "device_status": status}
    if brief:
        line["top_kernels"] = dict(list(kernels.items())[:4])
    else:
        line["kernels"] = kernels
    return line


def run_secondary_cli(args):
    """`--workload c1|c2|c4|c5`.  N > 1: independent replicas of the same batch on every GPU (samples are independent; no
    collective), value = items of all ranks / max-over-ranks time."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        dist.barrier()
    if rank != 0:
        args.no_cpu_baseline = True
    line = run_secondary(args.workload, args, local)
    if world > 1:
        items = line["value"] * line["ms_per_step"] * 1e-3
        e2e_ms = items / line["e2e"]["value"] * 1e3
        t = torch.tensor([line["ms_per_step"], e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line["ms_per_step"] = t[0].item()
        line["value"] = world * items / (t[0].item() * 1e-3)
        line["e2e"]["value"] = world * items / (t[1].item() * 1e-3)
        line["n_gpus"] = world
        line["config"]["parallelism"] = f"{world} independent replicas of the batch, no collective"
    if rank == 0:
        print(json.dumps(line), flush=True)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c3", choices=["c3", "c1", "c2", "c4", "c5"],
                    help="c3 = the decode benchmark (default); c1 = MLP 16 x 512 batch 32; c2 = GPT 4 layers d256 batch 8 x 64; "
                         "c4 = encoder-decoder forward, batch 64, 256 + 256 positions; c5 = ResNet-50 forward, batch 256")
    ap.add_argument("--micro", default=None, choices=["linear", "layernorm", "add", "mha", "conv"], help="profile one op instead of the decode workload")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="auto", choices=["auto", "fp32_simt", "fp32_3xtf32", "fp32_tf32_bf16x2", "bf16"],
                    help="bf16 = optional reduced-precision mode (bf16 tensor-core products, fp32 accumulation); not the headline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the opt-in decode variants and the secondary workloads (keeps profiler captures short)")
    ap.add_argument("--engine-option", action="append", default=[], metavar="NAME=VALUE",
                    help="integer field of FxfEngineOptions for the benchmark engine (tc_pair, tc_chunk_k, no_tp_fused_exchange, ...); repeatable")
    ap.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                    help="N > 1: tensor-parallel groups of 4 or 2 GPUs (default: the batch-32 decode sharded over heads, hidden units and "
                         "vocabulary) or N independent batch-32 replicas")
    args = ap.parse_args()
    if args.micro:
        return run_micro(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != "c3":
        return run_secondary_cli(args)
    run_ours(args)


if __name__ == "__main__":
    main()
