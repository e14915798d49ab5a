"""One-off check (not collected by pytest; takes minutes of CPU time): the complete GPT-2-small-shape greedy
decode — batch 32, 128 prompt + 128 generated tokens, 4096 argmax decisions — on the GPU against the CPU
oracle walking the same graph file through the reference's compiled CPU kernels.

    python tests/c3_full_decode_check.py [steps]

Prints whether all tokens are equal; if not, for every sequence the first differing position and the
oracle's top-1/top-2 logit margin there (a difference at a margin near the fp32 noise floor is a near-tie,
not an error in the path).
"""
import sys
import tempfile
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch

from fxfusion_b200 import lowering, wire
from fxfusion_b200.engine import ExecutionEngine
from oracle.graph_oracle import KERNELS, GraphOracle, make_static_buffer, static_decoder_mask
from oracle.ref_cpu.build import load as load_ref

B, T, PROMPT = 32, 256, 128
steps = int(sys.argv[1]) if len(sys.argv) > 1 else T - PROMPT
cfg = lowering.GPT2_SMALL
graph = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=B, seq=T, name="c3")
tokens = torch.from_numpy(lowering.decode_prompt(B, PROMPT, cfg.vocab))
buf = make_static_buffer(tokens, T)

with tempfile.TemporaryDirectory() as tmp:
    path = f"{tmp}/c3.bin"
    wire.dump(graph, path)
    eng = ExecutionEngine(path, "cuda:0")
    dev = buf.cuda()
    # device loop, `steps` steps only
    from fxfusion_b200 import _lib
    import ctypes as C
    lib = _lib.lib()
    tok_slot, mask_slot = eng.input_slots()
    tok_slot.copy_(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for cur in range(PROMPT, PROMPT + steps):
        _lib.check(lib.fxf_decode_build_mask(C.c_void_p(tok_slot.data_ptr()), C.c_void_p(mask_slot.data_ptr()), B, T, cur, 0, stream))
        _lib.check(lib.fxf_engine_run(eng.handle, (C.c_void_p * 2)(tok_slot.data_ptr(), mask_slot.data_ptr()), 2, stream))
        _lib.check(lib.fxf_engine_argmax_scatter(eng.handle, C.c_void_p(tok_slot.data_ptr()), cur, stream))
    torch.cuda.synchronize()
    gpu_tokens = tok_slot.cpu().clone()
    status = eng.device_status()

    ref = load_ref()
    kernels = None
    if ref is not None:
        def bind(op):
            def fn(reg, i, o, ints, floats):
                ref.call(op, [t if t is not None else torch.empty(0) for t in reg], list(i), list(o), list(ints), list(floats))
            return fn
        kernels = {op: bind(op) for op in KERNELS}
    orc = GraphOracle(graph, kernels=kernels)
    cpu = buf.clone()
    margins = torch.zeros(steps, B)
    t0 = time.time()
    # teacher-forced on the GPU's tokens as well: agreement of every decision given the same history
    forced_equal = 0
    first_div = [-1] * B
    for s, cur in enumerate(range(PROMPT, PROMPT + steps)):
        logits = orc.run([cpu, static_decoder_mask(cpu, cur)])[0]
        row = logits[:, cur - 1, :]
        top2 = torch.topk(row, 2, dim=-1).values
        margins[s] = top2[:, 0] - top2[:, 1]
        nxt = row.argmax(-1)
        cpu[:, cur] = nxt
        for b in range(B):
            if first_div[b] < 0 and int(nxt[b]) != int(gpu_tokens[b, cur]):
                first_div[b] = cur
        if s % 16 == 0:
            print(f"cpu step {s}/{steps} ({time.time() - t0:.0f} s)", flush=True)
    equal = torch.equal(cpu[:, :PROMPT + steps], gpu_tokens[:, :PROMPT + steps])
    print(f"device status {status}; oracle kernels: {'reference' if ref is not None else 'port'}")
    print(f"decisions {steps * B}; all tokens equal: {equal}")
    print(f"oracle top-2 margin: min {margins.min().item():.3e}, median {margins.median().item():.3e}")
    for b in range(B):
        if first_div[b] >= 0:
            s = first_div[b] - PROMPT
            print(f"  sequence {b}: first difference at position {first_div[b]}, oracle margin there {margins[s, b].item():.3e}")
    eng.close()
