"""Worker for the tensor-parallel tests; launched with torch.distributed.run (one process per rank).

    mode "cpu":  gloo ranks on the CPU check the sharding rule of fxfusion_b200.tp against the unsharded oracle
                 kernels (an MHA node, a FeedForward node, a vocabulary-sharded argmax).
    mode "gpu":  one GPU per rank; a tensor-parallel engine is compared with the CPU oracle (forward, greedy
                 decode with the vocabulary sharded) and with the single-GPU engine on rank 0.
"""
import math
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

from fxfusion_b200 import lowering, tp, wire
from oracle.graph_oracle import KERNELS, GraphOracle, decode_static, make_static_buffer, static_decoder_mask


def cpu_checks(rank, size):
    g = torch.Generator().manual_seed(0)
    B, T, H, hd, Fh = 2, 12, 4, 8, 64
    D = H * hd
    x = torch.randn(B, T, D, generator=g)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool)).view(1, 1, T, T).expand(B, 1, T, T).contiguous()
    wqkv, bqkv = torch.randn(3 * D, D, generator=g) / math.sqrt(D), torch.randn(3 * D, generator=g) * 0.1
    wo, bo = torch.randn(D, D, generator=g) / math.sqrt(D), torch.randn(D, generator=g) * 0.1
    # --- MHA: local heads only, partial output, all-reduce ---
    sh = tp.shard_mha(wqkv.numpy(), bqkv.numpy(), wo.numpy(), bo.numpy(), H, rank, size)
    Hl, Dl = sh["heads"], sh["heads"] * hd
    qkv = F.linear(x, torch.from_numpy(sh["wqkv"]), torch.from_numpy(sh["bqkv"]))
    q, k, v = (qkv[:, :, i * Dl:(i + 1) * Dl].view(B, T, Hl, hd).transpose(1, 2) for i in range(3))
    s = (q @ k.transpose(-2, -1)) / math.sqrt(hd)
    s = s.masked_fill(mask == 0, -math.inf)
    ctx = (torch.softmax(s, -1) @ v).transpose(1, 2).contiguous().view(B, T, Dl)
    part = F.linear(ctx, torch.from_numpy(np.ascontiguousarray(sh["wo"])), torch.from_numpy(sh["bo"]))
    dist.all_reduce(part)
    want = torch.zeros(B, T, D)
    KERNELS[wire.OP["MHA"]]([x, mask, wqkv, bqkv, wo, bo, want], [0, 1, 2, 3, 4, 5], [6], [H, hd, D, 3 * D], [math.sqrt(hd)])
    assert torch.allclose(part, want, atol=1e-5, rtol=1e-5), (part - want).abs().max()
    # --- CrossMHA: queries from x, keys/values from a longer memory, local heads only ---
    Tk = 17
    mem = torch.randn(B, Tk, D, generator=g)
    cmask = torch.ones(B, 1, 1, Tk, dtype=torch.bool)
    cmask[1, 0, 0, 11:] = False
    wq, bq = torch.randn(D, D, generator=g) / math.sqrt(D), torch.randn(D, generator=g) * 0.1
    wkv, bkv = torch.randn(2 * D, D, generator=g) / math.sqrt(D), torch.randn(2 * D, generator=g) * 0.1
    sc = tp.shard_cross_mha(wq.numpy(), bq.numpy(), wkv.numpy(), bkv.numpy(), wo.numpy(), bo.numpy(), H, rank, size)
    Hl, Dl = sc["heads"], sc["heads"] * hd
    q = F.linear(x, torch.from_numpy(sc["wq"]), torch.from_numpy(sc["bq"])).view(B, T, Hl, hd).transpose(1, 2)
    kv = F.linear(mem, torch.from_numpy(sc["wkv"]), torch.from_numpy(sc["bkv"]))
    k, v = (kv[:, :, i * Dl:(i + 1) * Dl].view(B, Tk, Hl, hd).transpose(1, 2) for i in range(2))
    s = ((q @ k.transpose(-2, -1)) / math.sqrt(hd)).masked_fill(cmask == 0, -math.inf)
    ctx = (torch.softmax(s, -1) @ v).transpose(1, 2).contiguous().view(B, T, Dl)
    part = F.linear(ctx, torch.from_numpy(np.ascontiguousarray(sc["wo"])), torch.from_numpy(sc["bo"]))
    dist.all_reduce(part)
    want = torch.zeros(B, T, D)
    KERNELS[wire.OP["CrossMHA"]]([x, mem, cmask, wq, bq, wkv, bkv, wo, bo, want], [0, 1, 2, 3, 4, 5, 6, 7, 8], [9], [H, hd, D, 2 * D], [math.sqrt(hd)])
    assert torch.allclose(part, want, atol=1e-5, rtol=1e-5), (part - want).abs().max()
    # --- FeedForward: column-parallel then row-parallel ---
    w1, b1 = torch.randn(Fh, D, generator=g) / math.sqrt(D), torch.randn(Fh, generator=g) * 0.1
    w2, b2 = torch.randn(D, Fh, generator=g) / math.sqrt(Fh), torch.randn(D, generator=g) * 0.1
    sf = tp.shard_feedforward(w1.numpy(), b1.numpy(), w2.numpy(), b2.numpy(), rank, size)
    part = F.linear(torch.relu(F.linear(x, torch.from_numpy(sf["w1"]), torch.from_numpy(sf["b1"]))),
                    torch.from_numpy(np.ascontiguousarray(sf["w2"])), torch.from_numpy(sf["b2"]))
    dist.all_reduce(part)
    want = torch.zeros(B, T, D)
    KERNELS[wire.OP["FeedForward"]]([x, w1, b1, w2, b2, want], [0, 1, 2, 3, 4], [5], [], [])
    assert torch.allclose(part, want, atol=1e-5, rtol=1e-5)
    # --- vocabulary-sharded argmax: local candidates, gather, first maximum wins ---
    V = 101
    logits = torch.randn(B, V, generator=g)
    logits[0, 7] = logits[0, 90] = 9.0  # a tie across shards: the lower index must win
    v0, v1 = tp.vocab_range(V, rank, size)
    local = logits[:, v0:v1]
    cand = torch.stack([local.max(-1).values, (local.argmax(-1) + v0).float()], -1)
    gathered = [torch.zeros_like(cand) for _ in range(size)]
    dist.all_gather(gathered, cand)
    allc = torch.stack(gathered)  # [size, B, 2]
    best = allc[..., 0].max(0).values
    idx = torch.where(allc[..., 0] == best, allc[..., 1], torch.full_like(best, float(V))).min(0).values.long()
    assert torch.equal(idx, logits.argmax(-1)), (idx, logits.argmax(-1))
    covered = sum(r1 - r0 for r0, r1 in (tp.vocab_range(V, r, size) for r in range(size)))
    assert covered == V
    # --- non-divisible head counts are replicated, not sharded: every rank computes the whole node, bias and residual
    # included, and nothing is summed over the ranks afterwards ---
    assert tp.head_range(12, rank, 8) == (0, 12) and tp.head_range(12, 1, 4) == (3, 6)
    H3, hd3 = 3, 8
    D3 = H3 * hd3
    x3 = torch.randn(B, T, D3, generator=g)
    w3, b3 = torch.randn(3 * D3, D3, generator=g) / math.sqrt(D3), torch.randn(3 * D3, generator=g) * 0.1
    wo3, bo3 = torch.randn(D3, D3, generator=g) / math.sqrt(D3), torch.randn(D3, generator=g) * 0.1
    s3 = tp.shard_mha(w3.numpy(), b3.numpy(), wo3.numpy(), bo3.numpy(), H3, rank, size)
    assert not s3["sharded"] and s3["heads"] == H3 and np.array_equal(s3["bo"], bo3.numpy())
    qkv = F.linear(x3, torch.from_numpy(s3["wqkv"]), torch.from_numpy(s3["bqkv"]))
    q, k, v = (qkv[:, :, i * D3:(i + 1) * D3].view(B, T, H3, hd3).transpose(1, 2) for i in range(3))
    sc3 = ((q @ k.transpose(-2, -1)) / math.sqrt(hd3)).masked_fill(mask == 0, -math.inf)
    ctx3 = (torch.softmax(sc3, -1) @ v).transpose(1, 2).contiguous().view(B, T, D3)
    full = F.linear(ctx3, torch.from_numpy(np.ascontiguousarray(s3["wo"])), torch.from_numpy(s3["bo"]))   # no all-reduce
    want = torch.zeros(B, T, D3)
    KERNELS[wire.OP["MHA"]]([x3, mask, w3, b3, wo3, bo3, want], [0, 1, 2, 3, 4, 5], [6], [H3, hd3, D3, 3 * D3], [math.sqrt(hd3)])
    assert torch.allclose(full, want, atol=1e-5, rtol=1e-5)


def gpu_checks(rank, size, tmp):
    from fxfusion_b200.engine import ExecutionEngine
    torch.cuda.set_device(rank)
    comm = tp.Communicator.from_process_group(rank)
    cfg = lowering.GPTConfig(256, 4, 1000, 4, 2)  # 4 heads of 64: divides over 2 and 4 ranks
    B, T, L0 = 4, 64, 40
    graph = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=B, seq=T, name="tp_gpt")
    path = os.path.join(tmp, f"tp_gpt_{rank}.bin")
    wire.dump(graph, path)
    tokens = torch.from_numpy(lowering.decode_prompt(B, L0, cfg.vocab))
    buf = make_static_buffer(tokens, T)
    mask = static_decoder_mask(buf, L0)
    oracle = GraphOracle(graph)
    want = oracle.run([buf, mask])[0]
    for precision, options in (("auto", {}), ("fp32_simt", {}), ("auto", {"no_tp_fused_exchange": 1}), ("auto", {"no_epilogue_fusion": 1})):
        eng = ExecutionEngine(path, f"cuda:{rank}", comm=comm, precision=precision, **options)
        text = eng.describe()
        fused = "+exchange(" in text
        assert fused == (not options.get("no_tp_fused_exchange")), f"rank {rank}: unexpected exchange fusion state with {options}:\n{text}"
        if fused:   # the residual stream between two exchanges stays row-sharded; Add and LayerNorm nodes launch nothing
            assert "[own rows]" in text and "folded into an earlier node" in text
        for _ in range(2):   # twice: the epochs of the peer barriers carry over from run to run
            got = eng.run([buf.cuda(), mask.cuda()])[0].cpu()
            err = (got - want).abs().max().item()
            assert err < 1e-4, f"rank {rank} {precision} {options}: TP forward differs from the oracle by {err}"
        assert eng.device_status() == 0
        eng.close()
    # row-pushed products: every rank owns whole 128-row tiles (8 x 64 = 512 rows over 2 or 4 ranks), so the products store
    # their rows into the owners' exchange windows and the exchange reads local memory
    B8 = 8
    graph8 = lowering.gpt_graph(cfg, lowering.gpt_params(cfg, 0), batch=B8, seq=T, name="tp_gpt8")
    path8 = os.path.join(tmp, f"tp_gpt8_{rank}.bin")
    wire.dump(graph8, path8)
    buf8 = make_static_buffer(torch.from_numpy(lowering.decode_prompt(B8, L0, cfg.vocab)), T)
    mask8 = static_decoder_mask(buf8, L0)
    want8 = GraphOracle(graph8).run([buf8, mask8])[0]
    for options in ({"tp_push": 1}, {}):
        eng = ExecutionEngine(path8, f"cuda:{rank}", comm=comm, **options)
        assert ("exchange window" in eng.describe()) == bool(options), eng.describe()
        for _ in range(3):   # the window is reused by every exchange of every run
            got8 = eng.run([buf8.cuda(), mask8.cuda()])[0].cpu()
            err = (got8 - want8).abs().max().item()
            assert err < 1e-4, f"rank {rank} {options}: TP forward with row-pushed products differs from the oracle by {err}"
        assert eng.device_status() == 0
        eng.close()
    # heads that do not divide over the ranks (3 heads): the MHA nodes are replicated on every rank (no exchange, bias and
    # residual on every rank), the FeedForward nodes are still sharded
    cfg3 = lowering.GPTConfig(192, 3, 300, 4, 2)
    g3 = lowering.gpt_graph(cfg3, lowering.gpt_params(cfg3, 5), batch=2, seq=32, name="tp_gpt3")
    path3 = os.path.join(tmp, f"tp_gpt3_{rank}.bin")
    wire.dump(g3, path3)
    tok3 = torch.from_numpy(lowering.decode_prompt(2, 20, cfg3.vocab))
    buf3 = make_static_buffer(tok3, 32)
    mask3 = static_decoder_mask(buf3, 20)
    want3 = GraphOracle(g3).run([buf3, mask3])[0]
    for options in ({}, {"no_tp_fused_exchange": 1}):
        eng = ExecutionEngine(path3, f"cuda:{rank}", comm=comm, **options)
        assert "replicated" in eng.describe()
        got3 = eng.run([buf3.cuda(), mask3.cuda()])[0].cpu()
        err = (got3 - want3).abs().max().item()
        assert err < 1e-4, f"rank {rank}: TP forward with replicated attention differs from the oracle by {err} ({options})"
        assert eng.device_status() == 0
        eng.close()
    # encoder-decoder graph: CrossMHA nodes are head-sharded like MHA
    ecfg = lowering.TransformerConfig(256, 4, 500, 2, 1, 2, pe_len=64)
    eg = lowering.transformer_graph(ecfg, lowering.transformer_params(ecfg, 1), batch=2, src_len=48, tgt_len=32, name="tp_encdec")
    epath = os.path.join(tmp, f"tp_encdec_{rank}.bin")
    wire.dump(eg, epath)
    gen = torch.Generator().manual_seed(3)
    esrc, etgt = torch.randint(1, 500, (2, 48), generator=gen), torch.randint(1, 500, (2, 32), generator=gen)
    esm = torch.ones(2, 1, 1, 48, dtype=torch.bool)
    esm[1, 0, 0, 40:] = False
    etm = torch.tril(torch.ones(32, 32, dtype=torch.bool)).view(1, 1, 32, 32).expand(2, 1, 32, 32).contiguous()
    ewant = GraphOracle(eg).run([esrc, etgt, esm, etm])[0]
    eng = ExecutionEngine(epath, f"cuda:{rank}", comm=comm)
    egot = eng.run([esrc.cuda(), etgt.cuda(), esm.cuda(), etm.cuda()])[0].cpu()
    err = (egot - ewant).abs().max().item()
    assert err < 1e-4, f"rank {rank}: TP encoder-decoder forward differs from the oracle by {err}"
    assert eng.device_status() == 0
    eng.close()
    # greedy decode with the vocabulary sharded as well: tokens must equal the oracle's on every rank
    eng = ExecutionEngine(path, f"cuda:{rank}", comm=comm, shard_output=True)
    dev = buf.cuda()
    eng.decode_static(dev, L0)
    torch.cuda.synchronize()
    want_tokens = decode_static(lambda b, m: oracle.run([b, m])[0], tokens, T)
    assert torch.equal(dev.cpu(), want_tokens), f"rank {rank}: TP greedy tokens differ from the oracle"
    dev = buf.cuda()
    eng.decode_static(dev, L0, last_row_only=True)
    torch.cuda.synchronize()
    assert torch.equal(dev.cpu(), want_tokens), f"rank {rank}: TP greedy tokens (last-row projection) differ from the oracle"
    eng.close()
    # failure detection, injected on the host: rank 0 runs a forward that the other ranks never join.  Its first exchange
    # runs into the 50 ms budget, records 121 and tells the peers; every later exchange of every rank returns at once.  The
    # late ranks then run their forward: it returns too, with status 123.  Nothing hangs and the engines are destroyed.
    eng = ExecutionEngine(path, f"cuda:{rank}", comm=comm, p2p_start_budget_ms=50, p2p_end_budget_ms=50)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        eng.run([buf.cuda(), mask.cuda()])
        st = eng.device_status()
        assert st == 121, f"rank 0: expected status 121 after a lonely forward, got {st}"
    dist.barrier()
    if rank != 0:
        eng.run([buf.cuda(), mask.cuda()])
        st = eng.device_status()
        assert st == 123, f"rank {rank}: expected status 123 (a peer gave up), got {st}"
    dist.barrier()
    eng.close()
    comm.close()


def main():
    mode = sys.argv[1]
    dist.init_process_group("gloo" if mode == "cpu" else "nccl")
    rank, size = dist.get_rank(), dist.get_world_size()
    if mode == "cpu":
        cpu_checks(rank, size)
    else:
        gpu_checks(rank, size, sys.argv[2])
    dist.barrier()
    if rank == 0:
        print(f"tp_worker {mode} ok on {size} ranks")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
