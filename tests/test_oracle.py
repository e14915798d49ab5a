"""Pins the CPU oracle: against the committed golden vectors (outputs of the reference's eager
models) and, where it has been built, against the reference's own compiled CPU kernels."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden_cases
from helpers import compare_outputs
from fxfusion_b200 import wire
from oracle.graph_oracle import KERNELS, GraphOracle, decode_static
from oracle.ref_cpu.build import load as load_ref


def _case(name):
    z = np.load(GOLDEN / f"{name}.npz")
    ins = [torch.from_numpy(z[f"in{i}"]) for i in range(sum(k.startswith("in") for k in z.files))]
    outs = [torch.from_numpy(z[f"out{i}"]) for i in range(sum(k.startswith("out") for k in z.files))]
    return z, ins, outs


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_reproduces_reference_eager_outputs(name):
    z, ins, outs = _case(name)
    got = GraphOracle(str(GOLDEN / f"{name}.bin")).run(ins)
    tight = name.startswith("gpt_forward")  # the reference's own GPT forward test uses 1e-5
    ok, info = compare_outputs(got, outs, atol=1e-5 if tight else 1e-4, rtol=1e-5 if tight else 1e-4)
    assert ok, info


@pytest.mark.parametrize("name", ["gpt_forward_static_shape", "gpt_2layer_decode"])
def test_oracle_greedy_decode_matches_reference_tokens(name):
    z, _, _ = _case(name)
    orc = GraphOracle(str(GOLDEN / f"{name}.bin"))
    T = orc.reg[orc.input_ids[0]].shape[1]
    got = decode_static(lambda buf, mask: orc.run([buf, mask])[0], torch.from_numpy(z["tokens"]), T)
    assert torch.equal(got, torch.from_numpy(z["expected_tokens"]))


def test_fully_masked_row_gives_nan_like_the_reference():
    z, ins, outs = _case("gpt_fully_masked_row")
    assert torch.isnan(outs[0]).any() and not torch.isnan(outs[0]).all()
    got = GraphOracle(str(GOLDEN / "gpt_fully_masked_row.bin")).run(ins)[0]
    assert torch.equal(torch.isnan(got), torch.isnan(outs[0]))


@pytest.mark.parametrize("name", golden_cases())
def test_restatement_is_bit_identical_to_reference_kernels(name):
    ref = load_ref()
    if ref is None:
        pytest.skip("oracle/_ref has not been built (python -m oracle.ref_cpu.build)")

    def bind(op):
        def fn(reg, i, o, ints, floats):
            ref.call(op, [t if t is not None else torch.empty(0) for t in reg], list(i), list(o), list(ints), list(floats))
        return fn

    _, ins, _ = _case(name)
    a = GraphOracle(str(GOLDEN / f"{name}.bin")).run(ins)
    # opcodes above 19 are this library's extensions: the reference has no kernel for them, the restatement stays
    b = GraphOracle(str(GOLDEN / f"{name}.bin"), kernels={op: (bind(op) if op <= 19 else KERNELS[op]) for op in KERNELS}).run(ins)
    for x, y in zip(a, b):
        assert torch.equal(torch.isnan(x), torch.isnan(y))
        assert torch.equal(torch.nan_to_num(x), torch.nan_to_num(y))


def test_golden_files_are_complete():
    names = golden_cases()
    assert len(names) >= 35
    ops_seen = set()
    for n in names:
        assert (GOLDEN / f"{n}.npz").exists()
        ops_seen |= {nd.op_code for nd in wire.load(GOLDEN / f"{n}.bin").nodes}
    assert ops_seen >= set(range(1, 20)), f"golden set misses opcodes {set(range(1, 20)) - ops_seen}"


def test_incremental_decode_equals_full_recompute():
    """The single-position step graph (CachedMHA, extension opcode 21) decodes the same tokens as the reference-shaped
    full-recompute graph, including a pad token inside a prompt (masked as a key from then on)."""
    from fxfusion_b200 import lowering
    from oracle.graph_oracle import decode_cached
    cfg = lowering.GPTConfig(64, 4, 200, 4, 2)
    params = lowering.gpt_params(cfg, 0, std=0.2)
    B, T, L0 = 3, 24, 6
    tokens = torch.from_numpy(lowering.decode_prompt(B, L0, cfg.vocab))
    tokens[1, 3] = 0
    full = GraphOracle(lowering.gpt_graph(cfg, params, batch=B, seq=T))
    step = GraphOracle(lowering.gpt_step_graph(cfg, params, batch=B, max_len=T))
    want = decode_static(lambda b, m: full.run([b, m])[0], tokens, T)
    got = decode_cached(lambda i, p, b: step.run([i, p, b])[0], tokens, T)
    assert torch.equal(got, want)
