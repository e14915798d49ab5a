"""GPU parity on the committed golden graphs: the graph files were lowered by the reference's own
passes, the expected outputs come from the reference's eager models.  Every case runs through the
C-ABI engine (fxf_engine_create / fxf_engine_run) and is compared with both the golden outputs and
the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden_cases
from helpers import compare_outputs
from oracle.graph_oracle import GraphOracle, decode_static

pytestmark = pytest.mark.gpu

# graphs made only of copies / gathers must be bit-exact
EXACT = {"embedding", "narrow", "narrow_offset", "narrow_dynamic_length", "size", "transpose_multidim",
         "transpose_then_view", "transpose_last2", "relu", "max_pool2d", "max_pool2d_ceil"}
ATOL, RTOL = 1e-4, 1e-3  # fp32 activation tolerance: max-abs 1e-4 / rel 1e-3


def _case(name):
    z = np.load(GOLDEN / f"{name}.npz")
    ins = [torch.from_numpy(z[f"in{i}"]) for i in range(sum(k.startswith("in") for k in z.files))]
    outs = [torch.from_numpy(z[f"out{i}"]) for i in range(sum(k.startswith("out") for k in z.files))]
    return z, ins, outs


@pytest.mark.parametrize("use_graph", [True, False], ids=["cudagraph", "eager"])
@pytest.mark.parametrize("name", golden_cases())
def test_engine_matches_reference_outputs(built_lib, name, use_graph):
    from fxfusion_b200.engine import ExecutionEngine
    z, ins, outs = _case(name)
    eng = ExecutionEngine(str(GOLDEN / f"{name}.bin"), "cuda:0", use_cuda_graph=use_graph)
    for _ in range(2):  # second run reuses the arena: stale data must not leak
        got = [t.clone() for t in eng.run([t.cuda() for t in ins])]
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    if name in EXACT:
        for g, e in zip(got, outs):
            assert torch.equal(g.cpu(), e), f"{name} must be bit-exact"
    ok, info = compare_outputs(got, outs, atol=ATOL, rtol=RTOL)
    assert ok, f"vs reference eager: {info}"
    ok, info = compare_outputs(got, GraphOracle(str(GOLDEN / f"{name}.bin")).run(ins), atol=ATOL, rtol=RTOL)
    assert ok, f"vs oracle: {info}"
    eng.close()


@pytest.mark.parametrize("name", ["gpt_forward_static_shape", "gpt_2layer_decode"])
def test_greedy_decode_tokens_are_bit_exact(built_lib, name):
    """Reference test_gpt_static_decode (py/tests/test_ops.py:441-488): tokens must be equal."""
    from fxfusion_b200.engine import ExecutionEngine
    from fxfusion_b200.decode import engine_decode_static
    z, ins, _ = _case(name)
    tokens, expected = torch.from_numpy(z["tokens"]), torch.from_numpy(z["expected_tokens"])
    eng = ExecutionEngine(str(GOLDEN / f"{name}.bin"), "cuda:0")
    T = ins[0].shape[1]
    # (a) host loop, the reference's engine_decode_static mirrored call by call
    got = engine_decode_static(eng, tokens.cuda(), max_seq_len=T)
    assert torch.equal(got.cpu(), expected)
    # (b) device-resident loop through fxf_decode_static
    buf = torch.zeros((tokens.shape[0], T), dtype=torch.int64, device="cuda")
    buf[:, :tokens.shape[1]] = tokens.cuda()
    eng.decode_static(buf, tokens.shape[1])
    assert torch.equal(buf.cpu(), expected)
    eng.close()


def test_fully_masked_row_nan_parity(built_lib):
    """Reference test_mha_fully_masked_row_nan_parity (py/tests/test_ops.py:491-509)."""
    from fxfusion_b200.engine import ExecutionEngine
    z, ins, outs = _case("gpt_fully_masked_row")
    eng = ExecutionEngine(str(GOLDEN / "gpt_fully_masked_row.bin"), "cuda:0")
    got = eng.run([t.cuda() for t in ins])[0].cpu()
    assert torch.isnan(got).any()
    assert torch.equal(torch.isnan(got), torch.isnan(outs[0]))
    eng.close()


def test_run_host_round_trip(built_lib):
    from fxfusion_b200.engine import ExecutionEngine
    z, ins, outs = _case("mlp")
    eng = ExecutionEngine(str(GOLDEN / "mlp.bin"), "cuda:0")
    out = np.empty(tuple(outs[0].shape), np.float32)
    eng.run_host([t.numpy() for t in ins], [out])
    ok, info = compare_outputs(torch.from_numpy(out), outs[0], atol=ATOL, rtol=RTOL)
    assert ok, info
    eng.close()


def test_engine_errors_match_the_reference_conditions(built_lib, tmp_path):
    from fxfusion_b200 import wire
    from fxfusion_b200.engine import ExecutionEngine
    eng = ExecutionEngine(str(GOLDEN / "add.bin"), "cuda:0")
    z, ins, _ = _case("add")
    with pytest.raises(RuntimeError, match="Input count mismatch"):
        eng.run([ins[0].cuda()])
    with pytest.raises(RuntimeError, match="device mismatch"):
        eng.run(ins)  # CPU tensors
    eng.close()
    with pytest.raises(RuntimeError, match="failed to open"):
        ExecutionEngine(str(tmp_path / "missing.bin"), "cuda:0")
    raw = (GOLDEN / "linear.bin").read_bytes()
    (tmp_path / "trunc.bin").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(RuntimeError, match="corrupt|out of bounds"):
        ExecutionEngine(str(tmp_path / "trunc.bin"), "cuda:0")
    g = wire.load(GOLDEN / "linear.bin", copy_constants=True)
    g.nodes[-2].op_code = 25
    wire.dump(g, tmp_path / "badop.bin")
    with pytest.raises(RuntimeError, match="Unsupported OpCode"):
        ExecutionEngine(str(tmp_path / "badop.bin"), "cuda:0")
    g = wire.load(GOLDEN / "linear.bin", copy_constants=True)
    for t in g.tensors:
        if t.kind == wire.KIND_CONSTANT:
            t.data = None
            break
    wire.dump(g, tmp_path / "nodata.bin")
    with pytest.raises(RuntimeError, match="Constant tensor missing data"):
        ExecutionEngine(str(tmp_path / "nodata.bin"), "cuda:0")
    g = wire.load(GOLDEN / "linear.bin", copy_constants=True)
    g.arena_size = 64
    wire.dump(g, tmp_path / "smallarena.bin")
    with pytest.raises(RuntimeError, match="outside the arena"):
        ExecutionEngine(str(tmp_path / "smallarena.bin"), "cuda:0")
