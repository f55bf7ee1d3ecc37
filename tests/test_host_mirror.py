"""CPU tests of the host side above the C ABI that goes beyond the reference's one-expression
emitter: the bytecode subset with conditionals, loops, calls and indexed loads (lowered programs
checked against numpy through the oracle's interpreter, emitted CUDA C checked by compiling it
with NVRTC for compute_100a — no GPU needed), the InstructionsCompiler contract, the Kernel
leftovers, the loop-routing rule and the packaging of tensors beside the bytecode."""
import asyncio
import os
import zipfile

import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import bytecode as B
from strict_b200 import native, packaging

FILTERS = sb.StrictType("Filters", [
    sb.Method("Clamp(value Number) Number", ["\tif value > 1", "\t\treturn 1", "\tif value < 0", "\t\treturn 0", "\tvalue"]),
    sb.Method("Brighten(pixel Number, initialDepth Number) Number", ["\tClamp(pixel + initialDepth)"]),
    sb.Method("Blur5(image Number) Number",
              ["\tmutable sum = 0", "\tconstant centre = index", "\tfor 5", "\t\tsum = sum + image(centre + index - 2)", "\tsum / 5"]),
    sb.Method("Checker(a Number, b Number) Number", ["\tif index % 2 is 0", "\t\ta", "\telse", "\t\tb * 2"]),
    sb.Method("Triangle(a Number) Number", ["\tmutable total = 0", "\tfor 3", "\t\tconstant row = index", "\t\tfor row + 1", "\t\t\ttotal = total + a * (row + index)", "\ttotal"]),
    sb.Method("Twice(a Number) Number", ["\tBrighten(a, 0.25) + Brighten(a * 2, 0.5)"]),
])


def nvrtc_or_skip(text, name):
    try:
        return native.compile_to_ptx(text, name)
    except NotImplementedError as e:
        pytest.skip(f"NVRTC is not installed: {e}")


def run_on_oracle(oracle, compiled, arrays, scalars, n):
    return oracle.ew_program2(np.array(compiled.code, np.int32), arrays, scalars, compiled.consts, n)


def test_bytecode_of_a_conditional():
    ins = sb.InstructionsToCuda().compile(FILTERS.by_name["Clamp"], FILTERS).instructions
    kinds = [type(i).__name__ for i in ins]
    assert kinds[:4] == ["LoadVariableToRegister", "LoadConstantInstruction", "BinaryInstruction", "JumpToId"]
    assert ins[2].IsConditional() and ins[2].InstructionType == B.GreaterThan and ins[3].InstructionType == B.JumpToIdIfFalse
    assert "ReturnInstruction" in kinds and "JumpToIdEnd" in kinds
    call = sb.InstructionsToCuda().compile(FILTERS.by_name["Brighten"], FILTERS).instructions
    invoke = [i for i in call if isinstance(i, B.Invoke)][0]
    assert invoke.MethodInfo.MethodName == "Clamp" and invoke.MethodInfo.ParameterNames == ["value"] and len(invoke.ArgumentRegisters) == 1
    loop = sb.InstructionsToCuda().compile(FILTERS.by_name["Blur5"], FILTERS).instructions
    assert any(isinstance(i, B.LoopBeginInstruction) for i in loop) and any(isinstance(i, B.ListCallInstruction) for i in loop)
    end = [i for i in loop if isinstance(i, B.LoopEndInstruction)][0]
    assert end.Begin is [i for i in loop if isinstance(i, B.LoopBeginInstruction)][0]


def test_extended_programs_match_numpy(oracle, rng):
    n = 1000
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    c = sb.InstructionsToCuda().compile
    clamp = lambda v: np.clip(v, 0, 1).astype(np.float32)  # noqa: E731
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Clamp"], FILTERS), [x], [], n), clamp(x))
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Brighten"], FILTERS), [x], [0.3], n), clamp(x + np.float32(0.3)))
    padded = np.concatenate([np.zeros(2, np.float32), x, np.zeros(2, np.float32)])  # loads outside [0, n) read 0
    want = np.zeros(n, np.float32)
    for k in range(5):
        want = want + padded[k:k + n]
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Blur5"], FILTERS), [x], [], n), want / np.float32(5))
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Checker"], FILTERS), [x, y], [], n), np.where(np.arange(n) % 2 == 0, x, y * 2).astype(np.float32))
    tri = np.zeros(n, np.float32)
    for row in range(3):
        for i in range(row + 1):
            tri = tri + x * np.float32(row + i)
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Triangle"], FILTERS), [x], [], n), tri)
    twice = clamp(x + np.float32(0.25)) + clamp(x * np.float32(2) + np.float32(0.5))
    assert np.array_equal(run_on_oracle(oracle, c(FILTERS.by_name["Twice"], FILTERS), [x], [], n), twice)


def test_reference_subset_goes_through_the_same_bytecode(oracle, rng):
    m = sb.InstructionsToCuda().compile(sb.Method("F(a Number, b Number, c Number) Number", ["\t(a + b) * c - 1"]))
    assert not m.extended and [type(i).__name__ for i in m.instructions].count("BinaryInstruction") == 3
    mod = sb.InstructionsToCuda().compile(sb.Method("F(a Number) Number", ["\ta % 2"]))  # Modulo: beyond the reference's four operators
    assert mod.extended and "fmodf(" in mod.cuda
    a = (rng.standard_normal(100) * 5).astype(np.float32)
    assert np.array_equal(run_on_oracle(oracle, mod, [a], [], 100), np.fmod(a, np.float32(2)))


@pytest.mark.parametrize("name", [m.Name for m in FILTERS.Methods])
def test_emitted_text_is_valid_cuda_c(name):
    compiled = sb.InstructionsToCuda().compile(FILTERS.by_name[name], FILTERS)
    ptx = nvrtc_or_skip(compiled.cuda, name)
    assert ".target sm_100a" in ptx and f".entry {name}(" in ptx


@pytest.mark.parametrize("sig,body", [("Add(first Number, second Number) Number", "first + second"),
                                      ("Process(input Number, width Number, height Number, initialDepth Number) Number", "initialDepth")])
def test_reference_texts_are_valid_cuda_c(sig, body):
    text = sb.InstructionsToCuda().Compile(sb.Method(sig, ["\t" + body]))
    assert ".visible .entry" in nvrtc_or_skip(text, sig.split("(")[0])


def test_limits_and_errors():
    c = sb.InstructionsToCuda().compile
    with pytest.raises(NotImplementedError):
        c(sb.Method("F(a Number) Number", ["\ta ^ 2"]))
    with pytest.raises(NotImplementedError):
        c(sb.Method("F(a Number) Number", ["\tb + 1"]))
    with pytest.raises(NotImplementedError):
        c(sb.Method("F(a Number) Number", ["\tmissing = 1", "\ta"]))
    rec = sb.StrictType("R", [sb.Method("F(a Number) Number", ["\tG(a)"]), sb.Method("G(a Number) Number", ["\tF(a)"])])
    with pytest.raises(NotImplementedError, match="recursive"):
        c(rec.by_name["F"], rec)
    deep = ["\t" * (d + 1) + "for 2" for d in range(5)] + ["\t" * 6 + "constant x = 1", "\ta"]
    with pytest.raises(NotImplementedError, match="nested"):
        c(sb.Method("F(a Number) Number", deep))
    try:
        native.compile_to_ptx("not cuda at all", "x")
        assert False
    except ValueError as e:
        assert "error" in str(e)
    except NotImplementedError:
        pass  # NVRTC not installed


def test_instructions_compiler_contract():
    """InstructionsCompiler.cs:114-115: abstract Compile(binary, platform) -> Task<string>, Extension."""
    assert issubclass(sb.InstructionsToCuda, sb.InstructionsCompiler) and sb.InstructionsToCuda().Extension == ".cu"
    with pytest.raises(NotImplementedError):
        sb.InstructionsCompiler().Compile(None, sb.Platform.Linux)
    program = sb.StrictType("Program", [sb.Method("Run Number", ["\tconstant five = 5", "\tfive * 2"])] + FILTERS.Methods)
    binary = sb.BinaryExecutable(program)
    assert [type(i).__name__ for i in binary.EntryPoint.instructions][-1] == "ReturnInstruction"
    text = asyncio.run(sb.InstructionsToCuda().Compile(binary, sb.Platform.Linux))
    assert 'extern "C" __global__ void Run(float *output, const int count)' in text  # entry point: Run, no parameters, a count (cs:14-15)
    twice = sb.InstructionsToCuda().compile(FILTERS.by_name["Twice"], FILTERS)
    found = sb.InstructionsCompiler.CollectMethods(twice.instructions, sb.BinaryExecutable(FILTERS))
    assert sorted(found) == ["Brighten(pixel, initialDepth) Number", "Clamp(value) Number"]
    assert sb.InstructionsCompiler.BuildMethodHeaderKey("Run", [], "None") == "Run"


def test_kernel_compile_and_save_ptx(tmp_path):
    k = sb.Kernel.__new__(sb.Kernel)  # no device here: the compile step needs none
    k.Context, k._handle = None, None
    path = str(tmp_path / "VectorAdd.ptx")
    try:
        ok = k.CompileKernelAndSaveAsPtxFile(path)
    except NotImplementedError as e:
        pytest.skip(str(e))
    assert ok and "saxpy" in open(path).read()
    assert k.Handle is k.Handle and not k.Handle.disposed


def test_loop_routing_rule(tmp_path):
    """InstructionsToMlir.cs:403-418 and the reference's own expectations
    (Strict.Compiler.Assembly.Tests/BlurPerformanceTests.cs:153-188): a 320x320 blur (30 body
    instructions) parallelises, 100,000 pixels of blur too, a small brightness loop does not."""
    assert (sb.ComplexityThreshold, sb.GpuComplexityThreshold) == (100_000, 10_000_000)
    assert sb.EstimateComplexity(320 * 320, 30) > sb.ComplexityThreshold and sb.ChooseStrategy(320 * 320, 30) == "scf.parallel"
    assert sb.ChooseStrategy(100_000, 30) == "scf.parallel" and sb.ChooseStrategy(100, 6) == "scf.for"
    assert sb.ChooseStrategy(2048 * 1024, 30) == "gpu.launch" and sb.ChooseStrategy(1280 * 720, 6) == "scf.parallel"
    assert sb.EstimateComplexity(10, 0) == 10
    src = tmp_path / "Filters.strict"
    src.write_text("")
    r = sb.Runner(str(src), sb.StrictType("Program", [sb.Method("Run Number", ["\t1 + 2"])]))
    out = r.Build(sb.Platform.Linux, sb.CompilerBackend.Cuda)
    assert out.endswith("Filters.cu") and "void Run(float *output, const int count)" in open(out).read()
    with pytest.raises(NotImplementedError):
        r.Build(sb.Platform.Linux, sb.CompilerBackend.Nasm)
    plan, compiled = sb.Runner(str(src), FILTERS).Plan("Blur5", 4_000_000)
    assert plan == "gpu.launch" and compiled.extended
    assert sb.Runner(str(src), FILTERS).Plan("Clamp", 1000)[0] == "scf.for"


def test_tensors_beside_the_bytecode(tmp_path, oracle):
    path = str(tmp_path / ("Model" + packaging.Extension))
    bytecode = bytes(range(200))
    with zipfile.ZipFile(path, "w") as z:  # what BinaryExecutable.Serialize writes: one .bytecode entry per type
        z.writestr("Strict/Examples/Model.bytecode", bytecode, compress_type=zipfile.ZIP_DEFLATED)
        z.writestr("Strict/Number.bytecode", b"\x01\x02", compress_type=zipfile.ZIP_DEFLATED)
    cfg = dict(arch=1, n_layers=1, d_model=256, n_q_heads=2, n_kv_heads=1, head_dim=128, d_ff=256, vocab=512, max_pos=64, tied=0, eps=1e-6, rope_theta=1e6)
    wq, ws = oracle.gen_qlinear(1, 2, 512, 256)
    tensors = {"layers.0.wqkv.q": wq, "layers.0.wqkv.s": ws, "normf.g": np.ones(256, np.float32)}
    packaging.add_model(path, cfg, tensors)
    assert sorted(packaging.bytecode_entries(path)) == ["Strict/Examples/Model", "Strict/Number"]
    with zipfile.ZipFile(path) as z:
        assert z.read("Strict/Examples/Model.bytecode") == bytecode  # the bytecode is untouched
        assert z.getinfo("model/layers.0.wqkv.q.tensor").compress_type == zipfile.ZIP_STORED
    got_cfg, got = packaging.read_model(path)
    assert got_cfg == cfg and sorted(got) == sorted(tensors)
    for k in tensors:
        assert got[k].dtype == tensors[k].dtype and np.array_equal(got[k], tensors[k])
    packaging.add_model(path, cfg, {"normf.g": np.zeros(256, np.float32)})  # replacing keeps the bytecode
    assert sorted(packaging.bytecode_entries(path)) == ["Strict/Examples/Model", "Strict/Number"] and list(packaging.read_model(path)[1]) == ["normf.g"]
    plain = str(tmp_path / "Plain.strictbinary")
    with zipfile.ZipFile(plain, "w") as z:
        z.writestr("A.bytecode", b"x")
    assert packaging.read_model(plain) == (None, {})
    bad = tmp_path / "Bad.strictbinary"
    bad.write_bytes(b"not a zip")
    with pytest.raises(packaging.InvalidFile):
        packaging.read_model(str(bad))
    with pytest.raises(ValueError):
        packaging.add_model(path, cfg, {"x": np.zeros(3, np.int64)})


def test_timeline_groups_blocks_into_launches_and_exposed_times_add_up():
    """strict_b200/timeline.py on hand-made records: two launches of one GEMM shape separated by a
    row kernel, blocks of a launch overlapping in time, marks optional; the exposed times telescope
    to the end of the last launch."""
    from strict_b200 import timeline as TL
    N_, K = 6144, 4096
    gemm = 1 | (((N_ ^ (K << 12)) & 0xFFFFFFFF) << 8)
    row = 2 | (77 << 8)

    def rec(t0, tw, t2, word, sm, marks=(0, 0, 0)):
        return [1000 + t0, 1000 + tw if tw else 0, 1000 + t2, word | (sm << 48), *[1000 + m if m else 0 for m in marks], 0]
    records = np.array([
        rec(0, 50, 400, gemm, 0), rec(10, 55, 420, gemm, 1), rec(5, 52, 390, gemm, 2),      # first GEMM launch, three blocks
        rec(100, 430, 600, row, 3, (450, 500, 0)), rec(110, 431, 610, row, 4, (452, 505, 0)),  # row kernel, resident early
        rec(500, 620, 900, gemm, 0), rec(505, 622, 950, gemm, 1),                             # second GEMM launch
    ], dtype=np.uint64)
    ll = TL.launches(records, {(N_, K): "gemm_qkv"})
    assert [d["kernel"] for d in ll] == ["gemm_qkv", "rownorm", "gemm_qkv"] and [d["blocks"] for d in ll] == [3, 2, 2]
    assert ll[0]["first_start"] == 0 and ll[0]["end"] == 420 and ll[0]["waited"] == 52
    assert ll[1]["marks"] == [451, 502, None] and ll[1]["exposed"] == 610 - 420
    assert sum(d["exposed"] for d in ll) == ll[-1]["end"] == 950
    per = TL.per_kernel(ll)
    assert per["gemm_qkv"] == (420 + (950 - 610), 2) and per["rownorm"] == (190, 1)
    assert TL.launches(np.zeros((0, 8), np.uint64)) == []


def test_build_identity_follows_the_sources(tmp_path):
    from strict_b200 import build
    a = build.source_id()
    assert a == build.source_id() and len(a) == 16 and int(a, 16) >= 0
