"""Routing of Strict's numeric loops to the library: the call site the reference lacks.

The reference's Runner.Build only instantiates the MLIR, LLVM and NASM back ends
(Strict/Runner.cs:71-82, Strict/CompilerBackend.cs:3-8); nothing routes a loop to its CUDA
project. Its MLIR emitter already decides per loop how to run it, from the product of iteration
count and body size (Strict.Compiler.Assembly/InstructionsToMlir.cs:396-418): sequential below
ComplexityThreshold, parallel on the CPU above it, on the GPU above GpuComplexityThreshold. This
module mirrors that rule and adds the missing branches: a `Cuda` back end for Build, which writes
the emitted kernel text next to the source as the other back ends write their IR
(Runner.cs:83-84), and TryRunOnGpu, which runs a data-parallel method over whole arrays through
the library when the rule says GPU and otherwise leaves it to the host's own VM (None) — the
library has no CPU path of its own.
"""
import asyncio
import os

from . import instructions_to_cuda as itc

ComplexityThreshold = 100_000          # InstructionsToMlir.cs:414
GpuComplexityThreshold = 10_000_000    # InstructionsToMlir.cs:418


class CompilerBackend:
    """Strict/CompilerBackend.cs:3-8, plus the CUDA back end."""
    MlirDefault, Llvm, Nasm, Cuda = "MlirDefault", "Llvm", "Nasm", "Cuda"


def EstimateComplexity(iterations, body_instruction_count):
    """iterations x max(body, 1) (Strict.Compiler.Assembly.Tests/BlurPerformanceTests.cs:166-167)."""
    return int(iterations) * max(int(body_instruction_count), 1)


def ChooseStrategy(iterations, body_instruction_count):
    """'scf.for' | 'scf.parallel' | 'gpu.launch', the three branches of InstructionsToMlir.cs:403-409."""
    complexity = EstimateComplexity(iterations, body_instruction_count)
    if complexity > GpuComplexityThreshold:
        return "gpu.launch"
    if complexity > ComplexityThreshold:
        return "scf.parallel"
    return "scf.for"


def BodyInstructionCount(compiled):
    """Instructions of the method's bytecode, the count CountLoopBodyInstructions takes between
    LoopBegin and LoopEnd (InstructionsToMlir.cs:420-432): here the whole method is the loop body."""
    return len(compiled.instructions)


class Runner:
    """The part of Strict/Runner.cs this path touches: Build with a chosen back end and the
    routing of data-parallel methods."""

    def __init__(self, strict_file_path, type_):
        self.strictFilePath = strict_file_path
        self.type = type_
        self.binary = itc.BinaryExecutable(type_)

    def Build(self, platform=itc.Platform.Linux, backend=CompilerBackend.Cuda):
        """Writes <source>.cu with the entry point's kernel and returns its path (Runner.cs:83-84).
        The other back ends belong to the reference's toolchain and are not part of this library."""
        if backend != CompilerBackend.Cuda:
            raise NotImplementedError(f"back end {backend} belongs to the reference's toolchain; this library provides {CompilerBackend.Cuda}")
        compiler = itc.InstructionsToCuda()
        text = asyncio.run(compiler.Compile(self.binary, platform))
        path = os.path.splitext(self.strictFilePath)[0] + compiler.Extension
        with open(path, "w") as f:
            f.write(text)
        return path

    def Plan(self, method_name, count):
        compiled = itc.CompiledMethod(self.type.by_name[method_name], self.type)
        return ChooseStrategy(count, BodyInstructionCount(compiled)), compiled

    def TryRunOnGpu(self, ctx, method_name, *args):
        """Runs `method_name` over its array arguments on the GPU if the complexity rule picks
        gpu.launch; returns the output DeviceVariable, or None when the loop stays with the host.
        args: as CompiledMethod.launch (parameters, output, [count])."""
        compiled = itc.CompiledMethod(self.type.by_name[method_name], self.type)
        if compiled.needs_count:
            count = int(args[-1])
        else:
            by_name = dict(zip(compiled.method.Parameters, args))
            count = int(by_name["width"]) * int(by_name["height"])
        if ChooseStrategy(count, BodyInstructionCount(compiled)) != "gpu.launch":
            return None
        return compiled.launch(ctx, *args)
