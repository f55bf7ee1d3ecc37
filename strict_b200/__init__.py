"""strict_b200 — host-side mirror of the Strict CUDA surface over libstrictb200.so (sm_100a).

Importing the package does not load the native library; the first Context()/lib() call does,
and raises if the library has not been built or no B200 is present (there is no CPU path).
"""
from .native import KernelException, lib, LIB_PATH  # noqa: F401
from .kernel import Context, DeviceVariable, FlatNumbers, Kernel, blur5x5_rgb8  # noqa: F401
from .instructions_to_cuda import (BinaryExecutable, CSharpToCudaTranspiler, CSharpType, InstructionsCompiler,  # noqa: F401
                                   InstructionsToCuda, InvalidCode, Method, MissingReturnStatement, Platform, StrictType)
from .model import CONFIGS, GPT2, QWEN3, KvCache, Model  # noqa: F401
from .runner import ChooseStrategy, CompilerBackend, ComplexityThreshold, EstimateComplexity, GpuComplexityThreshold, Runner  # noqa: F401
from . import packaging  # noqa: F401
