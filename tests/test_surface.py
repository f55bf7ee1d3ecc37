"""CPU tests of the host-side mirror: the emitted CUDA C text the reference's own tests pin
(Strict.Compiler.Cuda.Tests/InstructionsToCudaTests.cs:13-52), the C# scraper
(CSharpToCudaTranspilerTests.cs:20-41), and the C-ABI: the shared library loads and exports
every symbol include/strictb200.h declares (no compute calls: there is no GPU here)."""
import ctypes
import json
import os
import re

import numpy as np
import pytest

import strict_b200 as sb
from strict_b200 import native

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLD = json.load(open(os.path.join(HERE, "golden", "reference_known_answers.json")))


@pytest.mark.parametrize("case", GOLD["emitted_text"], ids=lambda c: c["signature"].split("(")[0])
def test_emitted_text_matches_reference_pins(case):
    cuda = sb.InstructionsToCuda().Compile(sb.Method(case["signature"], ["\t" + case["body"]]))
    for piece in case["contains"]:
        assert piece in cuda


def test_extension_and_count_parameter():
    assert sb.InstructionsToCuda.Extension == ".cu"
    m = sb.InstructionsToCuda().compile(sb.Method("Scale(input Number, width Number) Number", ["\tinput * 2.5"]))
    assert "const int width, float *output, const int count" in m.cuda  # count stays unless width AND height exist
    assert "idx >= count" in m.cuda and "output[idx] = input[idx] * 2.5" in m.cuda
    assert m.consts == [2.5]


def test_lowering_to_register_program():
    m = sb.InstructionsToCuda().compile(sb.Method("F(a Number, b Number, c Number) Number", ["\t(a + b) * c - 1"]))
    ops = [c[0] for c in m.code]
    assert ops == [0, 0, 3, 0, 5, 2, 4, 7]
    assert "output[idx] = ((a[idx] + b[idx]) * c[idx]) - 1" in m.cuda
    with pytest.raises(NotImplementedError):
        sb.Method("F(a Number) Number", ["\ta ^ 2"])
    with pytest.raises(NotImplementedError):
        sb.InstructionsToCuda().compile(sb.Method("F(a Number) Number", ["\tb + 1"]))


CS_ADD = "﻿public class AddNumbers\n{\n\tpublic float Add(float first, float second)\n\t{\n\t\treturn first + second;\n\t}\n}"
CS_DEPTH = ("namespace X;\n\npublic class InitializeDepths : DepthImageProcessor\n{\n"
            "\tpublic InitializeDepths(float initialDepth = 1) =>\n\t\tthis.initialDepth = initialDepth;\n\n"
            "\tprivate readonly float initialDepth;\n\n\tpublic void Process(DepthImage depthImage)\n\t{\n"
            "\t\tfor (var y = 0; y < depthImage.Height; y++)\n\t\tfor (var x = 0; x < depthImage.Width; x++)\n"
            "\t\t\tdepthImage.Depths[y * depthImage.Width + x] = initialDepth;\n\t}\n}")


def test_csharp_scraper():
    t = sb.CSharpToCudaTranspiler()
    with pytest.raises(sb.InvalidCode):
        t.Convert("")
    ty = t.ParseCSharp("AddNumbers.cs", CS_ADD)
    assert ty.Name == "AddNumbers" and len(ty.Methods) == 1 and ty.Methods[0].Name == "Add"
    assert ty.Methods[0].Parameters == ["first", "second"] and ty.Methods[0].body_text == "first + second"
    assert "output[idx] = first[idx] + second[idx]" in t.GenerateCuda(ty)
    ty = t.ParseCSharp("InitializeDepths.cs", CS_DEPTH)
    assert ty.Methods[0].Name == "Process" and ty.Methods[0].Parameters == ["input", "width", "height", "initialDepth"]
    assert "output[idx] = initialDepth" in t.GenerateCuda(ty)
    with pytest.raises(sb.MissingReturnStatement):
        t.ParseCSharp("MissingReturnStatement.cs", "\tfirst + second;")


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "strictb200.h")).read()
    declared = set(re.findall(r"\b(strictb200_[a-z0-9_]+)\s*\(", header))
    assert len(declared) > 50
    lib = native.lib()  # raises if the library was not built
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, missing
    # the ctypes table binds exactly the declared functions
    assert set(native.SIGNATURES) | {"strictb200_version", "strictb200_last_error", "strictb200_build_id"} == declared
    # the binary says which sources it was built from; after a build they are the ones beside it
    from strict_b200 import build
    assert lib.strictb200_build_id().decode().split()[0] == build.source_id()
    assert lib.strictb200_version() == int(re.search(r"#define STRICTB200_VERSION (\d+)", header).group(1))


def test_struct_layout_matches_header():
    assert ctypes.sizeof(native.ModelConfig) == 12 * 4
    c = sb.model.make_config(sb.CONFIGS["qwen3-8b"])
    assert (c.n_layers, c.d_model, c.n_q_heads, c.n_kv_heads, c.head_dim, c.d_ff, c.vocab, c.tied) == (36, 4096, 32, 8, 128, 12288, 151936, 0)


def test_null_handles_fail_cleanly_without_gpu():
    lib = native.lib()
    assert lib.strictb200_destroy(None) == 0  # destroy(NULL) is a no-op
    assert lib.strictb200_model_destroy(None) == 0 and lib.strictb200_kv_destroy(None) == 0
    assert lib.strictb200_synchronize(None) == native.ERR_INVALID_ARG
    assert b"null context" in lib.strictb200_last_error()
    with pytest.raises(ValueError):
        native.check(lib.strictb200_ew_binary(None, 0, None, None, None, 1))


def test_benchmark_configs():
    q8 = sb.CONFIGS["qwen3-8b"]
    D = q8["head_dim"]
    per_layer = (q8["n_q_heads"] + 2 * q8["n_kv_heads"]) * D * q8["d_model"] + q8["d_model"] * q8["n_q_heads"] * D + 3 * q8["d_model"] * q8["d_ff"]
    assert per_layer == 192_937_984 and per_layer * q8["n_layers"] == 6_945_767_424
    assert q8["vocab"] * q8["d_model"] == 622_329_856
    assert 2 * q8["n_kv_heads"] * D * 2 * q8["n_layers"] == 147_456  # KV bytes per token
    g = sb.CONFIGS["gpt2-small"]
    layers = g["n_layers"] * (4 * g["d_model"] ** 2 + 2 * g["d_model"] * g["d_ff"] + 4 * g["d_model"] + 3 * g["d_model"] + g["d_ff"] + g["d_model"] + 2 * g["d_model"])
    assert abs(layers - 85_054_464) < 200_000
