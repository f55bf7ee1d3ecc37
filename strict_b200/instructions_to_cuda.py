"""Mirror of Strict.Compiler.Cuda.InstructionsToCuda and CSharpToCudaTranspiler.

The reference turns a one-expression Strict method into the text of an element-wise CUDA C
kernel (Strict.Compiler.Cuda/InstructionsToCuda.cs:25-74) and, in its tests, compiles that
text with NVRTC. Here the same text is still produced (so string-level tests read the same),
but execution goes through an ahead-of-time sm_100a kernel: the method is lowered to the
instruction subset the emitter handles — LoadVariableToRegister, LoadConstantInstruction,
non-conditional BinaryInstruction, ReturnInstruction (cs:31-53) — and that register program
is what `strictb200_ew_program` (or `strictb200_ew_binary` for a single operator) runs.

One deliberate difference: the reference concatenates sub-expression strings without
parentheses (cs:44-48), so `(a + b) * c` is emitted as `a[idx] + b[idx] * c[idx]`. Nested
operands are parenthesised here, in the text and in the program alike.
"""
import ctypes as C
import re

import numpy as np

from . import native as N

SCALAR_PARAMETERS = ("width", "height", "initialDepth")  # InstructionsToCuda.cs:97-98
OPERATORS = {"+": 3, "-": 4, "*": 5, "/": 6}  # opcode of strictb200_ew_program
LOAD_ARRAY, LOAD_SCALAR, LOAD_CONST, RETURN = 0, 1, 2, 7


class InvalidCode(Exception):
    """CSharpToCudaTranspiler.InvalidCode (CSharpToCudaTranspiler.cs:28)."""


class MissingReturnStatement(Exception):
    """CSharpType.MissingReturnStatement (CSharpToCudaTranspiler.cs:77)."""


# ---------------------------------------------------------------- tiny expression front end
_TOKEN = re.compile(r"\s*(?:(\d+\.?\d*(?:[eE][-+]?\d+)?)|([A-Za-z_]\w*)|(.))")


def _tokenize(text):
    out = []
    for num, ident, op in _TOKEN.findall(text):
        if num:
            out.append(("num", num))
        elif ident:
            out.append(("id", ident))
        elif op.strip():
            out.append(("op", op))
    return out


class _Parser:
    """Binary + - * / with the usual precedence, left associative, parentheses."""

    def __init__(self, text):
        self.t = _tokenize(text)
        self.i = 0

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None)

    def take(self):
        tok = self.peek()
        self.i += 1
        return tok

    def parse(self):
        node = self.expr()
        if self.peek()[0] is not None:
            raise NotImplementedError(f"unsupported expression near {self.peek()[1]!r}")
        return node

    def expr(self):
        node = self.term()
        while self.peek() in (("op", "+"), ("op", "-")):
            op = self.take()[1]
            node = ("bin", op, node, self.term())
        return node

    def term(self):
        node = self.atom()
        while self.peek() in (("op", "*"), ("op", "/")):
            op = self.take()[1]
            node = ("bin", op, node, self.atom())
        return node

    def atom(self):
        kind, val = self.take()
        if kind == "num":
            return ("num", float(val), val)
        if kind == "id":
            return ("var", val)
        if (kind, val) == ("op", "("):
            node = self.expr()
            if self.take() != ("op", ")"):
                raise NotImplementedError("unbalanced parenthesis")
            return node
        raise NotImplementedError(f"unsupported expression near {val!r}")  # NotSupportedException, cs:108


class Method:
    """What the emitter reads of a Strict `Method`: Name, Parameters, one body expression.
    Built from the Strict lines the reference's tests use, e.g.
    Method("Add(first Number, second Number) Number", ["\\tfirst + second"])."""

    def __init__(self, signature_line, body_lines):
        m = re.match(r"\s*(\w+)\s*(?:\((.*)\))?\s*(\w+)?\s*$", signature_line)
        if not m:
            raise InvalidCode(signature_line)
        self.Name = m.group(1)
        self.Parameters = []
        if m.group(2):
            for part in m.group(2).split(","):
                bits = part.split()
                if len(bits) != 2 or bits[1] != "Number":
                    raise NotImplementedError(part.strip())
                self.Parameters.append(bits[0])
        body = [l.strip() for l in body_lines if l.strip()]
        if len(body) != 1:
            raise NotImplementedError("only one-expression methods are supported")
        self.body_text = body[0]
        self.body = _Parser(self.body_text).parse()


class CompiledMethod:
    """Result of InstructionsToCuda.compile: the CUDA C text plus the launchable program."""

    def __init__(self, method):
        self.method = method
        params = method.Parameters
        self.arrays = [p for p in params if p not in SCALAR_PARAMETERS]
        self.scalars = [p for p in params if p in SCALAR_PARAMETERS]
        self.needs_count = not ("width" in params and "height" in params)  # cs:76-77
        self.code, self.consts = [], []
        self._next = 0
        ret, self.expression = self._lower(method.body, top=True)
        self.code.append((RETURN, ret, 0, 0))
        if len(self.code) > 64 or len(self.consts) > 16:
            raise NotImplementedError("method too large for the element-wise kernel")
        self.cuda = self._emit()

    def _reg(self):
        if self._next >= 16:  # Strict.Bytecode/Register.cs:8-26
            raise NotImplementedError("expression needs more than 16 registers")
        self._next += 1
        return self._next - 1

    def _lower(self, node, top=False):
        kind = node[0]
        if kind == "var":
            name = node[1]
            r = self._reg()
            if name in self.arrays:
                self.code.append((LOAD_ARRAY, self.arrays.index(name), 0, r))
                return r, name + "[idx]"
            if name in self.scalars:
                self.code.append((LOAD_SCALAR, self.scalars.index(name), 0, r))
                return r, name
            raise NotImplementedError(f"unknown identifier {name}")
        if kind == "num":
            r = self._reg()
            self.consts.append(node[1])
            self.code.append((LOAD_CONST, len(self.consts) - 1, 0, r))
            text = node[2]
            return r, text
        _, op, lhs, rhs = node
        ra, ta = self._lower(lhs)
        rb, tb = self._lower(rhs)
        if lhs[0] == "bin":
            ta = "(" + ta + ")"
        if rhs[0] == "bin":
            tb = "(" + tb + ")"
        r = self._reg()
        self.code.append((OPERATORS[op], ra, rb, r))
        return r, f"{ta} {op} {tb}"

    def _emit(self):
        decl = []
        for p in self.method.Parameters:  # cs:85-96
            if p in ("width", "height"):
                decl.append(f"const int {p}")
            elif p in SCALAR_PARAMETERS:
                decl.append(f"const float {p}")
            else:
                decl.append(f"const float *{p}")
        decl.append("float *output")
        if self.needs_count:
            decl.append("const int count")
        bounds = "idx >= count" if self.needs_count else "x >= width || y >= height"  # cs:79-83
        return (f'extern "C" __global__ void {self.method.Name}({", ".join(decl)})\n{{\n'
                "\tint x = blockIdx.x * blockDim.x + threadIdx.x;\n"
                "\tint y = blockIdx.y * blockDim.y + threadIdx.y;\n"
                "\tint idx = y * blockDim.x + x;\n"
                f"  if ({bounds}) return;\n"
                f"\toutput[idx] = {self.expression};\n}}")

    def launch(self, ctx, *args):
        """args in the order of the emitted signature: parameters, output, [count]."""
        params = self.method.Parameters
        want = len(params) + 1 + (1 if self.needs_count else 0)
        if len(args) != want:
            raise ValueError(f"{self.method.Name} takes {want} arguments")
        by_name = dict(zip(params, args))
        output = args[len(params)]
        if self.needs_count:
            count = int(args[-1])
        else:
            count = int(by_name["width"]) * int(by_name["height"])
        arrays = [by_name[a] for a in self.arrays]
        # single operator over two arrays: the streaming fast path
        if len(self.code) == 4 and [c[0] for c in self.code[:2]] == [LOAD_ARRAY, LOAD_ARRAY] and self.code[2][0] in OPERATORS.values():
            a, b = arrays[self.code[0][1]], arrays[self.code[1][1]]
            N.check(N.lib().strictb200_ew_binary(ctx.h, self.code[2][0] - 3, a.p, b.p, output.p, count))
            return output
        code = np.array(self.code, np.int32)
        ptrs = (C.c_void_p * max(1, len(arrays)))(*[a.p.value for a in arrays])
        scal = np.array([float(by_name[s]) for s in self.scalars] or [0.0], np.float32)
        cons = np.array(self.consts or [0.0], np.float32)
        N.check(N.lib().strictb200_ew_program(ctx.h, N.ptr(code), len(self.code), ptrs, len(arrays), N.ptr(scal), len(self.scalars),
                                              N.ptr(cons), len(self.consts), output.p, count))
        return output


class InstructionsToCuda:
    """InstructionsToCuda (Strict.Compiler.Cuda/InstructionsToCuda.cs:12-20)."""

    Extension = ".cu"

    def compile(self, method):
        return CompiledMethod(method)

    def Compile(self, method):
        """Returns the CUDA C text, as the reference's Compile(Method) does."""
        return CompiledMethod(method).cuda


class CSharpType:
    """Line-prefix scrape of a C# file into a one-method type (CSharpToCudaTranspiler.cs:42-98)."""

    def __init__(self, type_name, text):
        self.Name = type_name
        method_name, return_type, params, ret = "", "", [], ""
        for line in text.replace("﻿", "").splitlines():
            if self._ignored(line, type_name):
                continue
            if line.startswith("\t\treturn") or line.startswith("\t\t\t"):
                value = line.strip().replace(";", "")
                if value.startswith("return "):
                    value = value[7:]
                elif " = " in value:
                    value = value[value.rindex(" = ") + 3:]
                ret = value
            else:
                parts = [p for p in re.split(r"[ (),]", line.strip()) if p]
                if parts[1] == "float":
                    return_type = " Number"
                method_name = parts[2]
                for i in range(3, len(parts), 2):
                    if parts[i] == "DepthImage":
                        params += ["input Number", "width Number", "height Number", "initialDepth Number"]
                    elif parts[i] != "float":
                        raise NotImplementedError(parts[i + 1])
                    else:
                        params.append(parts[i + 1] + " Number")
        if ret == "":
            raise MissingReturnStatement()
        sig = method_name + ("(" + ", ".join(params) + ")" if params else "") + return_type
        self.Methods = [Method(sig, ["\t" + ret])]

    @staticmethod
    def _ignored(line, type_name):
        return (line == "" or "{" in line or "}" in line or line.startswith("using ") or line.startswith("namespace ")
                or type_name in line or "this." in line or line.startswith("\tprivate ") or line.startswith("\t\tfor "))


class CSharpToCudaTranspiler:
    """CSharpToCudaTranspiler (Strict.Compiler.Cuda/CSharpToCudaTranspiler.cs:10-30)."""

    def ParseCSharp(self, file_path, text=None):
        if file_path == "":
            raise InvalidCode()
        import os
        if text is None:
            with open(file_path, encoding="utf-8-sig") as f:
                text = f.read()
        return CSharpType(os.path.splitext(os.path.basename(file_path))[0], text)

    @staticmethod
    def GenerateCuda(type_):
        return InstructionsToCuda().Compile(type_.Methods[0])

    def Convert(self, file_path):
        return self.GenerateCuda(self.ParseCSharp(file_path))
