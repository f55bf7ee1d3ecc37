"""Mirror of Strict.Compiler.Cuda.InstructionsToCuda, its base InstructionsCompiler, and
CSharpToCudaTranspiler.

The reference turns a one-expression Strict method into the text of an element-wise CUDA C
kernel (Strict.Compiler.Cuda/InstructionsToCuda.cs:25-74) and, in its tests, compiles that
text with NVRTC. Here the same text is still produced (so string-level tests read the same),
but execution goes through ahead-of-time sm_100a kernels: the method's bytecode
(strict_b200/bytecode.py) is lowered to a register program that `strictb200_ew_program` runs
(`strictb200_ew_binary` for a single operator over two arrays). Methods beyond the reference's
subset — conditionals, loops, calls of other methods of the type, loads at computed indices, the
gaps its plan lists (Strict.Compiler.Assembly/GpuSupportPlan.md:63-67) — lower to the larger
instruction set of `strictb200_ew_program2` and emit goto-style CUDA C, which NVRTC accepts.

One deliberate difference: the reference concatenates sub-expression strings without
parentheses (cs:44-48), so `(a + b) * c` is emitted as `a[idx] + b[idx] * c[idx]`. Nested
operands are parenthesised here, in the text and in the program alike.
"""
import ctypes as C
import re

import numpy as np

from . import bytecode as B
from . import native as N

SCALAR_PARAMETERS = ("width", "height", "initialDepth")  # InstructionsToCuda.cs:97-98
OPERATORS = {"+": 3, "-": 4, "*": 5, "/": 6}  # opcode of strictb200_ew_program
LOAD_ARRAY, LOAD_SCALAR, LOAD_CONST, RETURN = 0, 1, 2, 7
# further opcodes of strictb200_ew_program2
MOD, CMP_EQ, CMP_NE, CMP_LT, CMP_GT, JUMP, JUMP_IF_TRUE, JUMP_IF_FALSE, LOOP_BEGIN, LOOP_END, LOAD_AT, MOVE, LOAD_INDEX = range(8, 21)
_ARITH = {B.Add: 3, B.Subtract: 4, B.Multiply: 5, B.Divide: 6, B.Modulo: MOD}
_CMP = {B.Equal: CMP_EQ, B.NotEqual: CMP_NE, B.LessThan: CMP_LT, B.GreaterThan: CMP_GT}
_CTEXT = {3: "+", 4: "-", 5: "*", 6: "/", CMP_EQ: "==", CMP_NE: "!=", CMP_LT: "<", CMP_GT: ">"}
SLOTS, MAX_INSTRUCTIONS, MAX_LOOP_DEPTH = 32, 256, 4


class InvalidCode(Exception):
    """CSharpToCudaTranspiler.InvalidCode (CSharpToCudaTranspiler.cs:28)."""


class MissingReturnStatement(Exception):
    """CSharpType.MissingReturnStatement (CSharpToCudaTranspiler.cs:77)."""


class Method:
    """What the emitter reads of a Strict `Method`: Name, Parameters and the body. Built from
    Strict lines as the reference's tests write them, e.g.
    Method("Add(first Number, second Number) Number", ["\\tfirst + second"]). Bodies of several
    lines (constants, if/else, for, return, calls) follow strict_b200/bytecode.py."""

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
        self.scalars = [p for p in self.Parameters if p in SCALAR_PARAMETERS]
        body = [l for l in body_lines if l.strip()]
        self.statements = B.parse_body(body)
        self.body_text = body[0].strip() if len(body) == 1 else "\n".join(l.rstrip() for l in body)
        self.body = self.statements[0][1] if len(self.statements) == 1 and self.statements[0][0] == "return" else None


class StrictType:
    """A type with several methods that may call each other (an Invoke is resolved against the
    methods of the same type, as InstructionsCompiler.CollectMethods does by method header,
    Strict.Compiler/InstructionsCompiler.cs:53-86)."""

    def __init__(self, name, methods):
        self.Name = name
        self.Methods = list(methods)
        self.by_name = {m.Name: m for m in self.Methods}


def _generate(type_, method):
    others = {n: m for n, m in type_.by_name.items() if n != method.Name}
    return B.BinaryGenerator(type_.Name, method, others).Generate()


class CompiledMethod:
    """Result of InstructionsToCuda.compile: the bytecode, the CUDA C text and the launchable
    register program. One-expression methods produce the reference's text and the
    straight-line program of strictb200_ew_program; anything else the larger instruction set of
    strictb200_ew_program2 and goto-style CUDA C."""

    def __init__(self, method, type_=None):
        self.method = method
        self.type = type_ or StrictType("Kernel", [method])
        params = method.Parameters
        self.arrays = [p for p in params if p not in SCALAR_PARAMETERS]
        self.scalars = [p for p in params if p in SCALAR_PARAMETERS]
        self.needs_count = not ("width" in params and "height" in params)  # cs:76-77
        self.instructions = _generate(self.type, method)
        simple = method.body is not None and all(
            isinstance(i, (B.LoadVariableToRegister, B.LoadConstantInstruction, B.ReturnInstruction))
            or (isinstance(i, B.BinaryInstruction) and not i.IsConditional() and i.InstructionType != B.Modulo)
            for i in self.instructions)
        self.extended = not simple
        self.code, self.consts = [], []
        if simple:
            self._next = 0
            ret, self.expression = self._lower(method.body)
            self.code.append((RETURN, ret, 0, 0))
            if len(self.code) > 64 or len(self.consts) > 16:
                raise NotImplementedError("method too large for the element-wise kernel")
            self.cuda = self._signature() + f"\toutput[idx] = {self.expression};\n}}"
        else:
            self._lower_extended()
            self.cuda = self._emit_extended()

    # ------------------------------------------------------------ one expression (the reference's subset)
    def _reg(self):
        if self._next >= 16:  # Strict.Bytecode/Register.cs:8-26
            raise NotImplementedError("expression needs more than 16 registers")
        self._next += 1
        return self._next - 1

    def _lower(self, node):
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
            return r, node[2]
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

    def _signature(self):
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
                f"  if ({bounds}) return;\n")

    # ------------------------------------------------------------ conditionals, loops, calls, indexed loads
    def _const(self, value):
        if value not in self.consts:
            self.consts.append(value)
        return self.consts.index(value)

    def _lower_extended(self):
        """Instruction list -> quadruples of strictb200_ew_program2. Registers R0..R15 are slots
        0..15, variables get slots from 16 up, a called method's instructions are placed inline
        with its registers mapped to registers that are free at the call."""
        self.slots = {}          # variable name -> slot
        labels, fixups = {}, []  # jump key -> pc ; (pc, key)
        code = self.code

        def slot(name):
            if name not in self.slots:
                if 16 + len(self.slots) >= SLOTS:
                    raise NotImplementedError("more than 16 variables")
                self.slots[name] = 16 + len(self.slots)
            return self.slots[name]

        def place(instructions, reg, prefix, params, result, depth0, chain):
            """reg: register map; prefix: name space of the variables; params: name -> ('array', i) |
            ('scalar', i) | ('slot', s); result: (slot, end label) inside a call, else None."""
            loops = []
            for ins in instructions:
                if isinstance(ins, B.LoadConstantInstruction):
                    code.append((LOAD_CONST, self._const(ins.Constant), 0, reg[ins.Register]))
                elif isinstance(ins, B.LoadVariableToRegister):
                    name, dst = ins.Identifier, reg[ins.Register]
                    if name == "index" and loops:
                        code.append((MOVE, loops[-1][1], 0, dst))
                    elif name == "index" and name not in params:
                        code.append((LOAD_INDEX, 0, 0, dst))  # outside a loop: the element this thread computes
                    elif name in params:
                        kind, i = params[name]
                        code.append({"array": (LOAD_ARRAY, i, 0, dst), "scalar": (LOAD_SCALAR, i, 0, dst), "slot": (MOVE, i, 0, dst)}[kind])
                    else:
                        code.append((MOVE, slot(prefix + name), 0, dst))
                elif isinstance(ins, B.StoreFromRegisterInstruction):
                    code.append((MOVE, reg[ins.Register], 0, slot(prefix + ins.Identifier)))
                elif isinstance(ins, B.BinaryInstruction):
                    if ins.IsConditional():
                        code.append((_CMP[ins.InstructionType], reg[ins.Registers[0]], reg[ins.Registers[1]], 0))
                    else:
                        code.append((_ARITH[ins.InstructionType], reg[ins.Registers[0]], reg[ins.Registers[1]], reg[ins.Registers[2]]))
                elif isinstance(ins, B.JumpToId):
                    fixups.append((len(code), (prefix, ins.Id)))
                    code.append((JUMP_IF_FALSE if ins.InstructionType == B.JumpToIdIfFalse else JUMP_IF_TRUE, 0, 0, 0))
                elif isinstance(ins, B.Jump):
                    fixups.append((len(code), (prefix, ins.Id)))
                    code.append((JUMP, 0, 0, 0))
                elif isinstance(ins, B.JumpToIdEnd):
                    labels[(prefix, ins.Id)] = len(code)
                elif isinstance(ins, B.LoopBeginInstruction):
                    if depth0 + len(loops) >= MAX_LOOP_DEPTH:
                        raise NotImplementedError(f"loops nested deeper than {MAX_LOOP_DEPTH}")
                    index_slot = slot(f"index@{depth0 + len(loops)}")
                    loops.append((len(code), index_slot))
                    code.append((LOOP_BEGIN, reg[ins.Register], 0, index_slot))
                elif isinstance(ins, B.LoopEndInstruction):
                    begin, _ = loops.pop()
                    code.append((LOOP_END, begin, 0, 0))
                    op, a, _, c = code[begin]
                    code[begin] = (op, a, len(code), c)
                elif isinstance(ins, B.ListCallInstruction):
                    kind, i = params.get(ins.Identifier, (None, None))
                    if kind != "array":
                        raise NotImplementedError(f"{ins.Identifier}(index) needs an array parameter of the kernel")
                    code.append((LOAD_AT, i, reg[ins.IndexValueRegister], reg[ins.Register]))
                elif isinstance(ins, B.Invoke):
                    name = ins.MethodInfo.MethodName
                    if name in chain:
                        raise NotImplementedError(f"recursive call of {name}")
                    callee = self.type.by_name[name]
                    body = _generate(self.type, callee)
                    used = sorted({r for i2 in body for r in _registers_of(i2)})
                    free = [reg[r] for r in ins.FreeRegisters if r in reg]
                    if len(used) > len(free):
                        raise NotImplementedError(f"call of {name} needs {len(used)} registers, {len(free)} are free")
                    call_prefix = f"{prefix}{name}#{len(code)}."
                    call_params = {}
                    for pname, areg in zip(callee.Parameters, ins.ArgumentRegisters):
                        s_ = slot(call_prefix + pname)
                        code.append((MOVE, reg[areg], 0, s_))
                        call_params[pname] = ("slot", s_)
                    end = (call_prefix, "end")
                    # the callee's registers in use first, then its spare ones (for calls it makes itself), onto the free ones here
                    order = used + [v for v in range(B.REGISTERS) if v not in used]
                    place(body, dict(zip(order, free)), call_prefix, call_params, (reg[ins.Register], end), depth0 + len(loops), chain + [name])
                    labels[end] = len(code)
                elif isinstance(ins, B.ReturnInstruction):
                    if result is None:
                        code.append((RETURN, reg[ins.Register], 0, 0))
                    else:
                        code.append((MOVE, reg[ins.Register], 0, result[0]))
                        fixups.append((len(code), result[1]))
                        code.append((JUMP, 0, 0, 0))
                else:
                    raise NotImplementedError(type(ins).__name__)

        params = {a: ("array", i) for i, a in enumerate(self.arrays)}
        params.update({s: ("scalar", i) for i, s in enumerate(self.scalars)})
        place(self.instructions, {r: r for r in range(16)}, "", params, None, 0, [self.method.Name])
        for pc, key in fixups:
            op, _, b, c = code[pc]
            code[pc] = (op, labels[key], b, c)
        if len(code) > MAX_INSTRUCTIONS or len(self.consts) > 16:
            raise NotImplementedError("method too large for the element-wise kernel")

    def _emit_extended(self):
        """Goto-style CUDA C of the quadruples: one statement per instruction, a label where a
        jump lands, `for` blocks for the loops. Out-of-range indexed loads read 0."""
        targets = {q[1] for q in self.code if q[0] in (JUMP, JUMP_IF_TRUE, JUMP_IF_FALSE)}
        used = sorted({s for q in self.code for s in _slots_of(q)})
        names = {s: (f"r{s}" if s < 16 else f"v{s}") for s in used}
        lines = [self._signature().rstrip("\n")]
        if used:
            lines.append("\tfloat " + ", ".join(f"{names[s]} = 0.0f" for s in used) + ";")
        lines.append("\tbool flag = false;")
        depth = 0
        for pc, (op, a, b, c) in enumerate(self.code):
            if pc in targets:
                lines.append(f"L{pc}:;")
            ind = "\t" * (1 + depth)
            if op == LOAD_ARRAY:
                lines.append(f"{ind}{names[c]} = {self.arrays[a]}[idx];")
            elif op == LOAD_SCALAR:
                lines.append(f"{ind}{names[c]} = {self.scalars[a]};")
            elif op == LOAD_CONST:
                lines.append(f"{ind}{names[c]} = {self.consts[a]!r}f;")
            elif op in (3, 4, 5, 6):
                lines.append(f"{ind}{names[c]} = {names[a]} {_CTEXT[op]} {names[b]};")
            elif op == MOD:
                lines.append(f"{ind}{names[c]} = fmodf({names[a]}, {names[b]});")
            elif op in (CMP_EQ, CMP_NE, CMP_LT, CMP_GT):
                lines.append(f"{ind}flag = {names[a]} {_CTEXT[op]} {names[b]};")
            elif op == JUMP:
                lines.append(f"{ind}goto L{a};")
            elif op in (JUMP_IF_TRUE, JUMP_IF_FALSE):
                lines.append(f"{ind}if ({'' if op == JUMP_IF_TRUE else '!'}flag) goto L{a};")
            elif op == LOOP_BEGIN:
                lines.append(f"{ind}for (int i{depth} = 0; i{depth} < (int){names[a]}; i{depth}++) {{ {names[c]} = (float)i{depth};")
                depth += 1
            elif op == LOOP_END:
                depth -= 1
                lines.append("\t" * (1 + depth) + "}")
            elif op == LOAD_AT:
                lines.append(f"{ind}{names[c]} = ({names[b]} >= 0.0f && {names[b]} < (float)count) ? {self.arrays[a]}[(int){names[b]}] : 0.0f;")
            elif op == MOVE:
                lines.append(f"{ind}{names[c]} = {names[a]};")
            elif op == LOAD_INDEX:
                lines.append(f"{ind}{names[c]} = (float)idx;")
            elif op == RETURN:
                lines.append(f"{ind}{{ output[idx] = {names[a]}; return; }}")
        if len(self.code) in targets:
            lines.append(f"L{len(self.code)}:;")
        lines.append("\toutput[idx] = 0.0f;")  # a body that ends without a value returns 0 (cs:30)
        lines.append("}")
        return "\n".join(lines)

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
        if (not self.extended and len(self.code) == 4 and [c[0] for c in self.code[:2]] == [LOAD_ARRAY, LOAD_ARRAY]
                and self.code[2][0] in OPERATORS.values()):
            a, b = arrays[self.code[0][1]], arrays[self.code[1][1]]
            N.check(N.lib().strictb200_ew_binary(ctx.h, self.code[2][0] - 3, a.p, b.p, output.p, count))
            return output
        code = np.array(self.code, np.int32)
        ptrs = (C.c_void_p * max(1, len(arrays)))(*[a.p.value for a in arrays])
        scal = np.array([float(by_name[s]) for s in self.scalars] or [0.0], np.float32)
        cons = np.array(self.consts or [0.0], np.float32)
        entry = N.lib().strictb200_ew_program2 if self.extended else N.lib().strictb200_ew_program
        N.check(entry(ctx.h, N.ptr(code), len(self.code), ptrs, len(arrays), N.ptr(scal), len(self.scalars),
                      N.ptr(cons), len(self.consts), output.p, count))
        return output


def _registers_of(ins):
    regs = []
    for attr in ("Register", "IndexValueRegister"):
        if hasattr(ins, attr):
            regs.append(getattr(ins, attr))
    regs += list(getattr(ins, "Registers", [])) + list(getattr(ins, "ArgumentRegisters", []))
    return regs


def _slots_of(q):
    op, a, b, c = q
    if op in (LOAD_ARRAY, LOAD_SCALAR, LOAD_CONST, LOAD_INDEX):
        return [c]
    if op in (3, 4, 5, 6, MOD):
        return [a, b, c]
    if op in (CMP_EQ, CMP_NE, CMP_LT, CMP_GT):
        return [a, b]
    if op == RETURN:
        return [a]
    if op == LOOP_BEGIN:
        return [a, c]
    if op == LOAD_AT:
        return [b, c]
    if op == MOVE:
        return [a, c]
    return []


class Platform:
    """Strict.Compiler/Platform.cs."""
    Linux, Windows, MacOS = "Linux", "Windows", "MacOS"


class BinaryExecutable:
    """What InstructionsCompiler.Compile reads of a Strict.Bytecode.BinaryExecutable: the entry
    point's instruction list and the methods per type (BinaryExecutable.cs:19). Built here from a
    StrictType whose `Run` method (or first method) is the entry point."""

    class _Entry:
        def __init__(self, instructions):
            self.instructions = instructions

    def __init__(self, type_):
        self.type = type_
        self.entry_method = type_.by_name.get("Run", type_.Methods[0])
        self.EntryPoint = self._Entry(_generate(type_, self.entry_method))
        self.MethodsPerType = {type_.Name: {m.Name: m for m in type_.Methods}}


class InstructionsCompiler:
    """The contract every back end of the reference implements
    (Strict.Compiler/InstructionsCompiler.cs:9-116): `Compile(binary, platform)` returns the
    emitted source text (a Task<string> in C#: an awaitable here), `Extension` names the file
    type; CollectMethods gathers the methods an instruction list invokes, by method header."""

    Extension = ""

    def Compile(self, binary, platform):
        raise NotImplementedError("abstract: InstructionsCompiler.Compile(BinaryExecutable, Platform)")

    @staticmethod
    def BuildMethodHeaderKey(method_name, parameter_names, return_type="Number"):
        """InstructionsCompiler.cs:11-17: Name(p1, p2) ReturnType, or Name ReturnType without parameters."""
        if not parameter_names:
            return method_name if return_type == "None" else f"{method_name} {return_type}"
        return f"{method_name}({', '.join(parameter_names)}) {return_type}"

    @classmethod
    def CollectMethods(cls, instructions, binary):
        """Header key -> method for everything `instructions` invokes, transitively (cs:53-86)."""
        found, queue = {}, [i.MethodInfo for i in instructions if isinstance(i, B.Invoke)]
        while queue:
            info = queue.pop(0)
            key = cls.BuildMethodHeaderKey(info.MethodName, info.ParameterNames, info.ReturnTypeName)
            if key in found:
                continue
            methods = binary.MethodsPerType.get(info.TypeFullName, {})
            if info.MethodName not in methods:
                continue
            found[key] = methods[info.MethodName]
            queue += [i.MethodInfo for i in _generate(binary.type, methods[info.MethodName]) if isinstance(i, B.Invoke)]
        return found


class InstructionsToCuda(InstructionsCompiler):
    """InstructionsToCuda (Strict.Compiler.Cuda/InstructionsToCuda.cs:12-20)."""

    Extension = ".cu"

    def compile(self, method, type_=None):
        return CompiledMethod(method, type_)

    def Compile(self, method_or_binary, platform=None):
        """Compile(Method) returns the CUDA C text (cs:19-20). Compile(BinaryExecutable, Platform)
        is the InstructionsCompiler contract (cs:14-15): an awaitable that yields the text of the
        entry point's kernel — named Run, no parameters, with a count, as the reference builds it."""
        if isinstance(method_or_binary, BinaryExecutable):
            binary = method_or_binary

            async def task():
                return CompiledMethod(binary.entry_method, binary.type).cuda
            return task()
        return CompiledMethod(method_or_binary).cuda


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
