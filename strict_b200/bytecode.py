"""The part of Strict's register bytecode the CUDA back end consumes, and a generator for it.

The reference's CUDA emitter reads the instruction list a BinaryGenerator produces for a method
(Strict.Compiler.Cuda/InstructionsToCuda.cs:19-20) and handles LoadVariableToRegister,
LoadConstantInstruction, non-conditional BinaryInstruction and ReturnInstruction only
(cs:31-53); its plan lists what is missing for real data-parallel kernels: conditionals, loops,
method calls and per-element loads at computed indices
(Strict.Compiler.Assembly/GpuSupportPlan.md:63-67). This module mirrors the instruction classes
of Strict.Bytecode/Instructions (same names and fields, InstructionType values of
Strict.Bytecode/InstructionType.cs:9-47) for that larger subset and generates them from method
bodies written in a small subset of Strict:

    constant NAME = EXPR | mutable NAME = EXPR | NAME = EXPR
    if EXPR (is | is not | < | >) EXPR            (indented block, optional `else` block)
    for EXPR                                      (indented block; `index` counts from 0; outside a
                                                   loop `index` is the element the thread computes)
    return EXPR | EXPR                            (the last line's value is returned)

with expressions over + - * / %, numbers, parameters (array parameters mean "this thread's
element"), `index`, `NAME(EXPR)` on an array parameter (the element at that index) and
`NAME(EXPR, ...)` on another method of the same type (an Invoke). 16 registers
(Strict.Bytecode/Register.cs:8-26)."""
import re

# Strict.Bytecode/InstructionType.cs:9-47
LoadConstantToRegister, LoadVariableToRegisterType, StoreConstantToVariable, StoreRegisterToVariable, Set, ListCall = 0, 1, 2, 3, 4, 5
Add, Subtract, Multiply, Divide, Modulo = 11, 12, 13, 14, 15
ArithmeticSeparator = 20
Equal, NotEqual, LessThan, GreaterThan = 21, 22, 23, 24
BinaryOperatorsSeparator = 30
InvokeType, Return, LoopBegin, LoopEnd, JumpType, JumpIfTrue, JumpIfFalse, JumpIfNotZero, JumpEnd, JumpToIdIfFalse, JumpToIdIfTrue = range(31, 42)

ARITHMETIC = {"+": Add, "-": Subtract, "*": Multiply, "/": Divide, "%": Modulo}
COMPARISON = {"is": Equal, "is not": NotEqual, "<": LessThan, ">": GreaterThan}
SYMBOL = {Add: "+", Subtract: "-", Multiply: "*", Divide: "/"}
REGISTERS = 16


class Instruction:
    def __init__(self, instruction_type):
        self.InstructionType = instruction_type

    def __repr__(self):
        fields = ", ".join(f"{k}={v!r}" for k, v in self.__dict__.items() if k != "InstructionType")
        return f"{type(self).__name__}({fields})"


class RegisterInstruction(Instruction):
    def __init__(self, instruction_type, register):
        super().__init__(instruction_type)
        self.Register = register


class LoadConstantInstruction(RegisterInstruction):
    def __init__(self, register, constant):
        super().__init__(LoadConstantToRegister, register)
        self.Constant = float(constant)
        self.Text = constant if isinstance(constant, str) else repr(float(constant))


class LoadVariableToRegister(RegisterInstruction):
    def __init__(self, register, identifier):
        super().__init__(LoadVariableToRegisterType, register)
        self.Identifier = identifier


class StoreFromRegisterInstruction(RegisterInstruction):
    def __init__(self, register, identifier):
        super().__init__(StoreRegisterToVariable, register)
        self.Identifier = identifier


class BinaryInstruction(Instruction):
    def __init__(self, instruction_type, *registers):
        super().__init__(instruction_type)
        self.Registers = list(registers)

    def IsConditional(self):  # BinaryInstruction.cs: between the two separators
        return ArithmeticSeparator < self.InstructionType < BinaryOperatorsSeparator


class JumpToId(Instruction):
    def __init__(self, id_, instruction_type):
        super().__init__(instruction_type)
        self.Id = id_


class JumpToIdEnd(Instruction):
    def __init__(self, id_):
        super().__init__(JumpEnd)
        self.Id = id_


class Jump(Instruction):
    """Unconditional jump over the `else` block; resolved by Id like the conditional ones."""

    def __init__(self, id_):
        super().__init__(JumpType)
        self.Id = id_


class LoopBeginInstruction(RegisterInstruction):
    def __init__(self, register):
        super().__init__(LoopBegin, register)  # the register holds the iteration count


class LoopEndInstruction(Instruction):
    def __init__(self, begin):
        super().__init__(LoopEnd)
        self.Begin = begin


class ListCallInstruction(RegisterInstruction):
    def __init__(self, register, index_value_register, identifier):
        super().__init__(ListCall, register)
        self.IndexValueRegister = index_value_register
        self.Identifier = identifier


class InvokeMethodInfo:
    def __init__(self, type_full_name, method_name, parameter_names, return_type_name="Number"):
        self.TypeFullName, self.MethodName = type_full_name, method_name
        self.ParameterNames, self.ReturnTypeName = list(parameter_names), return_type_name


class Invoke(RegisterInstruction):
    """Arguments are in ArgumentRegisters, the result goes to Register (Invoke.cs)."""

    def __init__(self, register, method_info, argument_registers):
        super().__init__(InvokeType, register)
        self.MethodInfo = method_info
        self.ArgumentRegisters = list(argument_registers)


class ReturnInstruction(RegisterInstruction):
    def __init__(self, register):
        super().__init__(Return, register)


# ---------------------------------------------------------------- front end
_TOKEN = re.compile(r"\s*(?:(\d+\.?\d*(?:[eE][-+]?\d+)?)|([A-Za-z_]\w*)|(.))")


def tokenize(text):
    out = []
    for num, ident, op in _TOKEN.findall(text):
        if num:
            out.append(("num", num))
        elif ident:
            out.append(("id", ident))
        elif op.strip():
            out.append(("op", op))
    return out


class ExpressionParser:
    """+ - * / % with the usual precedence, left associative, parentheses, calls NAME(args)."""

    def __init__(self, tokens):
        self.t, self.i = tokens, 0

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
        while self.peek() in (("op", "*"), ("op", "/"), ("op", "%")):
            op = self.take()[1]
            node = ("bin", op, node, self.atom())
        return node

    def atom(self):
        kind, val = self.take()
        if kind == "num":
            return ("num", float(val), val)
        if kind == "id":
            if self.peek() == ("op", "("):
                self.take()
                args = []
                if self.peek() != ("op", ")"):
                    args.append(self.expr())
                    while self.peek() == ("op", ","):
                        self.take()
                        args.append(self.expr())
                if self.take() != ("op", ")"):
                    raise NotImplementedError("unbalanced parenthesis")
                return ("call", val, args)
            return ("var", val)
        if (kind, val) == ("op", "("):
            node = self.expr()
            if self.take() != ("op", ")"):
                raise NotImplementedError("unbalanced parenthesis")
            return node
        if (kind, val) == ("op", "-"):  # unary minus: 0 - x
            return ("bin", "-", ("num", 0.0, "0"), self.atom())
        raise NotImplementedError(f"unsupported expression near {val!r}")  # NotSupportedException, InstructionsToCuda.cs:108


def parse_expression(text):
    return ExpressionParser(tokenize(text)).parse()


def parse_condition(text):
    """EXPR (is not | is | < | >) EXPR at the top level of the line."""
    toks = tokenize(text)
    depth = 0
    for i, (kind, val) in enumerate(toks):
        if (kind, val) == ("op", "("):
            depth += 1
        elif (kind, val) == ("op", ")"):
            depth -= 1
        elif depth == 0:
            op, width = None, 1
            if (kind, val) == ("id", "is"):
                op = "is"
                if i + 1 < len(toks) and toks[i + 1] == ("id", "not"):
                    op, width = "is not", 2
            elif kind == "op" and val in "<>":
                op = val
            if op:
                return ("cond", op, ExpressionParser(toks[:i]).parse(), ExpressionParser(toks[i + width:]).parse())
    raise NotImplementedError(f"unsupported condition {text!r}")


def parse_block(lines, depth):
    """lines: list of (indent, text). Returns (statements, remaining lines)."""
    stmts = []
    while lines and lines[0][0] >= depth:
        indent, text = lines[0]
        if indent > depth:
            raise NotImplementedError(f"unexpected indentation before {text!r}")
        lines = lines[1:]
        m = re.match(r"(constant|mutable)\s+(\w+)\s*=\s*(.+)$", text)
        if m:
            stmts.append(("let", m.group(2), parse_expression(m.group(3))))
        elif text.startswith("if "):
            body, lines = parse_block(lines, depth + 1)
            other = []
            if lines and lines[0] == (depth, "else"):
                other, lines = parse_block(lines[1:], depth + 1)
            stmts.append(("if", parse_condition(text[3:]), body, other))
        elif text.startswith("for "):
            body, lines = parse_block(lines, depth + 1)
            stmts.append(("for", parse_expression(text[4:]), body))
        elif text.startswith("return "):
            stmts.append(("return", parse_expression(text[7:])))
        elif re.match(r"\w+\s*=[^=]", text):
            name, rhs = text.split("=", 1)
            stmts.append(("set", name.strip(), parse_expression(rhs)))
        else:
            stmts.append(("value", parse_expression(text)))
    return stmts, lines


def parse_body(body_lines):
    lines = []
    for raw in body_lines:
        if not raw.strip():
            continue
        indent = len(raw) - len(raw.lstrip("\t"))
        lines.append((indent, raw.strip()))
    if not lines:
        raise NotImplementedError("empty method body")
    stmts, rest = parse_block(lines, lines[0][0])
    if rest:
        raise NotImplementedError(f"unexpected indentation before {rest[0][1]!r}")
    _tail_returns(stmts)
    return stmts


def _tail_returns(stmts):
    """The value of a method is the value of its last line; where that line is an `if`, the last
    lines of its blocks."""
    if not stmts:
        return
    last = stmts[-1]
    if last[0] == "value":
        stmts[-1] = ("return", last[1])
    elif last[0] == "if":
        _tail_returns(last[2])
        _tail_returns(last[3])


# ---------------------------------------------------------------- generator
class BinaryGenerator:
    """Statements of one method -> instruction list (the role of Strict.Bytecode/BinaryGenerator
    for this subset). `arrays` and `scalars` are the method's parameter names by kind, `methods`
    the other methods of the type by name (for Invoke)."""

    def __init__(self, type_name, method, methods=None):
        self.type_name, self.method, self.methods = type_name, method, methods or {}
        self.instructions = []
        self.free = list(range(REGISTERS))
        self.locals = set()
        self.next_id = 0
        self.loop_depth = 0

    def reg(self):
        if not self.free:
            raise NotImplementedError("expression needs more than 16 registers")
        return self.free.pop(0)

    def release(self, r):
        if r not in self.free:
            self.free.insert(0, r)
            self.free.sort()

    def emit(self, ins):
        self.instructions.append(ins)
        return ins

    def Generate(self):
        self.block(self.method.statements)
        return self.instructions

    def expression(self, node):
        kind = node[0]
        if kind == "num":
            r = self.reg()
            self.emit(LoadConstantInstruction(r, node[2]))
            return r
        if kind == "var":
            name = node[1]
            if name != "index" and name not in self.locals and name not in self.method.Parameters:
                raise NotImplementedError(f"unknown identifier {name}")
            r = self.reg()
            self.emit(LoadVariableToRegister(r, name))
            return r
        if kind == "call":
            _, name, args = node
            if name in self.method.Parameters and name not in self.method.scalars:
                if len(args) != 1:
                    raise NotImplementedError(f"{name}(...) takes one index")
                ri = self.expression(args[0])
                r = self.reg()
                self.emit(ListCallInstruction(r, ri, name))
                self.release(ri)
                return r
            if name in self.methods:
                callee = self.methods[name]
                if len(args) != len(callee.Parameters):
                    raise NotImplementedError(f"{name} takes {len(callee.Parameters)} arguments")
                regs = [self.expression(a) for a in args]
                r = self.reg()
                call = self.emit(Invoke(r, InvokeMethodInfo(self.type_name, name, callee.Parameters), regs))
                call.FreeRegisters = list(self.free)  # registers the callee's body may use when placed inline
                for a in regs:
                    self.release(a)
                return r
            raise NotImplementedError(f"unknown method {name}")
        _, op, lhs, rhs = node
        ra, rb = self.expression(lhs), self.expression(rhs)
        r = self.reg()
        self.emit(BinaryInstruction(ARITHMETIC[op], ra, rb, r))
        self.release(ra)
        self.release(rb)
        return r

    def block(self, stmts):
        for st in stmts:
            kind = st[0]
            if kind in ("let", "set"):
                if kind == "set" and st[1] not in self.locals:
                    raise NotImplementedError(f"assignment to unknown variable {st[1]}")
                r = self.expression(st[2])
                self.emit(StoreFromRegisterInstruction(r, st[1]))
                self.locals.add(st[1])
                self.release(r)
            elif kind == "return":
                r = self.expression(st[1])
                self.emit(ReturnInstruction(r))
                self.release(r)
            elif kind == "value":
                self.release(self.expression(st[1]))
            elif kind == "if":
                _, (_, op, lhs, rhs), body, other = st
                ra, rb = self.expression(lhs), self.expression(rhs)
                self.emit(BinaryInstruction(COMPARISON[op], ra, rb))
                self.release(ra)
                self.release(rb)
                else_id = self.next_id
                self.next_id += 1
                self.emit(JumpToId(else_id, JumpToIdIfFalse))
                self.block(body)
                if other:
                    end_id = self.next_id
                    self.next_id += 1
                    self.emit(Jump(end_id))
                    self.emit(JumpToIdEnd(else_id))
                    self.block(other)
                    self.emit(JumpToIdEnd(end_id))
                else:
                    self.emit(JumpToIdEnd(else_id))
            elif kind == "for":
                r = self.expression(st[1])
                begin = self.emit(LoopBeginInstruction(r))
                self.loop_depth += 1
                self.block(st[2])
                self.loop_depth -= 1
                self.emit(LoopEndInstruction(begin))
                self.release(r)
            else:
                raise NotImplementedError(kind)
