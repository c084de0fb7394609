"""Recognises the canonical ``tt.dot`` K loop in the TTIR of a ``@triton.jit`` kernel.

The reference's extensions see a kernel as Triton IR: an ``scf.for`` over K whose body loads an A and a
B tile, optionally under ``scf.if %k < %split`` with unmasked loads on one side and masked loads on the
other (the shape LoopSplit rewrites, pass/LoopSplit/LoopSplit.cpp:107-144), feeds them to ``tt.dot`` with
the loop-carried fp32 accumulator, and stores the cast result (pass/LoopSplit/06-fused-attention.py:63,85
for the dots, :237-240 for the cast-and-store). This module reads that IR as text, evaluates every
integer and pointer value symbolically (sympy expressions over the kernel arguments, the program ids,
the induction variable and one index symbol per tile axis), and proves that the kernel computes

    C[m, n] = cast(alpha * sum_k A[m, k] * B[k, n])      for m < M, n < N, with zero fill past K

with affine addressing. The result is a :class:`DotKernelMatch`; :func:`bind` turns it, together with
the argument values and grid of one launch, into the operands of the library GEMM. A kernel that is
anything else raises :class:`NotCanonical` with the reason: nothing is approximated.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Optional

import sympy as sp


class NotCanonical(ValueError):
    """The kernel is not the K loop this backend lowers."""


# --------------------------------------------------------------------------------------------------
# Text -> operations
# --------------------------------------------------------------------------------------------------

_VAL = r"%[\w.$-]+(?:#\d+)?"
_VAL_RE = re.compile(_VAL)


@dataclass
class Op:
    results: list
    name: str
    operands: list
    rest: str
    regions: list = field(default_factory=list)
    extra: dict = field(default_factory=dict)


def strip_locations(text: str) -> str:
    """Remove ``loc(...)`` annotations and ``#loc`` definitions from a printed module."""
    out = []
    for line in text.splitlines():
        if line.lstrip().startswith("#loc"):
            continue
        res, i = [], 0
        while True:
            j = line.find(" loc(", i)
            if j < 0:
                res.append(line[i:])
                break
            res.append(line[i:j])
            depth, p = 0, j + 4
            while p < len(line):
                if line[p] == "(":
                    depth += 1
                elif line[p] == ")":
                    depth -= 1
                    if depth == 0:
                        break
                p += 1
            i = p + 1
        out.append("".join(res))
    return "\n".join(out)


def _split_types(rest: str) -> tuple:
    """(text before the type section, type section) of an operation's tail."""
    depth, last, i = 0, -1, 0
    while i < len(rest):
        ch = rest[i]
        if rest.startswith("->", i):
            i += 2
            continue
        if ch in "{[(<":
            depth += 1
        elif ch in "}])>":
            depth -= 1
        elif depth == 0 and rest.startswith(" : ", i):
            last = i
        i += 1
    if last < 0:
        return rest, ""
    return rest[:last], rest[last + 3:]


def _result_type(types: str) -> str:
    if " -> " in types:
        return types.rsplit(" -> ", 1)[1].strip()
    if " to " in types:
        return types.rsplit(" to ", 1)[1].strip()
    depth = 0
    for i, ch in enumerate(types):
        if ch in "<(":
            depth += 1
        elif ch in ">)":
            depth -= 1
        elif ch == "," and depth == 0:
            return types[:i].strip()
    return types.strip()


def parse_type(ty: str) -> tuple:
    """(shape, element type) of ``tensor<128x64xbf16>``, ``!tt.ptr<f16>``, ``i32`` ..."""
    ty = ty.strip()
    if ty.startswith("tensor<") and ty.endswith(">"):
        inner = ty[len("tensor<"):-1]
        shape = []
        while True:
            m = re.match(r"(\d+)x", inner)
            if not m:
                break
            shape.append(int(m.group(1)))
            inner = inner[m.end():]
        return tuple(shape), inner
    return (), ty


def _expand_results(lhs: str) -> list:
    out = []
    for tok in [t.strip() for t in lhs.split(",")]:
        if ":" in tok:
            name, n = tok.split(":")
            out += [f"{name}#{i}" for i in range(int(n))]
        else:
            out.append(tok)
    return out


_FUNC_ARG = re.compile(r"(%[\w.$-]+): (![\w.]+<(?:[^<>]|<[^<>]*>)*>|[\w]+)(?: \{[^{}]*\})?(?: loc\(\"([^\"]+)\"\()?")


def parse_module(text: str, arg_names: Optional[list] = None) -> tuple:
    """Parse one printed ``tt.func``. Returns (function name, [(ssa name, source name, type)], ops)."""
    lines = text.splitlines()
    header_at = next((i for i, l in enumerate(lines) if "tt.func" in l and "@" in l), None)
    if header_at is None:
        raise NotCanonical("no tt.func in the module")
    if sum(1 for l in lines if re.search(r"\btt\.func\b", l)) != 1:
        raise NotCanonical("more than one function: calls are not lowered")
    header = lines[header_at]
    fname = re.search(r"@([\w.$-]+)\(", header).group(1)
    arg_text = header[header.index("(") + 1:]
    args = []
    for i, m in enumerate(_FUNC_ARG.finditer(arg_text.split(") attributes")[0])):
        src = arg_names[i] if arg_names and i < len(arg_names) else (m.group(3) or m.group(1)[1:])
        args.append((m.group(1), src, m.group(2)))

    body = strip_locations("\n".join(lines[header_at + 1:])).splitlines()
    root: list = []
    stack = [root]
    owners: list = []
    for raw in body:
        line = raw.strip()
        if not line or line == "module {":
            continue
        if line == "}" or re.fullmatch(r"\} \{[^{}]*\}", line):  # a region's end, possibly with attributes
            if owners:
                owners.pop()
                stack.pop()
                continue
            break  # end of the function
        if line == "} else {":
            op = owners[-1]
            stack.pop()
            op.regions.append([])
            stack.append(op.regions[-1])
            continue
        results = []
        m = re.match(rf"^((?:{_VAL}(?::\d+)?(?:, )?)+) = (.*)$", line)
        if m:
            results = _expand_results(m.group(1))
            line = m.group(2)
        name, _, rest = line.partition(" ")
        if name == "scf.for":
            fm = re.match(rf"({_VAL}) = ({_VAL}) to ({_VAL}) step ({_VAL})(?: iter_args\((.*?)\) -> \((.*?)\))?", rest)
            if not fm or not line.endswith("{"):
                raise NotCanonical(f"unreadable scf.for: {line}")
            iters = []
            if fm.group(5):
                for part in fm.group(5).split(", "):
                    a, b = part.split(" = ")
                    iters.append((a.strip(), b.strip()))
            op = Op(results, name, [fm.group(2), fm.group(3), fm.group(4)], rest, [[]],
                    {"iv": fm.group(1), "iters": iters})
            stack[-1].append(op)
            owners.append(op)
            stack.append(op.regions[0])
            continue
        if name == "scf.if":
            cond = _VAL_RE.match(rest)
            if not cond or not line.endswith("{"):
                raise NotCanonical(f"unreadable scf.if: {line}")
            op = Op(results, name, [cond.group(0)], rest, [[]])
            stack[-1].append(op)
            owners.append(op)
            stack.append(op.regions[0])
            continue
        if line.endswith("{"):
            raise NotCanonical(f"operation with a region is not lowered: {name}")
        head, _types = _split_types(rest)
        stack[-1].append(Op(results, name, _VAL_RE.findall(head), rest))
    return fname, args, root


# --------------------------------------------------------------------------------------------------
# Symbolic values
# --------------------------------------------------------------------------------------------------

X0, X1, KIV = sp.symbols("x0 x1 k_iv", integer=True)
TIV = sp.Symbol("tile_iv", integer=True)  # induction variable of a persistent kernel's loop over tiles
PID = {a: sp.Symbol(f"pid_{a}", integer=True, nonnegative=True) for a in "xyz"}
NPROG = {a: sp.Symbol(f"nprog_{a}", integer=True, positive=True) for a in "xyz"}


@dataclass
class Int:
    shape: tuple
    expr: Any


@dataclass
class Ptr:
    base: str
    elem: str
    shape: tuple
    off: Any


@dataclass
class Cond:
    shape: tuple
    terms: tuple  # conjunction of (pred, lhs, rhs)


@dataclass
class Flt:
    kind: str  # const | arg | load | cast | scale | acc | dot | loop_dot
    shape: tuple
    data: dict


@dataclass
class Desc:
    """A 2-D tensor descriptor: loads and stores through it are bounded by `shape` with zero fill."""
    base: Ptr
    shape: tuple
    strides: tuple
    block: tuple


class _Opaque:
    """A value the analysis does not model; using it is an error."""

    def __init__(self, why: str):
        self.why = why


def _bshape(a: tuple, b: tuple) -> tuple:
    if a == b or b == ():
        return a
    if a == ():
        return b
    if len(a) == len(b) and all(x == y or x == 1 or y == 1 for x, y in zip(a, b)):
        return tuple(max(x, y) for x, y in zip(a, b))
    raise NotCanonical(f"shape mismatch {a} vs {b}")


def _subst(v: Any, mapping: dict) -> Any:
    if isinstance(v, Int):
        return Int(v.shape, v.expr.subs(mapping))
    if isinstance(v, Ptr):
        return Ptr(v.base, v.elem, v.shape, v.off.subs(mapping))
    if isinstance(v, Cond):
        return Cond(v.shape, tuple((p, l.subs(mapping), r.subs(mapping)) for p, l, r in v.terms))
    if isinstance(v, Flt):
        return Flt(v.kind, v.shape, {k: _subst(x, mapping) for k, x in v.data.items()})
    return v


_INT_BIN = {
    "arith.addi": lambda a, b: a + b,
    "arith.subi": lambda a, b: a - b,
    "arith.muli": lambda a, b: a * b,
    "arith.divsi": lambda a, b: sp.floor(a / b),
    "arith.divui": lambda a, b: sp.floor(a / b),
    "arith.floordivsi": lambda a, b: sp.floor(a / b),
    "arith.ceildivsi": lambda a, b: sp.ceiling(a / b),
    "arith.remsi": lambda a, b: sp.Mod(a, b),
    "arith.remui": lambda a, b: sp.Mod(a, b),
    "arith.minsi": lambda a, b: sp.Min(a, b),
    "arith.minui": lambda a, b: sp.Min(a, b),
    "arith.maxsi": lambda a, b: sp.Max(a, b),
    "arith.maxui": lambda a, b: sp.Max(a, b),
}
_INT_CASTS = {"arith.extsi", "arith.extui", "arith.trunci", "arith.index_cast"}
_FLT_CASTS = {"arith.extf", "arith.truncf", "tt.fp_to_fp"}
_PURE_TT_OPS = {"tt.bitcast", "tt.int_to_ptr", "tt.ptr_to_int", "tt.reshape", "tt.join", "tt.split", "tt.cat",
                "tt.clampf", "tt.precise_sqrt", "tt.precise_divf", "tt.mulhiui", "tt.unsplat", "tt.gather",
                "tt.histogram"}
_FLOAT_TYPES = {"f16", "bf16", "f32", "f64", "f8E4M3FN", "f8E5M2", "f8E4M3FNUZ", "f8E5M2FNUZ"}


def _terms_subset(small: Optional[Cond], big: Optional[Cond]) -> bool:
    """Every term of `small` (None = no mask) is also a term of `big`."""
    if small is None:
        return True
    if big is None:
        return not small.terms
    for p, l, r in small.terms:
        if not any(p == q and sp.expand(l - r - (l2 - r2)) == 0 for q, l2, r2 in big.terms):
            return False
    return True


def _walk(ops: list):
    for o in ops:
        yield o
        for r in o.regions:
            yield from _walk(r)


class _Evaluator:
    def __init__(self, args: list):
        self.stores: list = []
        self.loops = 0
        self.tile_loop: Optional[dict] = None
        self.arg_symbols: dict = {}
        self.env: dict = {}
        i = 0
        while i < len(args):
            ssa, src, ty = args[i]
            i += 1
            if ty.startswith("!tt.ptr<"):
                self.env[ssa] = Ptr(src, ty[len("!tt.ptr<"):-1], (), sp.Integer(0))
            elif ty.startswith("!tt.tensordesc<"):
                # A tensor descriptor built on the host: the front end passes it as the descriptor followed by its
                # shape (i32 each) and its strides (i64 each). They become the integer arguments <name>__shape<d>,
                # <name>__stride<d>, which the launcher reads from the descriptor object.
                block, elem = parse_type(ty[len("!tt.tensordesc<"):-1])
                rank = len(block)
                if rank != 2 or i + 2 * rank > len(args):
                    self.env[ssa] = _Opaque(f"tensor descriptor {src} of rank {rank}")
                    continue
                fields = []
                for d, (fs, _, fty) in enumerate(args[i:i + 2 * rank]):
                    name = f"{src}__{'shape' if d < rank else 'stride'}{d % rank}"
                    sym = sp.Symbol(name, integer=True)
                    self.arg_symbols[name] = sym
                    self.env[fs] = Int((), sym)
                    fields.append(sym)
                i += 2 * rank
                self.env[ssa] = Desc(Ptr(src, elem, (), sp.Integer(0)), tuple(fields[:rank]), tuple(fields[rank:]), block)
            elif ty in _FLOAT_TYPES:
                self.env[ssa] = Flt("arg", (), {"name": src})
            elif re.fullmatch(r"i\d+", ty):
                s = sp.Symbol(src, integer=True)
                self.arg_symbols[src] = s
                self.env[ssa] = Int((), s)
            else:
                self.env[ssa] = _Opaque(f"argument {src} of type {ty}")

    def get(self, env: dict, name: str) -> Any:
        v = env.get(name)
        if v is None:
            raise NotCanonical(f"use of unknown value {name}")
        if isinstance(v, _Opaque):
            raise NotCanonical(f"the kernel depends on {v.why}")
        return v

    # -- one block ------------------------------------------------------------------------------
    def run(self, ops: list, env: dict) -> Optional[list]:
        """Evaluate a block; returns the operands of its scf.yield (or None)."""
        for op in ops:
            if op.name == "scf.yield":
                return [self.get(env, o) for o in op.operands]
            if op.name == "tt.return":
                return None
            self.step(op, env)
        return None

    def step(self, op: Op, env: dict) -> None:
        n = op.name
        head, types = _split_types(op.rest)
        rshape, relem = parse_type(_result_type(types)) if types else ((), "")
        g = lambda i: self.get(env, op.operands[i])

        def put(v):
            env[op.results[0]] = v

        if n == "arith.constant":
            tok = head.strip()
            m = re.match(r"dense<(.*)>$", tok)
            lit = m.group(1) if m else tok
            if relem in _FLOAT_TYPES:
                put(Flt("const", rshape, {"value": float(lit)}))
            elif lit in ("true", "false"):
                put(Cond(rshape, ()) if lit == "true" else _Opaque("a constant-false condition"))
            else:
                put(Int(rshape, sp.Integer(int(lit))))
        elif n == "tt.get_program_id":
            put(Int((), PID[head.strip()]))
        elif n == "tt.get_num_programs":
            put(Int((), NPROG[head.strip()]))
        elif n == "tt.make_range":
            start = int(re.search(r"start = (-?\d+)", head).group(1))
            put(Int(rshape, X0 + start))
        elif n == "tt.splat":
            v = g(0)
            if isinstance(v, Int):
                put(Int(rshape, v.expr))
            elif isinstance(v, Ptr):
                put(Ptr(v.base, v.elem, rshape, v.off))
            elif isinstance(v, Flt) and v.kind in ("const", "arg"):
                put(Flt(v.kind, rshape, dict(v.data)))
            else:
                raise NotCanonical("tt.splat of a value that is not an integer, a pointer or a float scalar")
        elif n == "tt.expand_dims":
            v = g(0)
            axis = int(re.search(r"axis = (\d+)", head).group(1))
            ren = {X0: X1} if axis == 0 else {}
            if isinstance(v, Flt) and v.kind == "load" and len(v.shape) == 1:
                # a vector of per-row (axis 1 added) or per-column (axis 0 added) factors
                put(Flt("vec", rshape, {"src": _subst(v, ren), "along": "col" if axis == 0 else "row"}))
                return
            if not isinstance(v, (Int, Cond)) or len(v.shape) != 1:
                raise NotCanonical("tt.expand_dims is modelled for rank-1 tensors only")
            if isinstance(v, Int):
                put(Int(rshape, v.expr.subs(ren)))
            else:
                put(Cond(rshape, tuple((p, l.subs(ren), r.subs(ren)) for p, l, r in v.terms)))
        elif n == "tt.broadcast":
            v = g(0)
            if isinstance(v, Int):
                put(Int(rshape, v.expr))
            elif isinstance(v, Ptr):
                put(Ptr(v.base, v.elem, rshape, v.off))
            elif isinstance(v, Cond):
                put(Cond(rshape, v.terms))
            elif isinstance(v, Flt) and v.kind == "vec":
                put(Flt("vec", rshape, dict(v.data)))
            else:
                raise NotCanonical("tt.broadcast of a float tile")
        elif n in _INT_BIN:
            a, b = g(0), g(1)
            if not (isinstance(a, Int) and isinstance(b, Int)):
                raise NotCanonical(f"{n} on non-integer values")
            put(Int(_bshape(a.shape, b.shape), _INT_BIN[n](a.expr, b.expr)))
        elif n == "arith.andi":
            a, b = g(0), g(1)
            if not (isinstance(a, Cond) and isinstance(b, Cond)):
                raise NotCanonical("arith.andi is modelled for conditions only")
            put(Cond(_bshape(a.shape, b.shape), a.terms + b.terms))
        elif n in _INT_CASTS:
            put(g(0))
        elif n == "arith.cmpi":
            pred = head.strip().split(",")[0].strip()
            a, b = g(0), g(1)
            if not (isinstance(a, Int) and isinstance(b, Int)):
                raise NotCanonical("arith.cmpi on non-integer values")
            put(Cond(_bshape(a.shape, b.shape), ((pred, a.expr, b.expr),)))
        elif n == "tt.addptr":
            p, o = g(0), g(1)
            if not (isinstance(p, Ptr) and isinstance(o, Int)):
                raise NotCanonical("tt.addptr needs a pointer and an integer offset")
            put(Ptr(p.base, p.elem, _bshape(p.shape, o.shape), p.off + o.expr))
        elif n == "tt.load":
            p = g(0)
            if not isinstance(p, Ptr):
                raise NotCanonical("tt.load through something that is not a plain pointer")
            mask = g(1) if len(op.operands) > 1 else None
            other = g(2) if len(op.operands) > 2 else None
            if mask is not None and not isinstance(mask, Cond):
                raise NotCanonical("tt.load mask is not a comparison")
            if other is not None and not (isinstance(other, Flt) and other.kind == "const" and other.data["value"] == 0.0):
                raise NotCanonical("tt.load `other` must be zero")
            put(Flt("load", p.shape, {"ptr": p, "mask": mask, "guard": None}))
        elif n in _FLT_CASTS:
            v = g(0)
            if not isinstance(v, Flt):
                raise NotCanonical(f"{n} on a non-float value")
            put(Flt("cast", v.shape, {"src": v, "to": relem}))
        elif n == "tt.trans":
            v = g(0)
            if not (isinstance(v, Flt) and len(v.shape) == 2 and "1, 0" in head):
                raise NotCanonical("tt.trans is modelled as the transpose of a 2-D float tile")
            put(self.transpose(v))
        elif n == "arith.mulf":
            a, b = g(0), g(1)
            if isinstance(a, Flt) and a.kind in ("const", "arg", "vec"):
                a, b = b, a
            if not (isinstance(a, Flt) and isinstance(b, Flt) and b.kind in ("const", "arg", "vec")):
                raise NotCanonical("arith.mulf is modelled only as a scale by a scalar or by a row / column vector")
            if b.kind == "vec":
                put(Flt("vscale", _bshape(a.shape, b.shape), {"src": a, "vec": b}))
            else:
                put(Flt("scale", a.shape, {"src": a, "by": b}))
        elif n == "tt.dot":
            a, b, c = g(0), g(1), g(2)
            if not all(isinstance(v, Flt) for v in (a, b, c)):
                raise NotCanonical("tt.dot operands are not float tiles")
            if relem != "f32":
                raise NotCanonical(f"tt.dot accumulates in {relem}; the library kernel accumulates in f32")
            put(Flt("dot", c.shape, {"a": a, "b": b, "c": c}))
        elif n == "tt.make_tensor_descriptor":
            base = g(0)
            rest_ops = [g(i) for i in range(1, len(op.operands))]
            if not isinstance(base, Ptr) or base.shape != () or len(rest_ops) != 4 or \
                    not all(isinstance(v, Int) and v.shape == () for v in rest_ops):
                raise NotCanonical("tt.make_tensor_descriptor is modelled for 2-D descriptors on a plain pointer")
            bm = re.search(r"tensor<(\d+)x(\d+)x", types)
            put(Desc(base, (rest_ops[0].expr, rest_ops[1].expr), (rest_ops[2].expr, rest_ops[3].expr),
                     (int(bm.group(1)), int(bm.group(2)))))
        elif n in ("tt.descriptor_load", "tt.descriptor_store"):
            d, i, j = g(0), g(1), g(2)
            if not isinstance(d, Desc) or not all(isinstance(v, Int) and v.shape == () for v in (i, j)):
                raise NotCanonical(f"{n} needs a descriptor and two scalar coordinates")
            r, c = i.expr + X0, j.expr + X1
            ptr = Ptr(d.base.base, d.base.elem, d.block, d.base.off + r * d.strides[0] + c * d.strides[1])
            mask = Cond(d.block, (("slt", r, d.shape[0]), ("slt", c, d.shape[1])))
            if n == "tt.descriptor_load":
                put(Flt("load", d.block, {"ptr": ptr, "mask": mask, "guard": None}))
            else:
                v = g(3)
                if not isinstance(v, Flt):
                    raise NotCanonical("tt.descriptor_store of something that is not a float tile")
                self.stores.append((ptr, v, mask))
        elif n == "tt.store":
            p, v = g(0), g(1)
            mask = g(2) if len(op.operands) > 2 else None
            if not isinstance(p, Ptr) or not isinstance(v, Flt):
                raise NotCanonical("tt.store of something that is not a float tile through a plain pointer")
            if mask is not None and not isinstance(mask, Cond):
                raise NotCanonical("tt.store mask is not a comparison")
            self.stores.append((p, v, mask))
        elif n == "scf.if":
            self.eval_if(op, env)
        elif n == "scf.for":
            self.eval_for(op, env)
        elif n in ("tt.assume", "llvm.intr.assume"):
            pass
        elif op.results and (n.startswith("arith.") or n.startswith("math.") or n in _PURE_TT_OPS):
            # A value the analysis does not model: harmless while nothing the GEMM depends on uses it.
            for r in op.results:
                env[r] = _Opaque(f"the result of {n}")
        else:
            # Anything else may write memory or synchronise (atomics, calls, prints, inline assembly, ...).
            raise NotCanonical(f"operation that is not modelled and may have a side effect: {n}")

    @staticmethod
    def transpose(v: Flt) -> Flt:
        """The transposed tile of a load (through casts): the two index symbols change places."""
        if v.kind == "cast":
            inner = _Evaluator.transpose(v.data["src"])
            return Flt("cast", inner.shape, {"src": inner, "to": v.data["to"]})
        if v.kind != "load":
            raise NotCanonical("tt.trans of a value that is not a loaded tile")
        swap = {X0: X1, X1: X0}
        sw = lambda e: e.subs(swap, simultaneous=True)
        p, mask, guard = v.data["ptr"], v.data["mask"], v.data["guard"]
        shape = (v.shape[1], v.shape[0])
        return Flt("load", shape, {
            "ptr": Ptr(p.base, p.elem, shape, sw(p.off)),
            "mask": None if mask is None else Cond(shape, tuple((q, sw(l), sw(r)) for q, l, r in mask.terms)),
            "guard": guard})

    # -- regions --------------------------------------------------------------------------------
    def eval_if(self, op: Op, env: dict) -> None:
        cond = self.get(env, op.operands[0])
        if not isinstance(cond, Cond) or cond.shape != () or len(cond.terms) != 1:
            raise NotCanonical("scf.if on something that is not one scalar comparison")
        stores_before = len(self.stores)
        then_y = self.run(op.regions[0], dict(env))
        else_y = self.run(op.regions[1], dict(env)) if len(op.regions) > 1 else None
        if len(self.stores) != stores_before:
            raise NotCanonical("a store under scf.if is not lowered")
        if any(o.name == "scf.for" for r in op.regions for o in _walk(r)):
            raise NotCanonical("a loop under scf.if is not lowered")
        if not op.results:
            return
        if then_y is None or else_y is None or len(then_y) != len(op.results) or len(else_y) != len(op.results):
            raise NotCanonical("scf.if without matching yields")
        for r, t, e in zip(op.results, then_y, else_y):
            env[r] = self.merge(cond, t, e)

    @staticmethod
    def merge(cond: Cond, t: Any, e: Any) -> Any:
        """Both arms of the split: a load without the K mask where the compare holds (it may keep row or column
        masks), the fully masked load of the same addresses elsewhere. The merged value is the masked load,
        guarded by the compare."""
        if isinstance(t, Flt) and isinstance(e, Flt):
            ts, es = t, e
            casts = []
            while ts.kind == "cast" and es.kind == "cast" and ts.data["to"] == es.data["to"]:
                casts.append(ts.data["to"])
                ts, es = ts.data["src"], es.data["src"]
            if ts.kind == "load" and es.kind == "load":
                pt, pe = ts.data["ptr"], es.data["ptr"]
                same = pt.base == pe.base and pt.shape == pe.shape and sp.expand(pt.off - pe.off) == 0
                if same and _terms_subset(ts.data["mask"], es.data["mask"]) and ts.data["guard"] is None \
                        and es.data["guard"] is None:
                    v = Flt("load", es.shape, {"ptr": pe, "mask": es.data["mask"], "guard": cond})
                    for to in reversed(casts):
                        v = Flt("cast", v.shape, {"src": v, "to": to})
                    return v
        if isinstance(t, Int) and isinstance(e, Int) and t.shape == e.shape and sp.expand(t.expr - e.expr) == 0:
            return t
        return _Opaque("an scf.if whose arms are not the unmasked and the masked load of one tile")

    def eval_tile_loop(self, op: Op, env: dict) -> None:
        """The outer loop of a persistent kernel: each iteration is one tile (a K loop and a store). Its
        induction variable becomes a symbol of the tile origin; bind() walks it per program."""
        if self.tile_loop is not None or self.loops:
            raise NotCanonical("more than one loop over tiles, or a K loop before it")
        lo, hi, step = (self.get(env, o) for o in op.operands)
        if not all(isinstance(v, Int) and v.shape == () for v in (lo, hi, step)):
            raise NotCanonical("tile-loop bounds are not scalar integers")
        body = dict(env)
        body[op.extra["iv"]] = Int((), TIV)
        holders = []
        for i, (name, init_name) in enumerate(op.extra["iters"]):
            init = self.get(env, init_name)
            if not isinstance(init, Int):
                raise NotCanonical("the loop over tiles carries something that is not an integer")
            sym = sp.Symbol(f"tile_iter_{i}", integer=True)
            body[name] = Int(init.shape, sym)
            holders.append((sym, init))
        first_store = len(self.stores)
        yields = self.run(op.regions[0], body) or []
        if len(yields) != len(holders):
            raise NotCanonical("scf.for yield does not match its iter_args")
        trip = (TIV - lo.expr) / step.expr
        placeholders = {sym for sym, _ in holders}
        closed = {}
        for (sym, init), y in zip(holders, yields):
            if not isinstance(y, Int):
                raise NotCanonical("a tile-loop-carried integer is yielded as another kind of value")
            delta = sp.expand(y.expr - sym)
            if delta.free_symbols & (placeholders | {TIV, KIV}):
                raise NotCanonical("a tile-loop-carried integer does not advance by a loop-invariant amount")
            closed[sym] = init.expr + trip * delta
        for i in range(first_store, len(self.stores)):
            self.stores[i] = tuple(_subst(x, closed) for x in self.stores[i])
        for r in op.results:
            env[r] = _Opaque("the final value of a tile-loop-carried integer")
        self.tile_loop = {"lo": lo.expr, "hi": hi.expr, "step": step.expr}

    def eval_for(self, op: Op, env: dict) -> None:
        if any(o.name == "scf.for" for o in _walk(op.regions[0])):
            return self.eval_tile_loop(op, env)
        self.loops += 1
        if self.loops > 2:
            raise NotCanonical("more than two K loops in sequence")
        lo, hi, step = (self.get(env, o) for o in op.operands)
        if not all(isinstance(v, Int) and v.shape == () for v in (lo, hi, step)):
            raise NotCanonical("loop bounds are not scalar integers")
        if not step.expr.is_Integer or int(step.expr) <= 0:
            raise NotCanonical("the loop step is not a positive constant (LoopSplit.cpp:125-131 asks the same)")
        body = dict(env)
        body[op.extra["iv"]] = Int((), KIV)
        holders = []
        for i, (name, init_name) in enumerate(op.extra["iters"]):
            init = self.get(env, init_name)
            if isinstance(init, Int):
                s = sp.Symbol(f"iter_{i}", integer=True)
                body[name] = Int(init.shape, s)
            elif isinstance(init, Ptr):
                s = sp.Symbol(f"iter_{i}", integer=True)
                body[name] = Ptr(init.base, init.elem, init.shape, s)
            elif isinstance(init, Flt):
                s = None
                body[name] = Flt("acc", init.shape, {"index": i})
            else:
                raise NotCanonical("a loop-carried condition is not lowered")
            holders.append((s, init))
        stores_before = len(self.stores)
        yields = self.run(op.regions[0], body) or []
        if len(self.stores) != stores_before:
            raise NotCanonical("a store inside the K loop is not lowered")
        if len(yields) != len(holders):
            raise NotCanonical("scf.for yield does not match its iter_args")
        trip = (KIV - lo.expr) / step.expr
        closed = {}
        placeholders = {s for s, _ in holders if s is not None}
        for (s, init), y in zip(holders, yields):
            if s is None:
                continue
            cur = y.expr if isinstance(y, Int) else y.off if isinstance(y, Ptr) else None
            if cur is None:
                raise NotCanonical("a loop-carried integer is yielded as another kind of value")
            delta = sp.expand(cur - s)
            if delta.free_symbols & (placeholders | {KIV}):
                raise NotCanonical("a loop-carried offset does not advance by a loop-invariant amount")
            start = init.expr if isinstance(init, Int) else init.off
            closed[s] = start + trip * delta
        # What a carried offset holds after the loop: its start plus one advance per iteration. The trip count is
        # kept as one symbol so that a loop continuing from here can be compared with this one (_fuse_split_loops).
        trips = sp.Symbol(f"trips_{id(op)}", integer=True, nonnegative=True)
        trips_value = sp.ceiling(sp.Max(hi.expr - lo.expr, 0) / step.expr)
        deltas = {}
        for (s, init), y in zip(holders, yields):
            if s is not None:
                deltas[s] = sp.expand((y.expr if isinstance(y, Int) else y.off) - s)
        for idx, ((s, init), y) in enumerate(zip(holders, yields)):
            res = op.results[idx]
            if s is not None:
                if isinstance(init, Int):
                    env[res] = Int(init.shape, init.expr + trips * deltas[s])
                else:
                    env[res] = Ptr(init.base, init.elem, init.shape, init.off + trips * deltas[s])
                continue
            if not (isinstance(y, Flt) and y.kind == "dot" and y.data["c"].kind == "acc" and y.data["c"].data["index"] == idx):
                raise NotCanonical("the loop-carried float is not `acc = tt.dot(a, b, acc)`")
            env[res] = Flt("loop_dot", y.shape, {
                "a": _subst(y.data["a"], closed), "b": _subst(y.data["b"], closed), "init": init,
                "lo": lo.expr, "hi": hi.expr, "step": step.expr, "trips": trips, "trips_value": trips_value})


# --------------------------------------------------------------------------------------------------
# Matching
# --------------------------------------------------------------------------------------------------

# (exponent bits, mantissa bits): a cast keeps every value when neither shrinks
_FLOAT_BITS = {"f8E4M3FN": (4, 3), "f8E5M2": (5, 2), "f16": (5, 10), "bf16": (8, 7), "f32": (8, 23), "f64": (11, 52)}
_DTYPE_NAMES = {"f16": "f16", "bf16": "bf16", "f32": "f32", "f8E4M3FN": "f8e4m3", "f8E5M2": "f8e5m2"}


@dataclass
class DotKernelMatch:
    """What the K loop of a kernel computes, as expressions over its arguments and program ids."""
    kernel: str
    a_arg: str
    b_arg: str
    c_arg: str
    ab_dtype: str
    out_dtype: str
    block_m: int
    block_n: int
    block_k: int
    a_row_stride: str
    a_k_stride: str
    b_k_stride: str
    b_col_stride: str
    c_row_stride: str
    c_col_stride: str
    row0: str               # first row of the tile of program (pid_x, pid_y, pid_z)
    col0: str
    loop_lo: str
    loop_hi: str
    loop_step: int
    k_per_iv: int           # K elements per unit of the induction variable
    k_bound: Optional[str]  # the K the load masks compare with; None for unmasked loads
    m_bound: Optional[str]
    n_bound: Optional[str]
    split_pred: Optional[str]       # compare of the induction variable guarding the unmasked loads
    split_comparand: Optional[str]
    alpha: Optional[str]            # constant, or the name of a float argument
    int_args: list = field(default_factory=list)
    row_scale_arg: Optional[str] = None  # fp32 vector multiplied into the rows before the cast
    col_scale_arg: Optional[str] = None
    tile_loop: Optional[list] = None     # [lo, hi, step] of a persistent kernel's loop over tiles (tile_iv)
    batch_offsets: Optional[list] = None  # [A, B, C] element offsets of the program's matrices (batched GEMM)
    equal_at_launch: list = field(default_factory=list)  # [name, expr, expr]: bounds written differently that must agree
    split_is_loop_bound: bool = False  # the split point is where a first K loop ends (LoopSplit's output), not a compare

    def to_json(self) -> str:
        return json.dumps(self.__dict__, sort_keys=True)

    @staticmethod
    def from_json(text: str) -> "DotKernelMatch":
        return DotKernelMatch(**json.loads(text))


def _peel(v: Flt, vecs: Optional[list] = None) -> tuple:
    casts, alpha = [], None
    while v.kind in ("cast", "scale", "vscale"):
        if v.kind == "cast":
            casts.append(v.data["to"])
            v = v.data["src"]
        elif v.kind == "vscale":
            if vecs is None:
                raise NotCanonical("a tt.dot operand is scaled by a vector")
            vecs.append(v.data["vec"])
            v = v.data["src"]
        else:
            if alpha is not None:
                raise NotCanonical("more than one scalar scale in the epilogue")
            by = v.data["by"]
            alpha = repr(by.data["value"]) if by.kind == "const" else by.data["name"]
            v = v.data["src"]
    return v, casts, alpha


def _scale_vector(vec: Flt, origin: Any, index: Any, key: str, bounds: dict) -> str:
    """A scale vector must be an fp32 load of base[origin + index], masked (if at all) by the matrix bound."""
    load = vec.data["src"]
    p = load.data["ptr"]
    if p.elem != "f32":
        raise NotCanonical(f"the {vec.data['along']} scale vector is {p.elem}, not f32")
    if sp.expand(p.off - origin - index) != 0:
        raise NotCanonical(f"the {vec.data['along']} scale vector is not indexed by the tile's own {vec.data['along']}s")
    m = _classify_mask(load.data["mask"], {key: origin + index}, f"{vec.data['along']} scale mask")
    if key in m:
        if bounds.get(key) is not None and sp.expand(bounds[key] - m[key]) != 0:
            raise NotCanonical("a scale vector and the store disagree on the matrix bounds")
        bounds.setdefault(key, m[key])
    return p.base


def _affine(expr: Any, what: str) -> tuple:
    """Coefficients (x0, x1, k_iv, constant) of an address expression that must be affine in them."""
    try:
        poly = sp.Poly(sp.expand(expr), X0, X1, KIV)
    except sp.PolynomialError:
        raise NotCanonical(f"{what}: the address is not a polynomial in the tile indices")
    coef = {(1, 0, 0): 0, (0, 1, 0): 0, (0, 0, 1): 0, (0, 0, 0): 0}
    for mono, c in poly.terms():
        if mono not in coef:
            raise NotCanonical(f"{what}: the address is not affine in the tile indices")
        coef[mono] = c
    return coef[(1, 0, 0)], coef[(0, 1, 0)], coef[(0, 0, 1)], coef[(0, 0, 0)]


def _unwrap(expr: Any) -> tuple:
    """Replace every Mod(inner, modulus) whose modulus is loop- and tile-invariant by `inner`; the caller
    checks afterwards that the wrap cannot reach a stored element. Returns (expression, [(inner, modulus)])."""
    wraps = []
    for atom in list(expr.atoms(sp.Mod)):
        inner, modulus = atom.args
        if not (modulus.free_symbols & {X0, X1, KIV}) and (inner.free_symbols & {X0, X1}):
            wraps.append((sp.expand(inner), sp.expand(modulus)))
            expr = expr.subs(atom, inner)
    return expr, wraps


def _origin(const: Any, stride: Any, block: int, strides: set, what: str) -> tuple:
    """Split the constant part of an address into (tile origin in rows or columns, batch offset in elements).

    A term belongs to the origin when it is `stride` times a symbolic multiple of the block extent (tile origins
    are whole blocks); every other term is an offset of the whole matrix, as a batched kernel adds per program id.
    A term put on the wrong side cannot slip through: bind() checks numerically that the origins tile C exactly."""
    origin, batch = sp.Integer(0), sp.Integer(0)
    for term in sp.Add.make_args(sp.expand(const)):
        q = sp.cancel(term / (stride * block))
        if sp.denom(q) == 1 and not (q.free_symbols & strides):
            origin += q * block
        else:
            batch += term
    bad = {X0, X1, KIV}
    if (origin.free_symbols & bad) or (batch.free_symbols & bad):
        raise NotCanonical(f"{what}: the tile origin moves with the tile indices")
    return sp.expand(origin), sp.expand(batch)


def _classify_mask(cond: Optional[Cond], forms: dict, what: str) -> dict:
    """Each term must be `index < bound` for one of the index forms given; returns {form: bound}."""
    out: dict = {}
    if cond is None:
        return out
    for pred, l, r in cond.terms:
        if pred in ("sge", "uge") and any(sp.expand(l - r - form) == 0 for form in forms.values()):
            continue  # `index >= 0`, the lower half of a block pointer's boundary check: indices are never negative
        if pred in ("sgt", "ugt"):
            l, r, pred = r, l, "slt"
        if pred not in ("slt", "ult"):
            raise NotCanonical(f"{what}: mask predicate {pred} is not `<`")
        d = sp.expand(l - r)
        for key, form in forms.items():
            bound = sp.expand(form - d)
            if not (bound.free_symbols & {X0, X1, KIV}):
                if key in out and sp.expand(out[key] - bound) != 0:
                    raise NotCanonical(f"{what}: two different bounds on one index")
                out[key] = bound
                break
        else:
            raise NotCanonical(f"{what}: a mask term is not a bound on the row, column or K index")
    return out


def _fuse_split_loops(second: Flt) -> Flt:
    """Two K loops in sequence, the second starting from the first's result at the point where the first stops,
    are what LoopSplit makes of one loop whose compare `iv < mid` guarded the loads without a K mask
    (pass/LoopSplit/LoopSplit.cpp:169-190). Read them back as that one loop."""
    first = second.data["init"]
    if first.kind != "loop_dot":
        return second
    if first.data["init"].kind == "loop_dot":
        raise NotCanonical("more than two K loops in sequence")
    if sp.expand(first.data["hi"] - second.data["lo"]) != 0 or sp.expand(first.data["step"] - second.data["step"]) != 0:
        raise NotCanonical("the second K loop does not continue where the first stops")
    mid = sp.expand(first.data["hi"])
    # Offsets the second loop inherits hold `start + trips * advance`. The first loop runs (mid - lo) / step times when
    # mid is not below lo and a whole number of steps from it, which bind() checks for the launch's values.
    exact = {first.data["trips"]: (first.data["hi"] - first.data["lo"]) / first.data["step"]}
    fused = {}
    same_masks = True
    for key in ("a", "b"):
        f, f_casts, f_alpha = _peel(first.data[key])
        g, g_casts, g_alpha = _peel(_subst(second.data[key], exact))
        if f_alpha or g_alpha or f.kind != "load" or g.kind != "load" or f_casts != g_casts:
            raise NotCanonical("the two K loops do not feed the dot with the same kind of loads")
        pf, pg = f.data["ptr"], g.data["ptr"]
        if pf.base != pg.base or pf.elem != pg.elem or pf.shape != pg.shape or sp.expand(pf.off - pg.off) != 0:
            raise NotCanonical("the two K loops do not load from the same addresses")
        if f.data["guard"] is not None or g.data["guard"] is not None:
            raise NotCanonical("a split K loop still carries a compare on its induction variable")
        if not _terms_subset(f.data["mask"], g.data["mask"]):
            raise NotCanonical("the first K loop masks more than the second")
        same_masks = same_masks and _terms_subset(g.data["mask"], f.data["mask"])
        fused[key] = (g, g_casts)
    out = {}
    for key, (g, casts) in fused.items():
        guard = None if same_masks else Cond((), (("slt", KIV, mid),))
        v = Flt("load", g.shape, {"ptr": g.data["ptr"], "mask": g.data["mask"], "guard": guard})
        for to in reversed(casts):
            v = Flt("cast", v.shape, {"src": v, "to": to})
        out[key] = v
    return Flt("loop_dot", second.shape, {"a": out["a"], "b": out["b"], "init": first.data["init"],
                                          "lo": first.data["lo"], "hi": second.data["hi"], "step": second.data["step"],
                                          "trips": second.data["trips"], "trips_value": second.data["trips_value"],
                                          "fused": True})


def match_dot_kernel(text: str, arg_names: Optional[list] = None) -> DotKernelMatch:
    """Analyse the printed TTIR of one kernel. Raises NotCanonical unless it is the K loop described above."""
    try:
        return _match_dot_kernel(text, arg_names)
    except NotCanonical:
        raise
    except Exception as e:  # IR this reader was not written for: refuse, never guess
        raise NotCanonical(f"the IR could not be analysed ({type(e).__name__}: {e})") from e


def _match_dot_kernel(text: str, arg_names: Optional[list]) -> DotKernelMatch:
    fname, args, ops = parse_module(text, arg_names)
    ev = _Evaluator(args)
    ev.run(ops, ev.env)
    if len(ev.stores) != 1:
        raise NotCanonical(f"{len(ev.stores)} stores; the K loop has exactly one")
    c_ptr, value, c_mask = ev.stores[0]
    vecs: list = []
    value, out_casts, alpha = _peel(value, vecs)
    single = value.kind == "dot" and value.data["c"].kind == "const"
    if single:
        # One tt.dot outside any loop: a K loop of exactly one iteration over the whole K extent of the tiles.
        k_extent = value.data["a"].shape[1] if len(value.data["a"].shape) == 2 else 0
        value = Flt("loop_dot", value.shape, {"a": value.data["a"], "b": value.data["b"], "init": value.data["c"],
                                              "lo": sp.Integer(0), "hi": sp.Integer(k_extent), "step": sp.Integer(k_extent),
                                              "trips": sp.Symbol("trips_single"), "trips_value": sp.Integer(1)})
    if value.kind != "loop_dot":
        raise NotCanonical("the stored value is not the result of the K loop")
    value = _fuse_split_loops(value)
    init = value.data["init"]
    if not (init.kind == "const" and init.data["value"] == 0.0):
        raise NotCanonical("the accumulator does not start at zero")
    a, a_casts, a_alpha = _peel(value.data["a"])
    b, b_casts, b_alpha = _peel(value.data["b"])
    if a_alpha or b_alpha or a.kind != "load" or b.kind != "load":
        raise NotCanonical("the tt.dot operands are not plain loads")
    pa, pb = a.data["ptr"], b.data["ptr"]
    for elem, casts, which in ((pa.elem, a_casts, "A"), (pb.elem, b_casts, "B")):
        # A cast between the load and the dot must keep every value: the kernel multiplies what is in memory.
        for to in reversed(casts):
            if _FLOAT_BITS.get(to, (0, 0))[0] < _FLOAT_BITS.get(elem, (99, 99))[0] or \
                    _FLOAT_BITS.get(to, (0, 0))[1] < _FLOAT_BITS.get(elem, (99, 99))[1]:
                raise NotCanonical(f"operand {which} is narrowed from {elem} to {to} before the dot")
            elem = to
    if pa.elem not in ("f16", "bf16", "f8E4M3FN", "f8E5M2"):
        raise NotCanonical(f"operands of type {pa.elem} have no tensor-core path in the library")
    if out_casts not in ([], [c_ptr.elem]) or (not out_casts and c_ptr.elem != "f32"):
        raise NotCanonical("the epilogue is not a single cast of the f32 sum to the stored type")
    if len(pa.shape) != 2 or len(pb.shape) != 2 or len(c_ptr.shape) != 2:
        raise NotCanonical("tiles are not 2-D")
    (bm, bk), (bk2, bn) = pa.shape, pb.shape
    if bk != bk2 or c_ptr.shape != (bm, bn):
        raise NotCanonical("tile shapes of A, B and C do not agree")
    if pa.elem != pb.elem or pa.elem not in _DTYPE_NAMES or c_ptr.elem not in _DTYPE_NAMES:
        raise NotCanonical(f"element types {pa.elem}, {pb.elem} -> {c_ptr.elem} are not supported")

    a_off, a_wraps = _unwrap(pa.off)
    b_off, b_wraps = _unwrap(pb.off)
    sa_r, sa_k, sa_iv, ca = _affine(a_off, "A")
    sb_k, sb_c, sb_iv, cb = _affine(b_off, "B")
    sc_r, sc_c, sc_iv, cc = _affine(c_ptr.off, "C")
    if sc_iv != 0 or 0 in (sa_r, sa_k, sb_k, sb_c, sc_r, sc_c):
        raise NotCanonical("an operand has a zero stride or C moves with the loop")
    kpi_a, kpi_b = sp.cancel(sa_iv / sa_k), sp.cancel(sb_iv / sb_k)
    if single and kpi_a == 0 and kpi_b == 0:
        kpi_a = kpi_b = sp.Integer(1)  # no induction variable to advance along
    if not (kpi_a.is_Integer and kpi_a == kpi_b and int(kpi_a) > 0):
        raise NotCanonical("A and B do not advance along K by the same whole number of elements per iteration")
    kpi = int(kpi_a)
    step = int(value.data["step"])
    if kpi * step != bk:
        raise NotCanonical(f"the loop advances {kpi * step} K elements per iteration but the tiles hold {bk}")
    lo = sp.expand(value.data["lo"])
    if lo != 0:
        raise NotCanonical("the K loop does not start at 0")

    stride_syms = set()
    for s in (sa_r, sa_k, sb_k, sb_c, sc_r, sc_c):
        stride_syms |= s.free_symbols
    row0, a_batch = _origin(ca, sa_r, bm, stride_syms, "A")
    col0, b_batch = _origin(cb, sb_c, bn, stride_syms, "B")
    # What is left of C's address after the tile's rows and columns is the offset of its matrix.
    c_batch = sp.expand(cc - row0 * sc_r - col0 * sc_c)
    c_row, c_rest = _origin(c_batch, sc_r, bm, stride_syms, "C")
    c_col, c_rest = _origin(c_rest, sc_c, bn, stride_syms, "C")
    if c_row != 0 or c_col != 0 or (c_batch.free_symbols & {X0, X1, KIV}):
        raise NotCanonical("C is not stored at the rows of A and the columns of B")
    batched = any(e != 0 for e in (a_batch, b_batch, c_batch))

    kk = kpi * KIV if not (single and sa_iv == 0) else sp.Integer(0)
    a_m = _classify_mask(a.data["mask"], {"k": X1 + kk, "m": row0 + X0}, "A mask")
    b_m = _classify_mask(b.data["mask"], {"k": X0 + kk, "n": col0 + X1}, "B mask")
    c_m = _classify_mask(c_mask, {"m": row0 + X0, "n": col0 + X1}, "C mask")
    if ("k" in a_m) != ("k" in b_m):
        raise NotCanonical("A and B are not masked by the same K bound")
    # Bounds that are different expressions (the shapes of two host descriptors, say) must agree at every launch.
    equal_at_launch = []
    for what, x, y in (("K", a_m.get("k"), b_m.get("k")), ("M", a_m.get("m"), c_m.get("m")), ("N", b_m.get("n"), c_m.get("n"))):
        if x is not None and y is not None and sp.expand(x - y) != 0:
            if not (x.free_symbols and y.free_symbols):
                raise NotCanonical(f"loads and store disagree on the {what} bound")
            equal_at_launch.append([what, str(x), str(y)])
    bounds = {"m": c_m.get("m", a_m.get("m")), "n": c_m.get("n", b_m.get("n"))}
    row_scale = col_scale = None
    for vec in vecs:
        if vec.data["along"] == "row":
            if row_scale is not None:
                raise NotCanonical("more than one row scale vector")
            row_scale = _scale_vector(vec, row0, X0, "m", bounds)
        else:
            if col_scale is not None:
                raise NotCanonical("more than one column scale vector")
            col_scale = _scale_vector(vec, col0, X1, "n", bounds)
    m_bound, n_bound = bounds["m"], bounds["n"]
    # Rows of A (columns of B) taken modulo the matrix extent are the rows themselves wherever the store
    # writes; the wrapped ones only feed elements the store masks off.
    for wraps, index, bound, stored, what in ((a_wraps, row0 + X0, m_bound, "m" in c_m, "row"),
                                              (b_wraps, col0 + X1, n_bound, "n" in c_m, "column")):
        for inner, modulus in wraps:
            if sp.expand(inner - index) != 0 or bound is None or not stored or sp.expand(modulus - bound) != 0:
                raise NotCanonical(f"a {what} index is wrapped by something that is not the bound the store masks with")

    ga, gb = a.data["guard"], b.data["guard"]
    if (ga is None) != (gb is None):
        raise NotCanonical("only one operand is loaded under the split compare")
    split_pred = split_cmp = None
    if ga is not None:
        (pa_, la, ra), (pb_, lb, rb) = ga.terms[0], gb.terms[0]
        if pa_ != pb_ or sp.expand(la - lb) != 0 or sp.expand(ra - rb) != 0:
            raise NotCanonical("A and B are guarded by different compares")
        if sp.expand(la - KIV) != 0 or (ra.free_symbols & {KIV, X0, X1}) or pa_ not in ("slt", "ult"):
            raise NotCanonical("the split compare is not `induction variable < loop-invariant value`")
        if "k" not in a_m:
            raise NotCanonical("the guarded-off loads carry no K mask")
        split_pred, split_cmp = "slt", str(ra)

    return DotKernelMatch(
        kernel=fname, a_arg=pa.base, b_arg=pb.base, c_arg=c_ptr.base,
        ab_dtype=_DTYPE_NAMES[pa.elem], out_dtype=_DTYPE_NAMES[c_ptr.elem],
        block_m=bm, block_n=bn, block_k=bk,
        a_row_stride=str(sa_r), a_k_stride=str(sa_k), b_k_stride=str(sb_k), b_col_stride=str(sb_c),
        c_row_stride=str(sc_r), c_col_stride=str(sc_c), row0=str(row0), col0=str(col0),
        loop_lo=str(lo), loop_hi=str(sp.expand(value.data["hi"])), loop_step=step, k_per_iv=kpi,
        k_bound=str(a_m["k"]) if "k" in a_m else None,
        m_bound=str(m_bound) if m_bound is not None else None,
        n_bound=str(n_bound) if n_bound is not None else None,
        split_pred=split_pred, split_comparand=split_cmp, alpha=alpha,
        int_args=sorted(ev.arg_symbols), row_scale_arg=row_scale, col_scale_arg=col_scale,
        tile_loop=[str(sp.expand(ev.tile_loop[k])) for k in ("lo", "hi", "step")] if ev.tile_loop else None,
        batch_offsets=[str(a_batch), str(b_batch), str(c_batch)] if batched else None,
        equal_at_launch=equal_at_launch, split_is_loop_bound=bool(value.data.get("fused")) and split_cmp is not None)


# --------------------------------------------------------------------------------------------------
# Binding one launch
# --------------------------------------------------------------------------------------------------

@dataclass
class BoundDot:
    m: int
    n: int
    k: int
    a_layout: str   # "row" | "col"
    b_layout: str
    lda: int
    ldb: int
    ldc: int
    alpha: float
    block_k: int
    k_main: int     # K elements the unmasked iterations cover
    batches: Optional[list] = None  # batched GEMM: one (A, B, C) element-offset triple per matrix product
    swapped: bool = False           # the library computes C^T = B^T A^T: its A is the kernel's B and vice versa


def _value(expr: Optional[str], scalars: dict) -> Optional[int]:
    if expr is None:
        return None
    local = {name: sp.Symbol(name, integer=True) for name in scalars}
    e = sp.sympify(expr, locals=local)
    v = e.subs({local[n]: scalars[n] for n in local})
    if not v.is_Integer:
        raise NotCanonical(f"{expr} does not evaluate to an integer for this launch ({v})")
    return int(v)


def _tile_origins(match: DotKernelMatch, scalars: dict, grid: tuple) -> tuple:
    """Row and column origin of every tile the launch computes: one per program, or, for a persistent
    kernel, one per iteration of each program's loop over tiles."""
    import numpy as np

    gx, gy, gz = grid
    if gx * gy * gz > (1 << 24):
        raise NotCanonical("grid too large to check")
    px, py, pz = np.meshgrid(np.arange(gx), np.arange(gy), np.arange(gz), indexing="ij")
    env = {"pid_x": px.ravel(), "pid_y": py.ravel(), "pid_z": pz.ravel(),
           "nprog_x": gx, "nprog_y": gy, "nprog_z": gz, "tile_iv": 0}
    names = list(scalars) + list(env)
    local = {n: sp.Symbol(n, integer=True) for n in names}

    def evaluate(text: str) -> "np.ndarray":
        fn = sp.lambdify([local[n] for n in names], sp.sympify(text, locals=local), modules="numpy")
        size = np.asarray(env["pid_x"]).size
        with np.errstate(all="ignore"):
            v = np.broadcast_to(np.asarray(fn(*[scalars[n] for n in scalars], *[env[n] for n in env]), dtype=np.float64), size)
        if not np.isfinite(v).all():
            raise NotCanonical("the tile origin is undefined for some program ids of this grid (division by zero)")
        return v.astype(np.int64)

    if match.tile_loop is not None:
        lo, hi, step = (evaluate(t) for t in match.tile_loop)
        if (step <= 0).any():
            raise NotCanonical("the loop over tiles has a step that is not positive")
        count = np.maximum(0, -(-(hi - lo) // step))
        if int(count.sum()) > (1 << 24):
            raise NotCanonical("too many tiles to check")
        owner = np.repeat(np.arange(count.size), count)
        within = np.arange(owner.size) - np.repeat(np.cumsum(count) - count, count)
        for key in ("pid_x", "pid_y", "pid_z"):
            env[key] = env[key][owner]
        env["tile_iv"] = lo[owner] + within * step[owner]
    extra = [evaluate(t) for t in (match.batch_offsets or [])]
    return evaluate(match.row0), evaluate(match.col0), extra


def bind(match: DotKernelMatch, scalars: dict, grid: tuple, float_args: Optional[dict] = None) -> BoundDot:
    """Check one launch (integer argument values, grid) against the match and return the GEMM it is.

    Raises NotCanonical when this launch is outside what the library kernel reproduces: a layout with no
    unit stride, a grid that does not cover C exactly once, a split point past the last full K block.
    """
    import numpy as np

    grid = tuple(int(g) for g in grid) + (1,) * (3 - len(grid))
    sv = {k: int(v) for k, v in scalars.items()}
    a_r, a_k = _value(match.a_row_stride, sv), _value(match.a_k_stride, sv)
    b_k, b_c = _value(match.b_k_stride, sv), _value(match.b_col_stride, sv)
    c_r, c_c = _value(match.c_row_stride, sv), _value(match.c_col_stride, sv)
    transposed_out = c_c != 1
    if transposed_out and c_r != 1:
        raise NotCanonical(f"C has no unit stride ({c_r}, {c_c})")
    if a_k == 1:
        a_layout, lda = "row", a_r
    elif a_r == 1:
        a_layout, lda = "col", a_k
    else:
        raise NotCanonical(f"A has no unit stride ({a_r}, {a_k})")
    if b_c == 1:
        b_layout, ldb = "row", b_k
    elif b_k == 1:
        b_layout, ldb = "col", b_c
    else:
        raise NotCanonical(f"B has no unit stride ({b_k}, {b_c})")

    for what, x, y in match.equal_at_launch:
        if _value(x, sv) != _value(y, sv):
            raise NotCanonical(f"the operands disagree on {what}: {x} = {_value(x, sv)}, {y} = {_value(y, sv)}")
    hi = _value(match.loop_hi, sv)
    n_iter = max(0, -(-hi // match.loop_step))
    covered = n_iter * match.block_k
    k = _value(match.k_bound, sv)
    if k is None:
        k = covered
    elif covered < k:
        raise NotCanonical(f"the loop covers {covered} of K={k}")
    if k < 1:
        raise NotCanonical("empty K")

    rows, cols, offsets = _tile_origins(match, sv, grid)
    m = _value(match.m_bound, sv)
    n = _value(match.n_bound, sv)
    live = np.ones(rows.shape, bool)
    if m is not None:
        live &= rows < m
    if n is not None:
        live &= cols < n
    if m is None:
        m = int(rows.max()) + match.block_m
    if n is None:
        n = int(cols.max()) + match.block_n
    tm, tn = -(-m // match.block_m), -(-n // match.block_n)
    r, c = rows[live], cols[live]
    if (r % match.block_m).any() or (c % match.block_n).any() or (r < 0).any() or (c < 0).any():
        raise NotCanonical("tile origins are not multiples of the block shape")
    ids = (r // match.block_m) * tn + (c // match.block_n)
    batches = None
    if offsets:
        # One matrix product per distinct (A, B, C) offset triple; each must tile its C exactly once.
        triples = np.stack([o[live] for o in offsets], axis=1)
        uniq, inverse = np.unique(triples, axis=0, return_inverse=True)
        inverse = np.asarray(inverse).reshape(-1)
        if len(uniq) > 4096:
            raise NotCanonical(f"{len(uniq)} matrix products in one launch")
        if np.unique(uniq[:, 2]).size != len(uniq):
            raise NotCanonical("two matrix products of the launch store to the same C")
        for g in range(len(uniq)):
            mine = ids[inverse == g]
            if mine.size != tm * tn or np.unique(mine).size != tm * tn:
                raise NotCanonical(f"the grid {grid} does not cover the {tm}x{tn} tiles of every C exactly once")
        batches = [tuple(int(v) for v in row) for row in uniq]
    elif ids.size != tm * tn or np.unique(ids).size != tm * tn:
        raise NotCanonical(f"the grid {grid} does not cover the {tm}x{tn} tiles of C exactly once")

    k_main = (k // match.block_k) * match.block_k
    if match.split_comparand is not None:
        split = _value(match.split_comparand, sv)
        if match.split_is_loop_bound and split < hi and (split < 0 or split % match.loop_step):  # a second loop runs
            raise NotCanonical(f"split point {split} is not a whole number of steps of {match.loop_step} from 0")
        last = min(split, hi)
        if last > 0:
            iv_max = ((last - 1) // match.loop_step) * match.loop_step
            if iv_max * match.k_per_iv + match.block_k > k:
                raise NotCanonical(f"split point {split} lets an unmasked load run past K={k}")
        k_main = min(k_main, max(0, -(-last // match.loop_step)) * match.block_k)

    alpha = 1.0
    if match.alpha is not None:
        try:
            alpha = float(match.alpha)
        except ValueError:
            alpha = float((float_args or {})[match.alpha])
    for name, ld, need in (("A", lda, k if a_layout == "row" else m), ("B", ldb, n if b_layout == "row" else k),
                           ("C", c_r, n if not transposed_out else 0)):
        if ld < need:
            raise NotCanonical(f"{name}: leading dimension {ld} is smaller than its extent {need}")
    if transposed_out:
        # A column-major C is the row-major C^T = B^T A^T: the library runs with the operands exchanged. B^T[n, k]
        # sits at b + n * b_c + k * b_k (row-major when b_k == 1), A^T[k, m] at a + k * a_k + m * a_r.
        if c_c < m:
            raise NotCanonical(f"C: leading dimension {c_c} is smaller than its extent {m}")
        return BoundDot(m=n, n=m, k=k, a_layout="row" if b_layout == "col" else "col",
                        b_layout="row" if a_layout == "col" else "col", lda=ldb, ldb=lda, ldc=c_c, alpha=alpha,
                        block_k=match.block_k, k_main=k_main, swapped=True,
                        batches=[(ob, oa, oc) for oa, ob, oc in batches] if batches else None)
    return BoundDot(m=m, n=n, k=k, a_layout=a_layout, b_layout=b_layout, lda=lda, ldb=ldb, ldc=c_r,
                    alpha=alpha, block_k=match.block_k, k_main=k_main, batches=batches)
