"""LoopSplit on real Triton IR (text level): bisect an ``scf.for`` whose induction variable is compared with a
loop-invariant value, so that the compare is a constant in each half.

This is the transformation of the reference's pass (pass/LoopSplit/LoopSplit.cpp:124-196): the loop is cloned,
the first copy runs [lo, mid), the second [mid, hi) with the first copy's results as its initial values, and the
compare is replaced by ``true`` in one copy and ``false`` in the other; a canonicalisation afterwards (the lit
test's ``-canonicalize``, pass/LoopSplit/test/loop-split.mlir:1) removes the dead ``scf.if`` arms. Accepted loops
are the reference's (:107-144): a positive constant step, an ``arith.cmpi`` with predicate slt / sle / sgt / sge
(or their unsigned forms) on the induction variable, the other operand defined outside the loop; the first such
compare decides the split.

The mid point is computed so that the split keeps the meaning of the loop for every bound (the reference's
arithmetic adds one whole step when the distance is already a multiple of the step and does not clamp to the
loop's range; see the loop_split extension's "intent" mode, which this follows):

    T   = C for  iv < C / iv >= C,   C + 1 for  iv <= C / iv > C
    mid = min(lo + ceildiv(max(T - lo, 0), step) * step, max(hi, lo))

There are no MLIR C++ headers to build a pass against in this environment, so the rewrite works on the printed IR
and the result is checked by parsing it back with Triton's own MLIR context (compiler.B200DotBackend.make_loop_split).
"""
from __future__ import annotations

import re

from .ttir import _VAL, strip_locations

_FOR = re.compile(rf"^(\s*)(?:((?:{_VAL}(?::\d+)?)) = )?scf\.for ({_VAL}) = ({_VAL}) to ({_VAL}) step ({_VAL})"
                  rf"(?: iter_args\((.*?)\) -> \((.*?)\))?\s*(?: : (i\d+))? \{{$")
_CMP = re.compile(rf"^(\s*)({_VAL}) = arith\.cmpi (\w+), ({_VAL}), ({_VAL}) : (i\d+)$")
_CONST = re.compile(rf"^\s*({_VAL}) = arith\.constant (-?\d+) : i\d+$")
_DEF = re.compile(rf"^\s*((?:{_VAL}(?::\d+)?(?:, )?)+) = ")

# predicate -> (compare holds for iv < T, T = C + adjust); the rest hold for iv >= T
_LT = {"slt": 0, "ult": 0, "sle": 1, "ule": 1}
_GE = {"sge": 0, "uge": 0, "sgt": 1, "ugt": 1}
_SWAP = {"slt": "sgt", "sgt": "slt", "sle": "sge", "sge": "sle", "ult": "ugt", "ugt": "ult", "ule": "uge", "uge": "ule"}


def _region_end(lines: list, start: int) -> int:
    """Index of the line closing the region opened by lines[start]."""
    depth = 0
    for i in range(start, len(lines)):
        t = lines[i].strip()
        if t == "} else {":
            continue
        if t.endswith("{"):
            depth += 1
        elif t.startswith("}"):
            depth -= 1
            if depth == 0:
                return i
    raise ValueError("unbalanced regions in the IR text")


def _defined_inside(lines: list) -> set:
    names = set()
    for l in lines:
        m = _DEF.match(l)
        if m:
            for tok in m.group(1).split(", "):
                names.add(tok.split(":")[0])
        f = _FOR.match(l)
        if f:
            names.add(f.group(3))
            if f.group(7):
                names.update(p.split(" = ")[0].strip() for p in f.group(7).split(", "))
    return names


_INVERT = {"slt": "sge", "sge": "slt", "sle": "sgt", "sgt": "sle", "ult": "uge", "uge": "ult", "ule": "ugt", "ugt": "ule"}


def split_loops(text: str, mode: str = "intent") -> tuple:
    """Bisect every eligible loop of the printed module. Returns (new text, number of loops split).

    mode "intent" keeps the loop's meaning for every bound (module docstring). mode "as-written" emits exactly
    the reference's operations (LoopSplit.cpp:147-190): the comparand itself as the mid point, plus or minus one
    step for sge / sle, rounded by `mid_diff += step - mid_diff % step` when the step is not 1, no clamping, a
    compare with the induction variable on the right read with the inverted (not the swapped) predicate, and
    `false` / `true` for sgt-like compares in the first / second loop. It exists so that the reference's own lit
    test can be run against this rewrite; kernels are compiled with "intent"."""
    if mode not in ("intent", "as-written"):
        raise ValueError(mode)
    lines = strip_locations(text).splitlines()
    consts = {m.group(1): int(m.group(2)) for m in map(_CONST.match, lines) if m}
    out, i, n_split = [], 0, 0
    while i < len(lines):
        f = _FOR.match(lines[i])
        if not f:
            out.append(lines[i])
            i += 1
            continue
        end = _region_end(lines, i)
        body = lines[i + 1:end]
        indent, res, iv, lo, hi, step, iters, types, ity = f.groups()
        inside = _defined_inside(body)
        chosen = None
        if ity and consts.get(step, 0) > 0:
            for bi, bl in enumerate(body):
                c = _CMP.match(bl)
                if not c:
                    continue
                pred, x, y = c.group(3), c.group(4), c.group(5)
                if y == iv and x != iv:
                    pred, x, y = (_INVERT if mode == "as-written" else _SWAP).get(pred), y, x
                if x != iv or y == iv or pred not in _LT and pred not in _GE or y in inside:
                    continue
                chosen = (bi, c, pred, y)
                break
        if chosen is None:
            out.append(lines[i])  # not a loop to split; loops nested inside it are still looked at
            i += 1
            continue
        bi, c, pred, comparand = chosen
        tag = f"%ls{n_split}"
        holds_first = pred in _LT
        adjust = _LT[pred] if holds_first else _GE[pred]
        if mode == "as-written":
            greater, equal, stepv = pred in _GE, pred in ("sge", "sle", "uge", "ule"), consts[step]
            pre, midp = [], comparand
            if equal:
                pre += [f"{indent}{tag}_inc = arith.constant {-stepv if greater else stepv} : {ity}",
                        f"{indent}{tag}_t = arith.addi {comparand}, {tag}_inc : {ity}"]
                midp = f"{tag}_t"
            if stepv != 1:
                pre += [f"{indent}{tag}_d = arith.subi {midp}, {lo} : {ity}",
                        f"{indent}{tag}_r = arith.remui {tag}_d, {step} : {ity}",
                        f"{indent}{tag}_u = arith.subi {step}, {tag}_r : {ity}",
                        f"{indent}{tag}_e = arith.addi {tag}_d, {tag}_u : {ity}",
                        f"{indent}{tag}_mid = arith.addi {lo}, {tag}_e : {ity}"]
                midp = f"{tag}_mid"
            holds_first = not greater
        pre_intent = [f"{indent}{tag}_c0 = arith.constant 0 : {ity}"]
        thr = comparand
        if adjust:
            pre_intent += [f"{indent}{tag}_c1 = arith.constant 1 : {ity}",
                    f"{indent}{tag}_t = arith.addi {comparand}, {tag}_c1 : {ity}"]
            thr = f"{tag}_t"
        pre_intent += [f"{indent}{tag}_d = arith.subi {thr}, {lo} : {ity}",
                f"{indent}{tag}_p = arith.maxsi {tag}_d, {tag}_c0 : {ity}",
                f"{indent}{tag}_q = arith.ceildivsi {tag}_p, {step} : {ity}",
                f"{indent}{tag}_m = arith.muli {tag}_q, {step} : {ity}",
                f"{indent}{tag}_a = arith.addi {lo}, {tag}_m : {ity}",
                f"{indent}{tag}_h = arith.maxsi {hi}, {lo} : {ity}",
                f"{indent}{tag}_mid = arith.minsi {tag}_a, {tag}_h : {ity}"]
        if mode == "intent":
            pre, midp = pre_intent, f"{tag}_mid"

        def copy(first: bool) -> list:
            value = "true" if (first == holds_first) else "false"
            b = list(body)
            b[bi] = f"{c.group(1)}{c.group(2)} = arith.constant {value}"
            return b

        iter_pairs = [p.split(" = ") for p in iters.split(", ")] if iters else []
        n_res = len(iter_pairs)
        main = f"{tag}_main"
        main_refs = [main if n_res == 1 else f"{main}#{k}" for k in range(n_res)]
        head1 = f"{indent}" + (f"{main}{'' if n_res == 1 else ':' + str(n_res)} = " if n_res else "")
        head1 += f"scf.for {iv} = {lo} to {midp} step {step}"
        head2 = f"{indent}" + (f"{res} = " if res else "") + f"scf.for {iv} = {midp} to {hi} step {step}"
        if n_res:
            head1 += f" iter_args({iters}) -> ({types})"
            second = ", ".join(f"{a.strip()} = {r}" for (a, _), r in zip(iter_pairs, main_refs))
            head2 += f" iter_args({second}) -> ({types})"
        head1 += f"  : {ity} {{"
        head2 += f"  : {ity} {{"
        out += pre + [head1] + copy(True) + [lines[end], head2] + copy(False) + [lines[end]]
        n_split += 1
        i = end + 1
    return "\n".join(out) + "\n", n_split
