"""The pass-plugin C-ABI: symbols, registration at dlopen, enumerate / register / add semantics.

Expected behaviour is the reference's infra/pass/TritonExtPassInfra.cpp:7-52, except where
include/triton_ext_plugin.h documents a deliberate difference (enumeration fills every slot)."""
import ctypes
import os
import re
import subprocess

from triton_ext_b200 import plugin as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")


def _exported(lib_path):
    out = subprocess.run(["nm", "-D", "--defined-only", lib_path], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def _declared(header, prefix_regex):
    text = open(os.path.join(INCLUDE, header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(prefix_regex, text))


def test_infra_exports_the_four_plugin_symbols(built_libs):
    syms = _exported(P.infra_path())
    for s in ("tritonAddPluginPass", "tritonRegisterPluginPass", "tritonEnumeratePluginPasses", "TritonExtLoadPass"):
        assert s in syms


def test_every_declared_symbol_is_exported(built_libs):
    infra_syms = _exported(P.infra_path())
    dot_syms = _exported(P.plugin_path("b200_dot"))
    for name in _declared("triton_ext_dot_ir.h", r"\b(txir_\w+)\s*\("):
        assert name in infra_syms or name in dot_syms, name
    for name in _declared("b200_dot.h", r"\b(tx_dot_\w+)\s*\("):
        assert name in dot_syms, name
    split_syms = _exported(P.plugin_path("loop_split"))
    text_api = _declared("triton_ext_loop_split_text.h", r"\b(tx_loop_split_\w+)\s*\(")
    assert set(text_api) == {"tx_loop_split_text", "tx_loop_split_free"}
    for name in text_api:
        assert name in split_syms, name
    attn = _declared("b200_attention.h", r"\b(tx_attn_\w+)\s*\(")
    assert len(attn) >= 6
    for name in attn:
        assert name in dot_syms, name


def test_extensions_register_at_dlopen_in_load_order(built_libs):
    # Registration order is dlopen order, so ask a fresh interpreter: other tests of this process may
    # already have loaded the backend library on its own.
    import json
    import subprocess
    import sys

    code = ("import json; from triton_ext_b200 import plugin as P; P.load_default_plugins(); "
            "print(json.dumps(P.enumerate_passes()))")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    names = json.loads(out.stdout.strip().splitlines()[-1])
    assert names[:3] == ["loop_split", "dot_tile_select", "b200_dot"]
    # every slot is filled (the reference leaves all names in slot 0, TritonExtPassInfra.cpp:47-50)
    assert len(set(names)) == len(names)
    P.load_default_plugins()
    assert set(P.enumerate_passes()) >= {"loop_split", "dot_tile_select", "b200_dot"}


def test_enumerate_protocol(built_libs):
    P.load_default_plugins()
    lib = P.infra()
    assert lib.tritonEnumeratePluginPasses(None, None) == P.TP_GENERIC_FAILURE  # null count -> failure
    n = ctypes.c_uint32(0)
    assert lib.tritonEnumeratePluginPasses(ctypes.byref(n), None) == P.TP_SUCCESS  # count only
    assert n.value >= 3


def test_unknown_and_null_names_fail(built_libs):
    P.load_default_plugins()
    lib = P.infra()
    pm = P.PassManager()
    assert pm.add("no_such_pass") == P.TP_GENERIC_FAILURE
    assert P.register_pass("no_such_pass") == P.TP_GENERIC_FAILURE
    assert lib.tritonRegisterPluginPass(None) == P.TP_GENERIC_FAILURE
    assert lib.tritonAddPluginPass(pm._h, None) == P.TP_GENERIC_FAILURE
    assert lib.tritonAddPluginPass(None, b"loop_split") == P.TP_GENERIC_FAILURE
    assert pm.arguments() == []


def test_add_appends_in_order_and_register_is_idempotent(built_libs):
    P.load_default_plugins()
    pm = P.PassManager()
    assert pm.add("loop_split") == P.TP_SUCCESS
    assert pm.add("b200_dot") == P.TP_SUCCESS
    assert pm.add("loop_split") == P.TP_SUCCESS
    assert pm.arguments() == ["triton-loop-split", "triton-b200-dot", "triton-loop-split"]
    assert P.register_pass("loop_split") == P.TP_SUCCESS
    count = P.infra().txir_registered_pass_count()
    assert P.register_pass("loop_split") == P.TP_SUCCESS
    assert P.infra().txir_registered_pass_count() == count
    assert P.registered_pass_lookup("triton-loop-split") >= 0
    assert P.registered_pass_lookup("triton-nope") == -1


def test_load_pass_from_a_foreign_extension(built_libs, tmp_path):
    """A third-party extension written against the public headers only (C callbacks) can register."""
    src = tmp_path / "ext.c"
    src.write_text(r'''
#include "triton_ext_plugin.h"
static int registered = 0, added = 0;
static void reg(void) { registered++; }
static void add(TritonExtPassManagerRef pm) { (void)pm; added++; }
__attribute__((constructor)) static void init(void) { TritonExtLoadPass("foreign_ext", reg, add); }
__attribute__((visibility("default"))) int foreign_counts(void) { return registered * 100 + added; }
''')
    so = tmp_path / "libforeign_ext.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-I", INCLUDE, str(src), "-o", str(so),
                    "-L", os.path.dirname(P.infra_path()), "-lTritonExtPassInfra",
                    f"-Wl,-rpath,{os.path.dirname(P.infra_path())}"], check=True)
    P.load_plugins_from_env(str(so))
    assert "foreign_ext" in P.enumerate_passes()
    pm = P.PassManager()
    assert pm.add("foreign_ext") == P.TP_SUCCESS
    assert P.register_pass("foreign_ext") == P.TP_SUCCESS
    lib = ctypes.CDLL(str(so))
    assert lib.foreign_counts() == 101


def test_threaded_lookups(built_libs):
    import threading
    P.load_default_plugins()
    errs = []

    def work():
        for _ in range(200):
            pm = P.PassManager()
            if pm.add("loop_split") != P.TP_SUCCESS or "loop_split" not in P.enumerate_passes():
                errs.append(1)

    ts = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs


def test_loop_split_text_entry_point(built_libs):
    """tx_loop_split_text through its C-ABI: argument checks, a loop it must leave alone, one it must bisect."""
    lib = P.load_plugin(P.plugin_path("loop_split"))
    lib.tx_loop_split_text.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_int32)]
    lib.tx_loop_split_free.argtypes = [ctypes.c_void_p]
    out, n = ctypes.c_void_p(), ctypes.c_int32(-1)
    assert lib.tx_loop_split_text(None, 0, ctypes.byref(out), ctypes.byref(n)) == 1
    assert lib.tx_loop_split_text(b"module {\n}\n", 7, ctypes.byref(out), ctypes.byref(n)) == 1
    unbalanced = b"  scf.for %i = %a to %b step %c  : i32 {\n    %x = arith.addi %i, %i : i32\n"
    assert lib.tx_loop_split_text(unbalanced, 0, ctypes.byref(out), ctypes.byref(n)) == 2

    def run(text: str, mode: int = 0):
        o, k = ctypes.c_void_p(), ctypes.c_int32(-1)
        assert lib.tx_loop_split_text(text.encode(), mode, ctypes.byref(o), ctypes.byref(k)) == 0
        try:
            return ctypes.string_at(o).decode(), k.value
        finally:
            lib.tx_loop_split_free(o)

    loop = ("  %c4 = arith.constant 4 : i32\n"
            "  %r = scf.for %i = %lo to %hi step %c4 iter_args(%acc = %z) -> (i32)  : i32 {\n"
            "    %p = arith.cmpi PRED, %i, CMP : i32\n"
            "    %s = arith.select %p, %i, %acc : i32\n"
            "    scf.yield %s : i32\n"
            "  }\n")
    text, k = run(loop.replace("PRED", "slt").replace("CMP", "%mid"))
    assert k == 1 and text.count("scf.for") == 2
    assert "%ls0_main = scf.for %i = %lo to %ls0_mid step %c4 iter_args(%acc = %z) -> (i32)  : i32 {" in text
    assert "%r = scf.for %i = %ls0_mid to %hi step %c4 iter_args(%acc = %ls0_main) -> (i32)  : i32 {" in text
    assert text.index("%p = arith.constant true") < text.index("%p = arith.constant false")
    assert "arith.ceildivsi" in text and "arith.minsi" in text
    written, _ = run(loop.replace("PRED", "sge").replace("CMP", "%mid"), 1)
    assert "%ls0_inc = arith.constant -4 : i32" in written and "arith.remui" in written and "arith.minsi" not in written
    assert written.index("%p = arith.constant false") < written.index("%p = arith.constant true")
    # not split: equality compare; comparand defined inside the loop; non-constant step
    for variant in (loop.replace("PRED", "eq").replace("CMP", "%mid"),
                    loop.replace("PRED", "slt").replace("CMP", "%s"),
                    loop.replace("PRED", "slt").replace("CMP", "%mid").replace("step %c4", "step %step")):
        same, k = run(variant)
        assert k == 0 and same == variant


def test_loop_split_text_scopes_names_per_function_and_balances_while_regions(built_libs):
    """SSA names repeat from one tt.func to the next: the step constant (and, for the mask form, every definition) of a
    loop must be looked up in the function that holds the loop. And `} do {` of an scf.while closes one region and opens
    the next, like `} else {`: a loop behind a while must still be found, and its end must be the right brace."""
    lib = P.load_plugin(P.plugin_path("loop_split"))
    lib.tx_loop_split_text.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_int32)]
    lib.tx_loop_split_free.argtypes = [ctypes.c_void_p]

    def run(text: str, mode: int = 1):
        o, k = ctypes.c_void_p(), ctypes.c_int32(-1)
        assert lib.tx_loop_split_text(text.encode(), mode, ctypes.byref(o), ctypes.byref(k)) == 0
        try:
            return ctypes.string_at(o).decode(), k.value
        finally:
            lib.tx_loop_split_free(o)

    def func(name, step):
        return (f"  tt.func public @{name}(%lo: i32, %hi: i32, %mid: i32, %z: i32) {{\n"
                f"    %c = arith.constant {step} : i32\n"
                "    %r = scf.for %i = %lo to %hi step %c iter_args(%acc = %z) -> (i32)  : i32 {\n"
                "      %p = arith.cmpi sge, %i, %mid : i32\n"
                "      %s = arith.select %p, %i, %acc : i32\n"
                "      scf.yield %s : i32\n"
                "    }\n"
                "    tt.return\n"
                "  }\n")
    # as-written mode writes the step into the text (-step for sge): each function must get its own %c
    text, k = run("module {\n" + func("f", 4) + func("g", 16) + "}\n")
    assert k == 2
    first, second = text.split("tt.func public @g")
    assert "arith.constant -4 : i32" in first and "arith.constant -16 : i32" not in first
    assert "arith.constant -16 : i32" in second and "arith.constant -4 : i32" not in second
    # a loop in a function whose step is only defined in ANOTHER function is not split (no constant step in scope)
    stray = func("f", 4) + func("g", 16).replace("    %c = arith.constant 16 : i32\n", "").replace("(%lo: i32,", "(%c: i32, %lo: i32,")
    text, k = run("module {\n" + stray + "}\n")
    assert k == 1 and text.count("scf.for") == 3
    # scf.while before the loop: `} do {` must not unbalance the region count
    while_loop = ("  %w = scf.while (%a = %z) : (i32) -> i32 {\n"
                  "    %cond = arith.cmpi slt, %a, %hi : i32\n"
                  "    scf.condition(%cond) %a : i32\n"
                  "  } do {\n"
                  "  ^bb0(%b: i32):\n"
                  "    %n = arith.addi %b, %b : i32\n"
                  "    scf.yield %n : i32\n"
                  "  }\n")
    loop = ("  %c4 = arith.constant 4 : i32\n"
            "  %r = scf.for %i = %lo to %hi step %c4 iter_args(%acc = %w) -> (i32)  : i32 {\n"
            "    %p = arith.cmpi slt, %i, %mid : i32\n"
            "    %s = arith.select %p, %i, %acc : i32\n"
            "    scf.yield %s : i32\n"
            "  }\n")
    text, k = run(while_loop + loop, 0)
    assert k == 1 and text.count("scf.for") == 2 and text.count("scf.while") == 1
    # a loop INSIDE the while's body is found as well, and the while's closing brace stays where it was
    nested = while_loop.replace("    %n = arith.addi %b, %b : i32\n", loop.replace("\n  ", "\n    ").replace("  %c4", "    %c4", 1)
                                .replace("%acc = %w", "%acc = %b") + "    %n = arith.addi %r, %b : i32\n")
    text, k = run(nested, 0)
    assert k == 1 and text.count("scf.for") == 2 and text.rstrip().endswith("}")


def test_loop_split_text_peels_masked_remainder(built_libs):
    """The mask form through the C-ABI: tensor compares of (splat iv + range) with a splat bound."""
    lib = P.load_plugin(P.plugin_path("loop_split"))
    lib.tx_loop_split_text.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.POINTER(ctypes.c_int32)]
    lib.tx_loop_split_free.argtypes = [ctypes.c_void_p]
    text = ("  %c32 = arith.constant 32 : i32\n"
            "  %range = tt.make_range {end = 32 : i32, start = 0 : i32} : tensor<32xi32>\n"
            "  %r = scf.for %k = %c0 to %K step %c32 iter_args(%acc = %z) -> (tensor<16x16xf32>)  : i32 {\n"
            "    %s = tt.splat %k : i32 -> tensor<32xi32>\n"
            "    %idx = arith.addi %s, %range : tensor<32xi32>\n"
            "    %row = tt.expand_dims %idx {axis = 0 : i32} : tensor<32xi32> -> tensor<1x32xi32>\n"
            "    %kb = tt.splat %K : i32 -> tensor<1x32xi32>\n"
            "    %m = arith.cmpi slt, %row, %kb : tensor<1x32xi32>\n"
            "    %mb = tt.broadcast %m : tensor<1x32xi1> -> tensor<16x32xi1>\n"
            "    %a = tt.load %p, %mb, %zero : tensor<16x32x!tt.ptr<f16>>\n"
            "    scf.yield %acc : tensor<16x16xf32>\n"
            "  }\n")

    def run(t: str, mode: int):
        o, k = ctypes.c_void_p(), ctypes.c_int32(-1)
        assert lib.tx_loop_split_text(t.encode(), mode, ctypes.byref(o), ctypes.byref(k)) == 0
        try:
            return ctypes.string_at(o).decode(), k.value
        finally:
            lib.tx_loop_split_free(o)

    out, k = run(text, 0)
    assert k == 1 and out.count("scf.for") == 2
    assert "%ls0_e = arith.constant 31 : i32" in out and "%ls0_b = arith.subi %K, %ls0_e : i32" in out
    first, second = out.split("scf.for")[1:]
    assert "%m = arith.constant dense<true> : tensor<1x32xi1>" in first and "arith.cmpi" not in first
    assert "%m = arith.cmpi slt, %row, %kb : tensor<1x32xi32>" in second
    assert run(text, 1) == (text, 0)                                             # not in the as-written mode
    assert run(text.replace("tt.splat %K", "tt.splat %k"), 0)[1] == 0            # bound is the induction variable
    assert run(text.replace("start = 0", "start = 1"), 0)[1] == 0                # range does not start at 0
