"""Compiled map kernels on the CPU: the PTX the library writes for a register program (csrc/map_jit.cu) — for the
reference's materializec programs, user-style producers, sequential folds and random well-typed producers — assembles for
sm_100a with ptxas, rounds every f32 operation explicitly (so nothing can be contracted into an fma, the reference's
--fmad=false, catena-lang/src/runtime/artifact.rs:59-80), bakes the program's constants in and reads environment values from
the kernel parameters.  The text is produced without a GPU; running it is tests/test_map_program_gpu.py."""
import ctypes as C
import os
import re
import shutil
import subprocess

import numpy as np
import pytest

import catena_lang_b200 as cb
from catena_lang_b200 import lowering as lo
from catena_lang_b200.map_program import OP, Insn, MapProgram
import lowered_fixtures as fx
import random_programs as rp

PTXAS = shutil.which("ptxas") or ("/usr/local/cuda/bin/ptxas" if os.path.exists("/usr/local/cuda/bin/ptxas") else None)


def assemble(text, tmp_path, name="k"):
    if PTXAS is None:
        pytest.skip("ptxas is not installed")
    path = tmp_path / f"{name}.ptx"
    path.write_text(text)
    p = subprocess.run([PTXAS, "-arch=sm_100a", "-v", "-o", os.devnull, str(path)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    return p.stderr


def producers(mods):
    mm = lo.module_map(mods)
    seen = set()
    for m in mods:
        if not m.source_name or m.source_name in seen:
            continue
        seen.add(m.source_name)
        for a in m.entry.assignments:
            if a.op == "materializec":
                yield m.source_name, lo.map_program_for(a, mm)
            elif a.op == "reducec" and lo._touches_memory(a):
                plan = lo.fold_plan_for(a, mm)
                for k, p in enumerate(plan.sequential or []):
                    yield f"{m.source_name}.fold{k}", p
                if plan.staged is not None:
                    yield f"{m.source_name}.getter", plan.staged[0]


def test_every_fixture_program_assembles_for_sm_100a(tmp_path):
    count = 0
    for name, prog in producers(fx.materialize_programs() + fx.custom_map_programs() + fx.custom_fold_programs()):
        text = prog.ptx()
        assert ".target sm_100a" in text and ".entry catena_map_kernel" in text
        info = assemble(text, tmp_path, re.sub(r"[^A-Za-z0-9]", "_", name))
        assert "0 bytes spill stores" in info
        count += 1
    assert count >= 10


@pytest.mark.parametrize("seed", range(400, 408))
def test_random_producers_assemble(seed, tmp_path):
    mods, name = rp.generate(seed, n_ops=60, result="u64" if seed % 2 else "f32", control=seed % 3 != 0)
    mm = lo.module_map(mods)
    [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    text = prog.ptx()
    assemble(text, tmp_path)
    straight = all(c.op not in (OP["JMP"], OP["JZ"]) for c in prog.code)
    # four elements per thread in straight-line code, one when the program branches
    assert ("%l3_" in text) == straight


def test_f32_arithmetic_is_explicitly_rounded_and_constants_are_immediates():
    mm = lo.module_map(fx.custom_map_programs())
    [launch] = [a for a in mm["my.silu-map"].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    text = prog.ptx()
    body = [l.strip() for l in text.splitlines()]
    for l in body:
        m = re.match(r"(@!?%\w+ )?(add|sub|mul|div|fma|rcp)\.(\S+)", l)
        if m and m.group(3).endswith("f32"):
            assert ".rn." in l, l                      # an explicitly rounded operation is never contracted
    # nn.silu has no f32.fma: products and sums round separately.  The only fmas are the PRODUCTS of two elements at once,
    # a * b + (-0) with the -0 from a kernel parameter (a packed mul would be merged with the add behind it by ptxas)
    fmas = [l for l in body if l.startswith("fma")]
    assert fmas and all(l.startswith("fma.rn.f32x2") and l.endswith("%nz2;") for l in fmas)
    assert any(l.startswith("add.rn.f32x2") for l in body) and not any(l.startswith("mul.rn.f32x2") for l in body)
    # 1 / x is the correctly rounded reciprocal (both divisions of nn.sigmoid are 1 / x)
    assert any(l.startswith("rcp.rn.f32") for l in body) and not any(l.startswith("div.") for l in body)
    # the polynomial's coefficients are immediates; the only kernel-parameter preset would be an environment scalar (none here)
    assert "0x3FB8AA3B" in text and "ld.param.b32 %lc_" not in text
    # a producer with an environment scalar reads it from the parameters
    [launch] = [a for a in mm["my.clamp-map"].entry.assignments if a.op == "materializec"]
    assert "ld.param.b32 %lc_0, [p_init+0]" in lo.map_program_for(launch, mm).ptx()


def test_division_shortcuts_are_exact():
    """x / 2^k is emitted as x * 2^-k only while 2^-k is a normal number; any other constant divisor stays a division."""
    def ptx_for(divisor_bits):
        presets = [("const", divisor_bits)]
        code = [Insn(OP["U64_TO_F32"], 2, 1, 0, 0, 0, 0), Insn(OP["F32_DIV"], 2, 2, 0, 0, 0, 0), Insn(OP["HALT"], 0, 0, 0, 0, 0, 0)]
        return MapProgram("by-hand", code, presets, 3, 1, 2, [], 4).ptx()
    assert "mul.rn.f32 %l0_2, %l0_2, 0f3E800000" in ptx_for(0x40800000)          # / 4     -> * 0.25
    assert "mul.rn.f32 %l0_2, %l0_2, 0fBF000000" in ptx_for(0xC0000000)          # / -2    -> * -0.5
    assert "div.rn.f32" in ptx_for(0x40400000)                                   # / 3
    assert "div.rn.f32" in ptx_for(0x7F000000)                                   # / 2^127: the inverse would be subnormal
    assert "div.rn.f32" in ptx_for(0x00000000)                                   # / 0


def test_malformed_programs_get_no_text():
    L = cb.lib()
    need = C.c_uint64(0)

    def status(code, n_init=0, n_regs=4, index_reg=0, result_reg=0, n_buffers=0, elem=8):
        arr = (Insn * len(code))(*code)
        init = (C.c_uint64 * 4)()
        return L.catena_b200_map_ptx_s(arr, len(code), init, None, n_init, n_regs, index_reg, result_reg, n_buffers, elem, None, 0, C.byref(need))

    halt = Insn(OP["HALT"], 0, 0, 0, 0, 0, 0)
    assert status([halt]) == cb.OK and need.value > 100
    assert status([Insn(OP["MOV"], 1, 0, 0, 0, 0, 0)]) == cb.E_BAD_ARG                     # no HALT at the end
    assert status([Insn(OP["MOV"], 9, 0, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG               # register past the file
    assert status([Insn(OP["JMP"], 0, 0, 0, 0, 0, 7), halt]) == cb.E_BAD_ARG               # jump target past the program
    assert status([Insn(OP["LOAD_F32"], 1, 0, 0, 0, 0, 0), halt]) == cb.E_BAD_ARG          # buffer 0 of none
    assert status([halt], elem=2) == cb.E_BAD_ARG
    # a buffer too small for the text is reported, and what fits is terminated
    text = C.create_string_buffer(64)
    arr = (Insn * 1)(halt)
    init = (C.c_uint64 * 4)()
    assert L.catena_b200_map_ptx_s(arr, 1, init, None, 0, 4, 0, 0, 0, 8, text, 64, None) == cb.E_TOO_LARGE
    assert len(text.value) == 63


def test_a_long_branching_producer_compiles_beyond_the_interpreters_register_file(tmp_path):
    """Programs with branches get no register reuse from the host compiler, so a long one needs more than the interpreter's
    256 registers; a compiled kernel's registers are PTX virtual registers (up to 4096) and the assembler allocates the real ones."""
    from catena_lang_b200.map_program import MAX_REGS
    mods, name = rp.generate(1124, n_ops=130, result="u64", control=True)
    mm = lo.module_map(mods)
    [launch] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
    prog = lo.map_program_for(launch, mm)
    assert prog.n_regs > MAX_REGS
    info = assemble(prog.ptx(), tmp_path)
    assert "0 bytes spill stores" in info
    # the interpreter's entry point refuses the same program before any launch
    code = (Insn * len(prog.code))(*prog.code)
    init = (C.c_uint64 * len(prog.presets))()
    bufs = (cb.CatenaMem * 2)()
    out = cb.CatenaMem()
    assert cb.lib().catena_b200_map_program_s(code, len(prog.code), init, len(prog.presets), prog.n_regs, prog.index_reg, prog.result_reg,
                                              bufs, 2, prog.elem_bytes, 4, C.byref(out)) == cb.E_BAD_ARG
