"""Builds the C++ host mirror's test program (include/catena_b200.hpp + tests/cpp/host_mirror_test.cpp) with g++
against libcatena_b200.so and runs it: pre-call checks on CPU, the reference's known-answer vectors on the GPU."""
import os
import subprocess

import pytest

import catena_lang_b200 as cb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.dirname(cb.LIB_PATH)


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cpp") / "host_mirror_test")
    gxx = os.environ.get("CXX", "g++")
    cmd = [gxx, "-std=c++17", "-O1", "-Wall", "-ffp-contract=off", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include",
           os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"), "-o", out, "-L", LIBDIR, "-lcatena_b200",
           "-Wl,-rpath," + LIBDIR, "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.check_call(cmd)
    return out


def run(binary, mode):
    p = subprocess.run([binary, mode], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.strip().splitlines()[-1].startswith("ok ")


def test_cpp_host_mirror_pre_call_checks(binary):
    run(binary, "cpu")


@pytest.mark.gpu
def test_cpp_host_mirror_known_answers(binary):
    run(binary, "gpu")


def test_cpp_lowering_selector(tmp_path):
    """The C++ kernel selector over the lowered IR (include/catena_b200_lowering.hpp), same fixtures as test_lowering.py."""
    out = str(tmp_path / "lowering_test")
    subprocess.check_call([os.environ.get("CXX", "g++"), "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "lowering_test.cpp"), "-o", out])
    p = subprocess.run([out], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.strip().startswith("ok "), p.stdout + p.stderr


def test_cpp_host_evaluator(tmp_path):
    """The C++ host evaluator of lowered scalar modules (include/catena_b200_eval.hpp) on the reference's integer, bit,
    conditional and fold vectors; built with -ffp-contract=off, the reference's own rule for generated code."""
    out = str(tmp_path / "eval_test")
    subprocess.check_call([os.environ.get("CXX", "g++"), "-std=c++17", "-O1", "-Wall", "-ffp-contract=off", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "eval_test.cpp"), "-o", out])
    p = subprocess.run([out], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.strip().startswith("ok "), p.stdout + p.stderr


@pytest.fixture(scope="module")
def map_program_binary(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cpp") / "map_program_test")
    subprocess.check_call([os.environ.get("CXX", "g++"), "-std=c++17", "-O1", "-Wall", "-ffp-contract=off", "-I", os.path.join(ROOT, "include"),
                           "-I", "/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", "map_program_test.cpp"), "-o", out, "-L", LIBDIR,
                           "-lcatena_b200", "-Wl,-rpath," + LIBDIR, "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64"])
    return out


def test_cpp_map_program_compiler_agrees_with_python(map_program_binary):
    """The C++ and the Python compiler of register programs (include/catena_b200_map_program.hpp, map_program.py) give the same
    program — presets, registers, every instruction — for the reference's materializec programs, a conditional and a fold."""
    import lowered_fixtures as fx
    from catena_lang_b200 import lowering as lo
    p = subprocess.run([map_program_binary, "list"], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stdout + p.stderr
    mm = lo.module_map(fx.materialize_programs() + fx.custom_map_programs())
    lines = []
    for name in ("materialize-indexes", "materialize-copy-u64", "materialize-indexes-source", "my.clamp-map", "my.matvec", "my.poly-map"):
        [assign] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
        prog = lo.map_program_for(assign, mm)
        lines.append(f"program {name} regs={prog.n_regs} index={prog.index_reg} result={prog.result_reg} elem={prog.elem_bytes}")
        for what in prog.presets:
            lines.append(f"  preset {what[0]} {what[1]} {what[2] if what[0] == 'buflen' else 0}")
        for c in prog.code:
            lines.append(f"  insn {c.op} {c.dst} {c.a} {c.b} {c.c} {c.target}")
    fm = lo.module_map(fx.custom_fold_programs())
    [fold] = [a for a in fm["my.horner"].entry.assignments if a.op == "reducec"]
    prog = lo.fold_plan_for(fold, fm).sequential[0]
    lines.append(f"program my.horner regs={prog.n_regs} index={prog.index_reg} result={prog.result_reg} elem={prog.elem_bytes}")
    for what in prog.presets:
        lines.append(f"  preset {what[0]} {what[1]} {what[2] if what[0] == 'buflen' else 0}")
    for c in prog.code:
        lines.append(f"  insn {c.op} {c.dst} {c.a} {c.b} {c.c} {c.target}")
    assert p.stdout.strip().splitlines() == lines


def test_cpp_map_programs_compile_to_the_same_ptx_as_python(map_program_binary, tmp_path):
    """`Program::ptx` (C++) and `MapProgram.ptx` (Python) hand the same program to the library, so the kernel text is the
    same; every file assembles for sm_100a."""
    import shutil
    import lowered_fixtures as fx
    from catena_lang_b200 import lowering as lo
    p = subprocess.run([map_program_binary, "ptx", str(tmp_path)], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stdout + p.stderr
    mm = lo.module_map(fx.materialize_programs() + fx.custom_map_programs())
    programs = []
    for name in ("materialize-indexes", "materialize-copy-u64", "materialize-indexes-source", "my.clamp-map", "my.matvec", "my.poly-map"):
        [assign] = [a for a in mm[name].entry.assignments if a.op == "materializec"]
        programs.append(lo.map_program_for(assign, mm))
    fm = lo.module_map(fx.custom_fold_programs())
    [fold] = [a for a in fm["my.horner"].entry.assignments if a.op == "reducec"]
    programs.append(lo.fold_plan_for(fold, fm).sequential[0])
    ptxas = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    for k, prog in enumerate(programs):
        path = tmp_path / f"program_{k}.ptx"
        assert path.read_text() == prog.ptx()
        if os.path.exists(ptxas):
            subprocess.check_call([ptxas, "-arch=sm_100a", "-o", os.devnull, str(path)])


@pytest.mark.gpu
def test_cpp_map_program_on_the_gpu(map_program_binary):
    run(map_program_binary, "gpu")
