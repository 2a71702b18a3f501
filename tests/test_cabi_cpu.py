"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares, the
host-executed scalar programs are bit-exact with the oracle, and the host mirror of the reference's
Runtime surface behaves like catena-lang/tests/runtime.rs:128-168 expects.  No device compute here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import catena_lang_b200 as cb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "catena_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:program|catena_b200)_[A-Za-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = cb.lib()
    names = declared_symbols()
    assert len(names) > 60
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_symbol_mangling_matches_reference_rule():
    # codegen/mod.rs:379-388
    assert cb.symbol_for("nn.gelu-approx") == "program_nn_gelu_approx"
    assert cb.symbol_for("matmul-2x2-via-mem") == "program_matmul_2x2_via_mem"
    assert cb.symbol_for("2x") == "program__2x"


def test_scalar_programs_bit_exact_with_oracle(orc):
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.uniform(-20, 20, 4000), rng.uniform(-1, 1, 2000), [0.0, -0.0, 1.0, -1.0, 87.0, -87.0]]
                        ).astype(np.float32)
    L = cb.lib()
    for name in cb.SCALAR_PROGRAMS:
        inp = np.abs(xs) + np.float32(1e-3) if name in ("math.log-approx", "math.log2-approx",
                                                        "math.sin-approx-full-nonneg", "math.exp-approx-nonneg") else xs
        want = orc.map_unary(name, inp)
        fn = getattr(L, cb.symbol_for(name))
        got = np.empty_like(inp)
        out = C.c_float()
        for i, x in enumerate(inp):
            fn(C.c_float(x), C.byref(out))
            got[i] = out.value
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    out = C.c_float()
    for b, e in [(0.25, 0.5), (2.0, 3.0), (10.0, 0.25), (1.5, -1.0)]:
        L.program_math_powf(C.c_float(b), C.c_float(e), C.byref(out))
        assert np.float32(out.value).view(np.uint32) == np.float32(orc.scalar("math.powf", b, e)).view(np.uint32)


def test_runtime_surface_errors():
    rt = cb.Runtime.from_sources([""], cb.GpuDialect.Cuda)
    # tests/runtime.rs:128-168
    with pytest.raises(cb.ExecError) as e:
        rt.exec("does-not-exist", [])
    assert e.value.kind == "UnknownSourceFunction"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("math.sqrt", [])
    assert e.value.kind == "InputArityMismatch"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("math.sqrt", [cb.Value.f32(4.0)], n_outputs=2)
    assert e.value.kind == "OutputArityMismatch"
    with pytest.raises(cb.ExecError) as e:
        rt.exec("math.sqrt", [cb.Value.u64(4)])
    assert e.value.kind == "TypeMismatch"
    [r] = rt.exec("math.sqrt", [cb.Value.f32(9.0)])
    assert r.kind is cb.ValueKind.F32 and abs(r.v - 3.0) < 1e-4
    with pytest.raises(cb.InitError):
        cb.Runtime.from_sources([""], cb.GpuDialect.Hip)


def test_user_programs_need_a_definition():
    rt = cb.Runtime.from_sources([""])
    assert "matmul-2x2-via-mem" not in rt.signatures
    src = "(def program matmul-2x2-via-mem : ([n m k.] {}) -> ([n m k.] (cap.own mem)) = ())"
    rt = cb.Runtime.from_sources([src])
    assert rt.signatures["matmul-2x2-via-mem"][0] == "program_matmul_2x2_via_mem"


@pytest.mark.skipif(cb.lib().catena_b200_device_count() > 0, reason="a GPU is present")
def test_no_device_fails_loudly():
    m = cb.CatenaMem()
    s = cb.lib().catena_b200_mem_alloc(16, C.byref(m))
    assert s == cb.E_NO_DEVICE
    out = C.c_float(123.0)
    s = cb.lib().program_sum_f32_s(cb.CatenaMem(C.c_void_p(16), 16), C.byref(out))
    assert s == cb.E_NO_DEVICE
