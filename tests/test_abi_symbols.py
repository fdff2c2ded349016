"""The C-ABI library loads on a machine without a GPU, exports every symbol the header
declares, and refuses compute calls loudly instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "cleave_cuda.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cleave_cuda_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def built():
    from cleave_b200 import build
    return build.build()


def test_header_declares_the_operator_surface():
    names = _declared_symbols()
    for must in ("gemm_f32", "gemm_nt_f32", "gemm_tn_f32", "gemm_batched_f32", "add_f32", "sub_f32", "mul_f32",
                 "div_f32", "neg_f32", "relu_f32", "sigmoid_f32", "tanh_f32", "exp_f32", "sum_f32", "mean_f32",
                 "max_f32", "tanh_bwd_f32", "sigmoid_bwd_f32", "upload_f32", "download_f32", "get_f32"):
        assert f"cleave_cuda_{must}" in names


def test_library_exports_every_declared_symbol(built):
    L = ctypes.CDLL(built)
    missing = [n for n in _declared_symbols() if not hasattr(L, n)]
    assert not missing, missing


def test_python_binding_covers_every_declared_symbol(built):
    from cleave_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    _lib.lib()   # applies every signature; raises on a missing symbol


def test_no_cpu_fallback_without_a_device(built):
    import numpy as np

    import cleave_b200 as cb
    L = cb.lib()
    if L.cleave_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(cb.CleaveCudaError) as ei:
        cb.Tensor(np.ones(4, np.float32))
    assert ei.value.code == 1   # CLEAVE_CUDA_ERR_NO_DEVICE
    assert L.cleave_cuda_alloc_f32(16) is None
    assert L.cleave_cuda_last_error() == 1
    L.cleave_cuda_clear_error()
    assert L.cleave_cuda_last_error() == 0


def test_bad_handles_are_rejected_without_touching_them(built):
    import cleave_b200 as cb
    L = cb.lib()
    bogus = ctypes.c_void_p(0xDEAD0000)
    assert L.cleave_cuda_len(bogus) == -2            # CLEAVE_CUDA_ERR_BAD_HANDLE
    assert L.cleave_cuda_add_f32(bogus, bogus) is None
    assert L.cleave_cuda_last_error() == 2
    assert b"not a live tensor handle" in L.cleave_cuda_last_error_message()
    assert L.cleave_cuda_gemm_f32(None, None, 2, 2, 2) is None
    L.cleave_cuda_free(bogus)                        # must not crash
    L.cleave_cuda_clear_error()


def _cleave_externs():
    """(file, symbol, number of C-level arguments) for every ``extern(cleave_cuda_*) fn`` of the shipped
    cleave-side files.  An array parameter ``[T; N]`` is two C arguments, pointer and length
    (cleave/src/mlir_lower.rs:1096-1113); ``const`` is not valid inside a parameter list
    (cleave/src/grammar.pest:116) and is refused here."""
    out = []
    base = os.path.join(ROOT, "cleave_b200", "cleave")
    for dirpath, _, files in os.walk(base):
        for fn in files:
            if not fn.endswith(".cleave"):
                continue
            with open(os.path.join(dirpath, fn)) as f:
                text = re.sub(r"//[^\n]*", "", f.read())
            for sym, params in re.findall(r"extern\((cleave_cuda_\w+)\)\s*fn\s+\w+\s*\(([^)]*)\)", text):
                n = 0
                for prm in [x.strip() for x in params.split(",") if x.strip()]:
                    assert not prm.startswith("const "), f"{fn}: `{prm}`: const generics belong on the impl"
                    n += 2 if re.search(r":\s*\[", prm) else 1
                out.append((fn, sym, n))
    return out


def test_cleave_side_bindings_name_real_entry_points():
    from cleave_b200 import _lib
    externs = _cleave_externs()
    assert len(externs) >= 25
    for fn, sym, nargs in externs:
        assert sym in _lib.SIGNATURES, f"{fn}: {sym} is not in the C ABI"
        assert len(_lib.SIGNATURES[sym][1]) == nargs, f"{fn}: {sym} takes {len(_lib.SIGNATURES[sym][1])} arguments"


def test_generated_rust_bindings_are_current_and_complete():
    import subprocess
    import sys
    gen = os.path.join(ROOT, "cleave_b200", "cleave", "gen_rust_bindings.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0, "run gen_rust_bindings.py"
    with open(os.path.join(ROOT, "cleave_b200", "cleave", "rust", "cleave_cuda_sys.rs")) as f:
        text = f.read()
    for name in _declared_symbols():
        assert f"pub fn {name}(" in text and f'register_symbol("{name}"' in text, name


def test_cleave_files_keep_const_generics_out_of_parameter_lists():
    # cleave/src/grammar.pest:116 allows `const` only in generic_params (`impl<const N: i32> ...`, `fn f<const N: i32>`),
    # never inside a parameter list; a top-level extern fn cannot be generic at all (cleave/tests/callgraph.rs:227-233).
    base = os.path.join(ROOT, "cleave_b200", "cleave")
    seen = 0
    for dirpath, _, files in os.walk(base):
        for fn in files:
            if not fn.endswith(".cleave"):
                continue
            with open(os.path.join(dirpath, fn)) as f:
                text = re.sub(r"//[^\n]*", "", f.read())
            for name, params in re.findall(r"\bfn\s+(\w+)\s*(?:<[^>]*>)?\s*\(([^)]*)\)", text):
                seen += 1
                assert "const " not in params, f"{fn}: fn {name}({params.strip()})"
            for decl in re.findall(r"^\s*extern\s+fn\s+\w+\s*<", text, flags=re.M):
                raise AssertionError(f"{fn}: generic top-level extern fn: {decl.strip()}")
    assert seen > 60
