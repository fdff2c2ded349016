"""The reference-side change set (lowering hook, JIT registration, link lines, handle-typed export bindings) is
delivered as one unified diff.  No Rust toolchain exists where this suite runs, so "compiles" is not checked;
what is checked is that the diff applies cleanly to the reference files it names and leaves the hook in place."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATCH = os.path.join(ROOT, "cleave_b200", "cleave", "patches", "cleave_cuda_backend.patch")
# the reference checkout: CLEAVE_REFERENCE_DIR, else a directory named `reference` beside this repository
REFERENCE = os.environ.get("CLEAVE_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference"))


def _patched_files():
    with open(PATCH) as f:
        text = f.read()
    return sorted(set(re.findall(r"^\+\+\+ b/(\S+)", text, flags=re.M)))


def test_patch_names_the_documented_files():
    files = _patched_files()
    for must in ("cleave/src/mlir_lower.rs", "cleave/src/pipeline.rs", "cleave-build/src/lib.rs",
                 "cleave/src/rust_bindings.rs", "cleave/Cargo.toml", "cleave-cuda-sys/Cargo.toml"):
        assert must in files, must
    with open(PATCH) as f:
        text = f.read()
    # every symbol the hook calls is an entry point of the C ABI
    from cleave_b200 import _lib
    for sym in set(re.findall(r'"(cleave_cuda_\w+)"', text)):
        assert sym in _lib.SIGNATURES, sym


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="the reference tree is not present on this machine")
@pytest.mark.skipif(shutil.which("patch") is None, reason="no patch(1) on this machine")
def test_patch_applies_to_the_reference_tree(tmp_path):
    for rel in _patched_files():
        src = os.path.join(REFERENCE, rel)
        if os.path.exists(src):           # files the patch creates have no original
            dst = tmp_path / rel
            dst.parent.mkdir(parents=True, exist_ok=True)
            shutil.copy(src, dst)
    dry = subprocess.run(["patch", "--dry-run", "-p1", "-i", PATCH], cwd=tmp_path, capture_output=True, text=True)
    assert dry.returncode == 0, dry.stdout + dry.stderr
    assert "FAILED" not in dry.stdout and "fuzz" not in dry.stdout, dry.stdout
    real = subprocess.run(["patch", "-p1", "-i", PATCH], cwd=tmp_path, capture_output=True, text=True)
    assert real.returncode == 0, real.stdout + real.stderr
    lowered = (tmp_path / "cleave/src/mlir_lower.rs").read_text()
    assert "fn lower_tensor_op_to_device_call" in lowered and "cleave_cuda_host_gemm_f32" in lowered
    assert lowered.count("if device_backend_enabled()") == 1
    assert "register_cleave_cuda_symbols(engine)" in (tmp_path / "cleave/src/pipeline.rs").read_text()
    assert "rustc-link-lib=dylib=cleave_cuda" in (tmp_path / "cleave-build/src/lib.rs").read_text()
    # the generated declarations complete the new crate
    shutil.copy(os.path.join(ROOT, "cleave_b200", "cleave", "rust", "cleave_cuda_sys.rs"),
                tmp_path / "cleave-cuda-sys" / "src" / "lib.rs") if (tmp_path / "cleave-cuda-sys" / "src").exists() else None
    assert (tmp_path / "cleave-cuda-sys" / "Cargo.toml").exists() and (tmp_path / "cleave-cuda-sys" / "build.rs").exists()
