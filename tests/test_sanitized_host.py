"""The code that parses untrusted bytes - the prefix store, the ITKV decoder (both in the library's host-only part)
and the oracle's own decoders - rebuilt under AddressSanitizer and UndefinedBehaviorSanitizer and driven by the same
CPU tests, forged entries and forged snapshots included.  A sanitizer report aborts the child process, so a clean
exit means no out-of-bounds access, no use after free and no undefined arithmetic on those inputs.  CPU only."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DRIVER = textwrap.dedent("""
    import sys
    sys.path.insert(0, {root!r})
    sys.path.insert(0, {tests!r})
    from itak_torch_rebuild_b200 import _lib
    from oracle import oracle as orc
    # the sanitized builds stand in for the ordinary ones; the host-only library exports the store and the decoder
    _lib.SO_PATH = {lib!r}
    _lib.SIGNATURES = {{k: v for k, v in _lib.SIGNATURES.items() if k.startswith("itk_prefix_store") or k == "itk_itkv_check"}}
    orc._LIB_PATH = {oracle!r}
    orc.build = lambda force=False: orc._LIB_PATH
    import pytest
    sys.exit(pytest.main(["-x", "-q", "-p", "no:cacheprovider"] + {files!r}))
""")


def test_parsers_run_clean_under_the_sanitizers(tmp_path):
    from itak_torch_rebuild_b200 import build

    cxx = build.sanitizer_compiler()
    if cxx is None:
        pytest.skip("no compiler here links the sanitizer runtimes")
    lib = build.build_sanitized()
    made = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), f"CXX={cxx}", "liboracle_asan.so"],
                          capture_output=True, text=True)
    assert made.returncode == 0, made.stderr
    runtimes = []
    for name in ("libasan.so", "libubsan.so"):
        path = subprocess.run([cxx, f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
        assert os.path.isabs(path), f"{name} not found beside {cxx}"
        runtimes.append(os.path.realpath(path))
    files = [os.path.join(ROOT, "tests", f) for f in ("test_prefix_store.py", "test_itkv_codec.py", "test_oracle_snapshot.py")]
    script = tmp_path / "drive.py"
    script.write_text(DRIVER.format(root=ROOT, tests=os.path.join(ROOT, "tests"), lib=lib,
                                    oracle=os.path.join(ROOT, "oracle", "liboracle_asan.so"), files=files))
    env = dict(os.environ)
    env["LD_PRELOAD"] = ":".join(runtimes)
    # the interpreter itself is not instrumented: its own exit-time leaks are not the subject here
    env["ASAN_OPTIONS"] = "detect_leaks=0:abort_on_error=1:halt_on_error=1"
    env["UBSAN_OPTIONS"] = "halt_on_error=1:print_stacktrace=1"
    res = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=600)
    report = res.stdout[-3000:] + res.stderr[-3000:]
    assert res.returncode == 0, report
    assert "ERROR: AddressSanitizer" not in report and "runtime error:" not in report, report
    assert " passed" in res.stdout
