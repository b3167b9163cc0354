"""The reference-side adapter (integration/b200_nvfp4_mtp_provider.cpp) is real code: compiled with the
reference's own headers, linked with the reference's registry and program executor
(runtime/src/{model_descriptor,execution_provider,program_executor,sha256}.cpp, from where they lie)
and a stub of this library's C ABI, then driven the way the reference's
runtime/tests/cache_state_test.cpp drives its fixture provider -- artifact that declares this
provider's capability, negotiation, prepare_exact_decode over the bound tensors, session,
synchronisation, step, the executor's own re-validation of the result.  Needs the reference tree
(QLLM_REFERENCE or a `reference` directory beside the repository); skipped where it is absent."""
import os
import subprocess

import pytest

from oracle.binding import reference_root

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_adapter_compiles_links_and_runs_against_the_reference(tmp_path):
    reference = reference_root()
    if not reference or not os.path.isdir(os.path.join(reference, "runtime", "include")):
        pytest.skip("the reference tree is not present on this machine")
    runtime = os.path.join(reference, "runtime")
    integration = os.path.join(ROOT, "integration")
    binary = str(tmp_path / "adapter_link_test")
    compiler = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    sources = [os.path.join(integration, f) for f in ("adapter_link_test.cpp", "b200_nvfp4_mtp_provider.cpp",
                                                      "stub_qllm_abi.cpp")]
    sources += [os.path.join(runtime, "src", f) for f in ("model_descriptor.cpp", "execution_provider.cpp",
                                                          "program_executor.cpp", "sha256.cpp")]
    build = subprocess.run([compiler, "-std=c++20", "-O1", "-w", f"-I{runtime}/include", f"-I{ROOT}/include",
                            f"-I{integration}", *sources, "-o", binary], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-4000:]
    run = subprocess.run([binary], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "PASS adapter link test" in run.stdout, run.stdout + run.stderr


def test_stub_and_header_agree_on_every_entry_point_the_adapter_calls():
    # the stub must not drift from include/qllm_b200.h: every function it defines is declared there
    import re
    header = open(os.path.join(ROOT, "include", "qllm_b200.h")).read()
    stub = open(os.path.join(ROOT, "integration", "stub_qllm_abi.cpp")).read()
    defined = set(re.findall(r"\b(qllm_[a-z0-9_]+)\s*\([^;{]*\)\s*\{", stub)) - {"qllm_stub_last_provider"}
    assert defined and all(re.search(r"\b%s\s*\(" % name, header) for name in defined), defined
